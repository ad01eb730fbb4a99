"""Reduced instance of the Mamba-2 language-model training step: loss and every
parameter gradient of the C-ABI composition (r16 activations) against the
float64 CPU statement with autograd, then one Adam step against the oracle's
Adam on the same gradients."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_reduced_lm_step(mp, stream, orc):
    import torch
    from metaphor_b200.mamba_lm import LMConfig, MambaLM, init_weights
    from oracle import lm_oracle

    cfg = LMConfig(d_model=256, n_layer=2, vocab=1024, chunk=128)
    batch, seqlen = 2, 256
    w = init_weights(cfg, seed=0)
    rng = np.random.default_rng(1000)
    ids = rng.integers(0, cfg.vocab, size=batch * seqlen).astype(np.int32)
    targets = rng.integers(0, cfg.vocab, size=batch * seqlen).astype(np.int32)

    model = MambaLM(cfg, batch, seqlen, weights=w, stream=stream, loss_scale=256.0)
    torch.cuda.current_stream().synchronize()
    model.set_batch(torch.from_numpy(ids), torch.from_numpy(targets))
    model.forward()
    model.loss_and_logit_gradient()
    model.backward()
    model.fold_gradients()
    loss = model.loss()
    assert stream.status() == 0

    # the oracle sees the weights the contractions see: rounded to r16 (per-head parameters stay r32)
    small = ("dt_bias", "A_log", "D")
    wt = {k: torch.tensor(v.astype(np.float64) if k.split(".")[-1] in small else v.astype(np.float16).astype(np.float64), requires_grad=True)
          for k, v in w.items()}
    ref = lm_oracle.forward_loss(cfg, wt, torch.from_numpy(ids.astype(np.int64)), torch.from_numpy(targets.astype(np.int64)), batch, seqlen)
    ref.backward()
    ref_loss = float(ref.detach())
    assert abs(loss - ref_loss) <= 1e-2 * abs(ref_loss), (loss, ref_loss)   # r16 activations: the r16 tolerance
    assert abs(loss - ref_loss) <= 2e-3 * abs(ref_loss), ("loss is usually within 2e-3", loss, ref_loss)
    worst = {}
    for name in w:
        g, r = model.grad(name).astype(np.float64), wt[name].grad.numpy()
        err = np.max(np.abs(g - r)) / max(np.max(np.abs(r)), 1e-30)
        worst[name] = err
    print('loss', loss, ref_loss, 'gradient errors (max |got - ref| / max |ref|), worst first:')
    for k, v in sorted(worst.items(), key=lambda kv: -kv[1]):
        print(f"  {k:28s} {v:.3e}")
    # Every tensor is held to the r16 tolerance 1e-2, with one stated exception: A_log.  Its gradient is
    # sum_t dt_t g_a[t] with g_a the suffix sum of u_t - v_t (u = <gy, y>, v = <gx, x>), two nearly equal quantities
    # that come from two separate walks over r16 operand tiles; the difference keeps the rounding noise of both, and
    # where the true sum over a head is small the relative error of that head exceeds 1e-2 (measured 1.6e-2 - 1.9e-2
    # on layer 0 of this instance, below 3e-3 on every other tensor).
    limit = lambda name: 2.5e-2 if name.endswith("A_log") else 1e-2
    bad = {k: v for k, v in worst.items() if v > limit(k)}
    assert not bad, f"gradients outside the r16 tolerance of the float64 oracle: {bad}"

    # Adam on the flat buffer against the scalar oracle on the same gradient
    g32 = model.g32.cpu().numpy().copy()
    w32 = model.w32.cpu().numpy().copy()
    model.adam_step(lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8)
    stream.sync()
    mref, vref = np.zeros_like(w32), np.zeros_like(w32)
    wref, _, _ = orc.adam(w32.copy(), g32, mref, vref, 3e-4, 0.9, 0.95, 1e-8, 1.0 / 256.0, 1)
    got = model.w32.cpu().numpy()
    assert np.max(np.abs(got - wref)) <= 1e-6
    assert np.array_equal(model.w16.cpu().numpy(), got.astype(np.float16))
    assert not model.nonfinite_gradients()


def test_default_loss_scale_and_overflow_flag(mp, stream):
    """Default arguments at a realistic token count: the default loss scale keeps the r16 logit gradient out of the
    subnormal range (every weight gets a non-zero update), and a gradient that overflows is skipped and reported."""
    import torch
    from metaphor_b200.mamba_lm import LMConfig, MambaLM
    cfg = LMConfig(d_model=256, n_layer=1, vocab=4096, chunk=128)
    batch, seqlen = 8, 2048                      # T = 16384: 1/T = 6.1e-5 is already the smallest normal r16 number
    model = MambaLM(cfg, batch, seqlen, seed=0, stream=stream)
    assert model.loss_scale == 16384.0
    g = torch.Generator().manual_seed(5)
    tok = torch.randint(0, cfg.vocab, (batch * seqlen + 1,), generator=g, dtype=torch.int32)
    torch.cuda.current_stream().synchronize()
    model.set_batch(tok[:-1].contiguous(), tok[1:].contiguous())
    model.forward_backward()
    stream.sync()
    emb = model.grad("embedding")
    assert np.isfinite(emb).all()
    used = np.unique(tok.numpy())
    assert (np.abs(emb[used]).max(axis=1) > 0).mean() > 0.99      # rows of tokens that occur all carry gradient
    w_before = model.w32.cpu().numpy().copy()
    model.g32[7] = float("inf")
    torch.cuda.synchronize()
    model.adam_step()
    assert model.nonfinite_gradients()
    w_after = model.w32.cpu().numpy()
    assert w_after[7] == w_before[7] and np.isfinite(w_after).all()
    model.release()


def test_checkpoint_resume(mp, stream, tmp_path):
    """Two steps, save, one more step; a fresh model that loads the checkpoint reproduces that step: the same
    loss bit for bit (the forward pass is deterministic), the same weights up to the summation order of the
    atomically reduced parameter gradients."""
    import torch
    from metaphor_b200.mamba_lm import LMConfig, MambaLM
    cfg = LMConfig(d_model=256, n_layer=1, vocab=512, chunk=128)
    batch, seqlen = 1, 256
    rng = np.random.default_rng(7)
    ids = torch.from_numpy(rng.integers(0, cfg.vocab, size=batch * seqlen).astype(np.int32))
    tgt = torch.from_numpy(rng.integers(0, cfg.vocab, size=batch * seqlen).astype(np.int32))
    a = MambaLM(cfg, batch, seqlen, seed=3, stream=stream, loss_scale=128.0)
    torch.cuda.current_stream().synchronize()
    a.set_batch(ids, tgt)
    for _ in range(2):
        a.train_step()
    prefix = str(tmp_path / "ckpt")
    a.save(prefix)
    a.train_step()
    loss_a, w_a = a.loss(), a.w32.cpu().numpy().copy()
    b = MambaLM(cfg, batch, seqlen, seed=99, stream=stream, loss_scale=128.0)   # different initial weights
    torch.cuda.current_stream().synchronize()
    b.load(prefix)
    b.set_batch(ids, tgt)
    b.train_step()
    assert b.step_count == 3
    assert b.loss() == loss_a
    assert np.max(np.abs(b.w32.cpu().numpy() - w_a)) <= 1e-6
