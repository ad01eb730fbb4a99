"""Host composition of one data-parallel training step of a Mamba-2 language
model over the C ABI (include/mp_kernels.h): every computation is a ``launch_*``
call on the library's stream; torch is used for device memory only.

Layer (pre-norm residual block), T = batch * seqlen tokens, r16 activations:
    xn   = rmsnorm(h, norm_w)
    zx   = xn @ W_in                      columns [ z | x B C | dt ]
    x,B,C= silu(causal_conv1d(zx[x B C]))
    dt   = softplus(zx[dt] + dt_bias);  A = -exp(A_log)
    y    = ssd_scan(x, dt, A, B, C)
    u    = (y + D x) * silu(z)
    h    = h + rmsnorm(u, gnorm_w) @ W_out
Head: logits = rmsnorm(h, normf_w) @ E^T (tied embedding), mean cross-entropy.

Weights live in one flat r32 master buffer (plus Adam moments); contractions and
norms read a flat r16 copy.  Gradients: contractions and norm gains write r16
into a flat r16 gradient buffer, everything reduced with atomics (embedding rows,
conv taps, biases, D, A_log) goes straight to the flat r32 gradient.

The update is bucketed and overlapped with the reverse pass: the flat buffers are
in layer order, so as soon as the reverse of a group of layers has finished, a
second stream folds that bucket's r16 gradients into the r32 ones, all-reduces
the bucket (data-parallel runs) and applies the mixed-precision Adam step, which
also writes the bucket's refreshed r16 weights - while the first stream is
already in the reverse of the layers below.  Only the embedding bucket, whose
gradient is complete last, is exposed.  For replay the main-stream work is captured
as one CUDA graph per bucket (cut where a bucket's gradients are complete); the
bucket updates - and with them every NCCL call - are issued live between the
graph launches, on the second stream.
"""
from __future__ import annotations

import ctypes as C
import os
import math
from dataclasses import dataclass

from .runtime import Stream, launch, lib


@dataclass
class LMConfig:
    d_model: int = 768
    n_layer: int = 24
    expand: int = 2
    headdim: int = 64
    d_state: int = 128
    ngroups: int = 1
    d_conv: int = 4
    vocab: int = 50280
    chunk: int = 256
    eps: float = 1e-6

    @property
    def d_inner(self):
        return self.expand * self.d_model

    @property
    def heads(self):
        return self.d_inner // self.headdim

    @property
    def conv_dim(self):
        return self.d_inner + 2 * self.ngroups * self.d_state

    @property
    def d_in_proj(self):
        return 2 * self.d_inner + 2 * self.ngroups * self.d_state + self.heads

    def param_shapes(self):
        """(name, shape) in flat-buffer order."""
        out = [("embedding", (self.vocab, self.d_model))]
        for i in range(self.n_layer):
            p = f"layers.{i}."
            out += [(p + "norm_w", (self.d_model,)), (p + "in_proj", (self.d_model, self.d_in_proj)),
                    (p + "conv_w", (self.conv_dim, self.d_conv)), (p + "conv_b", (self.conv_dim,)),
                    (p + "dt_bias", (self.heads,)), (p + "A_log", (self.heads,)), (p + "D", (self.heads,)),
                    (p + "gnorm_w", (self.d_inner,)), (p + "out_proj", (self.d_inner, self.d_model))]
        out.append(("normf_w", (self.d_model,)))
        return out

    def n_params(self):
        return sum(math.prod(s) for _, s in self.param_shapes())


def init_weights(cfg: LMConfig, seed: int = 0):
    """Random initial weights as float32 numpy arrays (name -> array)."""
    import numpy as np
    r = np.random.default_rng(seed)
    w = {}
    for name, shape in cfg.param_shapes():
        leaf = name.split(".")[-1]
        if leaf in ("norm_w", "gnorm_w", "normf_w", "D"):
            a = np.ones(shape)
        elif leaf == "conv_b":
            a = np.zeros(shape)
        elif leaf == "conv_w":
            a = r.uniform(-1.0, 1.0, shape) / math.sqrt(cfg.d_conv)
        elif leaf == "dt_bias":   # softplus^-1 of step sizes drawn log-uniformly from [1e-3, 1e-1]
            dt = np.exp(r.uniform(math.log(1e-3), math.log(1e-1), shape))
            a = dt + np.log(-np.expm1(-dt))
        elif leaf == "A_log":
            a = np.log(r.uniform(1.0, 16.0, shape))
        else:
            a = r.standard_normal(shape) * 0.02
        w[name] = a.astype(np.float32)
    return w


ALIGN = 64   # elements: keeps every parameter 128-byte aligned in the r16 copy


class MambaLM:
    def __init__(self, cfg: LMConfig, batch: int, seqlen: int, weights=None, seed: int = 0, stream: Stream | None = None,
                 loss_scale: float | None = None, bucket_layers: int = 4, overlap: bool = True):
        """loss_scale multiplies the logit gradient before it is stored in r16 (the mean cross-entropy puts a factor
        1/T on it, which at realistic T drops typical entries into the r16 subnormal range).  Default: the largest
        power of two not above T, so that scale/T is in (1/2, 1].  The scale is static; Adam skips elements whose
        gradient overflowed and `nonfinite_gradients()` reports it."""
        import torch
        self.cfg, self.batch, self.seqlen = cfg, batch, seqlen
        self.T = batch * seqlen
        self.loss_scale = float(loss_scale) if loss_scale is not None else float(2 ** int(math.floor(math.log2(max(self.T, 1)))))
        self._own_stream = stream is None
        self.stream = stream if stream is not None else Stream()
        self._lib = lib()
        dev = "cuda"
        if seqlen % cfg.chunk != 0:
            raise ValueError("seqlen must be a multiple of the scan chunk")
        # ---- flat parameter buffers ------------------------------------------------
        self.offsets, off = {}, 0
        for name, shape in cfg.param_shapes():
            self.offsets[name] = (off, shape)
            off += (math.prod(shape) + ALIGN - 1) // ALIGN * ALIGN
        self.n_flat = off
        self.w32 = torch.zeros(off, dtype=torch.float32, device=dev)
        self.w16 = torch.zeros(off, dtype=torch.float16, device=dev)
        self.g32 = torch.zeros(off, dtype=torch.float32, device=dev)
        self.g16 = torch.zeros(off, dtype=torch.float16, device=dev)
        self.m = torch.zeros(off, dtype=torch.float32, device=dev)
        self.v = torch.zeros(off, dtype=torch.float32, device=dev)
        weights = weights if weights is not None else init_weights(cfg, seed)
        host = torch.zeros(off, dtype=torch.float32)
        for name, (o, shape) in self.offsets.items():
            host[o:o + math.prod(shape)] = torch.from_numpy(weights[name]).reshape(-1)
        self.w32.copy_(host)
        torch.cuda.synchronize()
        self._refresh_w16()
        self.step_count = 0
        self.tick = torch.zeros(4, dtype=torch.float32, device=dev)   # Adam's step number and bias corrections (launch_adam_tick)
        # ---- update buckets, in the order the reverse pass completes them ------------------------------
        # (lo, hi, first layer of the group or -1 for the embedding): layer groups from the top (the final norm's gain
        # sits right behind the last layer), then the embedding
        self.buckets = []
        hi = off
        top = cfg.n_layer
        while top > 0:
            first = max(0, top - max(1, bucket_layers))
            lo = self.offsets[f"layers.{first}.norm_w"][0]
            self.buckets.append((lo, hi, first))
            hi, top = lo, first
        self.buckets.append((0, hi, -1))
        self.overlap = overlap                    # False: the bucket updates run on the main stream, between the reverse kernels
        self.side = Stream()                      # carries gradient folding, all-reduce and Adam of finished buckets
        self._ev_bucket = [self._lib.mpEventCreate() for _ in self.buckets]
        self._ev_join = self._lib.mpEventCreate()
        # ---- activations -------------------------------------------------------------
        T, c = self.T, cfg
        f16 = lambda *s: torch.empty(*s, dtype=torch.float16, device=dev)
        f32 = lambda *s: torch.empty(*s, dtype=torch.float32, device=dev)
        gn = c.ngroups * c.d_state
        self.ids = torch.zeros(T, dtype=torch.int32, device=dev)
        self.targets = torch.zeros(T, dtype=torch.int32, device=dev)
        self.saved = [dict(h_in=f16(T, c.d_model), xn=f16(T, c.d_model), rstd1=f32(T), zx=f16(T, c.d_in_proj), xs=f16(T, c.d_inner),
                           Bs=f16(T, gn), Cs=f16(T, gn), dt=f32(T, c.heads), A=f32(c.heads), y=f16(T, c.d_inner),
                           un=f16(T, c.d_inner), rstd2=f32(T)) for _ in range(c.n_layer)]
        # residual stream: the input of layer i is saved[i]["h_in"], its output is written straight into the next
        # layer's h_in (the last one into h_out), so nothing is copied
        self.h_out = f16(T, c.d_model)
        self.hn = f16(T, c.d_model)
        self.rstdf = f32(T)
        self.logits = f16(T, c.vocab)
        self.loss_rows = f32(T)
        self.loss_sum = f32(1)
        # backward temporaries
        self.gh = f16(T, c.d_model)
        self.gt = f16(T, c.d_model)
        self.gun = f16(T, c.d_inner)
        self.gy = f16(T, c.d_inner)
        self.gxs = f16(T, c.d_inner)
        self.gBs = f16(T, gn)
        self.gCs = f16(T, gn)
        self.gdt = f32(T, c.heads)
        self.gA = f32(c.heads)
        self.gzx = f16(T, c.d_in_proj)
        dims = (batch, seqlen, c.heads, c.headdim, c.d_state, c.ngroups, c.chunk)
        self.ssd_dims = dims
        n_scr = max(self._lib.mpSsdScanScratchBytes(*dims, 0), self._lib.mpSsdScanScratchBytes(*dims, 1))
        self.ssd_scratch = torch.empty(n_scr, dtype=torch.uint8, device=dev)
        n_rms = max(self._lib.mpRmsnormReverseScratchBytes(T, c.d_model, self.stream.ctx),
                    self._lib.mpSsdGateRmsnormReverseScratchBytes(T, c.heads, c.headdim, self.stream.ctx))
        self.rms_scratch = torch.empty(max(n_rms, 16), dtype=torch.uint8, device=dev)
        torch.cuda.synchronize()

    # ------------------------------------------------------------------ helpers
    def _p(self, buf, name, extra=0):
        """Device address of a parameter (or of its gradient) inside a flat buffer."""
        return buf.data_ptr() + (self.offsets[name][0] + extra) * buf.element_size()

    def _timed(self, name, call, side=False):
        """Run `call()`; while a profile is being taken, bracket it with CUDA events on the stream it is issued to."""
        prof = getattr(self, "_prof", None)
        if prof is None:
            call()
            return
        import torch
        ts = self._prof_side_ts if side else self._prof_ts
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(ts)
        call()
        e1.record(ts)
        prof.append((name + (" (update stream)" if side else ""), e0, e1))

    def _L(self, name, *args):
        import torch
        label = name + "_r16"
        if name.startswith(("inner_product", "linear")):
            label += "[%dx%dx%d]" % tuple(args[-3:])
        self._timed(label, lambda: launch(name, torch.float16, *args, self.stream))

    def _L32(self, name, *args):
        import torch
        self._timed(name + "_r32", lambda: launch(name, torch.float32, *args, self.stream))

    def _refresh_w16(self):
        self._timed("convert_r32_r16", lambda: self._lib.launch_convert_r32_r16(
            C.c_void_p(self.w32.data_ptr()), C.c_void_p(self.w16.data_ptr()), self.n_flat, self.stream.ctx))

    def profile_step(self, comm=None, world=1, **adam):
        """One training step issued launcher by launcher (no graph replay) with a CUDA-event pair around
        every launcher call.  Returns {launcher: {"ms": total device time, "calls": count}}; a launcher that
        forks work onto the library's side streams is bracketed on the caller's stream, join included, and the
        bucket updates are bracketed on the update stream (they overlap the reverse pass)."""
        self.stream.sync(); self.side.sync()
        self._prof, self._prof_ts, self._prof_side_ts = [], self.stream.torch_stream(), self.side.torch_stream()
        try:
            self._issue_step(comm, world, **adam)
            self.stream.sync(); self.side.sync()
            out = {}
            for name, e0, e1 in self._prof:
                r = out.setdefault(name, {"ms": 0.0, "calls": 0})
                r["ms"] += e0.elapsed_time(e1)
                r["calls"] += 1
        finally:
            self._prof = None
        return out

    def set_batch(self, ids, targets):
        """ids, targets: int32 tensors of batch*seqlen tokens, on the host (pinned memory makes the copy
        asynchronous) or on the device; the copies are ordered on the library's stream."""
        for dst, src in ((self.ids, ids), (self.targets, targets)):
            src = src.reshape(-1)
            assert src.numel() == self.T and src.element_size() == 4
            if src.is_cuda:   # int32 and r32 are both 4-byte words and the copy kernel is bit-exact
                self._lib.launch_copy_r32(C.c_void_p(src.data_ptr()), C.c_void_p(dst.data_ptr()), src.numel(), self.stream.ctx)
            else:
                self._lib.mpMemcpyHtoD(C.c_void_p(dst.data_ptr()), C.c_void_p(src.data_ptr()), src.numel() * 4, self.stream.ctx)

    # ------------------------------------------------------------------ forward
    def forward(self):
        c, T, s = self.cfg, self.T, self.stream
        W = self.w16
        di, gn, H, P = c.d_inner, c.ngroups * c.d_state, c.heads, c.headdim
        seg_widths = (C.c_ulong * 3)(di, gn, gn)   # channels (= row pitch) of the conv's x, B and C outputs
        dip = c.d_in_proj
        esz = 2
        self._L("embedding", self._p(W, "embedding"), self.ids, self.saved[0]["h_in"], T, c.d_model, c.vocab)
        for i, sv in enumerate(self.saved):
            p = f"layers.{i}."
            h_next = self.saved[i + 1]["h_in"] if i + 1 < c.n_layer else self.h_out
            self._L("rmsnorm_ij_j", sv["h_in"], self._p(W, p + "norm_w"), c.eps, sv["xn"], sv["rstd1"], T, c.d_model)
            self._L("inner_product_ij_jk_ik", sv["xn"], self._p(W, p + "in_proj"), 1.0, sv["zx"], 0.0, T, c.d_model, dip)
            zx = sv["zx"].data_ptr()
            # one conv over the [x | B | C] columns, each segment into its own contiguous tensor
            self._L("causal_conv1d_silu_segments", zx + di * esz, dip, self._p(W, p + "conv_w"), self._p(W, p + "conv_b"),
                    (C.c_void_p * 3)(sv["xs"].data_ptr(), sv["Bs"].data_ptr(), sv["Cs"].data_ptr()), seg_widths, seg_widths, 3,
                    self.batch, self.seqlen, c.d_conv)
            # dt = softplus(raw + dt_bias) and A = -exp(A_log) are formed inside the scan and kept for the reverse pass
            self._L("ssd_scan_raw", sv["xs"], zx + (di + c.conv_dim) * esz, dip, self._p(self.w32, p + "dt_bias"), self._p(self.w32, p + "A_log"),
                    sv["Bs"], sv["Cs"], sv["y"], sv["dt"], sv["A"], self.ssd_scratch, *self.ssd_dims)
            # skip, gate and the gated norm in one pass; the gated activation itself is never stored
            self._L("ssd_gate_rmsnorm", sv["y"], sv["xs"], self._p(self.w32, p + "D"), zx, dip, self._p(W, p + "gnorm_w"), c.eps, sv["un"],
                    sv["rstd2"], T, H, P)
            # out-projection with the residual added in its epilogue: h_next = un W + h_in
            self._L("linear_ij_jk_ik_ik", sv["un"], self._p(W, p + "out_proj"), sv["h_in"], 1.0, h_next, 0.0, T, di, c.d_model)
        self._L("rmsnorm_ij_j", self.h_out, self._p(W, "normf_w"), c.eps, self.hn, self.rstdf, T, c.d_model)
        self._L("inner_product_ij_kj_ik", self.hn, self._p(W, "embedding"), 1.0, self.logits, 0.0, T, c.d_model, c.vocab)

    def loss_and_logit_gradient(self):
        """Mean cross-entropy (device scalar in loss_sum after the reduce) and, in place of the logits, its
        gradient times loss_scale."""
        c, T = self.cfg, self.T
        self._L("cross_entropy", self.logits, self.targets, self.loss_scale / T, self.loss_rows, self.logits, T, c.vocab)
        self._L32("reduce_ij_i", self.loss_rows, self.loss_sum, 0.0, 1, T)

    # ------------------------------------------------------------------ backward
    def _update_bucket(self, k, comm, world, adam):
        """Bucket k's gradients are complete on the main stream: hand them to the update stream."""
        lo, hi, _ = self.buckets[k]
        n = hi - lo
        side = self.side if self.overlap else self.stream
        if self.overlap:
            self._lib.mpEventRecord(self._ev_bucket[k], self.stream.ctx)
            self._lib.mpStreamWaitEvent(side.ctx, self._ev_bucket[k])
        P = lambda buf: C.c_void_p(buf.data_ptr() + lo * buf.element_size())
        g16 = P(self.g16)
        if comm is not None and world > 1:
            self._timed("convert_r16_r32", lambda: self._lib.launch_convert_r16_r32(g16, P(self.g32), 1.0, n, side.ctx), side=True)
            self._timed("all_reduce_sum", lambda: comm.all_reduce_sum(self.g32[lo:hi], side), side=True)
            g16 = C.c_void_p(0)
        self._timed("adam_mixed_r32", lambda: self._lib.launch_adam_mixed_r32(
            P(self.w32), P(self.w16), P(self.g32), g16, P(self.m), P(self.v), adam["lr"], adam["beta1"], adam["beta2"], adam["eps"],
            1.0 / (self.loss_scale * world), C.c_void_p(self.tick.data_ptr()), n, side.ctx), side=True)

    def backward(self, at_bucket=None):
        """Reverse pass.  `at_bucket(k)` is called on the host right after the last launch that writes a gradient of
        bucket k (the update of that bucket, or a cut of the graph capture); None leaves the gradients in g16 / g32
        (use `fold_gradients()` to read them)."""
        c, T = self.cfg, self.T
        W, G16, G32 = self.w16, self.g16, self.g32
        di, gn, H, P = c.d_inner, c.ngroups * c.d_state, c.heads, c.headdim
        seg_widths = (C.c_ulong * 3)(di, gn, gn)   # channels (= row pitch) of the conv's x, B and C outputs
        dip, esz = c.d_in_proj, 2
        self._L32("fill", G32, 0.0, self.n_flat)
        self._L("fill", G16, 0.0, self.n_flat)
        gl = self.logits   # holds d loss / d logits
        self._L("inner_product_ij_jk_ik", gl, self._p(W, "embedding"), 1.0, self.gt, 0.0, T, c.vocab, c.d_model)
        self._L("inner_product_ji_jk_ik", gl, self.hn, 1.0, self._p(G16, "embedding"), 0.0, c.vocab, T, c.d_model)
        self._L("rmsnorm_ij_j_reverse", self.h_out, self._p(W, "normf_w"), self.rstdf, self.gt, c.eps, self.gh, self._p(G16, "normf_w"),
                0.0, self.rms_scratch, T, c.d_model)
        group_first = {first: k for k, (_, _, first) in enumerate(self.buckets)}
        for i in reversed(range(c.n_layer)):
            sv, p = self.saved[i], f"layers.{i}."
            zx, gzx = sv["zx"].data_ptr(), self.gzx.data_ptr()
            # out_proj
            self._L("inner_product_ij_kj_ik", self.gh, self._p(W, p + "out_proj"), 1.0, self.gun, 0.0, T, c.d_model, di)
            self._L("inner_product_ji_jk_ik", sv["un"], self.gh, 1.0, self._p(G16, p + "out_proj"), 0.0, di, T, c.d_model)
            self._L("ssd_gate_rmsnorm_reverse", sv["y"], sv["xs"], self._p(self.w32, p + "D"), zx, dip, self._p(W, p + "gnorm_w"), sv["rstd2"],
                    self.gun, self.gy, gzx, dip, self._p(G32, p + "D"), self._p(G16, p + "gnorm_w"), 0.0, self.rms_scratch, T, H, P)
            if os.environ.get("MP_LM_SPLIT_SCAN_REVERSE"):   # A/B: the three launches the fused entry replaces
                self._L("ssd_scan_reverse", sv["xs"], sv["dt"], sv["A"], sv["Bs"], sv["Cs"], self.gy, self.gxs, self.gdt, self.gA,
                        self.gBs, self.gCs, self.ssd_scratch, *self.ssd_dims)
                self._L32("hadamard_reverse", self.gA, sv["A"], self._p(G32, p + "A_log"), H)
                self._L("softplus_bias_reverse", zx + (di + c.conv_dim) * esz, dip, self._p(self.w32, p + "dt_bias"), self.gdt,
                        gzx + (di + c.conv_dim) * esz, dip, self._p(G32, p + "dt_bias"), T, H)
            else:
              # the scan's reverse also hands back the gradients of the raw step sizes (through the softplus), of dt_bias and of A_log
              self._L("ssd_scan_reverse_raw", sv["xs"], sv["dt"], sv["A"], sv["Bs"], sv["Cs"], self.gy, zx + (di + c.conv_dim) * esz, dip,
                      self._p(self.w32, p + "dt_bias"), self.gxs, self.gdt, self.gA, gzx + (di + c.conv_dim) * esz, dip, self._p(G32, p + "dt_bias"),
                      self._p(G32, p + "A_log"), self.gBs, self.gCs, self.ssd_scratch, *self.ssd_dims)
            # the D skip's share of the x gradient (D[h] * gy) joins the scan's inside the convolution's reverse
            self._L("causal_conv1d_silu_segments_reverse_skip", zx + di * esz, dip, self._p(W, p + "conv_w"), self._p(W, p + "conv_b"),
                    (C.c_void_p * 3)(self.gxs.data_ptr(), self.gBs.data_ptr(), self.gCs.data_ptr()), seg_widths, seg_widths, 3,
                    (C.c_void_p * 3)(self.gy.data_ptr(), None, None), (C.c_ulong * 3)(di, 0, 0),
                    (C.c_void_p * 3)(self._p(self.w32, p + "D"), None, None), P,
                    gzx + di * esz, dip, self._p(G32, p + "conv_w"), self._p(G32, p + "conv_b"), self.batch, self.seqlen, c.d_conv)
            # in_proj
            self._L("inner_product_ij_kj_ik", self.gzx, self._p(W, p + "in_proj"), 1.0, self.gt, 0.0, T, dip, c.d_model)
            self._L("inner_product_ji_jk_ik", sv["xn"], self.gzx, 1.0, self._p(G16, p + "in_proj"), 0.0, c.d_model, T, dip)
            # the block's share joins the residual gradient already in gh
            self._L("rmsnorm_ij_j_reverse", sv["h_in"], self._p(W, p + "norm_w"), sv["rstd1"], self.gt, c.eps, self.gh,
                    self._p(G16, p + "norm_w"), 1.0, self.rms_scratch, T, c.d_model)
            # (alpha = 1 would also accumulate the gain gradient; G16 was zero-filled, so that is a plain write)
            if at_bucket is not None and i in group_first:
                at_bucket(group_first[i])
        self._L("embedding_reverse", self.ids, self.gh, self._p(G32, "embedding"), T, c.d_model, c.vocab)
        if at_bucket is not None:
            at_bucket(len(self.buckets) - 1)

    def fold_gradients(self):
        """g32 += g16 over the whole flat buffer (only for a reverse pass run without updates)."""
        self._timed("convert_r16_r32", lambda: self._lib.launch_convert_r16_r32(
            C.c_void_p(self.g16.data_ptr()), C.c_void_p(self.g32.data_ptr()), 1.0, self.n_flat, self.stream.ctx))

    # ------------------------------------------------------------------ the step
    def _issue_main(self, at_bucket, beta1, beta2):
        """The main-stream sequence of a step, with the host callback at every completed bucket."""
        self._timed("adam_tick", lambda: self._lib.launch_adam_tick(C.c_void_p(self.tick.data_ptr()), beta1, beta2, self.stream.ctx))
        self.forward()
        self.loss_and_logit_gradient()
        self.backward(at_bucket)

    def _join_updates(self):
        # the next step's forward reads the refreshed weights
        if not self.overlap:
            return
        self._lib.mpEventRecord(self._ev_join, self.side.ctx)
        self._lib.mpStreamWaitEvent(self.stream.ctx, self._ev_join)

    def _issue_step(self, comm, world, lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8):
        adam = dict(lr=lr, beta1=beta1, beta2=beta2, eps=eps)
        self._issue_main(lambda k: self._update_bucket(k, comm, world, adam), beta1, beta2)
        self._join_updates()

    def capture(self, comm=None, world=1, lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8):
        """Record the main-stream work of a step as one CUDA graph per update bucket (the step is over nine hundred
        launches, which the host cannot issue as fast as the device runs them); `train_step` then launches the
        graphs one after another and issues each bucket's update - gradient folding, all-reduce, Adam - live on the
        second stream right behind the graph that completes the bucket.  No collective is ever part of a graph.
        The sequence is first run once for real (a training step like any other), so that every one-time set-up
        has happened before the capture."""
        self._issue_step(comm, world, lr=lr, beta1=beta1, beta2=beta2, eps=eps)
        self.step_count += 1
        self.stream.sync(); self.side.sync()
        graphs = []
        last = len(self.buckets) - 1

        def cut(k):
            graphs.append(self._lib.mpGraphEndCapture(self.stream.ctx))
            if k < last:
                self._lib.mpGraphBeginCapture(self.stream.ctx)
        self._lib.mpGraphBeginCapture(self.stream.ctx)
        self._issue_main(cut, beta1, beta2)
        self.graphs = graphs

    def train_step(self, comm=None, world=1, lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8):
        """forward, loss, reverse, (all-reduce), Adam.  Returns nothing: the mean loss of the step is read
        with ``loss()`` after a stream synchronisation."""
        self.step_count += 1
        if getattr(self, "graphs", None):
            adam = dict(lr=lr, beta1=beta1, beta2=beta2, eps=eps)
            for k, graph in enumerate(self.graphs):
                self._lib.mpGraphLaunch(graph, self.stream.ctx)
                self._update_bucket(k, comm, world, adam)
            self._join_updates()
        else:
            self._issue_step(comm, world, lr=lr, beta1=beta1, beta2=beta2, eps=eps)

    def adam_step(self, lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, world=1):
        """Whole-buffer update from the folded r32 gradient (after `forward_backward`), on the main stream."""
        self.step_count += 1
        self._timed("adam_tick", lambda: self._lib.launch_adam_tick(C.c_void_p(self.tick.data_ptr()), beta1, beta2, self.stream.ctx))
        self._timed("adam_mixed_r32", lambda: self._lib.launch_adam_mixed_r32(
            C.c_void_p(self.w32.data_ptr()), C.c_void_p(self.w16.data_ptr()), C.c_void_p(self.g32.data_ptr()), C.c_void_p(0),
            C.c_void_p(self.m.data_ptr()), C.c_void_p(self.v.data_ptr()), lr, beta1, beta2, eps, 1.0 / (self.loss_scale * world),
            C.c_void_p(self.tick.data_ptr()), self.n_flat, self.stream.ctx))

    def forward_backward(self):
        """Gradients only (no update): forward, loss, reverse, then the r16 gradients folded into g32."""
        self.forward()
        self.loss_and_logit_gradient()
        self.backward()
        self.fold_gradients()

    def nonfinite_gradients(self) -> bool:
        """True if any Adam update so far met a gradient that was not finite (and skipped that element)."""
        self.stream.sync(); self.side.sync()
        import torch
        return bool(self.tick.view(torch.int32)[3].item() != 0)

    def all_reduce_description(self) -> str:
        sizes = ", ".join("%.0f MB" % ((hi - lo) * 4 / 1e6) for lo, hi, _ in self.buckets)
        return ("%d buckets in the order the reverse pass completes them (%s); each is folded to r32, all-reduced with mpAllReduceSum (NCCL) "
                "and updated on a second stream while the reverse pass continues; only the last (embedding) bucket is exposed" % (len(self.buckets), sizes))

    def release(self):
        """Destroy the captured graph (if any) and the stream; the device buffers go with the object."""
        self.stream.sync(); self.side.sync()
        for graph in getattr(self, "graphs", None) or []:
            self._lib.mpGraphDestroy(graph)
        self.graphs = None
        for e in self._ev_bucket + [self._ev_join]:
            self._lib.mpEventDestroy(e)
        self.side.close()
        if self._own_stream:
            self.stream.close()

    def loss(self) -> float:
        self.stream.sync()   # the step's last main-stream operation waits for the update stream
        return float(self.loss_sum.item()) / self.T

    def grad(self, name):
        """Gradient of a parameter (float32 host array, already divided by loss_scale)."""
        self.stream.sync()
        o, shape = self.offsets[name]
        return (self.g32[o:o + math.prod(shape)].reshape(shape) / self.loss_scale).cpu().numpy()

    # ------------------------------------------------------------------ checkpoint
    def save(self, prefix: str):
        """Raw-bytes checkpoint in leaf order, one file per tensor named "{prefix}_{idx}" (the naming of the
        reference's tensor_file.zig:36-40): idx = position in `param_shapes()` for the r32 master weights, then
        the two Adam moments in the same order, and "{prefix}_state" with the step count."""
        import hashlib
        import math
        import os
        self.stream.sync(); self.side.sync()
        n = len(self.offsets)

        def write_atomically(path, writer):      # a crash leaves either the old file or the new one, never a torn one
            tmp = path + ".tmp"
            writer(tmp)
            os.replace(tmp, path)
        for k, buf in enumerate((self.w32, self.m, self.v)):
            host = buf.cpu().numpy()
            for idx, (name, (o, shape)) in enumerate(self.offsets.items()):
                write_atomically(f"{prefix}_{k * n + idx}", lambda t, a=host[o:o + math.prod(shape)]: a.tofile(t))
        layout = hashlib.sha256(repr(self.cfg.param_shapes()).encode()).hexdigest()

        def write_state(t):
            with open(t, "w") as f:
                f.write(f"{self.step_count}\n{n}\n{layout}\n")
        write_atomically(f"{prefix}_state", write_state)    # written last: its presence marks a complete checkpoint

    def load(self, prefix: str):
        import hashlib
        import math
        import numpy as np
        import torch
        self.stream.sync(); self.side.sync()
        n = len(self.offsets)
        with open(f"{prefix}_state") as f:
            fields = f.read().split()
        step = int(fields[0])
        if len(fields) >= 3:     # tensor count and layout hash of the configuration the checkpoint was written with
            layout = hashlib.sha256(repr(self.cfg.param_shapes()).encode()).hexdigest()
            if int(fields[1]) != n or fields[2] != layout:
                raise ValueError(f"{prefix}_state was written for another parameter layout")
        for k, buf in enumerate((self.w32, self.m, self.v)):
            host = np.zeros(self.n_flat, dtype=np.float32)
            for idx, (name, (o, shape)) in enumerate(self.offsets.items()):
                cnt = math.prod(shape)
                a = np.fromfile(f"{prefix}_{k * n + idx}", dtype=np.float32)
                if a.size != cnt:
                    raise ValueError(f"{prefix}_{k * n + idx}: expected {cnt} values for {name}, found {a.size}")
                host[o:o + cnt] = a
            buf.copy_(torch.from_numpy(host))
        torch.cuda.synchronize()
        self.step_count = step
        self.tick.zero_()
        self.tick.view(torch.int32)[2] = step     # Adam's step number continues where the checkpoint left off
        torch.cuda.synchronize()
        self._refresh_w16()

    def launches_per_step(self, world: int = 1) -> int:
        """Kernel launches of one training step: the kernel nodes of the captured graphs plus the live launches of the
        bucket updates (0 before `capture`).  NCCL's own kernels are not counted."""
        graphs = getattr(self, "graphs", None)
        if not graphs:
            return 0
        return sum(int(self._lib.mpGraphKernelNodes(g)) for g in graphs) + (2 if world > 1 else 1) * len(self.buckets)
