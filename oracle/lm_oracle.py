"""Float64 CPU statement of the Mamba-2 language-model step composed in
metaphor_b200/mamba_lm.py, written from the formulas in that module's docstring
with the scan as the sequential recurrence S_t = exp(dt_t A) S_{t-1} + dt_t B_t x_t^T,
y_t = C_t^T S_t.  Gradients come from torch autograd in float64.

TEST INFRASTRUCTURE: imported only by tests/ (reduced instances; the
recurrence is a Python loop over time).
"""
from __future__ import annotations

import torch


def _rmsnorm(x, w, eps):
    return x * torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


def forward_loss(cfg, weights, ids, targets, batch, seqlen):
    """weights: name -> float64 tensor (requires_grad as wanted); ids, targets: int64 [batch*seqlen].
    Returns the mean cross-entropy."""
    di, gn, H, P, N = cfg.d_inner, cfg.ngroups * cfg.d_state, cfg.heads, cfg.headdim, cfg.d_state
    h = weights["embedding"][ids]                                   # [T, d]
    for i in range(cfg.n_layer):
        p = f"layers.{i}."
        xn = _rmsnorm(h, weights[p + "norm_w"], cfg.eps)
        zx = xn @ weights[p + "in_proj"]
        z, xbc, dtr = zx[:, :di], zx[:, di:di + cfg.conv_dim], zx[:, di + cfg.conv_dim:]
        xbc = xbc.reshape(batch, seqlen, cfg.conv_dim)
        pad = torch.cat([torch.zeros(batch, cfg.d_conv - 1, cfg.conv_dim, dtype=xbc.dtype), xbc], dim=1)
        pre = weights[p + "conv_b"] + sum(weights[p + "conv_w"][:, k] * pad[:, k:k + seqlen, :] for k in range(cfg.d_conv))
        act = pre * torch.sigmoid(pre)
        x = act[..., :di].reshape(batch, seqlen, H, P)
        Bm = act[..., di:di + gn].reshape(batch, seqlen, cfg.ngroups, N)
        Cm = act[..., di + gn:].reshape(batch, seqlen, cfg.ngroups, N)
        dt = torch.nn.functional.softplus(dtr + weights[p + "dt_bias"]).reshape(batch, seqlen, H)
        A = -torch.exp(weights[p + "A_log"])
        hpg = H // cfg.ngroups
        Bh = Bm.repeat_interleave(hpg, dim=2)                       # [b, l, H, N]
        Ch = Cm.repeat_interleave(hpg, dim=2)
        S = torch.zeros(batch, H, N, P, dtype=x.dtype)
        ys = []
        for t in range(seqlen):
            decay = torch.exp(dt[:, t] * A)                         # [b, H]
            S = decay[..., None, None] * S + (dt[:, t, :, None] * Bh[:, t])[..., None] * x[:, t, :, None, :]
            ys.append(torch.einsum("bhn,bhnp->bhp", Ch[:, t], S))
        y = torch.stack(ys, dim=1)                                  # [b, l, H, P]
        y = y + weights[p + "D"][None, None, :, None] * x
        u = y.reshape(batch * seqlen, di) * (z * torch.sigmoid(z))
        h = h + _rmsnorm(u, weights[p + "gnorm_w"], cfg.eps) @ weights[p + "out_proj"]
    hn = _rmsnorm(h, weights["normf_w"], cfg.eps)
    logits = hn @ weights["embedding"].T
    return torch.nn.functional.cross_entropy(logits, targets)
