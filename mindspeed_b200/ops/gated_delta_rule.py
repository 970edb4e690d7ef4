"""Gated delta rule (linear attention with a decaying, delta-updated state) in recurrent and chunked form.

State S [d_k, d_v] per head.  Per token t with decay g_t = exp(alpha_t) in (0, 1] and write strength beta_t:
      S_t = g_t * S_{t-1} + beta_t * k_t (v_t - (g_t * S_{t-1})^T k_t)^T ,      o_t = S_t^T q_t
``recurrent`` is the definition; ``chunked`` processes C tokens at a time with the WY representation: inside a chunk
the rank-C update is solved as a unit-lower-triangular system, so the sequential dependency is over chunks only and
the per-chunk work is matrix products.  Both are differentiable PyTorch; q and k are L2-normalised when
``use_qk_l2norm`` is set, matching the reference kernels.
reference: mindspeed/ops/triton/{chunk_delta_h,chunk_o,chunk_scaled_dot_kkt,wy_fast,solve_tril,cumsum,l2norm}.py.
"""
from __future__ import annotations

import torch


def _l2norm(x, eps=1e-6):
    return x * torch.rsqrt(x.float().pow(2).sum(-1, keepdim=True) + eps).to(x.dtype)


def gated_delta_rule_recurrent(q, k, v, g, beta, scale=None, initial_state=None, use_qk_l2norm=False):
    """q, k [B, T, H, dk]; v [B, T, H, dv]; g (log decay, <= 0), beta [B, T, H] -> (o [B, T, H, dv], final state)."""
    if use_qk_l2norm:
        q, k = _l2norm(q), _l2norm(k)
    B, T, H, dk = q.shape
    dv = v.shape[-1]
    scale = dk ** -0.5 if scale is None else scale
    S = q.new_zeros(B, H, dk, dv, dtype=torch.float32) if initial_state is None else initial_state.float()
    out = []
    qf, kf, vf = q.float() * scale, k.float(), v.float()
    for t in range(T):
        S = S * torch.exp(g[:, t].float())[..., None, None]
        kt = kf[:, t]
        pred = torch.einsum("bhkv,bhk->bhv", S, kt)
        S = S + torch.einsum("bhk,bhv->bhkv", kt, (vf[:, t] - pred) * beta[:, t].float().unsqueeze(-1))
        out.append(torch.einsum("bhkv,bhk->bhv", S, qf[:, t]))
    return torch.stack(out, dim=1).to(v.dtype), S


def gated_delta_rule_chunked(q, k, v, g, beta, scale=None, initial_state=None, chunk_size=64, use_qk_l2norm=False):
    if use_qk_l2norm:
        q, k = _l2norm(q), _l2norm(k)
    B, T, H, dk = q.shape
    dv = v.shape[-1]
    scale = dk ** -0.5 if scale is None else scale
    C = chunk_size
    pad = (-T) % C
    if pad:
        z = lambda t: torch.nn.functional.pad(t, (0, 0) * (t.dim() - 2) + (0, pad))
        q, k, v = z(q), z(k), z(v)
        g = torch.nn.functional.pad(g, (0, 0, 0, pad))
        beta = torch.nn.functional.pad(beta, (0, 0, 0, pad))
    Tp = T + pad
    n = Tp // C
    # [B, H, n, C, d]
    rs = lambda t: t.float().permute(0, 2, 1, 3).reshape(B, H, n, C, t.shape[-1])
    qc, kc, vc = rs(q) * scale, rs(k), rs(v)
    gc = g.float().permute(0, 2, 1).reshape(B, H, n, C).cumsum(-1)          # log decay accumulated inside the chunk
    bc = beta.float().permute(0, 2, 1).reshape(B, H, n, C)
    S = q.new_zeros(B, H, dk, dv, dtype=torch.float32) if initial_state is None else initial_state.float()
    tril = torch.tril(torch.ones(C, C, device=q.device, dtype=torch.bool), -1)
    tril_incl = torch.tril(torch.ones(C, C, device=q.device, dtype=torch.bool), 0)
    eye = torch.eye(C, device=q.device)
    outs = []
    for c in range(n):
        kk, vv, qq, gg, bb = kc[:, :, c], vc[:, :, c], qc[:, :, c], gc[:, :, c], bc[:, :, c]
        decay = torch.exp(gg.unsqueeze(-1) - gg.unsqueeze(-2))               # exp(G_i - G_j), used for i >= j
        # delta_i = beta_i (v_i - e^{G_i} S0^T k_i - sum_{j<i} e^{G_i - G_j} (k_j . k_i) delta_j)   ->  (I + A) Delta = R
        A = (torch.einsum("bhik,bhjk->bhij", kk, kk) * decay * bb.unsqueeze(-1)).masked_fill(~tril, 0.0)
        R = bb.unsqueeze(-1) * (vv - torch.exp(gg).unsqueeze(-1) * torch.einsum("bhkv,bhik->bhiv", S, kk))
        delta = torch.linalg.solve_triangular(A + eye, R, upper=False, unitriangular=True)
        # o_i = e^{G_i} S0^T q_i + sum_{j<=i} e^{G_i - G_j} (k_j . q_i) delta_j
        attn = (torch.einsum("bhik,bhjk->bhij", qq, kk) * decay).masked_fill(~tril_incl, 0.0)
        o = torch.exp(gg).unsqueeze(-1) * torch.einsum("bhkv,bhik->bhiv", S, qq) + torch.einsum("bhij,bhjv->bhiv", attn, delta)
        outs.append(o)
        # S_C = e^{G_C} S0 + sum_j e^{G_C - G_j} k_j delta_j^T
        last = gg[..., -1]
        w = torch.exp(last.unsqueeze(-1) - gg)
        S = S * torch.exp(last)[..., None, None] + torch.einsum("bhjk,bhjv->bhkv", kk * w.unsqueeze(-1), delta)
    o = torch.stack(outs, dim=2).reshape(B, H, Tp, dv).permute(0, 2, 1, 3)[:, :T]
    return o.to(v.dtype), S


def chunk_gated_delta_rule(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False, chunk_size=64,
                           use_qk_l2norm_in_kernel=False):
    """Entry point with the call shape of the reference op."""
    o, S = gated_delta_rule_chunked(q, k, v, g, beta, scale, initial_state, chunk_size, use_qk_l2norm_in_kernel)
    return o, (S if output_final_state else None)
