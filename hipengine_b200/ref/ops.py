"""Plain PyTorch fp32 reference ops: the oracle every CUDA kernel is tested against.

The numerics contract follows what the reference's NumPy oracle library defines
(``hipengine/kernels/cpu_reference/ops.py``): RMSNorm with fp32 statistics and
the GGUF weight used directly (``:26-30``); split-half (NeoX) rotation of the
first ``rope_dim`` dims of each head (``:1255-1290``); causal GQA attention with
an optional sigmoid output gate (``:2144-2256``); depthwise causal conv + SiLU
with a rolling state (``:1912-1964``); the serial Gated Delta Rule
(``:1967-2012``) and its chunkwise WY form (``:2015-2141``); MoE routing as
softmax over all experts, stable top-k, renormalise by ``max(sum, 6.1e-5)``
(``:575-621``); shared expert gated by a sigmoid (``:681-739``).

Everything here runs on CPU tensors (or CUDA, for large-shape GPU oracles) and
is written for clarity, not speed.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as F


def rmsnorm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float = 1e-6) -> torch.Tensor:
    xf = x.to(torch.float32)
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w.to(torch.float32)


def l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    xf = x.to(torch.float32)
    n = xf.pow(2).sum(-1, keepdim=True).sqrt().clamp(min=eps)
    return xf / n


def rope_neox(x: torch.Tensor, positions: torch.Tensor, theta: float, rope_dim: int) -> torch.Tensor:
    """x: [T, H, D]; rotate dims [0, rope_dim) in split-half pairing (i, i + rope_dim/2)."""
    xf = x.to(torch.float32)
    half = rope_dim // 2
    inv = theta ** (-torch.arange(half, dtype=torch.float32, device=x.device) * 2.0 / rope_dim)
    ang = positions.to(torch.float32)[:, None] * inv[None, :]
    c = ang.cos()[:, None, :]
    s = ang.sin()[:, None, :]
    a = xf[..., :half]
    b = xf[..., half:rope_dim]
    out = xf.clone()
    out[..., :half] = a * c - b * s
    out[..., half:rope_dim] = b * c + a * s
    return out


def causal_gqa_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_pos: torch.Tensor,
                         scale: float, window: int = 0, k_pos: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q: [T, H, D]; k, v: [S, Hkv, D(v)] cached rows at positions ``k_pos`` (default 0..S-1).

    Row t attends keys with ``k_pos <= q_pos[t]`` (and ``> q_pos[t] - window`` when windowed).
    """
    T, H, D = q.shape
    S, Hkv, _ = k.shape
    g = H // Hkv
    if k_pos is None:
        k_pos = torch.arange(S, device=q.device)
    qf = q.to(torch.float32).reshape(T, Hkv, g, D)
    kf = k.to(torch.float32)
    vf = v.to(torch.float32)
    s = torch.einsum("thgd,shd->thgs", qf, kf) * scale
    mask = k_pos[None, :] <= q_pos[:, None]
    if window > 0:
        mask = mask & (k_pos[None, :] > (q_pos[:, None] - window))
    s = s.masked_fill(~mask[:, None, None, :], float("-inf"))
    p = torch.softmax(s, dim=-1)
    o = torch.einsum("thgs,shd->thgd", p, vf)
    return o.reshape(T, H, vf.shape[-1])


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(x)


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    return F.gelu(x, approximate="tanh")


def softplus20(x: torch.Tensor) -> torch.Tensor:
    return torch.where(x > 20.0, x, torch.log1p(torch.exp(torch.clamp(x, max=20.0))))


def causal_conv1d_silu(x: torch.Tensor, w: torch.Tensor, state: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Depthwise causal conv + SiLU.

    x: [T, C]; w: [C, K]; state: [C, K-1] = the previous K-1 inputs (oldest first).
    Returns (out [T, C], new_state [C, K-1]).  out[t,c] = SiLU(sum_k w[c,k] * xx[t+k,c]) where xx
    is ``state`` followed by ``x``.
    """
    T, C = x.shape
    K = w.shape[1]
    xx = torch.cat([state.to(torch.float32).t(), x.to(torch.float32)], dim=0)  # [K-1+T, C]
    out = torch.zeros(T, C, dtype=torch.float32, device=x.device)
    for kk in range(K):
        out += xx[kk:kk + T] * w[:, kk].to(torch.float32)[None, :]
    new_state = xx[T:T + K - 1].t().contiguous()
    return silu(out), new_state


def gdn_gates(a: torch.Tensor, b: torch.Tensor, ssm_a: torch.Tensor, dt_bias: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """a, b: [T, Hv] projections.  Returns (decay [T, Hv], beta [T, Hv]).

    GGUF stores ``ssm_a`` as the negative coefficient ``-exp(a_log)`` so
    ``decay = exp(ssm_a * softplus(a + dt_bias))``.
    """
    beta = torch.sigmoid(b.to(torch.float32))
    g = ssm_a.to(torch.float32)[None, :] * softplus20(a.to(torch.float32) + dt_bias.to(torch.float32)[None, :])
    return torch.exp(g), beta


def gdn_recurrent(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, beta: torch.Tensor,
                  state: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Serial Gated Delta Rule.

    q, k: [T, Hv, Dk] (already L2-normalised, q scaled, K heads broadcast to V heads);
    v: [T, Hv, Dv]; decay, beta: [T, Hv]; state: [Hv, Dk, Dv].  Returns (o [T, Hv, Dv], state).
    """
    S = state.to(torch.float32).clone()
    T = q.shape[0]
    out = torch.empty_like(v, dtype=torch.float32)
    qf, kf, vf = q.to(torch.float32), k.to(torch.float32), v.to(torch.float32)
    for t in range(T):
        S = S * decay[t][:, None, None]
        kv = torch.einsum("hk,hkv->hv", kf[t], S)
        delta = (vf[t] - kv) * beta[t][:, None]
        S = S + kf[t][:, :, None] * delta[:, None, :]
        out[t] = torch.einsum("hk,hkv->hv", qf[t], S)
    return out, S


def gdn_chunked(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, beta: torch.Tensor,
                state: torch.Tensor, chunk: int = 64, dtype=torch.float64) -> Tuple[torch.Tensor, torch.Tensor]:
    """Chunkwise WY form of the same recurrence (algebra oracle for the tensor-core scan).

    Within a chunk with cumulative log-decay ``G_i`` the update solves
    ``(I + tril(diag(beta) (K K^T * exp(G_i - G_j)), -1)) U = diag(beta) (V - exp(G) K S0)``.
    """
    T, H, Dk = q.shape
    Dv = v.shape[-1]
    S = state.to(dtype).clone()
    out = torch.empty(T, H, Dv, dtype=dtype, device=q.device)
    qd, kd, vd = q.to(dtype), k.to(dtype), v.to(dtype)
    lg = torch.log(decay.to(dtype))
    bd = beta.to(dtype)
    for c0 in range(0, T, chunk):
        c1 = min(T, c0 + chunk)
        n = c1 - c0
        G = torch.cumsum(lg[c0:c1], dim=0)                   # [n, H]
        for h in range(H):
            Kc, Qc, Vc, g, b = kd[c0:c1, h], qd[c0:c1, h], vd[c0:c1, h], G[:, h], bd[c0:c1, h]
            diff = torch.exp((g[:, None] - g[None, :]).tril())     # masked below
            A = (Kc @ Kc.t()) * diff * b[:, None]
            A = torch.tril(A, -1)
            rhs = b[:, None] * (Vc - torch.exp(g)[:, None] * (Kc @ S[h]))
            U = torch.linalg.solve_triangular(torch.eye(n, dtype=dtype, device=q.device) + A, rhs, upper=False)
            QK = torch.tril((Qc @ Kc.t()) * diff)
            out[c0:c1, h] = torch.exp(g)[:, None] * (Qc @ S[h]) + QK @ U
            gl = g[-1]
            S[h] = torch.exp(gl) * S[h] + (Kc * torch.exp(gl - g)[:, None]).t() @ U
    return out.to(torch.float32), S.to(torch.float32)


def gated_rmsnorm(o: torch.Tensor, w: torch.Tensor, z: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """RMSNorm over the last dim with weight ``w`` then multiply by SiLU(z)."""
    return rmsnorm(o, w, eps) * silu(z.to(torch.float32))


def moe_route(logits: torch.Tensor, top_k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Softmax over all experts -> stable top-k (lower id wins ties) -> renormalise."""
    p = torch.softmax(logits.to(torch.float32), dim=-1)
    # stable descending sort keeps the lower expert id first among equals
    vals, idx = torch.sort(p, dim=-1, descending=True, stable=True)
    vals, idx = vals[..., :top_k], idx[..., :top_k]
    denom = vals.sum(-1, keepdim=True).clamp(min=6.1e-5)
    return idx, vals / denom


def swiglu(gate: torch.Tensor, up: torch.Tensor, act: str = "silu") -> torch.Tensor:
    g = gate.to(torch.float32)
    return (silu(g) if act == "silu" else gelu_tanh(g)) * up.to(torch.float32)


def bf16_round(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).to(torch.float32)


def q8_1_quantize(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-32 symmetric int8 activation quantisation used by the dp4a GEMV path.

    Returns (q int8 [..., K], d float32 [..., K/32]) with ``d = amax/127`` and ``q = rint(x/d)``.
    """
    xf = x.to(torch.float32)
    shp = xf.shape
    xb = xf.reshape(shp[:-1] + (shp[-1] // 32, 32))
    amax = xb.abs().amax(-1)
    d = amax / 127.0
    inv = torch.where(d > 0, 1.0 / d, torch.zeros_like(d))
    qv = torch.round(xb * inv[..., None]).clamp(-127, 127).to(torch.int8)
    return qv.reshape(shp), d


# ----------------------------------------------------------------------------- INT8 KV storage (per token and head)
def kv_int8_quantize(x: torch.Tensor, scale_dtype: torch.dtype = torch.float16) -> Tuple[torch.Tensor, torch.Tensor]:
    """K or V rows [..., D] -> (int8 values [..., D], one scale per row in ``scale_dtype``).

    Symmetric, per (token, head): ``scale = amax / 127`` rounded to the scale type FIRST, then ``q = rint(x / scale)``
    clipped to +-127, so that a reader multiplying by the stored scale reproduces exactly what the writer meant.  This
    is the reference's default INT8 KV format (``hipengine/kvcache/spans.py``: granularity ``per_token_head``, fp16 or
    fp32 scales; oracle ``hipengine/kernels/cpu_reference/ops.py:1313-1910``)."""
    xf = x.to(torch.float32)
    amax = xf.abs().amax(-1)
    scale = (amax / 127.0).to(scale_dtype)
    sf = scale.to(torch.float32)
    inv = torch.where(sf > 0, 1.0 / sf, torch.zeros_like(sf))
    q = torch.round(xf * inv[..., None]).clamp(-127, 127).to(torch.int8)
    return q, scale


def kv_int8_dequantize(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    return q.to(torch.float32) * scale.to(torch.float32)[..., None]


def kv_store_roundtrip(x: torch.Tensor, storage: str, scale_dtype: torch.dtype = torch.float16) -> torch.Tensor:
    """What attention reads back after ``x`` went through the KV store: bf16 rounding, or INT8 with a per-row scale."""
    if storage == "int8":
        return kv_int8_dequantize(*kv_int8_quantize(x, scale_dtype))
    if storage == "bf16":
        return x.to(torch.bfloat16).to(torch.float32)
    return x.to(torch.float32)
