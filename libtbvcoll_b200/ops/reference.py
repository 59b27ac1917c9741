"""Plain PyTorch statements of every operator, used as the numerics oracle in tests and by
the stock-PyTorch baseline model.  They run on CPU or GPU and follow HF Llama's bf16
semantics (each elementwise op rounds to bf16) so that the CUDA kernels can be compared
tightly; `*_f32` variants compute in fp32 throughout for tolerance-based checks."""
from __future__ import annotations

import torch


def rmsnorm(x: torch.Tensor, gamma: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    var = xf.pow(2).mean(-1, keepdim=True)
    return gamma * (xf * torch.rsqrt(var + eps)).to(x.dtype)


def add_rmsnorm(x: torch.Tensor, residual: torch.Tensor, gamma: torch.Tensor, eps: float):
    h = (x.float() + residual.float()).to(x.dtype)
    return rmsnorm(h, gamma, eps), h


def ar_residual_rmsnorm(partials, residual, gamma, eps):
    """fused collective oracle: bf16(sum in rank order, fp32) -> + residual -> RMSNorm"""
    acc = partials[0].float().clone()
    for p in partials[1:]:
        acc += p.float()
    s = acc.to(partials[0].dtype)
    return add_rmsnorm(s, residual, gamma, eps)


def rope(qk: torch.Tensor, positions: torch.Tensor, cos_sin: torch.Tensor) -> torch.Tensor:
    """qk: [T, heads, D]; HF rotate_half pairing, bf16 cos/sin, bf16 arithmetic."""
    D = qk.shape[-1]
    cs = cos_sin[positions.long()]
    cos = torch.cat((cs[:, : D // 2], cs[:, : D // 2]), -1).to(qk.dtype)[:, None, :]
    sin = torch.cat((cs[:, D // 2:], cs[:, D // 2:]), -1).to(qk.dtype)[:, None, :]
    x1, x2 = qk[..., : D // 2], qk[..., D // 2:]
    rot = torch.cat((-x2, x1), -1)
    return qk * cos + rot * sin


def silu_mul(x: torch.Tensor) -> torch.Tensor:
    I = x.shape[-1] // 2
    return torch.nn.functional.silu(x[..., :I]) * x[..., I:]


def gemm(x: torch.Tensor, w: torch.Tensor, bias=None) -> torch.Tensor:
    y = x.float() @ w.float().t()
    if bias is not None:
        y = y + bias.float()
    return y


def attention(q, k, v, scale, causal_offset=None):
    """q: [Tq, nq, D], k/v: [Tk, nkv, D]; fp32 softmax(QK^T)V with GQA head sharing.
    causal_offset: query row i sees keys 0..causal_offset+i (None = all keys)."""
    Tq, nq, D = q.shape
    Tk, nkv, _ = k.shape
    g = nq // nkv
    qf = q.float().permute(1, 0, 2)
    kf = k.float().permute(1, 0, 2).repeat_interleave(g, 0)
    vf = v.float().permute(1, 0, 2).repeat_interleave(g, 0)
    s = torch.einsum("hqd,hkd->hqk", qf, kf) * scale
    if causal_offset is not None:
        qi = torch.arange(Tq, device=q.device)[:, None] + causal_offset
        ki = torch.arange(Tk, device=q.device)[None, :]
        s = s.masked_fill(ki > qi, float("-inf"))
    p = torch.softmax(s, -1)
    return torch.einsum("hqk,hkd->hqd", p, vf).permute(1, 0, 2)


def argmax_first(logits: torch.Tensor):
    """(max value, lowest index holding it) per row"""
    v = logits.float()
    mx = v.max(-1, keepdim=True).values
    idx = torch.where(v == mx, torch.arange(v.shape[-1], device=v.device)[None, :], v.shape[-1]).min(-1).values
    return mx[:, 0], idx
