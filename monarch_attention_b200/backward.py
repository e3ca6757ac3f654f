"""Gradients for the forward kernels, by recomputation.

The reference trains through autograd of its eager implementation (reference:
ma/ma_torch.py:10-108; experiments/bart fine-tunes through it).  This module gives the CUDA forward the
same gradients without hand-written backward kernels: the forward pass is the library's kernels, and the
backward pass recomputes the forward ON THE SAME DEVICE with differentiable tensor operations that follow the
reference's four stage functions operation for operation (same rounding points, same epsilons and clamps),
and differentiates that graph.  It costs one eager forward plus its backward per call and the memory
of the block score tensors (E*H*N*(B + M) floats per stage); it is the training path, not the hot path.

Nothing here runs unless an input requires a gradient.
"""
from __future__ import annotations

import math

import torch
from torch import Tensor

_EPS = 1e-12  # reference: ma/ma_torch.py:10 (default eps of both right-factor stages)


def _blocked(x: Tensor, M: int, B: int, pre_pad: bool) -> Tensor:
    """Zero-pad the token axis to M*B (front or back) and view it as (M, B) (reference: ma/ma_torch.py:81-86)."""
    E, H, N, W = x.shape
    gap = M * B - N
    if gap:
        x = torch.nn.functional.pad(x, (0, 0, gap, 0) if pre_pad else (0, 0, 0, gap))
    return x.reshape(E, H, M, B, W)


def _validity(E: int, N: int, M: int, B: int, pre_pad: bool, attn_mask: Tensor | None, device) -> Tensor:
    """(M, B) or (E, 1, M, B) booleans: the position holds a real, un-masked token (reference: ma/ma_torch.py:92-98)."""
    gap = M * B - N
    pos = torch.arange(M * B, device=device).reshape(M, B)
    ok = pos >= gap if pre_pad else pos < N
    if attn_mask is not None:
        am = attn_mask.to(device) != 0
        if gap:
            am = torch.nn.functional.pad(am, (gap, 0) if pre_pad else (0, gap))
        ok = ok & am.reshape(E, 1, M, B)
    return ok


def _right(ar: Tensor, k: Tensor, cr: Tensor, sm_scale: float, key_ok: Tensor, v: Tensor | None):
    """Right-factor update of every key block (reference: ma/ma_torch.py:10-23, with v: :38-52)."""
    x = sm_scale * torch.matmul(ar, k.transpose(-1, -2)).to(torch.float32)
    x = x / (cr.unsqueeze(-1) + _EPS)
    x = x + torch.where(key_ok.unsqueeze(-2), 0.0, -math.inf)
    top = torch.clamp(x.amax(dim=-1, keepdim=True), min=_EPS)
    e = torch.exp(x - top)
    r = e / (e.sum(dim=-1, keepdim=True) + _EPS)
    r = torch.clamp(r, min=torch.finfo(r.dtype).tiny)
    cl = torch.special.xlogy(r, r).sum(dim=-1).transpose(-1, -2)
    al = sm_scale * torch.matmul(r.to(k.dtype), k).transpose(-2, -3)
    y = None if v is None else torch.matmul(r.to(v.dtype), v).transpose(-2, -3)
    return al, cl, y


def _left(al: Tensor, q_cols: Tensor, cl: Tensor, query_ok_cols: Tensor):
    """Left-factor update of every column (reference: ma/ma_torch.py:26-35)."""
    w = torch.matmul(al, q_cols.transpose(-1, -2)).to(torch.float32) - cl.unsqueeze(-1)
    lw = query_ok_cols.unsqueeze(-2) * torch.softmax(w, dim=-2)
    cr = lw.sum(dim=-1).transpose(-1, -2)
    ar = torch.matmul(lw.to(q_cols.dtype), q_cols).transpose(-2, -3)
    return ar, cr


def _output(al: Tensor, q_cols: Tensor, cl: Tensor, y: Tensor) -> Tensor:
    """Output stage (reference: ma/ma_torch.py:55-62)."""
    w = torch.matmul(q_cols, al.transpose(-1, -2)).to(torch.float32) - cl.unsqueeze(-2)
    return torch.matmul(torch.softmax(w, dim=-1).to(y.dtype), y).transpose(-2, -3)


def differentiable_forward(q: Tensor, k: Tensor, v: Tensor, attn_mask: Tensor | None, T: int, B: int,
                           pre_pad: bool) -> Tensor:
    """The forward pass in differentiable tensor operations on the inputs' device (reference: ma/ma_torch.py:65-108)."""
    E, H, N, D = q.shape
    M = -(-N // B)
    sm_scale = 1 / math.sqrt(D)
    qb, kb, vb = (_blocked(t, M, B, pre_pad) for t in (q, k, v))
    ok = _validity(E, N, M, B, pre_pad, attn_mask, q.device)
    ar, cr = qb, torch.ones(E, H, M, B, dtype=torch.float32, device=q.device)
    q_cols = qb.transpose(-2, -3)
    for _ in range(T - 1):
        al, cl, _ = _right(ar, kb, cr, sm_scale, ok, None)
        ar, cr = _left(al, q_cols, cl, ok.mT)
    al, cl, y = _right(ar, kb, cr, sm_scale, ok, vb)
    z = _output(al, q_cols, cl, y).reshape(E, H, M * B, v.shape[-1])
    gap = M * B - N
    return z[..., gap:, :] if pre_pad else z[..., :N, :]


class MonarchAttentionFunction(torch.autograd.Function):
    """forward: the library's kernels; backward: autograd through ``differentiable_forward``."""

    @staticmethod
    def forward(ctx, q, k, v, attn_mask, T, B, pre_pad, run_kernels):
        ctx.save_for_backward(q, k, v)
        ctx.attn_mask, ctx.T, ctx.B, ctx.pre_pad = attn_mask, T, B, pre_pad
        return run_kernels(q.detach(), k.detach(), v.detach())

    @staticmethod
    def backward(ctx, grad_out):
        q, k, v = ctx.saved_tensors
        needs = ctx.needs_input_grad[:3]
        with torch.enable_grad():
            leaves = [t.detach().requires_grad_(need) for t, need in zip((q, k, v), needs)]
            z = differentiable_forward(*leaves, ctx.attn_mask, ctx.T, ctx.B, ctx.pre_pad)
            wanted = [t for t, need in zip(leaves, needs) if need]
            grads = iter(torch.autograd.grad(z, wanted, grad_out.to(z.dtype)))
        return tuple(next(grads) if need else None for need in needs) + (None,) * 5
