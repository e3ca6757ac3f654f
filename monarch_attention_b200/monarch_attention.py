"""Host-side mirror of the reference's attention module for the B200 library.

Same constructor arguments, block size / iteration count meaning and the same
``forward(query, key, value[, attention_mask])`` shapes as the reference module
(reference: ma/monarch_attention.py:37-66), so the experiment models can construct
``MonarchAttention(config.block_size, config.num_steps, config.pad_type)`` and call
it unchanged (call sites: experiments/vit/model.py:97, experiments/roberta/model.py:104-106,
experiments/dit/attention_processor.py:143).

All arithmetic happens in the CUDA library behind the C ABI; PyTorch supplies device
memory and the current stream.  Inputs must live on a CUDA device: there is no CPU
path here.
"""
from __future__ import annotations

import ctypes as C
from collections.abc import Callable
from enum import StrEnum

import torch
import torch.nn as nn

from . import _cabi

Tensor = torch.Tensor
MonarchAttentionFn = Callable[[Tensor, Tensor, Tensor, "Tensor | None", int, int, bool], Tensor]

_DTYPE_CODE = {torch.float32: _cabi.F32, torch.bfloat16: _cabi.BF16, torch.float16: _cabi.F16}


class PadType(StrEnum):
    """Where the token axis is zero-padded to a multiple of the block size
    (reference: ma/monarch_attention.py:32-34)."""

    pre = "pre"
    post = "post"


# ---------------------------------------------------------------------------------
# Workspace cache: one scratch tensor per (device, stream), grown on demand.  It comes
# from PyTorch's caching allocator, so steady-state calls allocate nothing.
# ---------------------------------------------------------------------------------
_workspaces: dict[tuple[int, int], Tensor] = {}


def _workspace(device: torch.device, stream: int, nbytes: int) -> Tensor:
    key = (device.index if device.index is not None else torch.cuda.current_device(), stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def _tensor4(t: Tensor) -> _cabi.Tensor4:
    return _cabi.Tensor4(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2))


def _unit_inner(t: Tensor) -> Tensor:
    return t if t.stride(-1) == 1 or t.shape[-1] == 1 else t.contiguous()


def make_problem(q: Tensor, k: Tensor, v: Tensor, out: Tensor, mask: Tensor | None, T: int, B: int, pre_pad: bool,
                 kernel: int = _cabi.KERNEL_AUTO) -> _cabi.Problem:
    E, H, N, D = q.shape
    p = _cabi.Problem()
    p.abi_version = _cabi.ABI_VERSION
    p.E, p.H, p.N, p.D, p.Dv = E, H, N, D, v.shape[-1]
    p.block_size, p.num_steps, p.pre_pad = int(B), int(T), int(bool(pre_pad))
    p.qk_dtype, p.v_dtype = _DTYPE_CODE[q.dtype], _DTYPE_CODE[v.dtype]
    p.kernel = kernel
    p.q, p.k, p.v, p.out = _tensor4(q), _tensor4(k), _tensor4(v), _tensor4(out)
    if mask is not None:
        p.mask, p.mask_stride_e = mask.data_ptr(), mask.stride(0)
    else:
        p.mask, p.mask_stride_e = None, 0
    return p


def _check_inputs(q: Tensor, k: Tensor, v: Tensor, attn_mask: Tensor | None):
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError("query, key and value must have shape (batch, heads, tokens, width)")
    if not q.is_cuda:
        raise RuntimeError("monarch_attention_b200 runs on CUDA tensors only (there is no CPU path)")
    if k.device != q.device or v.device != q.device:
        raise ValueError("query, key and value must be on the same device")
    _check_device_free_inputs(q, k, v, attn_mask)


def _check_device_free_inputs(q: Tensor, k: Tensor, v: Tensor, attn_mask: Tensor | None):
    """Shape and dtype rules shared by the device and the host entry points."""
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError("query, key and value must have shape (batch, heads, tokens, width)")
    if k.shape != q.shape:
        raise ValueError(f"key shape {tuple(k.shape)} differs from query shape {tuple(q.shape)}")
    if v.shape[:3] != q.shape[:3]:
        raise ValueError(f"value shape {tuple(v.shape)} does not match query shape {tuple(q.shape)}")
    if q.dtype not in _DTYPE_CODE or v.dtype not in _DTYPE_CODE:
        raise ValueError(f"unsupported dtype {q.dtype} / {v.dtype}")
    if k.dtype != q.dtype:
        raise ValueError("query and key must have the same dtype")
    if attn_mask is not None and tuple(attn_mask.shape) != (q.shape[0], q.shape[2]):
        raise ValueError(f"attention_mask must have shape (batch, tokens) = {(q.shape[0], q.shape[2])}")


def _mask_bytes(attn_mask: Tensor | None, device) -> Tensor | None:
    """Any-dtype mask (non-zero = valid; reference: ma/ma_torch.py:96-98) -> uint8, unit inner stride."""
    if attn_mask is None:
        return None
    m = attn_mask.to(device)
    m = m.view(torch.uint8) if m.dtype == torch.bool else (m != 0).view(torch.uint8)
    return m if m.stride(-1) == 1 else m.contiguous()


def monarch_attention_b200(q: Tensor, k: Tensor, v: Tensor, attn_mask: Tensor | None, T: int, B: int, pre_pad: bool,
                           *, kernel: int = _cabi.KERNEL_AUTO, out: Tensor | None = None,
                           token_major_output: bool = False) -> Tensor:
    """Implementation function with the reference's registry signature
    (reference: ma/monarch_attention.py:11-19; computes what ma/ma_torch.py:65-108 computes).

    Returns a new (E, H, N, Dv) tensor of value's dtype on value's device.  With
    ``token_major_output`` the result is a (E, H, N, Dv) *view* of a (E, N, H, Dv) buffer, i.e. already
    in the layout the model adapters produce with ``permute(0, 2, 1, 3).contiguous()`` after the call
    (reference: experiments/vit/model.py:99-101), which then costs nothing.
    """
    _check_inputs(q, k, v, attn_mask)
    if torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad):
        # training: the kernels give the result, the gradients come from recomputation (backward.py)
        if out is not None:
            raise ValueError("out= cannot be combined with inputs that require a gradient")
        from .backward import MonarchAttentionFunction
        return MonarchAttentionFunction.apply(
            q, k, v, attn_mask, T, B, pre_pad,
            lambda a, b, c: monarch_attention_b200(a, b, c, attn_mask, T, B, pre_pad, kernel=kernel,
                                                   token_major_output=token_major_output))
    lib = _cabi.load()
    dev_index = q.device.index if q.device.index is not None else torch.cuda.current_device()
    # A bounded wait of an earlier asynchronous call on this device that gave up is reported here, at the
    # next call, without a synchronisation (the kernel leaves its code in mapped host memory).
    _cabi.raise_for_status(lib.ma_b200_poll_device_status(dev_index))
    q, k, v = _unit_inner(q), _unit_inner(k), _unit_inner(v)
    E, H, N, _ = q.shape
    if out is None:
        if token_major_output:
            out = torch.empty((E, N, H, v.shape[-1]), dtype=v.dtype, device=v.device).permute(0, 2, 1, 3)
        else:
            out = torch.empty((E, H, N, v.shape[-1]), dtype=v.dtype, device=v.device)
    mask = _mask_bytes(attn_mask, q.device)
    prob = make_problem(q, k, v, out, mask, T, B, pre_pad, kernel)
    with torch.cuda.device(q.device):
        need = lib.ma_b200_workspace_bytes(C.byref(prob))
        if need == 0:
            _cabi.raise_for_status(lib.ma_b200_workspace_layout_of(C.byref(prob), C.byref(_cabi.WorkspaceLayout())))
        stream = torch.cuda.current_stream(q.device).cuda_stream
        ws = _workspace(q.device, stream, need)
        rc = lib.ma_b200_forward(C.byref(prob), ws.data_ptr(), ws.numel(), stream)
    _cabi.raise_for_status(rc)
    return out


def _generic(q, k, v, m, T, B, pre_pad):
    return monarch_attention_b200(q, k, v, m, T, B, pre_pad, kernel=_cabi.KERNEL_GENERIC)


def _tcgen05(q, k, v, m, T, B, pre_pad):
    return monarch_attention_b200(q, k, v, m, T, B, pre_pad, kernel=_cabi.KERNEL_TCGEN05)


_IMPLEMENTATIONS: dict[str, MonarchAttentionFn] = {}


def register_impl(name: str, fn: MonarchAttentionFn) -> None:
    """Same registry hook as the reference (reference: ma/monarch_attention.py:15-19)."""
    _IMPLEMENTATIONS[name] = fn


register_impl("b200", monarch_attention_b200)
register_impl("b200-generic", _generic)
register_impl("b200-tcgen05", _tcgen05)
register_impl("b200-tcgen05-staged",
              lambda q, k, v, m, T, B, pp: monarch_attention_b200(q, k, v, m, T, B, pp, kernel=_cabi.KERNEL_TCGEN05_STAGED))
register_impl("b200-warp-mma",
              lambda q, k, v, m, T, B, pp: monarch_attention_b200(q, k, v, m, T, B, pp, kernel=_cabi.KERNEL_WARP_MMA))
register_impl("b200-head-fused",
              lambda q, k, v, m, T, B, pp: monarch_attention_b200(q, k, v, m, T, B, pp, kernel=_cabi.KERNEL_HEAD_FUSED))


class MonarchAttention(nn.Module):
    """Drop-in for the reference module (reference: ma/monarch_attention.py:37-66).

    ``impl`` selects the kernel family: "b200" (default: fused tensor-core kernel when the
    problem fits it, otherwise the generic path), "b200-generic", "b200-tcgen05" (fused, one
    launch), "b200-tcgen05-staged" (same kernel, one launch per stage),
    "b200-warp-mma" (warp-level tensor-core kernels for small blocks) or
    "b200-head-fused" (one CTA per head, one iteration, state in shared memory).  The reference's
    "torch" and "triton" implementations are not part of this library; asking for an
    unknown name raises ``ValueError`` exactly as the reference does.
    """

    def __init__(self, block_size, num_steps, pad_type, impl="b200"):
        super().__init__()
        self.block_size = block_size
        self.num_steps = num_steps
        self.pad_type = pad_type
        if impl not in _IMPLEMENTATIONS:
            available = ", ".join(sorted(_IMPLEMENTATIONS))
            raise ValueError(f"Unknown impl {impl!r}. Available: {available}")
        self._impl_fn = _IMPLEMENTATIONS[impl]
        # Set to True to get the result as a view of a (batch, tokens, heads, width) buffer (see
        # monarch_attention_b200); only the default implementation honours it.
        self.token_major_output = False

    def forward(self, query, key, value, attention_mask=None):
        if self.token_major_output and self._impl_fn is monarch_attention_b200:
            return monarch_attention_b200(query, key, value, attention_mask, self.num_steps, self.block_size,
                                          self.pad_type == PadType.pre, token_major_output=True)
        return self._impl_fn(query, key, value, attention_mask, self.num_steps, self.block_size,
                             self.pad_type == PadType.pre)

    def get_matrix(self, query, key, attention_mask=None):
        """Explicit (E, H, N, N) attention matrix: forward with V = identity
        (reference: ma/monarch_attention.py:61-66; fp32 identity, so an fp32 result)."""
        batch_size, num_heads, seq_len, _ = query.shape
        value = torch.eye(seq_len, device=query.device).expand(batch_size, num_heads, seq_len, seq_len)
        return self.forward(query, key, value, attention_mask)

    def extra_repr(self) -> str:
        return f"block_size={self.block_size}, num_steps={self.num_steps}, pad_type={str(self.pad_type)!r}"
