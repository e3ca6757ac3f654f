"""Forward pass on HOST tensors, with the PCIe copies overlapped with the kernels.

The reference module is handed device tensors by its callers (reference:
ma/monarch_attention.py:50-59); a caller whose q, k, v live in host memory pays
host-to-device and device-to-host copies around the call, and for the long-sequence
workloads those copies, not the kernels, are the time.  ``monarch_attention_b200_host``
binds the library's ``ma_b200_forward_host``, which cuts the (batch, head) pairs into chunks
of a few heads and pipelines H2D, kernels and D2H over three streams (see
``csrc/ma_host.cu``); this module only provides the device scratch and the pointers.
"""
from __future__ import annotations

import ctypes as C

import torch
from torch import Tensor

from . import _cabi
from .monarch_attention import _check_device_free_inputs, make_problem

_scratch: dict[int, Tensor] = {}


def plan_chunks(E: int, H: int, heads_per_chunk: int) -> list[tuple[int, int, int]]:
    """(batch index, first head, number of heads) of every chunk, in the order the library runs them."""
    if E < 0 or H < 0:
        raise ValueError("E and H must be non-negative")
    if heads_per_chunk < 1:
        raise ValueError("heads_per_chunk must be at least 1")
    out = []
    for e in range(E):
        h0 = 0
        while h0 < H:
            left = H - h0
            nh = min(heads_per_chunk, left)
            if e == E - 1 and nh > 1 and nh > left // 2:   # the last batch element tapers off
                nh = max(1, left // 2)
            out.append((e, h0, nh))
            h0 += nh
    return out


def monarch_attention_b200_host(q: Tensor, k: Tensor, v: Tensor, attn_mask: Tensor | None, T: int, B: int,
                                pre_pad: bool, *, out: Tensor | None = None, device=None,
                                heads_per_chunk: int = 8, wait: bool = True, streamed: bool = False,
                                kernel: int = _cabi.KERNEL_AUTO) -> Tensor:
    """Same computation as ``monarch_attention_b200`` for q, k, v (and the result) in host memory.

    q, k, v: CPU tensors (E, H, N, D) / (E, H, N, Dv) with unit inner stride; pinned for overlap.
    out:     optional CPU tensor (E, H, N, Dv) to receive the result (pinned for overlap).
    device:  CUDA device to run on (default: the current one).
    heads_per_chunk: heads per pipeline chunk (the last chunks are smaller: each at most half of what is
             left); 8 measured best for 16 heads of N = 16384 (2.20 ms per call against 2.60 ms unpipelined;
             4 gives 2.23 ms, 2 loses again to per-chunk start-up).
    wait:    block until the result is in ``out``; with ``wait=False`` the current stream has been made
             to wait for the last copy instead, and the caller synchronises it before reading ``out``
             (and keeps q, k, v, the mask and ``out`` alive until then).
    streamed: for a sequence of calls with ``wait=False`` whose host inputs are already valid when each call
             is made: the copy-in of a call starts while the kernels and the copy-out of the previous call
             are still running (``ma_b200_forward_host_streamed``), so that the host-to-device link never
             idles between calls.
    """
    _check_device_free_inputs(q, k, v, attn_mask)
    if q.is_cuda or k.is_cuda or v.is_cuda or (attn_mask is not None and attn_mask.is_cuda):
        raise ValueError("monarch_attention_b200_host takes host tensors; use monarch_attention_b200 for device ones")
    if heads_per_chunk < 1:
        raise ValueError("heads_per_chunk must be at least 1")
    E, H, N, _ = q.shape
    Dv = v.shape[-1]
    if out is None:
        out = torch.empty((E, H, N, Dv), dtype=v.dtype, pin_memory=True)
    elif out.is_cuda or tuple(out.shape) != (E, H, N, Dv) or out.dtype != v.dtype or out.stride(-1) != 1:
        raise ValueError("out must be a host tensor of shape (E, H, N, Dv), value's dtype and unit inner stride")
    if E == 0 or H == 0 or N == 0:
        return out
    lib = _cabi.load()
    q, k, v = (t if t.stride(-1) == 1 else t.contiguous() for t in (q, k, v))
    mask = None
    if attn_mask is not None:
        mask = attn_mask.view(torch.uint8) if attn_mask.dtype == torch.bool else (attn_mask != 0).view(torch.uint8)
        mask = mask if mask.stride(-1) == 1 else mask.contiguous()
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    prob = make_problem(q, k, v, out, mask, T, B, pre_pad, kernel)
    with torch.cuda.device(device):
        need = lib.ma_b200_host_scratch_bytes(C.byref(prob), heads_per_chunk)
        if need == 0:
            raise ValueError(lib.ma_b200_host_last_error().decode())
        idx = device.index if device.index is not None else torch.cuda.current_device()
        scratch = _scratch.get(idx)
        if scratch is None or scratch.numel() < need:
            torch.cuda.synchronize(device)  # an earlier call may still be using the old scratch
            scratch = _scratch[idx] = torch.empty(need, dtype=torch.uint8, device=device)
        stream = torch.cuda.current_stream(device)
        entry = lib.ma_b200_forward_host_streamed if streamed else lib.ma_b200_forward_host
        rc = entry(C.byref(prob), heads_per_chunk, scratch.data_ptr(), scratch.numel(), stream.cuda_stream)
        if rc != 0:
            _cabi.raise_for_status(rc, lib.ma_b200_host_last_error().decode())
        if wait:
            stream.synchronize()
    return out
