"""Generate tests/golden/golden.npz from the reference implementation itself.

Run where the reference is checked out (the machines that run the GPU tests do not
have it, which is why the vectors are committed):

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py --ref /path/to/reference

For every case in cases.py the script imports the reference's
``monarch_attention_torch`` (reference: ma/ma_torch.py:65) through its module
API (reference: ma/monarch_attention.py:37-59), runs it on the seeded CPU
inputs and stores

* ``<name>/out``   the output bits - all of them when the output has at most
                   2**17 elements, otherwise a fixed strided sample of 2**16
                   positions (16-bit dtypes are stored as their int16 bit
                   patterns);
* ``<name>/sums``  float64 per-(e,h) sums and sums of squares of the full output;
* ``<name>/qsum``  float64 sum of q, k, v (guards the input generator).

For the cases of ``GRAD_CASES`` it also differentiates the reference (autograd through its eager
implementation, the way the reference trains) with the seeded cotangent ``grad_weights(case)`` and stores
``<name>/out`` and ``<name>/dq``, ``<name>/dk``, ``<name>/dv`` (bit patterns; all elements of a small
tensor, a fixed strided sample of 2**14 positions of a large one).
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from cases import CASES, GRAD_CASES, grad_weights, make_inputs  # noqa: E402

FULL_LIMIT = 1 << 17
SAMPLE = 1 << 16


def to_bits(t: torch.Tensor) -> np.ndarray:
    t = t.contiguous()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.int16).numpy()
    return t.numpy()


def sample_positions(numel: int) -> np.ndarray:
    if numel <= FULL_LIMIT:
        return np.arange(numel)
    step = numel / SAMPLE
    return (np.arange(SAMPLE) * step).astype(np.int64)


def grad_sample_positions(numel: int) -> np.ndarray:
    """All positions of a small tensor, a fixed strided sample of 2**14 of a large one."""
    if numel <= (1 << 15):
        return np.arange(numel)
    return (np.arange(1 << 14) * (numel / (1 << 14))).astype(np.int64)


def summarize(out: torch.Tensor) -> dict:
    flat = to_bits(out).reshape(-1)
    o64 = out.to(torch.float64)
    sums = torch.stack([o64.sum(dim=(-1, -2)), (o64 * o64).sum(dim=(-1, -2))]).numpy()
    return {"out": flat[sample_positions(flat.size)], "sums": sums}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True, help="checkout of the reference repository")
    ap.add_argument("--out", default=os.path.join(HERE, "golden.npz"))
    args = ap.parse_args()
    sys.dont_write_bytecode = True
    sys.path.insert(0, args.ref)
    from ma.monarch_attention import MonarchAttention  # the reference module API

    torch.set_num_threads(os.cpu_count() or 1)
    blob = {}
    for case in CASES:
        q, k, v, mask = make_inputs(case)
        mod = MonarchAttention(case["B"], case["T"], "pre" if case["pre_pad"] else "post", impl="torch")
        with torch.no_grad():
            out = mod(q, k, v, mask)
        assert out.shape == (case["E"], case["H"], case["N"], case["Dv"]), out.shape
        assert not torch.isnan(out.float()).any(), case["name"]
        for key, val in summarize(out).items():
            blob[f"{case['name']}/{key}"] = val
        blob[f"{case['name']}/qsum"] = np.array(
            [x.to(torch.float64).sum().item() for x in (q, k, v)], dtype=np.float64)
        print(f"{case['name']:36s} out {tuple(out.shape)} {out.dtype}")
    for case in GRAD_CASES:
        q, k, v, mask = make_inputs(case)
        q, k, v = (t.requires_grad_(True) for t in (q, k, v))
        mod = MonarchAttention(case["B"], case["T"], "pre" if case["pre_pad"] else "post", impl="torch")
        out = mod(q, k, v, mask)
        out.backward(grad_weights(case).to(out.dtype))
        for key, t in (("out", out.detach()), ("dq", q.grad), ("dk", k.grad), ("dv", v.grad)):
            assert torch.isfinite(t.float()).all(), (case["name"], key)
            flat = to_bits(t).reshape(-1)
            blob[f"{case['name']}/{key}"] = flat[grad_sample_positions(flat.size)]
        print(f"{case['name']:36s} out {tuple(out.shape)} {out.dtype} + gradients")
    np.savez_compressed(args.out, **blob)
    print("wrote", args.out, os.path.getsize(args.out), "bytes")


if __name__ == "__main__":
    main()
