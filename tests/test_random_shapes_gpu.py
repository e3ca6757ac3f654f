"""Seeded random shapes: the warp-level tensor-core kernels (and the one-CTA-per-head kernel where it
applies) against the CPU oracle and against the generic kernels.
Covers what a fixed case list does not: every tile-size template, ragged last blocks, block sizes and
counts on both sides of 16 / 32 / 64 / 128, masks that empty whole key blocks, both padding sides."""
import random

import pytest
import torch

pytestmark = pytest.mark.gpu

BLOCKS = [1, 3, 7, 8, 15, 16, 17, 24, 31, 32, 33, 48, 64, 65, 100, 128, 129, 160, 200, 256]
COUNTS = [1, 2, 5, 14, 16, 17, 31, 32, 33, 60, 64, 65, 127, 128, 129, 150, 256]


def _draw(seed):
    rng = random.Random(seed)
    dt = rng.choice([torch.bfloat16, torch.float16])
    B, M = rng.choice(BLOCKS), rng.choice(COUNTS)
    if B * M > 40000:
        M = max(1, 40000 // B)
    D = rng.choice([8, 16, 32, 40, 64, 72, 80])
    if max(B, M) > 128 and D > 64:
        D = 64
    N = max(1, B * M - rng.randrange(0, B))
    E, H = rng.choice([(1, 1), (2, 3), (1, 4), (3, 2)])
    T = rng.choice([1, 1, 2, 2, 3])
    return dict(dt=dt, B=B, D=D, N=N, E=E, H=H, T=T, pre=rng.random() < 0.5,
                mask=rng.choice(["none", "none", "rand", "tail", "blocks"]), scale=rng.choice([1.0, 0.35, 2.0]))


@pytest.mark.parametrize("seed", range(64))
def test_warp_level_kernels_agree_with_generic_kernels(seed):
    import monarch_attention_b200 as ma
    c = _draw(seed)
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(seed * 7919 + 13)
    E, H, N, D, B, T = (c[x] for x in "EHNDBT")
    q, k, v = ((c["scale"] * torch.randn(E, H, N, D, generator=g)).to(c["dt"]).to(dev) for _ in range(3))
    mask = None
    if c["mask"] == "rand":
        mask = torch.rand(E, N, generator=g) > 0.3
        mask[:, 0] = True
    elif c["mask"] == "tail":
        mask = torch.ones(E, N, dtype=torch.bool)
        mask[0, N // 3 + 1:] = False
    elif c["mask"] == "blocks":           # every third key block fully masked
        mask = torch.ones(E, N, dtype=torch.bool)
        for m in range(0, -(-N // B), 3):
            mask[:, m * B:(m + 1) * B] = False
        mask[:, 0] = True
    md = None if mask is None else mask.to(dev)
    pad = "pre" if c["pre"] else "post"
    ref = ma.MonarchAttention(B, T, pad, impl="b200-generic")(q, k, v, md).float()
    out = ma.MonarchAttention(B, T, pad, impl="b200-warp-mma")(q, k, v, md).float()
    torch.cuda.synchronize()
    what = f"seed {seed}: {c}"
    assert torch.isfinite(out).all(), what
    scale = max(1.0, ref.abs().max().item())
    tol = 2e-2 if c["dt"] == torch.bfloat16 else 1e-2
    # Both sides are 16-bit pipelines that round at the same places but sum in different orders, so a
    # logit now and then lands on the other side of a rounding boundary; with sharp softmaxes and several
    # iterations one such flip moves a single output by a few ulp of its magnitude (the generic kernels
    # show the same against the CPU oracle).  Hence: the bound may be exceeded by isolated elements only,
    # never by more than a few ulp, and the Frobenius error stays small.
    diff = (out - ref).abs()
    assert (diff > tol * scale).float().mean().item() <= 1e-5, what
    assert diff.max().item() <= 4 * tol * scale, what
    assert (diff.norm() / ref.norm().clamp_min(1e-30)).item() <= 1e-2, what
    # and against the CPU oracle itself (relative Frobenius: the tolerance of the fixed parity cases)
    from oracle.monarch_oracle import monarch_attention_oracle
    want = monarch_attention_oracle(q.cpu(), k.cpu(), v.cpu(), mask, T, B, c["pre"]).float()
    fro = ((out.cpu() - want).norm() / want.norm().clamp_min(1e-30)).item()
    assert fro <= (1e-2 if c["dt"] == torch.bfloat16 else 4e-3), f"{what}: vs oracle {fro:.3e}"
    M = -(-N // B)
    if T == 1 and B <= 32 and M <= 32 and D <= 64:
        try:
            one = ma.MonarchAttention(B, T, pad, impl="b200-head-fused")(q, k, v, md).float()
        except ValueError:
            return                          # the head does not fit in shared memory
        torch.cuda.synchronize()
        d1 = (one - out).abs()
        assert (d1 > tol * scale).float().mean().item() <= 1e-5 and d1.max().item() <= 4 * tol * scale, what
