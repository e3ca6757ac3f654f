"""Seeded parity cases shared by the fixture generator, the oracle tests and the GPU tests.

Every case is a plain dict.  Inputs are drawn on the CPU from a per-case
``torch.Generator`` so that the CPU oracle and the GPU library see identical
bits.  Shapes come from three places:

* the reference's own test matrix (reference: ma/tests/test_ma.py:34-48,
  :70-80, :106-109, :125-133) - names ``ref_match_*``, ``ref_mask_*``,
  ``ref_t1_*``; inputs are unscaled ``randn`` as there;
* the five benchmark configurations, at full size where the CPU oracle
  finishes in seconds and scaled down in batch otherwise - names ``cfg*``;
* edge cases the reference's semantics define: fully masked key blocks,
  one surviving key, one block (plain softmax attention), value width
  different from the key width, value dtype different from the key dtype.
"""
from __future__ import annotations

import zlib

import torch

DTYPES = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}


def _c(name, E, H, N, D, B, T, pre_pad, dtype, *, Dv=None, mask=None, scale="unit", vdtype=None):
    return dict(name=name, E=E, H=H, N=N, D=D, Dv=D if Dv is None else Dv, B=B, T=T,
                pre_pad=bool(pre_pad), dtype=dtype, vdtype=vdtype or dtype, mask=mask, scale=scale)


def _ref_cases():
    out = []
    match = [
        (1, 1, 16, 16, 4, 2, False, "f16"), (1, 1, 16, 16, 4, 2, True, "f16"),
        (1, 4, 16, 16, 8, 3, False, "f16"), (1, 1, 19, 16, 4, 2, False, "f16"),
        (1, 1, 19, 16, 4, 2, True, "f16"), (2, 4, 32, 32, 8, 2, False, "f16"),
        (2, 1, 24, 16, 8, 3, False, "f16"), (2, 4, 16, 32, 4, 2, False, "bf16"),
        (1, 1, 16, 32, 4, 2, True, "bf16"), (1, 1, 24, 16, 8, 2, False, "bf16"),
    ]
    for i, (E, H, N, D, B, T, pp, dt) in enumerate(match):
        out.append(_c(f"ref_match_{i}", E, H, N, D, B, T, pp, dt))
    masked = [
        (1, 1, 16, 16, 4, 2, False, "f16"), (1, 1, 16, 16, 4, 2, True, "f16"),
        (1, 1, 19, 16, 4, 2, False, "f16"), (1, 4, 19, 16, 4, 3, True, "f16"),
        (1, 1, 32, 16, 8, 2, False, "f16"), (2, 4, 32, 32, 8, 2, False, "f16"),
        (1, 1, 16, 16, 4, 2, True, "bf16"), (2, 4, 16, 32, 4, 2, False, "bf16"),
    ]
    for i, (E, H, N, D, B, T, pp, dt) in enumerate(masked):
        out.append(_c(f"ref_mask_{i}", E, H, N, D, B, T, pp, dt, mask="block_safe"))
    t1 = [
        (1, 1, 16, 16, 4, False, "f16"), (2, 4, 19, 32, 8, True, "bf16"),
        (1, 1, 16, 16, 4, True, "f16"), (2, 4, 32, 32, 8, False, "f16"),
        (1, 1, 19, 16, 4, False, "f16"), (1, 1, 19, 16, 4, True, "f16"),
        (2, 4, 16, 32, 4, False, "bf16"),
    ]
    for i, (E, H, N, D, B, pp, dt) in enumerate(t1):
        out.append(_c(f"ref_t1_{i}", E, H, N, D, B, 1, pp, dt))
    # the same matrix in fp32, where the comparison is tight
    for i, (E, H, N, D, B, T, pp, dt) in enumerate(match[:7]):
        out.append(_c(f"ref_match_f32_{i}", E, H, N, D, B, T, pp, "f32"))
    for i, (E, H, N, D, B, T, pp, dt) in enumerate(masked[:6]):
        out.append(_c(f"ref_mask_f32_{i}", E, H, N, D, B, T, pp, "f32", mask="block_safe"))
    return out


def _config_cases():
    return [
        # config 1, full size
        _c("cfg1_f32", 2, 12, 256, 64, 16, 1, False, "f32", scale="rsqrt_d"),
        _c("cfg1_f32_t3", 2, 12, 256, 64, 16, 3, False, "f32", scale="rsqrt_d"),
        # config 2 (ViT): 197 tokens, b=15 -> 14 blocks; and the 225-token reading with 28 masked keys
        _c("cfg2_vit_bf16", 2, 12, 197, 64, 15, 1, True, "bf16", scale="activations"),
        _c("cfg2_vit_b14_bf16", 2, 12, 197, 64, 14, 2, True, "bf16", scale="activations"),
        _c("cfg2_vit225_bf16", 2, 12, 225, 64, 15, 1, True, "bf16", mask="tail28", scale="activations"),
        _c("cfg2_vit_f32", 1, 12, 197, 64, 15, 1, True, "f32", scale="activations"),
        # config 3 (op sweep), one or two heads of each size
        _c("cfg3_n4096_bf16", 1, 2, 4096, 64, 64, 2, False, "bf16", scale="rsqrt_d"),
        _c("cfg3_n16384_bf16", 1, 1, 16384, 64, 128, 2, False, "bf16", scale="rsqrt_d"),
        _c("cfg3_n4096_unit_bf16", 1, 2, 4096, 64, 64, 2, False, "bf16", scale="unit"),
        _c("cfg3_n16384_unit_bf16", 1, 1, 16384, 64, 128, 2, False, "bf16", scale="unit"),
        _c("cfg3_n4096_f16", 1, 1, 4096, 64, 64, 2, False, "f16", scale="unit"),
        _c("cfg3_n4096_f32", 1, 1, 4096, 64, 64, 2, False, "f32", scale="unit"),
        # the fused tensor-core kernel's other stage sequences (one iteration: no left-factor stage; three
        # and four: right-factor stages that read ar / cr), sharp logits, fp16 at block size 128, and head
        # counts that leave a partial last head group (12 heads in groups of 8; 33 heads of 4096 tokens)
        _c("cfg3_n16384_t1_bf16", 1, 1, 16384, 64, 128, 1, False, "bf16", scale="rsqrt_d"),
        _c("cfg3_n16384_t1_unit_bf16", 1, 1, 16384, 64, 128, 1, False, "bf16", scale="unit"),
        _c("cfg3_n16384_t3_bf16", 1, 1, 16384, 64, 128, 3, False, "bf16", scale="rsqrt_d"),
        _c("cfg3_n16384_t3_unit_bf16", 1, 1, 16384, 64, 128, 3, False, "bf16", scale="unit"),
        _c("cfg3_n16384_t4_bf16", 1, 1, 16384, 64, 128, 4, False, "bf16", scale="rsqrt_d"),
        _c("cfg3_n16384_t4_unit_bf16", 1, 1, 16384, 64, 128, 4, False, "bf16", scale="unit"),
        _c("cfg3_n16384_act_bf16", 1, 1, 16384, 64, 128, 2, False, "bf16", scale="activations"),
        _c("cfg3_n16384_t3_act_bf16", 1, 1, 16384, 64, 128, 3, False, "bf16", scale="activations"),
        _c("cfg3_n16384_unit_f16", 1, 1, 16384, 64, 128, 2, False, "f16", scale="unit"),
        _c("cfg3_n16384_t3_act_f16", 1, 1, 16384, 64, 128, 3, False, "f16", scale="activations"),
        _c("cfg3_n16384_e2h6_bf16", 2, 6, 16384, 64, 128, 2, False, "bf16", scale="rsqrt_d"),
        _c("cfg3_n4096_t1_bf16", 1, 2, 4096, 64, 64, 1, False, "bf16", scale="rsqrt_d"),
        _c("cfg3_n4096_t1_unit_bf16", 1, 2, 4096, 64, 64, 1, False, "bf16", scale="unit"),
        _c("cfg3_n4096_t3_bf16", 1, 2, 4096, 64, 64, 3, False, "bf16", scale="rsqrt_d"),
        _c("cfg3_n4096_t3_unit_bf16", 1, 2, 4096, 64, 64, 3, False, "bf16", scale="unit"),
        _c("cfg3_n4096_t4_unit_bf16", 1, 2, 4096, 64, 64, 4, False, "bf16", scale="unit"),
        _c("cfg3_n4096_act_bf16", 1, 2, 4096, 64, 64, 2, False, "bf16", scale="activations"),
        _c("cfg3_n4096_t3_act_f16", 1, 2, 4096, 64, 64, 3, False, "f16", scale="activations"),
        _c("cfg3_n4096_h33_bf16", 1, 33, 4096, 64, 64, 2, False, "bf16", scale="unit"),
        _c("cfg3_n65536_bf16", 1, 1, 65536, 64, 256, 2, False, "bf16", scale="activations"),
        _c("cfg3_n65536_unit_f16", 1, 1, 65536, 64, 256, 2, False, "f16", scale="unit"),
        # config 4 (RoBERTa): right padding produces fully masked key blocks
        _c("cfg4_roberta_bf16", 4, 12, 512, 64, 32, 1, False, "bf16", mask="right_pad", scale="activations"),
        _c("cfg4_roberta_t2_f32", 4, 2, 512, 64, 32, 2, False, "f32", mask="right_pad", scale="activations"),
        # config 5 (DiT): head width 72
        _c("cfg5_dit_bf16", 2, 4, 1024, 72, 32, 2, False, "bf16", scale="activations"),
        _c("cfg5_dit_f32", 1, 4, 1024, 72, 32, 2, False, "f32", scale="activations"),
    ]


def _edge_cases():
    return [
        _c("edge_one_block_softmax_f32", 1, 2, 24, 16, 32, 1, False, "f32"),
        _c("edge_one_block_prepad_f32", 1, 2, 24, 16, 32, 1, True, "f32"),
        _c("edge_dv_wider_f32", 1, 2, 40, 16, 8, 2, False, "f32", Dv=48),
        _c("edge_dv_narrow_bf16", 2, 2, 40, 32, 8, 2, True, "bf16", Dv=8),
        _c("edge_matrix_f32v_bf16", 1, 2, 36, 16, 6, 2, False, "bf16", Dv=36, vdtype="f32", scale="eye_v"),
        _c("edge_matrix_f32", 1, 2, 36, 16, 6, 2, True, "f32", Dv=36, scale="eye_v"),
        _c("edge_full_block_masked_f32", 2, 2, 64, 16, 8, 2, False, "f32", mask="right_pad_short"),
        _c("edge_full_block_masked_t3_bf16", 2, 2, 64, 32, 8, 3, True, "bf16", mask="right_pad_short"),
        _c("edge_single_key_f32", 1, 2, 32, 16, 8, 2, False, "f32", mask="single_key"),
        _c("edge_float_mask_f16", 2, 2, 48, 16, 8, 2, False, "f16", mask="float01"),
        _c("edge_int64_mask_bf16", 2, 2, 50, 16, 8, 2, True, "bf16", mask="int64"),
        _c("edge_b_gt_m_f32", 1, 3, 70, 24, 32, 2, False, "f32"),
        _c("edge_m_gt_b_f32", 1, 3, 70, 24, 4, 3, True, "f32"),
        _c("edge_odd_d_f32", 1, 2, 33, 20, 5, 2, False, "f32"),
        _c("edge_large_logits_f32", 1, 2, 64, 32, 8, 2, False, "f32", scale="large"),
        _c("edge_t4_f32", 1, 2, 64, 16, 8, 4, False, "f32"),
        _c("edge_b1_f32", 1, 1, 8, 16, 1, 2, False, "f32"),
        # block size and / or block count between 129 and 256, ragged, masked
        _c("edge_b200_m150_mask_bf16", 1, 2, 200 * 150 - 37, 64, 200, 2, True, "bf16", mask="block_safe"),
        _c("edge_b136_m40_f16", 2, 1, 136 * 40 - 5, 32, 136, 3, False, "f16", scale="rsqrt_d"),
        _c("edge_b24_m200_bf16", 1, 2, 24 * 200 - 3, 64, 24, 2, False, "bf16", mask="right_pad_short"),
        _c("edge_n1_f32", 1, 1, 1, 16, 4, 2, True, "f32"),
    ]


CASES = _ref_cases() + _config_cases() + _edge_cases()
CASES_BY_NAME = {c["name"]: c for c in CASES}
assert len(CASES_BY_NAME) == len(CASES)


def make_inputs(case):
    """(q, k, v, mask-or-None) on the CPU, deterministic in the case name."""
    g = torch.Generator(device="cpu")
    g.manual_seed(zlib.crc32(case["name"].encode()) & 0x7FFFFFFF)
    E, H, N, D, Dv, B = (case[x] for x in ("E", "H", "N", "D", "Dv", "B"))
    dt, vdt = DTYPES[case["dtype"]], DTYPES[case["vdtype"]]

    def draw(*shape):
        return torch.randn(*shape, generator=g, dtype=torch.float32)

    q, k, v = draw(E, H, N, D), draw(E, H, N, D), draw(E, H, N, Dv)
    sc = case["scale"]
    if sc == "rsqrt_d":
        q, k, v = q / D ** 0.5, k / D ** 0.5, v / D ** 0.5
    elif sc == "activations":   # stand-in for projected hidden states: O(1) logits, per-head offsets
        q = 1.5 * q + 0.3 * draw(E, H, 1, D)
        k = 1.5 * k + 0.3 * draw(E, H, 1, D)
    elif sc == "large":
        q, k = 4.0 * q, 4.0 * k
    elif sc == "eye_v":
        v = torch.eye(N, dtype=torch.float32).expand(E, H, N, N).contiguous()
    q, k, v = q.to(dt), k.to(dt), v.to(vdt)

    mk = case["mask"]
    mask = None
    if mk == "block_safe":      # reference: ma/tests/test_ma.py:18-29
        M = -(-N // B)
        mask = torch.rand(E, N, generator=g) > 0.3
        for e in range(E):
            for m in range(M):
                lo, hi = m * B, min(m * B + B, N)
                if not mask[e, lo:hi].any():
                    mask[e, lo] = True
    elif mk == "right_pad":     # a quarter of the sequences right-padded to a random length in [N/4, N]
        mask = torch.ones(E, N, dtype=torch.bool)
        n_short = max(1, E // 4)
        for e in range(n_short):
            ln = int(torch.randint(N // 4, N + 1, (1,), generator=g))
            mask[e, ln:] = False
    elif mk == "right_pad_short":   # first sequence keeps N/4+3 tokens: several fully masked blocks
        mask = torch.ones(E, N, dtype=torch.bool)
        mask[0, N // 4 + 3:] = False
    elif mk == "tail28":
        mask = torch.ones(E, N, dtype=torch.bool)
        mask[:, N - 28:] = False
    elif mk == "single_key":
        mask = torch.zeros(E, N, dtype=torch.bool)
        mask[:, ::B] = True
    elif mk == "float01":
        mask = (torch.rand(E, N, generator=g) > 0.4).to(torch.float32)
        mask[:, 0] = 1.0
    elif mk == "int64":
        mask = (torch.rand(E, N, generator=g) > 0.4).to(torch.int64)
        mask[:, -1] = 1
    return q, k, v, mask


# Cases whose gradients are stored (cotangent of the output = seeded weights): small enough for autograd through
# the reference on the CPU.  The reference trains through exactly this path (its eager implementation under
# autograd); the library's gradients are held to these.
GRAD_CASES = [
    _c("grad_f32_t2", 1, 2, 32, 16, 8, 2, False, "f32"),
    _c("grad_f32_mask_prepad_t3", 2, 2, 29, 16, 8, 3, True, "f32", mask="block_safe"),
    _c("grad_f32_t1_ragged", 1, 3, 50, 24, 16, 1, False, "f32"),
    _c("grad_bf16_t2", 1, 2, 64, 32, 8, 2, False, "bf16", scale="rsqrt_d"),
    _c("grad_f16_mask_t2", 2, 2, 48, 16, 8, 2, False, "f16", mask="block_safe", scale="rsqrt_d"),
    _c("grad_bf16_n4096_b64_t2", 1, 1, 4096, 64, 64, 2, False, "bf16", scale="rsqrt_d"),
]
GRAD_CASES_BY_NAME = {c["name"]: c for c in GRAD_CASES}


def grad_weights(case):
    """Seeded cotangent for the output of a case (float32, shape of the output)."""
    g = torch.Generator(device="cpu")
    g.manual_seed((zlib.crc32(case["name"].encode()) ^ 0x5bd1e995) & 0x7FFFFFFF)
    return torch.randn(case["E"], case["H"], case["N"], case["Dv"], generator=g, dtype=torch.float32)
