"""The CPU oracle against the reference's own outputs (tests/golden) and against
known answers.  Runs without a GPU."""
import numpy as np
import pytest
import torch

from helpers import CASES, CASES_BY_NAME, bits_to_float, error_metrics, golden, golden_sample, make_inputs, sample_of
from oracle.monarch_oracle import (OracleState, algorithmic_bytes, algorithmic_flops, monarch_attention_dense_f64,
                                   monarch_attention_oracle, softmax_attention_f64)

SMALL = [c for c in CASES if c["E"] * c["H"] * c["N"] <= 2048]


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_oracle_matches_reference_bits(case):
    q, k, v, mask = make_inputs(case)
    g = golden()
    qsum = np.array([x.to(torch.float64).sum().item() for x in (q, k, v)])
    np.testing.assert_array_equal(qsum, g[f"{case['name']}/qsum"], err_msg="input generator drifted")
    out = monarch_attention_oracle(q, k, v, mask, case["T"], case["B"], case["pre_pad"])
    assert out.shape == (case["E"], case["H"], case["N"], case["Dv"])
    assert out.dtype == v.dtype
    np.testing.assert_array_equal(sample_of(out), golden_sample(case["name"]))
    o64 = out.to(torch.float64)
    sums = torch.stack([o64.sum(dim=(-1, -2)), (o64 * o64).sum(dim=(-1, -2))]).numpy()
    np.testing.assert_array_equal(sums, g[f"{case['name']}/sums"])


@pytest.mark.parametrize("case", SMALL, ids=[c["name"] for c in SMALL])
def test_dense_f64_agrees_with_oracle(case):
    q, k, v, mask = make_inputs(case)
    ref = monarch_attention_oracle(q, k, v, mask, case["T"], case["B"], case["pre_pad"])
    dense = monarch_attention_dense_f64(q.float().numpy(), k.float().numpy(), v.float().numpy(),
                                        None if mask is None else mask.numpy(),
                                        case["T"], case["B"], case["pre_pad"])
    _, _, fro = error_metrics(ref.to(torch.float64).numpy(), dense)
    limit = {"f32": 2e-5, "bf16": 4e-2, "f16": 8e-3}[case["dtype"]]
    assert fro <= limit, (case["name"], fro)


def test_one_block_is_softmax_attention():
    # T=1 and a single block that holds every token: the Monarch matrix is the
    # dense softmax matrix (up to the eps in the denominator).
    for name in ("edge_one_block_softmax_f32", "edge_one_block_prepad_f32"):
        case = CASES_BY_NAME[name]
        q, k, v, _ = make_inputs(case)
        out = monarch_attention_oracle(q, k, v, None, 1, case["B"], case["pre_pad"])
        want = softmax_attention_f64(q.numpy(), k.numpy(), v.numpy())
        assert np.abs(out.numpy() - want).max() < 1e-5


def test_matrix_rows_sum_to_one():
    case = CASES_BY_NAME["edge_matrix_f32"]
    q, k, v, _ = make_inputs(case)
    a = monarch_attention_oracle(q, k, v, None, case["T"], case["B"], case["pre_pad"])
    assert a.shape[-1] == a.shape[-2]
    assert torch.allclose(a.sum(-1), torch.ones(a.shape[:-1]), atol=1e-5)
    assert (a >= 0).all()


def test_fully_masked_block_is_finite_and_state_shapes():
    case = CASES_BY_NAME["edge_full_block_masked_f32"]
    q, k, v, mask = make_inputs(case)
    M = -(-case["N"] // case["B"])
    assert any((~mask[e].reshape(M, case["B"])).all(dim=1).any() for e in range(case["E"])), \
        "case must contain a fully masked block"
    st = OracleState()
    out = monarch_attention_oracle(q, k, v, mask, case["T"], case["B"], case["pre_pad"], state=st)
    assert torch.isfinite(out).all()
    E, H, B, D = case["E"], case["H"], case["B"], case["D"]
    assert st.al.shape == (E, H, B, M, D) and st.cl.shape == (E, H, B, M)
    assert st.ar.shape == (E, H, M, B, D) and st.cr.shape == (E, H, M, B)
    assert st.y.shape == (E, H, B, M, case["Dv"])


def test_head_permutation_equivariance():
    case = CASES_BY_NAME["ref_match_5"]
    q, k, v, _ = make_inputs(case)
    out = monarch_attention_oracle(q, k, v, None, case["T"], case["B"], case["pre_pad"])
    perm = torch.tensor([2, 0, 3, 1])
    out_p = monarch_attention_oracle(q[:, perm], k[:, perm], v[:, perm], None, case["T"], case["B"], case["pre_pad"])
    assert torch.equal(out[:, perm], out_p)


def test_work_model_matches_published_table():
    # FLOPs / bytes of the op-sweep configuration (E=1,H=16,D=64,T=2,bf16)
    assert abs(algorithmic_flops(1, 16, 4096, 64, 64, 64, 2) / 4.83e9 - 1) < 2e-3
    assert abs(algorithmic_flops(1, 16, 16384, 64, 64, 128, 2) / 3.865e10 - 1) < 2e-3
    assert abs(algorithmic_flops(1, 16, 65536, 64, 64, 256, 2) / 3.092e11 - 1) < 2e-3
    assert algorithmic_bytes(1, 16, 16384, 64, 64, 2) == 134217728
    assert abs(algorithmic_flops(2, 12, 256, 64, 64, 16, 1) / 6.29e7 - 1) < 2e-3
