"""The entry point for callers that cannot allocate device memory.

Some hosts of the library (a process whose device memory already belongs to another pool,
a plug-in barred from the CUDA allocator, a latency-critical loop) cannot hand over a
workspace.  ``ma_b200_forward_static_scratch`` keeps the stage-to-stage state in a fixed
array inside the library instead.  This test calls it through the C ABI twice in a row -
the second call finds the first call's leftovers in the shared array - and checks both
results against the ordinary entry point on the same inputs (the generic kernels with a caller-owned
workspace, which tests/test_parity_gpu.py pins to the oracle and the reference's golden outputs on
these very cases).  The file name sorts last so
that a run stopping at the first failure has already exercised everything else.
"""
import ctypes as C

import pytest
import torch

from helpers import CASES_BY_NAME, check_close, make_inputs

pytestmark = pytest.mark.gpu


def _forward_both(lib, _cabi, make_problem, case_name, dev):
    case = CASES_BY_NAME[case_name]
    q, k, v, mask = make_inputs(case)
    q, k, v = q.to(dev), k.to(dev), v.to(dev)
    m8 = None if mask is None else (mask != 0).to(torch.uint8).to(dev)
    stream = torch.cuda.current_stream().cuda_stream

    want = torch.empty_like(v)
    prob = make_problem(q, k, v, want, m8, case["T"], case["B"], case["pre_pad"], _cabi.KERNEL_GENERIC)
    ws = torch.empty(lib.ma_b200_workspace_bytes(C.byref(prob)), dtype=torch.uint8, device=dev)
    _cabi.raise_for_status(lib.ma_b200_forward(C.byref(prob), ws.data_ptr(), ws.numel(), stream))

    got = torch.full_like(v, float("nan"))
    prob2 = make_problem(q, k, v, got, m8, case["T"], case["B"], case["pre_pad"])
    rc = lib.ma_b200_forward_static_scratch(C.byref(prob2), stream)
    assert rc == _cabi.OK, lib.ma_b200_static_scratch_last_error().decode()
    torch.cuda.synchronize()
    return got, want, case


def test_static_scratch_entry_matches_workspace_entry_twice_in_a_row():
    from monarch_attention_b200 import _cabi
    from monarch_attention_b200.monarch_attention import make_problem
    lib = _cabi.load()
    dev = torch.device("cuda:0")
    assert lib.ma_b200_static_scratch_bytes() == 8 << 20
    # two different problems back to back: masked bf16 with padding, then fp32 with three iterations
    for name in ("cfg2_vit225_bf16", "cfg1_f32_t3"):
        got, want, case = _forward_both(lib, _cabi, make_problem, name, dev)
        check_close(got.double().cpu().numpy(), want.double().cpu().numpy(), case["vdtype"],
                    f"static-scratch entry vs workspace entry, {name}")
        assert torch.equal(got, want)


def test_static_scratch_entry_refuses_oversized_problems():
    from monarch_attention_b200 import _cabi
    from monarch_attention_b200.monarch_attention import make_problem
    lib = _cabi.load()
    dev = torch.device("cuda:0")
    q = torch.zeros(1, 16, 16384, 64, dtype=torch.bfloat16, device=dev)   # needs ~100 MB of state
    out = torch.empty_like(q)
    prob = make_problem(q, q, q, out, None, 2, 128, False)
    rc = lib.ma_b200_forward_static_scratch(C.byref(prob), torch.cuda.current_stream().cuda_stream)
    assert rc == _cabi.WORKSPACE_TOO_SMALL
    assert "static scratch holds" in lib.ma_b200_static_scratch_last_error().decode()
    assert lib.ma_b200_forward_static_scratch(None, None) == _cabi.INVALID_ARGUMENT
