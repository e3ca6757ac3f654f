"""Host-side checks that need no GPU: the shared library loads and exports the declared
C ABI, argument validation, the module API's error behaviour, and the two-rank sharding
logic over gloo."""
import ctypes as C
import os
import re
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from monarch_attention_b200 import build, _cabi
    build.build()
    return _cabi.load()


def _problem(**kw):
    from monarch_attention_b200 import _cabi
    p = _cabi.Problem()
    p.abi_version = _cabi.ABI_VERSION
    p.E, p.H, p.N, p.D, p.Dv = 1, 2, 64, 16, 16
    p.block_size, p.num_steps, p.pre_pad = 8, 2, 0
    p.qk_dtype = p.v_dtype = _cabi.F32
    for k, v in kw.items():
        setattr(p, k, v)
    return p


def test_library_exports_every_declared_symbol(lib):
    header = open(os.path.join(ROOT, "include", "monarch_attention_b200.h")).read()
    declared = re.findall(r"MA_B200_API\s+[\w\s\*]+?\b(ma_b200_\w+)\s*\(", header)
    assert len(declared) >= 8
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    from monarch_attention_b200 import _cabi
    assert set(declared) == set(_cabi.EXPORTS)
    assert lib.ma_b200_abi_version() == 1


def test_status_strings(lib):
    seen = {lib.ma_b200_status_string(c).decode() for c in range(6)}
    assert len(seen) == 6 and "ok" in seen
    assert lib.ma_b200_status_string(99).decode() == "unknown status"


def test_workspace_layout_without_device(lib):
    from monarch_attention_b200 import _cabi
    p = _problem()
    L = _cabi.WorkspaceLayout()
    assert lib.ma_b200_workspace_layout_of(C.byref(p), C.byref(L)) == _cabi.OK
    assert L.M == 8 and L.kernel == _cabi.KERNEL_GENERIC
    assert L.status == 0 and L.ar % 256 == 0 and L.cr > L.ar and L.al > L.cr and L.cl > L.al and L.y > L.cl
    assert L.total == lib.ma_b200_workspace_bytes(C.byref(p))
    # ceil division for the block count, single step needs no left-factor state
    p2 = _problem(N=65, num_steps=1)
    assert lib.ma_b200_workspace_layout_of(C.byref(p2), C.byref(L)) == _cabi.OK
    assert L.M == 9 and L.ar == L.cr == L.al


@pytest.mark.parametrize("field,value", [("E", 0), ("N", -1), ("D", 0), ("block_size", 0), ("num_steps", 0),
                                         ("qk_dtype", 7), ("abi_version", 99), ("kernel", 5)])
def test_invalid_arguments_are_rejected(lib, field, value):
    from monarch_attention_b200 import _cabi
    p = _problem(**{field: value})
    assert lib.ma_b200_workspace_bytes(C.byref(p)) == 0
    assert lib.ma_b200_forward(C.byref(p), None, 0, None) == _cabi.INVALID_ARGUMENT
    assert lib.ma_b200_last_error().decode() != ""


def test_null_pointers_and_workspace_checks(lib):
    from monarch_attention_b200 import _cabi
    p = _problem()
    assert lib.ma_b200_forward(C.byref(p), None, 0, None) == _cabi.INVALID_ARGUMENT  # q is NULL
    assert lib.ma_b200_forward(None, None, 0, None) == _cabi.INVALID_ARGUMENT
    for t in (p.q, p.k, p.v, p.out):
        t.ptr, t.stride_e, t.stride_h, t.stride_n = 4096, 2048, 1024, 16
    assert lib.ma_b200_forward(C.byref(p), None, 0, None) == _cabi.INVALID_ARGUMENT  # workspace NULL
    assert lib.ma_b200_forward(C.byref(p), 4096 + 8, 1 << 30, None) == _cabi.INVALID_ARGUMENT  # misaligned
    assert lib.ma_b200_forward(C.byref(p), 4096, 16, None) == _cabi.WORKSPACE_TOO_SMALL
    p.q.ptr = 4097  # not aligned to 4 bytes
    assert lib.ma_b200_forward(C.byref(p), 4096, 1 << 30, None) == _cabi.INVALID_ARGUMENT
    p2 = _problem(qk_dtype=_cabi.F32, v_dtype=_cabi.BF16)
    assert lib.ma_b200_workspace_bytes(C.byref(p2)) == 0  # v narrower than q/k: unsupported
    p3 = _problem(kernel=_cabi.KERNEL_TCGEN05)
    L = _cabi.WorkspaceLayout()
    assert lib.ma_b200_workspace_layout_of(C.byref(p3), C.byref(L)) == _cabi.UNSUPPORTED


def test_module_api_mirrors_reference(lib):
    from monarch_attention_b200 import MonarchAttention, PadType
    m = MonarchAttention(16, 2, PadType.pre)
    assert (m.block_size, m.num_steps, m.pad_type) == (16, 2, "pre")
    assert list(m.parameters()) == [] and list(m.buffers()) == []
    assert PadType("post") is PadType.post and PadType.pre == "pre"
    with pytest.raises(ValueError, match="Unknown impl 'triton'. Available: "):
        MonarchAttention(16, 2, "pre", impl="triton")
    q = torch.zeros(1, 2, 32, 16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        m(q, q, q)
    with pytest.raises(ValueError):
        m(q[0], q[0], q[0])


def test_unit_range_partitions():
    from monarch_attention_b200.sharding import unit_range
    for total in (0, 1, 7, 16, 768):
        for world in (1, 2, 3, 4, 8):
            spans = [unit_range(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        unit_range(4, 4, 4)


_WORKER = r"""
import os, sys
sys.path.insert(0, {root!r}); sys.path.insert(0, os.path.join({root!r}, "tests", "golden"))
import torch, torch.distributed as dist
from cases import CASES_BY_NAME, make_inputs
from oracle.monarch_oracle import monarch_attention_oracle
from monarch_attention_b200.sharding import shard_heads, gather_to_rank0
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:{port}", rank=int(sys.argv[1]), world_size=2)
rank = dist.get_rank()
ok = True
for name in ("ref_match_5", "edge_b_gt_m_f32"):      # E=2 (split on batch), E=1,H=3 (flattened split)
    case = CASES_BY_NAME[name]
    q, k, v, _ = make_inputs(case)
    full = monarch_attention_oracle(q, k, v, None, case["T"], case["B"], case["pre_pad"])
    qs, ks, vs = shard_heads(q, k, v, rank, 2)
    part = monarch_attention_oracle(qs, ks, vs, None, case["T"], case["B"], case["pre_pad"])
    got = gather_to_rank0(part.reshape(-1, *part.shape[2:]))
    if rank == 0:
        joined = torch.cat(got, dim=0)
        ok &= torch.equal(joined, full.reshape(-1, *full.shape[2:]))
dist.barrier()
dist.destroy_process_group()
sys.exit(0 if ok else 1)
"""


def test_two_rank_sharding_over_gloo(tmp_path):
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    script = tmp_path / "worker.py"
    script.write_text(_WORKER.format(root=ROOT, port=port))
    procs = [subprocess.Popen([sys.executable, str(script), str(r)]) for r in range(2)]
    codes = [p.wait(timeout=240) for p in procs]
    assert codes == [0, 0]


def test_host_pipeline_chunk_plan():
    from monarch_attention_b200.host_pipeline import plan_chunks
    # full chunks, except that the last batch element tapers off (each chunk at most half of what is left)
    assert plan_chunks(2, 5, 2) == [(0, 0, 2), (0, 2, 2), (0, 4, 1), (1, 0, 2), (1, 2, 1), (1, 3, 1), (1, 4, 1)]
    assert plan_chunks(1, 3, 8) == [(0, 0, 1), (0, 1, 1), (0, 2, 1)]
    assert [n for _, _, n in plan_chunks(1, 16, 4)] == [4, 4, 4, 2, 1, 1]
    assert plan_chunks(0, 4, 2) == [] and plan_chunks(3, 0, 2) == []
    covered = sorted((e, h) for e, h0, n in plan_chunks(3, 7, 3) for h in range(h0, h0 + n))
    assert covered == [(e, h) for e in range(3) for h in range(7)]
    with pytest.raises(ValueError):
        plan_chunks(1, 4, 0)


def test_host_entry_rejects_bad_arguments_before_touching_a_gpu():
    import torch
    from monarch_attention_b200 import monarch_attention_b200_host
    q = torch.zeros(1, 2, 8, 16)
    with pytest.raises(ValueError):
        monarch_attention_b200_host(q, torch.zeros(1, 2, 9, 16), q, None, 1, 4, False)
    with pytest.raises(ValueError):
        monarch_attention_b200_host(q[0], q[0], q[0], None, 1, 4, False)


def test_host_scratch_size_is_host_arithmetic(lib):
    p = _problem(E=2, H=5, N=300, D=64, Dv=64, block_size=16, num_steps=2)
    one = lib.ma_b200_host_scratch_bytes(C.byref(p), 1)
    two = lib.ma_b200_host_scratch_bytes(C.byref(p), 2)
    big = lib.ma_b200_host_scratch_bytes(C.byref(p), 64)       # clamped to H
    five = lib.ma_b200_host_scratch_bytes(C.byref(p), 5)
    assert 0 < one < two < five == big
    # three slots of (q, k, v, result) for one head, at least
    assert one >= 3 * 4 * 300 * 64 * 4
    assert lib.ma_b200_host_scratch_bytes(C.byref(p), 0) == 0
    assert b"heads_per_chunk" in lib.ma_b200_host_last_error()
    # null host pointers are refused before any CUDA call
    assert lib.ma_b200_forward_host(C.byref(p), 2, None, 0, None) != 0


def test_caller_models_build_and_run_on_cpu():
    """The plain-PyTorch restatements of the three callers (ViT-B/16, RoBERTa-base encoder, DiT-XL/2) at
    reduced depth with a dense-attention stand-in: shapes and finiteness (no GPU involved)."""
    from monarch_attention_b200.models import DenseAttention, build_dit_xl2, build_roberta_base, build_vit_b16
    torch.manual_seed(0)
    with torch.no_grad():
        v = build_vit_b16(DenseAttention, dtype=torch.float32, device="cpu", depth=1)(torch.rand(1, 3, 224, 224))
        r = build_roberta_base(DenseAttention, dtype=torch.float32, device="cpu", depth=1)(
            torch.randint(3, 50265, (2, 32)), torch.ones(2, 32, dtype=torch.long))
        d = build_dit_xl2(DenseAttention, dtype=torch.float32, device="cpu", depth=1)(
            torch.randn(1, 4, 64, 64), torch.tensor([10]), torch.tensor([7]))
    assert v.shape == (1, 1000) and r.shape == (2, 32, 768) and d.shape == (1, 8, 64, 64)
    assert all(torch.isfinite(x).all() for x in (v, r, d))
