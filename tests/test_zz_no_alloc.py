"""iree_uk_b200_mmt4d_static_scratch: the mmt4d entry point for callers that cannot allocate.

IREE emits ukernel calls inside dispatches whose buffers were all planned by the compiler;
the call site has no allocator and may not call cudaMalloc, so it can hand the library
neither a workspace nor the means to make one. This entry point keeps the re-tiled operands
in a 32 MiB array inside the library instead. The test drives it through the C ABI twice in
a row — the second problem has another shape, so leftovers of the first call in the shared
array would show — and compares each result with what iree_uk_b200_mmt4d_ws gives for the
same inputs with caller-owned scratch: identical bytes for s8s8s32, relative Frobenius
error <= 1e-3 for bf16 (the tolerances of the parity tests). It also checks that a problem
too large for the array is refused and leaves the output untouched.

This file sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import numpy as np
import pytest
import torch

from iree_b200 import abi
from iree_b200 import ukernel as uk
from oracle import cases

import gpu_util as G

pytestmark = pytest.mark.gpu


def _run_both(case):
    lhs, rhs = G.to_device(case.lhs), G.to_device(case.rhs)
    out_a, out_b = G.to_device(case.out_init), G.to_device(case.out_init)
    pa = case.params(lhs.data_ptr(), rhs.data_ptr(), out_a.data_ptr())
    pb = case.params(lhs.data_ptr(), rhs.data_ptr(), out_b.data_ptr())
    need = uk.mmt4d_workspace_size(pa)
    assert 0 < need <= uk.STATIC_SCRATCH_BYTES
    uk.mmt4d_static_scratch(pa)
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    assert uk.mmt4d_path(pb, True) == abi.PATH_TCGEN05_RETILE
    uk.mmt4d(pb, workspace=ws)
    torch.cuda.synchronize()
    return out_a.cpu().numpy(), out_b.cpu().numpy()


def test_static_scratch_matches_workspace_entry_point_twice_in_a_row():
    first = cases.Mmt4dCase(abi.MMT4D_S8S8S32, 16, 16, 2, 24, 40, 200, 1, seed=21, loose=False)
    second = cases.Mmt4dCase(abi.MMT4D_BF16BF16F32, 16, 16, 2, 9, 17, 65, 0, seed=22,
                             mode="normal", loose=False)
    got, want = _run_both(first)
    assert np.array_equal(got, want)
    got, want = _run_both(second)
    assert cases.rel_frobenius(got.view(np.float32), want.view(np.float32)) <= 1e-3
    # and the first problem once more, after the array held the second one's operands
    got, want = _run_both(first)
    assert np.array_equal(got, want)
    G.check_device_status()


def test_static_scratch_runs_s16u4_with_many_rows_on_the_tensor_cores():
    """s16u4s32 1x32x8 with at least 16 rows is a scratch-using tensor-core problem for
    iree_uk_b200_mmt4d_ws, so it must be one here too (same kernel choice, same bytes), and a
    problem of that kind that does not fit the array must be refused."""
    case = cases.Mmt4dCase(abi.MMT4D_S16U4S32, 1, 32, 8, 200, 7, 33, 1, seed=24, mode="normal",
                           loose=False)
    for _ in range(2):
        got, want = _run_both(case)
        assert np.array_equal(got, want)
        assert np.array_equal(got, G.oracle_mmt4d(case))
    G.check_device_status()
    M, N, K = 4096, 448, 512  # 2 x 16 MiB byte planes + 56 MiB of widened weights
    lhs = torch.zeros(M * K * 8, dtype=torch.int16, device="cuda")
    rhs = torch.zeros(N * K * 128, dtype=torch.uint8, device="cuda")
    out = torch.full((M * N * 32,), 7, dtype=torch.int32, device="cuda")
    p = abi.Mmt4dParams()
    p.lhs_buffer, p.rhs_buffer, p.out_buffer = lhs.data_ptr(), rhs.data_ptr(), out.data_ptr()
    p.M, p.N, p.K, p.M0, p.N0, p.K0, p.flags = M, N, K, 1, 32, 8, abi.MMT4D_S16U4S32
    p.lhs_stride0, p.rhs_stride0, p.out_stride0 = K * 8, K * 256, N * 32
    assert uk.mmt4d_workspace_size(p) > uk.STATIC_SCRATCH_BYTES
    with pytest.raises(uk.UkernelError) as e:
        uk.mmt4d_static_scratch(p)
    assert e.value.status == abi.WORKSPACE_TOO_SMALL
    torch.cuda.synchronize()
    assert bool((out == 7).all())


def test_static_scratch_runs_s16s16_on_the_tensor_cores():
    """s16s16s32 16x16x2 uses scratch (byte planes of both operands) with iree_uk_b200_mmt4d_ws,
    so it does here too: same bytes as that call and as the reference, twice in a row."""
    case = cases.Mmt4dCase(abi.MMT4D_S16S16S32, 16, 16, 2, 24, 40, 130, 1, seed=26, mode="normal",
                           loose=False)
    for _ in range(2):
        got, want = _run_both(case)
        assert np.array_equal(got, want)
        assert np.array_equal(got, G.oracle_mmt4d(case))
    G.check_device_status()


def test_static_scratch_refuses_oversized_problem():
    M, N, K = 256, 256, 4096  # needs 64 MiB of re-tiled operands
    lhs = torch.zeros(M * K * 16, dtype=torch.float16, device="cuda")
    rhs = torch.zeros(N * K * 16, dtype=torch.float16, device="cuda")
    out = torch.full((M * N * 256,), 7.0, dtype=torch.float32, device="cuda")
    p = abi.Mmt4dParams()
    p.lhs_buffer, p.rhs_buffer, p.out_buffer = lhs.data_ptr(), rhs.data_ptr(), out.data_ptr()
    p.M, p.N, p.K, p.M0, p.N0, p.K0, p.flags = M, N, K, 16, 16, 1, abi.MMT4D_F16F16F32
    p.lhs_stride0, p.rhs_stride0, p.out_stride0 = K * 16, K * 16, N * 256
    assert uk.mmt4d_workspace_size(p) > uk.STATIC_SCRATCH_BYTES
    with pytest.raises(uk.UkernelError) as e:
        uk.mmt4d_static_scratch(p)
    assert e.value.status == abi.WORKSPACE_TOO_SMALL
    torch.cuda.synchronize()
    assert bool((out == 7.0).all())


def test_static_scratch_serves_scratch_free_shapes_too():
    case = cases.Mmt4dCase(abi.MMT4D_S8S8S32, 9, 6, 3, 5, 7, 13, 1, seed=23)
    lhs, rhs, out = G.to_device(case.lhs), G.to_device(case.rhs), G.to_device(case.out_init)
    uk.mmt4d_static_scratch(case.params(lhs.data_ptr(), rhs.data_ptr(), out.data_ptr()))
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), G.oracle_mmt4d(case))
