"""Parity of the fused row-major matmul (iree_uk_b200_matmul) with the reference's
pack -> mmt4d -> unpack chain (ukernel/tools/e2e_matmul_benchmark.c:173-300) run on the CPU
oracle: bit-exact for s8s8s32, relative Frobenius error <= 1e-3 for f16 / bf16."""
import numpy as np
import pytest

import oracle
from iree_b200 import abi
from oracle import cases

import gpu_util as G

pytestmark = pytest.mark.gpu

FLOAT_TOL = 1e-3  # relative Frobenius error allowed for the f16 / bf16 triples


def _operands(type_flag, M, N, K, seed):
    rng = np.random.default_rng(seed)
    if type_flag == abi.MMT4D_S8S8S32:
        return (rng.integers(-128, 128, (M, K), dtype=np.int8),
                rng.integers(-128, 128, (K, N), dtype=np.int8),
                rng.integers(-(1 << 20), 1 << 20, (M, N), dtype=np.int32))
    a = rng.standard_normal((M, K), dtype=np.float32)
    b = rng.standard_normal((K, N), dtype=np.float32)
    c = rng.standard_normal((M, N), dtype=np.float32)
    if type_flag == abi.MMT4D_F16F16F32:
        return a.astype(np.float16).view(np.uint16), b.astype(np.float16).view(np.uint16), c
    to_bf16 = lambda x: ((x.view(np.uint32) + 0x7FFF + ((x.view(np.uint32) >> 16) & 1)) >> 16).astype(np.uint16)
    return to_bf16(a), to_bf16(b), c


def _run_gpu(type_flag, lhs, rhs, acc, lhs_pad=0, rhs_pad=0, out_pad=0, lhs_off=0, rhs_off=0,
             out_off=0):
    """The matmul through the C ABI with the given row paddings and element offsets. Returns
    (result [M][N], whole output allocation, its initial content)."""
    import torch
    from iree_b200 import ukernel as uk
    M, K = lhs.shape
    N = rhs.shape[1]
    out_dtype = np.int32 if type_flag == abi.MMT4D_S8S8S32 else np.float32

    def embed(a, pad, off, fill):
        rows, cols = a.shape
        buf = np.full(off + rows * (cols + pad) + 3, fill, dtype=a.dtype)
        view = buf[off:off + rows * (cols + pad)].reshape(rows, cols + pad)
        view[:, :cols] = a
        return buf

    hl, hr = embed(lhs, lhs_pad, lhs_off, 1), embed(rhs, rhs_pad, rhs_off, 1)
    init = acc if acc is not None else np.full((M, N), 77, dtype=out_dtype)
    ho = embed(init.astype(out_dtype), out_pad, out_off, 55)
    dl, dr, do = (torch.from_numpy(x).cuda() for x in (hl, hr, ho.copy()))
    p = abi.MatmulParams()
    p.lhs_buffer, p.rhs_buffer, p.out_buffer = dl.data_ptr(), dr.data_ptr(), do.data_ptr()
    p.lhs_offset, p.rhs_offset, p.out_offset = lhs_off, rhs_off, out_off
    p.lhs_stride0, p.rhs_stride0, p.out_stride0 = K + lhs_pad, N + rhs_pad, N + out_pad
    p.M, p.N, p.K = M, N, K
    p.flags = type_flag | (abi.MMT4D_ACCUMULATE if acc is not None else 0)
    nws = uk.matmul_workspace_size(p)
    assert nws > 0
    ws = torch.empty(nws, dtype=torch.uint8, device="cuda")
    uk.matmul(p, ws)
    torch.cuda.synchronize()
    assert uk.device_status() == (0, 0)
    whole = do.cpu().numpy()
    res = whole[out_off:out_off + M * (N + out_pad)].reshape(M, N + out_pad)[:, :N]
    return res, whole, ho


def _untouched_outside(whole, init, M, N, out_pad, out_off):
    mask = np.ones(whole.shape, dtype=bool)
    body = mask[out_off:out_off + M * (N + out_pad)].reshape(M, N + out_pad)
    body[:, :N] = False
    return np.array_equal(whole[mask], init[mask])


SHAPES = [(1, 1, 1), (17, 33, 65), (128, 128, 128), (300, 200, 129), (130, 520, 96),
          (2560, 1032, 200)]  # the last one is served by the two-CTA kernel


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "%dx%dx%d" % s)
@pytest.mark.parametrize("accumulate", [0, 1])
def test_matmul_s8_exact(shape, accumulate):
    M, N, K = shape
    lhs, rhs, acc = _operands(abi.MMT4D_S8S8S32, M, N, K, seed=M * 7 + N)
    acc = acc if accumulate else None
    want = oracle.matmul_chain(lhs, rhs, acc, abi.MMT4D_S8S8S32, 16, 16, 2)
    got, _, _ = _run_gpu(abi.MMT4D_S8S8S32, lhs, rhs, acc)
    assert np.array_equal(got, want)


def test_matmul_result_does_not_depend_on_the_chain_tile_sizes():
    lhs, rhs, acc = _operands(abi.MMT4D_S8S8S32, 45, 70, 37, seed=3)
    got, _, _ = _run_gpu(abi.MMT4D_S8S8S32, lhs, rhs, acc)
    for M0, N0, K0 in [(16, 16, 2), (8, 8, 4), (1, 4, 8), (7, 3, 5)]:
        assert np.array_equal(got, oracle.matmul_chain(lhs, rhs, acc, abi.MMT4D_S8S8S32, M0, N0, K0))


@pytest.mark.parametrize("layout", [
    dict(lhs_pad=16, rhs_pad=16, out_pad=4),            # padded rows, everything aligned
    dict(lhs_pad=3, rhs_pad=5, out_pad=1),              # odd pitches: LHS copy, scalar stores
    dict(lhs_off=1, rhs_off=2, out_off=1),              # odd bases
    dict(lhs_off=16, rhs_off=16, out_off=4, out_pad=8),
], ids=["padded", "odd_pitch", "odd_base", "aligned_offsets"])
@pytest.mark.parametrize("t", [abi.MMT4D_S8S8S32, abi.MMT4D_F16F16F32], ids=["s8", "f16"])
def test_matmul_strides_and_offsets(t, layout):
    M, N, K = 150, 210, 77
    lhs, rhs, acc = _operands(t, M, N, K, seed=11)
    want = oracle.matmul_chain(lhs, rhs, acc, t, 16, 16, 2 if t == abi.MMT4D_S8S8S32 else 1)
    got, whole, init = _run_gpu(t, lhs, rhs, acc, **layout)
    if t == abi.MMT4D_S8S8S32:
        assert np.array_equal(got, want)
    else:
        assert cases.rel_frobenius(got, want) <= FLOAT_TOL
    assert _untouched_outside(whole, init, M, N, layout.get("out_pad", 0), layout.get("out_off", 0))


@pytest.mark.parametrize("t,K0", [(abi.MMT4D_F16F16F32, 1), (abi.MMT4D_BF16BF16F32, 2)],
                         ids=["f16", "bf16"])
@pytest.mark.parametrize("shape", [(1, 1, 1), (17, 33, 65), (300, 200, 129), (2560, 1024, 136)],
                         ids=lambda s: "%dx%dx%d" % s)
@pytest.mark.parametrize("accumulate", [0, 1])
def test_matmul_float_within_tolerance(t, K0, shape, accumulate):
    M, N, K = shape
    lhs, rhs, acc = _operands(t, M, N, K, seed=N)
    acc = acc if accumulate else None
    want = oracle.matmul_chain(lhs, rhs, acc, t, 16, 16, K0)
    got, _, _ = _run_gpu(t, lhs, rhs, acc)
    assert cases.rel_frobenius(got, want) <= FLOAT_TOL


def test_matmul_empty_reduction_and_rejections():
    import torch
    from iree_b200 import ukernel as uk
    out = torch.full((4, 8), 9, dtype=torch.int32, device="cuda")
    ws = torch.empty(1 << 20, dtype=torch.uint8, device="cuda")
    p = abi.MatmulParams()
    p.lhs_buffer = p.rhs_buffer = p.out_buffer = out.data_ptr()
    p.M, p.N, p.K = 4, 8, 0
    p.lhs_stride0, p.rhs_stride0, p.out_stride0 = 0, 8, 8
    p.flags = abi.MMT4D_S8S8S32
    uk.matmul(p, ws)                       # K = 0 without ACCUMULATE: zeros
    torch.cuda.synchronize()
    assert int(out.abs().sum()) == 0
    out.fill_(9)
    p.flags = abi.MMT4D_S8S8S32 | abi.MMT4D_ACCUMULATE
    uk.matmul(p, ws)                       # K = 0 with ACCUMULATE: unchanged
    torch.cuda.synchronize()
    assert int(out.sum()) == 9 * 32
    p.K, p.lhs_stride0 = 16, 16
    p.flags = abi.MMT4D_F32F32F32          # no tensor-core triple
    with pytest.raises(uk.UkernelError) as e:
        uk.matmul(p, ws)
    assert e.value.status == abi.UNSUPPORTED
    p.flags = abi.MMT4D_S8S8S32
    p.out_stride0 = 4                      # rows would overlap
    with pytest.raises(uk.UkernelError) as e:
        uk.matmul(p, ws)
    assert e.value.status == abi.INVALID_ARGUMENT
    p.out_stride0 = 8
    with pytest.raises(uk.UkernelError) as e:
        uk.matmul(p, ws[:256])             # scratch too small
    assert e.value.status == abi.WORKSPACE_TOO_SMALL
    assert int(out.sum()) == 9 * 32


def test_matmul_column_shards_equal_the_whole():
    """N-sharding of the row-major matmul needs no extra entry point: shard g passes
    rhs_offset = out_offset = its first column and its column count, with the full pitches."""
    import torch
    from iree_b200 import ukernel as uk
    M, N, K = 300, 520, 200
    lhs, rhs, _ = _operands(abi.MMT4D_BF16BF16F32, M, N, K, seed=4)
    whole, _, _ = _run_gpu(abi.MMT4D_BF16BF16F32, lhs, rhs, None)
    dl, dr = torch.from_numpy(lhs).cuda(), torch.from_numpy(rhs).cuda()
    out = torch.zeros(M, N, device="cuda")
    bounds = [0, 128, 136, 400, 520]   # uneven shards, one of them 8 columns wide
    for b, e in zip(bounds[:-1], bounds[1:]):
        p = abi.MatmulParams()
        p.lhs_buffer, p.rhs_buffer, p.out_buffer = dl.data_ptr(), dr.data_ptr(), out.data_ptr()
        p.rhs_offset = p.out_offset = b
        p.lhs_stride0, p.rhs_stride0, p.out_stride0 = K, N, N
        p.M, p.N, p.K, p.flags = M, e - b, K, abi.MMT4D_BF16BF16F32
        ws = torch.empty(uk.matmul_workspace_size(p), dtype=torch.uint8, device="cuda")
        uk.matmul(p, ws)
    torch.cuda.synchronize()
    assert uk.device_status() == (0, 0)
    assert np.array_equal(out.cpu().numpy(), whole)


@pytest.mark.parametrize("t,K0", [(abi.MMT4D_S8S8S32, 2), (abi.MMT4D_BF16BF16F32, 2)], ids=["s8", "bf16"])
@pytest.mark.parametrize("spec", [
    # M tiles, N tiles, K tiles, rows, cols, row pad, out offset
    (9, 17, 33, 9 * 16, 17 * 16, 0, 0),        # whole tiles, aligned: vector stores
    (9, 17, 33, 9 * 16 - 5, 17 * 16 - 3, 0, 0),  # ragged: the last tiles are cut
    (20, 24, 5, 20 * 16 - 15, 24 * 16 - 1, 7, 3),  # odd pitch and base: element stores
    (160, 64, 9, 160 * 16, 64 * 16 - 8, 8, 4),  # two-CTA kernel
], ids=["whole", "ragged", "odd_layout", "pair"])
@pytest.mark.parametrize("accumulate", [0, 1])
def test_mmt4d_with_unpack_folded_into_the_epilogue(t, K0, spec, accumulate):
    """iree_uk_b200_mmt4d_ws_unpacked against the reference's own sequence on the CPU oracle:
    (pack the accumulator,) mmt4d into tiles, unpack the tiles into the row-major matrix."""
    import torch
    from iree_b200 import ukernel as uk
    M, N, K, rows, cols, pad, off = spec
    is_int = t == abi.MMT4D_S8S8S32
    case = cases.Mmt4dCase(t, 16, 16, K0, M, N, K, 0, seed=33, mode="exact" if is_int else "normal",
                           loose=False)
    out_dtype = np.int32 if is_int else np.float32
    rng = np.random.default_rng(3)
    acc = (rng.integers(-1000, 1000, (rows, cols)).astype(np.int32) if is_int
           else rng.standard_normal((rows, cols), dtype=np.float32))
    # oracle: tiles <- pack(acc) when accumulating; mmt4d; unpack
    tiles = np.zeros(M * N * 256, dtype=out_dtype)
    if accumulate:
        pp = abi.PackParams()
        pp.in_buffer, pp.out_buffer = acc.ctypes.data, tiles.ctypes.data
        pp.in_size0, pp.in_size1, pp.in_stride0, pp.in_stride1 = rows, cols, cols, 1
        pp.out_size0, pp.out_size1, pp.out_size2, pp.out_size3 = M, N, 16, 16
        pp.out_stride1, pp.out_stride0 = 256, N * 256
        pp.flags = abi.PACK_I32I32 if is_int else abi.PACK_F32F32
        oracle.pack(pp)
    q = case.params(case.lhs, case.rhs, tiles)
    q.out_offset, q.out_stride0 = 0, N * 256
    q.flags = t | (abi.MMT4D_ACCUMULATE if accumulate else 0)
    oracle.mmt4d(q)
    want = np.zeros((rows, cols), dtype=out_dtype)
    u = abi.UnpackParams()
    u.in_buffer, u.out_buffer = tiles.ctypes.data, want.ctypes.data
    u.in_size0, u.in_size1, u.in_size2, u.in_size3 = M, N, 16, 16
    u.in_stride1, u.in_stride0 = 256, N * 256
    u.out_size0, u.out_size1, u.out_stride0, u.out_stride1 = rows, cols, cols, 1
    u.flags = abi.UNPACK_I32I32 if is_int else abi.UNPACK_F32F32
    oracle.unpack(u)
    # device: row-major output embedded in a larger buffer
    pitch = cols + pad
    host = np.full(off + rows * pitch + 5, 55, dtype=out_dtype)
    view = host[off:off + rows * pitch].reshape(rows, pitch)
    view[:, :cols] = acc if accumulate else 77
    init = host.copy()
    lhs, rhs, out = G.to_device(case.lhs), G.to_device(case.rhs), torch.from_numpy(host).cuda()
    p = case.params(lhs.data_ptr(), rhs.data_ptr(), out.data_ptr())
    p.out_offset, p.out_stride0 = off, pitch
    p.flags = q.flags
    ws = torch.empty(uk.mmt4d_workspace_size(p), dtype=torch.uint8, device="cuda")
    uk.mmt4d_unpacked(p, rows, cols, ws)
    torch.cuda.synchronize()
    assert uk.device_status() == (0, 0)
    whole = out.cpu().numpy()
    got = whole[off:off + rows * pitch].reshape(rows, pitch)[:, :cols]
    if is_int:
        assert np.array_equal(got, want)
    else:
        assert cases.rel_frobenius(got, want) <= FLOAT_TOL
    assert _untouched_outside(whole, init, rows, cols, pad, off)
