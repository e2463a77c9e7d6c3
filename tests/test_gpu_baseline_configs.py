"""The five benchmark configurations at their own sizes, GPU result against the reference
ukernels themselves (the library compiled in place under oracle/_ref, driven across the host's
threads as ukernel/README.md:26 prescribes for callers): integers, pack and unpack over the whole
output allocation bit for bit (the reference's own check, tools/mmt4d_test.c:430-440), floats by
relative Frobenius error <= 1e-3. Inputs are seeded and synthetic, with the value distributions
the configurations name; seeds are 1234 + configuration number."""
import os

import numpy as np
import pytest
import torch

import oracle
from iree_b200 import abi
from iree_b200 import ukernel as uk

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not oracle.ref_available(),
                                 reason="compiled reference ukernels not present")]

FLOAT_TOL = 1e-3
THREADS = os.cpu_count() or 1


def _mmt4d_params(flags, M, N, K, M0, N0, K0, lhs, rhs, out):
    p = abi.Mmt4dParams()
    p.lhs_buffer, p.rhs_buffer, p.out_buffer = lhs, rhs, out
    p.M, p.N, p.K, p.M0, p.N0, p.K0, p.flags = M, N, K, M0, N0, K0, flags
    lb, rb, _ = abi.MMT4D_BITS[flags & 0xFF]
    p.lhs_stride0, p.rhs_stride0, p.out_stride0 = K * M0 * K0, K * N0 * K0, N * M0 * N0
    return p


def _gpu_mmt4d(p_host, lhs, rhs, out_init, workspace=True):
    """Runs the host-described problem on device copies; returns the device output tensor."""
    d_lhs, d_rhs = torch.from_numpy(lhs).cuda(), torch.from_numpy(rhs).cuda()
    d_out = torch.from_numpy(out_init).cuda()
    p = abi.copy_params(p_host)
    p.lhs_buffer, p.rhs_buffer, p.out_buffer = d_lhs.data_ptr(), d_rhs.data_ptr(), d_out.data_ptr()
    ws = None
    if workspace:
        n = uk.mmt4d_workspace_size(p)
        ws = torch.empty(n, dtype=torch.uint8, device="cuda") if n else None
    path = uk.mmt4d_path(p, ws is not None)
    uk.mmt4d(p, workspace=ws)
    torch.cuda.synchronize()
    assert uk.device_status() == (0, 0)
    return d_out, path


def _rel_frobenius_gpu(got, want_host):
    """||got - want|| / ||want|| with `want` uploaded in pieces (bounded device temporaries)."""
    num = den = 0.0
    step = 1 << 26
    g = got.view(-1)
    for i in range(0, g.numel(), step):
        w = torch.from_numpy(want_host[i:i + step]).cuda().double()
        d = g[i:i + step].double() - w
        num += float((d * d).sum())
        den += float((w * w).sum())
    return (num / max(den, 1e-300)) ** 0.5


def _bf16(rng, n, scale):
    out = np.empty(n, dtype=np.uint16)
    step = 1 << 24
    for i in range(0, n, step):
        x = rng.standard_normal(min(step, n - i), dtype=np.float32) * np.float32(scale)
        u = x.view(np.uint32).astype(np.uint64)
        out[i:i + step] = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)  # RNE
    return out


def test_config1_s8_64x64x512_whole_buffer_exact():
    """mmt4d s8s8s32, M = N = 64, K = 512, tiles 16x16x2, no ACCUMULATE, output pre-filled with
    0xCD bytes to prove the overwrite; with and without scratch."""
    rng = np.random.default_rng(1234 + 1)
    lhs = rng.integers(-128, 128, 64 * 512 * 32, dtype=np.int8)
    rhs = rng.integers(-128, 128, 64 * 512 * 32, dtype=np.int8)
    init = np.full(64 * 64 * 256, 0xCDCDCDCD, dtype=np.uint32).view(np.int32)
    want = init.copy()
    p = _mmt4d_params(abi.MMT4D_S8S8S32, 64, 64, 512, 16, 16, 2, lhs.ctypes.data, rhs.ctypes.data,
                      want.ctypes.data)
    oracle.mmt4d_threaded(p, THREADS, "ref")
    for ws in (True, False):
        got, path = _gpu_mmt4d(p, lhs, rhs, init, workspace=ws)
        assert path == (abi.PATH_TCGEN05_RETILE if ws else abi.PATH_TCGEN05)
        assert np.array_equal(got.cpu().numpy(), want)


def test_config2_f16_accumulate_4096_cubed_against_reference():
    """mmt4d f16f16f32 | ACCUMULATE, M = N = 256, K = 4096, tiles 16x16x1, N(0,1) operands and
    accumulator: the whole output within 1e-3 of the reference's."""
    rng = np.random.default_rng(1234 + 2)
    lhs = rng.standard_normal(256 * 4096 * 16, dtype=np.float32).astype(np.float16)
    rhs = rng.standard_normal(256 * 4096 * 16, dtype=np.float32).astype(np.float16)
    init = rng.standard_normal(256 * 256 * 256, dtype=np.float32)
    want = init.copy()
    p = _mmt4d_params(abi.MMT4D_F16F16F32 | abi.MMT4D_ACCUMULATE, 256, 256, 4096, 16, 16, 1,
                      lhs.ctypes.data, rhs.ctypes.data, want.ctypes.data)
    oracle.mmt4d_threaded(p, THREADS, "ref")
    got, path = _gpu_mmt4d(p, lhs, rhs, init)
    assert path == abi.PATH_TCGEN05_RETILE
    assert _rel_frobenius_gpu(got, want) <= FLOAT_TOL


def test_config3_s16u4_decode_gemv_exact():
    """mmt4d s16u4s32, M = 1, N = 448, K = 512, tiles 1x32x8, full-range s16 activations and
    uniformly random weight bytes: all 14336 outputs bit for bit."""
    rng = np.random.default_rng(1234 + 3)
    lhs = rng.integers(-32768, 32768, 512 * 8, dtype=np.int16)
    rhs = rng.integers(0, 256, 448 * 512 * 128, dtype=np.uint8)
    init = np.full(448 * 32, 0x5A5A5A5A, dtype=np.int32)
    want = init.copy()
    p = _mmt4d_params(abi.MMT4D_S16U4S32, 1, 448, 512, 1, 32, 8, lhs.ctypes.data,
                      rhs.ctypes.data, want.ctypes.data)
    oracle.mmt4d_threaded(p, THREADS, "ref")
    got, path = _gpu_mmt4d(p, lhs, rhs, init)
    assert path == abi.PATH_GEMV
    assert np.array_equal(got.cpu().numpy(), want)


N4 = 8192


def _pack_params(src, dst, flags, in0, in1, o0, o1, t0, t1, pad=0):
    p = abi.PackParams()
    p.in_buffer, p.out_buffer = src, dst
    p.in_size0, p.in_size1, p.in_stride0, p.in_stride1 = in0, in1, N4, 1
    p.out_size0, p.out_size1, p.out_size2, p.out_size3 = o0, o1, t0, t1
    p.out_stride1 = t0 * t1
    p.out_stride0 = o1 * t0 * t1
    p.padding_value, p.flags = pad, flags
    return p


TI, TO = abi.PACK_TRANSPOSE_INNER, abi.PACK_TRANSPOSE_OUTER


@pytest.mark.parametrize("name,flags,in0,o0,o1,t0,t1,pad", [
    ("4a_lhs_style_16x1", abi.PACK_F32F32, N4, 512, N4, 16, 1, 0),
    ("4a_pad_8185_rows_nan_pattern", abi.PACK_F32F32, 8185, 512, N4, 16, 1, 0x7FC00000),
    ("4b_transpose_inner_1x16", abi.PACK_F32F32 | TI, N4, 512, N4, 1, 16, 0),
    ("4b_rhs_style_0x301", abi.PACK_F32F32 | TI | TO, N4, 512, N4, 16, 1, 0),
], ids=lambda v: v if isinstance(v, str) else None)
def test_config4_pack_8192_whole_output_exact(name, flags, in0, o0, o1, t0, t1, pad):
    """pack f32, 8192 x 8192 (or 8185 rows with 7 padded rows in the last tile row) into the
    tiled layouts the benchmark times; the whole 256 MiB output bit for bit. The 0x301 form is
    the RHS pack of tools/e2e_matmul_benchmark.c:238-254: [K][N] -> [N1][K1][16][1]."""
    rng = np.random.default_rng(1234 + 4)
    src = rng.standard_normal(N4 * N4, dtype=np.float32)
    init = np.full(N4 * N4, 0x5A5A5A5A, dtype=np.uint32)
    want = init.copy()
    oracle.pack(_pack_params(src.ctypes.data, want.ctypes.data, flags, in0, N4, o0, o1, t0, t1, pad),
                "ref")
    d_src, d_out = torch.from_numpy(src).cuda(), torch.from_numpy(init.view(np.int32)).cuda()
    p = _pack_params(d_src.data_ptr(), d_out.data_ptr(), flags, in0, N4, o0, o1, t0, t1, pad)
    assert uk.pack_path(p) == abi.PATH_FAST_COPY
    uk.pack(p)
    torch.cuda.synchronize()
    assert uk.device_status() == (0, 0)
    assert torch.equal(d_out, torch.from_numpy(want.view(np.int32)).cuda())


def test_config4c_unpack_i32_8192_whole_output_exact():
    """unpack i32 [512][512][16][16] -> 8192 x 8192, full-range values, bit for bit."""
    rng = np.random.default_rng(1234 + 4)
    src = rng.integers(-2**31, 2**31, N4 * N4, dtype=np.int64).astype(np.int32)
    init = np.full(N4 * N4, 0x5A5A5A5A, dtype=np.int32)
    want = init.copy()

    def params(s, d):
        q = abi.UnpackParams()
        q.in_buffer, q.out_buffer = s, d
        q.in_size0, q.in_size1, q.in_size2, q.in_size3 = 512, 512, 16, 16
        q.in_stride1, q.in_stride0 = 256, 512 * 256
        q.out_size0, q.out_size1, q.out_stride0, q.out_stride1 = N4, N4, N4, 1
        q.flags = abi.UNPACK_I32I32
        return q

    oracle.unpack(params(src.ctypes.data, want.ctypes.data), "ref")
    d_src, d_out = torch.from_numpy(src).cuda(), torch.from_numpy(init).cuda()
    q = params(d_src.data_ptr(), d_out.data_ptr())
    assert uk.unpack_path(q) == abi.PATH_FAST_COPY
    uk.unpack(q)
    torch.cuda.synchronize()
    assert torch.equal(d_out, torch.from_numpy(want).cuda())


def test_config5_bf16_headline_whole_output_and_shards_against_reference():
    """mmt4d bf16bf16f32, M = 512, K = 4096, N = 1792 tile rows of 16x16x2 (8192 x 8192 x 28672),
    activations N(0,1), weights N(0,0.02): the whole 896 MiB output within 1e-3 of the
    reference's, and, for the 2-way and 8-way splits of iree_uk_b200_mmt4d_shard_params, every
    rank's [M][N/G][16][16] slab within 1e-3 of the matching tile columns."""
    M1, N1, K1 = 512, 1792, 4096
    rng = np.random.default_rng(1234 + 5)
    lhs = _bf16(rng, M1 * K1 * 32, 1.0)
    rhs = _bf16(rng, N1 * K1 * 32, 0.02)
    want = np.zeros(M1 * N1 * 256, dtype=np.float32)
    ph = _mmt4d_params(abi.MMT4D_BF16BF16F32, M1, N1, K1, 16, 16, 2, lhs.ctypes.data,
                       rhs.ctypes.data, want.ctypes.data)
    oracle.mmt4d_threaded(ph, THREADS, "ref")

    d_lhs, d_rhs = torch.from_numpy(lhs).cuda(), torch.from_numpy(rhs).cuda()
    d_out = torch.full((M1 * N1 * 256,), float("nan"), dtype=torch.float32, device="cuda")
    full = _mmt4d_params(abi.MMT4D_BF16BF16F32, M1, N1, K1, 16, 16, 2, d_lhs.data_ptr(),
                         d_rhs.data_ptr(), d_out.data_ptr())
    ws = torch.empty(uk.mmt4d_workspace_size(full), dtype=torch.uint8, device="cuda")
    assert uk.mmt4d_path(full, True) == abi.PATH_TCGEN05_RETILE
    uk.mmt4d(full, workspace=ws)
    torch.cuda.synchronize()
    assert uk.device_status() == (0, 0)
    assert _rel_frobenius_gpu(d_out, want) <= FLOAT_TOL

    want_tiles = want.reshape(M1, N1, 256)
    for world in (2, 8):
        for rank in range(world):
            p, begin = uk.shard_params(full, rank, world, rhs_is_local=False, out_is_local=True)
            slab = torch.full((M1 * p.N * 256,), float("nan"), dtype=torch.float32, device="cuda")
            p.out_buffer = slab.data_ptr()
            uk.mmt4d(p, workspace=ws)
            torch.cuda.synchronize()
            w = np.ascontiguousarray(want_tiles[:, begin:begin + p.N]).reshape(-1)
            assert _rel_frobenius_gpu(slab, w) <= FLOAT_TOL, (world, rank)
    assert uk.device_status() == (0, 0)
