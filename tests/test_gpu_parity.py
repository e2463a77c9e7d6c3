"""GPU parity: the CUDA library, called through the C ABI, against the CPU oracle on the
reference tests' own case lists (tools/mmt4d_test.c:459-603, pack_test.c:137-241,
unpack_test.c:118-216). Integers, pack and unpack: whole output allocation bit-exact
(stride gaps and offset prefix included). Floats on the small-integer value ranges of
tools/util.c:136-168 are exact too."""
import os

import numpy as np
import pytest

import oracle
from iree_b200 import abi
from oracle import cases

import gpu_util as G

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _device_status_clean():
    yield
    G.check_device_status()


def _mmt4d_ids(tiles):
    return ["t%x_%dx%dx%d" % t for t in tiles]


@pytest.mark.parametrize("tile", cases.MMT4D_TILES + cases.MMT4D_TILES_EXTRA,
                         ids=_mmt4d_ids(cases.MMT4D_TILES + cases.MMT4D_TILES_EXTRA))
def test_mmt4d_reference_case_list(tile):
    n = 0
    for case in cases.all_mmt4d_cases([tile]):
        got, _ = G.run_mmt4d_case(case)
        want = G.oracle_mmt4d(case)
        assert np.array_equal(got, want), case.label()
        n += 1
    assert n > 0


@pytest.mark.parametrize("tile", cases.MMT4D_TILES_16BIT_OUT,
                         ids=lambda t: "t%x_%dx%dx%d" % t)
def test_mmt4d_16bit_output_triples(tile):
    """f16f16f16 / bf16bf16bf16 with and without SKIP_INTERMEDIATE_ROUNDINGS on the reference
    tests' shapes and small-integer values: bit-exact, rounding after every step included."""
    n = 0
    for case in cases.all_mmt4d_cases([tile]):
        got, _ = G.run_mmt4d_case(case)
        assert np.array_equal(got, G.oracle_mmt4d(case)), case.label()
        n += 1
    assert n > 0


@pytest.mark.parametrize("tile", [(abi.MMT4D_S8S8S32, 16, 16, 2), (abi.MMT4D_F16F16F32, 16, 16, 1),
                                  (abi.MMT4D_BF16BF16F32, 16, 16, 2),
                                  (abi.MMT4D_S8S8S32, 16, 16, 8), (abi.MMT4D_BF16BF16F32, 16, 16, 1),
                                  (abi.MMT4D_F32F32F32, 16, 16, 1), (abi.MMT4D_F32F32F32, 16, 16, 4)],
                         ids=lambda t: "t%x_%dx%dx%d" % t)
@pytest.mark.parametrize("shape", [(1, 1, 1), (8, 16, 64), (9, 17, 65), (3, 5, 7), (16, 32, 130),
                                   (24, 40, 31), (1, 1, 1000)], ids=lambda s: "%dx%dx%d" % s)
@pytest.mark.parametrize("accumulate", [0, 1])
def test_mmt4d_tensor_core_path_exact(tile, shape, accumulate):
    """Aligned, tight cases that the tensor-core path serves; small-integer values make the
    expected result exact for every accumulation order."""
    t, M0, N0, K0 = tile
    M, N, K = shape
    case = cases.Mmt4dCase(t, M0, N0, K0, M, N, K, accumulate, seed=7, mode="exact", loose=False)
    with G.f32_tensor_cores(t):
        got, path = G.run_mmt4d_case(case)
    assert path == abi.PATH_TCGEN05_RETILE
    want = G.oracle_mmt4d(case)
    assert np.array_equal(got, want), case.label()
    if t == abi.MMT4D_F32F32F32:  # default mode: the CUDA-core kernel, same exact result
        got, path = G.run_mmt4d_case(case)
        assert path == abi.PATH_GENERIC
        assert np.array_equal(got, want), case.label()


def test_mmt4d_tensor_core_loose_out_stride():
    """A non-tight out_stride0 (multiple of 16 bytes) keeps the tensor-core path and must not
    touch the gap between tile rows."""
    case = cases.Mmt4dCase(abi.MMT4D_S8S8S32, 16, 16, 2, 10, 9, 40, 0, seed=3, loose=False)
    case.out_stride0 += 8
    case.out_init = cases.random_elements("s32", case.out_offset + case.M * case.out_stride0,
                                          np.random.default_rng(5))
    got, path = G.run_mmt4d_case(case)
    assert path == abi.PATH_TCGEN05_RETILE
    assert np.array_equal(got, G.oracle_mmt4d(case))


def _half_bits_to_f32(a, is_bf16):
    u = a.view(np.uint16)
    if is_bf16:
        return (u.astype(np.uint32) << 16).view(np.float32)
    return u.view(np.float16).astype(np.float32)


@pytest.mark.parametrize("t,K0,is_bf16", [(abi.MMT4D_F16F16F16, 1, False),
                                          (abi.MMT4D_BF16BF16BF16, 2, True)], ids=["f16", "bf16"])
@pytest.mark.parametrize("shape", [(1, 1, 8), (9, 17, 65), (40, 24, 300), (160, 64, 64)],
                         ids=lambda s: "%dx%dx%d" % s)
@pytest.mark.parametrize("accumulate", [0, 1])
def test_mmt4d_16bit_output_on_tensor_cores(t, K0, is_bf16, shape, accumulate):
    """f16f16f16 / bf16bf16bf16 with SKIP_INTERMEDIATE_ROUNDINGS (f32 accumulation, one final
    rounding — what the reference's own benchmark runs, tools/mmt4d_benchmark.c:100) take the
    tensor-core kernel; N(0,1) operands, relative Frobenius error <= 1e-3 against the oracle.
    Without the flag the same problem stays on the generic kernel (rounding at every step)."""
    M, N, K = shape
    flags = t | abi.MMT4D_SKIP_INTERMEDIATE_ROUNDINGS
    case = cases.Mmt4dCase(flags, 16, 16, K0, M, N, K, accumulate, seed=17, mode="normal",
                           loose=False)
    got, path = G.run_mmt4d_case(case)
    assert path == abi.PATH_TCGEN05_RETILE
    want = G.oracle_mmt4d(case)
    err = cases.rel_frobenius(_half_bits_to_f32(got, is_bf16), _half_bits_to_f32(want, is_bf16))
    assert err <= 1e-3, err
    plain = cases.Mmt4dCase(t, 16, 16, K0, M, N, K, accumulate, seed=17, mode="normal", loose=False)
    _, path = G.run_mmt4d_case(plain)
    assert path == abi.PATH_GENERIC


@pytest.mark.parametrize("t,M0,N0,K0,M,N,K,acc,tol", [
    (abi.MMT4D_F16F16F32, 16, 16, 1, 16, 16, 512, 1, 1e-3),
    (abi.MMT4D_BF16BF16F32, 16, 16, 2, 24, 32, 256, 0, 1e-3),
    (abi.MMT4D_F16F16F32, 4, 6, 5, 5, 7, 13, 1, 1e-3),
    # f32 on the tensor cores (opt-in mode) as three tf32 products: error about 7e-9 x K
    (abi.MMT4D_F32F32F32, 16, 16, 1, 24, 40, 700, 0, 1e-5),
    (abi.MMT4D_F32F32F32, 16, 16, 2, 160, 64, 129, 1, 1e-5),
])
def test_mmt4d_float_normal_values(t, M0, N0, K0, M, N, K, acc, tol):
    """N(0,1) operands: relative Frobenius error <= 1e-3 against the oracle's f32
    accumulation (the tolerance the headline configurations state)."""
    case = cases.Mmt4dCase(t, M0, N0, K0, M, N, K, acc, seed=11, mode="normal", loose=False)
    with G.f32_tensor_cores(t):
        got, path = G.run_mmt4d_case(case)
    if M0 == 16:
        assert path == abi.PATH_TCGEN05_RETILE
    want = G.oracle_mmt4d(case)
    err = cases.rel_frobenius(got.view(np.float32), want.view(np.float32))
    assert err <= tol, err


def test_mmt4d_s16u4_gemv_path():
    # M = 1: the decode call; 2 <= M < 16: batches of rows, four per block sharing the weights
    for (M, N, K, acc) in [(1, 1, 1, 0), (1, 7, 33, 1), (3, 5, 64, 0), (1, 448, 512, 0),
                           (2, 3, 17, 1), (4, 2, 40, 0), (7, 3, 40, 1), (15, 2, 33, 0)]:
        case = cases.Mmt4dCase(abi.MMT4D_S16U4S32, 1, 32, 8, M, N, K, acc, seed=M + N, mode="normal",
                               loose=False)
        got, path = G.run_mmt4d_case(case)
        assert path == abi.PATH_GEMV
        assert np.array_equal(got, G.oracle_mmt4d(case)), (M, N, K, acc)


@pytest.mark.parametrize("shape", [(16, 3, 9), (32, 4, 16), (128, 8, 64), (200, 7, 33), (129, 5, 1),
                                   (256, 448, 40),
                                   # enough 256 x 128 tiles for the two-CTA form, ragged edges
                                   (2560, 32, 5), (2700, 35, 3)], ids=lambda s: "%dx%dx%d" % s)
@pytest.mark.parametrize("accumulate", [0, 1])
def test_mmt4d_s16u4_tensor_core_path(shape, accumulate):
    """s16u4s32 1x32x8 with many rows: signed-high / unsigned-low byte planes against u8 weights
    on the tensor cores, recombined as hi*256 + lo. Full-range s16 values, bit-exact."""
    M, N, K = shape
    case = cases.Mmt4dCase(abi.MMT4D_S16U4S32, 1, 32, 8, M, N, K, accumulate, seed=M + K,
                           mode="normal", loose=False)
    got, path = G.run_mmt4d_case(case)
    assert path == abi.PATH_TCGEN05_RETILE
    assert np.array_equal(got, G.oracle_mmt4d(case)), shape
    # the same problem without scratch runs the weight-streaming kernel and agrees
    got2, path2 = G.run_mmt4d_case(case, use_workspace=False)
    assert path2 == abi.PATH_GEMV
    assert np.array_equal(got2, got)


@pytest.mark.parametrize("shape", [(1, 1, 1), (8, 16, 64), (9, 17, 65), (3, 5, 7), (24, 40, 31),
                                   (1, 1, 1000), (16, 3, 260),
                                   # enough 256 x 128 tiles for the two-CTA form, ragged edges
                                   (160, 64, 9), (170, 67, 5),
                                   # enough tiles for the wide single-buffered accumulators
                                   # (256 / 160 columns), ragged in M and N
                                   (325, 67, 3)], ids=lambda s: "%dx%dx%d" % s)
@pytest.mark.parametrize("t,K0", [(abi.MMT4D_S16S16S32, 2), (abi.MMT4D_S16S8S32, 2),
                                  (abi.MMT4D_S8S4S32, 2), (abi.MMT4D_S8S4S32, 4),
                                  (abi.MMT4D_S8S4S32, 8), (abi.MMT4D_S8S4S32, 16)],
                         ids=["s16s16", "s16s8", "s8s4_k2", "s8s4_k4", "s8s4_k8", "s8s4_k16"])
@pytest.mark.parametrize("accumulate", [0, 1])
def test_mmt4d_byte_plane_types_on_the_tensor_cores(t, K0, shape, accumulate):
    """The integer triples wider or narrower than a byte, 16x16 tiles, as 8-bit tensor-core
    products. s16s16s32 16x16x2 (arch/x86_64/mmt4d_x86_64_avx512_base.c:312 has the ISA function):
    byte planes of both operands, four products per term into three accumulators, recombined
    modulo 2^32. s16s8s32: byte planes of the LHS, two products per term. s8s4s32: the nibbles
    sign-extended to bytes by the pre-pass (mmt4d_tile_generic.c:37-44), one product per term.
    Full-range values, so the sums wrap like the reference's int32 arithmetic; bit-exact. Without
    scratch the generic kernel serves the same problem and agrees."""
    M, N, K = shape
    case = cases.Mmt4dCase(t, 16, 16, K0, M, N, K, accumulate, seed=M + K, mode="normal",
                           loose=False)
    got, path = G.run_mmt4d_case(case)
    assert path == abi.PATH_TCGEN05_RETILE
    assert np.array_equal(got, G.oracle_mmt4d(case)), shape
    got2, path2 = G.run_mmt4d_case(case, use_workspace=False)
    assert path2 == abi.PATH_GENERIC
    assert np.array_equal(got2, got)


NARROW_TYPES = [(abi.MMT4D_S8S8S32, 2), (abi.MMT4D_F16F16F32, 1), (abi.MMT4D_BF16BF16F32, 2)]


@pytest.mark.parametrize("t,K0", NARROW_TYPES, ids=["s8", "f16", "bf16"])
@pytest.mark.parametrize("M0", [1, 2, 4, 8])
@pytest.mark.parametrize("shape", [(1, 1, 1), (1, 7, 33), (3, 5, 64), (1, 40, 1000), (2, 3, 129)],
                         ids=lambda s: "%dx%dx%d" % s)
@pytest.mark.parametrize("accumulate", [0, 1])
def test_mmt4d_narrowed_m0_weight_streaming(t, K0, M0, shape, accumulate):
    """Narrowed M0 x 16 tiles (arch/x86_64/mmt4d_x86_64_tiles.inl:30-60 has ISA functions for
    them): the weight-streaming kernel, with and without scratch. Small-integer values: exact."""
    M, N, K = shape
    case = cases.Mmt4dCase(t, M0, 16, K0, M, N, K, accumulate, seed=43, mode="exact", loose=False)
    want = G.oracle_mmt4d(case)
    for ws in (True, False):
        got, path = G.run_mmt4d_case(case, use_workspace=ws)
        assert path == abi.PATH_GEMV
        assert np.array_equal(got, want), case.label()


@pytest.mark.parametrize("t,K0", NARROW_TYPES[1:], ids=["f16", "bf16"])
def test_mmt4d_narrowed_m0_normal_values(t, K0):
    case = cases.Mmt4dCase(t, 4, 16, K0, 1, 96, 2048, 1, seed=47, mode="normal", loose=False)
    got, path = G.run_mmt4d_case(case)
    assert path == abi.PATH_GEMV
    want = G.oracle_mmt4d(case)
    assert cases.rel_frobenius(got.view(np.float32), want.view(np.float32)) <= 1e-3


def test_mmt4d_int_wraparound():
    """int32 sums wrap modulo 2^32 like the reference's (extreme s8 values, long K, and an
    initial accumulator near INT32_MAX)."""
    case = cases.Mmt4dCase(abi.MMT4D_S8S8S32, 16, 16, 2, 8, 16, 4096, 1, seed=1, loose=False)
    case.lhs[:] = 0x80  # -128
    case.rhs[:] = 0x80
    case.out_init.view(np.int32)[:] = 2**31 - 5
    want = G.oracle_mmt4d(case)
    for ws in (True, False):
        got, _ = G.run_mmt4d_case(case, use_workspace=ws)
        assert np.array_equal(got, want), ws


def test_mmt4d_int_overflow_inside_accumulator():
    """A sum that leaves the int32 range while it is still being accumulated (K = 140000
    products of -128 * -128) must wrap like the reference's, not saturate."""
    case = cases.Mmt4dCase(abi.MMT4D_S8S8S32, 16, 16, 2, 1, 1, 70000, 0, seed=1, loose=False)
    case.lhs[:] = 0x80
    case.rhs[:] = 0x80
    want = G.oracle_mmt4d(case)
    got, path = G.run_mmt4d_case(case)
    assert path == abi.PATH_TCGEN05_RETILE
    assert np.array_equal(got, want)


@pytest.mark.parametrize("tile", cases.PACK_TILES, ids=lambda t: "t%x_%dx%d" % t)
def test_pack_reference_case_list(tile):
    paths = set()
    for case in cases.all_pack_cases([tile]):
        got, path = G.run_pack_case(case)
        paths.add(path)
        assert np.array_equal(got, G.oracle_pack(case)), vars(case)
    assert paths


@pytest.mark.parametrize("tile", cases.UNPACK_TILES, ids=lambda t: "t%x_%dx%d" % t)
def test_unpack_reference_case_list(tile):
    for case in cases.all_unpack_cases([tile]):
        got, _ = G.run_unpack_case(case)
        assert np.array_equal(got, G.oracle_unpack(case)), vars(case)


@pytest.mark.parametrize("tile", cases.PACK_TILES, ids=lambda t: "t%x_%dx%d" % t)
def test_pack_aligned_vector_paths(tile):
    """Tight, 16-byte aligned cases (no random offsets) reach the vectorised branches."""
    seed = 100
    for outer in [(3, 2), (9, 33), (40, 70)]:
        for ti in (0, 1):
            for to in (0, 1):
                for pad in cases.PAD_MODES:
                    seed += 1
                    case = cases.PackCase(tile[0], tile[1], tile[2], outer, ti, to, pad, seed,
                                          loose=False)
                    got, _ = G.run_pack_case(case)
                    assert np.array_equal(got, G.oracle_pack(case)), vars(case)


@pytest.mark.parametrize("tile,outer", [
    ((abi.PACK_F32F32, 16, 1), (16, 32)), ((abi.PACK_F32F32, 16, 1), (64, 12)),
    ((abi.PACK_F16F16, 16, 1), (8, 64)),
    ((abi.PACK_BF16BF16, 16, 2), (8, 64)), ((abi.PACK_BF16BF16, 16, 2), (32, 24)),
    ((abi.PACK_I8I8, 16, 2), (12, 128)), ((abi.PACK_I8I8, 16, 2), (64, 8)),
], ids=lambda v: "x".join(str(x) for x in v))
@pytest.mark.parametrize("pad", ["none", "one_incomplete_tile"])
def test_pack_rhs_style_constant_shape_kernels(tile, outer, pad):
    """The RHS pack of a matmul ([K][N] -> [N1][K1][N0][K0], both transposes,
    tools/e2e_matmul_benchmark.c:238-254) on matrices that the constant-shape kernels divide:
    the long-row blocks and the many-short-rows blocks, whole blocks (bulk row copies) and
    blocks that hold padding."""
    case = cases.PackCase(tile[0], tile[1], tile[2], outer, 1, 1, pad, seed=77, loose=False)
    got, path = G.run_pack_case(case)
    assert path == abi.PATH_FAST_COPY
    assert np.array_equal(got, G.oracle_pack(case)), vars(case)
    G.check_device_status()


@pytest.mark.parametrize("tile", cases.UNPACK_TILES, ids=lambda t: "t%x_%dx%d" % t)
def test_unpack_aligned_vector_paths(tile):
    seed = 200
    for outer in [(3, 2), (9, 33), (40, 70)]:
        for ti in (0, 1):
            for to in (0, 1):
                for pad in cases.PAD_MODES:
                    seed += 1
                    case = cases.UnpackCase(tile[0], tile[1], tile[2], outer, ti, to, pad, seed,
                                            loose=False)
                    got, _ = G.run_unpack_case(case)
                    assert np.array_equal(got, G.oracle_unpack(case)), vars(case)


def test_generic_kernels_forced():
    """IREE_UK_B200_FORCE_GENERIC routes every call to the one-thread-per-element kernels."""
    os.environ["IREE_UK_B200_FORCE_GENERIC"] = "1"
    try:
        for case in cases.all_pack_cases([(abi.PACK_BF16BF16, 16, 2), (abi.PACK_F32F32, 3, 5)]):
            got, path = G.run_pack_case(case)
            assert path in (abi.PATH_GENERIC, abi.PATH_NONE)
            assert np.array_equal(got, G.oracle_pack(case))
        for case in cases.all_unpack_cases([(abi.UNPACK_I32I32, 16, 16), (abi.UNPACK_F16F16, 6, 7)]):
            got, path = G.run_unpack_case(case)
            assert path in (abi.PATH_GENERIC, abi.PATH_NONE)
            assert np.array_equal(got, G.oracle_unpack(case))
        case = cases.Mmt4dCase(abi.MMT4D_S8S8S32, 16, 16, 2, 8, 16, 64, 1, seed=2, loose=False)
        got, path = G.run_mmt4d_case(case)
        assert path == abi.PATH_GENERIC
        assert np.array_equal(got, G.oracle_mmt4d(case))
    finally:
        del os.environ["IREE_UK_B200_FORCE_GENERIC"]


def test_rejected_parameters_launch_nothing():
    from iree_b200 import ukernel as uk
    case = cases.Mmt4dCase(abi.MMT4D_S8S8S32, 16, 16, 2, 2, 2, 2, 0, loose=False)
    lhs, rhs, out = G.to_device(case.lhs), G.to_device(case.rhs), G.to_device(case.out_init)
    p = case.params(lhs.data_ptr(), rhs.data_ptr(), out.data_ptr())
    p.flags |= 0x800
    with pytest.raises(uk.UkernelError) as e:
        uk.mmt4d(p)
    assert e.value.status == abi.INVALID_ARGUMENT
    import torch
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), case.out_init)


def test_interleave_slabs_kernel():
    """[world][M][N/world][tile] -> [M][N][tile], the step after an all-gather of slabs."""
    import torch
    from iree_b200 import ukernel as uk
    world, M, N, tile = 4, 5, 12, 256
    rng = np.random.default_rng(3)
    gathered = rng.integers(-2**31, 2**31, size=(world, M, N // world, tile), dtype=np.int64)
    gathered = gathered.astype(np.int32)
    want = gathered.transpose(1, 0, 2, 3).reshape(M, N, tile)
    g = torch.from_numpy(gathered).cuda()
    out = torch.zeros(M * N * tile, dtype=torch.int32, device="cuda")
    uk.interleave_slabs(g, out, M, N, tile, 4, world)
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy().reshape(M, N, tile), want)


@pytest.mark.parametrize("spec", [
    (abi.MMT4D_S8S8S32, 16, 16, 2, 24, 40, 64, 1, "exact"),
    (abi.MMT4D_BF16BF16F32, 16, 16, 2, 9, 17, 33, 0, "exact"),
    (abi.MMT4D_S16U4S32, 1, 32, 8, 40, 9, 16, 1, "normal"),
    (abi.MMT4D_S16S16S32, 16, 16, 2, 9, 17, 33, 1, "normal"),
    (abi.MMT4D_S16S8S32, 16, 16, 2, 9, 17, 33, 0, "normal"),
    (abi.MMT4D_S8S4S32, 16, 16, 4, 9, 17, 33, 1, "normal"),
    (abi.MMT4D_S8S8S32, 9, 6, 3, 5, 7, 13, 1, "exact"),
    (abi.MMT4D_F16F16F16, 3, 5, 8, 5, 3, 4, 0, "exact"),
    (abi.MMT4D_S8S8S32, 16, 16, 2, 3, 5, 0, 0, "exact"),
], ids=lambda s: "t%x_%dx%dx%d_%dx%dx%d" % s[:7])
def test_mmt4d_host_buffers(spec):
    """The host-pointer entry point (the reference's own calling convention): loose strides and
    offsets on the host side, chunked and pipelined on the device, whole host output buffer
    bit-identical to the oracle's."""
    import torch
    from iree_b200 import ukernel as uk
    t, M0, N0, K0, M, N, K, acc, mode = spec
    case = cases.Mmt4dCase(t, M0, N0, K0, M, N, K, acc, seed=41, mode=mode, loose=True)
    want = G.oracle_mmt4d(case)
    lhs = torch.from_numpy(case.lhs.copy()).pin_memory()
    rhs = torch.from_numpy(case.rhs.copy()).pin_memory()
    out = torch.from_numpy(case.out_init.copy()).pin_memory()
    p = case.params(lhs.data_ptr(), rhs.data_ptr(), out.data_ptr())
    arena = torch.empty(max(uk.mmt4d_host_arena_size(p), 256), dtype=torch.uint8, device="cuda")
    uk.mmt4d_host(p, arena)
    torch.cuda.synchronize()
    assert np.array_equal(out.numpy(), want)


@pytest.mark.parametrize("spec", [
    (abi.MMT4D_S8S8S32, 16, 16, 2, 24, 40, 64, 1, "exact"),
    (abi.MMT4D_BF16BF16F32, 16, 16, 2, 9, 17, 33, 0, "exact"),
    (abi.MMT4D_S8S8S32, 9, 6, 3, 5, 7, 13, 1, "exact"),
], ids=lambda s: "t%x_%dx%dx%d_%dx%dx%d" % s[:7])
def test_mmt4d_host_buffers_with_device_resident_lhs(spec):
    """The host-pointer entry point with the LHS already on the device (the per-GPU step of the
    sharded host-buffer call): RHS and output stay host buffers with loose strides and offsets,
    the LHS is a device copy with its own row pitch; whole host output equal to the reference's."""
    import torch
    from iree_b200 import ukernel as uk
    t, M0, N0, K0, M, N, K, acc, mode = spec
    case = cases.Mmt4dCase(t, M0, N0, K0, M, N, K, acc, seed=43, mode=mode, loose=True)
    want = G.oracle_mmt4d(case)
    es = cases.KIND_BITS[case.kinds[0]] // 8
    row = K * M0 * K0
    pitch = (row * es + 15) // 16 * 16 // es + 16 // es     # a looser, 16-byte aligned row pitch
    host = np.zeros(M * pitch * es, dtype=np.uint8)
    src = case.lhs[case.lhs_offset * es:]
    for i in range(M):
        host[i * pitch * es:i * pitch * es + row * es] = src[i * case.lhs_stride0 * es:
                                                             i * case.lhs_stride0 * es + row * es]
    d_lhs = torch.from_numpy(host).cuda()
    rhs = torch.from_numpy(case.rhs.copy()).pin_memory()
    out = torch.from_numpy(case.out_init.copy()).pin_memory()
    p = case.params(0, rhs.data_ptr(), out.data_ptr())
    arena = torch.empty(max(uk.mmt4d_host_arena_size(p), 256), dtype=torch.uint8, device="cuda")
    uk.mmt4d_host_resident_lhs(p, d_lhs, pitch, arena)
    torch.cuda.synchronize()
    assert np.array_equal(out.numpy(), want)


@pytest.mark.parametrize("t", [abi.MMT4D_F16F16F32, abi.MMT4D_BF16BF16F32], ids=["f16", "bf16"])
@pytest.mark.parametrize("shape", [(1, 1, 1), (8, 16, 64), (9, 17, 65), (24, 40, 31), (16, 32, 200)],
                         ids=lambda s: "%dx%dx%d" % s)
@pytest.mark.parametrize("accumulate", [0, 1])
def test_mmt4d_tensor_core_without_workspace(t, shape, accumulate):
    """16-bit operands with K0 = 1 reach the tensor cores with no scratch at all: TMA stages
    the [tile][K1][16] panels as MN-major operands."""
    M, N, K = shape
    case = cases.Mmt4dCase(t, 16, 16, 1, M, N, K, accumulate, seed=17, mode="exact", loose=False)
    got, path = G.run_mmt4d_case(case, use_workspace=False)
    assert path == abi.PATH_TCGEN05
    assert np.array_equal(got, G.oracle_mmt4d(case)), case.label()


@pytest.mark.parametrize("tile", [
    (abi.MMT4D_S8S8S32, 1), (abi.MMT4D_S8S8S32, 2), (abi.MMT4D_S8S8S32, 4), (abi.MMT4D_S8S8S32, 8),
    (abi.MMT4D_S8S8S32, 16), (abi.MMT4D_BF16BF16F32, 2), (abi.MMT4D_F16F16F32, 4),
    (abi.MMT4D_BF16BF16F32, 8),
    (abi.MMT4D_BF16BF16BF16 | abi.MMT4D_SKIP_INTERMEDIATE_ROUNDINGS, 2),
], ids=lambda t: "t%x_k0_%d" % t)
@pytest.mark.parametrize("shape", [(1, 1, 1), (8, 16, 64), (9, 17, 65), (24, 40, 31), (3, 50, 300)],
                         ids=lambda s: "%dx%dx%d" % s)
@pytest.mark.parametrize("accumulate", [0, 1])
def test_mmt4d_scratch_free_kernel(tile, shape, accumulate):
    """Every other tensor-core triple without a workspace: the kernel whose producer warps
    re-tile the operands into shared memory themselves. Small-integer values: exact."""
    t, K0 = tile
    M, N, K = shape
    case = cases.Mmt4dCase(t, 16, 16, K0, M, N, K, accumulate, seed=19, mode="exact", loose=False)
    got, path = G.run_mmt4d_case(case, use_workspace=False)
    assert path == abi.PATH_TCGEN05
    assert np.array_equal(got, G.oracle_mmt4d(case)), case.label()


def test_mmt4d_scratch_free_kernel_normal_values():
    case = cases.Mmt4dCase(abi.MMT4D_BF16BF16F32, 16, 16, 2, 40, 24, 300, 1, seed=23, mode="normal",
                           loose=False)
    got, path = G.run_mmt4d_case(case, use_workspace=False)
    assert path == abi.PATH_TCGEN05
    want = G.oracle_mmt4d(case)
    assert cases.rel_frobenius(got.view(np.float32), want.view(np.float32)) <= 1e-3


@pytest.mark.parametrize("t,K0", [(abi.MMT4D_S8S8S32, 2), (abi.MMT4D_BF16BF16F32, 2),
                                  (abi.MMT4D_F16F16F32, 1)], ids=["s8", "bf16", "f16"])
def test_mmt4d_with_prepared_rhs(t, K0):
    """Weights re-tiled once and kept: the prepared form serves calls with different LHS row
    counts, and every result is identical to the ordinary workspace call (and the oracle)."""
    import torch
    from iree_b200 import ukernel as uk
    N, K = 40, 70
    prepared = None
    for M, acc in [(24, 0), (3, 1), (160, 0)]:
        case = cases.Mmt4dCase(t, 16, 16, K0, M, N, K, acc, seed=41, mode="exact", loose=False)
        if prepared is None:
            rhs_host = case.rhs  # the weights: the same for every M below
        case.rhs = rhs_host
        want = G.oracle_mmt4d(case)
        lhs, rhs, out = G.to_device(case.lhs), G.to_device(case.rhs), G.to_device(case.out_init)
        p = case.params(lhs.data_ptr(), rhs.data_ptr(), out.data_ptr())
        if prepared is None:
            prepared = torch.empty(uk.mmt4d_prepared_rhs_size(p), dtype=torch.uint8, device="cuda")
            assert prepared.numel() > 0
            uk.mmt4d_prepare_rhs(p, prepared)
        ws = torch.empty(uk.mmt4d_prepared_workspace_size(p), dtype=torch.uint8, device="cuda")
        assert 0 < ws.numel() < uk.mmt4d_workspace_size(p)
        p.rhs_buffer = 0  # not read once the RHS is prepared
        uk.mmt4d_prepared(p, prepared, ws)
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy(), want), (M, acc)
    G.check_device_status()
    # not applicable: s16s16s32, and an undersized scratch
    c = cases.Mmt4dCase(abi.MMT4D_S16S16S32, 16, 16, 2, 64, 4, 16, 0, seed=1, mode="normal", loose=False)
    assert uk.mmt4d_prepared_rhs_size(c.params(0, 0, 0)) == 0
    with pytest.raises(uk.UkernelError) as e:
        uk.mmt4d_prepared(p, prepared, ws[:256])
    assert e.value.status == abi.WORKSPACE_TOO_SMALL


def test_mmt4d_s16u4_with_prepared_weights():
    """s16u4s32 1x32x8: the u4 weights widened to bytes once and kept. The prepared call runs the
    tensor-core kernel for any number of rows (its pre-pass is then only the byte-plane split of
    the LHS) and gives the reference's bytes, also below the 16 rows from which the ordinary call
    would leave the weight-streaming kernel."""
    import torch
    from iree_b200 import ukernel as uk
    N, K = 9, 40
    prepared, rhs_host = None, None
    for M, acc in [(40, 0), (1, 1), (5, 0), (300, 1)]:
        case = cases.Mmt4dCase(abi.MMT4D_S16U4S32, 1, 32, 8, M, N, K, acc, seed=43, mode="normal",
                               loose=False)
        if rhs_host is None:
            rhs_host = case.rhs
        case.rhs = rhs_host
        want = G.oracle_mmt4d(case)
        lhs, rhs, out = G.to_device(case.lhs), G.to_device(case.rhs), G.to_device(case.out_init)
        p = case.params(lhs.data_ptr(), rhs.data_ptr(), out.data_ptr())
        if prepared is None:
            assert uk.mmt4d_prepared_rhs_size(p) == N * 32 * 384  # K * 8 = 320 bytes, 128-byte pitch
            prepared = torch.empty(uk.mmt4d_prepared_rhs_size(p), dtype=torch.uint8, device="cuda")
            uk.mmt4d_prepare_rhs(p, prepared)
        ws = torch.empty(uk.mmt4d_prepared_workspace_size(p), dtype=torch.uint8, device="cuda")
        assert ws.numel() > 0
        p.rhs_buffer = 0  # not read once the weights are prepared
        uk.mmt4d_prepared(p, prepared, ws)
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy(), want), (M, acc)
    G.check_device_status()


def test_concurrent_host_threads_on_their_own_streams():
    """The library keeps per-device caches behind mutexes and no per-call state: two host
    threads enqueue different problems on their own streams with their own scratch at the
    same time, many times over, and every result is the oracle's."""
    import threading
    import torch
    from iree_b200 import ukernel as uk
    specs = [(abi.MMT4D_S8S8S32, 2, (9, 17, 65)), (abi.MMT4D_BF16BF16F32, 2, (24, 40, 31))]
    errors = []

    def worker(t, K0, shape, use_ws):
        try:
            M, N, K = shape
            case = cases.Mmt4dCase(t, 16, 16, K0, M, N, K, 0, seed=29, mode="exact", loose=False)
            want = G.oracle_mmt4d(case)
            stream = torch.cuda.Stream()
            with torch.cuda.stream(stream):
                lhs, rhs = G.to_device(case.lhs), G.to_device(case.rhs)
                p0 = case.params(lhs.data_ptr(), rhs.data_ptr(), 0)
                ws = torch.empty(max(uk.mmt4d_workspace_size(p0), 256), dtype=torch.uint8,
                                 device="cuda") if use_ws else None
                for _ in range(50):
                    out = G.to_device(case.out_init)
                    p = case.params(lhs.data_ptr(), rhs.data_ptr(), out.data_ptr())
                    uk.mmt4d(p, stream, ws)
                    stream.synchronize()
                    if not np.array_equal(out.cpu().numpy(), want):
                        errors.append(case.label())
                        return
        except Exception as e:  # surfaced by the assertion below
            errors.append(repr(e))

    threads = [threading.Thread(target=worker, args=(t, k0, shape, i % 2 == 0))
               for i, (t, k0, shape) in enumerate(specs * 2)]
    for th in threads:
        th.start()
    for th in threads:
        th.join()
    assert not errors, errors
    G.check_device_status()


@pytest.mark.parametrize("kernel", ["one_cta", "two_cta", "two_cta_streamed", "scratch_free"])
def test_bounded_waits_report_a_timeout_instead_of_hanging(kernel):
    """Failure detection without faulting the GPU: a test hook makes the producers (the TMA warp,
    or the producer warps of the scratch-free kernel) never fill a stage, so the waits of the
    other roles run out (tens of milliseconds with the hook set); every kernel form must record
    the timeout, return, leave the context usable, and the next call must be correct. The
    two-CTA case has more tiles than CTA pairs, so both CTAs of every pair are mid-schedule
    when their waits expire."""
    import torch
    from iree_b200 import ukernel as uk
    if kernel.startswith("two_cta"):
        case = cases.Mmt4dCase(abi.MMT4D_S8S8S32, 16, 16, 2, 320, 96, 4, 0, seed=5, loose=False)
    else:
        case = cases.Mmt4dCase(abi.MMT4D_S8S8S32, 16, 16, 2, 8, 16, 64, 0, seed=5, loose=False)
    want = G.oracle_mmt4d(case)

    def run():
        lhs, rhs, out = G.to_device(case.lhs), G.to_device(case.rhs), G.to_device(case.out_init)
        p = case.params(lhs.data_ptr(), rhs.data_ptr(), out.data_ptr())
        if kernel == "scratch_free":
            assert uk.mmt4d_path(p, False) == abi.PATH_TCGEN05
            uk.mmt4d(p)
        else:
            ws = torch.empty(uk.mmt4d_workspace_size(p), dtype=torch.uint8, device="cuda")
            uk.testing_mmt4d_form(p, ws, FORMS[kernel])
        st, detail = uk.device_status()
        return st, detail, out.cpu().numpy()

    G.check_device_status()
    uk.testing_starve_producers(True)
    try:
        st, detail, _ = run()
    finally:
        uk.testing_starve_producers(False)
    assert st == abi.DEVICE_TIMEOUT and detail != 0, (st, detail)
    st, detail, got = run()
    assert st == abi.OK and detail == 0, (st, detail)
    assert np.array_equal(got, want)


FORMS = {"one_cta": 6, "two_cta": 5, "two_cta_streamed": 7}


@pytest.mark.parametrize("form", list(FORMS))
@pytest.mark.parametrize("t,K0,mode", [(abi.MMT4D_S8S8S32, 2, "exact"), (abi.MMT4D_BF16BF16F32, 2, "exact"),
                                       (abi.MMT4D_F16F16F32, 1, "exact")], ids=["s8", "bf16", "f16"])
@pytest.mark.parametrize("shape", [(1, 1, 1), (17, 9, 65), (40, 33, 130), (100, 40, 257),
                                   # more LHS tile rows than the pre-pass of the streamed form
                                   # covers (its workers re-tile rows 128 and up), ragged K
                                   (200, 40, 130), (300, 20, 33), (40, 500, 33)],
                         ids=lambda s: "%dx%dx%d" % s)
@pytest.mark.parametrize("accumulate", [0, 1])
def test_mmt4d_every_kernel_form_on_small_problems(form, t, K0, mode, shape, accumulate):
    """The library picks the kernel form by problem size; here every form (one CTA per tile, CTA
    pairs after a full pre-pass, CTA pairs whose own workers finish the re-tile behind ready
    counters) runs the same ragged problems and must give the reference's bytes."""
    import torch
    from iree_b200 import ukernel as uk
    M, N, K = shape
    case = cases.Mmt4dCase(t, 16, 16, K0, M, N, K, accumulate, seed=31, mode=mode, loose=False)
    lhs, rhs, out = G.to_device(case.lhs), G.to_device(case.rhs), G.to_device(case.out_init)
    p = case.params(lhs.data_ptr(), rhs.data_ptr(), out.data_ptr())
    ws = torch.empty(uk.mmt4d_workspace_size(p), dtype=torch.uint8, device="cuda")
    uk.testing_mmt4d_form(p, ws, FORMS[form])
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), G.oracle_mmt4d(case)), case.label()
    G.check_device_status()


@pytest.mark.parametrize("shape", [(385, 97, 3), (353, 127, 2), (465, 127, 2), (337, 49, 5)],
                         ids=lambda s: "%dx%dx%d" % s)
@pytest.mark.parametrize("t,K0", [(abi.MMT4D_S8S8S32, 2), (abi.MMT4D_BF16BF16F32, 2)], ids=["s8", "bf16"])
@pytest.mark.parametrize("accumulate", [0, 1])
def test_mmt4d_narrow_tail_tiles(shape, t, K0, accumulate):
    """Tile counts that leave a partial last round over the 74 CTA pairs of a B200: the
    two-CTA kernel cuts the tiles of that round into 2 or 4 narrower ones (accumulator widths
    256, 224, 192 and 160 columns are all covered by these shapes). Ragged M and N edges;
    small-integer values, so the reference's bytes are expected exactly."""
    M, N, K = shape
    case = cases.Mmt4dCase(t, 16, 16, K0, M, N, K, accumulate, seed=37, mode="exact", loose=False)
    got, path = G.run_mmt4d_case(case)
    assert path == abi.PATH_TCGEN05_RETILE
    assert np.array_equal(got, G.oracle_mmt4d(case)), case.label()
    G.check_device_status()


def test_undersized_workspace_is_refused_not_served_by_a_slower_kernel():
    import torch
    from iree_b200 import ukernel as uk
    case = cases.Mmt4dCase(abi.MMT4D_S8S8S32, 16, 16, 2, 8, 16, 64, 0, seed=5, loose=False)
    lhs, rhs, out = G.to_device(case.lhs), G.to_device(case.rhs), G.to_device(case.out_init)
    p = case.params(lhs.data_ptr(), rhs.data_ptr(), out.data_ptr())
    need = uk.mmt4d_workspace_size(p)
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    with pytest.raises(uk.UkernelError) as e:
        uk.mmt4d(p, workspace=ws[:need - 256])
    assert e.value.status == abi.WORKSPACE_TOO_SMALL
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), case.out_init)


def test_mmt4d_pooled_scratch_matches_the_workspace_call():
    """iree_uk_b200_mmt4d_pooled: the same kernels as the workspace call on memory of the
    library's stream-ordered pool; calls back to back, after a trim, and on a second stream."""
    import torch
    from iree_b200 import ukernel as uk
    case = cases.Mmt4dCase(abi.MMT4D_BF16BF16F32, 16, 16, 2, 24, 40, 300, 1, seed=9, mode="exact",
                           loose=False)
    want, path = G.run_mmt4d_case(case)
    assert path == abi.PATH_TCGEN05_RETILE
    side = torch.cuda.Stream()
    for round_ in range(4):
        lhs, rhs, out = G.to_device(case.lhs), G.to_device(case.rhs), G.to_device(case.out_init)
        p = case.params(lhs.data_ptr(), rhs.data_ptr(), out.data_ptr())
        if round_ == 3:
            side.wait_stream(torch.cuda.current_stream())
            uk.mmt4d_pooled(p, stream=side)
        else:
            uk.mmt4d_pooled(p)
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy(), want)
        if round_ == 1:
            uk.scratch_pool_trim(0)
    # a problem without scratch goes the usual way
    small = cases.Mmt4dCase(abi.MMT4D_S8S8S32, 9, 6, 3, 5, 7, 13, 0, seed=2, loose=False)
    lhs, rhs, out = G.to_device(small.lhs), G.to_device(small.rhs), G.to_device(small.out_init)
    uk.mmt4d_pooled(small.params(lhs.data_ptr(), rhs.data_ptr(), out.data_ptr()))
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), G.oracle_mmt4d(small))
