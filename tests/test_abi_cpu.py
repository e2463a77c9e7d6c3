"""Host-side checks that need no GPU: the shared library loads, exports every symbol the
public header declares, rejects what the reference's *_validate functions reject, and
selects kernels as documented."""
import ctypes as C
import os
import re

import pytest

from iree_b200 import abi
from iree_b200 import ukernel as uk
from iree_b200._lib import SIGNATURES, lib
from oracle import cases

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared(header_name):
    header = open(os.path.join(ROOT, "include", header_name)).read()
    return set(re.findall(r"\b(iree_uk_b200_[a-z0-9_]+)\s*\(", header))


def test_library_exports_every_declared_symbol():
    from iree_b200._lib import TESTING_SIGNATURES
    declared = _declared("iree_uk_b200.h")
    assert declared, "no declarations found"
    assert declared == set(SIGNATURES), declared ^ set(SIGNATURES)
    testing = _declared("iree_uk_b200_testing.h")
    assert testing == set(TESTING_SIGNATURES), testing ^ set(TESTING_SIGNATURES)
    for name in declared | testing:
        assert getattr(lib, name) is not None
    assert b"sm_100a" in lib.iree_uk_b200_version()
    # and nothing else is exported under the library's prefix
    import subprocess
    from iree_b200._lib import LIB_PATH
    out = subprocess.run(["nm", "-D", "--defined-only", LIB_PATH], capture_output=True, text=True)
    if out.returncode == 0:
        exported = set(re.findall(r"\b(iree_uk_b200_[a-z0-9_]+)\b", out.stdout))
        assert exported == declared | testing, exported ^ (declared | testing)


def test_workspace_entry_point_reports_bad_arguments_without_launching():
    """A NULL params pointer is an invalid argument, not a crash; an offered workspace that is
    too small for the kernel that would use it is refused instead of being ignored."""
    assert lib.iree_uk_b200_mmt4d_ws(None, 0x40000, 1 << 20, None) == abi.INVALID_ARGUMENT
    assert lib.iree_uk_b200_mmt4d_ws(None, None, 0, None) == abi.INVALID_ARGUMENT
    assert lib.iree_uk_b200_mmt4d_pooled(None, None) == abi.INVALID_ARGUMENT
    p = _mmt4d()
    need = uk.mmt4d_workspace_size(p)
    assert need > 256
    assert lib.iree_uk_b200_mmt4d_ws(C.addressof(p), 0x40000, need - 1, None) == abi.WORKSPACE_TOO_SMALL


def test_struct_layouts_match_reference():
    assert C.sizeof(abi.Mmt4dParams) == 120
    assert C.sizeof(abi.PackParams) == 136
    assert C.sizeof(abi.UnpackParams) == 128
    assert abi.Mmt4dParams.M0.offset == 96 and abi.Mmt4dParams.flags.offset == 108
    assert abi.Mmt4dParams.cpu_data.offset == 112
    assert abi.PackParams.padding_value.offset == 112 and abi.PackParams.flags.offset == 120
    assert abi.UnpackParams.flags.offset == 112 and abi.UnpackParams.cpu_data.offset == 120


def _mmt4d(flags=abi.MMT4D_S8S8S32, M=4, N=4, K=4, M0=16, N0=16, K0=2):
    p = abi.Mmt4dParams()
    p.lhs_buffer, p.rhs_buffer, p.out_buffer = 0x10000, 0x20000, 0x30000
    p.M, p.N, p.K, p.M0, p.N0, p.K0, p.flags = M, N, K, M0, N0, K0, flags
    p.lhs_stride0, p.rhs_stride0, p.out_stride0 = K * M0 * K0, K * N0 * K0, N * M0 * N0
    return p


def test_mmt4d_validation_mirrors_reference():
    # ukernel/mmt4d.c:12-48
    assert uk.mmt4d_path(_mmt4d()) == abi.PATH_TCGEN05_RETILE
    for mutate in (lambda p: setattr(p, "flags", p.flags | 0x800),       # unknown flag bit
                   lambda p: setattr(p, "flags", 0x0B),                  # type id out of range
                   lambda p: setattr(p, "flags", 0x00),                  # no type
                   lambda p: setattr(p, "M", -1),
                   lambda p: setattr(p, "K", 1 << 31),
                   lambda p: setattr(p, "M0", 1 << 15),
                   lambda p: setattr(p, "N0", -1)):
        p = _mmt4d()
        mutate(p)
        with pytest.raises(uk.UkernelError) as e:
            uk.mmt4d_path(p)
        assert e.value.status == abi.INVALID_ARGUMENT
    # u4 right-hand side: K0, stride and offset must be whole bytes
    p = _mmt4d(abi.MMT4D_S16U4S32, M0=1, N0=32, K0=8)
    assert uk.mmt4d_path(p) == abi.PATH_GEMV
    p.rhs_stride0 += 1
    with pytest.raises(uk.UkernelError):
        uk.mmt4d_path(p)
    p = _mmt4d(abi.MMT4D_S16U4S32, M0=5, N0=3, K0=3)
    with pytest.raises(uk.UkernelError):
        uk.mmt4d_path(p)
    # flags 0x200 / 0x400 are accepted and ignored
    p = _mmt4d()
    p.flags |= abi.MMT4D_ALLOW_GENERIC_FALLBACK | abi.MMT4D_SKIP_INTERMEDIATE_ROUNDINGS
    assert uk.mmt4d_path(p) == abi.PATH_TCGEN05_RETILE


def test_mmt4d_early_outs_and_paths():
    # ukernel/mmt4d.c:105-113
    assert uk.mmt4d_path(_mmt4d(M=0)) == abi.PATH_NONE
    assert uk.mmt4d_path(_mmt4d(N=0)) == abi.PATH_NONE
    assert uk.mmt4d_path(_mmt4d(abi.MMT4D_S8S8S32 | abi.MMT4D_ACCUMULATE, K=0)) == abi.PATH_NONE
    assert uk.mmt4d_path(_mmt4d(K=0)) == abi.PATH_ZERO_FILL
    # with a workspace: the re-tile pre-pass and the TMA-fed tensor-core kernels
    assert uk.mmt4d_path(_mmt4d(), with_workspace=True) == abi.PATH_TCGEN05_RETILE
    # without one the tensor-core triples still run on the tensor cores, operands read as they
    # lie (TMA staging for 16-bit K0 = 1, the scratch-free kernel for everything else)
    assert uk.mmt4d_path(_mmt4d(), with_workspace=False) == abi.PATH_TCGEN05
    assert uk.mmt4d_path(_mmt4d(abi.MMT4D_F16F16F32, K0=1), with_workspace=False) == abi.PATH_TCGEN05
    assert uk.mmt4d_path(_mmt4d(abi.MMT4D_BF16BF16F32, K0=2), with_workspace=False) == abi.PATH_TCGEN05
    assert uk.mmt4d_path(_mmt4d(abi.MMT4D_F32F32F32, K0=1), with_workspace=False) == abi.PATH_GENERIC
    # odd tile shapes and misaligned operands go to the generic kernel
    assert uk.mmt4d_path(_mmt4d(M0=9, N0=6, K0=3)) == abi.PATH_GENERIC
    p = _mmt4d()
    p.lhs_offset = 1
    assert uk.mmt4d_path(p) == abi.PATH_GENERIC
    assert uk.mmt4d_path(_mmt4d(abi.MMT4D_F32F32F32, K0=1)) == abi.PATH_GENERIC
    # 16-bit-output triples: generic kernel when every step is rounded, tensor cores when only
    # the final sum is (SKIP_INTERMEDIATE_ROUNDINGS)
    assert uk.mmt4d_path(_mmt4d(abi.MMT4D_F16F16F16, K0=1)) == abi.PATH_GENERIC
    assert uk.mmt4d_path(_mmt4d(abi.MMT4D_F16F16F16 | abi.MMT4D_SKIP_INTERMEDIATE_ROUNDINGS,
                                K0=1)) == abi.PATH_TCGEN05_RETILE
    # f32: CUDA cores unless the process opts into the tf32 x 3 mode
    prev = uk.set_f32_mode(uk.F32_MODE_TF32X3)
    try:
        assert uk.mmt4d_path(_mmt4d(abi.MMT4D_F32F32F32, K0=1)) == abi.PATH_TCGEN05_RETILE
    finally:
        uk.set_f32_mode(prev)
    assert uk.mmt4d_path(_mmt4d(abi.MMT4D_F32F32F32, K0=1)) == abi.PATH_GENERIC
    assert uk.mmt4d_path(_mmt4d(abi.MMT4D_BF16BF16BF16 | abi.MMT4D_SKIP_INTERMEDIATE_ROUNDINGS,
                                K=0)) == abi.PATH_ZERO_FILL


def test_mmt4d_info_and_workspace_size():
    assert uk.mmt4d_info(16, 16, 2, abi.MMT4D_S8S8S32) == 1
    assert uk.mmt4d_info(16, 16, 1, abi.MMT4D_F16F16F32) == 1
    assert uk.mmt4d_info(16, 16, 2, abi.MMT4D_BF16BF16F32) == 1
    assert uk.mmt4d_info(9, 6, 3, abi.MMT4D_S8S8S32) == 0
    assert uk.mmt4d_info(16, 16, 1, abi.MMT4D_F32F32F32) == 0
    assert uk.mmt4d_info(1, 32, 8, abi.MMT4D_S16U4S32) == 1
    big = _mmt4d(abi.MMT4D_S16U4S32, M=64, N=4, K=8, M0=1, N0=32, K0=8)
    assert uk.mmt4d_path(big) == abi.PATH_TCGEN05_RETILE
    assert uk.mmt4d_path(big, with_workspace=False) == abi.PATH_GEMV
    assert uk.mmt4d_workspace_size(big) == 2 * 64 * 128 + 4 * 32 * 128
    # s16s16s32 16x16x2: a high and a low byte plane of both operands, 128-byte row pitch
    s16 = _mmt4d(abi.MMT4D_S16S16S32, M=8, N=4, K=100, M0=16, N0=16, K0=2)
    assert uk.mmt4d_info(16, 16, 2, abi.MMT4D_S16S16S32) == 1
    assert uk.mmt4d_info(8, 8, 2, abi.MMT4D_S16S16S32) == 0
    assert uk.mmt4d_path(s16) == abi.PATH_TCGEN05_RETILE
    assert uk.mmt4d_path(s16, with_workspace=False) == abi.PATH_GENERIC
    assert uk.mmt4d_workspace_size(s16) == 2 * (8 + 4) * 16 * 256
    # s16s8s32 16x16x2: two LHS planes, one RHS plane; s8s4s32: sized like s8s8s32 (widened RHS)
    s16s8 = _mmt4d(abi.MMT4D_S16S8S32, M=8, N=4, K=100, M0=16, N0=16, K0=2)
    assert uk.mmt4d_info(16, 16, 2, abi.MMT4D_S16S8S32) == 1
    assert uk.mmt4d_path(s16s8) == abi.PATH_TCGEN05_RETILE
    assert uk.mmt4d_workspace_size(s16s8) == (2 * 8 + 4) * 16 * 256
    s8s4 = _mmt4d(abi.MMT4D_S8S4S32, M=8, N=4, K=100, M0=16, N0=16, K0=4)
    assert uk.mmt4d_info(16, 16, 4, abi.MMT4D_S8S4S32) == 1 and uk.mmt4d_info(16, 16, 6, abi.MMT4D_S8S4S32) == 0
    assert uk.mmt4d_path(s8s4) == abi.PATH_TCGEN05_RETILE
    assert uk.mmt4d_path(s8s4, with_workspace=False) == abi.PATH_GENERIC
    assert uk.mmt4d_workspace_size(s8s4) == uk.mmt4d_workspace_size(
        _mmt4d(abi.MMT4D_S8S8S32, M=8, N=4, K=100, M0=16, N0=16, K0=4))
    p = _mmt4d(abi.MMT4D_BF16BF16F32, M=512, N=1792, K=4096)
    # row-major copies of both operands, 128-byte row pitch; behind them the job cursor and
    # one ready counter per LHS tile row of the streamed pre-pass
    sync = (4 * (1 + 512) + 1023) // 1024 * 1024
    assert uk.mmt4d_workspace_size(p) == (512 + 1792) * 16 * 4096 * 2 * 2 + sync
    assert uk.mmt4d_workspace_size(_mmt4d(M0=9, N0=6, K0=3)) == 0


def _pack(flags=abi.PACK_F32F32, o=(4, 8), t=(16, 1), in_size=None):
    p = abi.PackParams()
    p.in_buffer, p.out_buffer = 0x10000, 0x20000
    p.flags = flags
    p.out_size0, p.out_size1, p.out_size2, p.out_size3 = o[0], o[1], t[0], t[1]
    p.out_stride1 = t[0] * t[1]
    p.out_stride0 = o[1] * p.out_stride1
    p.in_size0, p.in_size1 = in_size or (o[0] * t[0], o[1] * t[1])
    p.in_stride0, p.in_stride1 = p.in_size1, 1
    return p


def test_pack_validation_mirrors_reference():
    # ukernel/pack.c:51-104
    assert uk.pack_path(_pack()) == abi.PATH_FAST_COPY
    assert uk.pack_path(_pack(o=(0, 3))) == abi.PATH_NONE
    bad = [lambda p: setattr(p, "flags", 0x06), lambda p: setattr(p, "flags", p.flags | 0x400),
           lambda p: setattr(p, "out_stride1", 17), lambda p: setattr(p, "in_size0", 65),
           lambda p: setattr(p, "in_stride0", -1)]
    for mutate in bad:
        p = _pack()
        mutate(p)
        with pytest.raises(uk.UkernelError) as e:
            uk.pack_path(p)
        assert e.value.status == abi.INVALID_ARGUMENT
    # a tile larger than the reference's 4096-byte temporary is rejected (pack.c:9,43-46)
    with pytest.raises(uk.UkernelError):
        uk.pack_path(_pack(t=(64, 32)))
    assert uk.pack_path(_pack(t=(32, 32))) == abi.PATH_FAST_COPY


def test_unpack_validation_mirrors_reference():
    # ukernel/unpack.c:31-82
    p = abi.UnpackParams()
    p.in_buffer, p.out_buffer = 0x10000, 0x20000
    p.flags = abi.UNPACK_I32I32
    p.in_size0, p.in_size1, p.in_size2, p.in_size3 = 4, 4, 16, 16
    p.in_stride1, p.in_stride0 = 256, 1024
    p.out_size0, p.out_size1, p.out_stride0, p.out_stride1 = 64, 64, 64, 1
    assert uk.unpack_path(p) == abi.PATH_FAST_COPY
    p.flags = 0x02  # I8I8 exists for pack only (exported_bits.h:76)
    with pytest.raises(uk.UkernelError):
        uk.unpack_path(p)
    p.flags = abi.UNPACK_I32I32
    p.out_size0 = 65
    with pytest.raises(uk.UkernelError):
        uk.unpack_path(p)
    p.out_size0 = 0
    assert uk.unpack_path(p) == abi.PATH_NONE


def test_query_tile_sizes():
    # roles: LHS -> (M0,K0), RHS -> (N0,K0), RESULT -> (M0,N0)  (query_tile_sizes.c:43-63)
    assert uk.query_tile_sizes_2d(0x0201) == (16, 2)
    assert uk.query_tile_sizes_2d(0x0502) == (16, 2)
    assert uk.query_tile_sizes_2d(0x0303) == (16, 16)
    assert uk.query_tile_sizes_2d(0x0301) == (16, 1)
    with pytest.raises(uk.UkernelError):
        uk.query_tile_sizes_2d(0x0701)
    with pytest.raises(uk.UkernelError):
        uk.query_tile_sizes_2d(0x0204)


def test_query_tile_sizes_reference_answers_under_the_compat_flag():
    """With the compat flag the call answers what the reference's x86-64 build answers for a
    cpu_data word; checked against the compiled reference itself where it is present, for every
    operation, role and feature level."""
    import oracle
    bit = lambda *bs: sum(1 << b for b in bs)
    avx2 = bit(15, 11, 14)
    avx512 = avx2 | bit(20, 21, 22, 23, 24)
    levels = [0, avx2, avx512, avx512 | bit(28), avx512 | bit(28, 31)]
    expect_f32 = {0: (8, 1, 4), avx2: (8, 1, 8)}
    for d in levels:
        for op in range(1, 7):
            for role in (1, 2, 3):
                flags = (op << 8) | role
                got = uk.query_tile_sizes_2d(flags | uk.QUERY_REFERENCE_X86_64, cpu_data0=d)
                if oracle.ref_available():
                    assert got == oracle.query_tile_sizes_2d_ref(flags, d), (hex(d), op, role)
    assert uk.query_tile_sizes_2d(0x0103 | uk.QUERY_REFERENCE_X86_64, cpu_data0=0) == (8, 4)
    assert uk.query_tile_sizes_2d(0x0203 | uk.QUERY_REFERENCE_X86_64, cpu_data0=avx512 | bit(28)) == (16, 16)
    assert uk.query_tile_sizes_2d(0x0501 | uk.QUERY_REFERENCE_X86_64, cpu_data0=avx512) == (8, 4)
    with pytest.raises(uk.UkernelError):   # the compat answer needs cpu_data
        uk.query_tile_sizes_2d(0x0101 | uk.QUERY_REFERENCE_X86_64)


def test_shard_params_partition_n():
    full = _mmt4d(abi.MMT4D_BF16BF16F32, M=8, N=30, K=16)
    covered = []
    for world in (1, 2, 4, 8):
        nb = 0
        for r in range(world):
            sh, begin = uk.shard_params(full, r, world, rhs_is_local=False, out_is_local=False)
            assert begin == nb
            assert sh.rhs_offset == full.rhs_offset + begin * full.rhs_stride0
            assert sh.out_offset == full.out_offset + begin * 256
            assert sh.out_stride0 == full.out_stride0 and sh.M == full.M and sh.K == full.K
            nb += sh.N
            sl, _ = uk.shard_params(full, r, world, rhs_is_local=True, out_is_local=True)
            assert sl.rhs_offset == full.rhs_offset and sl.out_stride0 == sl.N * 256
        assert nb == full.N
        covered.append(world)
    with pytest.raises(uk.UkernelError):
        uk.shard_params(full, 2, 2)


def test_status_strings():
    assert lib.iree_uk_b200_status_string(0) == b"OK"
    assert lib.iree_uk_b200_status_string(abi.DEVICE_TIMEOUT) == b"DEVICE_TIMEOUT"


def test_scratch_sizes_are_consistent():
    """Sizes depend on the shape and type only: the ordinary scratch is the LHS part plus the
    RHS part that a caller may instead prepare once (each scratch ends with the small block of
    counters of the streamed pre-pass); f32 in its tensor-core mode needs two planes of each;
    triples without a tensor-core path need none."""
    p = _mmt4d(abi.MMT4D_BF16BF16F32, M=512, N=1792, K=4096)
    sync = (4 * (1 + 512) + 1023) // 1024 * 1024
    whole = uk.mmt4d_workspace_size(p)
    assert whole == (512 + 1792) * 16 * 8192 * 2 + sync   # the headline problem: 576 MiB
    assert uk.mmt4d_prepared_rhs_size(p) + uk.mmt4d_prepared_workspace_size(p) == whole
    assert uk.mmt4d_prepared_rhs_size(p) == 1792 * 16 * 8192 * 2
    q = _mmt4d(abi.MMT4D_BF16BF16F32, M=7, N=1792, K=4096)   # another M, the same weights
    assert uk.mmt4d_prepared_rhs_size(q) == uk.mmt4d_prepared_rhs_size(p)
    assert uk.mmt4d_workspace_size(_mmt4d(M0=8, N0=8)) == 0
    # s16u4s32: the prepared form is the weights widened to bytes, the scratch then the two LHS planes
    s = _mmt4d(abi.MMT4D_S16U4S32, M=64, N=4, K=16, M0=1, N0=32, K0=8)
    assert uk.mmt4d_prepared_rhs_size(s) == 4 * 32 * 128
    assert uk.mmt4d_prepared_workspace_size(s) == 2 * 64 * 128
    assert uk.mmt4d_prepared_rhs_size(s) + uk.mmt4d_prepared_workspace_size(s) == uk.mmt4d_workspace_size(s)
    assert uk.mmt4d_prepared_rhs_size(_mmt4d(abi.MMT4D_S16S16S32, M0=16, N0=16, K0=2)) == 0
    f = _mmt4d(abi.MMT4D_F32F32F32, K0=1)
    assert uk.mmt4d_workspace_size(f) == 0
    prev = uk.set_f32_mode(uk.F32_MODE_TF32X3)
    try:
        assert uk.mmt4d_workspace_size(f) == 2 * (4 + 4) * 16 * 128 + 1024
        assert uk.mmt4d_prepared_rhs_size(f) == 0
    finally:
        uk.set_f32_mode(prev)


def test_header_compiles_as_c_and_cxx_and_struct_sizes_match_the_reference(tmp_path):
    """include/iree_uk_b200.h is plain C usable from C++ (the reference's own common.h refuses
    C++, ukernel/common.h:10-12), and a C program sees the reference's struct sizes: 120 / 136 /
    128 bytes (mmt4d_internal.h:14-32, pack_internal.h:12-30, unpack_internal.h:12-29)."""
    import shutil
    import subprocess
    header = os.path.join(ROOT, "include", "iree_uk_b200.h")
    if not shutil.which("gcc") or not shutil.which("g++"):
        pytest.skip("no host compiler")
    subprocess.check_call(["gcc", "-std=c11", "-Wall", "-Werror", "-fsyntax-only", "-x", "c", header])
    subprocess.check_call(["g++", "-std=c++17", "-Wall", "-Werror", "-fsyntax-only", "-x", "c++", header])
    src = tmp_path / "sizes.c"
    src.write_text('#include <stdio.h>\n#include "iree_uk_b200.h"\n'
                   'int main(void) { printf("%zu %zu %zu %zu\\n", sizeof(iree_uk_mmt4d_params_t), '
                   'sizeof(iree_uk_pack_params_t), sizeof(iree_uk_unpack_params_t), '
                   'sizeof(iree_uk_b200_matmul_params_t)); return 0; }\n')
    exe = tmp_path / "sizes"
    subprocess.check_call(["gcc", "-std=c11", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)])
    out = subprocess.check_output([str(exe)], text=True).split()
    assert out[:3] == ["120", "136", "128"]
    assert int(out[3]) == C.sizeof(abi.MatmulParams)
