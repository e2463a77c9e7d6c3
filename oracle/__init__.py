"""CPU checkers for the mmt4d / pack / unpack path. TEST INFRASTRUCTURE ONLY.

Two implementations sit behind one interface (ctypes params structs holding HOST
pointers):

* ``impl="oracle"`` — ``libuk_oracle.so``, the plain-C restatement in ``uk_oracle.c``;
* ``impl="ref"``    — ``_ref/libiree_uk_ref.so``, the reference ukernels themselves,
  compiled in place from a reference checkout by ``make ref`` (present only where that
  checkout was available at build time; ``ref_available()`` tells).

Only the tests, the smoke check and the bench's CPU-baseline legs import this package;
the shipped library never does.
"""
import ctypes as C
import os
import subprocess
from concurrent.futures import ThreadPoolExecutor

from iree_b200 import abi

_HERE = os.path.dirname(os.path.abspath(__file__))
_ORACLE_SO = os.path.join(_HERE, "libuk_oracle.so")
_REF_SO = os.path.join(_HERE, "_ref", "libiree_uk_ref.so")


def _reference_src():
    """``runtime/src`` of a reference checkout: the IREE_REFERENCE_SRC environment variable, or
    a checkout named ``reference`` beside this repository; None when neither exists."""
    cands = [os.environ.get("IREE_REFERENCE_SRC"),
             os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference", "runtime", "src")]
    for c in cands:
        if c and os.path.isdir(os.path.join(c, "iree", "builtins", "ukernel")):
            return c
    return None

_oracle = None
_ref = None


def build(reference_src=None, quiet=True):
    """Compile the C restatement, and the reference ukernels when a checkout is present."""
    out = subprocess.DEVNULL if quiet else None
    subprocess.check_call(["make", "-C", _HERE, "oracle"], stdout=out)
    src = reference_src or _reference_src()
    if src:
        subprocess.check_call(["make", "-C", _HERE, "ref", "REF=" + src], stdout=out)


def lib():
    """The C restatement, built on first use if the shared object is missing."""
    global _oracle
    if _oracle is None:
        if not os.path.exists(_ORACLE_SO):
            subprocess.check_call(["make", "-C", _HERE, "oracle"], stdout=subprocess.DEVNULL)
        _oracle = C.CDLL(_ORACLE_SO)
        for name in ("uk_oracle_mmt4d", "uk_oracle_pack", "uk_oracle_unpack"):
            getattr(_oracle, name).restype = C.c_int
            getattr(_oracle, name).argtypes = [C.c_void_p]
    return _oracle


def ref_available():
    return os.path.exists(_REF_SO)


def ref():
    """The compiled reference ukernels (None when they were not built)."""
    global _ref
    if _ref is None and ref_available():
        _ref = C.CDLL(_REF_SO)
        I, P = abi.index_t, C.c_void_p
        _ref.iree_uk_mmt4d.restype = None
        _ref.iree_uk_mmt4d.argtypes = [P, I, I, P, I, I, P, I, I, I, I, I, C.c_int32,
                                       C.c_int32, C.c_int32, C.c_uint32, P]
        _ref.iree_uk_mmt4d_info.restype = C.c_uint32
        _ref.iree_uk_mmt4d_info.argtypes = [C.c_int32, C.c_int32, C.c_int32, C.c_uint32, P]
        _ref.iree_uk_pack.restype = None
        _ref.iree_uk_pack.argtypes = [P, I, I, I, P, I, I, I, I, I, I, I, I, I, C.c_uint64,
                                      C.c_uint32, P]
        _ref.iree_uk_unpack.restype = None
        _ref.iree_uk_unpack.argtypes = [P, I, I, I, P, I, I, I, I, I, I, I, I, I,
                                        C.c_uint32, P]
    return _ref


# cpu_data[0] bit positions, runtime/src/iree/schemas/cpu_feature_bits.inl:85-112
_X86_BITS = {"sse3": 0, "ssse3": 1, "sse4_1": 2, "sse4_2": 3, "sse4a": 4, "avx": 10,
             "fma": 11, "fma4": 12, "xop": 13, "f16c": 14, "avx2": 15, "avx512f": 20,
             "avx512cd": 21, "avx512vl": 22, "avx512dq": 23, "avx512bw": 24,
             "avx512ifma": 25, "avx512vbmi": 26, "avx512_vpopcntdq": 27, "avx512_vnni": 28,
             "avx512_vbmi2": 29, "avx512_bitalg": 30, "avx512_bf16": 31, "avx512_fp16": 32}
_cpu_data = None


def cpu_data(features="host"):
    """A uint64[8] ``cpu_data`` array: the running host's features, or all zero
    (``features="none"``), which with ALLOW_GENERIC_FALLBACK forces the reference's
    portable tile functions (ukernel/mmt4d.c:124-138)."""
    global _cpu_data
    arr = (C.c_uint64 * 8)()
    if features == "none":
        return arr
    if _cpu_data is None:
        word = 0
        try:
            with open("/proc/cpuinfo") as f:
                for line in f:
                    if line.startswith("flags"):
                        flags = set(line.split(":", 1)[1].split())
                        for name, bit in _X86_BITS.items():
                            if name in flags:
                                word |= 1 << bit
                        break
        except OSError:
            pass
        _cpu_data = word
    arr[0] = _cpu_data
    return arr


def mmt4d(p, impl="oracle", features="host"):
    """Run mmt4d on host buffers described by an ``abi.Mmt4dParams``."""
    if impl == "oracle":
        rc = lib().uk_oracle_mmt4d(C.addressof(p))
        if rc:
            raise ValueError("type triple not restated in the oracle: 0x%x" % p.flags)
        return
    cd = cpu_data(features)
    ref().iree_uk_mmt4d(p.lhs_buffer, p.lhs_offset, p.lhs_stride0, p.rhs_buffer, p.rhs_offset,
                        p.rhs_stride0, p.out_buffer, p.out_offset, p.out_stride0, p.M, p.N,
                        p.K, p.M0, p.N0, p.K0, p.flags | abi.MMT4D_ALLOW_GENERIC_FALLBACK,
                        C.addressof(cd))


def mmt4d_info(M0, N0, K0, flags, features="host"):
    """Bit 0: the compiled reference has an ISA-specific tile function for this shape."""
    cd = cpu_data(features)
    return ref().iree_uk_mmt4d_info(M0, N0, K0, flags, C.addressof(cd))


def pack(p, impl="oracle", features="host"):
    if impl == "oracle":
        if lib().uk_oracle_pack(C.addressof(p)):
            raise ValueError("bad pack type 0x%x" % p.flags)
        return
    cd = cpu_data(features)
    ref().iree_uk_pack(p.in_buffer, p.in_offset, p.in_stride0, p.in_stride1, p.out_buffer,
                       p.out_offset, p.out_stride0, p.out_stride1, p.in_size0, p.in_size1,
                       p.out_size0, p.out_size1, p.out_size2, p.out_size3, p.padding_value,
                       p.flags, C.addressof(cd))


def unpack(p, impl="oracle", features="host"):
    if impl == "oracle":
        if lib().uk_oracle_unpack(C.addressof(p)):
            raise ValueError("bad unpack type 0x%x" % p.flags)
        return
    cd = cpu_data(features)
    ref().iree_uk_unpack(p.in_buffer, p.in_offset, p.in_stride0, p.in_stride1, p.out_buffer,
                         p.out_offset, p.out_stride0, p.out_stride1, p.in_size0, p.in_size1,
                         p.in_size2, p.in_size3, p.out_size0, p.out_size1, p.flags,
                         C.addressof(cd))


def query_tile_sizes_2d_ref(flags, cpu_data0):
    """The compiled reference's iree_uk_query_tile_sizes_2d for one cpu_data[0] word:
    (tile_size0, tile_size1)."""
    r = ref()
    cd = (C.c_uint64 * 8)(cpu_data0)
    p = abi.QueryTileSizes2dParams(flags=flags, size0=0, size1=0, cpu_data=C.cast(cd, C.c_void_p))
    o = abi.QueryTileSizes2dOut()
    r.iree_uk_query_tile_sizes_2d.restype = None
    r.iree_uk_query_tile_sizes_2d.argtypes = [C.c_void_p, C.c_void_p]
    r.iree_uk_query_tile_sizes_2d(C.addressof(p), C.addressof(o))
    return int(o.tile_size0), int(o.tile_size1)


def _chunks(total, parts):
    parts = max(1, min(parts, total))
    base, rem = divmod(total, parts)
    begin = 0
    for i in range(parts):
        size = base + (1 if i < rem else 0)
        yield begin, size
        begin += size


def mmt4d_threaded(p, threads, impl="ref"):
    """mmt4d across ``threads`` host threads. The ukernel is single-threaded by design and
    callers slice the work (ukernel/README.md:26): tile rows (M) are split into contiguous
    chunks, one per thread, by advancing lhs_offset / out_offset; a single-row problem
    (the GEMV case) splits N instead. ctypes releases the GIL during each call."""
    jobs = []
    if p.M > 1 or p.N <= 1:
        for begin, size in _chunks(p.M, threads):
            q = abi.copy_params(p)
            q.M = size
            q.lhs_offset = p.lhs_offset + begin * p.lhs_stride0
            q.out_offset = p.out_offset + begin * p.out_stride0
            jobs.append(q)
    else:
        for begin, size in _chunks(p.N, threads):
            q = abi.copy_params(p)
            q.N = size
            q.rhs_offset = p.rhs_offset + begin * p.rhs_stride0
            q.out_offset = p.out_offset + begin * p.M0 * p.N0
            jobs.append(q)
    if len(jobs) <= 1:
        for q in jobs:
            mmt4d(q, impl)
        return len(jobs)
    with ThreadPoolExecutor(len(jobs)) as ex:
        list(ex.map(lambda q: mmt4d(q, impl), jobs))
    return len(jobs)


def matmul_chain(lhs, rhs, acc, type_flag, M0, N0, K0, impl="oracle"):
    """Row-major matmul through the chain of ukernel/tools/e2e_matmul_benchmark.c:173-300:
    pack the LHS, pack the RHS with TRANSPOSE_INNER | TRANSPOSE_OUTER, pack the accumulator
    (when ``acc`` is given, which also sets ACCUMULATE), mmt4d, unpack; padding is zero.
    ``lhs`` [M][K], ``rhs`` [K][N] and ``acc`` [M][N] are C-contiguous numpy arrays whose
    item sizes match the type triple (int8 / uint16 bit patterns for f16 and bf16; int32 or
    float32 for ``acc``). Returns the [M][N] result."""
    import numpy as np
    pack_in = {abi.MMT4D_S8S8S32: abi.PACK_I8I8, abi.MMT4D_F16F16F32: abi.PACK_F16F16,
               abi.MMT4D_BF16BF16F32: abi.PACK_BF16BF16}[type_flag]
    is_int = type_flag == abi.MMT4D_S8S8S32
    pack_out = abi.PACK_I32I32 if is_int else abi.PACK_F32F32
    unpack_out = abi.UNPACK_I32I32 if is_int else abi.UNPACK_F32F32
    out_dtype = np.int32 if is_int else np.float32
    M, K = lhs.shape
    K2, N = rhs.shape
    assert K == K2
    M1, N1, K1 = -(-M // M0), -(-N // N0), -(-K // K0)
    packed_lhs = np.zeros(M1 * K1 * M0 * K0, dtype=lhs.dtype)
    packed_rhs = np.zeros(N1 * K1 * N0 * K0, dtype=rhs.dtype)
    packed_out = np.zeros(M1 * N1 * M0 * N0, dtype=out_dtype)
    result = np.zeros((M, N), dtype=out_dtype)

    def pack_params(src, dst, flags, s0, s1, o0, o1, t0, t1):
        p = abi.PackParams()
        p.in_buffer, p.out_buffer = src.ctypes.data, dst.ctypes.data
        p.in_size0, p.in_size1, p.in_stride0, p.in_stride1 = s0, s1, s1, 1
        p.out_size0, p.out_size1, p.out_size2, p.out_size3 = o0, o1, t0, t1
        p.out_stride1 = t0 * t1
        p.out_stride0 = o1 * t0 * t1
        p.padding_value, p.flags = 0, flags
        return p

    lhs, rhs = np.ascontiguousarray(lhs), np.ascontiguousarray(rhs)
    pack(pack_params(lhs, packed_lhs, pack_in, M, K, M1, K1, M0, K0), impl)
    pack(pack_params(rhs, packed_rhs,
                     pack_in | abi.PACK_TRANSPOSE_INNER | abi.PACK_TRANSPOSE_OUTER,
                     K, N, N1, K1, N0, K0), impl)
    flags = type_flag
    if acc is not None:
        acc = np.ascontiguousarray(acc.astype(out_dtype, copy=False))
        pack(pack_params(acc, packed_out, pack_out, M, N, M1, N1, M0, N0), impl)
        flags |= abi.MMT4D_ACCUMULATE
    q = abi.Mmt4dParams()
    q.lhs_buffer, q.rhs_buffer, q.out_buffer = (packed_lhs.ctypes.data, packed_rhs.ctypes.data,
                                                packed_out.ctypes.data)
    q.M, q.N, q.K, q.M0, q.N0, q.K0, q.flags = M1, N1, K1, M0, N0, K0, flags
    q.lhs_stride0, q.rhs_stride0, q.out_stride0 = K1 * M0 * K0, K1 * N0 * K0, N1 * M0 * N0
    mmt4d(q, impl)
    u = abi.UnpackParams()
    u.in_buffer, u.out_buffer = packed_out.ctypes.data, result.ctypes.data
    u.in_size0, u.in_size1, u.in_size2, u.in_size3 = M1, N1, M0, N0
    u.in_stride1, u.in_stride0 = M0 * N0, N1 * M0 * N0
    u.out_size0, u.out_size1, u.out_stride0, u.out_stride1 = M, N, N, 1
    u.flags = unpack_out
    unpack(u, impl)
    return result
