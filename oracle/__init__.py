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
_DEFAULT_REF_SRC = "/root/reference/runtime/src"

_oracle = None
_ref = None


def build(reference_src=None, quiet=True):
    """Compile the C restatement, and the reference ukernels when a checkout is present."""
    out = subprocess.DEVNULL if quiet else None
    subprocess.check_call(["make", "-C", _HERE, "oracle"], stdout=out)
    src = reference_src or os.environ.get("IREE_REFERENCE_SRC", _DEFAULT_REF_SRC)
    if os.path.isdir(os.path.join(src, "iree", "builtins", "ukernel")):
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
