"""Loads ``libiree_uk_b200.so`` and declares the C ABI of ``include/iree_uk_b200.h``.

There is no fallback: if the shared library is missing or lacks a symbol, importing this
module raises. Build it with ``python -m iree_b200.build``.
"""
import ctypes as C
import os

from . import abi

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libiree_uk_b200.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        "%s not found: the CUDA library is not built (python -m iree_b200.build). "
        "There is no CPU or PyTorch fallback for this path." % LIB_PATH)

lib = C.CDLL(LIB_PATH)

_P, _I, _i32, _u32, _u64, _sz = C.c_void_p, abi.index_t, C.c_int32, C.c_uint32, C.c_uint64, C.c_size_t

#: every symbol the public header declares: name -> (restype, argtypes)
SIGNATURES = {
    "iree_uk_b200_status_string": (C.c_char_p, [C.c_int]),
    "iree_uk_b200_version": (C.c_char_p, []),
    "iree_uk_b200_mmt4d": (C.c_int, [_P, _P]),
    "iree_uk_b200_mmt4d_workspace_size": (_sz, [_P]),
    "iree_uk_b200_mmt4d_ws": (C.c_int, [_P, _P, _sz, _P]),
    "iree_uk_b200_mmt4d_static_scratch": (C.c_int, [_P, _P]),
    "iree_uk_b200_mmt4d_pooled": (C.c_int, [_P, _P]),
    "iree_uk_b200_scratch_pool_trim": (C.c_int, [C.c_size_t]),
    "iree_uk_b200_mmt4d_host_arena_size": (_sz, [_P]),
    "iree_uk_b200_mmt4d_host": (C.c_int, [_P, _P, _sz, _P]),
    "iree_uk_b200_mmt4d_host_resident_lhs": (C.c_int, [_P, _P, _I, _P, _sz, _P]),
    "iree_uk_b200_mmt4d_ws_peers": (C.c_int, [_P, _P, C.c_int, _P, _sz, _P]),
    "iree_uk_b200_mmt4d_ws_multicast": (C.c_int, [_P, _P, _P, _sz, _P]),
    "iree_uk_b200_mmt4d_ws_unpacked": (C.c_int, [_P, _I, _I, _P, _sz, _P]),
    "iree_uk_b200_mmt4d_prepared_rhs_size": (_sz, [_P]),
    "iree_uk_b200_mmt4d_prepared_workspace_size": (_sz, [_P]),
    "iree_uk_b200_mmt4d_prepare_rhs": (C.c_int, [_P, _P, _sz, _P]),
    "iree_uk_b200_mmt4d_ws_prepared": (C.c_int, [_P, _P, _P, _sz, _P]),
    "iree_uk_b200_set_f32_mode": (C.c_int, [C.c_int]),
    "iree_uk_b200_mmt4d_sharded": (C.c_int, [C.c_int, _P, _P, _P, _P, _P, C.c_int]),
    "iree_uk_b200_peer_export": (C.c_int, [_P, _P]),
    "iree_uk_b200_peer_open": (C.c_int, [_P, _P]),
    "iree_uk_b200_peer_close": (C.c_int, [_P]),
    "iree_uk_b200_matmul_workspace_size": (_sz, [_P]),
    "iree_uk_b200_matmul": (C.c_int, [_P, _P, _sz, _P]),
    "iree_uk_b200_mmt4d_flat": (C.c_int, [_P, _I, _I, _P, _I, _I, _P, _I, _I, _I, _I, _I, _i32,
                                          _i32, _i32, _u32, _P, _P, _sz, _P]),
    "iree_uk_b200_mmt4d_info": (_u32, [_i32, _i32, _i32, _u32]),
    "iree_uk_b200_mmt4d_path": (C.c_int, [_P, C.c_int]),
    "iree_uk_b200_mmt4d_shard_params": (C.c_int, [_P, C.c_int, C.c_int, C.c_int, C.c_int, _P, _P]),
    "iree_uk_b200_interleave_slabs": (C.c_int, [_P, _P, _I, _I, _I, C.c_int, C.c_int, _P]),
    "iree_uk_b200_pack": (C.c_int, [_P, _P]),
    "iree_uk_b200_pack_flat": (C.c_int, [_P, _I, _I, _I, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I,
                                         _u64, _u32, _P, _P]),
    "iree_uk_b200_pack_path": (C.c_int, [_P]),
    "iree_uk_b200_unpack": (C.c_int, [_P, _P]),
    "iree_uk_b200_unpack_flat": (C.c_int, [_P, _I, _I, _I, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I,
                                           _u32, _P, _P]),
    "iree_uk_b200_unpack_path": (C.c_int, [_P]),
    "iree_uk_b200_query_tile_sizes_2d": (C.c_int, [_P, _P]),
    "iree_uk_b200_device_status": (C.c_int, [_P, _P]),
    "iree_uk_b200_kernel_timing": (C.c_int, [C.c_int]),
    "iree_uk_b200_kernel_timing_mean_ms": (C.c_int, [_P, _P, _P]),
}

for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)  # AttributeError if the library lacks a declared symbol
    _fn.restype = _res
    _fn.argtypes = _args

# test hooks, declared in include/iree_uk_b200_testing.h
TESTING_SIGNATURES = {
    "iree_uk_b200_testing_starve_producers": (C.c_int, [C.c_int]),
    "iree_uk_b200_testing_mmt4d_form": (C.c_int, [_P, _P, _sz, C.c_int, _P]),
}
for _name, (_res, _args) in TESTING_SIGNATURES.items():
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args
