"""ctypes view of ``include/iree_uk_b200.h``: flag constants and parameter structs.

The structs are field-for-field the reference's
(runtime/src/iree/builtins/ukernel/mmt4d_internal.h:14-32, pack_internal.h:12-30,
unpack_internal.h:12-29), so the same ``Structure`` instance can be handed to this
library (device pointers) or to a CPU implementation of the ukernels (host pointers).
Flag values are the frozen ones of ukernel/exported_bits.h:29-83.
"""
import ctypes as C

index_t = C.c_int64

# --- mmt4d flags (exported_bits.h:29-46) ---
MMT4D_TYPE_MASK = 0xFF
MMT4D_F32F32F32 = 0x01
MMT4D_S8S8S32 = 0x02
MMT4D_F16F16F32 = 0x03
MMT4D_F16F16F16 = 0x04
MMT4D_BF16BF16F32 = 0x05
MMT4D_BF16BF16BF16 = 0x06
MMT4D_S16S16S32 = 0x07
MMT4D_S16U4S32 = 0x08
MMT4D_S16S8S32 = 0x09
MMT4D_S8S4S32 = 0x0A
MMT4D_ACCUMULATE = 0x100
MMT4D_ALLOW_GENERIC_FALLBACK = 0x200
MMT4D_SKIP_INTERMEDIATE_ROUNDINGS = 0x400

# --- pack flags (exported_bits.h:56-66) ---
PACK_F32F32 = 0x01
PACK_I8I8 = 0x02
PACK_I32I32 = 0x03
PACK_F16F16 = 0x04
PACK_BF16BF16 = 0x05
PACK_TRANSPOSE_INNER = 0x100
PACK_TRANSPOSE_OUTER = 0x200

# --- unpack flags (exported_bits.h:73-83) ---
UNPACK_F32F32 = 0x01
UNPACK_I32I32 = 0x03
UNPACK_F16F16 = 0x04
UNPACK_BF16BF16 = 0x05
UNPACK_TRANSPOSE_INNER = 0x100
UNPACK_TRANSPOSE_OUTER = 0x200

# status codes (iree_uk_b200_status_t)
OK, INVALID_ARGUMENT, UNSUPPORTED, CUDA_ERROR, WORKSPACE_TOO_SMALL, DEVICE_TIMEOUT = range(6)

# kernel paths (iree_uk_b200_path_t)
PATH_NONE, PATH_GENERIC, PATH_TCGEN05, PATH_TCGEN05_RETILE, PATH_GEMV, PATH_FAST_COPY, \
    PATH_ZERO_FILL = range(7)

#: bits per element of (lhs, rhs, out) per mmt4d type id (mmt4d_internal.h:40-61)
MMT4D_BITS = {
    MMT4D_F32F32F32: (32, 32, 32), MMT4D_S8S8S32: (8, 8, 32), MMT4D_F16F16F32: (16, 16, 32),
    MMT4D_F16F16F16: (16, 16, 16), MMT4D_BF16BF16F32: (16, 16, 32),
    MMT4D_BF16BF16BF16: (16, 16, 16), MMT4D_S16S16S32: (16, 16, 32),
    MMT4D_S16U4S32: (16, 4, 32), MMT4D_S16S8S32: (16, 8, 32), MMT4D_S8S4S32: (8, 4, 32),
}
#: bytes per element per pack / unpack type id (pack_internal.h:34-41)
PACK_ELEM_SIZE = {PACK_F32F32: 4, PACK_I8I8: 1, PACK_I32I32: 4, PACK_F16F16: 2,
                  PACK_BF16BF16: 2}
UNPACK_ELEM_SIZE = {UNPACK_F32F32: 4, UNPACK_I32I32: 4, UNPACK_F16F16: 2, UNPACK_BF16BF16: 2}


class Mmt4dParams(C.Structure):
    """iree_uk_mmt4d_params_t (120 bytes)."""
    _fields_ = [
        ("lhs_buffer", C.c_void_p), ("lhs_offset", index_t), ("lhs_stride0", index_t),
        ("rhs_buffer", C.c_void_p), ("rhs_offset", index_t), ("rhs_stride0", index_t),
        ("out_buffer", C.c_void_p), ("out_offset", index_t), ("out_stride0", index_t),
        ("M", index_t), ("N", index_t), ("K", index_t),
        ("M0", C.c_int32), ("N0", C.c_int32), ("K0", C.c_int32),
        ("flags", C.c_uint32), ("cpu_data", C.c_void_p),
    ]


class MatmulParams(C.Structure):
    """iree_uk_b200_matmul_params_t: row-major lhs [M][K], rhs [K][N], out [M][N]."""
    _fields_ = [
        ("lhs_buffer", C.c_void_p), ("lhs_offset", index_t), ("lhs_stride0", index_t),
        ("rhs_buffer", C.c_void_p), ("rhs_offset", index_t), ("rhs_stride0", index_t),
        ("out_buffer", C.c_void_p), ("out_offset", index_t), ("out_stride0", index_t),
        ("M", index_t), ("N", index_t), ("K", index_t),
        ("flags", C.c_uint32),
    ]


class PeerHandle(C.Structure):
    """iree_uk_b200_peer_handle_t: CUDA IPC handle of an allocation + offset of the buffer."""
    _fields_ = [("ipc", C.c_ubyte * 64), ("offset", C.c_uint64)]


class PackParams(C.Structure):
    """iree_uk_pack_params_t (136 bytes)."""
    _fields_ = [
        ("in_buffer", C.c_void_p), ("in_offset", index_t), ("in_stride0", index_t),
        ("in_stride1", index_t),
        ("out_buffer", C.c_void_p), ("out_offset", index_t), ("out_stride0", index_t),
        ("out_stride1", index_t),
        ("in_size0", index_t), ("in_size1", index_t),
        ("out_size0", index_t), ("out_size1", index_t), ("out_size2", index_t),
        ("out_size3", index_t),
        ("padding_value", C.c_uint64), ("flags", C.c_uint32), ("cpu_data", C.c_void_p),
    ]


class UnpackParams(C.Structure):
    """iree_uk_unpack_params_t (128 bytes)."""
    _fields_ = [
        ("in_buffer", C.c_void_p), ("in_offset", index_t), ("in_stride0", index_t),
        ("in_stride1", index_t),
        ("out_buffer", C.c_void_p), ("out_offset", index_t), ("out_stride0", index_t),
        ("out_stride1", index_t),
        ("in_size0", index_t), ("in_size1", index_t), ("in_size2", index_t),
        ("in_size3", index_t),
        ("out_size0", index_t), ("out_size1", index_t),
        ("flags", C.c_uint32), ("cpu_data", C.c_void_p),
    ]


class QueryTileSizes2dParams(C.Structure):
    """iree_uk_query_tile_sizes_2d_params_t."""
    _fields_ = [("flags", C.c_uint32), ("size0", index_t), ("size1", index_t),
                ("cpu_data", C.c_void_p)]


class QueryTileSizes2dOut(C.Structure):
    """iree_uk_query_tile_sizes_2d_out_params_t."""
    _fields_ = [("tile_size0", index_t), ("tile_size1", index_t)]


assert C.sizeof(Mmt4dParams) == 120 and C.sizeof(PackParams) == 136
assert C.sizeof(UnpackParams) == 128


def copy_params(p):
    """A field-by-field copy of a params struct."""
    q = type(p)()
    C.memmove(C.byref(q), C.byref(p), C.sizeof(p))
    return q
