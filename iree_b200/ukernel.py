"""Host-side mirror of the reference's ukernel interface, over the C ABI.

The three operations keep the reference's names and argument meaning
(``iree_uk_mmt4d`` / ``iree_uk_pack`` / ``iree_uk_unpack``,
runtime/src/iree/builtins/ukernel/mmt4d.h:14-22, pack.h:26-34, unpack.h:17-25); buffers are
CUDA device pointers and each call is enqueued on a CUDA stream. A non-zero status from the
library raises ``UkernelError`` (the reference asserts instead).

torch is used only for device memory and streams.
"""
import ctypes as C

from . import abi
from ._lib import lib


class UkernelError(RuntimeError):
    def __init__(self, status, what):
        self.status = status
        super().__init__("%s: %s" % (what, lib.iree_uk_b200_status_string(status).decode()))


def _stream_handle(stream):
    if stream is None:
        import torch
        return torch.cuda.current_stream().cuda_stream
    return getattr(stream, "cuda_stream", stream)


def _check(status, what):
    if status != abi.OK:
        raise UkernelError(status, what)


def mmt4d_workspace_size(params):
    """Scratch bytes ``mmt4d(..., workspace=...)`` can use for ``params`` (0: none)."""
    return int(lib.iree_uk_b200_mmt4d_workspace_size(C.addressof(params)))


def mmt4d(params, stream=None, workspace=None):
    """``iree_uk_mmt4d_p`` on device buffers. ``workspace``: a torch uint8 CUDA tensor of at
    least ``mmt4d_workspace_size(params)`` bytes, or None (then no scratch is used)."""
    s = _stream_handle(stream)
    if workspace is None:
        _check(lib.iree_uk_b200_mmt4d(C.addressof(params), s), "mmt4d")
    else:
        _check(lib.iree_uk_b200_mmt4d_ws(C.addressof(params), workspace.data_ptr(),
                                         workspace.numel() * workspace.element_size(), s), "mmt4d")


def mmt4d_host_arena_size(params):
    """Device bytes ``mmt4d_host`` needs for ``params`` (host pointers)."""
    return int(lib.iree_uk_b200_mmt4d_host_arena_size(C.addressof(params)))


def mmt4d_host(params, arena, stream=None):
    """``iree_uk_mmt4d_p`` with HOST buffers in ``params`` (the reference's own convention):
    copies in, computes on the device, copies the result back, pipelined over chunks of RHS tile
    rows. ``arena``: a torch uint8 CUDA tensor of at least ``mmt4d_host_arena_size(params)``
    bytes. Asynchronous: synchronise the stream before reading the output."""
    _check(lib.iree_uk_b200_mmt4d_host(C.addressof(params), arena.data_ptr(),
                                       arena.numel() * arena.element_size(),
                                       _stream_handle(stream)), "mmt4d_host")


def mmt4d_host_resident_lhs(params, device_lhs, device_lhs_stride0, arena, stream=None):
    """``mmt4d_host`` with the LHS already on the device (``device_lhs``: a CUDA tensor of tile
    rows ``device_lhs_stride0`` elements apart); RHS and output are host buffers in ``params``."""
    _check(lib.iree_uk_b200_mmt4d_host_resident_lhs(
        C.addressof(params), device_lhs.data_ptr(), device_lhs_stride0, arena.data_ptr(),
        arena.numel() * arena.element_size(), _stream_handle(stream)), "mmt4d_host_resident_lhs")


def mmt4d_peers(params, peer_out_ptrs, workspace, stream=None):
    """mmt4d whose output tiles are also stored, by the same kernel, to the buffers at
    ``peer_out_ptrs`` (device addresses valid on this GPU, usually other GPUs' memory opened
    with ``peer_open``); each stands for ``params.out_buffer`` in one more copy of the output.
    Tensor-core problems only (raises UNSUPPORTED otherwise)."""
    n = len(peer_out_ptrs)
    arr = (C.c_void_p * max(n, 1))(*peer_out_ptrs)
    _check(lib.iree_uk_b200_mmt4d_ws_peers(C.addressof(params), arr, n, workspace.data_ptr(),
                                           workspace.numel() * workspace.element_size(),
                                           _stream_handle(stream)), "mmt4d_peers")


F32_MODE_CUDA_CORES, F32_MODE_TF32X3 = 0, 1


def set_f32_mode(mode):
    """Process-wide: how f32f32f32 with 16x16 tiles is computed when scratch is supplied —
    ``F32_MODE_CUDA_CORES`` (default, the reference's accumulation order) or ``F32_MODE_TF32X3``
    (tensor cores, three tf32 products per term). Returns the previous mode."""
    return int(lib.iree_uk_b200_set_f32_mode(mode))


def mmt4d_sharded(device_ids, per_gpu_params, workspaces, streams, replicate_output=False):
    """The N-sharded mmt4d from one process that owns several GPUs: enqueues
    ``per_gpu_params[g]`` on ``device_ids[g]`` / ``streams[g]`` with ``workspaces[g]`` (torch
    uint8 tensors on that device). With ``replicate_output`` every GPU's full-size output
    buffer receives all tile columns through peer stores."""
    n = len(device_ids)
    ids = (C.c_int * n)(*device_ids)
    params = (abi.Mmt4dParams * n)(*per_gpu_params)
    ws = (C.c_void_p * n)(*[w.data_ptr() for w in workspaces])
    nb = (C.c_size_t * n)(*[w.numel() * w.element_size() for w in workspaces])
    st = (C.c_void_p * n)(*[getattr(s, "cuda_stream", s) for s in streams])
    _check(lib.iree_uk_b200_mmt4d_sharded(n, ids, params, ws, nb, st,
                                          1 if replicate_output else 0), "mmt4d_sharded")


def mmt4d_unpacked(params, out_size0, out_size1, workspace, stream=None):
    """mmt4d whose epilogue writes the row-major ``out_size0 x out_size1`` matrix that
    ``unpack`` would produce from the output tiles; ``params.out_*`` describe that matrix."""
    _check(lib.iree_uk_b200_mmt4d_ws_unpacked(C.addressof(params), out_size0, out_size1,
                                              workspace.data_ptr(),
                                              workspace.numel() * workspace.element_size(),
                                              _stream_handle(stream)), "mmt4d_unpacked")


def mmt4d_prepared_rhs_size(params):
    """Bytes of the re-tiled RHS a caller may keep across calls (0: not applicable)."""
    return int(lib.iree_uk_b200_mmt4d_prepared_rhs_size(C.addressof(params)))


def mmt4d_prepared_workspace_size(params):
    """Scratch bytes ``mmt4d_prepared`` needs (the LHS part only)."""
    return int(lib.iree_uk_b200_mmt4d_prepared_workspace_size(C.addressof(params)))


def mmt4d_prepare_rhs(params, prepared, stream=None):
    """Re-tiles ``params.rhs_buffer`` once into ``prepared`` (a torch uint8 CUDA tensor of at
    least ``mmt4d_prepared_rhs_size(params)`` bytes) for later ``mmt4d_prepared`` calls."""
    _check(lib.iree_uk_b200_mmt4d_prepare_rhs(C.addressof(params), prepared.data_ptr(),
                                              prepared.numel() * prepared.element_size(),
                                              _stream_handle(stream)), "mmt4d_prepare_rhs")


def mmt4d_prepared(params, prepared, workspace, stream=None):
    """mmt4d with the RHS already re-tiled (weights prepared once): only the LHS is re-tiled
    per call. Same results as ``mmt4d(..., workspace=...)``."""
    _check(lib.iree_uk_b200_mmt4d_ws_prepared(C.addressof(params), prepared.data_ptr(),
                                              workspace.data_ptr(),
                                              workspace.numel() * workspace.element_size(),
                                              _stream_handle(stream)), "mmt4d_prepared")


def mmt4d_multicast(params, multicast_out_ptr, workspace, stream=None):
    """mmt4d whose output tiles are stored once through an NVLink multicast mapping and
    replicated by the switch into every GPU's buffer; ``multicast_out_ptr`` is the address in
    that mapping that stands for ``params.out_buffer``."""
    _check(lib.iree_uk_b200_mmt4d_ws_multicast(C.addressof(params), multicast_out_ptr,
                                               workspace.data_ptr(),
                                               workspace.numel() * workspace.element_size(),
                                               _stream_handle(stream)), "mmt4d_multicast")


def peer_export(device_ptr):
    """Bytes another process on this machine can pass to ``peer_open`` to address the device
    buffer at ``device_ptr`` (an int, or a tensor)."""
    ptr = device_ptr.data_ptr() if hasattr(device_ptr, "data_ptr") else int(device_ptr)
    h = abi.PeerHandle()
    _check(lib.iree_uk_b200_peer_export(ptr, C.addressof(h)), "peer_export")
    return bytes(h)


def peer_open(handle_bytes):
    """Device address, valid in this process on the current device, of a buffer another
    process exported with ``peer_export``."""
    h = abi.PeerHandle.from_buffer_copy(handle_bytes)
    out = C.c_void_p()
    _check(lib.iree_uk_b200_peer_open(C.addressof(h), C.addressof(out)), "peer_open")
    return int(out.value)


def peer_close(ptr):
    _check(lib.iree_uk_b200_peer_close(ptr), "peer_close")


def matmul_workspace_size(params):
    """Scratch bytes ``matmul`` needs for ``params`` (an ``abi.MatmulParams``)."""
    return int(lib.iree_uk_b200_matmul_workspace_size(C.addressof(params)))


def matmul(params, workspace, stream=None):
    """Row-major matmul with the results of the reference's pack -> mmt4d -> unpack chain
    (``ukernel/tools/e2e_matmul_benchmark.c:173-300``), on the tensor-core kernels and without
    packed copies of the LHS or the result. ``workspace``: a torch uint8 CUDA tensor of at least
    ``matmul_workspace_size(params)`` bytes."""
    _check(lib.iree_uk_b200_matmul(C.addressof(params), workspace.data_ptr(),
                                   workspace.numel() * workspace.element_size(),
                                   _stream_handle(stream)), "matmul")


STATIC_SCRATCH_BYTES = 32 << 20


def mmt4d_static_scratch(params, stream=None):
    """mmt4d for callers that cannot allocate or pass device scratch: same results as
    ``mmt4d(..., workspace=...)``, with the re-tiled operands kept in a 32 MiB array that
    lives inside the library on each GPU. Raises WORKSPACE_TOO_SMALL when the problem needs
    more than that. Calls that may overlap on the GPU share (and would race on) that array;
    make the first call on a device before beginning any stream capture there."""
    _check(lib.iree_uk_b200_mmt4d_static_scratch(C.addressof(params), _stream_handle(stream)),
           "mmt4d_static_scratch")


def mmt4d_pooled(params, stream=None):
    """mmt4d with scratch from the library's stream-ordered memory pool (taken and returned on
    ``stream``): the kernels of ``mmt4d(..., workspace=...)`` behind the reference's plain
    signature, for callers that may allocate."""
    _check(lib.iree_uk_b200_mmt4d_pooled(C.addressof(params), _stream_handle(stream)),
           "mmt4d_pooled")


def scratch_pool_trim(keep_bytes=0):
    """Hands the unused memory of the current device's scratch pool back, down to ``keep_bytes``."""
    _check(lib.iree_uk_b200_scratch_pool_trim(keep_bytes), "scratch_pool_trim")


def mmt4d_path(params, with_workspace=True):
    """Which kernel serves the call (``abi.PATH_*``); raises on rejected parameters."""
    r = lib.iree_uk_b200_mmt4d_path(C.addressof(params), 1 if with_workspace else 0)
    if r < 0:
        raise UkernelError(-r, "mmt4d_path")
    return r


def mmt4d_info(M0, N0, K0, flags):
    """``iree_uk_mmt4d_info``: bit 0 set when a tensor-core kernel exists for the tile."""
    return int(lib.iree_uk_b200_mmt4d_info(M0, N0, K0, flags))


def pack(params, stream=None):
    """``iree_uk_pack_p`` on device buffers."""
    _check(lib.iree_uk_b200_pack(C.addressof(params), _stream_handle(stream)), "pack")


def pack_path(params):
    r = lib.iree_uk_b200_pack_path(C.addressof(params))
    if r < 0:
        raise UkernelError(-r, "pack_path")
    return r


def unpack(params, stream=None):
    """``iree_uk_unpack_p`` on device buffers."""
    _check(lib.iree_uk_b200_unpack(C.addressof(params), _stream_handle(stream)), "unpack")


def unpack_path(params):
    r = lib.iree_uk_b200_unpack_path(C.addressof(params))
    if r < 0:
        raise UkernelError(-r, "unpack_path")
    return r


QUERY_REFERENCE_X86_64 = 0x10000


def query_tile_sizes_2d(flags, size0=0, size1=0, cpu_data0=None):
    """``iree_uk_query_tile_sizes_2d``: (tile_size0, tile_size1). With ``QUERY_REFERENCE_X86_64``
    in ``flags`` and ``cpu_data0`` (the first cpu_data word) the reference's x86-64 answer."""
    words = (C.c_uint64 * 8)(cpu_data0 or 0) if cpu_data0 is not None else None
    p = abi.QueryTileSizes2dParams(flags=flags, size0=size0, size1=size1,
                                   cpu_data=C.cast(words, C.c_void_p) if words is not None else None)
    o = abi.QueryTileSizes2dOut()
    _check(lib.iree_uk_b200_query_tile_sizes_2d(C.addressof(p), C.addressof(o)),
           "query_tile_sizes_2d")
    return int(o.tile_size0), int(o.tile_size1)


def device_status(stream=None):
    """Synchronises the stream and returns (status, detail word) of the bounded device waits."""
    detail = C.c_uint32(0)
    st = lib.iree_uk_b200_device_status(_stream_handle(stream), C.addressof(detail))
    return st, int(detail.value)


def kernel_timing(every):
    """Every ``every``-th later tensor-core mmt4d call on the current device records CUDA events
    around its pre-pass and its main kernel (0 switches the recording off)."""
    _check(lib.iree_uk_b200_kernel_timing(int(every)), "kernel_timing")


def kernel_timing_mean_ms():
    """(mean pre-pass ms, mean main-kernel ms, calls) over the remembered recorded calls."""
    a, b, n = C.c_float(0), C.c_float(0), C.c_int(0)
    _check(lib.iree_uk_b200_kernel_timing_mean_ms(C.addressof(a), C.addressof(b), C.addressof(n)),
           "kernel_timing_mean_ms")
    return float(a.value), float(b.value), int(n.value)


FORM_TWO_CTA, FORM_ONE_CTA, FORM_TWO_CTA_STREAMED = 5, 6, 7


def testing_starve_producers(enable):
    """Test hook: the producers of the tensor-core kernels fill nothing while enabled, so the
    bounded device-side waits run out. Returns the previous setting."""
    return int(lib.iree_uk_b200_testing_starve_producers(1 if enable else 0))


def testing_mmt4d_form(params, workspace, form, stream=None):
    """Test hook: a tensor-core mmt4d on one given kernel form (``FORM_*``)."""
    _check(lib.iree_uk_b200_testing_mmt4d_form(C.addressof(params), workspace.data_ptr(),
                                               workspace.numel() * workspace.element_size(), form,
                                               _stream_handle(stream)), "testing_mmt4d_form")


def shard_params(full, rank, world, rhs_is_local=False, out_is_local=True):
    """Parameters of ``rank`` when the RHS tile rows (N) are split across ``world`` GPUs.
    Returns (params, first owned tile row)."""
    shard = abi.Mmt4dParams()
    begin = abi.index_t(0)
    _check(lib.iree_uk_b200_mmt4d_shard_params(C.addressof(full), rank, world,
                                               1 if rhs_is_local else 0,
                                               1 if out_is_local else 0, C.addressof(shard),
                                               C.addressof(begin)), "mmt4d_shard_params")
    return shard, int(begin.value)


def interleave_slabs(gathered, out, M, N, tile_elems, elem_size, world, stream=None):
    """[world][M][N/world][tile] -> [M][N][tile] on device (after an all-gather of slabs)."""
    _check(lib.iree_uk_b200_interleave_slabs(gathered.data_ptr(), out.data_ptr(), M, N,
                                             tile_elems, elem_size, world,
                                             _stream_handle(stream)), "interleave_slabs")
