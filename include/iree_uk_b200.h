/*
 * iree_uk_b200.h — C ABI of the B200 (sm_100a) data-tiled contraction library.
 *
 * The library is a drop-in for the three IREE microkernels
 *   iree_uk_mmt4d   (runtime/src/iree/builtins/ukernel/mmt4d.h:14-22)
 *   iree_uk_pack    (runtime/src/iree/builtins/ukernel/pack.h:26-34)
 *   iree_uk_unpack  (runtime/src/iree/builtins/ukernel/unpack.h:17-25)
 * with the same parameter structs, the same flag values and the same 4-D tiled
 * layouts, except that every buffer is a CUDA device pointer and every call takes the
 * CUDA stream the work is enqueued on (for IREE that is the dispatch stream owned by
 * the CUDA HAL device, runtime/src/iree/hal/drivers/cuda/cuda_device.c:542-547).
 *
 * Contract shared by all entry points
 *   - asynchronous: kernels are enqueued on `cu_stream` in call order; the stream is
 *     never synchronised and no other stream is touched;
 *   - no implicit device allocation: scratch memory, when a fast path wants it, is
 *     passed in by the caller (see iree_uk_b200_mmt4d_ws);
 *   - arguments are validated on the host with the reference's rules
 *     (mmt4d.c:12-48, pack.c:51-104, unpack.c:31-82) and a violation returns
 *     IREE_UK_B200_INVALID_ARGUMENT instead of asserting; nothing is launched then;
 *   - bytes of the output allocation that the reference does not write are never
 *     written (pinned by the whole-buffer memcmp of tools/mmt4d_test.c:430-440);
 *   - offsets and strides are in elements, exactly as in the reference; for the u4
 *     right-hand side they must be even (whole bytes, mmt4d.c:39-46);
 *   - `cpu_data` is ignored and may be NULL;
 *   - thread-safe; one CUDA device per call (the one `cu_stream` belongs to must be
 *     current on the calling thread).
 *
 * This header is plain C99 and also valid C++.
 */
#ifndef IREE_UK_B200_H_
#define IREE_UK_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define IREE_UK_B200_EXPORT __declspec(dllexport)
#else
#define IREE_UK_B200_EXPORT __attribute__((visibility("default")))
#endif

/* iree_uk_index_t is int64 on 64-bit hosts (ukernel/common.h:269-275). */
typedef int64_t iree_uk_index_t;

/*===----------------------------------------------------------------------===*/
/* Flags — values frozen by ukernel/exported_bits.h:29-83                      */
/*===----------------------------------------------------------------------===*/

#define IREE_UK_FLAG_MMT4D_TYPE_MASK 0xFF
#define IREE_UK_FLAG_MMT4D_TYPE_NONE 0x00
#define IREE_UK_FLAG_MMT4D_TYPE_F32F32F32 0x01
#define IREE_UK_FLAG_MMT4D_TYPE_S8S8S32 0x02
#define IREE_UK_FLAG_MMT4D_TYPE_F16F16F32 0x03
#define IREE_UK_FLAG_MMT4D_TYPE_F16F16F16 0x04
#define IREE_UK_FLAG_MMT4D_TYPE_BF16BF16F32 0x05
#define IREE_UK_FLAG_MMT4D_TYPE_BF16BF16BF16 0x06
#define IREE_UK_FLAG_MMT4D_TYPE_S16S16S32 0x07
#define IREE_UK_FLAG_MMT4D_TYPE_S16U4S32 0x08
#define IREE_UK_FLAG_MMT4D_TYPE_S16S8S32 0x09
#define IREE_UK_FLAG_MMT4D_TYPE_S8S4S32 0x0A
#define IREE_UK_FLAG_MMT4D_TYPE_END 0x0B
#define IREE_UK_FLAG_MMT4D_ACCUMULATE 0x100
#define IREE_UK_FLAG_MMT4D_ALLOW_GENERIC_FALLBACK_TILE_FUNCTION 0x200
#define IREE_UK_FLAG_MMT4D_SKIP_INTERMEDIATE_ROUNDINGS 0x400
#define IREE_UK_FLAG_MMT4D_INFO_HAVE_ARCHITECTURE_SPECIFIC_TILE_FUNCTION 0x1

#define IREE_UK_FLAG_PACK_TYPE_MASK 0xFF
#define IREE_UK_FLAG_PACK_TYPE_NONE 0x00
#define IREE_UK_FLAG_PACK_TYPE_F32F32 0x01
#define IREE_UK_FLAG_PACK_TYPE_I8I8 0x02
#define IREE_UK_FLAG_PACK_TYPE_I32I32 0x03
#define IREE_UK_FLAG_PACK_TYPE_F16F16 0x04
#define IREE_UK_FLAG_PACK_TYPE_BF16BF16 0x05
#define IREE_UK_FLAG_PACK_TRANSPOSE_INNER 0x100
#define IREE_UK_FLAG_PACK_TRANSPOSE_OUTER 0x200

#define IREE_UK_FLAG_UNPACK_TYPE_MASK 0xFF
#define IREE_UK_FLAG_UNPACK_TYPE_NONE 0x00
#define IREE_UK_FLAG_UNPACK_TYPE_F32F32 0x01
#define IREE_UK_FLAG_UNPACK_TYPE_I32I32 0x03
#define IREE_UK_FLAG_UNPACK_TYPE_F16F16 0x04
#define IREE_UK_FLAG_UNPACK_TYPE_BF16BF16 0x05
#define IREE_UK_FLAG_UNPACK_TRANSPOSE_INNER 0x100
#define IREE_UK_FLAG_UNPACK_TRANSPOSE_OUTER 0x200

#define IREE_UK_FLAG_QUERY_TILE_SIZES_OPERAND_ROLE_MASK 0xFF
#define IREE_UK_FLAG_QUERY_TILE_SIZES_OPERAND_ROLE_LHS 0x01
#define IREE_UK_FLAG_QUERY_TILE_SIZES_OPERAND_ROLE_RHS 0x02
#define IREE_UK_FLAG_QUERY_TILE_SIZES_OPERAND_ROLE_RESULT 0x03
#define IREE_UK_FLAG_QUERY_TILE_SIZES_OPERATION_MASK 0xFF00
#define IREE_UK_FLAG_QUERY_TILE_SIZES_OPERATION_MATMUL_F32F32F32 0x0100
#define IREE_UK_FLAG_QUERY_TILE_SIZES_OPERATION_MATMUL_I8I8I32 0x0200
#define IREE_UK_FLAG_QUERY_TILE_SIZES_OPERATION_MATMUL_F16F16F32 0x0300
#define IREE_UK_FLAG_QUERY_TILE_SIZES_OPERATION_MATMUL_F16F16F16 0x0400
#define IREE_UK_FLAG_QUERY_TILE_SIZES_OPERATION_MATMUL_BF16BF16F32 0x0500
#define IREE_UK_FLAG_QUERY_TILE_SIZES_OPERATION_MATMUL_BF16BF16BF16 0x0600
/* Not a reference flag (the reference uses bits 0-15 only): answer what the reference's own
 * x86-64 build answers for params->cpu_data instead of this library's tile choice. */
#define IREE_UK_B200_FLAG_QUERY_TILE_SIZES_REFERENCE_X86_64 0x10000

/*===----------------------------------------------------------------------===*/
/* Parameter structs — field-for-field the reference's                         */
/*===----------------------------------------------------------------------===*/

/* ukernel/mmt4d_internal.h:14-32. 120 bytes on LP64.
 * out[i][j][i0][j0] (+)= sum_{k,k0} lhs[i][k][i0][k0] * rhs[j][k][j0][k0]
 * lhs element index: lhs_offset + i*lhs_stride0 + k*M0*K0 + i0*K0 + k0
 * rhs element index: rhs_offset + j*rhs_stride0 + k*N0*K0 + j0*K0 + k0
 * out element index: out_offset + i*out_stride0 + j*M0*N0 + i0*N0 + j0 */
typedef struct iree_uk_mmt4d_params_t {
  const void* lhs_buffer; /* device pointer */
  iree_uk_index_t lhs_offset;
  iree_uk_index_t lhs_stride0;
  const void* rhs_buffer; /* device pointer */
  iree_uk_index_t rhs_offset;
  iree_uk_index_t rhs_stride0;
  void* out_buffer; /* device pointer */
  iree_uk_index_t out_offset;
  iree_uk_index_t out_stride0;
  iree_uk_index_t M; /* number of LHS tile rows   (M1) */
  iree_uk_index_t N; /* number of RHS tile rows   (N1) */
  iree_uk_index_t K; /* number of tiles along K   (K1) */
  int32_t M0;
  int32_t N0;
  int32_t K0;
  uint32_t flags;
  const uint64_t* cpu_data; /* ignored */
} iree_uk_mmt4d_params_t;

/* ukernel/pack_internal.h:12-30. 136 bytes on LP64. */
typedef struct iree_uk_pack_params_t {
  const void* in_buffer; /* device pointer */
  iree_uk_index_t in_offset;
  iree_uk_index_t in_stride0;
  iree_uk_index_t in_stride1;
  void* out_buffer; /* device pointer */
  iree_uk_index_t out_offset;
  iree_uk_index_t out_stride0;
  iree_uk_index_t out_stride1; /* must equal out_size2*out_size3 (pack.c:72) */
  iree_uk_index_t in_size0;
  iree_uk_index_t in_size1;
  iree_uk_index_t out_size0;
  iree_uk_index_t out_size1;
  iree_uk_index_t out_size2;
  iree_uk_index_t out_size3;
  uint64_t padding_value; /* low elem-size bytes are the fill pattern (pack.h:16-25) */
  uint32_t flags;
  const uint64_t* cpu_data; /* ignored */
} iree_uk_pack_params_t;

/* ukernel/unpack_internal.h:12-29. 128 bytes on LP64. */
typedef struct iree_uk_unpack_params_t {
  const void* in_buffer; /* device pointer */
  iree_uk_index_t in_offset;
  iree_uk_index_t in_stride0;
  iree_uk_index_t in_stride1; /* must equal in_size2*in_size3 (unpack.c:49) */
  void* out_buffer;           /* device pointer */
  iree_uk_index_t out_offset;
  iree_uk_index_t out_stride0;
  iree_uk_index_t out_stride1;
  iree_uk_index_t in_size0;
  iree_uk_index_t in_size1;
  iree_uk_index_t in_size2;
  iree_uk_index_t in_size3;
  iree_uk_index_t out_size0;
  iree_uk_index_t out_size1;
  uint32_t flags;
  const uint64_t* cpu_data; /* ignored */
} iree_uk_unpack_params_t;

/* ukernel/query_tile_sizes.h:17-24. */
typedef struct iree_uk_query_tile_sizes_2d_params_t {
  uint32_t flags;
  iree_uk_index_t size0;
  iree_uk_index_t size1;
  const uint64_t* cpu_data; /* ignored */
} iree_uk_query_tile_sizes_2d_params_t;

/* ukernel/query_tile_sizes.h:26-29. */
typedef struct iree_uk_query_tile_sizes_2d_out_params_t {
  iree_uk_index_t tile_size0;
  iree_uk_index_t tile_size1;
} iree_uk_query_tile_sizes_2d_out_params_t;

/*===----------------------------------------------------------------------===*/
/* Status codes (the reference returns void and asserts; this ABI reports)     */
/*===----------------------------------------------------------------------===*/

typedef enum iree_uk_b200_status_t {
  IREE_UK_B200_OK = 0,
  IREE_UK_B200_INVALID_ARGUMENT = 1, /* a reference *_validate rule is violated   */
  IREE_UK_B200_UNSUPPORTED = 2,      /* valid for the reference, not served here  */
  IREE_UK_B200_CUDA_ERROR = 3,       /* a CUDA runtime/driver call failed         */
  IREE_UK_B200_WORKSPACE_TOO_SMALL = 4,
  IREE_UK_B200_DEVICE_TIMEOUT = 5 /* a bounded device-side wait gave up          */
} iree_uk_b200_status_t;

IREE_UK_B200_EXPORT const char* iree_uk_b200_status_string(int status);

/*===----------------------------------------------------------------------===*/
/* Which kernel serves a call (reported, never a CPU path)                     */
/*===----------------------------------------------------------------------===*/

typedef enum iree_uk_b200_path_t {
  IREE_UK_B200_PATH_NONE = 0,         /* early-out: nothing is launched            */
  IREE_UK_B200_PATH_GENERIC = 1,      /* CUDA-core kernel, any tile shape / stride */
  IREE_UK_B200_PATH_TCGEN05 = 2,      /* tcgen05 + TMEM, operands read as they lie */
  IREE_UK_B200_PATH_TCGEN05_RETILE = 3, /* re-tile pre-pass into workspace, then 2 */
  IREE_UK_B200_PATH_GEMV = 4,         /* s16u4s32 M0=1 weight-streaming kernel     */
  IREE_UK_B200_PATH_FAST_COPY = 5,    /* pack/unpack 16-byte vectorised relayout   */
  IREE_UK_B200_PATH_ZERO_FILL = 6     /* K==0 without ACCUMULATE: zero the tiles   */
} iree_uk_b200_path_t;

/*===----------------------------------------------------------------------===*/
/* mmt4d                                                                       */
/*===----------------------------------------------------------------------===*/

/* Replaces iree_uk_mmt4d_p (ukernel/mmt4d.c:115-141). Uses no scratch memory. The
 * tensor-core triples with 16x16 tiles still run on the tensor cores: 16-bit K0 = 1
 * operands are staged by TMA as they lie, every other layout by a kernel whose producer warps
 * re-tile the operands on their way into shared memory (measured 0.38 of the rate that
 * iree_uk_b200_mmt4d_ws reaches with its pre-pass into caller-owned scratch). Everything
 * else runs the generic CUDA-core kernel. */
IREE_UK_B200_EXPORT int iree_uk_b200_mmt4d(const iree_uk_mmt4d_params_t* params,
                                           void* cu_stream);

/* Bytes of scratch iree_uk_b200_mmt4d_ws can use for `params` (0 when the call is served
 * without scratch). The size depends on M,N,K,M0,N0,K0 and the type only. */
IREE_UK_B200_EXPORT size_t
iree_uk_b200_mmt4d_workspace_size(const iree_uk_mmt4d_params_t* params);

/* Same operation as iree_uk_b200_mmt4d with caller-owned scratch (256-byte aligned
 * device memory, at least iree_uk_b200_mmt4d_workspace_size bytes, free to reuse once
 * the enqueued work has completed). Replaces iree_uk_mmt4d_p (ukernel/mmt4d.c:115-141).
 * workspace == NULL (or workspace_bytes == 0) is the scratch-free call above. A workspace that
 * is offered but smaller than the kernel that would use it needs is refused with
 * IREE_UK_B200_WORKSPACE_TOO_SMALL and nothing is launched; the call never falls back to a
 * slower kernel on its own. */
IREE_UK_B200_EXPORT int iree_uk_b200_mmt4d_ws(const iree_uk_mmt4d_params_t* params,
                                              void* workspace, size_t workspace_bytes,
                                              void* cu_stream);

/* mmt4d followed by the unpack of its result, as one call: the tiles never exist in memory, the
 * epilogue writes the row-major matrix that iree_uk_unpack (ukernel/unpack.c:259-285, type
 * I32I32 / F32F32, no transposes) would produce from them. params->out_buffer, out_offset and
 * out_stride0 describe that matrix ([out_size0][out_size1], out_stride0 = its row pitch in
 * elements, out_size0 <= M * M0, out_size1 <= N * N0; elements outside it are never written,
 * exactly as unpack does). With ACCUMULATE the matrix holds the accumulator on entry (what
 * packing it into tiles first would feed mmt4d). Tensor-core triples with a 32-bit output and
 * 16x16 tiles only; scratch as for iree_uk_b200_mmt4d_ws. */
IREE_UK_B200_EXPORT int iree_uk_b200_mmt4d_ws_unpacked(const iree_uk_mmt4d_params_t* params,
                                                       iree_uk_index_t out_size0,
                                                       iree_uk_index_t out_size1, void* workspace,
                                                       size_t workspace_bytes, void* cu_stream);

/* Weights prepared once. The tensor-core path re-tiles both operands before every call; when
 * the RHS is a weight matrix that does not change between calls, its re-tiled form can be
 * produced once and kept by the caller (the analogue of IREE packing constant weights ahead of
 * time, compiler/.../ConstEval):
 *   iree_uk_b200_mmt4d_prepared_rhs_size(params)   bytes of the prepared form (0: not applicable;
 *       depends on N, K, K0 and the type only — M may differ from call to call),
 *   iree_uk_b200_mmt4d_prepare_rhs(params, buf, bytes, stream)   fills it from params->rhs_buffer,
 *   iree_uk_b200_mmt4d_ws_prepared(params, buf, ws, ws_bytes, stream)   the mmt4d itself; only the
 *       LHS is re-tiled, into `ws` of iree_uk_b200_mmt4d_prepared_workspace_size(params) bytes.
 * `buf` and `ws` are 256-byte aligned device memory. Results are identical to
 * iree_uk_b200_mmt4d_ws. The prepared form is valid while the RHS contents, N, K, K0 and the type
 * stay the same; params->rhs_buffer is not read by iree_uk_b200_mmt4d_ws_prepared. For the
 * s8s8s32 / f16 / bf16 triples with 16x16 tiles, and for s16u4s32 1x32x8, whose prepared form is
 * the weights widened to bytes: the prepared call then runs the tensor-core kernel for any
 * number of rows (not the f32 mode, not s16s16 / s16s8 / s8s4). */
IREE_UK_B200_EXPORT size_t
iree_uk_b200_mmt4d_prepared_rhs_size(const iree_uk_mmt4d_params_t* params);
IREE_UK_B200_EXPORT size_t
iree_uk_b200_mmt4d_prepared_workspace_size(const iree_uk_mmt4d_params_t* params);
IREE_UK_B200_EXPORT int iree_uk_b200_mmt4d_prepare_rhs(const iree_uk_mmt4d_params_t* params,
                                                       void* prepared_rhs, size_t prepared_bytes,
                                                       void* cu_stream);
IREE_UK_B200_EXPORT int iree_uk_b200_mmt4d_ws_prepared(const iree_uk_mmt4d_params_t* params,
                                                       const void* prepared_rhs, void* workspace,
                                                       size_t workspace_bytes, void* cu_stream);

/* How f32f32f32 with 16x16xK0 tiles is computed when scratch is supplied. The reference adds
 * f32 products in k order; the default here does the same on the CUDA cores. TF32X3 moves the
 * work to the tensor cores: each operand is split into a tf32 part and a remainder and every
 * product becomes three tf32 products accumulated in f32 (measured 266 TFLOP/s at 8192^3, f32
 * operations counted once). The result then differs
 * from the reference's by a relative Frobenius error of about 7e-9 x K (1e-6 at K = 129, 5e-6
 * at K = 700): tensor-core accumulation truncates. Process-wide, like a math mode; returns the
 * previous mode. */
#define IREE_UK_B200_F32_MODE_CUDA_CORES 0
#define IREE_UK_B200_F32_MODE_TF32X3 1
IREE_UK_B200_EXPORT int iree_uk_b200_set_f32_mode(int mode);

/* Most peer output buffers one call of iree_uk_b200_mmt4d_ws_peers can store to. */
#define IREE_UK_B200_MAX_PEERS 16

/* mmt4d fused with the replication of its output: every output tile is stored to
 * params->out_buffer and, from the same kernel, to `num_peers` further buffers that usually
 * live on other GPUs (NVLink peer memory), so that an N-sharded mmt4d (each GPU owning a range
 * of RHS tile rows, ukernel/mmt4d.c:84-98) leaves the whole [M][N][M0][N0] result on every GPU
 * without a separate all-gather. peer_out_buffers[i] stands for params->out_buffer in copy i:
 * out_offset and out_stride0 apply to it unchanged. The pointers must be valid on the current
 * device (see iree_uk_b200_peer_open) and have params->out_buffer's alignment modulo 32 bytes.
 * ACCUMULATE reads the old values from params->out_buffer only. The stores to a peer are
 * complete when this GPU's stream reaches the end of the call; the peer must not read them
 * before it has synchronised with this GPU (a barrier among the ranks, or an event).
 * Served only by the tensor-core kernels (s8s8s32, f16f16f32, bf16bf16f32 with 16x16 tiles and
 * scratch): any other problem returns IREE_UK_B200_UNSUPPORTED and launches nothing. No
 * counterpart in the reference, whose ukernels are single-device. */
IREE_UK_B200_EXPORT int iree_uk_b200_mmt4d_ws_peers(const iree_uk_mmt4d_params_t* params,
                                                    const void* const* peer_out_buffers,
                                                    int num_peers, void* workspace,
                                                    size_t workspace_bytes, void* cu_stream);

/* As iree_uk_b200_mmt4d_ws_peers, but through an NVLink multicast mapping (NVSwitch systems):
 * `multicast_out_buffer` is the address, in the multicast mapping bound to the same-shaped
 * output buffers of all GPUs of a group (this GPU's included), that stands for
 * params->out_buffer. Every output tile is stored once with multimem.st and replicated to all
 * bound buffers by the switch, so the result leaves this GPU once instead of once per peer.
 * The mapping is created by the caller (cuMulticastCreate / cuMulticastBindMem, or a library
 * that wraps them); params->out_buffer stays this GPU's ordinary address of its own buffer
 * (ACCUMULATE reads the old values through it). Same completion and synchronisation rules as
 * iree_uk_b200_mmt4d_ws_peers. */
IREE_UK_B200_EXPORT int iree_uk_b200_mmt4d_ws_multicast(const iree_uk_mmt4d_params_t* params,
                                                        const void* multicast_out_buffer,
                                                        void* workspace, size_t workspace_bytes,
                                                        void* cu_stream);

/* The N-sharded mmt4d driven from ONE process that owns several GPUs. For g in [0, n_gpus):
 * makes device_ids[g] current and enqueues per_gpu[g] (as produced by
 * iree_uk_b200_mmt4d_shard_params, with buffers on that device) on streams[g] with
 * workspaces[g] / workspace_bytes[g]; the caller's current device is restored afterwards.
 * replicate_output = 0: every GPU writes only its own buffer (no data-path collective).
 * replicate_output = 1: per_gpu[g].out_buffer must be a full [M][N][M0][N0] buffer on GPU g
 * addressed with out_is_local = 0; peer access between the devices is enabled as needed and
 * every GPU stores its tile columns into all n_gpus buffers (iree_uk_b200_mmt4d_ws_peers), so
 * that after all streams have completed each buffer holds the whole result. Returns the first
 * non-zero status; work enqueued before it stays enqueued. n_gpus <= IREE_UK_B200_MAX_PEERS + 1. */
IREE_UK_B200_EXPORT int iree_uk_b200_mmt4d_sharded(int n_gpus, const int* device_ids,
                                                   const iree_uk_mmt4d_params_t* per_gpu,
                                                   void* const* workspaces,
                                                   const size_t* workspace_bytes,
                                                   void* const* cu_streams, int replicate_output);

/* What one process hands to another (same machine) so that the other can address this
 * process's device buffer: a CUDA IPC handle of the allocation plus the buffer's offset in it. */
typedef struct iree_uk_b200_peer_handle_t {
  unsigned char ipc[64];
  uint64_t offset;
} iree_uk_b200_peer_handle_t;

/* Fills `handle` for `device_ptr` (memory of the current device obtained from cudaMalloc,
 * directly or through an allocator built on it). */
IREE_UK_B200_EXPORT int iree_uk_b200_peer_export(const void* device_ptr,
                                                 iree_uk_b200_peer_handle_t* handle);
/* Maps another process's buffer into this process for the current device (peer access is
 * enabled as needed). Each handle may be open once per process at a time. */
IREE_UK_B200_EXPORT int iree_uk_b200_peer_open(const iree_uk_b200_peer_handle_t* handle,
                                               void** device_ptr);
/* Unmaps a pointer returned by iree_uk_b200_peer_open, once no enqueued work uses it. */
IREE_UK_B200_EXPORT int iree_uk_b200_peer_close(void* device_ptr);

/* Capacity of the library-owned scratch used by iree_uk_b200_mmt4d_static_scratch. */
#define IREE_UK_B200_STATIC_SCRATCH_BYTES (32u << 20)

/* mmt4d for call sites that have no way to obtain device memory of their own. It has no
 * counterpart in the reference: there the ukernels need no scratch at all.
 *
 * Who needs it: a ukernel call that IREE emits sits inside an already-planned dispatch. The
 * compiler has laid out every buffer ahead of time, the ukernel contract forbids allocating
 * (ukernel/README.md:17-26), and at that point of the HAL command stream there is no
 * allocator to ask and no place to call cudaMalloc from. Such a caller can pass neither a
 * workspace nor allocate one, so with iree_uk_b200_mmt4d it would be stuck on the generic
 * kernel. This entry point gives it the tensor-core path anyway: the re-tiled operand
 * copies go into a fixed IREE_UK_B200_STATIC_SCRATCH_BYTES (32 MiB) array that is part of
 * the library image in each GPU's memory (every GPU that loads the library holds those
 * 32 MiB until the process exits). The call itself allocates nothing, on host or device.
 *
 * Same operation, arguments and results as iree_uk_b200_mmt4d_ws, and the same choice of
 * kernel: whatever iree_uk_b200_mmt4d_ws would run with scratch (the tensor-core triples with
 * 16x16 tiles, s16s16s32 / s16s8s32 16x16x2, s8s4s32 16x16x{2,4,8,16}, and s16u4s32 1x32x8 with at
 * least 16 rows) runs here on the array; problems
 * that use no scratch anyway (the weight-streaming s16u4s32 kernel below 16 rows, the generic
 * kernel, the zero fill) are served exactly as by iree_uk_b200_mmt4d. Differences:
 *  - a problem whose scratch need (iree_uk_b200_mmt4d_workspace_size) exceeds the array is
 *    refused with IREE_UK_B200_WORKSPACE_TOO_SMALL and nothing is launched; it is never
 *    silently served by a slower kernel;
 *  - the first call on each device looks up the array's device address
 *    (cudaGetSymbolAddress, with that device current). Make that first call during
 *    set-up, before any stream capture is begun on that device;
 *  - all calls on a device share the one array. Nothing in it has to start at zero (the
 *    pre-pass rewrites every byte the main kernel reads, so the previous call's leftovers
 *    are harmless), but two calls whose kernels can overlap on the GPU — different streams
 *    without an ordering between them — race on it. Keep calls on one stream, or order
 *    them with events. */
IREE_UK_B200_EXPORT int iree_uk_b200_mmt4d_static_scratch(
    const iree_uk_mmt4d_params_t* params, void* cu_stream);

/* mmt4d with scratch taken from a stream-ordered memory pool that the library owns (one per
 * device, created on first use; no reference counterpart). For a caller of the reference's
 * plain three-pointer signature that may allocate but has no buffer planned for scratch: the
 * call takes iree_uk_b200_mmt4d_workspace_size bytes from the pool with
 * cudaMallocFromPoolAsync on `cu_stream`, runs exactly what iree_uk_b200_mmt4d_ws would run
 * on them, and returns them with cudaFreeAsync on the same stream. The pool keeps what it has
 * been given (release threshold: unlimited), so after the first call of a given size no
 * device memory is obtained from the driver; iree_uk_b200_scratch_pool_trim hands memory back.
 * Problems that use no scratch are served exactly as by iree_uk_b200_mmt4d. Nothing in the
 * library calls this on its own: a caller that cannot allocate uses
 * iree_uk_b200_mmt4d_static_scratch or iree_uk_b200_mmt4d. */
IREE_UK_B200_EXPORT int iree_uk_b200_mmt4d_pooled(const iree_uk_mmt4d_params_t* params,
                                                  void* cu_stream);
/* Releases the current device's scratch pool down to `keep_bytes` of unused memory
 * (cudaMemPoolTrimTo); memory of calls still in flight is not touched. */
IREE_UK_B200_EXPORT int iree_uk_b200_scratch_pool_trim(size_t keep_bytes);

/* Flat-argument twin of iree_uk_mmt4d (ukernel/mmt4d.h:14-22, mmt4d.c:151-177) with the
 * workspace and the stream appended; `cpu_data` is kept in the list so a call site can be
 * substituted one for one. */
IREE_UK_B200_EXPORT int iree_uk_b200_mmt4d_flat(
    const void* lhs_buffer, iree_uk_index_t lhs_offset, iree_uk_index_t lhs_stride0,
    const void* rhs_buffer, iree_uk_index_t rhs_offset, iree_uk_index_t rhs_stride0,
    void* out_buffer, iree_uk_index_t out_offset, iree_uk_index_t out_stride0,
    iree_uk_index_t M, iree_uk_index_t N, iree_uk_index_t K, int32_t M0, int32_t N0,
    int32_t K0, uint32_t flags, const uint64_t* cpu_data, void* workspace,
    size_t workspace_bytes, void* cu_stream);

/* Row-major matmul: the chain of iree_uk_e2e_matmul (ukernel/tools/e2e_matmul_benchmark.c:173-300:
 * pack LHS, pack RHS with TRANSPOSE_INNER|TRANSPOSE_OUTER, pack the accumulator, mmt4d, unpack)
 * as one operation on row-major operands, with no packed copy of the LHS or of the result.
 * lhs is [M][K], rhs is [K][N], out is [M][N]; M, N, K count ELEMENTS; offsets and strides are
 * in elements of the respective buffer; padding is zero as in the chain. `flags` is one of the
 * tensor-core type triples (IREE_UK_FLAG_MMT4D_TYPE_S8S8S32, _F16F16F32, _BF16BF16F32),
 * optionally | IREE_UK_FLAG_MMT4D_ACCUMULATE (out holds the accumulator on entry). The result
 * equals that of the chain for any tile sizes: exactly for s8s8s32, up to the order of the f32
 * additions for the float triples. */
typedef struct iree_uk_b200_matmul_params_t {
  const void* lhs_buffer;
  iree_uk_index_t lhs_offset;
  iree_uk_index_t lhs_stride0;
  const void* rhs_buffer;
  iree_uk_index_t rhs_offset;
  iree_uk_index_t rhs_stride0;
  void* out_buffer;
  iree_uk_index_t out_offset;
  iree_uk_index_t out_stride0;
  iree_uk_index_t M;
  iree_uk_index_t N;
  iree_uk_index_t K;
  uint32_t flags;
} iree_uk_b200_matmul_params_t;

/* Scratch bytes iree_uk_b200_matmul needs (a K-major copy of the RHS, and room for a copy of
 * the LHS that is used only when the LHS base or row pitch is not 16-byte aligned); 0 when the
 * parameters are rejected. */
IREE_UK_B200_EXPORT size_t
iree_uk_b200_matmul_workspace_size(const iree_uk_b200_matmul_params_t* params);

/* Enqueues the matmul on `cu_stream`. `workspace`: 256-byte aligned device memory of at least
 * iree_uk_b200_matmul_workspace_size bytes, in use until the work has completed. */
IREE_UK_B200_EXPORT int iree_uk_b200_matmul(const iree_uk_b200_matmul_params_t* params,
                                            void* workspace, size_t workspace_bytes,
                                            void* cu_stream);

/* Device bytes iree_uk_b200_mmt4d_host needs for `params` (device copies of both operands and
 * of the output, plus the tensor-core scratch of one chunk); 0 when the parameters are rejected. */
IREE_UK_B200_EXPORT size_t
iree_uk_b200_mmt4d_host_arena_size(const iree_uk_mmt4d_params_t* params);

/* iree_uk_mmt4d_p (ukernel/mmt4d.c:115-141) with the reference's own calling convention for
 * the buffers: lhs_buffer, rhs_buffer and out_buffer are HOST pointers, as in the reference.
 * The operands are copied to the device, the contraction runs on the kernels of this library
 * and the result is copied back into out_buffer; the RHS tile rows are processed in up to 8
 * chunks so that host-to-device copies, kernels and device-to-host copies overlap. All device
 * memory is the caller's `device_arena` (256-byte aligned, at least
 * iree_uk_b200_mmt4d_host_arena_size bytes, in use until the work has completed). The call
 * returns once everything is enqueued; out_buffer is complete when work enqueued on `cu_stream`
 * after this call runs (or after synchronising it). Host buffers should be page-locked, or the
 * copies will not overlap. Uses three internal streams per device, created on first use; calls
 * for one device from several host threads take turns enqueueing and run one after another. */
IREE_UK_B200_EXPORT int iree_uk_b200_mmt4d_host(const iree_uk_mmt4d_params_t* params,
                                                void* device_arena, size_t arena_bytes,
                                                void* cu_stream);

/* As iree_uk_b200_mmt4d_host, for a caller that has already brought the LHS to the device:
 * params->lhs_buffer / lhs_offset / lhs_stride0 are ignored and the LHS tile rows are read from
 * `device_lhs`, `device_lhs_stride0` elements apart (device memory of the current device, 16-byte
 * aligned rows for the tensor-core kernels, ready once the work already enqueued on `cu_stream`
 * has run); RHS and output stay host buffers. This is the per-GPU step of an N-sharded
 * host-buffer mmt4d in which the LHS crosses PCIe once - each GPU uploads 1/G of its tile rows -
 * and is then all-gathered over NVLink, instead of being uploaded in full to every GPU. No
 * counterpart in the reference, whose callers never shard. */
IREE_UK_B200_EXPORT int iree_uk_b200_mmt4d_host_resident_lhs(
    const iree_uk_mmt4d_params_t* params, const void* device_lhs,
    iree_uk_index_t device_lhs_stride0, void* device_arena, size_t arena_bytes, void* cu_stream);

/* Replaces iree_uk_mmt4d_info (ukernel/mmt4d.h:25-27, mmt4d.c:143-149): bit 0 is set when
 * a tensor-core (tcgen05) kernel exists for this (types, M0, N0, K0). */
IREE_UK_B200_EXPORT uint32_t iree_uk_b200_mmt4d_info(int32_t M0, int32_t N0, int32_t K0,
                                                     uint32_t flags);

/* Which kernel iree_uk_b200_mmt4d_ws (with_workspace != 0) or iree_uk_b200_mmt4d
 * (with_workspace == 0) would launch for `params`; an iree_uk_b200_path_t, or a negative
 * status when the parameters are rejected. Mirrors the tile-function selection of
 * ukernel/mmt4d.c:124-138. */
IREE_UK_B200_EXPORT int iree_uk_b200_mmt4d_path(const iree_uk_mmt4d_params_t* params,
                                                int with_workspace);

/* Parameters of GPU `rank` of `world` when the N dimension (RHS tile rows = weight tiles)
 * is split contiguously across GPUs: rank r owns tile rows [r*N/world, (r+1)*N/world)
 * (remainder spread over the first ranks). `rhs_is_local` != 0 means the caller's
 * rhs_buffer already holds only this rank's rows (rhs_offset is kept); otherwise the
 * offset is advanced inside a full RHS. `out_is_local` != 0 means out_buffer is a slab
 * [M][N_local][M0][N0] (out_stride0 is set to N_local*M0*N0); otherwise the slab is
 * addressed inside a full [M][N][M0][N0] output through out_offset. The j loop of
 * ukernel/mmt4d.c:84-98 only advances rhs_panel and out_tile, which is why this needs no
 * reduction. Returns the first owned tile row in *n_begin (may be NULL). */
IREE_UK_B200_EXPORT int iree_uk_b200_mmt4d_shard_params(
    const iree_uk_mmt4d_params_t* full, int rank, int world, int rhs_is_local,
    int out_is_local, iree_uk_mmt4d_params_t* shard, iree_uk_index_t* n_begin);

/* Interleaves `world` gathered output slabs [r][M][N_r][M0*N0] (the layout an all-gather of
 * equal slabs produces) into one [M][N][M0*N0] buffer; elem_size in bytes. N must be
 * divisible by world. No counterpart in the reference (its callers never shard). */
IREE_UK_B200_EXPORT int iree_uk_b200_interleave_slabs(const void* gathered, void* out,
                                                      iree_uk_index_t M, iree_uk_index_t N,
                                                      iree_uk_index_t tile_elems,
                                                      int elem_size, int world,
                                                      void* cu_stream);

/*===----------------------------------------------------------------------===*/
/* pack / unpack                                                               */
/*===----------------------------------------------------------------------===*/

/* Replaces iree_uk_pack_p (ukernel/pack.c:315-322). */
IREE_UK_B200_EXPORT int iree_uk_b200_pack(const iree_uk_pack_params_t* params,
                                          void* cu_stream);

/* Flat-argument twin of iree_uk_pack (ukernel/pack.h:26-34, pack.c:325-352). */
IREE_UK_B200_EXPORT int iree_uk_b200_pack_flat(
    const void* in_buffer, iree_uk_index_t in_offset, iree_uk_index_t in_stride0,
    iree_uk_index_t in_stride1, void* out_buffer, iree_uk_index_t out_offset,
    iree_uk_index_t out_stride0, iree_uk_index_t out_stride1, iree_uk_index_t in_size0,
    iree_uk_index_t in_size1, iree_uk_index_t out_size0, iree_uk_index_t out_size1,
    iree_uk_index_t out_size2, iree_uk_index_t out_size3, uint64_t padding_value,
    uint32_t flags, const uint64_t* cpu_data, void* cu_stream);

/* Which kernel serves the pack call (iree_uk_b200_path_t) or a negative status. Mirrors
 * iree_uk_pack_select_tile_func (ukernel/pack_tile.c:57-71). */
IREE_UK_B200_EXPORT int iree_uk_b200_pack_path(const iree_uk_pack_params_t* params);

/* Replaces iree_uk_unpack_p (ukernel/unpack.c:249-257). */
IREE_UK_B200_EXPORT int iree_uk_b200_unpack(const iree_uk_unpack_params_t* params,
                                            void* cu_stream);

/* Flat-argument twin of iree_uk_unpack (ukernel/unpack.h:17-25, unpack.c:259-285). */
IREE_UK_B200_EXPORT int iree_uk_b200_unpack_flat(
    const void* in_buffer, iree_uk_index_t in_offset, iree_uk_index_t in_stride0,
    iree_uk_index_t in_stride1, void* out_buffer, iree_uk_index_t out_offset,
    iree_uk_index_t out_stride0, iree_uk_index_t out_stride1, iree_uk_index_t in_size0,
    iree_uk_index_t in_size1, iree_uk_index_t in_size2, iree_uk_index_t in_size3,
    iree_uk_index_t out_size0, iree_uk_index_t out_size1, uint32_t flags,
    const uint64_t* cpu_data, void* cu_stream);

/* Which kernel serves the unpack call, as for pack. Mirrors
 * iree_uk_unpack_select_tile_func (ukernel/unpack_tile.c:57-71). */
IREE_UK_B200_EXPORT int iree_uk_b200_unpack_path(const iree_uk_unpack_params_t* params);

/*===----------------------------------------------------------------------===*/
/* query_tile_sizes                                                            */
/*===----------------------------------------------------------------------===*/

/* Replaces iree_uk_query_tile_sizes_2d (ukernel/query_tile_sizes.c:65-76): the (M0,K0),
 * (N0,K0) or (M0,N0) tile a caller should pack with so that mmt4d lands on the tensor-core
 * path: M0xN0xK0 = 16x16x1 for f16, 16x16x2 for bf16 and i8 — the shapes the reference's
 * x86-64 encoder picks (compiler/src/iree/compiler/Codegen/ExternalInterfaces/
 * CPUEncodingExternalModels.cpp:479-585) — and, for f32 (no tensor-core kernel here), the
 * 16x16x1 the reference answers on AVX-512 (ukernel/arch/x86_64/
 * query_tile_sizes_x86_64_entry_point.c:10-25).
 * With IREE_UK_B200_FLAG_QUERY_TILE_SIZES_REFERENCE_X86_64 set in params->flags the call answers
 * exactly what the reference's x86-64 build answers for params->cpu_data (then required, not
 * ignored): f32 16x1x16 / 8x1x8 / 8x1x4 and i8 16x2x16 / 8x2x8 / 8x2x4 by AVX-512 / AVX2 / neither
 * (query_tile_sizes_x86_64_entry_point.c:10-64), and the generic 8x4x8 for the other operations
 * (query_tile_sizes.c:35-41) - for callers that keep a CPU pipeline's packed layouts. */
IREE_UK_B200_EXPORT int iree_uk_b200_query_tile_sizes_2d(
    const iree_uk_query_tile_sizes_2d_params_t* params,
    iree_uk_query_tile_sizes_2d_out_params_t* out_params);

/*===----------------------------------------------------------------------===*/
/* Device-side status                                                          */
/*===----------------------------------------------------------------------===*/

/* Every device-side wait in this library (mbarrier phases of the TMA/MMA pipeline) is
 * bounded; a wait that runs out records a code in a per-device status word and the kernel
 * returns. This call synchronises `cu_stream`, reads and clears that word and returns
 * IREE_UK_B200_OK or IREE_UK_B200_DEVICE_TIMEOUT; *detail (may be NULL) receives the raw
 * word. It is the only entry point that synchronises. No counterpart in the reference. */
IREE_UK_B200_EXPORT int iree_uk_b200_device_status(void* cu_stream, uint32_t* detail);

/*===----------------------------------------------------------------------===*/
/* Kernel timing (benchmarks)                                                  */
/*===----------------------------------------------------------------------===*/

/* Off by default. iree_uk_b200_kernel_timing(n) with n > 0 makes every n-th later tensor-core
 * mmt4d call on the CURRENT device record three CUDA events on its stream: before its pre-pass,
 * between pre-pass and main kernel, and after the main kernel (a recorded call therefore runs
 * its two kernels without their usual overlap); n = 0 switches it off. The last 64 recorded
 * calls are remembered per device. iree_uk_b200_kernel_timing_mean_ms waits for the last
 * recorded call and returns the mean pre-pass and main-kernel milliseconds over the remembered
 * calls and their number (IREE_UK_B200_INVALID_ARGUMENT when nothing was recorded). This is how
 * a benchmark separates the main kernel's duration from the step it is part of. No counterpart
 * in the reference. */
IREE_UK_B200_EXPORT int iree_uk_b200_kernel_timing(int every);
IREE_UK_B200_EXPORT int iree_uk_b200_kernel_timing_mean_ms(float* prepass_ms, float* main_ms,
                                                           int* count);

/* Library build identification: "iree_uk_b200 <version> sm_100a". */
IREE_UK_B200_EXPORT const char* iree_uk_b200_version(void);

#ifdef __cplusplus
} /* extern "C" */
#endif

#if defined(__cplusplus)
static_assert(sizeof(iree_uk_mmt4d_params_t) == 120, "mmt4d params layout");
static_assert(sizeof(iree_uk_pack_params_t) == 136, "pack params layout");
static_assert(sizeof(iree_uk_unpack_params_t) == 128, "unpack params layout");
static_assert(offsetof(iree_uk_mmt4d_params_t, M0) == 96, "mmt4d params layout");
static_assert(offsetof(iree_uk_mmt4d_params_t, flags) == 108, "mmt4d params layout");
static_assert(offsetof(iree_uk_mmt4d_params_t, cpu_data) == 112, "mmt4d params layout");
static_assert(offsetof(iree_uk_pack_params_t, padding_value) == 112, "pack params layout");
static_assert(offsetof(iree_uk_pack_params_t, flags) == 120, "pack params layout");
static_assert(offsetof(iree_uk_unpack_params_t, flags) == 112, "unpack params layout");
#else
_Static_assert(sizeof(iree_uk_mmt4d_params_t) == 120, "mmt4d params layout");
_Static_assert(sizeof(iree_uk_pack_params_t) == 136, "pack params layout");
_Static_assert(sizeof(iree_uk_unpack_params_t) == 128, "unpack params layout");
#endif

#endif /* IREE_UK_B200_H_ */
