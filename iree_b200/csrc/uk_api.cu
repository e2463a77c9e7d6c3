// extern "C" entry points of libiree_uk_b200.so: validation, kernel selection, launch.
#include <cstdio>
#include <cstring>
#include <atomic>
#include <initializer_list>
#include <mutex>
#include <vector>

#include <cuda.h>

#include "uk_common.h"
#include "../../include/iree_uk_b200_testing.h"

namespace uk {

// Written by kernels whose bounded waits ran out; lives in each device's static memory, so
// nothing is allocated for it.
__device__ uint32_t g_status_word;

uint32_t* device_status_word() {
  constexpr int kMaxDevices = 64;
  static uint32_t* addr[kMaxDevices] = {};
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!addr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) return nullptr;
    addr[dev] = static_cast<uint32_t*>(p);
  }
  return addr[dev];
}

static std::atomic<int> g_f32_mode{0};
int f32_mode() { return g_f32_mode.load(std::memory_order_relaxed); }

KernelTiming* kernel_timing() {
  constexpr int kMaxDevices = 64;
  static KernelTiming rings[kMaxDevices];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  return &rings[dev];
}

static std::atomic<int> g_starve{0};
bool testing_starve_producers() { return g_starve.load(std::memory_order_relaxed) != 0; }

namespace {

enum class Mmt4dPath { None, Generic, Tc, TcRetile, TcSw, Gemv, Narrow, ZeroFill };

// Kernel selection, the analogue of ukernel/mmt4d.c:105-138 (early-out, then an
// architecture-specific tile function, else the generic one).
int select_mmt4d(const iree_uk_mmt4d_params_t* p, bool have_ws, Mmt4dPath* path) {
  const int rc = validate_mmt4d(p);
  if (rc) return rc;
  const bool acc = (p->flags & IREE_UK_FLAG_MMT4D_ACCUMULATE) != 0;
  if (p->M == 0 || p->N == 0 || (p->K == 0 && acc)) { *path = Mmt4dPath::None; return 0; }
  Mmt4dTypes t;
  mmt4d_types(p->flags, &t);
  // A zero-sized inner tile addresses no output element.
  if (p->M0 == 0 || p->N0 == 0) { *path = Mmt4dPath::None; return 0; }
  if (p->K == 0 || p->K0 == 0) { *path = Mmt4dPath::ZeroFill; return 0; }
  const bool force_generic = env_flag("IREE_UK_B200_FORCE_GENERIC");
  if (!force_generic) {
    // s16u4s32: the tensor-core path from 16 rows on, below that the GEMV. Measured per call at
    // N = 14336, K = 4096: the tensor-core path 40-45 us whatever M (its pre-pass widens all the
    // weights), the GEMV with four rows per block 15 / 24 / 41 / 59 / 74 us for 4 / 8 / 16 / 24 / 31 rows.
    if (have_ws && p->M >= 16 && mmt4d_tc_s16u4_eligible(p)) { *path = Mmt4dPath::TcRetile; return 0; }
    if (mmt4d_gemv_s16u4_eligible(p)) { *path = Mmt4dPath::Gemv; return 0; }
    // narrowed M0 with N0 = 16: weight streaming, with or without scratch
    if (mmt4d_narrow_eligible(p)) { *path = Mmt4dPath::Narrow; return 0; }
    if (have_ws && mmt4d_tc_eligible(p)) { *path = Mmt4dPath::TcRetile; return 0; }
    // s16s16s32 16x16x2: byte planes on the tensor cores (scratch only; generic kernel without)
    if (have_ws && mmt4d_tc_s16s16_eligible(p)) { *path = Mmt4dPath::TcRetile; return 0; }
    if (have_ws && mmt4d_tc_s16s8_eligible(p)) { *path = Mmt4dPath::TcRetile; return 0; }
    // s8s4s32 16x16xK0: nibbles widened by the pre-pass, then the s8s8s32 kernels (scratch only)
    if (have_ws && mmt4d_tc_s8s4_eligible(p)) { *path = Mmt4dPath::TcRetile; return 0; }
    // Without scratch, a 16-bit K0 = 1 operand ([tile][K1][16]) can still be read by TMA as an
    // MN-major tensor-core operand; K0 = 2 operands cannot and fall to the generic kernel.
    if (!have_ws && mmt4d_tc_direct_eligible(p)) { *path = Mmt4dPath::Tc; return 0; }
    // Any other tensor-core triple without scratch: the kernel whose producer warps re-tile the
    // operands on their way into shared memory.
    if (!have_ws && mmt4d_tc_sw_eligible(p)) { *path = Mmt4dPath::TcSw; return 0; }
  }
  *path = Mmt4dPath::Generic;
  return 0;
}

int path_code(Mmt4dPath p) {
  switch (p) {
    case Mmt4dPath::None: return IREE_UK_B200_PATH_NONE;
    case Mmt4dPath::Generic: return IREE_UK_B200_PATH_GENERIC;
    case Mmt4dPath::Tc: return IREE_UK_B200_PATH_TCGEN05;
    case Mmt4dPath::TcSw: return IREE_UK_B200_PATH_TCGEN05;
    case Mmt4dPath::TcRetile: return IREE_UK_B200_PATH_TCGEN05_RETILE;
    case Mmt4dPath::Gemv: return IREE_UK_B200_PATH_GEMV;
    case Mmt4dPath::Narrow: return IREE_UK_B200_PATH_GEMV;
    default: return IREE_UK_B200_PATH_ZERO_FILL;
  }
}

int run_mmt4d(const iree_uk_mmt4d_params_t* p, void* ws, size_t ws_bytes, bool have_ws,
              void* cu_stream) {
  Mmt4dPath path;
  const int rc = select_mmt4d(p, have_ws, &path);
  if (rc) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(cu_stream);
  switch (path) {
    case Mmt4dPath::None: return IREE_UK_B200_OK;
    case Mmt4dPath::ZeroFill: return launch_mmt4d_zero_fill(p, stream);
    case Mmt4dPath::Gemv: return launch_mmt4d_gemv_s16u4(p, stream);
    case Mmt4dPath::Narrow: return launch_mmt4d_narrow(p, stream);
    case Mmt4dPath::TcRetile: return launch_mmt4d_tc(p, ws, ws_bytes, kTcVariantDefault, stream);
    case Mmt4dPath::Tc: return launch_mmt4d_tc(p, nullptr, 0, kTcVariantDirect, stream);
    case Mmt4dPath::TcSw: return launch_mmt4d_tc_sw(p, stream);
    default: return launch_mmt4d_generic(p, stream);
  }
}

}  // namespace
}  // namespace uk

using namespace uk;

extern "C" {

const char* iree_uk_b200_status_string(int status) {
  switch (status) {
    case IREE_UK_B200_OK: return "OK";
    case IREE_UK_B200_INVALID_ARGUMENT: return "INVALID_ARGUMENT";
    case IREE_UK_B200_UNSUPPORTED: return "UNSUPPORTED";
    case IREE_UK_B200_CUDA_ERROR: return "CUDA_ERROR";
    case IREE_UK_B200_WORKSPACE_TOO_SMALL: return "WORKSPACE_TOO_SMALL";
    case IREE_UK_B200_DEVICE_TIMEOUT: return "DEVICE_TIMEOUT";
    default: return "UNKNOWN";
  }
}

const char* iree_uk_b200_version(void) { return "iree_uk_b200 0.1 sm_100a"; }

int iree_uk_b200_mmt4d(const iree_uk_mmt4d_params_t* params, void* cu_stream) {
  return run_mmt4d(params, nullptr, 0, false, cu_stream);
}

size_t iree_uk_b200_mmt4d_workspace_size(const iree_uk_mmt4d_params_t* params) {
  Mmt4dPath path;
  if (select_mmt4d(params, true, &path) || path != Mmt4dPath::TcRetile) {
    // Alignment of the buffers may differ between this query and the call; size by shape.
    if (!params || validate_mmt4d(params)) return 0;
  }
  return mmt4d_tc_workspace_size(params);
}

int iree_uk_b200_mmt4d_ws(const iree_uk_mmt4d_params_t* params, void* workspace,
                          size_t workspace_bytes, void* cu_stream) {
  // No workspace at all is the scratch-free call. A workspace that is offered but too small for
  // the kernel that would use it is reported, never quietly replaced by a slower kernel.
  if (!workspace || workspace_bytes == 0) return run_mmt4d(params, nullptr, 0, false, cu_stream);
  Mmt4dPath path;
  const int rc = select_mmt4d(params, true, &path);
  if (rc) return rc;
  if (path == Mmt4dPath::TcRetile && workspace_bytes < mmt4d_tc_workspace_size(params))
    return IREE_UK_B200_WORKSPACE_TOO_SMALL;
  return run_mmt4d(params, workspace, workspace_bytes, true, cu_stream);
}

namespace {
// The current device's scratch pool, created on first use; nullptr on failure.
cudaMemPool_t scratch_pool() {
  constexpr int kMaxDevices = 64;
  static cudaMemPool_t pools[kMaxDevices] = {};
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!pools[dev]) {
    cudaMemPoolProps props = {};
    props.allocType = cudaMemAllocationTypePinned;
    props.handleTypes = cudaMemHandleTypeNone;
    props.location.type = cudaMemLocationTypeDevice;
    props.location.id = dev;
    cudaMemPool_t pool = nullptr;
    if (cudaMemPoolCreate(&pool, &props) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    uint64_t keep = ~uint64_t(0);
    if (cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep) != cudaSuccess) {
      cudaGetLastError();
      cudaMemPoolDestroy(pool);
      return nullptr;
    }
    pools[dev] = pool;
  }
  return pools[dev];
}
}  // namespace

int iree_uk_b200_mmt4d_pooled(const iree_uk_mmt4d_params_t* params, void* cu_stream) {
  Mmt4dPath path;
  const int rc = select_mmt4d(params, true, &path);
  if (rc) return rc;
  if (path != Mmt4dPath::TcRetile) return run_mmt4d(params, nullptr, 0, false, cu_stream);
  const size_t bytes = mmt4d_tc_workspace_size(params);
  cudaMemPool_t pool = scratch_pool();
  if (!pool) return IREE_UK_B200_CUDA_ERROR;
  cudaStream_t stream = static_cast<cudaStream_t>(cu_stream);
  void* ws = nullptr;
  if (cudaMallocFromPoolAsync(&ws, bytes, pool, stream) != cudaSuccess) {
    cudaGetLastError();
    return IREE_UK_B200_CUDA_ERROR;
  }
  const int run = run_mmt4d(params, ws, bytes, true, cu_stream);
  // Stream-ordered: the memory returns to the pool after the kernels enqueued above.
  if (cudaFreeAsync(ws, stream) != cudaSuccess) {
    cudaGetLastError();
    return run ? run : IREE_UK_B200_CUDA_ERROR;
  }
  return run;
}

int iree_uk_b200_scratch_pool_trim(size_t keep_bytes) {
  cudaMemPool_t pool = scratch_pool();
  if (!pool) return IREE_UK_B200_CUDA_ERROR;
  return cuda_status(cudaMemPoolTrimTo(pool, keep_bytes));
}

int iree_uk_b200_mmt4d_flat(const void* lhs_buffer, iree_uk_index_t lhs_offset,
                            iree_uk_index_t lhs_stride0, const void* rhs_buffer,
                            iree_uk_index_t rhs_offset, iree_uk_index_t rhs_stride0,
                            void* out_buffer, iree_uk_index_t out_offset,
                            iree_uk_index_t out_stride0, iree_uk_index_t M, iree_uk_index_t N,
                            iree_uk_index_t K, int32_t M0, int32_t N0, int32_t K0, uint32_t flags,
                            const uint64_t* cpu_data, void* workspace, size_t workspace_bytes,
                            void* cu_stream) {
  iree_uk_mmt4d_params_t p;
  p.lhs_buffer = lhs_buffer; p.lhs_offset = lhs_offset; p.lhs_stride0 = lhs_stride0;
  p.rhs_buffer = rhs_buffer; p.rhs_offset = rhs_offset; p.rhs_stride0 = rhs_stride0;
  p.out_buffer = out_buffer; p.out_offset = out_offset; p.out_stride0 = out_stride0;
  p.M = M; p.N = N; p.K = K; p.M0 = M0; p.N0 = N0; p.K0 = K0;
  p.flags = flags; p.cpu_data = cpu_data;
  return iree_uk_b200_mmt4d_ws(&p, workspace, workspace_bytes, cu_stream);
}

uint32_t iree_uk_b200_mmt4d_info(int32_t M0, int32_t N0, int32_t K0, uint32_t flags) {
  const uint32_t type = flags & IREE_UK_FLAG_MMT4D_TYPE_MASK;
  const bool skip = (flags & IREE_UK_FLAG_MMT4D_SKIP_INTERMEDIATE_ROUNDINGS) != 0;
  const bool tc_type = type == IREE_UK_FLAG_MMT4D_TYPE_S8S8S32 ||
                       type == IREE_UK_FLAG_MMT4D_TYPE_F16F16F32 ||
                       type == IREE_UK_FLAG_MMT4D_TYPE_BF16BF16F32 ||
                       (skip && (type == IREE_UK_FLAG_MMT4D_TYPE_F16F16F16 ||
                                 type == IREE_UK_FLAG_MMT4D_TYPE_BF16BF16BF16)) ||
                       (type == IREE_UK_FLAG_MMT4D_TYPE_F32F32F32 && f32_mode() == IREE_UK_B200_F32_MODE_TF32X3);
  const int es = type == IREE_UK_FLAG_MMT4D_TYPE_S8S8S32 ? 1 : (type == IREE_UK_FLAG_MMT4D_TYPE_F32F32F32 ? 4 : 2);
  const int g = K0 * es;
  if (tc_type && M0 == 16 && N0 == 16 && (g == 1 || g == 2 || g == 4 || g == 8 || g == 16))
    return IREE_UK_FLAG_MMT4D_INFO_HAVE_ARCHITECTURE_SPECIFIC_TILE_FUNCTION;
  if (type == IREE_UK_FLAG_MMT4D_TYPE_S16U4S32 && M0 == 1 && N0 == 32 && K0 == 8)
    return IREE_UK_FLAG_MMT4D_INFO_HAVE_ARCHITECTURE_SPECIFIC_TILE_FUNCTION;
  if ((type == IREE_UK_FLAG_MMT4D_TYPE_S16S16S32 || type == IREE_UK_FLAG_MMT4D_TYPE_S16S8S32) &&
      M0 == 16 && N0 == 16 && K0 == 2)
    return IREE_UK_FLAG_MMT4D_INFO_HAVE_ARCHITECTURE_SPECIFIC_TILE_FUNCTION;
  if (type == IREE_UK_FLAG_MMT4D_TYPE_S8S4S32 && M0 == 16 && N0 == 16 &&
      (K0 == 2 || K0 == 4 || K0 == 8 || K0 == 16))
    return IREE_UK_FLAG_MMT4D_INFO_HAVE_ARCHITECTURE_SPECIFIC_TILE_FUNCTION;
  // narrowed M0: the weight-streaming kernel
  const bool narrow_type = (type == IREE_UK_FLAG_MMT4D_TYPE_S8S8S32 && K0 == 2) ||
                           (type == IREE_UK_FLAG_MMT4D_TYPE_F16F16F32 && K0 == 1) ||
                           (type == IREE_UK_FLAG_MMT4D_TYPE_BF16BF16F32 && K0 == 2);
  if (narrow_type && N0 == 16 && (M0 == 1 || M0 == 2 || M0 == 4 || M0 == 8))
    return IREE_UK_FLAG_MMT4D_INFO_HAVE_ARCHITECTURE_SPECIFIC_TILE_FUNCTION;
  return 0;
}

int iree_uk_b200_set_f32_mode(int mode) {
  if (mode != IREE_UK_B200_F32_MODE_CUDA_CORES && mode != IREE_UK_B200_F32_MODE_TF32X3)
    return g_f32_mode.load();
  return g_f32_mode.exchange(mode);
}

int iree_uk_b200_mmt4d_ws_peers(const iree_uk_mmt4d_params_t* params,
                                const void* const* peer_out_buffers, int num_peers,
                                void* workspace, size_t workspace_bytes, void* cu_stream) {
  if (num_peers < 0 || num_peers > IREE_UK_B200_MAX_PEERS || (num_peers && !peer_out_buffers))
    return IREE_UK_B200_INVALID_ARGUMENT;
  Mmt4dPath path;
  const int rc = select_mmt4d(params, true, &path);
  if (rc) return rc;
  if (path != Mmt4dPath::TcRetile ||
      (params->flags & IREE_UK_FLAG_MMT4D_TYPE_MASK) == IREE_UK_FLAG_MMT4D_TYPE_S16U4S32)
    return IREE_UK_B200_UNSUPPORTED;
  if (!workspace || workspace_bytes < mmt4d_tc_workspace_size(params))
    return IREE_UK_B200_WORKSPACE_TOO_SMALL;
  return launch_mmt4d_tc(params, workspace, workspace_bytes, kTcVariantDefault,
                         static_cast<cudaStream_t>(cu_stream), peer_out_buffers, num_peers);
}

int iree_uk_b200_mmt4d_ws_multicast(const iree_uk_mmt4d_params_t* params,
                                    const void* multicast_out_buffer, void* workspace,
                                    size_t workspace_bytes, void* cu_stream) {
  if (!multicast_out_buffer) return IREE_UK_B200_INVALID_ARGUMENT;
  Mmt4dPath path;
  const int rc = select_mmt4d(params, true, &path);
  if (rc) return rc;
  if (path != Mmt4dPath::TcRetile ||
      (params->flags & IREE_UK_FLAG_MMT4D_TYPE_MASK) == IREE_UK_FLAG_MMT4D_TYPE_S16U4S32)
    return IREE_UK_B200_UNSUPPORTED;
  if (!workspace || workspace_bytes < mmt4d_tc_workspace_size(params))
    return IREE_UK_B200_WORKSPACE_TOO_SMALL;
  return launch_mmt4d_tc(params, workspace, workspace_bytes, kTcVariantDefault,
                         static_cast<cudaStream_t>(cu_stream), nullptr, 0, multicast_out_buffer);
}

int iree_uk_b200_mmt4d_ws_unpacked(const iree_uk_mmt4d_params_t* params, iree_uk_index_t out_size0,
                                   iree_uk_index_t out_size1, void* workspace,
                                   size_t workspace_bytes, void* cu_stream) {
  const int rc = validate_mmt4d(params);
  if (rc) return rc;
  const iree_uk_mmt4d_params_t& p = *params;
  if (out_size0 < 0 || out_size1 < 0 || out_size0 > p.M * p.M0 || out_size1 > p.N * p.N0 ||
      p.out_stride0 < out_size1)
    return IREE_UK_B200_INVALID_ARGUMENT;
  const bool acc = (p.flags & IREE_UK_FLAG_MMT4D_ACCUMULATE) != 0;
  if (out_size0 == 0 || out_size1 == 0 || (p.K == 0 && acc)) return IREE_UK_B200_OK;
  const uint32_t type = p.flags & IREE_UK_FLAG_MMT4D_TYPE_MASK;
  if (type == IREE_UK_FLAG_MMT4D_TYPE_S16U4S32 || !mmt4d_tc_operands_eligible(params)) {
    if (p.K == 0 || p.K0 == 0) {
      // an empty reduction without ACCUMULATE: zeros, for any type with a 32-bit output
      Mmt4dTypes t;
      if (!mmt4d_types(p.flags, &t) || elem_bits(t.out) != 32) return IREE_UK_B200_UNSUPPORTED;
      return cudaMemset2DAsync(static_cast<char*>(p.out_buffer) + p.out_offset * 4,
                               size_t(p.out_stride0) * 4, 0, size_t(out_size1) * 4,
                               size_t(out_size0), static_cast<cudaStream_t>(cu_stream)) == cudaSuccess
                 ? IREE_UK_B200_OK : IREE_UK_B200_CUDA_ERROR;
    }
    return IREE_UK_B200_UNSUPPORTED;
  }
  const RowMajorOut rm = {out_size0, out_size1};
  return launch_mmt4d_tc(params, workspace, workspace_bytes, kTcVariantDefault,
                         static_cast<cudaStream_t>(cu_stream), nullptr, 0, nullptr, nullptr, &rm);
}

size_t iree_uk_b200_mmt4d_prepared_rhs_size(const iree_uk_mmt4d_params_t* params) {
  if (!params || validate_mmt4d(params)) return 0;
  return mmt4d_tc_prepared_rhs_size(params);
}

size_t iree_uk_b200_mmt4d_prepared_workspace_size(const iree_uk_mmt4d_params_t* params) {
  if (!params || validate_mmt4d(params)) return 0;
  return mmt4d_tc_prepared_workspace_size(params);
}

int iree_uk_b200_mmt4d_prepare_rhs(const iree_uk_mmt4d_params_t* params, void* prepared_rhs,
                                   size_t prepared_bytes, void* cu_stream) {
  const int rc = validate_mmt4d(params);
  if (rc) return rc;
  return launch_mmt4d_tc_prepare_rhs(params, prepared_rhs, prepared_bytes,
                                     static_cast<cudaStream_t>(cu_stream));
}

int iree_uk_b200_mmt4d_ws_prepared(const iree_uk_mmt4d_params_t* params, const void* prepared_rhs,
                                   void* workspace, size_t workspace_bytes, void* cu_stream) {
  if (!prepared_rhs) return IREE_UK_B200_INVALID_ARGUMENT;
  Mmt4dPath path;
  const int rc = select_mmt4d(params, true, &path);
  if (rc) return rc;
  if (path == Mmt4dPath::None) return IREE_UK_B200_OK;
  // s16u4s32 with prepared weights takes the tensor-core kernel whatever M: nothing is left of
  // the pre-pass but the byte-plane split of the LHS
  const bool s16u4 = (params->flags & IREE_UK_FLAG_MMT4D_TYPE_MASK) == IREE_UK_FLAG_MMT4D_TYPE_S16U4S32 &&
                     path != Mmt4dPath::ZeroFill && mmt4d_tc_s16u4_eligible(params);
  if ((path != Mmt4dPath::TcRetile && !s16u4) || !mmt4d_tc_prepared_rhs_size(params))
    return IREE_UK_B200_UNSUPPORTED;
  return launch_mmt4d_tc(params, workspace, workspace_bytes, kTcVariantDefault,
                         static_cast<cudaStream_t>(cu_stream), nullptr, 0, nullptr, prepared_rhs);
}

int iree_uk_b200_mmt4d_sharded(int n_gpus, const int* device_ids,
                               const iree_uk_mmt4d_params_t* per_gpu, void* const* workspaces,
                               const size_t* workspace_bytes, void* const* cu_streams,
                               int replicate_output) {
  if (n_gpus < 1 || n_gpus > IREE_UK_B200_MAX_PEERS + 1 || !device_ids || !per_gpu || !workspaces ||
      !workspace_bytes || !cu_streams)
    return IREE_UK_B200_INVALID_ARGUMENT;
  int previous = 0;
  if (cudaGetDevice(&previous) != cudaSuccess) return IREE_UK_B200_CUDA_ERROR;
  int rc = IREE_UK_B200_OK;
  for (int g = 0; g < n_gpus && rc == IREE_UK_B200_OK; ++g) {
    if (cudaSetDevice(device_ids[g]) != cudaSuccess) { rc = IREE_UK_B200_CUDA_ERROR; break; }
    if (!replicate_output || n_gpus == 1) {
      rc = iree_uk_b200_mmt4d_ws(&per_gpu[g], workspaces[g], workspace_bytes[g], cu_streams[g]);
      continue;
    }
    const void* peers[IREE_UK_B200_MAX_PEERS];
    int n = 0;
    for (int h = 0; h < n_gpus && rc == IREE_UK_B200_OK; ++h) {
      if (h == g) continue;
      if (device_ids[h] != device_ids[g]) {
        const cudaError_t e = cudaDeviceEnablePeerAccess(device_ids[h], 0);
        if (e == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
        else if (e != cudaSuccess) { cudaGetLastError(); rc = IREE_UK_B200_CUDA_ERROR; }
      }
      peers[n++] = per_gpu[h].out_buffer;
    }
    if (rc == IREE_UK_B200_OK)
      rc = iree_uk_b200_mmt4d_ws_peers(&per_gpu[g], peers, n, workspaces[g], workspace_bytes[g],
                                       cu_streams[g]);
  }
  cudaSetDevice(previous);
  return rc;
}

namespace {
struct PeerMapping {
  void* base;
  void* ptr;
};
std::mutex g_peer_mu;
std::vector<PeerMapping> g_peer_mappings;
}  // namespace

int iree_uk_b200_peer_export(const void* device_ptr, iree_uk_b200_peer_handle_t* handle) {
  if (!device_ptr || !handle) return IREE_UK_B200_INVALID_ARGUMENT;
  // base of the allocation that holds device_ptr
  typedef CUresult (*GetRange)(CUdeviceptr*, size_t*, CUdeviceptr);
  static GetRange get_range = [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      fn = nullptr;
    return reinterpret_cast<GetRange>(fn);
  }();
  if (!get_range) return IREE_UK_B200_CUDA_ERROR;
  CUdeviceptr base = 0;
  size_t size = 0;
  if (get_range(&base, &size, reinterpret_cast<CUdeviceptr>(device_ptr)) != CUDA_SUCCESS)
    return IREE_UK_B200_CUDA_ERROR;
  cudaIpcMemHandle_t h;
  static_assert(sizeof h == sizeof handle->ipc, "IPC handle size");
  if (cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base)) != cudaSuccess) {
    cudaGetLastError();
    return IREE_UK_B200_CUDA_ERROR;
  }
  std::memcpy(handle->ipc, &h, sizeof h);
  handle->offset = uint64_t(reinterpret_cast<CUdeviceptr>(device_ptr) - base);
  return IREE_UK_B200_OK;
}

int iree_uk_b200_peer_open(const iree_uk_b200_peer_handle_t* handle, void** device_ptr) {
  if (!handle || !device_ptr) return IREE_UK_B200_INVALID_ARGUMENT;
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle->ipc, sizeof h);
  void* base = nullptr;
  if (cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
    cudaGetLastError();
    return IREE_UK_B200_CUDA_ERROR;
  }
  *device_ptr = static_cast<char*>(base) + handle->offset;
  std::lock_guard<std::mutex> lock(g_peer_mu);
  g_peer_mappings.push_back({base, *device_ptr});
  return IREE_UK_B200_OK;
}

int iree_uk_b200_peer_close(void* device_ptr) {
  void* base = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_peer_mu);
    for (size_t i = 0; i < g_peer_mappings.size(); ++i)
      if (g_peer_mappings[i].ptr == device_ptr) {
        base = g_peer_mappings[i].base;
        g_peer_mappings.erase(g_peer_mappings.begin() + i);
        break;
      }
  }
  if (!base) return IREE_UK_B200_INVALID_ARGUMENT;
  return cudaIpcCloseMemHandle(base) == cudaSuccess ? IREE_UK_B200_OK : IREE_UK_B200_CUDA_ERROR;
}

static int validate_matmul(const iree_uk_b200_matmul_params_t* p, int* es) {
  if (!p) return IREE_UK_B200_INVALID_ARGUMENT;
  if (p->flags & ~(IREE_UK_FLAG_MMT4D_TYPE_MASK | IREE_UK_FLAG_MMT4D_ACCUMULATE))
    return IREE_UK_B200_INVALID_ARGUMENT;
  switch (p->flags & IREE_UK_FLAG_MMT4D_TYPE_MASK) {
    case IREE_UK_FLAG_MMT4D_TYPE_S8S8S32: *es = 1; break;
    case IREE_UK_FLAG_MMT4D_TYPE_F16F16F32:
    case IREE_UK_FLAG_MMT4D_TYPE_BF16BF16F32: *es = 2; break;
    default: return IREE_UK_B200_UNSUPPORTED;
  }
  if (p->M < 0 || p->N < 0 || p->K < 0) return IREE_UK_B200_INVALID_ARGUMENT;
  if (p->lhs_stride0 < p->K || p->rhs_stride0 < p->N || p->out_stride0 < p->N)
    return IREE_UK_B200_INVALID_ARGUMENT;
  if (p->M && p->N && !p->out_buffer) return IREE_UK_B200_INVALID_ARGUMENT;
  if (p->M && p->N && p->K && (!p->lhs_buffer || !p->rhs_buffer)) return IREE_UK_B200_INVALID_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(p->out_buffer) & 3) ||
      (reinterpret_cast<uintptr_t>(p->lhs_buffer) & (*es - 1)) ||
      (reinterpret_cast<uintptr_t>(p->rhs_buffer) & (*es - 1)))
    return IREE_UK_B200_INVALID_ARGUMENT;
  return IREE_UK_B200_OK;
}

size_t iree_uk_b200_matmul_workspace_size(const iree_uk_b200_matmul_params_t* params) {
  int es = 0;
  if (validate_matmul(params, &es)) return 0;
  return matmul_workspace_size(params->flags, params->M, params->N, params->K);
}

int iree_uk_b200_matmul(const iree_uk_b200_matmul_params_t* params, void* workspace,
                        size_t workspace_bytes, void* cu_stream) {
  int es = 0;
  const int rc = validate_matmul(params, &es);
  if (rc) return rc;
  const iree_uk_b200_matmul_params_t& p = *params;
  cudaStream_t stream = static_cast<cudaStream_t>(cu_stream);
  if (p.M == 0 || p.N == 0) return IREE_UK_B200_OK;
  char* out = static_cast<char*>(p.out_buffer) + p.out_offset * 4;
  if (p.K == 0) {
    // an empty reduction: the accumulator is kept, or the result is zero
    if (p.flags & IREE_UK_FLAG_MMT4D_ACCUMULATE) return IREE_UK_B200_OK;
    return cudaMemset2DAsync(out, size_t(p.out_stride0) * 4, 0, size_t(p.N) * 4, size_t(p.M),
                             stream) == cudaSuccess ? IREE_UK_B200_OK : IREE_UK_B200_CUDA_ERROR;
  }
  return launch_matmul_rowmajor(
      p.flags, static_cast<const char*>(p.lhs_buffer) + p.lhs_offset * es, p.lhs_stride0 * es,
      static_cast<const char*>(p.rhs_buffer) + p.rhs_offset * es, p.rhs_stride0 * es, out,
      p.out_stride0, p.M, p.N, p.K, workspace, workspace_bytes, stream);
}

int iree_uk_b200_mmt4d_path(const iree_uk_mmt4d_params_t* params, int with_workspace) {
  Mmt4dPath path;
  const int rc = select_mmt4d(params, with_workspace != 0, &path);
  if (rc) return -rc;
  return path_code(path);
}

int iree_uk_b200_mmt4d_shard_params(const iree_uk_mmt4d_params_t* full, int rank, int world,
                                    int rhs_is_local, int out_is_local,
                                    iree_uk_mmt4d_params_t* shard, iree_uk_index_t* n_begin) {
  if (!full || !shard || world < 1 || rank < 0 || rank >= world) return IREE_UK_B200_INVALID_ARGUMENT;
  const int rc = validate_mmt4d(full);
  if (rc) return rc;
  const int64_t base = full->N / world, rem = full->N % world;
  const int64_t begin = rank * base + (rank < rem ? rank : rem);
  const int64_t count = base + (rank < rem ? 1 : 0);
  *shard = *full;
  shard->N = count;
  if (!rhs_is_local) shard->rhs_offset = full->rhs_offset + begin * full->rhs_stride0;
  if (out_is_local) {
    shard->out_stride0 = count * int64_t(full->M0) * full->N0;
  } else {
    shard->out_offset = full->out_offset + begin * int64_t(full->M0) * full->N0;
  }
  if (n_begin) *n_begin = begin;
  return IREE_UK_B200_OK;
}

int iree_uk_b200_interleave_slabs(const void* gathered, void* out, iree_uk_index_t M,
                                  iree_uk_index_t N, iree_uk_index_t tile_elems, int elem_size,
                                  int world, void* cu_stream) {
  if (!gathered || !out || M < 0 || N < 0 || tile_elems <= 0 || elem_size <= 0)
    return IREE_UK_B200_INVALID_ARGUMENT;
  return launch_interleave_slabs(gathered, out, M, N, tile_elems, elem_size, world,
                                 static_cast<cudaStream_t>(cu_stream));
}

// ---- pack ----

static int select_pack(const iree_uk_pack_params_t* p, int* path) {
  const int rc = validate_pack(p);
  if (rc) return rc;
  if (p->out_size0 == 0 || p->out_size1 == 0 || p->out_size2 == 0 || p->out_size3 == 0) {
    *path = IREE_UK_B200_PATH_NONE;  // ukernel/pack.c:106-109
    return 0;
  }
  *path = (!env_flag("IREE_UK_B200_FORCE_GENERIC") && pack_staged_eligible(p))
              ? IREE_UK_B200_PATH_FAST_COPY
              : IREE_UK_B200_PATH_GENERIC;
  return 0;
}

int iree_uk_b200_pack(const iree_uk_pack_params_t* params, void* cu_stream) {
  int path;
  const int rc = select_pack(params, &path);
  if (rc) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(cu_stream);
  if (path == IREE_UK_B200_PATH_NONE) return IREE_UK_B200_OK;
  if (path == IREE_UK_B200_PATH_FAST_COPY) return launch_pack_staged(params, stream);
  return launch_pack_generic(params, stream);
}

int iree_uk_b200_pack_path(const iree_uk_pack_params_t* params) {
  int path;
  const int rc = select_pack(params, &path);
  return rc ? -rc : path;
}

int iree_uk_b200_pack_flat(const void* in_buffer, iree_uk_index_t in_offset,
                           iree_uk_index_t in_stride0, iree_uk_index_t in_stride1,
                           void* out_buffer, iree_uk_index_t out_offset,
                           iree_uk_index_t out_stride0, iree_uk_index_t out_stride1,
                           iree_uk_index_t in_size0, iree_uk_index_t in_size1,
                           iree_uk_index_t out_size0, iree_uk_index_t out_size1,
                           iree_uk_index_t out_size2, iree_uk_index_t out_size3,
                           uint64_t padding_value, uint32_t flags, const uint64_t* cpu_data,
                           void* cu_stream) {
  iree_uk_pack_params_t p;
  p.in_buffer = in_buffer; p.in_offset = in_offset; p.in_stride0 = in_stride0;
  p.in_stride1 = in_stride1; p.out_buffer = out_buffer; p.out_offset = out_offset;
  p.out_stride0 = out_stride0; p.out_stride1 = out_stride1; p.in_size0 = in_size0;
  p.in_size1 = in_size1; p.out_size0 = out_size0; p.out_size1 = out_size1;
  p.out_size2 = out_size2; p.out_size3 = out_size3; p.padding_value = padding_value;
  p.flags = flags; p.cpu_data = cpu_data;
  return iree_uk_b200_pack(&p, cu_stream);
}

// ---- unpack ----

static int select_unpack(const iree_uk_unpack_params_t* p, int* path) {
  const int rc = validate_unpack(p);
  if (rc) return rc;
  if (p->out_size0 == 0 || p->out_size1 == 0 || p->in_size0 == 0 || p->in_size1 == 0 ||
      p->in_size2 == 0 || p->in_size3 == 0) {
    *path = IREE_UK_B200_PATH_NONE;  // ukernel/unpack.c:84-86
    return 0;
  }
  *path = (!env_flag("IREE_UK_B200_FORCE_GENERIC") && unpack_staged_eligible(p))
              ? IREE_UK_B200_PATH_FAST_COPY
              : IREE_UK_B200_PATH_GENERIC;
  return 0;
}

int iree_uk_b200_unpack(const iree_uk_unpack_params_t* params, void* cu_stream) {
  int path;
  const int rc = select_unpack(params, &path);
  if (rc) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(cu_stream);
  if (path == IREE_UK_B200_PATH_NONE) return IREE_UK_B200_OK;
  if (path == IREE_UK_B200_PATH_FAST_COPY) return launch_unpack_staged(params, stream);
  return launch_unpack_generic(params, stream);
}

int iree_uk_b200_unpack_path(const iree_uk_unpack_params_t* params) {
  int path;
  const int rc = select_unpack(params, &path);
  return rc ? -rc : path;
}

int iree_uk_b200_unpack_flat(const void* in_buffer, iree_uk_index_t in_offset,
                             iree_uk_index_t in_stride0, iree_uk_index_t in_stride1,
                             void* out_buffer, iree_uk_index_t out_offset,
                             iree_uk_index_t out_stride0, iree_uk_index_t out_stride1,
                             iree_uk_index_t in_size0, iree_uk_index_t in_size1,
                             iree_uk_index_t in_size2, iree_uk_index_t in_size3,
                             iree_uk_index_t out_size0, iree_uk_index_t out_size1, uint32_t flags,
                             const uint64_t* cpu_data, void* cu_stream) {
  iree_uk_unpack_params_t p;
  p.in_buffer = in_buffer; p.in_offset = in_offset; p.in_stride0 = in_stride0;
  p.in_stride1 = in_stride1; p.out_buffer = out_buffer; p.out_offset = out_offset;
  p.out_stride0 = out_stride0; p.out_stride1 = out_stride1; p.in_size0 = in_size0;
  p.in_size1 = in_size1; p.in_size2 = in_size2; p.in_size3 = in_size3;
  p.out_size0 = out_size0; p.out_size1 = out_size1; p.flags = flags; p.cpu_data = cpu_data;
  return iree_uk_b200_unpack(&p, cu_stream);
}

// ---- query_tile_sizes ----

int iree_uk_b200_query_tile_sizes_2d(const iree_uk_query_tile_sizes_2d_params_t* params,
                                     iree_uk_query_tile_sizes_2d_out_params_t* out_params) {
  if (!params || !out_params) return IREE_UK_B200_INVALID_ARGUMENT;
  int64_t m = 16, n = 16, k = 1;
  const bool reference = (params->flags & IREE_UK_B200_FLAG_QUERY_TILE_SIZES_REFERENCE_X86_64) != 0;
  if (params->flags & ~(IREE_UK_FLAG_QUERY_TILE_SIZES_OPERAND_ROLE_MASK |
                        IREE_UK_FLAG_QUERY_TILE_SIZES_OPERATION_MASK |
                        IREE_UK_B200_FLAG_QUERY_TILE_SIZES_REFERENCE_X86_64))
    return IREE_UK_B200_INVALID_ARGUMENT;
  if (reference) {
    // The reference's x86-64 answers (arch/x86_64/query_tile_sizes_x86_64_entry_point.c:10-64,
    // feature predicates arch/x86_64/common_x86_64.h:26-53, bit positions
    // schemas/cpu_feature_bits.inl:85-112); other operations get query_tile_sizes.c:35-41.
    if (!params->cpu_data) return IREE_UK_B200_INVALID_ARGUMENT;
    const uint64_t d = params->cpu_data[0];
    auto all = [&](std::initializer_list<int> bits) {
      for (int b : bits) if (!((d >> b) & 1)) return false;
      return true;
    };
    const bool avx2 = all({15, 11, 14});                       // AVX2, FMA, F16C
    const bool avx512 = avx2 && all({20, 24, 23, 22, 21});     // F, BW, DQ, VL, CD
    const bool vnni = avx512 && all({28});
    switch (params->flags & IREE_UK_FLAG_QUERY_TILE_SIZES_OPERATION_MASK) {
      case IREE_UK_FLAG_QUERY_TILE_SIZES_OPERATION_MATMUL_F32F32F32:
        k = 1; m = avx512 ? 16 : 8; n = avx512 ? 16 : (avx2 ? 8 : 4); break;
      case IREE_UK_FLAG_QUERY_TILE_SIZES_OPERATION_MATMUL_I8I8I32:
        k = 2; m = vnni ? 16 : 8; n = vnni ? 16 : (avx2 ? 8 : 4); break;
      case IREE_UK_FLAG_QUERY_TILE_SIZES_OPERATION_MATMUL_F16F16F32:
      case IREE_UK_FLAG_QUERY_TILE_SIZES_OPERATION_MATMUL_F16F16F16:
      case IREE_UK_FLAG_QUERY_TILE_SIZES_OPERATION_MATMUL_BF16BF16F32:
      case IREE_UK_FLAG_QUERY_TILE_SIZES_OPERATION_MATMUL_BF16BF16BF16:
        m = 8; k = 4; n = 8; break;
      default: return IREE_UK_B200_INVALID_ARGUMENT;
    }
  } else
  switch (params->flags & IREE_UK_FLAG_QUERY_TILE_SIZES_OPERATION_MASK) {
    case IREE_UK_FLAG_QUERY_TILE_SIZES_OPERATION_MATMUL_F32F32F32: k = 1; break;
    case IREE_UK_FLAG_QUERY_TILE_SIZES_OPERATION_MATMUL_I8I8I32: k = 2; break;
    case IREE_UK_FLAG_QUERY_TILE_SIZES_OPERATION_MATMUL_F16F16F32: k = 1; break;
    case IREE_UK_FLAG_QUERY_TILE_SIZES_OPERATION_MATMUL_F16F16F16: k = 1; break;
    case IREE_UK_FLAG_QUERY_TILE_SIZES_OPERATION_MATMUL_BF16BF16F32: k = 2; break;
    case IREE_UK_FLAG_QUERY_TILE_SIZES_OPERATION_MATMUL_BF16BF16BF16: k = 2; break;
    default: return IREE_UK_B200_INVALID_ARGUMENT;  // query_tile_sizes.c:20-21
  }
  switch (params->flags & IREE_UK_FLAG_QUERY_TILE_SIZES_OPERAND_ROLE_MASK) {
    case IREE_UK_FLAG_QUERY_TILE_SIZES_OPERAND_ROLE_LHS:
      out_params->tile_size0 = m; out_params->tile_size1 = k; break;
    case IREE_UK_FLAG_QUERY_TILE_SIZES_OPERAND_ROLE_RHS:
      out_params->tile_size0 = n; out_params->tile_size1 = k; break;
    case IREE_UK_FLAG_QUERY_TILE_SIZES_OPERAND_ROLE_RESULT:
      out_params->tile_size0 = m; out_params->tile_size1 = n; break;
    default: return IREE_UK_B200_INVALID_ARGUMENT;  // query_tile_sizes.c:22-25
  }
  return IREE_UK_B200_OK;
}

// ---- device status ----

int iree_uk_b200_device_status(void* cu_stream, uint32_t* detail) {
  uint32_t* word = device_status_word();
  if (!word) return IREE_UK_B200_CUDA_ERROR;
  cudaStream_t stream = static_cast<cudaStream_t>(cu_stream);
  uint32_t host = 0;
  if (cudaMemcpyAsync(&host, word, sizeof host, cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
      cudaStreamSynchronize(stream) != cudaSuccess)
    return IREE_UK_B200_CUDA_ERROR;
  if (detail) *detail = host;
  if (host) {
    if (cudaMemsetAsync(word, 0, sizeof host, stream) != cudaSuccess ||
        cudaStreamSynchronize(stream) != cudaSuccess)
      return IREE_UK_B200_CUDA_ERROR;
    return IREE_UK_B200_DEVICE_TIMEOUT;
  }
  return IREE_UK_B200_OK;
}

// ---- kernel timing (benchmarks) ----

int iree_uk_b200_kernel_timing(int every) {
  KernelTiming* t = kernel_timing();
  if (!t) return IREE_UK_B200_CUDA_ERROR;
  t->enabled.store(false);
  if (every > 0 && !t->ev[0][0]) {
    for (int c = 0; c < KernelTiming::kRing; ++c)
      for (int i = 0; i < 3; ++i)
        if (cudaEventCreate(&t->ev[c][i]) != cudaSuccess) {
          cudaGetLastError();
          return IREE_UK_B200_CUDA_ERROR;
        }
  }
  t->every.store(every > 1 ? every : 1);
  t->calls.store(0);
  t->seen.store(0);
  t->enabled.store(every > 0);
  return IREE_UK_B200_OK;
}

int iree_uk_b200_kernel_timing_mean_ms(float* prepass_ms, float* main_ms, int* count) {
  KernelTiming* t = kernel_timing();
  if (!t) return IREE_UK_B200_CUDA_ERROR;
  const long long calls = t->calls.load();
  if (!t->enabled.load() || calls == 0) return IREE_UK_B200_INVALID_ARGUMENT;
  const long long n = calls < KernelTiming::kRing ? calls : KernelTiming::kRing;
  double a = 0.0, b = 0.0;
  for (long long i = 0; i < n; ++i) {
    cudaEvent_t* e = t->ev[(calls - 1 - i) % KernelTiming::kRing];
    if (cudaEventSynchronize(e[2]) != cudaSuccess) return IREE_UK_B200_CUDA_ERROR;
    float x = 0.f, y = 0.f;
    if (cudaEventElapsedTime(&x, e[0], e[1]) != cudaSuccess ||
        cudaEventElapsedTime(&y, e[1], e[2]) != cudaSuccess)
      return IREE_UK_B200_CUDA_ERROR;
    a += x;
    b += y;
  }
  if (prepass_ms) *prepass_ms = float(a / n);
  if (main_ms) *main_ms = float(b / n);
  if (count) *count = int(n);
  return IREE_UK_B200_OK;
}

// ---- test hooks (include/iree_uk_b200_testing.h) ----

int iree_uk_b200_testing_starve_producers(int enable) { return g_starve.exchange(enable ? 1 : 0); }

int iree_uk_b200_testing_mmt4d_form(const iree_uk_mmt4d_params_t* params, void* workspace,
                                    size_t workspace_bytes, int form, void* cu_stream) {
  const int rc = validate_mmt4d(params);
  if (rc) return rc;
  if (form != IREE_UK_B200_TESTING_FORM_ONE_CTA && form != IREE_UK_B200_TESTING_FORM_TWO_CTA &&
      form != IREE_UK_B200_TESTING_FORM_TWO_CTA_STREAMED)
    return IREE_UK_B200_INVALID_ARGUMENT;
  if (params->M < 1 || params->N < 1 || params->K < 1) return IREE_UK_B200_UNSUPPORTED;
  if (!mmt4d_tc_eligible(params)) return IREE_UK_B200_UNSUPPORTED;
  return launch_mmt4d_tc(params, workspace, workspace_bytes, form,
                         static_cast<cudaStream_t>(cu_stream));
}

}  // extern "C"
