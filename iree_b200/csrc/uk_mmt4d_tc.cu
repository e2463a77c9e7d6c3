// mmt4d on the 5th-generation tensor cores (sm_100a), host side: tensor maps, shared-memory
// and instruction descriptors, kernel selection and launch. The data path is
//   TMA -> shared memory -> tcgen05.mma -> TMEM -> tcgen05.ld -> [M1][N1][16][16] output tiles
// for s8s8s32 (kind::i8), f16f16f32 / bf16bf16f32 and their 16-bit-output forms (kind::f16),
// f32f32f32 on request (kind::tf32, three products per term) and s16u4s32 (two kind::i8
// products per term), all with M0 = N0 = 16 (s16u4s32: 1 x 32 x 8).
//
// How the operands reach shared memory is described by runtime parameters (tensor maps, box
// coordinates, shared-memory descriptor fields), not by the kernel bodies:
//   * K-major, SWIZZLE_128B, from scratch that retile_kernel fills from the mmt4d panel layout
//     [tile][K1][16][K0] (works for every K0) - the product path when a workspace is given;
//   * MN-major, SWIZZLE_32B, read directly from a 16-bit K0 = 1 operand - no scratch, half rate;
//   * no TMA at all: mmt4d_tc_sw_kernel's producer warps re-tile into the swizzled stages;
//   * row-major matmul operands: K-major LHS in place, MN-major SWIZZLE_128B RHS in place.
//
// Every wait on an mbarrier in the kernels is bounded (clock64 deadline). A wait that runs out
// records a code in the per-device status word, raises a CTA-wide abort flag, and all roles
// leave their loops; the producer then waits (bounded) for its own copies in flight, TMEM is
// freed and the kernel returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <type_traits>

#include "uk_common.h"
#include "uk_tc_device.cuh"
#include "uk_tc_prepass.cuh"
#include "uk_tc_kernels.cuh"

namespace uk {
namespace {

// ---------------------------------------------------------------------------------------
// host side: tensor maps, descriptors, launch
// ---------------------------------------------------------------------------------------


// Wait policy of a launch: every device-side wait gives up after about a second; with the
// starve test hook set, the producers fill nothing and the limit drops to a few tens of
// milliseconds, because several waits then run out one after the other.
void set_wait_policy(TcParams* P) {
  P->starve = testing_starve_producers() ? 1 : 0;
  P->wait_cycles = P->starve ? (1ll << 26) : kWaitCycles;
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

struct TypeInfo {
  int es;         // operand element bytes
  bool is_int;
  uint32_t fmt;   // a/b format field of the instruction descriptor
  uint32_t cfmt;  // accumulator format
  CUtensorMapDataType tm_type;
  int out_es;     // output element bytes: 4, or 2 for the f16 / bf16 output triples
  bool triple = false;  // f32 x f32: split into tf32 hi/lo planes, three products per K slice
};

bool tc_type_info(uint32_t flags, TypeInfo* ti) {
  // The 16-bit-output triples accumulate in f32 on the tensor cores and round once at the end,
  // which is what the reference computes only under SKIP_INTERMEDIATE_ROUNDINGS
  // (mmt4d_tile_generic.c:395-404); without that flag they stay on the generic kernel.
  const bool skip = (flags & IREE_UK_FLAG_MMT4D_SKIP_INTERMEDIATE_ROUNDINGS) != 0;
  switch (flags & IREE_UK_FLAG_MMT4D_TYPE_MASK) {
    case IREE_UK_FLAG_MMT4D_TYPE_S8S8S32: *ti = {1, true, 1u, 2u, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4}; return true;
    case IREE_UK_FLAG_MMT4D_TYPE_F16F16F32: *ti = {2, false, 0u, 1u, CU_TENSOR_MAP_DATA_TYPE_UINT16, 4}; return true;
    case IREE_UK_FLAG_MMT4D_TYPE_BF16BF16F32: *ti = {2, false, 1u, 1u, CU_TENSOR_MAP_DATA_TYPE_UINT16, 4}; return true;
    case IREE_UK_FLAG_MMT4D_TYPE_F32F32F32: *ti = {4, false, 2u, 1u, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, true}; return f32_mode() == IREE_UK_B200_F32_MODE_TF32X3;
    case IREE_UK_FLAG_MMT4D_TYPE_F16F16F16: *ti = {2, false, 0u, 1u, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2}; return skip;
    case IREE_UK_FLAG_MMT4D_TYPE_BF16BF16BF16: *ti = {2, false, 1u, 1u, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2}; return skip;
    default: return false;
  }
}

uint32_t make_idesc(const TypeInfo& ti, int n, bool mn_major, int m = BM) {
  return (ti.cfmt << 4) | (ti.fmt << 7) | (ti.fmt << 10) | (uint32_t(mn_major) << 15) |
         (uint32_t(mn_major) << 16) | (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}

// The two-CTA kernel's instantiations: [is_int][form], form 0 = everything re-tiled by the
// pre-pass kernel, 1 / 2 = streamed pre-pass (the kernel's own workers finish the re-tile) for
// 2- / 4-byte granules.
using PairKernel = void (*)(const TcParams);
constexpr int kPairForms = 3;
int streamed_form_of_granule(int G) { return G == 2 ? 1 : (G == 4 ? 2 : 0); }
PairKernel pair_kernel(bool is_int, int form) {
  static const PairKernel table[2][kPairForms] = {
      {mmt4d_tc2_kernel<false, 0>, mmt4d_tc2_kernel<false, 2>, mmt4d_tc2_kernel<false, 4>},
      {mmt4d_tc2_kernel<true, 0>, mmt4d_tc2_kernel<true, 2>, mmt4d_tc2_kernel<true, 4>}};
  return table[is_int ? 1 : 0][form];
}
int pair_threads(int form) { return form ? kStreamedThreads : kThreads; }

// Co-resident 2-CTA clusters of a pair kernel on the current device (0 on failure).
int max_pair_clusters(PairKernel kernel, int threads, size_t smem) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2, 1, 1);
  cfg.blockDim = dim3(unsigned(threads), 1, 1);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) return 0;
  return n;
}

// What the launchers need to know about the current device, found once per device: the
// kernels' dynamic shared memory limit is raised to the device maximum at that point, so the
// per-call path makes no attribute or occupancy calls.
struct DeviceInfo {
  bool ok = false;
  int sms = 0;
  int max_smem = 0;           // dynamic shared memory per block the kernels may be launched with
  int pair_clusters[2][kPairForms] = {};  // co-resident CTA pairs of mmt4d_tc2_kernel [is_int][form]
};

const DeviceInfo* device_info() {
  constexpr int kMaxDevices = 64;
  static DeviceInfo info[kMaxDevices];
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  DeviceInfo& d = info[dev];
  if (!d.ok) {
    if (cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&d.max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess)
      return nullptr;
    // dynamic limit of each kernel = the device's opt-in maximum minus its static shared memory
    int dyn_limit = d.max_smem;
    auto raise_limit = [&](const void* fn) {
      cudaFuncAttributes fa;
      if (cudaFuncGetAttributes(&fa, fn) != cudaSuccess) return false;
      const int dyn = d.max_smem - int(fa.sharedSizeBytes);
      dyn_limit = std::min(dyn_limit, dyn);
      return cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, dyn) == cudaSuccess;
    };
    bool raised = raise_limit(reinterpret_cast<const void*>(mmt4d_tc_kernel<false>)) &&
                  raise_limit(reinterpret_cast<const void*>(mmt4d_tc_kernel<true>));
    for (int i = 0; i < 2 && raised; ++i)
      for (int f = 0; f < kPairForms && raised; ++f)
        raised = raise_limit(reinterpret_cast<const void*>(pair_kernel(i != 0, f)));
    if (!raised) {
      cudaGetLastError();
      return nullptr;
    }
    d.max_smem = dyn_limit;
    const size_t smem_probe = size_t(6) * (BM * 128 + 128 * 128) + 1024;
    for (int i = 0; i < 2; ++i)
      for (int f = 0; f < kPairForms; ++f)
        d.pair_clusters[i][f] = max_pair_clusters(pair_kernel(i != 0, f), pair_threads(f), smem_probe);
    d.ok = true;
  }
  return &d;
}

// Cost of the last, partial round of `rem` tiles of width bn over `clusters` CTA pairs (in the
// unit of pick_bn_pair: columns, plus 96 per tile) and the split that gives it: the tiles stay
// whole or are cut along N into 2 or 4 narrow ones when that shortens the round.
int64_t tail_round_cost(int rem, int bn, int clusters, bool may_split, int* split_out) {
  int best = 1;
  int64_t best_cost = rem > 0 ? int64_t(bn + 96) : 0;
  if (rem > 0 && may_split) {
    for (int split : {2, 4}) {
      if ((bn / split) % 16 != 0 || bn % split != 0) continue;
      const int64_t rounds = (int64_t(rem) * split + clusters - 1) / clusters;
      const int64_t cost = rounds * (bn / split + 96);
      if (cost < best_cost) { best_cost = cost; best = split; }
    }
  }
  if (split_out) *split_out = best;
  return best_cost;
}

// Accumulator width for the pair kernel: among the multiples of 32 columns up to 256, the one
// that minimises the estimated time = full rounds of 256 x bn tiles over `clusters` pairs, each
// bn columns plus a fixed part, plus the last partial round (narrow tail tiles counted when the
// kernel can cut them).
int pick_bn_pair(int64_t M1, int64_t N1, int clusters, bool may_split) {
  {
    const int bn = debug_int("IREE_UK_B200_DEBUG_PAIR_BN", 0);
    if (bn >= 32 && bn <= 256 && bn % 32 == 0) return bn;
  }
  const int64_t m_tiles = (M1 * 16 + 255) / 256, cols = N1 * 16;
  int best = 256;
  int64_t best_cost = -1;
  for (int bn = 256; bn >= 128; bn -= 32) {
    const int64_t tiles = m_tiles * ((cols + bn - 1) / bn);
    // tile time: the MMAs plus a fixed part (96 columns' worth: with 32 the 4096^3 problem chose
    // 192 columns and five waves, which measured 4 % slower than 256 columns and four waves)
    const int64_t full = tiles / clusters;
    const int rem = int(tiles % clusters);
    const int64_t cost = full * (bn + 96) + tail_round_cost(rem, bn, clusters, may_split && tiles > clusters, nullptr);
    // a narrower tile has to win by more than 2 %: 256-column MMAs are the most efficient (the
    // 8-way shard of the headline problem: estimate 2240 for 224 columns against 2272 for 256,
    // measured 0.3964 against 0.3931 ms)
    if (best_cost < 0 || cost * 100 < best_cost * 98) { best_cost = cost; best = bn; }
  }
  return best;
}

// Upper word of a shared-memory matrix descriptor: stride byte offset, version 1
// (Blackwell), swizzle mode (2 = 128 B, 4 = 64 B, 6 = 32 B, 0 = none).
uint32_t desc_hi(uint32_t sbo_bytes, uint32_t layout) {
  return ((sbo_bytes >> 4) & 0x3FFFu) | (1u << 14) | (layout << 29);
}

int64_t round_up(int64_t v, int64_t q) { return (v + q - 1) / q * q; }

int pick_bn(int64_t M1, int64_t N1) {
  {
    const int bn = debug_int("IREE_UK_B200_DEBUG_BN", 0);
    if (bn >= 16 && bn <= 256 && bn % 16 == 0) return bn;
  }
  const int64_t m_tiles = (M1 + 7) / 8;
  for (int bn : {256, 128, 64}) {
    const int64_t n_tiles = (N1 * 16 + bn - 1) / bn;
    if (m_tiles * n_tiles >= 148 || bn == 64) {
      // never wider than the problem (rounded up to 16 columns)
      const int64_t cap = round_up(N1 * 16, 16);
      return int(std::min<int64_t>(bn, std::max<int64_t>(cap, 16)));
    }
  }
  return 64;
}

bool encode_map(CUtensorMap* map, CUtensorMapDataType type, void* base, const uint64_t dims[3],
                const uint64_t strides_b[2], const uint32_t box[3], CUtensorMapSwizzle swz) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  cuuint64_t gd[3] = {dims[0], dims[1], dims[2]};
  cuuint64_t gs[2] = {strides_b[0], strides_b[1]};
  cuuint32_t bx[3] = {box[0], box[1], box[2]};
  cuuint32_t es[3] = {1, 1, 1};
  return fn(map, type, 3, base, gd, gs, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

// ---- s16u4s32 (M0 = 1, N0 = 32, K0 = 8) on the tensor cores ----------------------------------

bool mmt4d_tc_s16u4_eligible(const iree_uk_mmt4d_params_t* p) {
  if ((p->flags & IREE_UK_FLAG_MMT4D_TYPE_MASK) != IREE_UK_FLAG_MMT4D_TYPE_S16U4S32) return false;
  if (p->M0 != 1 || p->N0 != 32 || p->K0 != 8 || p->K < 1 || p->M < 1 || p->N < 1) return false;
  const uintptr_t lhs = reinterpret_cast<uintptr_t>(p->lhs_buffer) + uintptr_t(p->lhs_offset * 2);
  const uintptr_t rhs = reinterpret_cast<uintptr_t>(p->rhs_buffer) + uintptr_t(p->rhs_offset / 2);
  const uintptr_t out = reinterpret_cast<uintptr_t>(p->out_buffer) + uintptr_t(p->out_offset * 4);
  if ((lhs | rhs | out) & 15) return false;
  if ((p->lhs_stride0 * 2) % 16 || (p->rhs_stride0 / 2) % 16 || (p->out_stride0 * 4) % 16) return false;
  if ((p->M + 127) / 128 * ((p->N + 0) / 1 + 1) > 0x3FFFFFFF) return false;
  return true;
}

bool mmt4d_tc_s16s16_eligible(const iree_uk_mmt4d_params_t* p) {
  if ((p->flags & IREE_UK_FLAG_MMT4D_TYPE_MASK) != IREE_UK_FLAG_MMT4D_TYPE_S16S16S32) return false;
  if (p->M0 != 16 || p->N0 != 16 || p->K0 != 2 || p->K < 1 || p->M < 1 || p->N < 1) return false;
  const uintptr_t lhs = reinterpret_cast<uintptr_t>(p->lhs_buffer) + uintptr_t(p->lhs_offset * 2);
  const uintptr_t rhs = reinterpret_cast<uintptr_t>(p->rhs_buffer) + uintptr_t(p->rhs_offset * 2);
  const uintptr_t out = reinterpret_cast<uintptr_t>(p->out_buffer) + uintptr_t(p->out_offset * 4);
  if ((lhs | rhs | out) & 15) return false;
  if ((p->lhs_stride0 * 2) % 16 || (p->rhs_stride0 * 2) % 16 || (p->out_stride0 * 4) % 16) return false;
  if ((p->M + 7) / 8 * ((p->N + 3) / 4) > 0x3FFFFFFF) return false;
  return true;
}

bool mmt4d_tc_s16s8_eligible(const iree_uk_mmt4d_params_t* p) {
  if ((p->flags & IREE_UK_FLAG_MMT4D_TYPE_MASK) != IREE_UK_FLAG_MMT4D_TYPE_S16S8S32) return false;
  if (p->M0 != 16 || p->N0 != 16 || p->K0 != 2 || p->K < 1 || p->M < 1 || p->N < 1) return false;
  const uintptr_t lhs = reinterpret_cast<uintptr_t>(p->lhs_buffer) + uintptr_t(p->lhs_offset * 2);
  const uintptr_t rhs = reinterpret_cast<uintptr_t>(p->rhs_buffer) + uintptr_t(p->rhs_offset);
  const uintptr_t out = reinterpret_cast<uintptr_t>(p->out_buffer) + uintptr_t(p->out_offset * 4);
  if ((lhs | rhs | out) & 15) return false;
  if ((p->lhs_stride0 * 2) % 16 || p->rhs_stride0 % 16 || (p->out_stride0 * 4) % 16) return false;
  if ((p->M + 7) / 8 * ((p->N + 3) / 4) > 0x3FFFFFFF) return false;
  return true;
}

bool mmt4d_tc_s8s4_eligible(const iree_uk_mmt4d_params_t* p) {
  if ((p->flags & IREE_UK_FLAG_MMT4D_TYPE_MASK) != IREE_UK_FLAG_MMT4D_TYPE_S8S4S32) return false;
  if (p->M0 != 16 || p->N0 != 16 || p->K < 1 || p->M < 1 || p->N < 1) return false;
  if (p->K0 != 2 && p->K0 != 4 && p->K0 != 8 && p->K0 != 16) return false;
  if (p->rhs_offset & 1) return false;  // the RHS starts on a byte
  const uintptr_t lhs = reinterpret_cast<uintptr_t>(p->lhs_buffer) + uintptr_t(p->lhs_offset);
  const uintptr_t rhs = reinterpret_cast<uintptr_t>(p->rhs_buffer) + uintptr_t(p->rhs_offset / 2);
  const uintptr_t out = reinterpret_cast<uintptr_t>(p->out_buffer) + uintptr_t(p->out_offset * 4);
  if ((lhs | rhs | out) & 15) return false;
  if (p->lhs_stride0 % 16 || (p->rhs_stride0 & 1) || (p->rhs_stride0 / 2) % 16 || (p->out_stride0 * 4) % 16)
    return false;
  if ((p->M + 7) / 8 * ((p->N + 3) / 4) > 0x3FFFFFFF) return false;
  return true;
}

namespace {

struct S16U4Layout {
  int64_t pitch, plane_bytes, w_bytes;
};
S16U4Layout s16u4_layout(const iree_uk_mmt4d_params_t* p) {
  S16U4Layout l;
  l.pitch = round_up(p->K * 8, 128);
  l.plane_bytes = round_up(p->M * l.pitch, 1024);
  l.w_bytes = round_up(p->N * 32 * l.pitch, 1024);
  return l;
}

// f32 -> tf32 planes, in place: hi is x rounded to sign, exponent and 10 mantissa bits (what
// kind::tf32 reads), lo = x - hi (exact in f32) goes to the second plane.
__global__ void __launch_bounds__(256) split_tf32_kernel(uint4* __restrict__ hi, uint4* __restrict__ lo,
                                                         int64_t vecs) {
  pdl_launch_dependents();
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < vecs;
       i += int64_t(gridDim.x) * blockDim.x) {
    const uint4 x = hi[i];
    const uint32_t v[4] = {x.x, x.y, x.z, x.w};
    uint32_t h[4], l[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      // round to nearest tf32 (truncate instead where rounding up would overflow to infinity)
      const bool top = (v[j] & 0x7F800000u) == 0x7F000000u;
      h[j] = (top ? v[j] : v[j] + 0x1000u) & 0xFFFFE000u;
      const float d = __uint_as_float(v[j]) - __uint_as_float(h[j]);
      // inf - inf and nan - nan must not poison the sum twice: the hi plane carries them
      l[j] = ((v[j] & 0x7F800000u) == 0x7F800000u) ? 0u : __float_as_uint(d);
    }
    hi[i] = make_uint4(h[0], h[1], h[2], h[3]);
    lo[i] = make_uint4(l[0], l[1], l[2], l[3]);
  }
}

// Launches a main kernel (one-CTA form when cluster == 1, CTA pairs when cluster == 2) with
// programmatic stream serialisation, so that it may overlap the tail of the pre-pass kernel
// enqueued just before it (see pdl_wait).
template <typename Kernel>
cudaError_t launch_main(Kernel kernel, int grid, int cluster, size_t smem, cudaStream_t stream,
                        const TcParams& P, int threads = kThreads) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned(grid), 1, 1);
  cfg.blockDim = dim3(unsigned(threads), 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  int n = 0;
  attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attrs[n].val.programmaticStreamSerializationAllowed = 1;
  ++n;
  if (cluster > 1) {
    attrs[n].id = cudaLaunchAttributeClusterDimension;
    attrs[n].val.clusterDim.x = unsigned(cluster);
    attrs[n].val.clusterDim.y = 1;
    attrs[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = unsigned(n);
  return cudaLaunchKernelEx(&cfg, kernel, P);
}

// `prepared` (optional): the weights already widened to bytes by launch_mmt4d_tc_prepare_rhs and
// kept by the caller; the scratch then holds the two LHS byte planes only.
int launch_mmt4d_tc_s16u4(const iree_uk_mmt4d_params_t* p, void* ws, size_t ws_bytes,
                          cudaStream_t stream, const void* prepared = nullptr) {
  if (!mmt4d_tc_s16u4_eligible(p)) return IREE_UK_B200_UNSUPPORTED;
  uint32_t* status = device_status_word();
  if (!status) return IREE_UK_B200_CUDA_ERROR;
  const S16U4Layout l = s16u4_layout(p);
  if (!ws || ws_bytes < size_t(2 * l.plane_bytes + (prepared ? 0 : l.w_bytes))) return IREE_UK_B200_WORKSPACE_TOO_SMALL;
  if ((reinterpret_cast<uintptr_t>(ws) | reinterpret_cast<uintptr_t>(prepared)) & 255) return IREE_UK_B200_INVALID_ARGUMENT;
  KernelTiming* timing = kernel_timing();
  cudaEvent_t* tev = timing ? timing->next_slot() : nullptr;
  if (tev) KernelTiming::record(tev[0], stream);

  const char* lhs = static_cast<const char*>(p->lhs_buffer) + p->lhs_offset * 2;
  const char* rhs = static_cast<const char*>(p->rhs_buffer) + p->rhs_offset / 2;
  char* hi = static_cast<char*>(ws);
  char* lo = hi + l.plane_bytes;
  char* w8 = prepared ? const_cast<char*>(static_cast<const char*>(prepared)) : lo + l.plane_bytes;
  {
    const int64_t total = p->M * p->K;
    const int64_t blocks = std::min<int64_t>((total + 255) / 256, 148 * 16);
    split_s16_kernel<<<int(blocks), 256, 0, stream>>>(lhs, p->lhs_stride0 * 2, hi, lo, l.pitch, p->M, p->K);
    if (!prepared) {
      const int64_t kchunks = (p->K + 63) / 64;
      if (p->N * kchunks > 0x7FFFFFFF) return IREE_UK_B200_UNSUPPORTED;
      unpack_u4_kernel<<<int(p->N * kchunks), 256, 0, stream>>>(rhs, p->rhs_stride0 / 2, w8, l.pitch,
                                                              p->K, int(kchunks));
    }
    if (cudaGetLastError() != cudaSuccess) return IREE_UK_B200_CUDA_ERROR;
  }

  TcParams P;
  std::memset(&P, 0, sizeof P);
  const int64_t kbytes = p->K * 8, ncols = p->N * 32;
  // (256 columns with one accumulator buffer measured slower here: 0.712 against 0.693 ms)
  const int bn = int(std::min<int64_t>(128, ncols));
  const uint64_t da[3] = {uint64_t(kbytes), uint64_t(p->M), 2};
  const uint64_t db[3] = {uint64_t(kbytes), uint64_t(ncols), 1};
  const uint64_t sa[2] = {uint64_t(l.pitch), uint64_t(l.plane_bytes)};
  const uint64_t sb[2] = {uint64_t(l.pitch), uint64_t(l.pitch) * uint64_t(ncols)};
  // The two-CTA form (256 rows x 128 columns per CTA pair, two accumulators of 128 columns, double
  // buffered = all 512 TMEM columns) once every pair has a tile; the one-CTA form otherwise.
  const DeviceInfo* di = device_info();
  if (!di) return IREE_UK_B200_CUDA_ERROR;
  const int pair_clusters = di->pair_clusters[1][0];
  const bool pair = bn == 128 && p->M >= 256 && pair_clusters >= 1 &&
                    ((p->M + 255) / 256) * ((ncols + 127) / 128) >= 74 &&
                    !debug_int("IREE_UK_B200_DEBUG_S16U4_ONE_CTA", 0);
  const int tile_m = pair ? 2 * BM : BM;
  const int b_rows = pair ? bn / 2 : bn;
  const uint32_t ba[3] = {128, BM, 1};
  const uint32_t bb[3] = {128, uint32_t(b_rows), 1};
  if (!encode_map(&P.map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, hi, da, sa, ba, CU_TENSOR_MAP_SWIZZLE_128B) ||
      !encode_map(&P.map_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, w8, db, sb, bb, CU_TENSOR_MAP_SWIZZLE_128B))
    return IREE_UK_B200_CUDA_ERROR;
  // box 0: high plane, box 1: low plane
  P.sa = {2, BM * 128, {128, 0, 0}, {0, tile_m, 0}, {0, 0, 1}, {0, pair ? BM : 0, 0}};
  P.sb = {1, b_rows * 128, {128, 0, 0}, {0, bn, 0}, {0, 0, 0}, {0, pair ? b_rows : 0, 0}};
  P.desc_hi_a = P.desc_hi_b = desc_hi(1024, 2);
  P.desc_lbo_a = P.desc_lbo_b = 1;
  P.kadv_a = P.kadv_b = 2;
  P.kbox_units_a = uint32_t(BM * 128) >> 4;  // distance from the high to the low plane tile
  P.kbox_units_b = 0;
  // accumulate s32; LHS high bytes signed, low bytes unsigned; weights unsigned
  const uint32_t common = (2u << 4) | (uint32_t(bn >> 3) << 17) | (uint32_t(tile_m >> 4) << 24);
  P.idesc = common | (1u << 7);
  P.idesc2 = common;
  P.dual = 1;
  P.acc_bufs = 2 * 2 * bn <= 512 ? 2 : 1;
  P.kboxes = 1;
  P.mma_per_box = 4;
  P.stage_bytes_a = 2 * BM * 128;
  P.stage_bytes_b = b_rows * 128;
  P.num_kb = int((kbytes + 127) / 128);
  P.bn = bn;
  P.m_tiles = int((p->M + tile_m - 1) / tile_m);
  P.n_tiles = int((ncols + bn - 1) / bn);
  P.num_work = P.tail_first = P.m_tiles * P.n_tiles;
  P.tail_split = 1;
  P.group_m = std::min(P.m_tiles, pair ? 8 : 16);
  P.out = static_cast<char*>(p->out_buffer) + p->out_offset * 4;
  P.out_stride0 = p->out_stride0;
  P.M1 = p->M;
  P.N1 = p->N;
  P.accumulate = (p->flags & IREE_UK_FLAG_MMT4D_ACCUMULATE) ? 1 : 0;
  P.out_is_int = 1;
  P.status = status;
  set_wait_policy(&P);
  const int stage_bytes = P.stage_bytes_a + P.stage_bytes_b;
  P.num_stages = std::max(2, std::min(kMaxStages, 200 * 1024 / stage_bytes));
  const size_t smem = size_t(P.num_stages) * stage_bytes + 1024;
  if (smem > size_t(di->max_smem)) return IREE_UK_B200_CUDA_ERROR;
  if (tev) KernelTiming::record(tev[1], stream);
  cudaError_t e;
  if (pair) {
    const int grid = 2 * std::min(P.m_tiles * P.n_tiles, pair_clusters);
    e = launch_main(pair_kernel(true, 0), grid, 2, smem, stream, P);
  } else {
    const int grid = std::min(P.m_tiles * P.n_tiles, di->sms);
    e = launch_main(mmt4d_tc_kernel<true>, grid, 1, smem, stream, P);
  }
  if (e != cudaSuccess) return IREE_UK_B200_CUDA_ERROR;
  if (tev) {
    KernelTiming::record(tev[2], stream);
    timing->calls.fetch_add(1, std::memory_order_relaxed);
  }
  return cuda_status(cudaGetLastError());
}

// ---- s16s16s32 (M0 = N0 = 16, K0 = 2) on the tensor cores -----------------------------------
// x = 256 * hi + lo with hi the signed high byte and lo the unsigned low byte of an s16, so
// sum(a * b) = 65536 * sum(ha * hb) + 256 * (sum(ha * lb) + sum(la * hb)) + sum(la * lb): four
// 8-bit tensor-core products per term into three s32 accumulators, recombined modulo 2^32 by the
// epilogue - which is the reference's own wrapping int32 arithmetic (mmt4d_tile_generic.c).
struct S16S16Layout {
  int64_t pitch, plane_a, plane_b;
};
S16S16Layout s16s16_layout(const iree_uk_mmt4d_params_t* p) {
  S16S16Layout l;
  l.pitch = round_up(p->K * 2, 128);
  l.plane_a = round_up(p->M * 16 * l.pitch, 1024);
  l.plane_b = round_up(p->N * 16 * l.pitch, 1024);
  return l;
}

// Also serves s16s8s32 16x16x2 (`rhs_s8`): the RHS is then a single plane of signed bytes, every
// term takes two products (high x b, low x b) into two accumulators, double buffered.
int launch_mmt4d_tc_s16s16(const iree_uk_mmt4d_params_t* p, void* ws, size_t ws_bytes,
                           cudaStream_t stream) {
  const bool rhs_s8 = (p->flags & IREE_UK_FLAG_MMT4D_TYPE_MASK) == IREE_UK_FLAG_MMT4D_TYPE_S16S8S32;
  if (!(rhs_s8 ? mmt4d_tc_s16s8_eligible(p) : mmt4d_tc_s16s16_eligible(p))) return IREE_UK_B200_UNSUPPORTED;
  uint32_t* status = device_status_word();
  if (!status) return IREE_UK_B200_CUDA_ERROR;
  const S16S16Layout l = s16s16_layout(p);
  const int b_planes = rhs_s8 ? 1 : 2;
  if (!ws || ws_bytes < size_t(2 * l.plane_a + b_planes * l.plane_b)) return IREE_UK_B200_WORKSPACE_TOO_SMALL;
  if (reinterpret_cast<uintptr_t>(ws) & 255) return IREE_UK_B200_INVALID_ARGUMENT;
  const DeviceInfo* di = device_info();
  if (!di) return IREE_UK_B200_CUDA_ERROR;
  KernelTiming* timing = kernel_timing();
  cudaEvent_t* tev = timing ? timing->next_slot() : nullptr;
  if (tev) KernelTiming::record(tev[0], stream);

  char* a_hi = static_cast<char*>(ws);
  char* b_hi = a_hi + 2 * l.plane_a;
  {
    const int64_t kchunks = (p->K + 255) / 256;
    const SplitOperand a = {static_cast<const char*>(p->lhs_buffer) + p->lhs_offset * 2,
                            p->lhs_stride0 * 2, a_hi, l.plane_a, p->M * kchunks};
    const SplitOperand b = {static_cast<const char*>(p->rhs_buffer) + p->rhs_offset * 2,
                            p->rhs_stride0 * 2, b_hi, l.plane_b, rhs_s8 ? 0 : p->N * kchunks};
    if (a.blocks + b.blocks > 0x7FFFFFFF) return IREE_UK_B200_UNSUPPORTED;
    retile_split_s16_kernel<<<int(a.blocks + b.blocks), 256, 0, stream>>>(a, b, l.pitch, p->K,
                                                                        int(kchunks));
    if (cudaGetLastError() != cudaSuccess) return IREE_UK_B200_CUDA_ERROR;
    if (rhs_s8) {  // the s8 RHS [N1][K1][16][2]: a plain re-tile with 2-byte granules
      const int rc = launch_retile(nullptr, 0, nullptr, 0,
                                   static_cast<const char*>(p->rhs_buffer) + p->rhs_offset,
                                   p->rhs_stride0, b_hi, p->N, l.pitch, p->K, 2, stream);
      if (rc) return rc;
    }
  }

  TcParams P;
  std::memset(&P, 0, sizeof P);
  const int64_t kbytes = p->K * 2, rows = p->M * 16, ncols = p->N * 16;
  // Accumulator width. 128 columns by default: two accumulators then fit TMEM twice (the
  // epilogue overlaps the next tile), three only once. Problems that fill the CTA pairs with
  // wider tiles take them, with ONE accumulator buffer: 256 columns in the two-product mode
  // (measured 0.719 against 0.765 ms at 8192 x 14336 x 4096: wider MMAs re-read the LHS planes
  // from shared memory half as often, which outweighs the lost overlap), 160 in the four-product
  // mode (3 x 160 = 480 of the 512 columns; 1.230 against 1.259 ms).
  int bn = int(std::min<int64_t>(128, round_up(ncols, 16)));
  {
    const int wide = rhs_s8 ? 256 : 160;
    if (rows >= 256 && ((rows + 255) / 256) * ((ncols + wide - 1) / wide) >= 74) bn = wide;
  }
  const int pair_clusters = di->pair_clusters[1][0];
  const bool pair = bn >= 128 && rows >= 256 && pair_clusters >= 1 &&
                    ((rows + 255) / 256) * ((ncols + 127) / 128) >= 74;
  const int tile_m = pair ? 2 * BM : BM;
  const int b_rows = pair ? bn / 2 : bn;
  const uint64_t da[3] = {uint64_t(kbytes), uint64_t(rows), 2};
  const uint64_t db[3] = {uint64_t(kbytes), uint64_t(ncols), uint64_t(b_planes)};
  const uint64_t sa[2] = {uint64_t(l.pitch), uint64_t(l.plane_a)};
  const uint64_t sb[2] = {uint64_t(l.pitch), uint64_t(l.plane_b)};
  const uint32_t ba[3] = {128, BM, 1};
  const uint32_t bb[3] = {128, uint32_t(b_rows), 1};
  if (!encode_map(&P.map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, a_hi, da, sa, ba, CU_TENSOR_MAP_SWIZZLE_128B) ||
      !encode_map(&P.map_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, b_hi, db, sb, bb, CU_TENSOR_MAP_SWIZZLE_128B))
    return IREE_UK_B200_CUDA_ERROR;
  // box 0: high plane, box 1: low plane
  P.sa = {2, BM * 128, {128, 0, 0}, {0, tile_m, 0}, {0, 0, 1}, {0, pair ? BM : 0, 0}};
  P.sb = {b_planes, b_rows * 128, {128, 0, 0}, {0, bn, 0}, {0, 0, 1}, {0, pair ? b_rows : 0, 0}};
  P.desc_hi_a = P.desc_hi_b = desc_hi(1024, 2);
  P.desc_lbo_a = P.desc_lbo_b = 1;
  P.kadv_a = P.kadv_b = 2;
  P.kbox_units_a = uint32_t(BM * 128) >> 4;      // from the high to the low plane tile
  P.kbox_units_b = rhs_s8 ? 0u : uint32_t(b_rows * 128) >> 4;
  // accumulate s32; in the four-product mode the operands' sign bits are set per product by the
  // issuing thread, in the two-product mode the RHS is signed and the LHS planes differ
  const uint32_t common = (2u << 4) | (uint32_t(bn >> 3) << 17) | (uint32_t(tile_m >> 4) << 24);
  if (rhs_s8) {
    P.idesc = common | (1u << 7) | (1u << 10);
    P.idesc2 = common | (1u << 10);
    P.dual = 2;
    P.acc_bufs = 2 * 2 * bn <= 512 ? 2 : 1;
  } else {
    P.idesc = common;
    P.quad = 1;
    P.acc_bufs = 2 * 3 * bn <= 512 ? 2 : 1;
  }
  P.kboxes = 1;
  P.mma_per_box = 4;
  P.stage_bytes_a = 2 * BM * 128;
  P.stage_bytes_b = b_planes * b_rows * 128;
  P.num_kb = int((kbytes + 127) / 128);
  P.bn = bn;
  P.m_tiles = int((rows + tile_m - 1) / tile_m);
  P.n_tiles = int((ncols + bn - 1) / bn);
  P.num_work = P.tail_first = P.m_tiles * P.n_tiles;
  P.tail_split = 1;
  P.group_m = std::min(P.m_tiles, pair ? 8 : 16);
  P.out = static_cast<char*>(p->out_buffer) + p->out_offset * 4;
  P.out_stride0 = p->out_stride0;
  P.M1 = p->M;
  P.N1 = p->N;
  P.accumulate = (p->flags & IREE_UK_FLAG_MMT4D_ACCUMULATE) ? 1 : 0;
  P.out_is_int = 1;
  P.status = status;
  set_wait_policy(&P);
  const int stage_bytes = P.stage_bytes_a + P.stage_bytes_b;
  P.num_stages = std::max(2, std::min(kMaxStages, 200 * 1024 / stage_bytes));
  const size_t smem = size_t(P.num_stages) * stage_bytes + 1024;
  if (smem > size_t(di->max_smem)) return IREE_UK_B200_CUDA_ERROR;
  if (tev) KernelTiming::record(tev[1], stream);
  cudaError_t e;
  if (pair) {
    const int grid = 2 * std::min(P.m_tiles * P.n_tiles, pair_clusters);
    e = launch_main(pair_kernel(true, 0), grid, 2, smem, stream, P);
  } else {
    const int grid = std::min(P.m_tiles * P.n_tiles, di->sms);
    e = launch_main(mmt4d_tc_kernel<true>, grid, 1, smem, stream, P);
  }
  if (e != cudaSuccess) return IREE_UK_B200_CUDA_ERROR;
  if (tev) {
    KernelTiming::record(tev[2], stream);
    timing->calls.fetch_add(1, std::memory_order_relaxed);
  }
  return cuda_status(cudaGetLastError());
}

}  // namespace

// Operand side of the tensor-core path's conditions: a tensor-core triple, 16x16 tiles, a K0
// whose granule the re-tile handles, 16-byte aligned operand panels.
bool mmt4d_tc_operands_eligible(const iree_uk_mmt4d_params_t* p) {
  TypeInfo ti;
  if (!tc_type_info(p->flags, &ti)) return false;
  if (p->M0 != 16 || p->N0 != 16 || p->K0 < 1 || p->K < 1 || p->M < 1 || p->N < 1) return false;
  const int G = p->K0 * ti.es;
  if (G != 1 && G != 2 && G != 4 && G != 8 && G != 16) return false;
  const uintptr_t lhs = reinterpret_cast<uintptr_t>(p->lhs_buffer) + uintptr_t(p->lhs_offset * ti.es);
  const uintptr_t rhs = reinterpret_cast<uintptr_t>(p->rhs_buffer) + uintptr_t(p->rhs_offset * ti.es);
  if ((lhs | rhs) & 15) return false;
  if ((p->lhs_stride0 * ti.es) % 16 || (p->rhs_stride0 * ti.es) % 16) return false;
  if ((p->M + 7) / 8 * ((p->N + 3) / 4) > 0x3FFFFFFF) return false;
  return true;
}

bool mmt4d_tc_eligible(const iree_uk_mmt4d_params_t* p) {
  TypeInfo ti;
  if (!mmt4d_tc_operands_eligible(p) || !tc_type_info(p->flags, &ti)) return false;
  // tiled output: every 16-value tile row is accessed with 16-byte vectors
  const uintptr_t out = reinterpret_cast<uintptr_t>(p->out_buffer) + uintptr_t(p->out_offset * ti.out_es);
  return (out & 15) == 0 && (p->out_stride0 * ti.out_es) % 16 == 0;
}

bool mmt4d_tc_direct_eligible(const iree_uk_mmt4d_params_t* p) {
  TypeInfo ti;
  return tc_type_info(p->flags, &ti) && ti.es == 2 && p->K0 == 1 && mmt4d_tc_eligible(p);
}

namespace {
// Job cursor + one ready counter per LHS tile row (streamed LHS pre-pass).
size_t sync_block_bytes(const iree_uk_mmt4d_params_t* p) {
  return size_t((4 * (1 + p->M) + 1023) / 1024 * 1024);
}
}  // namespace

size_t mmt4d_tc_workspace_size(const iree_uk_mmt4d_params_t* p) {
  if ((p->flags & IREE_UK_FLAG_MMT4D_TYPE_MASK) == IREE_UK_FLAG_MMT4D_TYPE_S16U4S32) {
    if (p->M0 != 1 || p->N0 != 32 || p->K0 != 8 || p->K < 1 || p->M < 1 || p->N < 1) return 0;
    const S16U4Layout l = s16u4_layout(p);
    return size_t(2 * l.plane_bytes + l.w_bytes);
  }
  if ((p->flags & IREE_UK_FLAG_MMT4D_TYPE_MASK) == IREE_UK_FLAG_MMT4D_TYPE_S16S16S32 ||
      (p->flags & IREE_UK_FLAG_MMT4D_TYPE_MASK) == IREE_UK_FLAG_MMT4D_TYPE_S16S8S32) {
    if (p->M0 != 16 || p->N0 != 16 || p->K0 != 2 || p->K < 1 || p->M < 1 || p->N < 1) return 0;
    const S16S16Layout l = s16s16_layout(p);
    const bool rhs_s8 = (p->flags & IREE_UK_FLAG_MMT4D_TYPE_MASK) == IREE_UK_FLAG_MMT4D_TYPE_S16S8S32;
    return size_t(2 * l.plane_a + (rhs_s8 ? 1 : 2) * l.plane_b);
  }
  if ((p->flags & IREE_UK_FLAG_MMT4D_TYPE_MASK) == IREE_UK_FLAG_MMT4D_TYPE_S8S4S32) {
    // sized like the s8s8s32 problem of the same shape: the RHS is widened to bytes
    if (p->K0 != 2 && p->K0 != 4 && p->K0 != 8 && p->K0 != 16) return 0;
    iree_uk_mmt4d_params_t q = *p;
    q.flags = (p->flags & ~uint32_t(IREE_UK_FLAG_MMT4D_TYPE_MASK)) | IREE_UK_FLAG_MMT4D_TYPE_S8S8S32;
    return mmt4d_tc_workspace_size(&q);
  }
  TypeInfo ti;
  if (!tc_type_info(p->flags, &ti)) return 0;
  if (p->M0 != 16 || p->N0 != 16 || p->K0 < 1 || p->K < 1 || p->M < 1 || p->N < 1) return 0;
  const int64_t pitch = round_up(p->K * p->K0 * ti.es, 128);
  const size_t one = size_t(round_up(p->M * 16 * pitch, 1024) + round_up(p->N * 16 * pitch, 1024));
  // f32: a hi and a lo plane of both operands. Behind the operands: the job cursor and the
  // per-tile-row ready counters of the streamed LHS pre-pass.
  return (ti.triple ? 2 * one : one) + sync_block_bytes(p);
}

// Re-tiled RHS kept by the caller across calls (weights): its size, the scratch a call then
// still needs (the LHS part), and the pre-pass that fills it.
size_t mmt4d_tc_prepared_rhs_size(const iree_uk_mmt4d_params_t* p) {
  if ((p->flags & IREE_UK_FLAG_MMT4D_TYPE_MASK) == IREE_UK_FLAG_MMT4D_TYPE_S16U4S32) {
    // the u4 weights widened to bytes, K-major
    if (p->M0 != 1 || p->N0 != 32 || p->K0 != 8 || p->K < 1 || p->N < 1) return 0;
    return size_t(s16u4_layout(p).w_bytes);
  }
  TypeInfo ti;
  if (!tc_type_info(p->flags, &ti) || ti.triple) return 0;
  if (p->M0 != 16 || p->N0 != 16 || p->K0 < 1 || p->K < 1 || p->N < 1) return 0;
  const int64_t pitch = round_up(p->K * p->K0 * ti.es, 128);
  return size_t(round_up(p->N * 16 * pitch, 1024));
}
size_t mmt4d_tc_prepared_workspace_size(const iree_uk_mmt4d_params_t* p) {
  if ((p->flags & IREE_UK_FLAG_MMT4D_TYPE_MASK) == IREE_UK_FLAG_MMT4D_TYPE_S16U4S32) {
    if (p->M0 != 1 || p->N0 != 32 || p->K0 != 8 || p->K < 1 || p->M < 1) return 0;
    return size_t(2 * s16u4_layout(p).plane_bytes);  // the two byte planes of the LHS
  }
  TypeInfo ti;
  if (!tc_type_info(p->flags, &ti) || ti.triple) return 0;
  if (p->M0 != 16 || p->N0 != 16 || p->K0 < 1 || p->K < 1 || p->M < 1) return 0;
  const int64_t pitch = round_up(p->K * p->K0 * ti.es, 128);
  return size_t(round_up(p->M * 16 * pitch, 1024)) + sync_block_bytes(p);
}
int launch_mmt4d_tc_prepare_rhs(const iree_uk_mmt4d_params_t* p, void* prepared, size_t bytes,
                                cudaStream_t stream) {
  if ((p->flags & IREE_UK_FLAG_MMT4D_TYPE_MASK) == IREE_UK_FLAG_MMT4D_TYPE_S16U4S32) {
    const size_t need = mmt4d_tc_prepared_rhs_size(p);
    if (!need) return IREE_UK_B200_UNSUPPORTED;
    if (!prepared || bytes < need) return IREE_UK_B200_WORKSPACE_TOO_SMALL;
    const uintptr_t rhs = reinterpret_cast<uintptr_t>(p->rhs_buffer) + uintptr_t(p->rhs_offset / 2);
    if ((reinterpret_cast<uintptr_t>(prepared) & 255) || (rhs & 15) || (p->rhs_offset & 1) ||
        (p->rhs_stride0 & 1) || (p->rhs_stride0 / 2) % 16)
      return IREE_UK_B200_INVALID_ARGUMENT;
    const int64_t kchunks = (p->K + 63) / 64;
    if (p->N * kchunks > 0x7FFFFFFF) return IREE_UK_B200_UNSUPPORTED;
    unpack_u4_kernel<<<int(p->N * kchunks), 256, 0, stream>>>(
        reinterpret_cast<const char*>(rhs), p->rhs_stride0 / 2, static_cast<char*>(prepared),
        s16u4_layout(p).pitch, p->K, int(kchunks));
    return cuda_status(cudaGetLastError());
  }
  TypeInfo ti;
  if (!tc_type_info(p->flags, &ti) || ti.triple) return IREE_UK_B200_UNSUPPORTED;
  const size_t need = mmt4d_tc_prepared_rhs_size(p);
  if (!need) return IREE_UK_B200_UNSUPPORTED;
  if (!prepared || bytes < need) return IREE_UK_B200_WORKSPACE_TOO_SMALL;
  const uintptr_t rhs = reinterpret_cast<uintptr_t>(p->rhs_buffer) + uintptr_t(p->rhs_offset * ti.es);
  if ((reinterpret_cast<uintptr_t>(prepared) & 255) || (rhs & 15) || (p->rhs_stride0 * ti.es) % 16)
    return IREE_UK_B200_INVALID_ARGUMENT;
  const int G = p->K0 * ti.es;
  if (G != 1 && G != 2 && G != 4 && G != 8 && G != 16) return IREE_UK_B200_UNSUPPORTED;
  const int64_t pitch = round_up(p->K * p->K0 * ti.es, 128);
  return launch_retile(nullptr, 0, nullptr, 0, reinterpret_cast<const char*>(rhs),
                       p->rhs_stride0 * ti.es, static_cast<char*>(prepared), p->N, pitch, p->K, G,
                       stream);
}

namespace {
// The two-CTA kernel works on 256-row tiles with at most 74 CTA pairs in flight; it pays once
// there are enough 256 x 128 tiles to occupy every pair.
bool pair_kernel_pays(const iree_uk_mmt4d_params_t* p) {
  const int64_t m_tiles = (p->M * 16 + 255) / 256, n_tiles = (p->N * 16 + 127) / 128;
  return p->M * 16 >= 256 && p->N * 16 >= 128 && m_tiles * n_tiles >= 74;
}
}  // namespace

int launch_mmt4d_tc(const iree_uk_mmt4d_params_t* p, void* ws, size_t ws_bytes, int variant,
                    cudaStream_t stream, const void* const* peer_out_buffers, int num_peers,
                    const void* multicast_out, const void* prepared_rhs, const RowMajorOut* rm) {
  if (multicast_out && num_peers) return IREE_UK_B200_INVALID_ARGUMENT;
  if (rm && (num_peers || multicast_out)) return IREE_UK_B200_INVALID_ARGUMENT;
  if (num_peers < 0 || num_peers > IREE_UK_B200_MAX_PEERS || (num_peers && !peer_out_buffers))
    return IREE_UK_B200_INVALID_ARGUMENT;
  // Peer copies exist for the plain tiled epilogue only.
  const uint32_t type = p->flags & IREE_UK_FLAG_MMT4D_TYPE_MASK;
  const bool planes = type == IREE_UK_FLAG_MMT4D_TYPE_S16U4S32 || type == IREE_UK_FLAG_MMT4D_TYPE_S16S16S32;
  if ((num_peers || multicast_out || rm) && planes) return IREE_UK_B200_UNSUPPORTED;
  if (prepared_rhs && type == IREE_UK_FLAG_MMT4D_TYPE_S16S16S32) return IREE_UK_B200_UNSUPPORTED;
  if (type == IREE_UK_FLAG_MMT4D_TYPE_S16U4S32) return launch_mmt4d_tc_s16u4(p, ws, ws_bytes, stream, prepared_rhs);
  if (type == IREE_UK_FLAG_MMT4D_TYPE_S16S16S32) return launch_mmt4d_tc_s16s16(p, ws, ws_bytes, stream);
  if (type == IREE_UK_FLAG_MMT4D_TYPE_S16S8S32) {
    if (num_peers || multicast_out || prepared_rhs || rm) return IREE_UK_B200_UNSUPPORTED;
    return launch_mmt4d_tc_s16s16(p, ws, ws_bytes, stream);
  }
  if (type == IREE_UK_FLAG_MMT4D_TYPE_S8S4S32) {
    if (num_peers || multicast_out || prepared_rhs || rm) return IREE_UK_B200_UNSUPPORTED;
    return launch_mmt4d_tc_s8s4(p, ws, ws_bytes, variant, stream);
  }
  TypeInfo ti;
  if (!tc_type_info(p->flags, &ti) || !(rm ? mmt4d_tc_operands_eligible(p) : mmt4d_tc_eligible(p)))
    return IREE_UK_B200_UNSUPPORTED;
  if ((num_peers || multicast_out || rm) && ti.out_es != 4) return IREE_UK_B200_UNSUPPORTED;  // 32-bit only
  if (rm && (rm->rows < 0 || rm->cols < 0 || rm->rows > p->M * 16 || rm->cols > p->N * 16 ||
             (reinterpret_cast<uintptr_t>(p->out_buffer) & 3)))
    return IREE_UK_B200_INVALID_ARGUMENT;
  uint32_t* status = device_status_word();
  const DeviceInfo* di = device_info();
  if (!status || !di) return IREE_UK_B200_CUDA_ERROR;

  TcParams P;
  std::memset(&P, 0, sizeof P);
  KernelTiming* timing = kernel_timing();
  cudaEvent_t* tev = timing ? timing->next_slot() : nullptr;
  if (tev) KernelTiming::record(tev[0], stream);
  int bn = pick_bn(p->M, p->N);
  bool pair = false;
  int pair_clusters = 0;
  const int64_t kelems = p->K * p->K0;
  char* lhs = const_cast<char*>(static_cast<const char*>(p->lhs_buffer)) + p->lhs_offset * ti.es;
  char* rhs = const_cast<char*>(static_cast<const char*>(p->rhs_buffer)) + p->rhs_offset * ti.es;
  const int kblk_elems = 128 / ti.es;  // one 128-byte swizzle row of K per TMA box
  // Variant 0 = automatic: the two-CTA kernel when the problem gives every CTA pair work,
  // the one-CTA kernel otherwise. 5 / 6 force the two-CTA / one-CTA kernel; 3 is the
  // scratch-free MN-major staging of 16-bit K0 = 1 operands.
  // Variant 0 = automatic (below). kTcVariantTwoCta / kTcVariantOneCta force a kernel with the
  // whole re-tile in the pre-pass; kTcVariantStreamed forces the two-CTA kernel with the
  // streamed pre-pass.
  const int streamed_granule_form = ti.triple ? 0 : streamed_form_of_granule(p->K0 * ti.es);
  bool want_streamed = false, variant_forced_streamed = false;
  if (variant == 0) {
    variant = pair_kernel_pays(p) ? kTcVariantTwoCta : kTcVariantOneCta;
    want_streamed = variant == kTcVariantTwoCta && streamed_granule_form != 0 &&
                    !debug_int("IREE_UK_B200_DEBUG_NO_STREAMED", 0);
  } else if (variant == kTcVariantStreamed) {
    if (!streamed_granule_form) return IREE_UK_B200_UNSUPPORTED;
    variant = kTcVariantTwoCta;
    want_streamed = true;
    variant_forced_streamed = true;
  }
  int stream_form = 0;  // set below once the startup set is known to leave work for the workers
  // K boxes per stage: two for the two-CTA kernel (64 KB stages, half the barrier round trips
  // per MMA), one for the one-CTA kernel (its stage is already 48 KB).
  int kboxes = debug_int("IREE_UK_B200_DEBUG_KBOXES", variant == kTcVariantTwoCta ? 2 : 1) == 2 ? 2 : 1;
  const int mma_k = 32 / ti.es;        // K per tcgen05.mma: 16 (16-bit) or 32 (8-bit)

  if (variant == kTcVariantTwoCta || variant == kTcVariantOneCta) {
    // K-major operands from the re-tiled scratch: the one-CTA kernel (6) on 128 x bn tiles, or
    // the two-CTA kernel (5) on 256 x bn tiles per CTA pair.
    if (prepared_rhs && ti.triple) return IREE_UK_B200_UNSUPPORTED;
    const size_t need = prepared_rhs ? mmt4d_tc_prepared_workspace_size(p) : mmt4d_tc_workspace_size(p);
    if (!ws || ws_bytes < need) return IREE_UK_B200_WORKSPACE_TOO_SMALL;
    if ((reinterpret_cast<uintptr_t>(ws) | reinterpret_cast<uintptr_t>(prepared_rhs)) & 255)
      return IREE_UK_B200_INVALID_ARGUMENT;
    pair = variant == kTcVariantTwoCta;
    if (pair) {
      pair_clusters = di->pair_clusters[ti.is_int ? 1 : 0][want_streamed ? streamed_granule_form : 0];
      if (pair_clusters < 1) return IREE_UK_B200_CUDA_ERROR;
      bn = pick_bn_pair(p->M, p->N, pair_clusters, !ti.triple);
    }
    if (ti.triple) kboxes = 1;  // the two boxes of a stage are the hi and lo planes
    const int64_t pitch = round_up(kelems * ti.es, 128);
    const int64_t a_bytes = round_up(p->M * 16 * pitch, 1024), b_bytes = round_up(p->N * 16 * pitch, 1024);
    char* ws_a = static_cast<char*>(ws);
    // A prepared RHS is this pre-pass's output kept by the caller: only the LHS is re-tiled.
    char* ws_b = prepared_rhs ? const_cast<char*>(static_cast<const char*>(prepared_rhs)) : ws_a + a_bytes;
    const int G = p->K0 * ti.es;
    // Streamed LHS pre-pass: the pre-pass kernel re-tiles the RHS and the LHS rows of the first
    // group of m-tiles; the main kernel's workers re-tile the LHS rows of the later groups.
    int64_t a_first = p->M;
    if (want_streamed) {
      const int m_tiles = int((p->M * 16 + 2 * BM - 1) / (2 * BM));
      const int gm = std::min(m_tiles, debug_int("IREE_UK_B200_DEBUG_GROUP_M", 8));
      const int64_t first = std::min<int64_t>(p->M, int64_t(gm) * (2 * BM / 16));
      const int kj = G == 4 ? warp_job_k1<4>() : warp_job_k1<2>();
      const int64_t kch = (p->K + kj - 1) / kj;
      const int64_t jobs = (p->M - first) * kch;
      // Worth it once the rows the workers take over are a good part of the whole pre-pass
      // (at least a quarter of all tile rows of both operands): measured +1 % on the 8-way
      // shard of the headline problem, nothing on the unsharded one, whose pre-pass is mostly RHS.
      const bool pays = (p->M - first) * 4 >= p->M + (prepared_rhs ? 0 : p->N) ||
                        variant_forced_streamed;
      if (jobs > 0 && jobs < (1ll << 31) && pays) {
        stream_form = streamed_granule_form;
        a_first = first;
        P.src_a = lhs;
        P.src_stride_a = p->lhs_stride0 * ti.es;
        P.K1 = p->K;
        P.rt_dst_a = ws_a;
        P.rt_pitch = pitch;
        P.rt_sync = reinterpret_cast<uint32_t*>(ws_a + a_bytes + (prepared_rhs ? 0 : b_bytes));
        P.rt_a_first = a_first;
        P.rt_jobs = uint32_t(jobs);
        P.rt_kchunks = int32_t(kch);
      } else if (pair) {  // occupancy of the plain form decides the grid
        pair_clusters = di->pair_clusters[ti.is_int ? 1 : 0][0];
      }
    }
    const int rc = launch_retile(lhs, p->lhs_stride0 * ti.es, ws_a, a_first, rhs,
                                 p->rhs_stride0 * ti.es, ws_b, prepared_rhs ? 0 : p->N, pitch,
                                 p->K, G, stream, stream_form ? P.rt_sync : nullptr,
                                 stream_form ? int(1 + p->M) : 0);
    if (rc) return rc;
    const int64_t plane_bytes = a_bytes + b_bytes;  // [A hi | B hi][A lo | B lo]
    if (ti.triple) {
      const int64_t vecs = plane_bytes / 16;
      const int blocks = int(std::min<int64_t>((vecs + 255) / 256, int64_t(di->sms) * 16));
      split_tf32_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<uint4*>(ws_a),
                                                    reinterpret_cast<uint4*>(ws_a + plane_bytes), vecs);
      if (cudaGetLastError() != cudaSuccess) return IREE_UK_B200_CUDA_ERROR;
    }
    const int b_rows = pair ? bn / 2 : bn;  // RHS rows one CTA stages
    const int tile_m = pair ? 2 * BM : BM;
    const uint64_t planes = ti.triple ? 2 : 1;
    const uint64_t da[3] = {uint64_t(kelems), uint64_t(p->M * 16), planes};
    const uint64_t db[3] = {uint64_t(kelems), uint64_t(p->N * 16), planes};
    const uint64_t sa[2] = {uint64_t(pitch), ti.triple ? uint64_t(plane_bytes) : uint64_t(pitch) * uint64_t(p->M * 16)};
    const uint64_t sb[2] = {uint64_t(pitch), ti.triple ? uint64_t(plane_bytes) : uint64_t(pitch) * uint64_t(p->N * 16)};
    const uint32_t ba[3] = {uint32_t(kblk_elems), BM, 1};
    const uint32_t bb[3] = {uint32_t(kblk_elems), uint32_t(b_rows), 1};
    if (!encode_map(&P.map_a, ti.tm_type, ws_a, da, sa, ba, CU_TENSOR_MAP_SWIZZLE_128B) ||
        !encode_map(&P.map_b, ti.tm_type, ws_b, db, sb, bb, CU_TENSOR_MAP_SWIZZLE_128B))
      return IREE_UK_B200_CUDA_ERROR;
    if (ti.triple) {
      P.sa = {2, BM * 128, {kblk_elems, 0, 0}, {0, tile_m, 0}, {0, 0, 1}, {0, pair ? BM : 0, 0}};
      P.sb = {2, b_rows * 128, {kblk_elems, 0, 0}, {0, bn, 0}, {0, 0, 1}, {0, pair ? b_rows : 0, 0}};
      P.triple = 1;
    } else {
      P.sa = {kboxes, BM * 128, {kboxes * kblk_elems, 0, 0}, {0, tile_m, 0}, {kblk_elems, 0, 0}, {0, pair ? BM : 0, 0}};
      P.sb = {kboxes, b_rows * 128, {kboxes * kblk_elems, 0, 0}, {0, bn, 0}, {kblk_elems, 0, 0}, {0, pair ? b_rows : 0, 0}};
    }
    const int boxes = ti.triple ? 2 : kboxes;
    P.desc_hi_a = P.desc_hi_b = desc_hi(1024, 2);
    P.desc_lbo_a = P.desc_lbo_b = 1;
    P.kadv_a = P.kadv_b = 2;  // 32 bytes of K per MMA inside the 128-byte swizzle row
    P.kbox_units_a = uint32_t(BM * 128) >> 4;
    P.kbox_units_b = uint32_t(b_rows * 128) >> 4;
    P.idesc = make_idesc(ti, bn, false, tile_m);
    P.kboxes = kboxes;
    P.mma_per_box = 4;
    P.stage_bytes_a = boxes * BM * 128;
    P.stage_bytes_b = boxes * b_rows * 128;
    P.num_kb = int((kelems + kboxes * kblk_elems - 1) / (kboxes * kblk_elems));
  } else {
    // MN-major, straight from a K0 = 1 16-bit operand [tile][K1][16]: for a fixed k the 16 rows
    // of a tile are 32 contiguous bytes, so TMA stages boxes of 16 elements x kblk k-steps x
    // (rows / 16) tiles with the 32-byte swizzle. In shared memory 8 k-steps of one tile are a
    // 256-byte atom (stride byte offset); the next tile is kblk * 32 bytes on (leading byte
    // offset). No scratch is needed; the main loop runs at about half the K-major rate.
    if (ti.es != 2 || p->K0 != 1 || variant != kTcVariantDirect) return IREE_UK_B200_UNSUPPORTED;
    const int kblk = 64;
    const uint64_t da[3] = {16, uint64_t(p->K), uint64_t(p->M)};
    const uint64_t db[3] = {16, uint64_t(p->K), uint64_t(p->N)};
    const uint64_t sa[2] = {32, uint64_t(p->lhs_stride0 * 2)};
    const uint64_t sb[2] = {32, uint64_t(p->rhs_stride0 * 2)};
    const uint32_t ba[3] = {16, uint32_t(kblk), BM / 16};
    const uint32_t bb[3] = {16, uint32_t(kblk), uint32_t(bn / 16)};
    if (!encode_map(&P.map_a, ti.tm_type, lhs, da, sa, ba, CU_TENSOR_MAP_SWIZZLE_32B) ||
        !encode_map(&P.map_b, ti.tm_type, rhs, db, sb, bb, CU_TENSOR_MAP_SWIZZLE_32B))
      return IREE_UK_B200_CUDA_ERROR;
    P.sa = {1, BM * kblk * 2, {0, kblk, 0}, {0, 0, BM / 16}, {0, 0, 0}};
    P.sb = {1, bn * kblk * 2, {0, kblk, 0}, {0, 0, bn / 16}, {0, 0, 0}};
    P.desc_hi_a = P.desc_hi_b = desc_hi(256, 6);
    P.desc_lbo_a = P.desc_lbo_b = uint32_t(kblk * 32) >> 4;
    P.kadv_a = P.kadv_b = (16 * 32) >> 4;
    P.stage_bytes_a = BM * kblk * 2;
    P.stage_bytes_b = bn * kblk * 2;
    P.idesc = make_idesc(ti, bn, true);
    P.kboxes = 1;
    P.mma_per_box = kblk / mma_k;
    P.num_kb = int((p->K + kblk - 1) / kblk);
  }

  const int tile_m = pair ? 2 * BM : BM;
  P.bn = bn;
  P.m_tiles = int((p->M * 16 + tile_m - 1) / tile_m);
  P.n_tiles = int((p->N * 16 + bn - 1) / bn);
  P.num_work = P.tail_first = P.m_tiles * P.n_tiles;
  P.tail_split = 1;
  if (pair && !ti.triple) {
    // Tail of the schedule: the tiles of the last, partial round over the CTA pairs are cut
    // along N into 2 or 4 narrow tiles when that shortens the round (tile time ~ width + 96
    // columns' worth, as in pick_bn_pair).
    const int tiles = P.num_work, rem = tiles % pair_clusters;
    if (tiles > pair_clusters && rem != 0) {
      int best = 1;
      tail_round_cost(rem, bn, pair_clusters, true, &best);
      best = debug_int("IREE_UK_B200_DEBUG_TAIL_SPLIT", best);
      if (best > 1) {
        const int b_rows_narrow = bn / best / 2;
        const int64_t pitch = round_up(kelems * ti.es, 128);
        const uint64_t db[3] = {uint64_t(kelems), uint64_t(p->N * 16), 1};
        const uint64_t sb[2] = {uint64_t(pitch), uint64_t(pitch) * uint64_t(p->N * 16)};
        const uint32_t bb[3] = {uint32_t(kblk_elems), uint32_t(b_rows_narrow), 1};
        char* ws_b = prepared_rhs ? const_cast<char*>(static_cast<const char*>(prepared_rhs))
                                  : static_cast<char*>(ws) + round_up(p->M * 16 * pitch, 1024);
        if (!encode_map(&P.map_b_narrow, ti.tm_type, ws_b, db, sb, bb, CU_TENSOR_MAP_SWIZZLE_128B))
          return IREE_UK_B200_CUDA_ERROR;
        P.tail_first = tiles - rem;
        P.tail_split = best;
        P.num_work = P.tail_first + rem * best;
      }
    }
  }
  P.group_m = std::min(P.m_tiles, debug_int("IREE_UK_B200_DEBUG_GROUP_M", pair ? 8 : 16));
  P.out = static_cast<char*>(p->out_buffer) + p->out_offset * ti.out_es;
  P.out_stride0 = p->out_stride0;
  P.M1 = p->M;
  P.N1 = p->N;
  P.accumulate = (p->flags & IREE_UK_FLAG_MMT4D_ACCUMULATE) ? 1 : 0;
  P.out_is_int = ti.is_int ? 1 : 0;
  P.out_vec32 = ((reinterpret_cast<uintptr_t>(P.out) & 31) == 0 && (p->out_stride0 * ti.out_es) % 32 == 0) ? 1 : 0;
  P.out16 = ti.out_es == 2 ? (ti.fmt == 0u ? 1 : 2) : 0;
  if (rm) {  // the unpack folded into the epilogue: rows x cols of a row-major matrix
    P.out_row_major = 1;
    P.rows = rm->rows;
    P.cols = rm->cols;
    P.out_vec16 = ((reinterpret_cast<uintptr_t>(P.out) & 15) == 0 && (p->out_stride0 * 4) % 16 == 0) ? 1 : 0;
    P.out_vec32 = ((reinterpret_cast<uintptr_t>(P.out) & 31) == 0 && (p->out_stride0 * 4) % 32 == 0) ? 1 : 0;
  }
  if (multicast_out) {
    P.use_multicast = 1;
    P.mc_delta = int64_t(reinterpret_cast<intptr_t>(multicast_out) -
                         reinterpret_cast<intptr_t>(p->out_buffer));
    if (P.mc_delta % 16) return IREE_UK_B200_INVALID_ARGUMENT;
  }
  P.num_peers = num_peers;
  for (int g = 0; g < num_peers; ++g) {
    const char* peer = static_cast<const char*>(peer_out_buffers[g]);
    if (!peer) return IREE_UK_B200_INVALID_ARGUMENT;
    P.peer_delta[g] = int64_t(reinterpret_cast<intptr_t>(peer) -
                              reinterpret_cast<intptr_t>(p->out_buffer));
    // a peer buffer must allow the same vector width as the local one
    if (P.peer_delta[g] % (P.out_vec32 ? 32 : 16)) return IREE_UK_B200_INVALID_ARGUMENT;
  }
  P.status = status;
  set_wait_policy(&P);

  const int stage_bytes = P.stage_bytes_a + P.stage_bytes_b;
  const int smem_budget = 200 * 1024;
  P.num_stages = std::max(2, std::min(kMaxStages, smem_budget / stage_bytes));
  // In the two-CTA kernel, 32-bit output tiles that are only written leave through shared memory as
  // whole 1 KB bulk copies (1-2 % faster than 32-byte stores from registers on the headline
  // shape; no gain for small problems or when the old tile is read first).
  P.staged_epilogue = (pair && !rm && !P.out16 && !multicast_out && !P.accumulate &&
                       debug_int("IREE_UK_B200_DEBUG_STAGED_EPILOGUE", 1)) ? 1 : 0;
  const size_t epi_bytes = (num_peers || multicast_out || P.staged_epilogue) ? 4 * kEpiStageBytes : 0;
  const size_t smem = size_t(P.num_stages) * stage_bytes + 1024 + epi_bytes;

  if (smem > size_t(di->max_smem)) return IREE_UK_B200_CUDA_ERROR;
  cudaError_t e;
  if (tev) KernelTiming::record(tev[1], stream);
  if (pair) {
    const int grid = 2 * std::min(P.num_work, pair_clusters);
    e = launch_main(pair_kernel(ti.is_int, stream_form), grid, 2, smem, stream, P,
                    pair_threads(stream_form));
  } else {
    const int grid = std::min(P.m_tiles * P.n_tiles, di->sms);
    e = ti.is_int ? launch_main(mmt4d_tc_kernel<true>, grid, 1, smem, stream, P)
                  : launch_main(mmt4d_tc_kernel<false>, grid, 1, smem, stream, P);
  }
  if (e != cudaSuccess) return IREE_UK_B200_CUDA_ERROR;
  if (tev) {
    KernelTiming::record(tev[2], stream);
    timing->calls.fetch_add(1, std::memory_order_relaxed);
  }
  return cuda_status(cudaGetLastError());
}

}  // namespace uk

namespace uk {

// s8s4s32 with 16x16xK0 tiles: the RHS nibbles are sign-extended to bytes and re-tiled in one
// pre-pass (widen_s4_kernel), which leaves exactly what a prepared s8s8s32 RHS is; the call
// then runs as s8s8s32 with that prepared RHS (one 8-bit tensor-core product per term, the LHS
// re-tile streamed as usual). Workspace: [LHS scratch + sync block][widened RHS].
int launch_mmt4d_tc_s8s4(const iree_uk_mmt4d_params_t* p, void* ws, size_t ws_bytes, int variant,
                         cudaStream_t stream) {
  if (!mmt4d_tc_s8s4_eligible(p)) return IREE_UK_B200_UNSUPPORTED;
  iree_uk_mmt4d_params_t q = *p;
  q.flags = (p->flags & ~uint32_t(IREE_UK_FLAG_MMT4D_TYPE_MASK)) | IREE_UK_FLAG_MMT4D_TYPE_S8S8S32;
  const size_t lhs_part = mmt4d_tc_prepared_workspace_size(&q), rhs_part = mmt4d_tc_prepared_rhs_size(&q);
  if (!lhs_part || !rhs_part) return IREE_UK_B200_UNSUPPORTED;
  if (!ws || ws_bytes < lhs_part + rhs_part) return IREE_UK_B200_WORKSPACE_TOO_SMALL;
  if (reinterpret_cast<uintptr_t>(ws) & 255) return IREE_UK_B200_INVALID_ARGUMENT;
  char* widened = static_cast<char*>(ws) + lhs_part;
  const int64_t pitch = round_up(p->K * p->K0, 128);
  const int rc = launch_widen_s4(static_cast<const char*>(p->rhs_buffer) + p->rhs_offset / 2,
                                 p->rhs_stride0 / 2, widened, p->N, pitch, p->K, p->K0, stream);
  if (rc) return rc;
  // the s8s8s32 call never reads its RHS operand itself: it is described by the prepared copy
  q.rhs_buffer = widened;
  q.rhs_offset = 0;
  q.rhs_stride0 = p->K * 16 * p->K0;
  return launch_mmt4d_tc(&q, ws, lhs_part, variant, stream, nullptr, 0, nullptr, widened);
}

namespace {

using SwKernel = void (*)(const TcParams);
// [is_int][log2 G]
SwKernel sw_kernel(bool is_int, int G) {
  int lg = 0;
  while ((1 << lg) < G) ++lg;
  static const SwKernel table[2][5] = {
      {mmt4d_tc_sw_kernel<false, 1>, mmt4d_tc_sw_kernel<false, 2>, mmt4d_tc_sw_kernel<false, 4>,
       mmt4d_tc_sw_kernel<false, 8>, mmt4d_tc_sw_kernel<false, 16>},
      {mmt4d_tc_sw_kernel<true, 1>, mmt4d_tc_sw_kernel<true, 2>, mmt4d_tc_sw_kernel<true, 4>,
       mmt4d_tc_sw_kernel<true, 8>, mmt4d_tc_sw_kernel<true, 16>}};
  return table[is_int ? 1 : 0][lg];
}

// Raises the dynamic shared-memory limit of every scratch-free kernel once per device.
bool sw_kernels_ready(const DeviceInfo* di, int* max_dyn) {
  constexpr int kMaxDevices = 64;
  static int limit[kMaxDevices] = {};
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return false;
  std::lock_guard<std::mutex> lock(mu);
  if (!limit[dev]) {
    int optin = 0;
    if (cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess)
      return false;
    int lim = optin;
    for (int is_int = 0; is_int < 2; ++is_int)
      for (int G = 1; G <= 16; G *= 2) {
        const void* fn = reinterpret_cast<const void*>(sw_kernel(is_int != 0, G));
        cudaFuncAttributes fa;
        if (cudaFuncGetAttributes(&fa, fn) != cudaSuccess) return false;
        const int dyn = optin - int(fa.sharedSizeBytes);
        if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, dyn) != cudaSuccess) {
          cudaGetLastError();
          return false;
        }
        lim = std::min(lim, dyn);
      }
    limit[dev] = lim;
  }
  (void)di;
  *max_dyn = limit[dev];
  return true;
}

}  // namespace

bool mmt4d_tc_sw_eligible(const iree_uk_mmt4d_params_t* p) {
  TypeInfo ti;
  return tc_type_info(p->flags, &ti) && !ti.triple && mmt4d_tc_eligible(p);
}

// Tensor-core mmt4d without scratch: one launch of mmt4d_tc_sw_kernel.
int launch_mmt4d_tc_sw(const iree_uk_mmt4d_params_t* p, cudaStream_t stream) {
  TypeInfo ti;
  if (!tc_type_info(p->flags, &ti) || ti.triple || !mmt4d_tc_eligible(p)) return IREE_UK_B200_UNSUPPORTED;
  uint32_t* status = device_status_word();
  const DeviceInfo* di = device_info();
  int max_dyn = 0;
  if (!status || !di || !sw_kernels_ready(di, &max_dyn)) return IREE_UK_B200_CUDA_ERROR;
  TcParams P;
  std::memset(&P, 0, sizeof P);
  KernelTiming* timing = kernel_timing();
  cudaEvent_t* tev = timing ? timing->next_slot() : nullptr;
  if (tev) { KernelTiming::record(tev[0], stream); KernelTiming::record(tev[1], stream); }
  const int G = p->K0 * ti.es;
  const int bn = pick_bn(p->M, p->N);
  P.src_a = static_cast<const char*>(p->lhs_buffer) + p->lhs_offset * ti.es;
  P.src_b = static_cast<const char*>(p->rhs_buffer) + p->rhs_offset * ti.es;
  P.src_stride_a = p->lhs_stride0 * ti.es;
  P.src_stride_b = p->rhs_stride0 * ti.es;
  P.K1 = p->K;
  const int kps = 128 / G;  // k1 steps per 128-byte swizzle row
  P.desc_hi_a = P.desc_hi_b = desc_hi(1024, 2);
  P.desc_lbo_a = P.desc_lbo_b = 1;
  P.kadv_a = P.kadv_b = 2;
  P.kbox_units_a = uint32_t(BM * 128) >> 4;
  P.kbox_units_b = uint32_t(bn * 128) >> 4;
  P.idesc = make_idesc(ti, bn, false);
  P.kboxes = 1;
  P.mma_per_box = 4;
  P.stage_bytes_a = BM * 128;
  P.stage_bytes_b = bn * 128;
  P.num_kb = int((p->K + kps - 1) / kps);
  P.bn = bn;
  P.m_tiles = int((p->M * 16 + BM - 1) / BM);
  P.n_tiles = int((p->N * 16 + bn - 1) / bn);
  P.group_m = std::min(P.m_tiles, 16);
  P.out = static_cast<char*>(p->out_buffer) + p->out_offset * ti.out_es;
  P.out_stride0 = p->out_stride0;
  P.M1 = p->M;
  P.N1 = p->N;
  P.accumulate = (p->flags & IREE_UK_FLAG_MMT4D_ACCUMULATE) ? 1 : 0;
  P.out_is_int = ti.is_int ? 1 : 0;
  P.out_vec32 = ((reinterpret_cast<uintptr_t>(P.out) & 31) == 0 && (p->out_stride0 * ti.out_es) % 32 == 0) ? 1 : 0;
  P.out16 = ti.out_es == 2 ? (ti.fmt == 0u ? 1 : 2) : 0;
  P.status = status;
  set_wait_policy(&P);
  const int stage_bytes = P.stage_bytes_a + P.stage_bytes_b;
  P.num_stages = std::max(2, std::min(kMaxStages, 200 * 1024 / stage_bytes));
  const size_t smem = size_t(P.num_stages) * stage_bytes + 1024;
  if (smem > size_t(max_dyn)) return IREE_UK_B200_CUDA_ERROR;
  const int grid = std::min(P.m_tiles * P.n_tiles, di->sms);
  sw_kernel(ti.is_int, G)<<<grid, kSwThreads, smem, stream>>>(P);
  if (tev) {
    KernelTiming::record(tev[2], stream);
    timing->calls.fetch_add(1, std::memory_order_relaxed);
  }
  return cuda_status(cudaGetLastError());
}

}  // namespace uk

// ---------------------------------------------------------------------------------------
// mmt4d with library-owned scratch, for callers that cannot allocate
// ---------------------------------------------------------------------------------------
namespace uk {
namespace {

// Part of the library image on every device that loads it. In host code this name is only a
// handle for cudaGetSymbolAddress, never a pointer to hand to a kernel.
static __device__ __align__(256) unsigned char g_static_scratch[IREE_UK_B200_STATIC_SCRATCH_BYTES];

// Device address of g_static_scratch on the current device, looked up once per device.
void* static_scratch_address() {
  constexpr int kMaxDevices = 64;
  static void* addr[kMaxDevices] = {};
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!addr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_static_scratch) != cudaSuccess)
      return nullptr;
    addr[dev] = p;
  }
  return addr[dev];
}

}  // namespace
}  // namespace uk

extern "C" int iree_uk_b200_mmt4d_static_scratch(const iree_uk_mmt4d_params_t* params,
                                                 void* cu_stream) {
  const int rc = uk::validate_mmt4d(params);
  if (rc) return rc;
  // Only the kernels that iree_uk_b200_mmt4d_ws would run with scratch need the array: the
  // tensor-core triples with 16x16 tiles, and s16u4s32 1x32x8 once there are 16 rows (below
  // that the weight-streaming kernel serves it, without scratch). Everything else goes the
  // usual way.
  const int path = iree_uk_b200_mmt4d_path(params, 1);
  if (path < 0) return -path;
  if (path != IREE_UK_B200_PATH_TCGEN05_RETILE) return iree_uk_b200_mmt4d(params, cu_stream);
  if (uk::mmt4d_tc_workspace_size(params) > size_t(IREE_UK_B200_STATIC_SCRATCH_BYTES))
    return IREE_UK_B200_WORKSPACE_TOO_SMALL;
  void* scratch = uk::static_scratch_address();
  if (!scratch) return IREE_UK_B200_CUDA_ERROR;
  return iree_uk_b200_mmt4d_ws(params, scratch, size_t(IREE_UK_B200_STATIC_SCRATCH_BYTES),
                               cu_stream);
}

// ---------------------------------------------------------------------------------------
// fused row-major matmul: what pack -> mmt4d -> unpack computes, without the packed copies
// ---------------------------------------------------------------------------------------
namespace uk {
namespace {

// [K][N] row-major -> [N][K] row-major with a pitch, through a 64 x 64 shared-memory tile.
template <int ES>
__global__ void __launch_bounds__(256) transpose_kn_kernel(const char* __restrict__ src,
                                                           int64_t src_pitch_b, char* __restrict__ dst,
                                                           int64_t dst_pitch_b, int64_t K, int64_t N) {
  using E = typename std::conditional<ES == 1, uint8_t, uint16_t>::type;
  constexpr int T = 64;
  __shared__ E tile[T][T + 2 * (4 / ES) + 0];  // [n][k], padded
  pdl_launch_dependents();
  const int64_t k_base = int64_t(blockIdx.y) * T, n_base = int64_t(blockIdx.x) * T;
  for (int e = threadIdx.x; e < T * T; e += blockDim.x) {
    const int k = e / T, n = e - k * T;
    const int64_t gk = k_base + k, gn = n_base + n;
    tile[n][k] = (gk < K && gn < N) ? *reinterpret_cast<const E*>(src + gk * src_pitch_b + gn * ES)
                                     : E(0);
  }
  __syncthreads();
  constexpr int NV = 16 / ES;       // elements per 16-byte vector
  constexpr int VPR = T / NV;       // vectors per tile row
  for (int v = threadIdx.x; v < T * VPR; v += blockDim.x) {
    const int n = v / VPR, kv = v - n * VPR;
    const int64_t gn = n_base + n, gk = k_base + int64_t(kv) * NV;
    if (gn >= N || gk >= K) continue;
    char* dp = dst + gn * dst_pitch_b + gk * ES;
    if (gk + NV <= K) {
      uint32_t w[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint32_t x = 0;
#pragma unroll
        for (int j = 0; j < 4 / ES; ++j) x |= uint32_t(tile[n][kv * NV + q * (4 / ES) + j]) << (8 * ES * j);
        w[q] = x;
      }
      *reinterpret_cast<uint4*>(dp) = make_uint4(w[0], w[1], w[2], w[3]);
    } else {
      for (int j = 0; j < NV && gk + j < K; ++j) reinterpret_cast<E*>(dp)[j] = tile[n][kv * NV + j];
    }
  }
}

struct MatmulLayout {
  int64_t pitch, rhs_t_bytes, lhs_copy_bytes;
};
MatmulLayout matmul_layout(int64_t M, int64_t N, int64_t K, int es) {
  MatmulLayout l;
  l.pitch = round_up(K * es, 128);
  l.rhs_t_bytes = round_up(N * l.pitch, 1024);
  l.lhs_copy_bytes = round_up(M * l.pitch, 1024);
  return l;
}

}  // namespace

size_t matmul_workspace_size(uint32_t flags, int64_t M, int64_t N, int64_t K) {
  TypeInfo ti;
  if (!tc_type_info(flags, &ti) || M < 1 || N < 1 || K < 1) return 0;
  const MatmulLayout l = matmul_layout(M, N, K, ti.es);
  return size_t(l.rhs_t_bytes + l.lhs_copy_bytes);
}

// lhs [M][K] (row pitch lhs_pitch_b), rhs [K][N] (row pitch rhs_pitch_b), out [M][N] 32-bit.
int launch_matmul_rowmajor(uint32_t flags, const char* lhs, int64_t lhs_pitch_b, const char* rhs,
                           int64_t rhs_pitch_b, char* out, int64_t out_stride0, int64_t M, int64_t N,
                           int64_t K, void* ws, size_t ws_bytes, cudaStream_t stream) {
  TypeInfo ti;
  if (!tc_type_info(flags, &ti)) return IREE_UK_B200_UNSUPPORTED;
  if (M > 0x7FFFFFFF || N > 0x7FFFFFFF || K > 0x7FFFFFFF) return IREE_UK_B200_UNSUPPORTED;
  const MatmulLayout l = matmul_layout(M, N, K, ti.es);
  if (!ws || ws_bytes < size_t(l.rhs_t_bytes + l.lhs_copy_bytes)) return IREE_UK_B200_WORKSPACE_TOO_SMALL;
  if (reinterpret_cast<uintptr_t>(ws) & 255) return IREE_UK_B200_INVALID_ARGUMENT;
  uint32_t* status = device_status_word();
  const DeviceInfo* di = device_info();
  if (!status || !di) return IREE_UK_B200_CUDA_ERROR;
  KernelTiming* timing = kernel_timing();
  cudaEvent_t* tev = timing ? timing->next_slot() : nullptr;
  if (tev) KernelTiming::record(tev[0], stream);

  // RHS: transposed once into K-major rows. LHS: used in place when TMA can address it,
  // else copied with a TMA-friendly pitch.
  char* rhs_t = static_cast<char*>(ws);
  char* lhs_copy = rhs_t + l.rhs_t_bytes;
  // A 16-bit row-major RHS is itself a legal tensor-core operand: N-contiguous ("MN-major")
  // rows that TMA stages as 64-column x K swizzled boxes. It needs TMA's alignment; 8-bit
  // operands must be K-major, so they are always transposed.
  const bool b_direct = ti.es == 2 && (reinterpret_cast<uintptr_t>(rhs) & 15) == 0 &&
                        (rhs_pitch_b & 15) == 0 && !debug_int("IREE_UK_B200_DEBUG_MATMUL_TRANSPOSE", 0);
  if (!b_direct) {
    dim3 grid(unsigned((N + 63) / 64), unsigned((K + 63) / 64));
    if (grid.y > 65535) return IREE_UK_B200_UNSUPPORTED;
    if (ti.es == 1) transpose_kn_kernel<1><<<grid, 256, 0, stream>>>(rhs, rhs_pitch_b, rhs_t, l.pitch, K, N);
    else transpose_kn_kernel<2><<<grid, 256, 0, stream>>>(rhs, rhs_pitch_b, rhs_t, l.pitch, K, N);
    if (cudaGetLastError() != cudaSuccess) return IREE_UK_B200_CUDA_ERROR;
  }
  const char* a_ptr = lhs;
  int64_t a_pitch = lhs_pitch_b;
  if ((reinterpret_cast<uintptr_t>(lhs) & 15) || (lhs_pitch_b & 15)) {
    if (cudaMemcpy2DAsync(lhs_copy, size_t(l.pitch), lhs, size_t(lhs_pitch_b), size_t(K * ti.es),
                          size_t(M), cudaMemcpyDeviceToDevice, stream) != cudaSuccess)
      return IREE_UK_B200_CUDA_ERROR;
    a_ptr = lhs_copy;
    a_pitch = l.pitch;
  }

  TcParams P;
  std::memset(&P, 0, sizeof P);
  const int kblk_elems = 128 / ti.es;
  // tile counts in units of the 16-row tiles the schedulers reason in
  const int64_t M1 = (M + 15) / 16, N1 = (N + 15) / 16;
  const bool want_pair = M >= 256 && N >= 128 && ((M + 255) / 256) * ((N + 127) / 128) >= 74;
  bool pair = false;
  int pair_clusters = 0, bn = pick_bn(M1, N1), kboxes = 1;
  if (want_pair) {
    pair_clusters = di->pair_clusters[ti.is_int ? 1 : 0][0];
    if (pair_clusters >= 1) {
      pair = true;
      kboxes = 2;
      bn = pick_bn_pair(M1, N1, pair_clusters, false);  // the fused matmul cuts no tail tiles
    }
  }
  if (b_direct) {
    // whole 64-column swizzle atoms per CTA: 128 or 256 columns per CTA pair, 64..256 per CTA
    if (pair) {
      const int64_t mt = (M + 255) / 256;
      auto cost = [&](int w) {
        const int64_t tiles = mt * ((N + w - 1) / w);
        return ((tiles + pair_clusters - 1) / pair_clusters) * (w + 96);
      };
      bn = cost(128) < cost(256) ? 128 : 256;
    } else {
      bn = N > 128 ? 256 : (N > 64 ? 128 : 64);
    }
  }
  const int b_rows = pair ? bn / 2 : bn;  // RHS rows (output columns) one CTA stages
  const int tile_m = pair ? 2 * BM : BM;
  const uint64_t da[3] = {uint64_t(K), uint64_t(M), 1};
  const uint64_t sa[2] = {uint64_t(a_pitch), uint64_t(a_pitch) * uint64_t(M)};
  const uint32_t ba[3] = {uint32_t(kblk_elems), BM, 1};
  if (!encode_map(&P.map_a, ti.tm_type, const_cast<char*>(a_ptr), da, sa, ba, CU_TENSOR_MAP_SWIZZLE_128B))
    return IREE_UK_B200_CUDA_ERROR;
  P.sa = {kboxes, BM * 128, {kboxes * kblk_elems, 0, 0}, {0, tile_m, 0}, {kblk_elems, 0, 0}, {0, BM, 0}};
  P.desc_hi_a = P.desc_hi_b = desc_hi(1024, 2);
  P.desc_lbo_a = P.desc_lbo_b = 1;
  P.kadv_a = P.kadv_b = 2;
  P.kbox_units_a = uint32_t(BM * 128) >> 4;
  P.idesc = make_idesc(ti, bn, false, tile_m);
  if (b_direct) {
    // [K][N] as it lies: boxes of 64 columns (one 128-byte swizzle row) x all K rows of a stage.
    // In shared memory a box is [k][64 columns]; 8 K rows form one 1 KB swizzle atom (stride
    // byte offset), the next 64 columns are the next box (leading byte offset).
    const int stage_rows = kboxes * kblk_elems;
    const uint64_t db[3] = {uint64_t(N), uint64_t(K), 1};
    const uint64_t sb[2] = {uint64_t(rhs_pitch_b), uint64_t(rhs_pitch_b) * uint64_t(K)};
    const uint32_t bb[3] = {64, uint32_t(stage_rows), 1};
    if (!encode_map(&P.map_b, ti.tm_type, const_cast<char*>(rhs), db, sb, bb, CU_TENSOR_MAP_SWIZZLE_128B))
      return IREE_UK_B200_CUDA_ERROR;
    const int box_bytes = stage_rows * 128;
    P.sb = {b_rows / 64, box_bytes, {0, stage_rows, 0}, {bn, 0, 0}, {64, 0, 0}, {b_rows, 0, 0}};
    P.desc_lbo_b = uint32_t(box_bytes) >> 4;
    P.kadv_b = (16 * 128) >> 4;                 // 16 K rows per MMA
    P.kbox_units_b = (kblk_elems * 128) >> 4;   // K rows covered by one K box of the LHS
    P.idesc |= 1u << 16;                        // B is MN-major
  } else {
    const uint64_t db[3] = {uint64_t(K), uint64_t(N), 1};
    const uint64_t sb[2] = {uint64_t(l.pitch), uint64_t(l.pitch) * uint64_t(N)};
    const uint32_t bb[3] = {uint32_t(kblk_elems), uint32_t(b_rows), 1};
    if (!encode_map(&P.map_b, ti.tm_type, rhs_t, db, sb, bb, CU_TENSOR_MAP_SWIZZLE_128B))
      return IREE_UK_B200_CUDA_ERROR;
    P.sb = {kboxes, b_rows * 128, {kboxes * kblk_elems, 0, 0}, {0, bn, 0}, {kblk_elems, 0, 0}, {0, b_rows, 0}};
    P.kbox_units_b = uint32_t(b_rows * 128) >> 4;
  }
  P.kboxes = kboxes;
  P.mma_per_box = 4;
  P.stage_bytes_a = kboxes * BM * 128;
  P.stage_bytes_b = kboxes * b_rows * 128;
  P.num_kb = int((K + kboxes * kblk_elems - 1) / (kboxes * kblk_elems));
  P.bn = bn;
  P.m_tiles = int((M + tile_m - 1) / tile_m);
  P.n_tiles = int((N + bn - 1) / bn);
  P.num_work = P.tail_first = P.m_tiles * P.n_tiles;
  P.tail_split = 1;
  P.group_m = std::min(P.m_tiles, pair ? 8 : 16);
  P.out = out;
  P.out_stride0 = out_stride0;
  P.M1 = M1;
  P.N1 = N1;
  P.rows = M;
  P.cols = N;
  P.out_row_major = 1;
  P.out_vec16 = ((reinterpret_cast<uintptr_t>(out) & 15) == 0 && (out_stride0 * 4) % 16 == 0) ? 1 : 0;
  P.out_vec32 = ((reinterpret_cast<uintptr_t>(out) & 31) == 0 && (out_stride0 * 4) % 32 == 0) ? 1 : 0;
  P.accumulate = (flags & IREE_UK_FLAG_MMT4D_ACCUMULATE) ? 1 : 0;
  P.out_is_int = ti.is_int ? 1 : 0;
  P.status = status;
  set_wait_policy(&P);
  const int stage_bytes = P.stage_bytes_a + P.stage_bytes_b;
  P.num_stages = std::max(2, std::min(kMaxStages, 200 * 1024 / stage_bytes));
  const size_t smem = size_t(P.num_stages) * stage_bytes + 1024;
  if (tev) KernelTiming::record(tev[1], stream);
  cudaError_t e;
  if (pair) {
    const int grid = 2 * std::min(P.m_tiles * P.n_tiles, pair_clusters);
    e = launch_main(pair_kernel(ti.is_int, 0), grid, 2, smem, stream, P);
  } else {
    const int grid = std::min(P.m_tiles * P.n_tiles, di->sms);
    e = ti.is_int ? launch_main(mmt4d_tc_kernel<true>, grid, 1, smem, stream, P)
                  : launch_main(mmt4d_tc_kernel<false>, grid, 1, smem, stream, P);
  }
  if (e != cudaSuccess) return IREE_UK_B200_CUDA_ERROR;
  if (tev) {
    KernelTiming::record(tev[2], stream);
    timing->calls.fetch_add(1, std::memory_order_relaxed);
  }
  return cuda_status(cudaGetLastError());
}

}  // namespace uk

