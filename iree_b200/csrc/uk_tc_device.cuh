// Device-side building blocks of the tensor-core mmt4d kernels (sm_100a): the kernel parameter
// block, PTX wrappers (mbarrier, TMA, tcgen05, TMEM, bulk copies, programmatic dependent
// launch), the epilogues that move TMEM accumulators to the output, and the routines that issue
// one stage's TMA loads and tcgen05.mma instructions. Included by uk_mmt4d_tc.cu only.
#ifndef IREE_UK_B200_CSRC_UK_TC_DEVICE_CUH_
#define IREE_UK_B200_CSRC_UK_TC_DEVICE_CUH_

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdint>
#include <type_traits>

#include "uk_common.h"

namespace uk {
namespace {


constexpr int kMaxStages = 8;
constexpr int kThreads = 192;
constexpr long long kWaitCycles = 1ll << 31;  // ~1.1 s at 1.9 GHz
constexpr int BM = 128;

struct OperandStage {
  int32_t nbox;       // TMA boxes per stage
  int32_t box_bytes;  // shared-memory bytes per box
  int32_t kstep[3];   // coordinate = kb*kstep + tile*tstep + box*bstep
  int32_t tstep[3];
  int32_t bstep[3];
  int32_t rstep[3];   // two-CTA kernel only: added once for the CTA of cluster rank 1
};

struct TcParams {
  CUtensorMap map_a;
  CUtensorMap map_b;
  CUtensorMap map_b_narrow;  // two-CTA kernel: the RHS with the box of a narrow tail tile
  int32_t num_work;          // work items (tiles, the tail ones counted tail_split times)
  int32_t tail_first;        // first narrow item = first tile of the tail (num_work when none)
  int32_t tail_split;        // narrow tiles per tail tile
  OperandStage sa, sb;
  uint32_t desc_hi_a, desc_hi_b;    // bits 32..63 of the shared-memory descriptors
  uint32_t desc_lbo_a, desc_lbo_b;  // leading byte offset >> 4
  uint32_t kadv_a, kadv_b;          // start-address advance per MMA along K, in 16-byte units
  uint32_t kbox_units_a, kbox_units_b;  // 16-byte units between the K boxes of one stage
  uint32_t idesc;
  uint32_t idesc2;      // dual-LHS mode: instruction descriptor of the second (low-byte) MMA
  int32_t dual;         // two LHS planes (signed high / unsigned low bytes) per stage:
                        // 1 = s16u4s32 (row-major output, M0 = 1), 2 = s16s8s32 (16x16 output tiles)
  int32_t quad;         // s16s16s32: two byte planes of both operands, four MMAs per K slice
  int32_t acc_bufs;     // accumulator buffers in TMEM: 2 (epilogue overlaps the next tile), or 1
  int32_t kboxes;       // K boxes per stage (1 or 2)
  int32_t mma_per_box;  // tcgen05.mma per K box
  int32_t stage_bytes_a, stage_bytes_b;
  int32_t num_stages;
  int32_t num_kb;
  int32_t m_tiles, n_tiles, group_m;
  int32_t bn;  // accumulator columns per CTA tile
  char* out;
  int64_t out_stride0;  // elements
  int64_t M1, N1;
  int32_t accumulate;
  int32_t out_is_int;
  int32_t out_vec32;     // output rows may be accessed with 32-byte vectors
  // scratch-free kernel: the operands as they lie, [tile][K1][16][K0]
  const char* src_a;
  const char* src_b;
  int64_t src_stride_a, src_stride_b;  // bytes between tile rows
  int64_t K1;
  // streamed LHS pre-pass (two-CTA kernel): what the kernel's own worker warps re-tile, from
  // src_a above into the scratch that map_a describes
  char* rt_dst_a;
  int64_t rt_pitch;        // row pitch of the scratch, bytes
  uint32_t* rt_sync;       // [0]: job cursor; [1 + r]: jobs done for LHS tile row r
  int64_t rt_a_first;      // first LHS tile row that the workers re-tile
  uint32_t rt_jobs;        // jobs in all
  int32_t rt_kchunks;      // jobs per tile row
  int32_t triple;        // f32 operands as hi/lo tf32 planes, three MMAs per K slice
  int32_t out16;         // 0: 32-bit output; 1: f16 output, 2: bf16 output (rounded once, RNE)
  int32_t use_multicast; // output tiles are stored through an NVLink multicast mapping
  int64_t mc_delta;      // byte distance from `out` to that mapping
  int32_t staged_epilogue;  // local output through shared memory and 1 KB bulk copies too
  int32_t num_peers;     // copies of every output tile also stored to this many peer buffers
  int64_t peer_delta[IREE_UK_B200_MAX_PEERS];  // byte distance from `out` to each peer's buffer
  int32_t out_row_major; // fused matmul: the output is a row-major rows x cols matrix
  int32_t out_vec16;     // row-major output rows may be accessed with 16-byte vectors
  int64_t rows, cols;    // extent of the row-major output
  int32_t starve;        // test hook: the producers never fill a stage, so the bounded waits run out
  int64_t wait_cycles;   // clock64 ticks a device-side wait may take before it gives up
  uint32_t* status;
};

// ---------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// One lane of a converged warp. The surrounding code stays warp-uniform, so descriptors,
// coordinates and barrier addresses can live in uniform registers, which is what the TMA and
// tcgen05 instructions take.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "elect.sync _|p, 0xFFFFFFFF;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait. False when the deadline passed or another role already aborted.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          long long limit) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long deadline = clock64() + limit;
  while (!mbar_try_wait(bar, parity)) {
    if (*abort_flag || clock64() > deadline) return false;
  }
  return true;
}

// The same wait executed by a whole converged warp with one shared verdict.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                               long long limit) {
  return __all_sync(0xFFFFFFFFu, mbar_wait(bar, parity, abort_flag, limit));
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot),
               "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
               : "memory");
}
// Programmatic dependent launch. A pre-pass kernel calls pdl_launch_dependents() at its start:
// the main kernel that follows it in the stream may then be scheduled while the pre-pass's last
// blocks still run, and overlaps its own set-up (barriers, TMEM allocation) with them. Every
// thread of a main kernel calls pdl_wait() after that set-up and before it touches global
// memory: it returns once the preceding kernel has completed and its writes are visible.
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
template <bool IS_INT>
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                       uint32_t idesc, uint32_t accumulate) {
  if (IS_INT) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
// mbarrier arrives once all tcgen05.mma issued so far by this thread have completed.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
// ---- two-CTA (cta_group::2) forms -------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n"
               "barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of the same shared-memory variable in the CTA of rank `rank` of this cluster.
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}
// Raises the abort flag of this CTA and of its peer in the pair, so that every role of both
// CTAs leaves its loop at its next bounded wait instead of running its own wait out. The peer
// cannot have exited: it leaves only through the cluster barrier that this CTA has not reached.
__device__ __forceinline__ void raise_abort_pair(int* flag, uint32_t rank) {
  *reinterpret_cast<volatile int*>(flag) = 1;
  const uint32_t remote = mapa_shared(smem_u32(flag), rank ^ 1u);
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(remote), "r"(1) : "memory");
}
// TMA load of one CTA of a pair; the completion bytes go to the mbarrier at `bar`, a
// shared::cluster address that may belong to the peer CTA. No multicast.
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                                 int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot),
               "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
               : "memory");
}
// kind::tf32: 32-bit operands of which the tensor core uses sign, exponent and 10 mantissa bits.
template <bool PAIR>
__device__ __forceinline__ void tc_mma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                            uint32_t idesc, uint32_t accumulate) {
  if (PAIR) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}

template <bool IS_INT>
__device__ __forceinline__ void tc_mma_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                            uint32_t idesc, uint32_t accumulate) {
  if (IS_INT) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
// Arrives on the mbarrier at the same shared-memory offset in every CTA of `cta_mask` once all
// tcgen05.mma issued so far by this thread (for both CTAs of the pair) have completed.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
      "[%0], %1;" ::"r"(bar), "h"(cta_mask)
      : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tile_coords(const TcParams& P, int tile, int* mt, int* nt) {
  const int per_group = P.group_m * P.n_tiles;
  const int g = tile / per_group, r = tile - g * per_group;
  const int gm = min(P.group_m, P.m_tiles - g * P.group_m);
  *nt = r / gm;
  *mt = g * P.group_m + (r - *nt * gm);
}

// Work items of the two-CTA kernel. Items [0, tail_first) are whole tiles in schedule order.
// When the tile count is not a multiple of the number of CTA pairs, the tiles of the last,
// partial round are cut along N into tail_split narrower tiles each (items tail_first and up),
// so that the round keeps every pair busy for a fraction of a tile's time instead of a few
// pairs for a whole one.
struct WorkItem {
  int mt, nt;    // tile coordinates
  int col0;      // first output column, in elements
  int width;     // accumulator columns of this item (bn, or bn / tail_split)
  bool narrow;
};
__device__ __forceinline__ WorkItem work_item(const TcParams& P, int w) {
  WorkItem it;
  int tile = w, part = 0;
  it.width = P.bn;
  it.narrow = w >= P.tail_first;
  if (it.narrow) {
    const int r = w - P.tail_first;
    tile = P.tail_first + r / P.tail_split;
    part = r - (tile - P.tail_first) * P.tail_split;
    it.width = P.bn / P.tail_split;
  }
  tile_coords(P, tile, &it.mt, &it.nt);
  it.col0 = it.nt * P.bn + part * it.width;
  return it;
}

enum : uint32_t {
  kStatusProducerTimeout = 1u << 0,
  kStatusMmaTimeout = 1u << 1,
  kStatusEpilogueTimeout = 1u << 2,
  kStatusDrainTimeout = 1u << 3,
  // bits 4 and 5: the weight-streaming GEMV and the pack bulk-row wait (other files)
  kStatusRetileTimeout = 1u << 6,  // rows re-tiled by the kernel's own workers never became ready
};

__device__ __forceinline__ void st_global_v8(void* p, const uint32_t* r) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(r[0]),
               "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
__device__ __forceinline__ void ld_global_v8(const void* p, uint32_t (&r)[8]) {
  asm volatile("ld.global.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
                 "=r"(r[7])
               : "l"(p)
               : "memory");
}

// Row-major output (fused matmul): lane owns output row `row`, `chunks` groups of 16 columns
// from column col0. Whole, aligned groups use 16-byte accesses; ragged or unaligned ones are
// written element by element, never past `cols`. All 32 lanes must call this.
__device__ __forceinline__ void epilogue_rows_rowmajor(const TcParams& P, uint32_t taddr0,
                                                       int64_t row, int64_t col0, int chunks) {
  for (int c = 0; c < chunks; ++c) {
    uint32_t r[16];
    tmem_ld16(taddr0 + uint32_t(c * 16), r);
    tmem_ld_wait();
    const int64_t col = col0 + c * 16;
    if (row >= P.rows || col >= P.cols) continue;
    uint32_t* dst = reinterpret_cast<uint32_t*>(P.out) + row * P.out_stride0 + col;
    if (P.out_vec32 && !P.accumulate && col + 16 <= P.cols) {
      // write-only, 32-byte aligned rows: two whole-sector stores
      st_global_v8(dst, &r[0]);
      st_global_v8(dst + 8, &r[8]);
    } else if (P.out_vec16 && col + 16 <= P.cols) {
      uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        if (P.accumulate) {
          const uint4 old = d4[v];
          const uint32_t o[4] = {old.x, old.y, old.z, old.w};
#pragma unroll
          for (int j = 0; j < 4; ++j)
            r[4 * v + j] = P.out_is_int
                               ? r[4 * v + j] + o[j]
                               : __float_as_uint(__uint_as_float(r[4 * v + j]) + __uint_as_float(o[j]));
        }
        d4[v] = make_uint4(r[4 * v + 0], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        if (col + j < P.cols) {
          uint32_t v = r[j];
          if (P.accumulate)
            v = P.out_is_int ? v + dst[j]
                             : __float_as_uint(__uint_as_float(v) + __uint_as_float(dst[j]));
          dst[j] = v;
        }
      }
    }
  }
}

// Bulk copy of `bytes` (a multiple of 16) from this CTA's shared memory to global memory,
// which may be a peer GPU's; completion is tracked by the issuing thread's bulk groups.
__device__ __forceinline__ void bulk_store(void* gdst, uint32_t ssrc, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               :: "l"(gdst), "r"(ssrc), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" :: "n"(N) : "memory");
}

constexpr int kEpiStageBytes = 4096;  // per epilogue warp: two buffers of 32 rows x 64 bytes

// Epilogue through shared memory, with or without peer copies: the warp's 32 rows x 16 columns (two whole 16x16 output tiles of
// 1 KB each) are staged in shared memory and leave as 1 KB bulk copies, one per tile and
// destination: the local output and every peer buffer. Whole-tile writes are what NVLink
// carries efficiently; 32-byte stores from registers reach a fraction of the link rate.
// `stage` is this warp's kEpiStageBytes of shared memory. All 32 lanes must call this.
__device__ __forceinline__ void epilogue_rows_peers(const TcParams& P, uint32_t taddr0,
                                                    int64_t row, int64_t n1_0, int chunks,
                                                    uint32_t stage, int lane) {
  const int64_t m1 = row >> 4;
  const int m0 = int(row & 15);
  const int64_t m1_first = (row - lane) >> 4;  // lanes 0-15: this tile row, 16-31: the next
  const int copies = 2 * (1 + P.num_peers);    // (tile of the pair) x (destination)
  for (int c = 0; c < chunks; ++c) {
    uint32_t r[16];
    tmem_ld16(taddr0 + uint32_t(c * 16), r);
    tmem_ld_wait();
    const int64_t n1 = n1_0 + c;
    if (P.accumulate && m1 < P.M1 && n1 < P.N1) {
      const uint4* d4 = reinterpret_cast<const uint4*>(
          P.out + (m1 * P.out_stride0 + n1 * 256 + m0 * 16) * 4);
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        const uint4 old = d4[v];
        const uint32_t o[4] = {old.x, old.y, old.z, old.w};
#pragma unroll
        for (int j = 0; j < 4; ++j)
          r[4 * v + j] = P.out_is_int
                             ? r[4 * v + j] + o[j]
                             : __float_as_uint(__uint_as_float(r[4 * v + j]) + __uint_as_float(o[j]));
      }
    }
    const uint32_t buf = stage + uint32_t(c & 1) * 2048u;
    bulk_wait_read<1>();  // the copies that read this buffer two chunks ago are done with it
    __syncwarp();
#pragma unroll
    for (int v = 0; v < 4; ++v)
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                   :: "r"(buf + uint32_t(lane) * 64u + uint32_t(v) * 16u), "r"(r[4 * v + 0]),
                      "r"(r[4 * v + 1]), "r"(r[4 * v + 2]), "r"(r[4 * v + 3]) : "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
    if (n1 < P.N1) {
      for (int j = lane; j < copies; j += 32) {
        const int t = j & 1, g = (j >> 1) - 1;  // g = -1: the local output
        if (m1_first + t < P.M1) {
          char* dst = P.out + ((m1_first + t) * P.out_stride0 + n1 * 256) * 4;
          if (g >= 0) dst += P.peer_delta[g];
          bulk_store(dst, buf + uint32_t(t) * 1024u, 1024u);
        }
      }
    }
    bulk_commit();
  }
  bulk_wait_read<0>();  // shared memory is reused by the next tile, or released at exit
  __syncwarp();
}

// Epilogue through an NVLink multicast mapping: one multimem.st reaches the output buffer of
// every GPU bound to the mapping (this one included), replicated by the switch, so the result
// leaves this GPU once instead of once per peer. The warp's 32 rows x 16 columns are staged in
// shared memory and read back so that each store instruction covers 512 contiguous bytes of
// an output tile. All 32 lanes must call this.
__device__ __forceinline__ void epilogue_rows_multicast(const TcParams& P, uint32_t taddr0,
                                                        int64_t row, int64_t n1_0, int chunks,
                                                        uint32_t stage, int lane) {
  const int64_t m1 = row >> 4;
  const int m0 = int(row & 15);
  const int64_t m1_first = (row - lane) >> 4;
  for (int c = 0; c < chunks; ++c) {
    uint32_t r[16];
    tmem_ld16(taddr0 + uint32_t(c * 16), r);
    tmem_ld_wait();
    const int64_t n1 = n1_0 + c;
    if (P.accumulate && m1 < P.M1 && n1 < P.N1) {
      const uint4* d4 = reinterpret_cast<const uint4*>(
          P.out + (m1 * P.out_stride0 + n1 * 256 + m0 * 16) * 4);
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        const uint4 old = d4[v];
        const uint32_t o[4] = {old.x, old.y, old.z, old.w};
#pragma unroll
        for (int j = 0; j < 4; ++j)
          r[4 * v + j] = P.out_is_int
                             ? r[4 * v + j] + o[j]
                             : __float_as_uint(__uint_as_float(r[4 * v + j]) + __uint_as_float(o[j]));
      }
    }
    __syncwarp();  // the previous chunk has been read out of the staging buffer
#pragma unroll
    for (int v = 0; v < 4; ++v)
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                   :: "r"(stage + uint32_t(lane) * 64u + uint32_t(v) * 16u), "r"(r[4 * v + 0]),
                      "r"(r[4 * v + 1]), "r"(r[4 * v + 2]), "r"(r[4 * v + 3]) : "memory");
    __syncwarp();
    if (n1 < P.N1) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {  // 4 x 512 bytes = the two 1 KB tiles
        const int t = i >> 1;
        if (m1_first + t < P.M1) {
          float x, y, z, w;
          asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                       : "=f"(x), "=f"(y), "=f"(z), "=f"(w)
                       : "r"(stage + uint32_t(i) * 512u + uint32_t(lane) * 16u) : "memory");
          char* dst = P.out + P.mc_delta + ((m1_first + t) * P.out_stride0 + n1 * 256) * 4 +
                      (i & 1) * 512 + lane * 16;
          asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                       :: "l"(dst), "f"(x), "f"(y), "f"(z), "f"(w) : "memory");
        }
      }
    }
  }
  __syncwarp();
}

// 16-bit output (f16f16f16 / bf16bf16bf16 with one final rounding): lane owns row (m1, m0) of
// 16x16 tiles of 512 bytes; its 16 values of a tile are one 32-byte row.
__device__ __forceinline__ uint32_t pack_out16(float lo, float hi, int kind) {
  if (kind == 1) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
  const __nv_bfloat162 b = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&b);
}
__device__ __forceinline__ float2 unpack_out16(uint32_t v, int kind) {
  if (kind == 1) return __half22float2(*reinterpret_cast<const __half2*>(&v));
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v));
}
__device__ __forceinline__ void epilogue_rows_out16(const TcParams& P, uint32_t taddr0, int64_t row,
                                                    int64_t n1_0, int chunks) {
  const int64_t m1 = row >> 4;
  const int m0 = int(row & 15);
  for (int c = 0; c < chunks; ++c) {
    uint32_t r[16];
    tmem_ld16(taddr0 + uint32_t(c * 16), r);
    tmem_ld_wait();
    const int64_t n1 = n1_0 + c;
    if (m1 < P.M1 && n1 < P.N1) {
      uint4* d4 = reinterpret_cast<uint4*>(P.out + (m1 * P.out_stride0 + n1 * 256 + m0 * 16) * 2);
      uint32_t w[8];
      if (P.accumulate) {
        const uint4 o0 = d4[0], o1 = d4[1];
        const uint32_t o[8] = {o0.x, o0.y, o0.z, o0.w, o1.x, o1.y, o1.z, o1.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float2 old = unpack_out16(o[j], P.out16);
          w[j] = pack_out16(__uint_as_float(r[2 * j]) + old.x, __uint_as_float(r[2 * j + 1]) + old.y,
                            P.out16);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          w[j] = pack_out16(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]), P.out16);
      }
      d4[0] = make_uint4(w[0], w[1], w[2], w[3]);
      d4[1] = make_uint4(w[4], w[5], w[6], w[7]);
    }
  }
}

// Epilogue of one accumulator tile for one warp: lanes own rows row0 .. row0+31 of the output
// (row = m1*16 + m0), `chunks` groups of 16 columns starting at tile column n1_0. Each thread
// moves one 64-byte row of a 16x16 output tile per chunk. All 32 lanes must call this.
__device__ __forceinline__ void epilogue_rows(const TcParams& P, uint32_t taddr0, int64_t row,
                                              int64_t n1_0, int chunks, uint32_t epi_stage,
                                              int lane) {
  if (P.use_multicast) {
    epilogue_rows_multicast(P, taddr0, row, n1_0, chunks, epi_stage, lane);
    return;
  }
  if (P.num_peers || P.staged_epilogue) {
    epilogue_rows_peers(P, taddr0, row, n1_0, chunks, epi_stage, lane);
    return;
  }
  if (P.out16) {
    epilogue_rows_out16(P, taddr0, row, n1_0, chunks);
    return;
  }
  if (P.out_row_major) {
    epilogue_rows_rowmajor(P, taddr0, row, n1_0 * 16, chunks);
    return;
  }
  const int64_t m1 = row >> 4;
  const int m0 = int(row & 15);
  for (int c = 0; c < chunks; ++c) {
    uint32_t r[16];
    tmem_ld16(taddr0 + uint32_t(c * 16), r);
    tmem_ld_wait();
    const int64_t n1 = n1_0 + c;
    if (m1 < P.M1 && n1 < P.N1) {
      char* dst = P.out + (m1 * P.out_stride0 + n1 * 256 + m0 * 16) * 4;
      if (P.out_vec32) {
        // 32-byte accesses: every store fills a whole 32-byte sector.
        if (P.accumulate) {
#pragma unroll
          for (int v = 0; v < 2; ++v) {
            uint32_t o[8];
            ld_global_v8(dst + 32 * v, o);
#pragma unroll
            for (int j = 0; j < 8; ++j)
              r[8 * v + j] = P.out_is_int
                                 ? r[8 * v + j] + o[j]
                                 : __float_as_uint(__uint_as_float(r[8 * v + j]) + __uint_as_float(o[j]));
          }
        }
        st_global_v8(dst, &r[0]);
        st_global_v8(dst + 32, &r[8]);
      } else {
        uint4* d4 = reinterpret_cast<uint4*>(dst);
        if (P.accumulate) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const uint4 old = d4[v];
            const uint32_t o[4] = {old.x, old.y, old.z, old.w};
#pragma unroll
            for (int j = 0; j < 4; ++j)
              r[4 * v + j] = P.out_is_int
                                 ? r[4 * v + j] + o[j]
                                 : __float_as_uint(__uint_as_float(r[4 * v + j]) + __uint_as_float(o[j]));
          }
        }
#pragma unroll
        for (int v = 0; v < 4; ++v)
          d4[v] = make_uint4(r[4 * v + 0], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
      }
    }
  }
}

// Epilogue of the dual-LHS mode: the output is row-major (M0 = 1): lane owns output row `row`,
// `chunks` groups of 16 columns starting at column col0; value = (hi << 8) + lo (+ old).
__device__ __forceinline__ void epilogue_rows_dual(const TcParams& P, uint32_t taddr_hi,
                                                   uint32_t taddr_lo, int64_t row, int64_t col0,
                                                   int chunks) {
  const int64_t ncols = P.N1 * 32;
  for (int c = 0; c < chunks; ++c) {
    uint32_t h[16], r[16];
    tmem_ld16(taddr_hi + uint32_t(c * 16), h);
    tmem_ld16(taddr_lo + uint32_t(c * 16), r);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 16; ++j) r[j] += h[j] << 8;
    const int64_t col = col0 + c * 16;
    if (row < P.M1 && col < ncols) {
      uint4* d4 = reinterpret_cast<uint4*>(P.out + (row * P.out_stride0 + col) * 4);
      if (P.accumulate) {
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          const uint4 old = d4[v];
          r[4 * v + 0] += old.x; r[4 * v + 1] += old.y; r[4 * v + 2] += old.z; r[4 * v + 3] += old.w;
        }
      }
#pragma unroll
      for (int v = 0; v < 4; ++v)
        d4[v] = make_uint4(r[4 * v + 0], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
    }
  }
}

// Epilogue of the dual-LHS mode with 16x16 output tiles (s16s8s32): two accumulators of `bn`
// columns (high byte plane, low byte plane); value = (hi << 8) + lo (+ old) modulo 2^32.
__device__ __forceinline__ void epilogue_rows_dual_tiled(const TcParams& P, uint32_t taddr_hi,
                                                         int64_t row, int64_t n1_0, int chunks) {
  const int64_t m1 = row >> 4;
  const int m0 = int(row & 15);
  for (int c = 0; c < chunks; ++c) {
    uint32_t h[16], r[16];
    tmem_ld16(taddr_hi + uint32_t(c * 16), h);
    tmem_ld16(taddr_hi + uint32_t(P.bn) + uint32_t(c * 16), r);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 16; ++j) r[j] += h[j] << 8;
    const int64_t n1 = n1_0 + c;
    if (m1 < P.M1 && n1 < P.N1) {
      uint4* d4 = reinterpret_cast<uint4*>(P.out + (m1 * P.out_stride0 + n1 * 256 + m0 * 16) * 4);
      if (P.accumulate) {
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          const uint4 old = d4[v];
          r[4 * v + 0] += old.x; r[4 * v + 1] += old.y; r[4 * v + 2] += old.z; r[4 * v + 3] += old.w;
        }
      }
#pragma unroll
      for (int v = 0; v < 4; ++v)
        d4[v] = make_uint4(r[4 * v + 0], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
    }
  }
}

// Epilogue of the four-product mode (s16s16s32, 16x16 tiles): three accumulators of `bn` columns
// (high x high, the two cross products, low x low); value = (hh << 16) + (cross << 8) + ll
// (+ old), all modulo 2^32 like the reference's int32 arithmetic.
__device__ __forceinline__ void epilogue_rows_quad(const TcParams& P, uint32_t taddr_hh, int64_t row,
                                                   int64_t n1_0, int chunks) {
  const int64_t m1 = row >> 4;
  const int m0 = int(row & 15);
  const uint32_t bn = uint32_t(P.bn);
  for (int c = 0; c < chunks; ++c) {
    uint32_t r[16], x[16];
    tmem_ld16(taddr_hh + uint32_t(c * 16), r);
    tmem_ld16(taddr_hh + bn + uint32_t(c * 16), x);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 16; ++j) r[j] = (r[j] << 16) + (x[j] << 8);
    tmem_ld16(taddr_hh + 2u * bn + uint32_t(c * 16), x);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 16; ++j) r[j] += x[j];
    const int64_t n1 = n1_0 + c;
    if (m1 < P.M1 && n1 < P.N1) {
      uint4* d4 = reinterpret_cast<uint4*>(P.out + (m1 * P.out_stride0 + n1 * 256 + m0 * 16) * 4);
      if (P.accumulate) {
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          const uint4 old = d4[v];
          r[4 * v + 0] += old.x; r[4 * v + 1] += old.y; r[4 * v + 2] += old.z; r[4 * v + 3] += old.w;
        }
      }
#pragma unroll
      for (int v = 0; v < 4; ++v)
        d4[v] = make_uint4(r[4 * v + 0], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
    }
  }
}

// One stage's TMA loads for one operand. `c` holds the coordinates of box 0 for this k-block.
template <bool PAIR>
__device__ __forceinline__ void issue_operand_loads(const CUtensorMap* map, const OperandStage& st,
                                                    uint32_t smem, uint32_t bar, const int (&c)[3]) {
  for (int b = 0; b < st.nbox; ++b) {
    const uint32_t dst = smem + uint32_t(b * st.box_bytes);
    const int c0 = c[0] + b * st.bstep[0], c1 = c[1] + b * st.bstep[1], c2 = c[2] + b * st.bstep[2];
    if (PAIR) tma_load_3d_pair(dst, map, bar, c0, c1, c2);
    else tma_load_3d(dst, map, bar, c0, c1, c2);
  }
}

// All tcgen05.mma of one stage. Everything but the two stage addresses is loop-invariant and
// lives in registers of the single issuing thread.
struct MmaIssue {
  uint32_t lo_a, lo_b, hi_a, hi_b, kadv_a, kadv_b, kbox_a, kbox_b, idesc, idesc2;
  int kboxes, mma_per_box, dual, triple, quad;
};
__device__ __forceinline__ MmaIssue make_mma_issue(const TcParams& P) {
  MmaIssue m;
  m.lo_a = P.desc_lbo_a << 16; m.lo_b = P.desc_lbo_b << 16;
  m.hi_a = P.desc_hi_a; m.hi_b = P.desc_hi_b;
  m.kadv_a = P.kadv_a; m.kadv_b = P.kadv_b;
  m.kbox_a = P.kbox_units_a; m.kbox_b = P.kbox_units_b;
  m.idesc = P.idesc; m.kboxes = P.kboxes; m.mma_per_box = P.mma_per_box;
  m.idesc2 = P.idesc2; m.dual = P.dual; m.triple = P.triple; m.quad = P.quad;
  return m;
}
// Dual-LHS stage (s16u4s32): shared memory holds [high-byte plane | low-byte plane | RHS]; each K
// slice feeds two MMAs that share the RHS descriptor and accumulate into two TMEM regions
// (d_tmem and d_tmem + bn), recombined as hi*256 + lo by the epilogue.
template <bool PAIR>
__device__ __forceinline__ void issue_stage_mmas_dual(const MmaIssue& m, uint32_t d_hi, uint32_t d_lo,
                                                      uint32_t a_units, uint32_t b_units,
                                                      bool first_kblock) {
  uint32_t acc = first_kblock ? 0u : 1u;
  uint32_t au = a_units, bu = b_units;
  for (int j = 0; j < m.mma_per_box; ++j) {
    const uint64_t da_hi = (uint64_t(m.hi_a) << 32) | uint64_t((au & 0x3FFFu) | m.lo_a);
    const uint64_t da_lo = (uint64_t(m.hi_a) << 32) | uint64_t(((au + m.kbox_a) & 0x3FFFu) | m.lo_a);
    const uint64_t db = (uint64_t(m.hi_b) << 32) | uint64_t((bu & 0x3FFFu) | m.lo_b);
    if (PAIR) {
      tc_mma_pair<true>(d_hi, da_hi, db, m.idesc, acc);
      tc_mma_pair<true>(d_lo, da_lo, db, m.idesc2, acc);
    } else {
      tc_mma<true>(d_hi, da_hi, db, m.idesc, acc);
      tc_mma<true>(d_lo, da_lo, db, m.idesc2, acc);
    }
    acc = 1u;
    au += m.kadv_a;
    bu += m.kadv_b;
  }
}

// Four-product stage (s16s16s32): shared memory holds [high | low] byte planes of both operands
// (x = 256 * hi + lo with hi the signed high byte and lo the unsigned low byte). Each K slice
// feeds hi*hi into d, hi*lo and lo*hi into d + bn, lo*lo into d + 2 bn; m.idesc carries neither
// operand's sign bit (bit 7: A signed, bit 10: B signed).
template <bool PAIR>
__device__ __forceinline__ void issue_stage_mmas_quad(const MmaIssue& m, uint32_t d, uint32_t bn,
                                                      uint32_t a_units, uint32_t b_units,
                                                      bool first_kblock) {
  uint32_t acc = first_kblock ? 0u : 1u;
  uint32_t au = a_units, bu = b_units;
  const uint32_t a_signed = 1u << 7, b_signed = 1u << 10;
  for (int j = 0; j < m.mma_per_box; ++j) {
    const uint64_t a_hi = (uint64_t(m.hi_a) << 32) | uint64_t((au & 0x3FFFu) | m.lo_a);
    const uint64_t a_lo = (uint64_t(m.hi_a) << 32) | uint64_t(((au + m.kbox_a) & 0x3FFFu) | m.lo_a);
    const uint64_t b_hi = (uint64_t(m.hi_b) << 32) | uint64_t((bu & 0x3FFFu) | m.lo_b);
    const uint64_t b_lo = (uint64_t(m.hi_b) << 32) | uint64_t(((bu + m.kbox_b) & 0x3FFFu) | m.lo_b);
    if (PAIR) {
      tc_mma_pair<true>(d, a_hi, b_hi, m.idesc | a_signed | b_signed, acc);
      tc_mma_pair<true>(d + bn, a_hi, b_lo, m.idesc | a_signed, acc);
      tc_mma_pair<true>(d + bn, a_lo, b_hi, m.idesc | b_signed, 1u);
      tc_mma_pair<true>(d + 2u * bn, a_lo, b_lo, m.idesc, acc);
    } else {
      tc_mma<true>(d, a_hi, b_hi, m.idesc | a_signed | b_signed, acc);
      tc_mma<true>(d + bn, a_hi, b_lo, m.idesc | a_signed, acc);
      tc_mma<true>(d + bn, a_lo, b_hi, m.idesc | b_signed, 1u);
      tc_mma<true>(d + 2u * bn, a_lo, b_lo, m.idesc, acc);
    }
    acc = 1u;
    au += m.kadv_a;
    bu += m.kadv_b;
  }
}

template <bool IS_INT, bool PAIR>
__device__ __forceinline__ void issue_stage_mmas(const MmaIssue& m, uint32_t d_tmem, uint32_t a_units,
                                                 uint32_t b_units, bool first_kblock) {
  uint32_t acc = first_kblock ? 0u : 1u;
  if (!IS_INT && m.triple) {
    // f32 as three tf32 products: shared memory holds [hi plane | lo plane] of each operand
    // (x = hi + lo, hi = the tf32 part); hi*hi + lo*hi + hi*lo, the lo*lo term is below f32's
    // own rounding error. Small terms first.
    uint32_t au = a_units, bu = b_units;
    for (int j = 0; j < m.mma_per_box; ++j) {
      const uint64_t a_hi = (uint64_t(m.hi_a) << 32) | uint64_t((au & 0x3FFFu) | m.lo_a);
      const uint64_t a_lo = (uint64_t(m.hi_a) << 32) | uint64_t(((au + m.kbox_a) & 0x3FFFu) | m.lo_a);
      const uint64_t b_hi = (uint64_t(m.hi_b) << 32) | uint64_t((bu & 0x3FFFu) | m.lo_b);
      const uint64_t b_lo = (uint64_t(m.hi_b) << 32) | uint64_t(((bu + m.kbox_b) & 0x3FFFu) | m.lo_b);
      tc_mma_tf32<PAIR>(d_tmem, a_lo, b_hi, m.idesc, acc);
      tc_mma_tf32<PAIR>(d_tmem, a_hi, b_lo, m.idesc, 1u);
      tc_mma_tf32<PAIR>(d_tmem, a_hi, b_hi, m.idesc, 1u);
      acc = 1u;
      au += m.kadv_a;
      bu += m.kadv_b;
    }
    return;
  }
  for (int kb = 0; kb < m.kboxes; ++kb) {
    uint32_t au = a_units + uint32_t(kb) * m.kbox_a, bu = b_units + uint32_t(kb) * m.kbox_b;
    for (int j = 0; j < m.mma_per_box; ++j) {
      const uint64_t da = (uint64_t(m.hi_a) << 32) | uint64_t((au & 0x3FFFu) | m.lo_a);
      const uint64_t db = (uint64_t(m.hi_b) << 32) | uint64_t((bu & 0x3FFFu) | m.lo_b);
      if (PAIR) tc_mma_pair<IS_INT>(d_tmem, da, db, m.idesc, acc);
      else tc_mma<IS_INT>(d_tmem, da, db, m.idesc, acc);
      acc = 1u;
      au += m.kadv_a;
      bu += m.kadv_b;
    }
  }
}


}  // namespace
}  // namespace uk

#endif  // IREE_UK_B200_CSRC_UK_TC_DEVICE_CUH_
