// mmt4d on the 5th-generation tensor cores (sm_100a): TMA -> shared memory -> tcgen05.mma
// -> TMEM -> tcgen05.ld -> [M1][N1][16][16] output tiles.
//
// One persistent, warp-specialised kernel serves s8s8s32 (kind::i8), f16f16f32 and
// bf16bf16f32 (kind::f16) with M0 = N0 = 16:
//
//   warp 0      TMA producer: one elected lane issues cp.async.bulk.tensor loads (never
//               with cluster multicast) into a ring of shared-memory stages
//   warp 1      MMA issuer: one elected lane issues tcgen05.mma (M = 128, N = BN <= 256)
//               into one of two TMEM accumulator buffers; also owns TMEM alloc / dealloc
//   warps 2..5  epilogue: tcgen05.ld 32 lanes x 16 columns -> one 64-byte row of one
//               16x16 output tile per thread (+ the old tile when ACCUMULATE) -> st.global
//
// The CTA tile is 128 rows (8 LHS tile rows) x BN columns (BN/16 RHS tile rows). Tiles are
// walked in a grouped order so that the CTAs of one wave share LHS / RHS panels in L2.
//
// How the operands reach shared memory is described by runtime parameters (tensor maps,
// box coordinates, shared-memory descriptor fields), not by the kernel body. "Variants":
//   0  K-major, SWIZZLE_128B: both operands are first re-tiled by retile_kernel from the
//      mmt4d panel layout [tile][K1][16][K0] into row-major [row][K] scratch; this is the
//      canonical tcgen05 layout and works for every K0
//   1..4  MN-major, read directly from a K0 = 1, 16-bit mmt4d operand ([tile][K1][16] is
//      already "16 contiguous M/N elements per k"); 1/2 use 128-byte swizzle with four
//      tile rows side by side, 3/4 use 32-byte swizzle; even numbers swap the roles of the
//      descriptor's two byte offsets. Experimental until validated on hardware.
//
// Every wait on an mbarrier is bounded (clock64 deadline). A wait that runs out records a
// code in the per-device status word, raises a CTA-wide abort flag, and all roles leave
// their loops; the producer then waits (bounded) for its own copies in flight, TMEM is
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
  OperandStage sa, sb;
  uint32_t desc_hi_a, desc_hi_b;    // bits 32..63 of the shared-memory descriptors
  uint32_t desc_lbo_a, desc_lbo_b;  // leading byte offset >> 4
  uint32_t kadv_a, kadv_b;          // start-address advance per MMA along K, in 16-byte units
  uint32_t kbox_units_a, kbox_units_b;  // 16-byte units between the K boxes of one stage
  uint32_t idesc;
  uint32_t idesc2;      // dual-LHS mode: instruction descriptor of the second (low-byte) MMA
  int32_t dual;         // s16u4s32: two LHS planes (signed high / unsigned low bytes) per stage
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
  int32_t triple;        // f32 operands as hi/lo tf32 planes, three MMAs per K slice
  int32_t out16;         // 0: 32-bit output; 1: f16 output, 2: bf16 output (rounded once, RNE)
  int32_t use_multicast; // output tiles are stored through an NVLink multicast mapping
  int64_t mc_delta;      // byte distance from `out` to that mapping
  int32_t num_peers;     // copies of every output tile also stored to this many peer buffers
  int64_t peer_delta[IREE_UK_B200_MAX_PEERS];  // byte distance from `out` to each peer's buffer
  int32_t out_row_major; // fused matmul: the output is a row-major rows x cols matrix
  int32_t out_vec16;     // row-major output rows may be accessed with 16-byte vectors
  int64_t rows, cols;    // extent of the row-major output
  uint32_t debug_flags;  // experiments only: 1 = no output stores, 2 = no TMEM reads, 4 = no TMA
                         // loads, 8 = the producer never fills a stage (exercises the bounded waits)
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
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long deadline = clock64() + kWaitCycles;
  while (!mbar_try_wait(bar, parity)) {
    if (*abort_flag || clock64() > deadline) return false;
  }
  return true;
}

// The same wait executed by a whole converged warp with one shared verdict.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  return __all_sync(0xFFFFFFFFu, mbar_wait(bar, parity, abort_flag));
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

enum : uint32_t {
  kStatusProducerTimeout = 1u << 0,
  kStatusMmaTimeout = 1u << 1,
  kStatusEpilogueTimeout = 1u << 2,
  kStatusDrainTimeout = 1u << 3,
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
    if (row >= P.rows || col >= P.cols || (P.debug_flags & 1u)) continue;
    uint32_t* dst = reinterpret_cast<uint32_t*>(P.out) + row * P.out_stride0 + col;
    if (P.out_vec16 && col + 16 <= P.cols) {
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

// Epilogue with peer copies: the warp's 32 rows x 16 columns (two whole 16x16 output tiles of
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
    if (n1 < P.N1 && !(P.debug_flags & 1u)) {
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
    if (n1 < P.N1 && !(P.debug_flags & 1u)) {
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
    if (m1 < P.M1 && n1 < P.N1 && !(P.debug_flags & 1u)) {
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
  if (P.debug_flags & 2u) return;
  if (P.use_multicast) {
    epilogue_rows_multicast(P, taddr0, row, n1_0, chunks, epi_stage, lane);
    return;
  }
  if (P.num_peers) {
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
    if (m1 < P.M1 && n1 < P.N1 && !(P.debug_flags & 1u)) {
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
  if (P.debug_flags & 2u) return;
  const int64_t ncols = P.N1 * 32;
  for (int c = 0; c < chunks; ++c) {
    uint32_t h[16], r[16];
    tmem_ld16(taddr_hi + uint32_t(c * 16), h);
    tmem_ld16(taddr_lo + uint32_t(c * 16), r);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 16; ++j) r[j] += h[j] << 8;
    const int64_t col = col0 + c * 16;
    if (row < P.M1 && col < ncols && !(P.debug_flags & 1u)) {
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
  int kboxes, mma_per_box, dual, triple;
};
__device__ __forceinline__ MmaIssue make_mma_issue(const TcParams& P) {
  MmaIssue m;
  m.lo_a = P.desc_lbo_a << 16; m.lo_b = P.desc_lbo_b << 16;
  m.hi_a = P.desc_hi_a; m.hi_b = P.desc_hi_b;
  m.kadv_a = P.kadv_a; m.kadv_b = P.kadv_b;
  m.kbox_a = P.kbox_units_a; m.kbox_b = P.kbox_units_b;
  m.idesc = P.idesc; m.kboxes = P.kboxes; m.mma_per_box = P.mma_per_box;
  m.idesc2 = P.idesc2; m.dual = P.dual; m.triple = P.triple;
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

// ---------------------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------------------
template <bool IS_INT>
__global__ void __launch_bounds__(kThreads, 1) mmt4d_tc_kernel(const __grid_constant__ TcParams P) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kMaxStages];
  __shared__ __align__(8) uint64_t empty_bar[kMaxStages];
  __shared__ __align__(8) uint64_t tmem_full_bar[2];
  __shared__ __align__(8) uint64_t tmem_empty_bar[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t stage_base = (smem_u32(smem_raw) + 1023u) & ~1023u;  // swizzle atoms: 1 KB
  const uint32_t stage_bytes = uint32_t(P.stage_bytes_a + P.stage_bytes_b);
  const int S = P.num_stages;
  const int num_tiles = P.m_tiles * P.n_tiles;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&tmem_full_bar[b]), 1);
      mbar_init(smem_u32(&tmem_empty_bar[b]), 4);  // one arrive per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  volatile int* abortp = &abort_flag;
  pdl_wait();

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------
    {
      int stage = 0;
      uint32_t phase = 0;
      long long issued = 0;
      bool ok = true;
      const OperandStage sa_st = P.sa, sb_st = P.sb;
      const int num_kb = P.num_kb;
      const uint32_t a_bytes = uint32_t(P.stage_bytes_a);
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int mt, nt;
        tile_coords(P, tile, &mt, &nt);
        int ca[3] = {mt * sa_st.tstep[0], mt * sa_st.tstep[1], mt * sa_st.tstep[2]};
        int cb[3] = {nt * sb_st.tstep[0], nt * sb_st.tstep[1], nt * sb_st.tstep[2]};
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_warp(smem_u32(&empty_bar[stage]), phase ^ 1u, abortp)) {
            if (lane == 0) atomicOr(P.status, kStatusProducerTimeout);
            abort_flag = 1;
            ok = false;
            break;
          }
          const uint32_t bar = smem_u32(&full_bar[stage]);
          const uint32_t sa = stage_base + uint32_t(stage) * stage_bytes;
          const bool starve = (P.debug_flags & 8u) != 0;  // test hook: nothing ever arrives
          if (!starve && elect_one()) {
            if (P.debug_flags & 4u) {
              mbar_arrive(bar);
            } else {
              mbar_expect_tx(bar, stage_bytes);
              issue_operand_loads<false>(&P.map_a, sa_st, sa, bar, ca);
              issue_operand_loads<false>(&P.map_b, sb_st, sa + a_bytes, bar, cb);
            }
          }
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 3; ++i) { ca[i] += sa_st.kstep[i]; cb[i] += sb_st.kstep[i]; }
          if (!starve) ++issued;
          if (++stage == S) { stage = 0; phase ^= 1u; }
        }
      }
      if ((!ok || *abortp) && lane == 0) {
        // Aborting: let this CTA's own copies land before its shared memory is released.
        const long long n = issued < S ? issued : S;
        for (long long i = 0; i < n; ++i) {
          const long long idx = issued - 1 - i;
          const int s = int(idx % S);
          const uint32_t par = uint32_t((idx / S) & 1);
          const long long deadline = clock64() + kWaitCycles;
          while (!mbar_try_wait(smem_u32(&full_bar[s]), par)) {
            if (clock64() > deadline) { atomicOr(P.status, kStatusDrainTimeout); break; }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    {
      int stage = 0;
      uint32_t phase = 0;
      int buf = 0;
      uint32_t buf_phase = 0;
      bool ok = true;
      const MmaIssue mi = make_mma_issue(P);
      const uint32_t a_bytes = uint32_t(P.stage_bytes_a);
      const int num_kb = P.num_kb;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait_warp(smem_u32(&tmem_empty_bar[buf]), buf_phase ^ 1u, abortp)) {
          if (lane == 0) atomicOr(P.status, kStatusMmaTimeout);
          abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + uint32_t(buf * P.bn * (mi.dual ? 2 : 1));
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_warp(smem_u32(&full_bar[stage]), phase, abortp)) {
            if (lane == 0) atomicOr(P.status, kStatusMmaTimeout);
            abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = stage_base + uint32_t(stage) * stage_bytes;
          if (elect_one()) {
            if (IS_INT && mi.dual)
              issue_stage_mmas_dual<false>(mi, d_tmem, d_tmem + uint32_t(P.bn), sa >> 4, (sa + a_bytes) >> 4, kb == 0);
            else
              issue_stage_mmas<IS_INT, false>(mi, d_tmem, sa >> 4, (sa + a_bytes) >> 4, kb == 0);
            tc_commit(smem_u32(&empty_bar[stage]));  // stage reusable once these MMAs finish
            if (kb == num_kb - 1) tc_commit(smem_u32(&tmem_full_bar[buf]));  // accumulator complete
          }
          __syncwarp();
          if (++stage == S) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        if (++buf == 2) { buf = 0; buf_phase ^= 1u; }
      }
    }
  } else {
    // ------------------------------- epilogue -------------------------------
    const int q = warp & 3;  // TMEM lane quadrant this warp may read
    const int m_local = q * 32 + lane;
    const uint32_t epi_stage = stage_base + uint32_t(S) * stage_bytes + uint32_t(q) * kEpiStageBytes;
    int buf = 0;
    uint32_t buf_phase = 0;
    const int chunks = P.bn >> 4;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      int mt, nt;
      tile_coords(P, tile, &mt, &nt);
      // Warp-uniform outcome: tcgen05.ld below needs all 32 lanes.
      if (!__all_sync(0xFFFFFFFFu, mbar_wait(smem_u32(&tmem_full_bar[buf]), buf_phase, abortp))) {
        if (lane == 0) atomicOr(P.status, kStatusEpilogueTimeout);
        abort_flag = 1;
        break;
      }
      tc_fence_after();
      const int64_t row = int64_t(mt) * BM + m_local;
      if (P.dual) {
        const uint32_t t_hi = tmem_base + (uint32_t(q * 32) << 16) + uint32_t(buf * 2 * P.bn);
        epilogue_rows_dual(P, t_hi, t_hi + uint32_t(P.bn), row, int64_t(nt) * P.bn, chunks);
      } else {
        const uint32_t taddr0 = tmem_base + (uint32_t(q * 32) << 16) + uint32_t(buf * P.bn);
        epilogue_rows(P, taddr0, row, int64_t(nt) * chunks, chunks, epi_stage, lane);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&tmem_empty_bar[buf]));
      if (++buf == 2) { buf = 0; buf_phase ^= 1u; }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------------------
// the scratch-free kernel: operands re-tiled on the way into shared memory
// ---------------------------------------------------------------------------------------
// Same MMA and epilogue roles as mmt4d_tc_kernel, but the stages are filled by four producer
// warps instead of TMA: a mmt4d operand [tile][K1][16][K0] holds, for one tile and the K range
// of one stage (128 bytes per row), exactly 2 KB of contiguous memory; the producers read it
// with 16-byte loads and scatter the G = K0 * element-size byte granules to their places in the
// K-major 128-byte-swizzled stage (row = m0, 16-byte chunk index XOR (row & 7)). No pre-pass and
// no scratch: this is what a call without a workspace gets. The shared-memory stores cost issue
// slots and bandwidth the TMA form does not spend, so with a workspace the TMA kernels are used.
constexpr int kSwGroups = 3;                       // producer groups of 4 warps; group g fills stages g, g+3, ...
constexpr int kSwProducerWarps = 4 * kSwGroups;    // warps 0..11
constexpr int kSwMmaWarp = kSwProducerWarps + 4;   // warps 12..15 epilogue, 16 MMA issuer
constexpr int kSwThreads = (kSwMmaWarp + 1) * 32;

template <int G>
__device__ __forceinline__ void st_granule(uint32_t addr, const uint32_t (&v)[4], int i) {
  // granule i of the 16-byte vector v (G bytes each)
  if (G == 16) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" :: "r"(addr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]) : "memory");
  } else if (G == 8) {
    asm volatile("st.shared.v2.b32 [%0], {%1, %2};" :: "r"(addr), "r"(v[2 * i]), "r"(v[2 * i + 1]) : "memory");
  } else if (G == 4) {
    asm volatile("st.shared.b32 [%0], %1;" :: "r"(addr), "r"(v[i]) : "memory");
  } else if (G == 2) {
    const uint32_t w = v[i >> 1] >> ((i & 1) * 16);
    asm volatile("st.shared.b16 [%0], %1;" :: "r"(addr), "h"(uint16_t(w)) : "memory");
  } else {
    const uint32_t w = v[i >> 2] >> ((i & 3) * 8);
    asm volatile("st.shared.b8 [%0], %1;" :: "r"(addr), "r"(w & 0xFFu) : "memory");
  }
}

// One stage: BM/16 LHS tiles then bn/16 RHS tiles, each 16 rows x 128 bytes of K (k1 steps
// [k1_0, k1_0 + 128/G)). Thread t of a group's 128 owns vector t of every tile's 2 KB; the loads
// of the next batch of tiles are issued before the current batch is stored, so one global-memory
// latency is exposed per stage, not one per batch.
// Which of a tile's 128 vectors (k1 step, group of 16/G rows) thread t of a producer group
// owns. The natural order (t = k1 * G + group) makes lanes of a warp whose rows agree in
// (row & 7) store to the same banks in the same step for 2- and 4-byte granules; these orders
// give every lane of a warp its own bank (lanes that share a 32-bit word merge):
//   G = 4: a warp takes 16 k1 steps x 2 neighbouring row groups (rows r and r + 4),
//   G = 2: a warp takes 32 k1 steps x 1 row group.
template <int G>
__device__ __forceinline__ void sw_vector_of_thread(int t, int* k1_local, int* sub) {
  const int w = t >> 5, l = t & 31;
  if (G == 4) {
    *sub = (l & 1) + 2 * (w & 1);
    *k1_local = (l >> 1) + 16 * (w >> 1);
  } else if (G == 2) {
    *sub = w & 1;
    *k1_local = l + 32 * (w >> 1);
  } else {
    *k1_local = t / G;
    *sub = t - *k1_local * G;
  }
}

struct SwStageSrc {
  const char* a;      // LHS tile row of the first tile, at k1_0
  const char* b;      // RHS likewise
  int64_t stride_a, stride_b;
  int a_valid, b_valid;  // tiles that exist (the rest of the stage keeps stale rows nobody reads)
};

// `n` tiles of one operand (n <= 8) from `p` (first tile, this thread's vector), `stride` bytes
// apart, the first `valid` of which exist; `off[i]` is the shared-memory offset of granule i
// inside a tile's 2 KB of rows.
template <int G>
__device__ __forceinline__ void sw_load_batch(uint4 (&v)[8], const char* p, int64_t stride, int n,
                                              int valid, bool k_ok) {
#pragma unroll
  for (int b = 0; b < 8; ++b) {
    const bool ok = k_ok && b < n && b < valid;
    v[b] = ok ? __ldg(reinterpret_cast<const uint4*>(p + int64_t(b) * stride)) : make_uint4(0u, 0u, 0u, 0u);
  }
}
template <int G>
__device__ __forceinline__ void sw_store_batch(const uint4 (&v)[8], int n, uint32_t smem,
                                               const uint32_t (&off)[16 / G]) {
#pragma unroll
  for (int b = 0; b < 8; ++b) {
    if (b < n) {
      const uint32_t w[4] = {v[b].x, v[b].y, v[b].z, v[b].w};
#pragma unroll
      for (int i = 0; i < 16 / G; ++i) st_granule<G>(smem + uint32_t(b) * 2048u + off[i], w, i);
    }
  }
}

template <int G>
__device__ __forceinline__ void sw_fill_stage(const SwStageSrc& src, int a_tiles, int b_tiles,
                                              bool k_ok, uint32_t smem, int t) {
  constexpr int RPV = 16 / G;            // rows covered by one 16-byte vector
  int k1_local, sub;
  sw_vector_of_thread<G>(t, &k1_local, &sub);
  const int vec = k1_local * G + sub;    // index of this thread's vector in a tile's 2 KB
  const uint32_t col = uint32_t(k1_local * G);
  const uint32_t chunk = col >> 4, within = col & 15u;
  uint32_t off[RPV];
#pragma unroll
  for (int i = 0; i < RPV; ++i) {
    const uint32_t row = uint32_t(sub * RPV + i);
    off[i] = row * 128u + ((chunk ^ (row & 7u)) << 4) + within;
  }
  // LHS tiles (a_tiles = 8) are one batch, RHS tiles (b_tiles <= 16) up to two; the next batch
  // is loaded before the current one is stored.
  const char* pa = src.a + vec * 16;
  const char* pb = src.b + vec * 16;
  uint4 v0[8], v1[8];
  sw_load_batch<G>(v0, pa, src.stride_a, a_tiles, src.a_valid, k_ok);
  sw_load_batch<G>(v1, pb, src.stride_b, b_tiles, src.b_valid, k_ok);
  sw_store_batch<G>(v0, a_tiles, smem, off);
  const uint32_t smem_b = smem + uint32_t(a_tiles) * 2048u;
  if (b_tiles > 8)
    sw_load_batch<G>(v0, pb + 8 * src.stride_b, src.stride_b, b_tiles - 8, src.b_valid - 8, k_ok);
  sw_store_batch<G>(v1, b_tiles, smem_b, off);
  if (b_tiles > 8) sw_store_batch<G>(v0, b_tiles - 8, smem_b + 8u * 2048u, off);
}

template <bool IS_INT, int G>
__global__ void __launch_bounds__(kSwThreads, 1) mmt4d_tc_sw_kernel(const __grid_constant__ TcParams P) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kMaxStages];
  __shared__ __align__(8) uint64_t empty_bar[kMaxStages];
  __shared__ __align__(8) uint64_t tmem_full_bar[2];
  __shared__ __align__(8) uint64_t tmem_empty_bar[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t stage_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t stage_bytes = uint32_t(P.stage_bytes_a + P.stage_bytes_b);
  const int S = P.num_stages;
  const int num_tiles = P.m_tiles * P.n_tiles;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 128);  // every thread of the filling group arrives
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&tmem_full_bar[b]), 1);
      mbar_init(smem_u32(&tmem_empty_bar[b]), 4);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == kSwMmaWarp) {
    tmem_alloc(smem_u32(&tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  volatile int* abortp = &abort_flag;
  pdl_wait();

  if (warp < kSwProducerWarps) {
    // ------------------------------- producers -------------------------------
    // Group g (four warps) fills every kSwGroups-th stage of the running sequence of k-blocks, so
    // up to kSwGroups stages are being fetched at the same time.
    const int group = warp >> 2;
    const int t = threadIdx.x & 127;
    bool ok = true;
    const int num_kb = P.num_kb;
    constexpr int kps = 128 / G;  // k1 steps per stage
    const int b_tiles = P.bn >> 4;
    long long seq = 0;            // k-blocks since the start of the kernel, over all tiles
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int mt, nt;
      tile_coords(P, tile, &mt, &nt);
      const int64_t a0 = int64_t(mt) * (BM / 16), b0 = int64_t(nt) * b_tiles;
      for (int kb = 0; kb < num_kb; ++kb, ++seq) {
        if (int(seq % kSwGroups) != group) continue;
        const int stage = int(seq % S);
        const uint32_t phase = uint32_t((seq / S) & 1);
        if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1u, abortp)) {
          atomicOr(P.status, kStatusProducerTimeout);
          abort_flag = 1;
          ok = false;
          break;
        }
        const uint32_t sa = stage_base + uint32_t(stage) * stage_bytes;
        if (!(P.debug_flags & 4u)) {
          const int64_t k1_0 = int64_t(kb) * kps;
          SwStageSrc src;
          src.a = P.src_a + a0 * P.src_stride_a + k1_0 * (16 * G);
          src.b = P.src_b + b0 * P.src_stride_b + k1_0 * (16 * G);
          src.stride_a = P.src_stride_a;
          src.stride_b = P.src_stride_b;
          src.a_valid = int(min(int64_t(BM / 16), P.M1 - a0));
          src.b_valid = int(min(int64_t(b_tiles), P.N1 - b0));
          int k1_local, sub;
          sw_vector_of_thread<G>(t, &k1_local, &sub);
          sw_fill_stage<G>(src, BM / 16, b_tiles, k1_0 + k1_local < P.K1, sa, t);
        }
        // make the generic-proxy stores visible to the tensor core (async proxy), then signal
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        if (!(P.debug_flags & 8u)) mbar_arrive(smem_u32(&full_bar[stage]));
      }
    }
  } else if (warp == kSwMmaWarp) {
    // ------------------------------- MMA issuer -------------------------------
    int stage = 0;
    uint32_t phase = 0;
    int buf = 0;
    uint32_t buf_phase = 0;
    bool ok = true;
    const MmaIssue mi = make_mma_issue(P);
    const uint32_t a_bytes = uint32_t(P.stage_bytes_a);
    const int num_kb = P.num_kb;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      if (!mbar_wait_warp(smem_u32(&tmem_empty_bar[buf]), buf_phase ^ 1u, abortp)) {
        if (lane == 0) atomicOr(P.status, kStatusMmaTimeout);
        abort_flag = 1;
        break;
      }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + uint32_t(buf * P.bn);
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!mbar_wait_warp(smem_u32(&full_bar[stage]), phase, abortp)) {
          if (lane == 0) atomicOr(P.status, kStatusMmaTimeout);
          abort_flag = 1;
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t sa = stage_base + uint32_t(stage) * stage_bytes;
        if (elect_one()) {
          issue_stage_mmas<IS_INT, false>(mi, d_tmem, sa >> 4, (sa + a_bytes) >> 4, kb == 0);
          tc_commit(smem_u32(&empty_bar[stage]));
          if (kb == num_kb - 1) tc_commit(smem_u32(&tmem_full_bar[buf]));
        }
        __syncwarp();
        if (++stage == S) { stage = 0; phase ^= 1u; }
      }
      if (!ok) break;
      if (++buf == 2) { buf = 0; buf_phase ^= 1u; }
    }
  } else {
    // ------------------------------- epilogue -------------------------------
    const int q = warp & 3;
    const int m_local = q * 32 + lane;
    const uint32_t epi_stage = stage_base + uint32_t(S) * stage_bytes + uint32_t(q) * kEpiStageBytes;
    int buf = 0;
    uint32_t buf_phase = 0;
    const int chunks = P.bn >> 4;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      int mt, nt;
      tile_coords(P, tile, &mt, &nt);
      if (!__all_sync(0xFFFFFFFFu, mbar_wait(smem_u32(&tmem_full_bar[buf]), buf_phase, abortp))) {
        if (lane == 0) atomicOr(P.status, kStatusEpilogueTimeout);
        abort_flag = 1;
        break;
      }
      tc_fence_after();
      const int64_t row = int64_t(mt) * BM + m_local;
      const uint32_t taddr0 = tmem_base + (uint32_t(q * 32) << 16) + uint32_t(buf * P.bn);
      epilogue_rows(P, taddr0, row, int64_t(nt) * chunks, chunks, epi_stage, lane);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&tmem_empty_bar[buf]));
      if (++buf == 2) { buf = 0; buf_phase ^= 1u; }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kSwMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------------------
// the two-CTA kernel (cta_group::2)
// ---------------------------------------------------------------------------------------
// A cluster of two CTAs on neighbouring SMs works on one 256 x BN tile. Each CTA stages its own
// 128 rows of the LHS and its own half (BN/2 rows) of the RHS, so a CTA moves 2/3 of the bytes
// per k-block that the one-CTA kernel moves for the same math; one tcgen05.mma issued by the
// leader (cluster rank 0) drives both SMs' tensor cores, reads the RHS halves from both CTAs'
// shared memory and accumulates 128 rows x BN columns in each CTA's TMEM. Barriers:
//   full[s]       leader's only; armed by the leader's producer with the bytes of both CTAs;
//                 both CTAs' TMA loads complete on it (the peer through a mapped address)
//   empty[s]      one per CTA; the leader's tcgen05.commit arrives on both (multicast commit)
//   tmem_full[b]  one per CTA; multicast commit after the last k-block of a tile
//   tmem_empty[b] leader's only, 8 arrivals: the four epilogue warps of each CTA
// No TMA load uses cluster multicast.
template <bool IS_INT>
__global__ void __launch_bounds__(kThreads, 1) mmt4d_tc2_kernel(const __grid_constant__ TcParams P) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kMaxStages];
  __shared__ __align__(8) uint64_t empty_bar[kMaxStages];
  __shared__ __align__(8) uint64_t tmem_full_bar[2];
  __shared__ __align__(8) uint64_t tmem_empty_bar[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const uint32_t stage_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t stage_bytes = uint32_t(P.stage_bytes_a + P.stage_bytes_b);  // per CTA
  const int S = P.num_stages;
  const int num_tiles = P.m_tiles * P.n_tiles;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&tmem_full_bar[b]), 1);
      mbar_init(smem_u32(&tmem_empty_bar[b]), 8);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(&tmem_slot), 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anything signals them remotely
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  volatile int* abortp = &abort_flag;
  pdl_wait();

  if (warp == 0) {
    // ------------------------------- TMA producer (both CTAs) -------------------------------
    {
      int stage = 0;
      uint32_t phase = 0;
      long long issued = 0;
      bool ok = true;
      const int r = int(rank);
      const OperandStage sa_st = P.sa, sb_st = P.sb;
      const int num_kb = P.num_kb;
      const uint32_t a_bytes = uint32_t(P.stage_bytes_a);
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        int mt, nt;
        tile_coords(P, tile, &mt, &nt);
        int ca[3], cb[3];
#pragma unroll
        for (int i = 0; i < 3; ++i) {
          ca[i] = mt * sa_st.tstep[i] + r * sa_st.rstep[i];
          cb[i] = nt * sb_st.tstep[i] + r * sb_st.rstep[i];
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_warp(smem_u32(&empty_bar[stage]), phase ^ 1u, abortp)) {
            if (lane == 0) atomicOr(P.status, kStatusProducerTimeout);
            abort_flag = 1;
            ok = false;
            break;
          }
          const uint32_t own_bar = smem_u32(&full_bar[stage]);
          const uint32_t bar = mapa_shared(own_bar, 0);
          const uint32_t sa = stage_base + uint32_t(stage) * stage_bytes;
          if (elect_one()) {
            if (P.debug_flags & 4u) {
              if (leader) mbar_arrive(own_bar);
            } else {
              if (leader) mbar_expect_tx(own_bar, 2u * stage_bytes);
              issue_operand_loads<true>(&P.map_a, sa_st, sa, bar, ca);
              issue_operand_loads<true>(&P.map_b, sb_st, sa + a_bytes, bar, cb);
            }
          }
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 3; ++i) { ca[i] += sa_st.kstep[i]; cb[i] += sb_st.kstep[i]; }
          ++issued;
          if (++stage == S) { stage = 0; phase ^= 1u; }
        }
      }
      if ((!ok || *abortp) && leader && lane == 0) {
        // Aborting: the leader's full barriers count the copies of both CTAs; let them land
        // before either CTA's shared memory is released (the cluster barrier below orders the
        // peer's exit after this).
        const long long n = issued < S ? issued : S;
        for (long long i = 0; i < n; ++i) {
          const long long idx = issued - 1 - i;
          const int s = int(idx % S);
          const uint32_t par = uint32_t((idx / S) & 1);
          const long long deadline = clock64() + kWaitCycles;
          while (!mbar_try_wait(smem_u32(&full_bar[s]), par)) {
            if (clock64() > deadline) { atomicOr(P.status, kStatusDrainTimeout); break; }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer (leader only) -------------------------------
    if (leader) {
      int stage = 0;
      uint32_t phase = 0;
      int buf = 0;
      uint32_t buf_phase = 0;
      bool ok = true;
      const MmaIssue mi = make_mma_issue(P);
      const uint32_t a_bytes = uint32_t(P.stage_bytes_a);
      const int num_kb = P.num_kb;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        if (!mbar_wait_warp(smem_u32(&tmem_empty_bar[buf]), buf_phase ^ 1u, abortp)) {
          if (lane == 0) atomicOr(P.status, kStatusMmaTimeout);
          abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + uint32_t(buf * P.bn * (mi.dual ? 2 : 1));
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_warp(smem_u32(&full_bar[stage]), phase, abortp)) {
            if (lane == 0) atomicOr(P.status, kStatusMmaTimeout);
            abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = stage_base + uint32_t(stage) * stage_bytes;
          if (elect_one()) {
            if (IS_INT && mi.dual)
              issue_stage_mmas_dual<true>(mi, d_tmem, d_tmem + uint32_t(P.bn), sa >> 4, (sa + a_bytes) >> 4, kb == 0);
            else
              issue_stage_mmas<IS_INT, true>(mi, d_tmem, sa >> 4, (sa + a_bytes) >> 4, kb == 0);
            tc_commit_pair(smem_u32(&empty_bar[stage]), 3);  // both CTAs may refill the stage
            if (kb == num_kb - 1) tc_commit_pair(smem_u32(&tmem_full_bar[buf]), 3);  // accumulators done
          }
          __syncwarp();
          if (++stage == S) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        if (++buf == 2) { buf = 0; buf_phase ^= 1u; }
      }
    }
  } else {
    // ------------------------------- epilogue (both CTAs) -------------------------------
    const int q = warp & 3;
    const uint32_t epi_stage = stage_base + uint32_t(S) * stage_bytes + uint32_t(q) * kEpiStageBytes;
    int buf = 0;
    uint32_t buf_phase = 0;
    const int chunks = P.bn >> 4;
    for (int tile = pair; tile < num_tiles; tile += num_pairs) {
      int mt, nt;
      tile_coords(P, tile, &mt, &nt);
      if (!__all_sync(0xFFFFFFFFu, mbar_wait(smem_u32(&tmem_full_bar[buf]), buf_phase, abortp))) {
        if (lane == 0) atomicOr(P.status, kStatusEpilogueTimeout);
        abort_flag = 1;
        break;
      }
      tc_fence_after();
      const int64_t row = int64_t(mt) * 256 + int64_t(rank) * 128 + q * 32 + lane;
      if (P.dual) {
        const uint32_t t_hi = tmem_base + (uint32_t(q * 32) << 16) + uint32_t(buf * 2 * P.bn);
        epilogue_rows_dual(P, t_hi, t_hi + uint32_t(P.bn), row, int64_t(nt) * P.bn, chunks);
      } else {
        const uint32_t taddr0 = tmem_base + (uint32_t(q * 32) << 16) + uint32_t(buf * P.bn);
        epilogue_rows(P, taddr0, row, int64_t(nt) * chunks, chunks, epi_stage, lane);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&tmem_empty_bar[buf]), 0));
      if (++buf == 2) { buf = 0; buf_phase ^= 1u; }
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA frees TMEM or exits while its peer may still touch it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------------------
// re-tile: mmt4d panels [tile][K1][16][K0] -> row-major [tile*16 + r][K1*K0] scratch
// ---------------------------------------------------------------------------------------
// G = K0 * element bytes is the granule that stays contiguous; per tile row the kernel
// transposes a [K1][16] matrix of granules into [16][K1]. A block moves 1024/G k1 steps of
// one tile row (16 KB) through shared memory: contiguous 16-byte loads, 16-byte stores of
// 1 KB row segments, four of each in flight per thread. The shared-memory pitch per k1 is 16*G + 4 bytes so that walking
// k1 at a fixed row is bank-conflict free.
struct RetileOperand {
  const char* src;       // first panel
  int64_t src_stride_b;  // bytes between panels (tile rows)
  char* dst;             // row-major scratch
  int64_t blocks;        // tile rows x k chunks
};

// Both operands of a mmt4d call in one launch: blocks [0, a.blocks) re-tile the LHS, the rest
// the RHS.
template <int G>
__global__ void __launch_bounds__(256) retile_kernel(RetileOperand opa, RetileOperand opb,
                                                     int64_t dst_pitch_b, int64_t K1, int kchunks) {
  pdl_launch_dependents();
  const bool is_a = int64_t(blockIdx.x) < opa.blocks;
  const char* __restrict__ src = is_a ? opa.src : opb.src;
  const int64_t src_stride_b = is_a ? opa.src_stride_b : opb.src_stride_b;
  char* __restrict__ dst = is_a ? opa.dst : opb.dst;
  const int64_t block = is_a ? int64_t(blockIdx.x) : int64_t(blockIdx.x) - opa.blocks;
  constexpr int KC = 1024 / G;            // k1 steps per block: 16 KB in, 16 rows x 1 KB out
  constexpr int PITCH = 16 * G + 4;       // bytes per k1 in shared memory
  constexpr int GV = 16 / G;              // granules per 16-byte vector
  __shared__ __align__(16) unsigned char sm[KC * PITCH];
  const int64_t tile = block / kchunks;
  const int chunk = int(block - tile * kchunks);
  const int64_t k_base = int64_t(chunk) * KC;
  const int kn = int(min(int64_t(KC), K1 - k_base));
  const char* sp = src + tile * src_stride_b + k_base * (16 * G);
  // load: kn * 16 granules contiguous = kn * G vectors of 16 bytes
  const int nvec = kn * G;
#pragma unroll 4
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    const uint4 x = __ldg(reinterpret_cast<const uint4*>(sp) + v);
    const int byte = v * 16;
    const int k = byte / (16 * G), within = byte - k * (16 * G);
    uint32_t* d = reinterpret_cast<uint32_t*>(sm + k * PITCH + within);
    d[0] = x.x; d[1] = x.y; d[2] = x.z; d[3] = x.w;
  }
  __syncthreads();
  // store: 16 rows x kn granules; a thread builds 16 bytes = GV consecutive k1 of one row
  if (G == 2) {
    // 2-byte granules: a 32-bit shared-memory word holds one k of two neighbouring rows, so a
    // thread reads 8 words (8 k) and emits the 16-byte vectors of both rows: half the
    // shared-memory loads of the one-row-at-a-time scheme below.
    const int full = kn / GV;  // whole vectors per row
    const int full8 = (full + 7) & ~7;
#pragma unroll 2
    for (int v = threadIdx.x; v < 8 * full8; v += blockDim.x) {
      const int rp = (v >> 3) & 7, kv = ((v >> 6) << 3) | (v & 7);
      if (kv >= full) continue;
      const int k0 = kv * GV;
      uint32_t x[8];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        x[j] = *reinterpret_cast<const uint32_t*>(sm + (k0 + j) * PITCH + rp * 4);
      uint4 even, odd;
      even.x = __byte_perm(x[0], x[1], 0x5410); odd.x = __byte_perm(x[0], x[1], 0x7632);
      even.y = __byte_perm(x[2], x[3], 0x5410); odd.y = __byte_perm(x[2], x[3], 0x7632);
      even.z = __byte_perm(x[4], x[5], 0x5410); odd.z = __byte_perm(x[4], x[5], 0x7632);
      even.w = __byte_perm(x[6], x[7], 0x5410); odd.w = __byte_perm(x[6], x[7], 0x7632);
      char* dp = dst + (tile * 16 + 2 * rp) * dst_pitch_b + (k_base + k0) * G;
      *reinterpret_cast<uint4*>(dp) = even;
      *reinterpret_cast<uint4*>(dp + dst_pitch_b) = odd;
    }
    const int rem = kn - full * GV;  // trailing k of a ragged last chunk
    for (int e = threadIdx.x; e < 16 * rem; e += blockDim.x) {
      const int r = e / rem, k = full * GV + (e - r * rem);
      *reinterpret_cast<uint16_t*>(dst + (tile * 16 + r) * dst_pitch_b + (k_base + k) * G) =
          *reinterpret_cast<const uint16_t*>(sm + k * PITCH + r * G);
    }
    return;
  }
  // Lane mapping: 8 consecutive vectors of a row (128 bytes), then the next row; keeps the
  // shared-memory reads spread over banks and the global stores in 128-byte pieces.
  const int vec_per_row = (kn + GV - 1) / GV;
  const int vec_per_row8 = (vec_per_row + 7) & ~7;
#pragma unroll 4
  for (int v = threadIdx.x; v < 16 * vec_per_row8; v += blockDim.x) {
    const int r = (v >> 3) & 15, kv = ((v >> 7) << 3) | (v & 7);
    if (kv >= vec_per_row) continue;
    const int k0 = kv * GV;
    char* dp = dst + (tile * 16 + r) * dst_pitch_b + (k_base + k0) * G;
    if (k0 + GV <= kn) {
      uint32_t w[4];
      if (G == 16) {
        const uint32_t* s = reinterpret_cast<const uint32_t*>(sm + k0 * PITCH + r * G);
        w[0] = s[0]; w[1] = s[1]; w[2] = s[2]; w[3] = s[3];
      } else if (G == 8) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const uint32_t* s = reinterpret_cast<const uint32_t*>(sm + (k0 + j) * PITCH + r * G);
          w[2 * j] = s[0]; w[2 * j + 1] = s[1];
        }
      } else if (G == 4) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          w[j] = *reinterpret_cast<const uint32_t*>(sm + (k0 + j) * PITCH + r * G);
      } else if (G == 2) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t lo = *reinterpret_cast<const uint16_t*>(sm + (k0 + 2 * j) * PITCH + r * G);
          const uint32_t hi = *reinterpret_cast<const uint16_t*>(sm + (k0 + 2 * j + 1) * PITCH + r * G);
          w[j] = lo | (hi << 16);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t x = 0;
#pragma unroll
          for (int b = 0; b < 4; ++b) x |= uint32_t(sm[(k0 + 4 * j + b) * PITCH + r * G]) << (8 * b);
          w[j] = x;
        }
      }
      *reinterpret_cast<uint4*>(dp) = make_uint4(w[0], w[1], w[2], w[3]);
    } else {
      for (int k = k0; k < kn; ++k)
        for (int b = 0; b < G; ++b) dp[(k - k0) * G + b] = char(sm[k * PITCH + r * G + b]);
    }
  }
}

int launch_retile(const char* lhs, int64_t lhs_stride_b, char* dst_a, int64_t tiles_a,
                  const char* rhs, int64_t rhs_stride_b, char* dst_b, int64_t tiles_b,
                  int64_t dst_pitch_b, int64_t K1, int G, cudaStream_t stream) {
  if (K1 <= 0 || tiles_a + tiles_b <= 0) return IREE_UK_B200_OK;
  const int KC = 1024 / G;
  const int64_t kchunks = (K1 + KC - 1) / KC;
  const RetileOperand a = {lhs, lhs_stride_b, dst_a, tiles_a * kchunks};
  const RetileOperand b = {rhs, rhs_stride_b, dst_b, tiles_b * kchunks};
  const int64_t blocks = a.blocks + b.blocks;
  if (blocks > 0x7FFFFFFF) return IREE_UK_B200_UNSUPPORTED;
  switch (G) {
    case 1: retile_kernel<1><<<int(blocks), 256, 0, stream>>>(a, b, dst_pitch_b, K1, int(kchunks)); break;
    case 2: retile_kernel<2><<<int(blocks), 256, 0, stream>>>(a, b, dst_pitch_b, K1, int(kchunks)); break;
    case 4: retile_kernel<4><<<int(blocks), 256, 0, stream>>>(a, b, dst_pitch_b, K1, int(kchunks)); break;
    case 8: retile_kernel<8><<<int(blocks), 256, 0, stream>>>(a, b, dst_pitch_b, K1, int(kchunks)); break;
    case 16: retile_kernel<16><<<int(blocks), 256, 0, stream>>>(a, b, dst_pitch_b, K1, int(kchunks)); break;
    default: return IREE_UK_B200_UNSUPPORTED;
  }
  return cuda_status(cudaGetLastError());
}

// ---------------------------------------------------------------------------------------
// s16u4s32 pre-pass: byte planes for the LHS, byte-wide row-major weights for the RHS
// ---------------------------------------------------------------------------------------
// x = hi*256 + lo exactly, with hi the signed high byte and lo the unsigned low byte of the
// s16, so sum(x*w) = 256*sum(hi*w) + sum(lo*w): two 8-bit tensor-core products. The LHS
// [M][K1][1][8] (row-major M x K s16) becomes two row-major byte planes.
__global__ void __launch_bounds__(256) split_s16_kernel(const char* __restrict__ lhs,
                                                        int64_t lhs_stride_b, char* __restrict__ hi,
                                                        char* __restrict__ lo, int64_t pitch_b,
                                                        int64_t M, int64_t K1) {
  const int64_t total = M * K1;
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < total;
       i += int64_t(gridDim.x) * blockDim.x) {
    const int64_t row = i / K1, k1 = i - row * K1;
    const uint4 x = __ldg(reinterpret_cast<const uint4*>(lhs + row * lhs_stride_b) + k1);
    const uint2 l = make_uint2(__byte_perm(x.x, x.y, 0x6420), __byte_perm(x.z, x.w, 0x6420));
    const uint2 h = make_uint2(__byte_perm(x.x, x.y, 0x7531), __byte_perm(x.z, x.w, 0x7531));
    *reinterpret_cast<uint2*>(lo + row * pitch_b + k1 * 8) = l;
    *reinterpret_cast<uint2*>(hi + row * pitch_b + k1 * 8) = h;
  }
}

// RHS [N1][K1][32][8 x u4] (tile = 128 bytes, low nibble = even k0) -> row-major u8
// [N1*32][K1*8]. A block widens 64 k1 steps of one tile row through shared memory: contiguous
// 16-byte loads, 16-byte stores of 512-byte row segments.
__global__ void __launch_bounds__(256) unpack_u4_kernel(const char* __restrict__ rhs,
                                                        int64_t rhs_stride_b, char* __restrict__ dst,
                                                        int64_t pitch_b, int64_t K1, int kchunks) {
  pdl_launch_dependents();
  constexpr int KC = 64, PITCH = KC * 8 + 16;
  __shared__ __align__(16) unsigned char sm[32 * PITCH];
  const int64_t n1 = blockIdx.x / kchunks;
  const int chunk = int(blockIdx.x - n1 * kchunks);
  const int64_t k_base = int64_t(chunk) * KC;
  const int kn = int(min(int64_t(KC), K1 - k_base));
  const uint4* src = reinterpret_cast<const uint4*>(rhs + n1 * rhs_stride_b + k_base * 128);
#pragma unroll 2
  for (int v = threadIdx.x; v < kn * 8; v += blockDim.x) {
    const int k = v >> 3, g = v & 7;
    const uint4 w = __ldg(src + v);
    const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const uint32_t even = ws[r] & 0x0F0F0F0Fu, odd = (ws[r] >> 4) & 0x0F0F0F0Fu;
      // bytes k0 = 0..7 in order: even0, odd0, even1, odd1, ...
      const uint2 o = make_uint2(__byte_perm(even, odd, 0x5140), __byte_perm(even, odd, 0x7362));
      *reinterpret_cast<uint2*>(sm + (4 * g + r) * PITCH + k * 8) = o;
    }
  }
  __syncthreads();
  const int row_bytes = kn * 8;
  const int vec_per_row = row_bytes / 16;
  for (int v = threadIdx.x; v < 32 * vec_per_row; v += blockDim.x) {
    const int n0 = v / vec_per_row, kv = v - n0 * vec_per_row;
    *reinterpret_cast<uint4*>(dst + (n1 * 32 + n0) * pitch_b + k_base * 8 + kv * 16) =
        *reinterpret_cast<const uint4*>(sm + n0 * PITCH + kv * 16);
  }
  if (row_bytes & 15) {  // odd number of k1 in the last chunk: the final 8 bytes of each row
    if (threadIdx.x < 32) {
      const int n0 = threadIdx.x;
      *reinterpret_cast<uint2*>(dst + (n1 * 32 + n0) * pitch_b + k_base * 8 + vec_per_row * 16) =
          *reinterpret_cast<const uint2*>(sm + n0 * PITCH + vec_per_row * 16);
    }
  }
}

// ---------------------------------------------------------------------------------------
// host side: tensor maps, descriptors, launch
// ---------------------------------------------------------------------------------------

// Experiment knobs, honoured only when IREE_UK_B200_DEBUG is set in the environment.
int debug_int(const char* name, int fallback) {
  static const bool enabled = std::getenv("IREE_UK_B200_DEBUG") != nullptr;
  if (!enabled) return fallback;
  const char* v = std::getenv(name);
  return v ? std::atoi(v) : fallback;
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

// Co-resident 2-CTA clusters of the pair kernel on the current device (0 on failure).
template <bool IS_INT>
int max_pair_clusters(size_t smem) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, mmt4d_tc2_kernel<IS_INT>, &cfg) != cudaSuccess) return 0;
  return n;
}

// What the launchers need to know about the current device, found once per device: the
// kernels' dynamic shared memory limit is raised to the device maximum at that point, so the
// per-call path makes no attribute or occupancy calls.
struct DeviceInfo {
  bool ok = false;
  int sms = 0;
  int max_smem = 0;           // dynamic shared memory per block the kernels may be launched with
  int pair_clusters[2] = {};  // co-resident CTA pairs of mmt4d_tc2_kernel<false / true>
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
    if (!raise_limit(reinterpret_cast<const void*>(mmt4d_tc_kernel<false>)) ||
        !raise_limit(reinterpret_cast<const void*>(mmt4d_tc_kernel<true>)) ||
        !raise_limit(reinterpret_cast<const void*>(mmt4d_tc2_kernel<false>)) ||
        !raise_limit(reinterpret_cast<const void*>(mmt4d_tc2_kernel<true>))) {
      cudaGetLastError();
      return nullptr;
    }
    d.max_smem = dyn_limit;
    const size_t smem_probe = size_t(6) * (BM * 128 + 128 * 128) + 1024;
    d.pair_clusters[0] = max_pair_clusters<false>(smem_probe);
    d.pair_clusters[1] = max_pair_clusters<true>(smem_probe);
    d.ok = true;
  }
  return &d;
}

// Accumulator width for the pair kernel: among the multiples of 32 columns up to 256, the one
// that minimises (waves of 256 x bn tiles over `clusters` pairs) x bn, i.e. the estimated time.
int pick_bn_pair(int64_t M1, int64_t N1, int clusters) {
  {
    const int bn = debug_int("IREE_UK_B200_DEBUG_PAIR_BN", 0);
    if (bn >= 32 && bn <= 256 && bn % 32 == 0) return bn;
  }
  const int64_t m_tiles = (M1 * 16 + 255) / 256, cols = N1 * 16;
  int best = 256;
  int64_t best_cost = -1;
  for (int bn = 256; bn >= 128; bn -= 32) {
    const int64_t tiles = m_tiles * ((cols + bn - 1) / bn);
    const int64_t waves = (tiles + clusters - 1) / clusters;
    const int64_t cost = waves * (bn + 32);  // tile time: the MMAs plus a small fixed part
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = bn; }
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
                        const TcParams& P) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned(grid), 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
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

int launch_mmt4d_tc_s16u4(const iree_uk_mmt4d_params_t* p, void* ws, size_t ws_bytes,
                          cudaStream_t stream) {
  if (!mmt4d_tc_s16u4_eligible(p)) return IREE_UK_B200_UNSUPPORTED;
  uint32_t* status = device_status_word();
  if (!status) return IREE_UK_B200_CUDA_ERROR;
  const S16U4Layout l = s16u4_layout(p);
  if (!ws || ws_bytes < size_t(2 * l.plane_bytes + l.w_bytes)) return IREE_UK_B200_WORKSPACE_TOO_SMALL;
  if (reinterpret_cast<uintptr_t>(ws) & 255) return IREE_UK_B200_INVALID_ARGUMENT;
  KernelTiming& timing = kernel_timing();
  cudaEvent_t* tev = timing.next_slot();
  if (tev) cudaEventRecord(tev[0], stream);

  const char* lhs = static_cast<const char*>(p->lhs_buffer) + p->lhs_offset * 2;
  const char* rhs = static_cast<const char*>(p->rhs_buffer) + p->rhs_offset / 2;
  char* hi = static_cast<char*>(ws);
  char* lo = hi + l.plane_bytes;
  char* w8 = lo + l.plane_bytes;
  {
    const int64_t total = p->M * p->K;
    const int64_t blocks = std::min<int64_t>((total + 255) / 256, 148 * 16);
    split_s16_kernel<<<int(blocks), 256, 0, stream>>>(lhs, p->lhs_stride0 * 2, hi, lo, l.pitch, p->M, p->K);
    const int64_t kchunks = (p->K + 63) / 64;
    if (p->N * kchunks > 0x7FFFFFFF) return IREE_UK_B200_UNSUPPORTED;
    unpack_u4_kernel<<<int(p->N * kchunks), 256, 0, stream>>>(rhs, p->rhs_stride0 / 2, w8, l.pitch,
                                                            p->K, int(kchunks));
    if (cudaGetLastError() != cudaSuccess) return IREE_UK_B200_CUDA_ERROR;
  }

  TcParams P;
  std::memset(&P, 0, sizeof P);
  const int64_t kbytes = p->K * 8, ncols = p->N * 32;
  const int bn = int(std::min<int64_t>(128, ncols));
  const uint64_t da[3] = {uint64_t(kbytes), uint64_t(p->M), 2};
  const uint64_t db[3] = {uint64_t(kbytes), uint64_t(ncols), 1};
  const uint64_t sa[2] = {uint64_t(l.pitch), uint64_t(l.plane_bytes)};
  const uint64_t sb[2] = {uint64_t(l.pitch), uint64_t(l.pitch) * uint64_t(ncols)};
  // The two-CTA form (256 rows x 128 columns per CTA pair, two accumulators of 128 columns, double
  // buffered = all 512 TMEM columns) once every pair has a tile; the one-CTA form otherwise.
  const DeviceInfo* di = device_info();
  if (!di) return IREE_UK_B200_CUDA_ERROR;
  const int pair_clusters = di->pair_clusters[1];
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
  P.kboxes = 1;
  P.mma_per_box = 4;
  P.stage_bytes_a = 2 * BM * 128;
  P.stage_bytes_b = b_rows * 128;
  P.num_kb = int((kbytes + 127) / 128);
  P.bn = bn;
  P.m_tiles = int((p->M + tile_m - 1) / tile_m);
  P.n_tiles = int((ncols + bn - 1) / bn);
  P.group_m = std::min(P.m_tiles, pair ? 8 : 16);
  P.out = static_cast<char*>(p->out_buffer) + p->out_offset * 4;
  P.out_stride0 = p->out_stride0;
  P.M1 = p->M;
  P.N1 = p->N;
  P.accumulate = (p->flags & IREE_UK_FLAG_MMT4D_ACCUMULATE) ? 1 : 0;
  P.out_is_int = 1;
  P.status = status;
  P.debug_flags = uint32_t(debug_int("IREE_UK_B200_DEBUG_FLAGS", 0));
  const int stage_bytes = P.stage_bytes_a + P.stage_bytes_b;
  P.num_stages = std::max(2, std::min(kMaxStages, 200 * 1024 / stage_bytes));
  const size_t smem = size_t(P.num_stages) * stage_bytes + 1024;
  if (smem > size_t(di->max_smem)) return IREE_UK_B200_CUDA_ERROR;
  if (tev) cudaEventRecord(tev[1], stream);
  cudaError_t e;
  if (pair) {
    const int grid = 2 * std::min(P.m_tiles * P.n_tiles, pair_clusters);
    e = launch_main(mmt4d_tc2_kernel<true>, grid, 2, smem, stream, P);
  } else {
    const int grid = std::min(P.m_tiles * P.n_tiles, di->sms);
    e = launch_main(mmt4d_tc_kernel<true>, grid, 1, smem, stream, P);
  }
  if (e != cudaSuccess) return IREE_UK_B200_CUDA_ERROR;
  if (tev) {
    cudaEventRecord(tev[2], stream);
    ++timing.calls;
  }
  return cuda_status(cudaGetLastError());
}

}  // namespace

bool mmt4d_tc_eligible(const iree_uk_mmt4d_params_t* p) {
  TypeInfo ti;
  if (!tc_type_info(p->flags, &ti)) return false;
  if (p->M0 != 16 || p->N0 != 16 || p->K0 < 1 || p->K < 1 || p->M < 1 || p->N < 1) return false;
  const int G = p->K0 * ti.es;
  if (G != 1 && G != 2 && G != 4 && G != 8 && G != 16) return false;
  const uintptr_t lhs = reinterpret_cast<uintptr_t>(p->lhs_buffer) + uintptr_t(p->lhs_offset * ti.es);
  const uintptr_t rhs = reinterpret_cast<uintptr_t>(p->rhs_buffer) + uintptr_t(p->rhs_offset * ti.es);
  const uintptr_t out = reinterpret_cast<uintptr_t>(p->out_buffer) + uintptr_t(p->out_offset * ti.out_es);
  if ((lhs | rhs | out) & 15) return false;
  if ((p->lhs_stride0 * ti.es) % 16 || (p->rhs_stride0 * ti.es) % 16 ||
      (p->out_stride0 * ti.out_es) % 16)
    return false;
  if ((p->M + 7) / 8 * ((p->N + 3) / 4) > 0x3FFFFFFF) return false;
  return true;
}

bool mmt4d_tc_direct_eligible(const iree_uk_mmt4d_params_t* p) {
  TypeInfo ti;
  return tc_type_info(p->flags, &ti) && ti.es == 2 && p->K0 == 1 && mmt4d_tc_eligible(p);
}

size_t mmt4d_tc_workspace_size(const iree_uk_mmt4d_params_t* p) {
  if ((p->flags & IREE_UK_FLAG_MMT4D_TYPE_MASK) == IREE_UK_FLAG_MMT4D_TYPE_S16U4S32) {
    if (p->M0 != 1 || p->N0 != 32 || p->K0 != 8 || p->K < 1 || p->M < 1 || p->N < 1) return 0;
    const S16U4Layout l = s16u4_layout(p);
    return size_t(2 * l.plane_bytes + l.w_bytes);
  }
  TypeInfo ti;
  if (!tc_type_info(p->flags, &ti)) return 0;
  if (p->M0 != 16 || p->N0 != 16 || p->K0 < 1 || p->K < 1 || p->M < 1 || p->N < 1) return 0;
  const int64_t pitch = round_up(p->K * p->K0 * ti.es, 128);
  const size_t one = size_t(round_up(p->M * 16 * pitch, 1024) + round_up(p->N * 16 * pitch, 1024));
  return ti.triple ? 2 * one : one;  // f32: a hi and a lo plane of both operands
}

// Re-tiled RHS kept by the caller across calls (weights): its size, the scratch a call then
// still needs (the LHS part), and the pre-pass that fills it.
size_t mmt4d_tc_prepared_rhs_size(const iree_uk_mmt4d_params_t* p) {
  TypeInfo ti;
  if (!tc_type_info(p->flags, &ti) || ti.triple) return 0;
  if (p->M0 != 16 || p->N0 != 16 || p->K0 < 1 || p->K < 1 || p->N < 1) return 0;
  const int64_t pitch = round_up(p->K * p->K0 * ti.es, 128);
  return size_t(round_up(p->N * 16 * pitch, 1024));
}
size_t mmt4d_tc_prepared_workspace_size(const iree_uk_mmt4d_params_t* p) {
  TypeInfo ti;
  if (!tc_type_info(p->flags, &ti) || ti.triple) return 0;
  if (p->M0 != 16 || p->N0 != 16 || p->K0 < 1 || p->K < 1 || p->M < 1) return 0;
  const int64_t pitch = round_up(p->K * p->K0 * ti.es, 128);
  return size_t(round_up(p->M * 16 * pitch, 1024));
}
int launch_mmt4d_tc_prepare_rhs(const iree_uk_mmt4d_params_t* p, void* prepared, size_t bytes,
                                cudaStream_t stream) {
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
                    const void* multicast_out, const void* prepared_rhs) {
  if (multicast_out && num_peers) return IREE_UK_B200_INVALID_ARGUMENT;
  if (num_peers < 0 || num_peers > IREE_UK_B200_MAX_PEERS || (num_peers && !peer_out_buffers))
    return IREE_UK_B200_INVALID_ARGUMENT;
  // Peer copies exist for the plain tiled epilogue only.
  if ((num_peers || multicast_out) && (p->flags & IREE_UK_FLAG_MMT4D_TYPE_MASK) == IREE_UK_FLAG_MMT4D_TYPE_S16U4S32)
    return IREE_UK_B200_UNSUPPORTED;
  if ((p->flags & IREE_UK_FLAG_MMT4D_TYPE_MASK) == IREE_UK_FLAG_MMT4D_TYPE_S16U4S32)
    return launch_mmt4d_tc_s16u4(p, ws, ws_bytes, stream);
  TypeInfo ti;
  if (!tc_type_info(p->flags, &ti) || !mmt4d_tc_eligible(p)) return IREE_UK_B200_UNSUPPORTED;
  if ((num_peers || multicast_out) && ti.out_es != 4) return IREE_UK_B200_UNSUPPORTED;  // 32-bit tiles only
  uint32_t* status = device_status_word();
  const DeviceInfo* di = device_info();
  if (!status || !di) return IREE_UK_B200_CUDA_ERROR;

  TcParams P;
  std::memset(&P, 0, sizeof P);
  KernelTiming& timing = kernel_timing();
  cudaEvent_t* tev = timing.next_slot();
  if (tev) cudaEventRecord(tev[0], stream);
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
  if (variant == 0) variant = pair_kernel_pays(p) ? 5 : 6;
  // K boxes per stage: two for the two-CTA kernel (64 KB stages, half the barrier round trips
  // per MMA), one for the one-CTA kernel (its stage is already 48 KB).
  int kboxes = debug_int("IREE_UK_B200_DEBUG_KBOXES", variant == 5 ? 2 : 1) == 2 ? 2 : 1;
  const int mma_k = 32 / ti.es;        // K per tcgen05.mma: 16 (16-bit) or 32 (8-bit)

  if (variant == 5 || variant == 6) {
    // K-major operands from the re-tiled scratch: the one-CTA kernel (6) on 128 x bn tiles, or
    // the two-CTA kernel (5) on 256 x bn tiles per CTA pair.
    if (prepared_rhs && ti.triple) return IREE_UK_B200_UNSUPPORTED;
    const size_t need = prepared_rhs ? mmt4d_tc_prepared_workspace_size(p) : mmt4d_tc_workspace_size(p);
    if (!ws || ws_bytes < need) return IREE_UK_B200_WORKSPACE_TOO_SMALL;
    if ((reinterpret_cast<uintptr_t>(ws) | reinterpret_cast<uintptr_t>(prepared_rhs)) & 255)
      return IREE_UK_B200_INVALID_ARGUMENT;
    pair = variant == 5;
    if (pair) {
      pair_clusters = di->pair_clusters[ti.is_int ? 1 : 0];
      if (pair_clusters < 1) return IREE_UK_B200_CUDA_ERROR;
      bn = pick_bn_pair(p->M, p->N, pair_clusters);
    }
    if (ti.triple) kboxes = 1;  // the two boxes of a stage are the hi and lo planes
    const int64_t pitch = round_up(kelems * ti.es, 128);
    const int64_t a_bytes = round_up(p->M * 16 * pitch, 1024), b_bytes = round_up(p->N * 16 * pitch, 1024);
    char* ws_a = static_cast<char*>(ws);
    // A prepared RHS is this pre-pass's output kept by the caller: only the LHS is re-tiled.
    char* ws_b = prepared_rhs ? const_cast<char*>(static_cast<const char*>(prepared_rhs)) : ws_a + a_bytes;
    const int G = p->K0 * ti.es;
    const int rc = launch_retile(lhs, p->lhs_stride0 * ti.es, ws_a, p->M, rhs,
                                 p->rhs_stride0 * ti.es, ws_b, prepared_rhs ? 0 : p->N, pitch,
                                 p->K, G, stream);
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
  P.group_m = std::min(P.m_tiles, pair ? 8 : 16);
  P.out = static_cast<char*>(p->out_buffer) + p->out_offset * ti.out_es;
  P.out_stride0 = p->out_stride0;
  P.M1 = p->M;
  P.N1 = p->N;
  P.accumulate = (p->flags & IREE_UK_FLAG_MMT4D_ACCUMULATE) ? 1 : 0;
  P.out_is_int = ti.is_int ? 1 : 0;
  P.out_vec32 = ((reinterpret_cast<uintptr_t>(P.out) & 31) == 0 && (p->out_stride0 * ti.out_es) % 32 == 0) ? 1 : 0;
  P.out16 = ti.out_es == 2 ? (ti.fmt == 0u ? 1 : 2) : 0;
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
  P.debug_flags = uint32_t(debug_int("IREE_UK_B200_DEBUG_FLAGS", 0));

  const int stage_bytes = P.stage_bytes_a + P.stage_bytes_b;
  const int smem_budget = 200 * 1024;
  P.num_stages = std::max(2, std::min(kMaxStages, smem_budget / stage_bytes));
  const size_t smem = size_t(P.num_stages) * stage_bytes + 1024 + ((num_peers || multicast_out) ? 4 * kEpiStageBytes : 0);

  if (smem > size_t(di->max_smem)) return IREE_UK_B200_CUDA_ERROR;
  cudaError_t e;
  if (tev) cudaEventRecord(tev[1], stream);
  if (pair) {
    const int grid = 2 * std::min(P.m_tiles * P.n_tiles, pair_clusters);
    e = ti.is_int ? launch_main(mmt4d_tc2_kernel<true>, grid, 2, smem, stream, P)
                  : launch_main(mmt4d_tc2_kernel<false>, grid, 2, smem, stream, P);
  } else {
    const int grid = std::min(P.m_tiles * P.n_tiles, di->sms);
    e = ti.is_int ? launch_main(mmt4d_tc_kernel<true>, grid, 1, smem, stream, P)
                  : launch_main(mmt4d_tc_kernel<false>, grid, 1, smem, stream, P);
  }
  if (e != cudaSuccess) return IREE_UK_B200_CUDA_ERROR;
  if (tev) {
    cudaEventRecord(tev[2], stream);
    ++timing.calls;
  }
  return cuda_status(cudaGetLastError());
}

}  // namespace uk

namespace uk {
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
  KernelTiming& timing = kernel_timing();
  cudaEvent_t* tev = timing.next_slot();
  if (tev) { cudaEventRecord(tev[0], stream); cudaEventRecord(tev[1], stream); }
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
  P.debug_flags = uint32_t(debug_int("IREE_UK_B200_DEBUG_FLAGS", 0));
  const int stage_bytes = P.stage_bytes_a + P.stage_bytes_b;
  P.num_stages = std::max(2, std::min(kMaxStages, 200 * 1024 / stage_bytes));
  const size_t smem = size_t(P.num_stages) * stage_bytes + 1024;
  if (smem > size_t(max_dyn)) return IREE_UK_B200_CUDA_ERROR;
  const int grid = std::min(P.m_tiles * P.n_tiles, di->sms);
  sw_kernel(ti.is_int, G)<<<grid, kSwThreads, smem, stream>>>(P);
  if (tev) {
    cudaEventRecord(tev[2], stream);
    ++timing.calls;
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
  // Only the tensor-core path uses scratch; everything else goes the usual way.
  const bool trivial = params->M == 0 || params->N == 0 || params->K == 0 ||
                       params->M0 == 0 || params->N0 == 0 || params->K0 == 0;
  if (trivial || uk::mmt4d_gemv_s16u4_eligible(params) || !uk::mmt4d_tc_eligible(params))
    return iree_uk_b200_mmt4d(params, cu_stream);
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
  KernelTiming& timing = kernel_timing();
  cudaEvent_t* tev = timing.next_slot();
  if (tev) cudaEventRecord(tev[0], stream);

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
    pair_clusters = di->pair_clusters[ti.is_int ? 1 : 0];
    if (pair_clusters >= 1) {
      pair = true;
      kboxes = 2;
      bn = pick_bn_pair(M1, N1, pair_clusters);
    }
  }
  if (b_direct) {
    // whole 64-column swizzle atoms per CTA: 128 or 256 columns per CTA pair, 64..256 per CTA
    if (pair) {
      const int64_t mt = (M + 255) / 256;
      auto cost = [&](int w) {
        const int64_t tiles = mt * ((N + w - 1) / w);
        return ((tiles + pair_clusters - 1) / pair_clusters) * (w + 32);
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
  P.group_m = std::min(P.m_tiles, pair ? 8 : 16);
  P.out = out;
  P.out_stride0 = out_stride0;
  P.M1 = M1;
  P.N1 = N1;
  P.rows = M;
  P.cols = N;
  P.out_row_major = 1;
  P.out_vec16 = ((reinterpret_cast<uintptr_t>(out) & 15) == 0 && (out_stride0 * 4) % 16 == 0) ? 1 : 0;
  P.accumulate = (flags & IREE_UK_FLAG_MMT4D_ACCUMULATE) ? 1 : 0;
  P.out_is_int = ti.is_int ? 1 : 0;
  P.status = status;
  P.debug_flags = uint32_t(debug_int("IREE_UK_B200_DEBUG_FLAGS", 0));
  const int stage_bytes = P.stage_bytes_a + P.stage_bytes_b;
  P.num_stages = std::max(2, std::min(kMaxStages, 200 * 1024 / stage_bytes));
  const size_t smem = size_t(P.num_stages) * stage_bytes + 1024;
  if (tev) cudaEventRecord(tev[1], stream);
  cudaError_t e;
  if (pair) {
    const int grid = 2 * std::min(P.m_tiles * P.n_tiles, pair_clusters);
    e = ti.is_int ? launch_main(mmt4d_tc2_kernel<true>, grid, 2, smem, stream, P)
                  : launch_main(mmt4d_tc2_kernel<false>, grid, 2, smem, stream, P);
  } else {
    const int grid = std::min(P.m_tiles * P.n_tiles, di->sms);
    e = ti.is_int ? launch_main(mmt4d_tc_kernel<true>, grid, 1, smem, stream, P)
                  : launch_main(mmt4d_tc_kernel<false>, grid, 1, smem, stream, P);
  }
  if (e != cudaSuccess) return IREE_UK_B200_CUDA_ERROR;
  if (tev) {
    cudaEventRecord(tev[2], stream);
    ++timing.calls;
  }
  return cuda_status(cudaGetLastError());
}

}  // namespace uk

