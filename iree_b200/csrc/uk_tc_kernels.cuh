// The three tensor-core mmt4d kernels: mmt4d_tc_kernel (one CTA per 128 x BN tile, TMA-fed),
// mmt4d_tc_sw_kernel (the same roles with producer warps that re-tile the operands themselves,
// no scratch) and mmt4d_tc2_kernel (CTA pairs, cta_group::2, 256 x BN tiles). Included by
// uk_mmt4d_tc.cu after uk_tc_device.cuh.
#ifndef IREE_UK_B200_CSRC_UK_TC_KERNELS_CUH_
#define IREE_UK_B200_CSRC_UK_TC_KERNELS_CUH_

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdint>
#include <type_traits>

#include "uk_common.h"

namespace uk {
namespace {

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
  const long long wait_limit = P.wait_cycles;
  // accumulators of one tile: bn columns, two (dual-LHS mode) or three (four-product mode) of them
  const int acc_cols = P.bn * (P.quad ? 3 : (P.dual ? 2 : 1));
  const int nbuf = P.acc_bufs == 1 ? 1 : 2;
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
          if (!mbar_wait_warp(smem_u32(&empty_bar[stage]), phase ^ 1u, abortp, wait_limit)) {
            if (lane == 0) atomicOr(P.status, kStatusProducerTimeout);
            abort_flag = 1;
            ok = false;
            break;
          }
          const uint32_t bar = smem_u32(&full_bar[stage]);
          const uint32_t sa = stage_base + uint32_t(stage) * stage_bytes;
          const bool starve = P.starve != 0;  // test hook: nothing ever arrives
          if (!starve && elect_one()) {
            mbar_expect_tx(bar, stage_bytes);
            issue_operand_loads<false>(&P.map_a, sa_st, sa, bar, ca);
            issue_operand_loads<false>(&P.map_b, sb_st, sa + a_bytes, bar, cb);
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
          const long long deadline = clock64() + wait_limit;
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
        if (!mbar_wait_warp(smem_u32(&tmem_empty_bar[buf]), buf_phase ^ 1u, abortp, wait_limit)) {
          if (lane == 0) atomicOr(P.status, kStatusMmaTimeout);
          abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + uint32_t(buf * acc_cols);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_warp(smem_u32(&full_bar[stage]), phase, abortp, wait_limit)) {
            if (lane == 0) atomicOr(P.status, kStatusMmaTimeout);
            abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = stage_base + uint32_t(stage) * stage_bytes;
          if (elect_one()) {
            if (IS_INT && mi.quad)
              issue_stage_mmas_quad<false>(mi, d_tmem, uint32_t(P.bn), sa >> 4, (sa + a_bytes) >> 4, kb == 0);
            else if (IS_INT && mi.dual)
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
        if (++buf == nbuf) { buf = 0; buf_phase ^= 1u; }
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
      if (!__all_sync(0xFFFFFFFFu, mbar_wait(smem_u32(&tmem_full_bar[buf]), buf_phase, abortp, wait_limit))) {
        if (lane == 0) atomicOr(P.status, kStatusEpilogueTimeout);
        abort_flag = 1;
        break;
      }
      tc_fence_after();
      const int64_t row = int64_t(mt) * BM + m_local;
      const uint32_t taddr0 = tmem_base + (uint32_t(q * 32) << 16) + uint32_t(buf * acc_cols);
      if (P.quad)
        epilogue_rows_quad(P, taddr0, row, int64_t(nt) * chunks, chunks);
      else if (P.dual == 2)
        epilogue_rows_dual_tiled(P, taddr0, row, int64_t(nt) * chunks, chunks);
      else if (P.dual)
        epilogue_rows_dual(P, taddr0, taddr0 + uint32_t(P.bn), row, int64_t(nt) * P.bn, chunks);
      else
        epilogue_rows(P, taddr0, row, int64_t(nt) * chunks, chunks, epi_stage, lane);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&tmem_empty_bar[buf]));
      if (++buf == nbuf) { buf = 0; buf_phase ^= 1u; }
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
  const long long wait_limit = P.wait_cycles;
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
        if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1u, abortp, wait_limit)) {
          atomicOr(P.status, kStatusProducerTimeout);
          abort_flag = 1;
          ok = false;
          break;
        }
        const uint32_t sa = stage_base + uint32_t(stage) * stage_bytes;
        {
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
        if (!P.starve) mbar_arrive(smem_u32(&full_bar[stage]));
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
      if (!mbar_wait_warp(smem_u32(&tmem_empty_bar[buf]), buf_phase ^ 1u, abortp, wait_limit)) {
        if (lane == 0) atomicOr(P.status, kStatusMmaTimeout);
        abort_flag = 1;
        break;
      }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + uint32_t(buf * P.bn);
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!mbar_wait_warp(smem_u32(&full_bar[stage]), phase, abortp, wait_limit)) {
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
      if (!__all_sync(0xFFFFFFFFu, mbar_wait(smem_u32(&tmem_full_bar[buf]), buf_phase, abortp, wait_limit))) {
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
//
// Streamed LHS pre-pass (G != 0). The re-tile of an operand into K-major scratch is pure data
// movement that the tensor-core main loop does not need all at once: a tile needs only its own
// LHS rows. The tile schedule walks the LHS in groups of m-tiles, so in this form the pre-pass
// kernel re-tiles the RHS and just the first group of LHS rows; eight more warps per CTA
// ("workers") re-tile the later groups while the main loop runs on the earlier ones. That takes
// most of the LHS re-tile - the part of a call that does not shrink when the RHS is sharded
// across GPUs - off the critical path. Each worker warp claims jobs (8 KB: one tile row,
// warp_job_k1<G>() k1 steps, re-tiled in registers) from a cursor in global memory and counts
// finished jobs per tile row; the TMA producer of a tile first checks, with a bounded acquire
// wait, that the counters of the eight LHS tile rows it is about to load have reached the number
// of jobs per row, then orders its TMA loads after what it observed with a proxy fence. Workers
// never wait for anything and any CTA's workers can take any job, so the re-tile makes progress
// whichever CTAs of the launch happen to be resident: nothing in this kernel waits on a CTA that
// may not be running. (Streaming the RHS the same way was measured too: its re-tile is five
// times the LHS's at the headline size, and run beside the main loop it slowed that loop by
// almost what the pre-pass had cost.)
constexpr int kWorkerWarps = 8;
constexpr int kWorkerThreads = kWorkerWarps * 32;
constexpr int kWorkerFirstWarp = kThreads / 32;            // warps 6..13
constexpr int kStreamedThreads = kThreads + kWorkerThreads;  // 448

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

template <bool IS_INT, int G>
__global__ void __launch_bounds__(G ? kStreamedThreads : kThreads, 1)
mmt4d_tc2_kernel(const __grid_constant__ TcParams P) {
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
  const long long wait_limit = P.wait_cycles;
  // accumulators of one tile: bn columns, two (dual-LHS mode) or three (four-product mode) of them
  const int acc_cols = P.bn * (P.quad ? 3 : (P.dual ? 2 : 1));
  const int nbuf = P.acc_bufs == 1 ? 1 : 2;
  pdl_wait();

  if (G != 0 && warp >= kWorkerFirstWarp) {
    // ------------------------------- re-tile workers (streamed pre-pass) --------------------
    if constexpr (G != 0) {
      constexpr int KJ = warp_job_k1<G>();
      const uint32_t kch = uint32_t(P.rt_kchunks);
      uint32_t claimed = 0;  // lane 0: the job claimed ahead of time
      if (lane == 0) claimed = atomicAdd(P.rt_sync, 1u);
      while (true) {
        // lane 0 decides for the warp
        uint32_t j = (lane == 0 && !*abortp) ? claimed : 0xFFFFFFFFu;
        j = __shfl_sync(0xFFFFFFFFu, j, 0);
        if (j >= P.rt_jobs) break;
        // the next job's number travels while this job is being done
        if (lane == 0) claimed = atomicAdd(P.rt_sync, 1u);
        const uint32_t r = j / kch;
        const int chunk = int(j - r * kch);
        const int64_t row = P.rt_a_first + r;
        retile_warp_job<G>(P.src_a + row * P.src_stride_a, P.rt_dst_a, P.rt_pitch, row, P.K1,
                           int64_t(chunk) * KJ, lane);
        // every lane's stores are ordered before the count that announces them
        __threadfence();
        __syncwarp();
        if (lane == 0) atomicAdd(P.rt_sync + 1 + row, 1u);
      }
    }
  } else if (warp == 0) {
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
      for (int w = pair; w < P.num_work && ok; w += num_pairs) {
        const WorkItem it = work_item(P, w);
        const int mt = it.mt, nt = it.nt;
        int ca[3], cb[3];
#pragma unroll
        for (int i = 0; i < 3; ++i) {
          ca[i] = mt * sa_st.tstep[i] + r * sa_st.rstep[i];
          cb[i] = nt * sb_st.tstep[i] + r * sb_st.rstep[i];
        }
        // A narrow tail tile: K-major RHS rows [col0, col0 + width), half of them per CTA, through
        // the tensor map whose box has that many rows; the stage keeps its layout (the boxes
        // just hold fewer rows), only the bytes to expect change.
        const CUtensorMap* map_b = &P.map_b;
        uint32_t tx_bytes = 2u * stage_bytes;
        if (it.narrow) {
          cb[1] = it.col0 + r * (it.width >> 1);
          map_b = &P.map_b_narrow;
          tx_bytes = 2u * (a_bytes + uint32_t(sb_st.nbox) * uint32_t(it.width >> 1) * 128u);
        }
        if (G != 0) {
          // Streamed pre-pass: lanes 0-7 vouch for this CTA's eight LHS tile rows. Rows below
          // rt_a_first were re-tiled by the pre-pass kernel; the others are ready once their
          // counter has reached the jobs per row.
          const uint32_t* ctr = nullptr;
          if (lane < 8) {
            const int64_t row = int64_t(mt) * (2 * BM / 16) + int64_t(r) * (BM / 16) + lane;
            if (row >= P.rt_a_first && row < P.M1) ctr = P.rt_sync + 1 + row;
          }
          bool ready = true;
          if (ctr) {
            const uint32_t need = uint32_t(P.rt_kchunks);
            const long long deadline = clock64() + wait_limit;
            while (ld_acquire_gpu(ctr) < need) {
              if (*abortp || clock64() > deadline) { ready = false; break; }
            }
          }
          if (!__all_sync(0xFFFFFFFFu, ready)) {
            if (lane == 0) atomicOr(P.status, kStatusRetileTimeout);
            raise_abort_pair(&abort_flag, rank);
            ok = false;
            break;
          }
          // order the TMA (async proxy) reads after the workers' writes observed above
          asm volatile("fence.proxy.async.global;" ::: "memory");
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_warp(smem_u32(&empty_bar[stage]), phase ^ 1u, abortp, wait_limit)) {
            if (lane == 0) atomicOr(P.status, kStatusProducerTimeout);
            raise_abort_pair(&abort_flag, rank);
            ok = false;
            break;
          }
          const uint32_t own_bar = smem_u32(&full_bar[stage]);
          const uint32_t bar = mapa_shared(own_bar, 0);
          const uint32_t sa = stage_base + uint32_t(stage) * stage_bytes;
          const bool starve = P.starve != 0;  // test hook: nothing ever arrives
          if (!starve && elect_one()) {
            if (leader) mbar_expect_tx(own_bar, tx_bytes);
            issue_operand_loads<true>(&P.map_a, sa_st, sa, bar, ca);
            issue_operand_loads<true>(map_b, sb_st, sa + a_bytes, bar, cb);
          }
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 3; ++i) { ca[i] += sa_st.kstep[i]; cb[i] += sb_st.kstep[i]; }
          if (!starve) ++issued;
          if (++stage == S) { stage = 0; phase ^= 1u; }
        }
      }
      if ((!ok || *abortp) && !leader && lane == 0 && issued > 0) {
        // Aborting: this CTA's copies complete on the leader's barriers, which only the leader can
        // wait on, and the two producers may have left their loops at different stages. Give the
        // copies this CTA issued last a fixed grace period (a TMA load lands within microseconds)
        // before the cluster barrier below lets its shared memory go.
        const long long until = clock64() + (1ll << 18);
        while (clock64() < until) {}
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
          const long long deadline = clock64() + wait_limit;
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
      MmaIssue mi_narrow = mi;  // the same MMAs with the N of a narrow tail tile
      mi_narrow.idesc = (mi.idesc & ~(0x3Fu << 17)) | (uint32_t((P.bn / max(P.tail_split, 1)) >> 3) << 17);
      for (int w = pair; w < P.num_work && ok; w += num_pairs) {
        const bool narrow = w >= P.tail_first;
        if (!mbar_wait_warp(smem_u32(&tmem_empty_bar[buf]), buf_phase ^ 1u, abortp, wait_limit)) {
          if (lane == 0) atomicOr(P.status, kStatusMmaTimeout);
          raise_abort_pair(&abort_flag, rank);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + uint32_t(buf * acc_cols);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_warp(smem_u32(&full_bar[stage]), phase, abortp, wait_limit)) {
            if (lane == 0) atomicOr(P.status, kStatusMmaTimeout);
            raise_abort_pair(&abort_flag, rank);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = stage_base + uint32_t(stage) * stage_bytes;
          if (elect_one()) {
            if (IS_INT && mi.quad)
              issue_stage_mmas_quad<true>(mi, d_tmem, uint32_t(P.bn), sa >> 4, (sa + a_bytes) >> 4, kb == 0);
            else if (IS_INT && mi.dual)
              issue_stage_mmas_dual<true>(mi, d_tmem, d_tmem + uint32_t(P.bn), sa >> 4, (sa + a_bytes) >> 4, kb == 0);
            else
              issue_stage_mmas<IS_INT, true>(narrow ? mi_narrow : mi, d_tmem, sa >> 4, (sa + a_bytes) >> 4, kb == 0);
            tc_commit_pair(smem_u32(&empty_bar[stage]), 3);  // both CTAs may refill the stage
            if (kb == num_kb - 1) tc_commit_pair(smem_u32(&tmem_full_bar[buf]), 3);  // accumulators done
          }
          __syncwarp();
          if (++stage == S) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        if (++buf == nbuf) { buf = 0; buf_phase ^= 1u; }
      }
    }
  } else {
    // ------------------------------- epilogue (both CTAs) -------------------------------
    const int q = warp & 3;
    const uint32_t epi_stage = stage_base + uint32_t(S) * stage_bytes + uint32_t(q) * kEpiStageBytes;
    int buf = 0;
    uint32_t buf_phase = 0;
    for (int w = pair; w < P.num_work; w += num_pairs) {
      const WorkItem it = work_item(P, w);
      const int mt = it.mt, nt = it.nt;
      const int chunks = it.width >> 4;
      if (!__all_sync(0xFFFFFFFFu, mbar_wait(smem_u32(&tmem_full_bar[buf]), buf_phase, abortp, wait_limit))) {
        if (lane == 0) atomicOr(P.status, kStatusEpilogueTimeout);
        raise_abort_pair(&abort_flag, rank);
        break;
      }
      tc_fence_after();
      const int64_t row = int64_t(mt) * 256 + int64_t(rank) * 128 + q * 32 + lane;
      const uint32_t taddr0 = tmem_base + (uint32_t(q * 32) << 16) + uint32_t(buf * acc_cols);
      if (P.quad)
        epilogue_rows_quad(P, taddr0, row, int64_t(it.col0 >> 4), chunks);
      else if (P.dual == 2)
        epilogue_rows_dual_tiled(P, taddr0, row, int64_t(it.col0 >> 4), chunks);
      else if (P.dual)
        epilogue_rows_dual(P, taddr0, taddr0 + uint32_t(P.bn), row, int64_t(nt) * P.bn, chunks);
      else
        epilogue_rows(P, taddr0, row, int64_t(it.col0 >> 4), chunks, epi_stage, lane);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&tmem_empty_bar[buf]), 0));
      if (++buf == nbuf) { buf = 0; buf_phase ^= 1u; }
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


}  // namespace
}  // namespace uk

#endif  // IREE_UK_B200_CSRC_UK_TC_KERNELS_CUH_
