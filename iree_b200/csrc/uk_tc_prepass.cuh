// Pre-pass kernels of the tensor-core mmt4d path: the re-tile of mmt4d panels into K-major
// rows, and the s16 byte-plane split / u4 widening of the s16u4s32 mode. Included by
// uk_mmt4d_tc.cu after uk_tc_device.cuh.
#ifndef IREE_UK_B200_CSRC_UK_TC_PREPASS_CUH_
#define IREE_UK_B200_CSRC_UK_TC_PREPASS_CUH_

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdint>
#include <cstdlib>
#include <type_traits>

#include "uk_common.h"

namespace uk {
namespace {

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

// One re-tile job: k1 steps [chunk * KC, +KC) of tile row `tile` (16 rows), through the
// shared-memory buffer `sm` (KC * (16 * G + 4) bytes). Executed by `nthreads` threads that
// synchronise through `sync()` (the whole block in the pre-pass kernel, a named barrier among the
// worker warps of the main kernel). KC = k1 steps per job.
template <int G, int KC, class Sync>
__device__ __forceinline__ void retile_job(const char* __restrict__ src, int64_t src_stride_b,
                                           char* __restrict__ dst, int64_t dst_pitch_b, int64_t K1,
                                           int64_t tile, int chunk, unsigned char* sm, int tid,
                                           int nthreads, Sync sync) {
  constexpr int PITCH = 16 * G + 4;       // bytes per k1 in shared memory
  constexpr int GV = 16 / G;              // granules per 16-byte vector
  const int64_t k_base = int64_t(chunk) * KC;
  const int kn = int(min(int64_t(KC), K1 - k_base));
  const char* sp = src + tile * src_stride_b + k_base * (16 * G);
  // load: kn * 16 granules contiguous = kn * G vectors of 16 bytes
  const int nvec = kn * G;
#pragma unroll 4
  for (int v = tid; v < nvec; v += nthreads) {
    const uint4 x = __ldg(reinterpret_cast<const uint4*>(sp) + v);
    const int byte = v * 16;
    const int k = byte / (16 * G), within = byte - k * (16 * G);
    uint32_t* d = reinterpret_cast<uint32_t*>(sm + k * PITCH + within);
    d[0] = x.x; d[1] = x.y; d[2] = x.z; d[3] = x.w;
  }
  sync();
  // store: 16 rows x kn granules; a thread builds 16 bytes = GV consecutive k1 of one row
  if (G == 2) {
    // 2-byte granules: a 32-bit shared-memory word holds one k of two neighbouring rows, so a
    // thread reads 8 words (8 k) and emits the 16-byte vectors of both rows: half the
    // shared-memory loads of the one-row-at-a-time scheme below.
    const int full = kn / GV;  // whole vectors per row
    const int full8 = (full + 7) & ~7;
#pragma unroll 2
    for (int v = tid; v < 8 * full8; v += nthreads) {
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
    for (int e = tid; e < 16 * rem; e += nthreads) {
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
  for (int v = tid; v < 16 * vec_per_row8; v += nthreads) {
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

// The same re-tile done by one warp entirely in registers, for 2- and 4-byte granules: 8 KB of
// one tile row (16 rows x warp_job_k1<G>() k1 steps). Every lane loads sixteen 16-byte vectors
// - a vector holds one k1 step of 16 / G neighbouring rows - such that 16 / G of them are
// consecutive k1 steps of the same rows; transposing those inside the thread yields, per row,
// 16 contiguous bytes of that row's K-major form. No shared memory, no barrier: a warp is an
// independent worker with all of its loads in flight at once. Vectors past K1 are read as zero
// and not stored (a stored vector may reach past K1 * G inside the row's padded pitch).
template <int G>
__host__ __device__ constexpr int warp_job_k1() { return 2048 / (4 * G); }  // G = 4: 128, G = 2: 256

template <int G>
__device__ __forceinline__ void retile_warp_job(const char* __restrict__ src_row,
                                                char* __restrict__ dst, int64_t dst_pitch_b,
                                                int64_t tile_row, int64_t K1, int64_t k1_begin,
                                                int lane) {
  static_assert(G == 2 || G == 4, "register re-tile: 2- and 4-byte granules");
  constexpr int RPV = 16 / G;        // rows per vector = k1 steps gathered per output vector
  constexpr int RG = 16 / RPV;       // row groups of a tile: lanes rg = lane % RG
  constexpr int KQ = 32 / RG;        // k1 groups per sub-pass: kq = lane / RG
  constexpr int SUB = 16 / RPV;      // sub-passes: 16 vectors per lane in all
  const int rg = lane % RG, kq = lane / RG;
  auto load_sub = [&](uint4 (&v)[RPV], int s) {
    const int64_t base = k1_begin + int64_t(s) * (KQ * RPV) + int64_t(kq) * RPV;
#pragma unroll
    for (int i = 0; i < RPV; ++i) {
      const int64_t k1 = base + i;
      v[i] = k1 < K1 ? __ldg(reinterpret_cast<const uint4*>(src_row + k1 * (16 * G) + rg * 16))
                     : make_uint4(0u, 0u, 0u, 0u);
    }
  };
  auto store_sub = [&](const uint4 (&v)[RPV], int s) {
    const int64_t base = k1_begin + int64_t(s) * (KQ * RPV) + int64_t(kq) * RPV;
    if (base >= K1) return;
    char* drow = dst + (tile_row * 16 + rg * RPV) * dst_pitch_b + base * G;
#pragma unroll
    for (int c = 0; c < RPV; ++c) {
      uint4 o;
      if (G == 4) {
        // row c of the group: word c of each of the four k1 steps
        const uint32_t w[4][4] = {{v[0].x, v[0].y, v[0].z, v[0].w},
                                  {v[1].x, v[1].y, v[1].z, v[1].w},
                                  {v[2].x, v[2].y, v[2].z, v[2].w},
                                  {v[3].x, v[3].y, v[3].z, v[3].w}};
        o = make_uint4(w[0][c], w[1][c], w[2][c], w[3][c]);
      } else {
        // row c of the group: halfword c of each of the eight k1 steps (even rows in the low half)
        const uint32_t sel = (c & 1) ? 0x7632u : 0x5410u;
        uint32_t w[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint4 x = v[i];
          const uint32_t words[4] = {x.x, x.y, x.z, x.w};
          w[i] = words[c >> 1];
        }
        o = make_uint4(__byte_perm(w[0], w[1], sel), __byte_perm(w[2], w[3], sel),
                       __byte_perm(w[4], w[5], sel), __byte_perm(w[6], w[7], sel));
      }
      *reinterpret_cast<uint4*>(drow + int64_t(c) * dst_pitch_b) = o;
    }
  };
  uint4 v[SUB][RPV];
#pragma unroll
  for (int s = 0; s < SUB; ++s) load_sub(v[s], s);
#pragma unroll
  for (int s = 0; s < SUB; ++s) store_sub(v[s], s);
}

// Both operands of a mmt4d call in one launch: blocks [0, a.blocks) re-tile the LHS, the rest
// the RHS. `clear` / `clear_words` (optional): 32-bit words that block 0 zeroes - the ready
// counters and the job cursor of a main kernel that finishes the re-tile itself (see
// StreamedRetile); nothing else touches them while this kernel runs.
template <int G>
__global__ void __launch_bounds__(256) retile_kernel(RetileOperand opa, RetileOperand opb,
                                                     int64_t dst_pitch_b, int64_t K1, int kchunks,
                                                     uint32_t* clear, int clear_words) {
  pdl_launch_dependents();
  constexpr int KC = 1024 / G;            // k1 steps per block: 16 KB in, 16 rows x 1 KB out
  __shared__ __align__(16) unsigned char sm[KC * (16 * G + 4)];
  if (blockIdx.x == 0)
    for (int i = threadIdx.x; i < clear_words; i += blockDim.x) clear[i] = 0u;
  const bool is_a = int64_t(blockIdx.x) < opa.blocks;
  const RetileOperand& op = is_a ? opa : opb;
  const int64_t block = is_a ? int64_t(blockIdx.x) : int64_t(blockIdx.x) - opa.blocks;
  const int64_t tile = block / kchunks;
  const int chunk = int(block - tile * kchunks);
  retile_job<G, KC>(op.src, op.src_stride_b, op.dst, dst_pitch_b, K1, tile, chunk, sm,
                    int(threadIdx.x), int(blockDim.x), [] { __syncthreads(); });
}

int launch_retile(const char* lhs, int64_t lhs_stride_b, char* dst_a, int64_t tiles_a,
                  const char* rhs, int64_t rhs_stride_b, char* dst_b, int64_t tiles_b,
                  int64_t dst_pitch_b, int64_t K1, int G, cudaStream_t stream,
                  uint32_t* clear = nullptr, int clear_words = 0) {
  if (K1 <= 0 || tiles_a + tiles_b <= 0) {
    if (clear_words > 0 && cudaMemsetAsync(clear, 0, size_t(clear_words) * 4, stream) != cudaSuccess)
      return IREE_UK_B200_CUDA_ERROR;
    return IREE_UK_B200_OK;
  }
  const int KC = 1024 / G;
  const int64_t kchunks = (K1 + KC - 1) / KC;
  const RetileOperand a = {lhs, lhs_stride_b, dst_a, tiles_a * kchunks};
  const RetileOperand b = {rhs, rhs_stride_b, dst_b, tiles_b * kchunks};
  const int64_t blocks = a.blocks + b.blocks;
  if (blocks > 0x7FFFFFFF) return IREE_UK_B200_UNSUPPORTED;
  switch (G) {
    case 1: retile_kernel<1><<<int(blocks), 256, 0, stream>>>(a, b, dst_pitch_b, K1, int(kchunks), clear, clear_words); break;
    case 2: retile_kernel<2><<<int(blocks), 256, 0, stream>>>(a, b, dst_pitch_b, K1, int(kchunks), clear, clear_words); break;
    case 4: retile_kernel<4><<<int(blocks), 256, 0, stream>>>(a, b, dst_pitch_b, K1, int(kchunks), clear, clear_words); break;
    case 8: retile_kernel<8><<<int(blocks), 256, 0, stream>>>(a, b, dst_pitch_b, K1, int(kchunks), clear, clear_words); break;
    case 16: retile_kernel<16><<<int(blocks), 256, 0, stream>>>(a, b, dst_pitch_b, K1, int(kchunks), clear, clear_words); break;
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

// s16s16s32 pre-pass: a [tile][K1][16][2] s16 operand becomes two K-major byte planes
// [tile * 16 + r][K1 * 2] (high bytes, low bytes). A block moves 256 k1 steps of one tile row
// (16 KB) through shared memory, 68 bytes per k1 like the plain re-tile; a thread then reads the
// 8 words (8 k1 steps x 2 s16) of one row and stores 16 bytes to each plane. Lanes cover 8 rows
// x 4 k1 groups, which keeps the shared-memory reads on 32 different banks.
struct SplitOperand {
  const char* src;       // first panel
  int64_t src_stride_b;  // bytes between panels (tile rows)
  char* hi;              // high-byte plane; the low-byte plane follows at +plane_bytes
  int64_t plane_bytes;
  int64_t blocks;        // tile rows x k chunks
};
__global__ void __launch_bounds__(256) retile_split_s16_kernel(SplitOperand opa, SplitOperand opb,
                                                               int64_t pitch_b, int64_t K1,
                                                               int kchunks) {
  pdl_launch_dependents();
  constexpr int KC = 256, PITCH = 68;
  __shared__ __align__(16) unsigned char sm[KC * PITCH];
  const bool is_a = int64_t(blockIdx.x) < opa.blocks;
  const SplitOperand& op = is_a ? opa : opb;
  const int64_t block = is_a ? int64_t(blockIdx.x) : int64_t(blockIdx.x) - opa.blocks;
  const int64_t tile = block / kchunks;
  const int chunk = int(block - tile * kchunks);
  const int64_t k_base = int64_t(chunk) * KC;
  const int kn = int(min(int64_t(KC), K1 - k_base));
  const uint4* sp = reinterpret_cast<const uint4*>(op.src + tile * op.src_stride_b + k_base * 64);
  const int tid = int(threadIdx.x);
#pragma unroll 4
  for (int v = tid; v < kn * 4; v += 256) {
    const uint4 x = __ldg(sp + v);
    uint32_t* d = reinterpret_cast<uint32_t*>(sm + (v >> 2) * PITCH + (v & 3) * 16);
    d[0] = x.x; d[1] = x.y; d[2] = x.z; d[3] = x.w;
  }
  // k1 steps past the end of a ragged last chunk read as zero
  for (int v = kn * 16 + tid; v < ((kn + 7) & ~7) * 16; v += 256)
    *reinterpret_cast<uint32_t*>(sm + (v >> 4) * PITCH + (v & 15) * 4) = 0u;
  __syncthreads();
  const int groups = (kn + 7) >> 3;  // 16-byte vectors per row and plane
  const int groups4 = (groups + 3) & ~3;
  // task t: row = (t & 7) | ((t >> 5) & 1) << 3, group = ((t >> 3) & 3) | (t >> 6) << 2
  for (int t = tid; t < 16 * groups4; t += 256) {
    const int r = (t & 7) | (((t >> 5) & 1) << 3);
    const int g = ((t >> 3) & 3) | ((t >> 6) << 2);
    if (g >= groups) continue;
    uint32_t w[8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
      w[j] = *reinterpret_cast<const uint32_t*>(sm + (g * 8 + j) * PITCH + r * 4);
    const uint4 lo = make_uint4(__byte_perm(w[0], w[1], 0x6420), __byte_perm(w[2], w[3], 0x6420),
                                __byte_perm(w[4], w[5], 0x6420), __byte_perm(w[6], w[7], 0x6420));
    const uint4 hi = make_uint4(__byte_perm(w[0], w[1], 0x7531), __byte_perm(w[2], w[3], 0x7531),
                                __byte_perm(w[4], w[5], 0x7531), __byte_perm(w[6], w[7], 0x7531));
    char* dp = op.hi + (tile * 16 + r) * pitch_b + (k_base + g * 8) * 2;
    *reinterpret_cast<uint4*>(dp) = hi;
    *reinterpret_cast<uint4*>(dp + op.plane_bytes) = lo;
  }
}

// s8s4s32 pre-pass for the RHS: [N1][K1][16][K0 x s4] (K0 / 2 bytes per row and k1 step, low
// nibble = even k0) -> K-major s8 rows [N1 * 16 + r][K1 * K0], every nibble sign-extended to a
// byte: what the s8s8s32 kernels consume as a re-tiled RHS. GS = K0 / 2 source bytes per granule.
// A block widens 1024 / K0 k1 steps of one tile row (8 KB in, 16 rows x 1 KB out) through
// shared memory.
template <int GS>
__global__ void __launch_bounds__(256) widen_s4_kernel(const char* __restrict__ rhs,
                                                       int64_t rhs_stride_b, char* __restrict__ dst,
                                                       int64_t pitch_b, int64_t K1, int kchunks) {
  pdl_launch_dependents();
  constexpr int K0 = 2 * GS, KC = 1024 / K0, PITCH = 16 * GS + 4;
  __shared__ __align__(16) unsigned char sm[KC * PITCH];
  const int64_t n1 = blockIdx.x / kchunks;
  const int chunk = int(blockIdx.x - n1 * kchunks);
  const int64_t k_base = int64_t(chunk) * KC;
  const int kn = int(min(int64_t(KC), K1 - k_base));
  const uint4* src = reinterpret_cast<const uint4*>(rhs + n1 * rhs_stride_b + k_base * (16 * GS));
  const int tid = int(threadIdx.x);
  for (int v = tid; v < kn * GS; v += 256) {
    const uint4 x = __ldg(src + v);
    const int byte = v * 16;
    const int k = byte / (16 * GS), within = byte - k * (16 * GS);
    uint32_t* d = reinterpret_cast<uint32_t*>(sm + k * PITCH + within);
    d[0] = x.x; d[1] = x.y; d[2] = x.z; d[3] = x.w;
  }
  __syncthreads();
  // 16 rows x (kn * K0 / 16) vectors of 16 widened bytes = 8 source bytes each
  const int vec_per_row = (kn * K0 + 15) / 16;
  const int vec_per_row8 = (vec_per_row + 7) & ~7;
  for (int v = tid; v < 16 * vec_per_row8; v += 256) {
    const int r = (v >> 3) & 15, kv = ((v >> 7) << 3) | (v & 7);
    if (kv >= vec_per_row) continue;
    uint32_t w[4] = {0u, 0u, 0u, 0u};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int sb = kv * 8 + j;       // source byte of this row within the chunk
      const int k = sb / GS, within = sb - k * GS;
      const int b = k < kn ? int(int8_t(sm[k * PITCH + r * GS + within])) : 0;
      const uint32_t lo = uint32_t(int32_t(int8_t(uint8_t(b << 4))) >> 4) & 0xFFu;
      const uint32_t hi = uint32_t(b >> 4) & 0xFFu;  // arithmetic shift of the signed byte
      w[j >> 1] |= (lo | (hi << 8)) << (16 * (j & 1));
    }
    *reinterpret_cast<uint4*>(dst + (n1 * 16 + r) * pitch_b + k_base * K0 + int64_t(kv) * 16) =
        make_uint4(w[0], w[1], w[2], w[3]);
  }
}

int launch_widen_s4(const char* rhs, int64_t rhs_stride_b, char* dst, int64_t tiles,
                    int64_t pitch_b, int64_t K1, int K0, cudaStream_t stream) {
  if (tiles <= 0 || K1 <= 0) return IREE_UK_B200_OK;
  const int KC = 1024 / K0;
  const int64_t kchunks = (K1 + KC - 1) / KC;
  if (tiles * kchunks > 0x7FFFFFFF) return IREE_UK_B200_UNSUPPORTED;
  const int blocks = int(tiles * kchunks);
  switch (K0) {
    case 2: widen_s4_kernel<1><<<blocks, 256, 0, stream>>>(rhs, rhs_stride_b, dst, pitch_b, K1, int(kchunks)); break;
    case 4: widen_s4_kernel<2><<<blocks, 256, 0, stream>>>(rhs, rhs_stride_b, dst, pitch_b, K1, int(kchunks)); break;
    case 8: widen_s4_kernel<4><<<blocks, 256, 0, stream>>>(rhs, rhs_stride_b, dst, pitch_b, K1, int(kchunks)); break;
    case 16: widen_s4_kernel<8><<<blocks, 256, 0, stream>>>(rhs, rhs_stride_b, dst, pitch_b, K1, int(kchunks)); break;
    default: return IREE_UK_B200_UNSUPPORTED;
  }
  return cuda_status(cudaGetLastError());
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


}  // namespace
}  // namespace uk

#endif  // IREE_UK_B200_CSRC_UK_TC_PREPASS_CUH_
