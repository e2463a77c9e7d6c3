// Pre-pass kernels of the tensor-core mmt4d path: the re-tile of mmt4d panels into K-major
// rows, and the s16 byte-plane split / u4 widening of the s16u4s32 mode. Included by
// uk_mmt4d_tc.cu after uk_tc_device.cuh.
#ifndef IREE_UK_B200_CSRC_UK_TC_PREPASS_CUH_
#define IREE_UK_B200_CSRC_UK_TC_PREPASS_CUH_

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdint>
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


}  // namespace
}  // namespace uk

#endif  // IREE_UK_B200_CSRC_UK_TC_PREPASS_CUH_
