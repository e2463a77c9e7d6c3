// mmt4d on CUDA cores: the kernel that serves every tile shape, stride and offset the
// reference accepts (ukernel/mmt4d.c:26-46), plus the K==0 zero fill and the s16u4s32
// weight-streaming GEMV. The tensor-core kernels of uk_mmt4d_tc.cu take over for the tile
// shapes they specialise; this file is what the rest falls to — never a CPU path.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdlib>
#include <type_traits>

#include "uk_common.h"

namespace uk {
namespace {

struct GenericArgs {
  const char* lhs;  // first addressed byte (offset applied)
  const char* rhs;
  char* out;
  int64_t lhs_stride_b, rhs_stride_b;  // bytes between tile rows
  int64_t out_stride0;                 // elements
  int64_t M, N, K;
  int32_t M0, N0, K0;
  int32_t accumulate;
};

template <uint32_t TYPE> struct Traits;
template <> struct Traits<IREE_UK_FLAG_MMT4D_TYPE_F32F32F32> {
  using Acc = float;
  static __device__ float lhs(const char* p, int64_t e) { return reinterpret_cast<const float*>(p)[e]; }
  static __device__ float rhs(const char* p, int64_t e) { return reinterpret_cast<const float*>(p)[e]; }
};
template <> struct Traits<IREE_UK_FLAG_MMT4D_TYPE_F16F16F32> {
  using Acc = float;
  static __device__ float lhs(const char* p, int64_t e) { return __half2float(reinterpret_cast<const __half*>(p)[e]); }
  static __device__ float rhs(const char* p, int64_t e) { return __half2float(reinterpret_cast<const __half*>(p)[e]); }
};
template <> struct Traits<IREE_UK_FLAG_MMT4D_TYPE_BF16BF16F32> {
  using Acc = float;
  static __device__ float lhs(const char* p, int64_t e) { return __uint_as_float(uint32_t(reinterpret_cast<const uint16_t*>(p)[e]) << 16); }
  static __device__ float rhs(const char* p, int64_t e) { return lhs(p, e); }
};
template <> struct Traits<IREE_UK_FLAG_MMT4D_TYPE_S8S8S32> {
  using Acc = uint32_t;
  static __device__ int32_t lhs(const char* p, int64_t e) { return reinterpret_cast<const int8_t*>(p)[e]; }
  static __device__ int32_t rhs(const char* p, int64_t e) { return reinterpret_cast<const int8_t*>(p)[e]; }
};
template <> struct Traits<IREE_UK_FLAG_MMT4D_TYPE_S16S16S32> {
  using Acc = uint32_t;
  static __device__ int32_t lhs(const char* p, int64_t e) { return reinterpret_cast<const int16_t*>(p)[e]; }
  static __device__ int32_t rhs(const char* p, int64_t e) { return reinterpret_cast<const int16_t*>(p)[e]; }
};
template <> struct Traits<IREE_UK_FLAG_MMT4D_TYPE_S16S8S32> {
  using Acc = uint32_t;
  static __device__ int32_t lhs(const char* p, int64_t e) { return reinterpret_cast<const int16_t*>(p)[e]; }
  static __device__ int32_t rhs(const char* p, int64_t e) { return reinterpret_cast<const int8_t*>(p)[e]; }
};
// 4-bit right-hand sides: element e is in byte e/2, low nibble when e is even
// (ukernel/mmt4d_tile_generic.c:35-44 signed, :130-136 unsigned).
template <> struct Traits<IREE_UK_FLAG_MMT4D_TYPE_S16U4S32> {
  using Acc = uint32_t;
  static __device__ int32_t lhs(const char* p, int64_t e) { return reinterpret_cast<const int16_t*>(p)[e]; }
  static __device__ int32_t rhs(const char* p, int64_t e) {
    const uint32_t b = reinterpret_cast<const uint8_t*>(p)[e >> 1];
    return int32_t((e & 1) ? (b >> 4) : (b & 0xF));
  }
};
template <> struct Traits<IREE_UK_FLAG_MMT4D_TYPE_S8S4S32> {
  using Acc = uint32_t;
  static __device__ int32_t lhs(const char* p, int64_t e) { return reinterpret_cast<const int8_t*>(p)[e]; }
  static __device__ int32_t rhs(const char* p, int64_t e) {
    const uint32_t b = reinterpret_cast<const uint8_t*>(p)[e >> 1];
    int32_t v = int32_t((e & 1) ? (b >> 4) : (b & 0xF));
    return (v & 8) ? v - 16 : v;
  }
};

__device__ __forceinline__ float mac(float acc, float a, float b) { return fmaf(a, b, acc); }
__device__ __forceinline__ uint32_t mac(uint32_t acc, int32_t a, int32_t b) {
  return acc + uint32_t(a * b);  // wraps modulo 2^32 like the reference's int32 sums
}

// One thread per output element; the K loop is the reference's: k-major, then k0
// (ukernel/mmt4d_tile_generic.c:65-75).
template <uint32_t TYPE>
__global__ void __launch_bounds__(256) mmt4d_generic_kernel(GenericArgs a) {
  using T = Traits<TYPE>;
  using Acc = typename T::Acc;
  const int64_t tile_elems = int64_t(a.M0) * a.N0;
  const int64_t total = a.M * a.N * tile_elems;
  const int64_t lhs_k_step = int64_t(a.M0) * a.K0, rhs_k_step = int64_t(a.N0) * a.K0;
  for (int64_t idx = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; idx < total;
       idx += int64_t(gridDim.x) * blockDim.x) {
    const int64_t tile = idx / tile_elems;
    const int32_t e = int32_t(idx - tile * tile_elems);
    const int64_t i = tile / a.N, j = tile - i * a.N;
    const int32_t i0 = e / a.N0, j0 = e - i0 * a.N0;
    const char* lp = a.lhs + i * a.lhs_stride_b;
    const char* rp = a.rhs + j * a.rhs_stride_b;
    Acc* op = reinterpret_cast<Acc*>(a.out) + i * a.out_stride0 + j * tile_elems + e;
    Acc acc = a.accumulate ? *op : Acc(0);
    int64_t le = int64_t(i0) * a.K0, re = int64_t(j0) * a.K0;
    for (int64_t k = 0; k < a.K; ++k) {
      for (int32_t k0 = 0; k0 < a.K0; ++k0) acc = mac(acc, T::lhs(lp, le + k0), T::rhs(rp, re + k0));
      le += lhs_k_step;
      re += rhs_k_step;
    }
    *op = acc;
  }
}

// f16f16f16 / bf16bf16bf16 (ukernel/mmt4d_tile_generic.c:226-286, :316-376): without
// SKIP_INTERMEDIATE_ROUNDINGS the accumulator is 16-bit and rounded (to nearest even) after
// every multiply-add; with it the sum stays in f32 and is rounded once at the end. Multiply
// and add are separate roundings, as in the reference's portable code.
template <bool IS_BF16>
__global__ void __launch_bounds__(256) mmt4d_generic_out16_kernel(GenericArgs a, int skip_round) {
  auto to_f32 = [](uint16_t v) -> float {
    if (IS_BF16) return __uint_as_float(uint32_t(v) << 16);
    return __half2float(__ushort_as_half(v));
  };
  auto from_f32 = [](float f) -> uint16_t {
    if (IS_BF16) return __bfloat16_as_ushort(__float2bfloat16_rn(f));
    return __half_as_ushort(__float2half_rn(f));
  };
  const int64_t tile_elems = int64_t(a.M0) * a.N0;
  const int64_t total = a.M * a.N * tile_elems;
  const int64_t lhs_k_step = int64_t(a.M0) * a.K0, rhs_k_step = int64_t(a.N0) * a.K0;
  for (int64_t idx = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; idx < total;
       idx += int64_t(gridDim.x) * blockDim.x) {
    const int64_t tile = idx / tile_elems;
    const int32_t e = int32_t(idx - tile * tile_elems);
    const int64_t i = tile / a.N, j = tile - i * a.N;
    const int32_t i0 = e / a.N0, j0 = e - i0 * a.N0;
    const uint16_t* lp = reinterpret_cast<const uint16_t*>(a.lhs + i * a.lhs_stride_b);
    const uint16_t* rp = reinterpret_cast<const uint16_t*>(a.rhs + j * a.rhs_stride_b);
    uint16_t* op = reinterpret_cast<uint16_t*>(a.out) + i * a.out_stride0 + j * tile_elems + e;
    uint16_t acc16 = a.accumulate ? *op : uint16_t(0);
    float acc32 = to_f32(acc16);
    int64_t le = int64_t(i0) * a.K0, re = int64_t(j0) * a.K0;
    for (int64_t k = 0; k < a.K; ++k) {
      for (int32_t k0 = 0; k0 < a.K0; ++k0) {
        const float prod = __fmul_rn(to_f32(lp[le + k0]), to_f32(rp[re + k0]));
        if (skip_round) {
          acc32 = __fadd_rn(acc32, prod);
        } else {
          acc16 = from_f32(__fadd_rn(to_f32(acc16), prod));
        }
      }
      le += lhs_k_step;
      re += rhs_k_step;
    }
    *op = skip_round ? from_f32(acc32) : acc16;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) mmt4d_zero_fill_kernel(char* out, int64_t out_stride0,
                                                              int64_t M, int64_t row_elems) {
  // K == 0 without ACCUMULATE: every addressed out tile becomes zero, stride gaps are left
  // alone (ukernel/mmt4d.c:105-113 falls through to a tile function with an empty K loop).
  const int64_t total = M * row_elems;
  for (int64_t idx = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; idx < total;
       idx += int64_t(gridDim.x) * blockDim.x) {
    const int64_t i = idx / row_elems, c = idx - i * row_elems;
    reinterpret_cast<T*>(out)[i * out_stride0 + c] = T(0);
  }
}

// ---------------------------------------------------------------------------------------
// s16u4s32, M0 = 1, N0 = 32, K0 = 8: weight-streaming GEMV.
// RHS tile (n1, k1) is 128 contiguous bytes [n0 = 32][4 bytes = 8 nibbles, low nibble =
// even k0]; the whole RHS row n1 is K*128 contiguous bytes. One block per (m, n1) pair
// keeps 32 int32 sums; each lane takes 16 bytes (4 n0 rows of one k1) per step, four k1
// per warp step, and the eight warps interleave along K in chunks. HBM-bound by construction:
// every weight byte is read once. The nibbles are widened to bytes in registers (even and odd
// ones apart) and multiplied with the s16 activations by dp2a, four per 8 weights; the
// activations of a chunk are paired for that once per k1 step and shared through a staging row
// per warp, not re-arranged by each of the eight lanes that meet the same k1.
// ---------------------------------------------------------------------------------------

// a: two signed 16-bit values, b: four unsigned bytes of which the low (high) two are used:
// d = c + a.lo * b.byte0 + a.hi * b.byte1 (b.byte2, b.byte3)
__device__ __forceinline__ int32_t dp2a_lo(uint32_t a, uint32_t b, int32_t c) {
  int32_t d;
  asm("dp2a.lo.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ int32_t dp2a_hi(uint32_t a, uint32_t b, int32_t c) {
  int32_t d;
  asm("dp2a.hi.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// The weights reach shared memory by bulk asynchronous copies (cp.async.bulk, completion on an
// mbarrier): each of the 8 warps owns a 4 KB buffer and walks its own chunks of 32 k1 steps
// (chunk c belongs to warp c mod 8), so every warp has a whole chunk in flight without holding
// it in registers, and with 32 KB per block all blocks of the decode shape are resident at
// once. (A version with register-staged 16-byte loads, eight in flight per thread, took 10.9 us
// per call where this one takes 7.3 us.) Waits are bounded.
constexpr int kGemvBulkWarps = 8;
constexpr int kGemvChunkK1 = 32;                       // k1 steps per chunk

__device__ __forceinline__ uint32_t gemv_smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// R = LHS rows (M0 = 1 tiles) one block serves: a batch of tokens shares one pass over the
// weights and the nibble split of every weight word (R = 1: the decode call proper).
template <int R>
__global__ void __launch_bounds__(kGemvBulkWarps * 32)
mmt4d_gemv_s16u4_kernel(GenericArgs a, uint32_t* status) {
  // chunk of k1 steps per bulk copy: 32 (4 KB) for the decode call, 16 with four rows per block
  // so that the staging rows of the four rows' activations still fit 48 KB of static memory
  constexpr int CK = R == 1 ? kGemvChunkK1 : kGemvChunkK1 / 2;
  __shared__ __align__(128) unsigned char wbuf[kGemvBulkWarps][CK * 128];
  __shared__ __align__(8) uint64_t bar[kGemvBulkWarps];
  __shared__ int32_t partial[kGemvBulkWarps][R][32];
  __shared__ uint4 xs[kGemvBulkWarps][R][CK];  // per warp: the chunk's activations, paired
  const int64_t mg = blockIdx.x / a.N, n1 = blockIdx.x - mg * a.N;
  const int64_t m = mg * R;                              // first LHS row of this block
  const int rows = int(min(int64_t(R), a.M - m));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kq = lane >> 3, ng = lane & 7;
  const char* rhs = a.rhs + n1 * a.rhs_stride_b;
  const uint32_t my_bar = gemv_smem_u32(&bar[warp]);
  const uint32_t my_buf = gemv_smem_u32(&wbuf[warp][0]);
  if (lane == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(my_bar) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  int32_t acc[R][4];
#pragma unroll
  for (int i = 0; i < R; ++i)
#pragma unroll
    for (int r = 0; r < 4; ++r) acc[i][r] = 0;
  const int64_t chunks = (a.K + CK - 1) / CK;
  uint32_t parity = 0;
  bool ok = true;
  for (int64_t c = warp; c < chunks && ok; c += kGemvBulkWarps) {
    const int64_t k0 = c * CK;
    const int steps = int(min(int64_t(CK), a.K - k0));
    if (lane == 0) {
      const uint32_t bytes = uint32_t(steps) * 128u;
      // earlier reads of this buffer (generic proxy) come before the copy's writes (async proxy)
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(my_bar), "r"(bytes) : "memory");
      asm volatile(
          "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
          :: "r"(my_buf), "l"(rhs + k0 * 128), "r"(bytes), "r"(my_bar) : "memory");
    }
    // The activations of this chunk, while the weights are on their way: lane l takes k1 step l,
    // pairs its eight s16 values the way dp2a consumes them against the even and the odd nibbles
    // - (x0,x2) (x4,x6) (x1,x3) (x5,x7) - and leaves the four words in this warp's staging row.
#pragma unroll
    for (int i = 0; i < R; ++i) {
      uint4 x = make_uint4(0u, 0u, 0u, 0u);
      if (i < rows && lane < steps)
        x = __ldg(reinterpret_cast<const uint4*>(a.lhs + (m + i) * a.lhs_stride_b) + k0 + lane);
      const uint4 pairs = make_uint4(__byte_perm(x.x, x.y, 0x5410), __byte_perm(x.z, x.w, 0x5410),
                                     __byte_perm(x.x, x.y, 0x7632), __byte_perm(x.z, x.w, 0x7632));
      if (lane < CK) xs[warp][i][lane] = pairs;
    }
    __syncwarp();
    // bounded wait for the chunk
    {
      const long long deadline = clock64() + (1ll << 31);
      uint32_t done = 0;
      while (true) {
        asm volatile(
            "{\n.reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(done) : "r"(my_bar), "r"(parity) : "memory");
        if (done) break;
        if (clock64() > deadline) { ok = false; break; }
      }
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) {
        if (lane == 0) {
          atomicOr(status, 1u << 4);
          // one more bounded wait: the copy must not still be in flight into this warp's
          // buffer when the block's shared memory is released
          const long long drain = clock64() + (1ll << 31);
          uint32_t landed = 0;
          while (!landed && clock64() < drain) {
            asm volatile(
                "{\n.reg .pred p;\n"
                "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
                "selp.u32 %0, 1, 0, p;\n}\n"
                : "=r"(landed) : "r"(my_bar), "r"(parity) : "memory");
          }
        }
        __syncwarp();
        break;
      }
    }
    parity ^= 1u;
#pragma unroll
    for (int s = 0; s < CK / 4; ++s) {
      const int k = s * 4 + kq;
      uint4 wv = make_uint4(0u, 0u, 0u, 0u);
      if (k < steps)
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(wv.x), "=r"(wv.y), "=r"(wv.z), "=r"(wv.w)
                     : "r"(my_buf + uint32_t(k) * 128u + uint32_t(ng) * 16u) : "memory");
      const uint32_t ws[4] = {wv.x, wv.y, wv.z, wv.w};
      uint32_t w_even[4], w_odd[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        w_even[r] = ws[r] & 0x0F0F0F0Fu;
        w_odd[r] = (ws[r] >> 4) & 0x0F0F0F0Fu;
      }
#pragma unroll
      for (int i = 0; i < R; ++i) {
        if (i >= rows) break;
        const uint4 x = xs[warp][i][k];  // the eight lanes of one k read the same row
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          acc[i][r] = dp2a_lo(x.x, w_even[r], acc[i][r]);
          acc[i][r] = dp2a_hi(x.y, w_even[r], acc[i][r]);
          acc[i][r] = dp2a_lo(x.z, w_odd[r], acc[i][r]);
          acc[i][r] = dp2a_hi(x.w, w_odd[r], acc[i][r]);
        }
      }
    }
    __syncwarp();  // every lane is done with the buffer before lane 0 refills it
  }
#pragma unroll
  for (int i = 0; i < R; ++i) {
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      acc[i][r] += __shfl_xor_sync(0xFFFFFFFFu, acc[i][r], 8);
      acc[i][r] += __shfl_xor_sync(0xFFFFFFFFu, acc[i][r], 16);
    }
    if (lane < 8) {
#pragma unroll
      for (int r = 0; r < 4; ++r) partial[warp][i][ng * 4 + r] = acc[i][r];
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < rows * 32; e += blockDim.x) {
    const int i = e >> 5, n0 = e & 31;
    int32_t s = 0;
#pragma unroll
    for (int w = 0; w < kGemvBulkWarps; ++w) s += partial[w][i][n0];
    int32_t* op = reinterpret_cast<int32_t*>(a.out) + (m + i) * a.out_stride0 + n1 * 32 + n0;
    *op = a.accumulate ? int32_t(uint32_t(*op) + uint32_t(s)) : s;
  }
}

// ---------------------------------------------------------------------------------------
// Narrowed M0 (1, 2, 4 or 8 rows) with N0 = 16: the tiles the reference's encoder picks when M
// is small (decode, GEMV-like shapes; compiler/.../CPUEncodingExternalModels.cpp narrows M0 to
// the next power of two) and for which it ships ISA tile functions
// (arch/x86_64/mmt4d_x86_64_tiles.inl): s8s8s32 K0 = 2, f16f16f32 K0 = 1, bf16bf16f32 K0 = 2.
// With so few LHS rows the call is a weight stream: every RHS byte is read once per LHS tile
// row and used for M0 multiply-adds, so HBM bounds it - as long as the arithmetic keeps up,
// which on the CUDA cores it does for M0 = 1 (and 2); the wider tiles take the warp-level
// tensor-core instruction (mmt4d_narrow_mma_kernel below).
// One block per (LHS tile row, RHS tile row); its 8 warps interleave along K, each lane reads
// 16-byte vectors of the RHS row - a vector holds one k1 step of 4 (bf16) or 8 (s8, f16)
// neighbouring n0 rows, and a lane always meets the same rows - with four loads in flight, takes
// the matching LHS values through L1 (the LHS tile row is a few KB), and keeps M0 x rows sums.
// f32 sums are formed in another order than the reference's (k interleaved over lanes and
// warps); integers are exact.
// ---------------------------------------------------------------------------------------
enum class NarrowType : int { S8, F16, BF16 };

template <NarrowType T, int M0>
__global__ void __launch_bounds__(256) mmt4d_narrow_kernel(GenericArgs a) {
  constexpr int ROWS = T == NarrowType::BF16 ? 4 : 8;   // n0 rows per 16-byte vector
  constexpr int VPT = 16 / ROWS;                        // vectors per RHS tile
  constexpr int KSUB = 32 / VPT;                        // k1 steps per warp-wide load
  constexpr int TILE_B = VPT * 16;                      // RHS tile bytes
  constexpr int XB = T == NarrowType::BF16 ? 4 : 2;     // LHS bytes per (k1, m0): K0 elements
  constexpr int U = 4;                                  // loads in flight per lane
  using Acc = typename std::conditional<T == NarrowType::S8, int32_t, float>::type;
  __shared__ Acc partial[8][M0][16];
  const int64_t m1 = blockIdx.x / a.N, n1 = blockIdx.x - m1 * a.N;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int v = lane % VPT, ksub = lane / VPT;
  const char* rhs = a.rhs + n1 * a.rhs_stride_b + v * 16;
  const char* lhs = a.lhs + m1 * a.lhs_stride_b;
  Acc acc[M0][ROWS];
#pragma unroll
  for (int m = 0; m < M0; ++m)
#pragma unroll
    for (int r = 0; r < ROWS; ++r) acc[m][r] = Acc(0);

  for (int64_t kb = int64_t(warp) * (U * KSUB); kb < a.K; kb += 8 * U * KSUB) {
    uint4 w[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t k1 = kb + u * KSUB + ksub;
      w[u] = k1 < a.K ? __ldg(reinterpret_cast<const uint4*>(rhs + k1 * TILE_B))
                      : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t k1 = kb + u * KSUB + ksub;
      if (k1 >= a.K) continue;
      const uint32_t ww[4] = {w[u].x, w[u].y, w[u].z, w[u].w};
      const char* xp = lhs + k1 * (M0 * XB);
#pragma unroll
      for (int m = 0; m < M0; ++m) {
        if (T == NarrowType::BF16) {
          const uint32_t x = __ldg(reinterpret_cast<const uint32_t*>(xp + m * 4));
          const float x0 = __uint_as_float(x << 16), x1 = __uint_as_float(x & 0xFFFF0000u);
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            acc[m][r] = fmaf(__uint_as_float(ww[r] << 16), x0, acc[m][r]);
            acc[m][r] = fmaf(__uint_as_float(ww[r] & 0xFFFF0000u), x1, acc[m][r]);
          }
        } else if (T == NarrowType::F16) {
          const float x = __half2float(__ushort_as_half(__ldg(reinterpret_cast<const uint16_t*>(xp + m * 2))));
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&ww[j]));
            acc[m][2 * j] = fmaf(f.x, x, acc[m][2 * j]);
            acc[m][2 * j + 1] = fmaf(f.y, x, acc[m][2 * j + 1]);
          }
        } else {
          // two s8 of the LHS as two s16; a weight word holds rows 2j (low half) and 2j + 1
          const uint32_t xb = __ldg(reinterpret_cast<const uint16_t*>(xp + m * 2));
          const int32_t x0 = int8_t(xb & 0xFF), x1 = int8_t(xb >> 8);
          const uint32_t xs = (uint32_t(x0) & 0xFFFFu) | (uint32_t(x1) << 16);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            int32_t lo, hi;
            asm("dp2a.lo.s32.s32 %0, %1, %2, %3;" : "=r"(lo) : "r"(xs), "r"(ww[j]), "r"(int32_t(acc[m][2 * j])));
            asm("dp2a.hi.s32.s32 %0, %1, %2, %3;" : "=r"(hi) : "r"(xs), "r"(ww[j]), "r"(int32_t(acc[m][2 * j + 1])));
            acc[m][2 * j] = Acc(lo);
            acc[m][2 * j + 1] = Acc(hi);
          }
        }
      }
    }
  }
  // lanes that differ only in their k1 position hold partial sums of the same rows
#pragma unroll
  for (int m = 0; m < M0; ++m)
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      Acc x = acc[m][r];
#pragma unroll
      for (int d = VPT; d < 32; d <<= 1) x += __shfl_xor_sync(0xFFFFFFFFu, x, d);
      acc[m][r] = x;
    }
  if (lane < VPT) {
#pragma unroll
    for (int m = 0; m < M0; ++m)
#pragma unroll
      for (int r = 0; r < ROWS; ++r) partial[warp][m][v * ROWS + r] = acc[m][r];
  }
  __syncthreads();
  for (int e = threadIdx.x; e < M0 * 16; e += blockDim.x) {
    const int m = e >> 4, n0 = e & 15;
    Acc sum = Acc(0);
#pragma unroll
    for (int w8 = 0; w8 < 8; ++w8) sum += partial[w8][m][n0];
    Acc* op = reinterpret_cast<Acc*>(a.out) + m1 * a.out_stride0 + n1 * (M0 * 16) + e;
    if (T == NarrowType::S8) {
      uint32_t* uo = reinterpret_cast<uint32_t*>(op);
      *uo = a.accumulate ? *uo + uint32_t(sum) : uint32_t(sum);  // wraps like the reference's int32
    } else {
      *op = a.accumulate ? *op + sum : sum;
    }
  }
}

// The same weight stream where the CUDA-core form above is bound by its multiply-adds (M0 per
// weight; every M0 for bf16, from M0 = 2 for s8, from 4 for f16): the warp-level tensor-core
// instruction mma.sync m16n8k16 (bf16, f16) / m16n8k32 (s8) has exactly this shape when the 16
// rows of an RHS tile are its M and the up to 8 rows of the LHS tile its N. Fragments come
// straight from global memory: for bf16 (K0 = 2) one k1 step of one n0 row is the 4-byte pair an
// A register holds, so a lane takes 8 bytes = rows 2g, 2g+1 (the instruction's rows g and g+8)
// at k1 = kb+t and again at kb+t+4; for f16 (K0 = 1) and s8 (K0 = 2) one k1 step of one row is
// 2 bytes, two neighbouring k1 steps make a register (a byte permute of two 4-byte loads). The
// LHS tile is a few KB and comes through L1. Eight warps interleave along K, four MMAs' worth
// of loads in flight per warp; sums in another order than the reference's (integers exact).
template <NarrowType T>
__device__ __forceinline__ void narrow_mma(uint32_t (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  if (T == NarrowType::BF16)
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
  else if (T == NarrowType::F16)
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
  else
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

template <NarrowType T, int M0>
__global__ void __launch_bounds__(256) mmt4d_narrow_mma_kernel(GenericArgs a) {
  constexpr bool G4 = T == NarrowType::BF16;  // 4-byte granules (one k1 step of one row)
  constexpr int KM = G4 ? 8 : 16;             // k1 steps per MMA
  constexpr int U = 4;                        // MMAs whose loads are in flight together
  using Acc = typename std::conditional<T == NarrowType::S8, int32_t, float>::type;
  __shared__ Acc partial[8][M0][16];
  const int64_t m1 = blockIdx.x / a.N, n1 = blockIdx.x - m1 * a.N;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const char* rhs = a.rhs + n1 * a.rhs_stride_b;
  const char* lhs = a.lhs + m1 * a.lhs_stride_b;
  const int64_t K = a.K;
  const int gm = g < M0 ? g : M0 - 1;  // the LHS row this lane reads (rows past M0 count as zero)
  const bool row_live = g < M0;
  uint32_t d[4] = {0u, 0u, 0u, 0u};
  constexpr int WB = G4 ? 64 : 32;            // RHS bytes per k1 step
  constexpr int XB = (G4 ? 4 : 2) * M0;       // LHS bytes per k1 step
  // this lane's first addresses within a group of KM k1 steps
  const char* wp = rhs + (G4 ? t * WB + g * 8 : 2 * t * WB + g * 4);
  const char* xp = lhs + (G4 ? t * XB + gm * 4 : 2 * t * XB + gm * 2);
  // One group's fragments. FULL: all KM k1 steps exist, every load is unconditional at a
  // constant offset from the lane's pointers; else each k1 step is checked against K.
  auto load_group = [&](int64_t grp, uint32_t (&fa)[4], uint32_t (&fb)[2], auto full) {
    constexpr bool FULL = decltype(full)::value;
    const int64_t kb = grp * KM;
    const char* w = wp + kb * WB;
    const char* x = xp + kb * XB;
    if (G4) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const bool live = FULL || kb + t + 4 * h < K;
        uint2 wv = make_uint2(0u, 0u);
        uint32_t xv = 0u;
        if (live) wv = __ldg(reinterpret_cast<const uint2*>(w + 4 * h * WB));
        if (live && row_live) xv = __ldg(reinterpret_cast<const uint32_t*>(x + 4 * h * XB));
        fa[2 * h] = wv.x;      // n0 = 2g   -> row g of the instruction
        fa[2 * h + 1] = wv.y;  // n0 = 2g+1 -> row g + 8
        fb[h] = xv;
      }
    } else {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int64_t k1 = kb + 8 * h + 2 * t;
        uint32_t w0 = 0u, w1 = 0u, x0 = 0u, x1 = 0u;
        const bool live0 = FULL || k1 < K, live1 = FULL || k1 + 1 < K;
        if (live0) w0 = __ldg(reinterpret_cast<const uint32_t*>(w + 8 * h * WB));
        if (live1) w1 = __ldg(reinterpret_cast<const uint32_t*>(w + (8 * h + 1) * WB));
        if (live0 && row_live) x0 = __ldg(reinterpret_cast<const uint16_t*>(x + 8 * h * XB));
        if (live1 && row_live) x1 = __ldg(reinterpret_cast<const uint16_t*>(x + (8 * h + 1) * XB));
        fa[2 * h] = __byte_perm(w0, w1, 0x5410);      // row 2g at k1, k1 + 1
        fa[2 * h + 1] = __byte_perm(w0, w1, 0x7632);  // row 2g+1
        fb[h] = x0 | (x1 << 16);
      }
    }
  };
  const int64_t groups = (K + KM - 1) / KM, full_groups = K / KM;
  int64_t grp = int64_t(warp) * U;
  for (; grp + U <= full_groups; grp += 8 * U) {
    uint32_t fa[U][4], fb[U][2];
#pragma unroll
    for (int u = 0; u < U; ++u) load_group(grp + u, fa[u], fb[u], std::true_type());
#pragma unroll
    for (int u = 0; u < U; ++u) narrow_mma<T>(d, fa[u], fb[u]);
  }
  // what is left of this warp's share: fewer than U groups, the last one possibly ragged
  for (int u = 0; u < U && grp + u < groups; ++u) {
    uint32_t fa[4], fb[2];
    load_group(grp + u, fa, fb, std::false_type());
    narrow_mma<T>(d, fa, fb);
  }
  // d0, d1: n0 = 2g, m0 = 2t, 2t+1; d2, d3: n0 = 2g+1
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m0 = 2 * t + (i & 1), n0 = 2 * g + (i >> 1);
    if (m0 < M0) {
      Acc v;
      if (T == NarrowType::S8) v = Acc(int32_t(d[i]));
      else v = Acc(__uint_as_float(d[i]));
      partial[warp][m0][n0] = v;
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < M0 * 16; e += blockDim.x) {
    const int m = e >> 4, n0 = e & 15;
    Acc sum = Acc(0);
#pragma unroll
    for (int w8 = 0; w8 < 8; ++w8) sum += partial[w8][m][n0];
    Acc* op = reinterpret_cast<Acc*>(a.out) + m1 * a.out_stride0 + n1 * (M0 * 16) + e;
    if (T == NarrowType::S8) {
      uint32_t* uo = reinterpret_cast<uint32_t*>(op);
      *uo = a.accumulate ? *uo + uint32_t(sum) : uint32_t(sum);  // wraps like the reference's int32
    } else {
      *op = a.accumulate ? *op + sum : sum;
    }
  }
}

bool fill_args(const iree_uk_mmt4d_params_t* p, GenericArgs* a) {
  Mmt4dTypes t;
  if (!mmt4d_types(p->flags, &t)) return false;
  const int lb = elem_bits(t.lhs), rb = elem_bits(t.rhs), ob = elem_bits(t.out);
  a->lhs = static_cast<const char*>(p->lhs_buffer) + p->lhs_offset * lb / 8;
  a->rhs = static_cast<const char*>(p->rhs_buffer) + p->rhs_offset * rb / 8;
  a->out = static_cast<char*>(p->out_buffer) + p->out_offset * (ob / 8);
  a->lhs_stride_b = p->lhs_stride0 * lb / 8;
  a->rhs_stride_b = p->rhs_stride0 * rb / 8;
  a->out_stride0 = p->out_stride0;
  a->M = p->M; a->N = p->N; a->K = p->K;
  a->M0 = p->M0; a->N0 = p->N0; a->K0 = p->K0;
  a->accumulate = (p->flags & IREE_UK_FLAG_MMT4D_ACCUMULATE) ? 1 : 0;
  return true;
}

template <uint32_t TYPE>
int launch_generic_typed(const GenericArgs& a, cudaStream_t stream) {
  const int64_t total = a.M * a.N * a.M0 * a.N0;
  if (total <= 0) return IREE_UK_B200_OK;
  const int64_t blocks = std::min<int64_t>((total + 255) / 256, 148 * 64);
  mmt4d_generic_kernel<TYPE><<<int(blocks), 256, 0, stream>>>(a);
  return cuda_status(cudaGetLastError());
}

}  // namespace

int launch_mmt4d_generic(const iree_uk_mmt4d_params_t* p, cudaStream_t stream) {
  GenericArgs a;
  if (!fill_args(p, &a)) return IREE_UK_B200_INVALID_ARGUMENT;
  switch (p->flags & IREE_UK_FLAG_MMT4D_TYPE_MASK) {
    case IREE_UK_FLAG_MMT4D_TYPE_F32F32F32: return launch_generic_typed<IREE_UK_FLAG_MMT4D_TYPE_F32F32F32>(a, stream);
    case IREE_UK_FLAG_MMT4D_TYPE_S8S8S32: return launch_generic_typed<IREE_UK_FLAG_MMT4D_TYPE_S8S8S32>(a, stream);
    case IREE_UK_FLAG_MMT4D_TYPE_F16F16F32: return launch_generic_typed<IREE_UK_FLAG_MMT4D_TYPE_F16F16F32>(a, stream);
    case IREE_UK_FLAG_MMT4D_TYPE_BF16BF16F32: return launch_generic_typed<IREE_UK_FLAG_MMT4D_TYPE_BF16BF16F32>(a, stream);
    case IREE_UK_FLAG_MMT4D_TYPE_S16S16S32: return launch_generic_typed<IREE_UK_FLAG_MMT4D_TYPE_S16S16S32>(a, stream);
    case IREE_UK_FLAG_MMT4D_TYPE_S16U4S32: return launch_generic_typed<IREE_UK_FLAG_MMT4D_TYPE_S16U4S32>(a, stream);
    case IREE_UK_FLAG_MMT4D_TYPE_S16S8S32: return launch_generic_typed<IREE_UK_FLAG_MMT4D_TYPE_S16S8S32>(a, stream);
    case IREE_UK_FLAG_MMT4D_TYPE_S8S4S32: return launch_generic_typed<IREE_UK_FLAG_MMT4D_TYPE_S8S4S32>(a, stream);
    case IREE_UK_FLAG_MMT4D_TYPE_F16F16F16:
    case IREE_UK_FLAG_MMT4D_TYPE_BF16BF16BF16: {
      const int64_t total = a.M * a.N * a.M0 * a.N0;
      if (total <= 0) return IREE_UK_B200_OK;
      const int64_t blocks = std::min<int64_t>((total + 255) / 256, 148 * 64);
      const int skip = (p->flags & IREE_UK_FLAG_MMT4D_SKIP_INTERMEDIATE_ROUNDINGS) ? 1 : 0;
      if ((p->flags & IREE_UK_FLAG_MMT4D_TYPE_MASK) == IREE_UK_FLAG_MMT4D_TYPE_F16F16F16)
        mmt4d_generic_out16_kernel<false><<<int(blocks), 256, 0, stream>>>(a, skip);
      else
        mmt4d_generic_out16_kernel<true><<<int(blocks), 256, 0, stream>>>(a, skip);
      return cuda_status(cudaGetLastError());
    }
    default: return IREE_UK_B200_UNSUPPORTED;
  }
}

int launch_mmt4d_zero_fill(const iree_uk_mmt4d_params_t* p, cudaStream_t stream) {
  GenericArgs a;
  if (!fill_args(p, &a)) return IREE_UK_B200_INVALID_ARGUMENT;
  Mmt4dTypes t;
  mmt4d_types(p->flags, &t);
  const int64_t row_elems = a.N * a.M0 * a.N0;
  const int64_t total = a.M * row_elems;
  if (total <= 0) return IREE_UK_B200_OK;
  const int64_t blocks = std::min<int64_t>((total + 255) / 256, 148 * 16);
  if (elem_bits(t.out) == 32)
    mmt4d_zero_fill_kernel<uint32_t><<<int(blocks), 256, 0, stream>>>(a.out, a.out_stride0, a.M, row_elems);
  else
    mmt4d_zero_fill_kernel<uint16_t><<<int(blocks), 256, 0, stream>>>(a.out, a.out_stride0, a.M, row_elems);
  return cuda_status(cudaGetLastError());
}

bool mmt4d_narrow_eligible(const iree_uk_mmt4d_params_t* p) {
  const uint32_t type = p->flags & IREE_UK_FLAG_MMT4D_TYPE_MASK;
  int k0 = 0, es = 0;
  switch (type) {
    case IREE_UK_FLAG_MMT4D_TYPE_S8S8S32: k0 = 2; es = 1; break;
    case IREE_UK_FLAG_MMT4D_TYPE_F16F16F32: k0 = 1; es = 2; break;
    case IREE_UK_FLAG_MMT4D_TYPE_BF16BF16F32: k0 = 2; es = 2; break;
    default: return false;
  }
  if (p->N0 != 16 || p->K0 != k0 || p->K < 1) return false;
  if (p->M0 != 1 && p->M0 != 2 && p->M0 != 4 && p->M0 != 8) return false;
  if (p->M * p->N > 0x7FFFFFFF) return false;
  // 16-byte loads of the RHS rows, K0-element loads of the LHS
  const uintptr_t lhs = reinterpret_cast<uintptr_t>(p->lhs_buffer) + uintptr_t(p->lhs_offset * es);
  const uintptr_t rhs = reinterpret_cast<uintptr_t>(p->rhs_buffer) + uintptr_t(p->rhs_offset * es);
  const uintptr_t out = reinterpret_cast<uintptr_t>(p->out_buffer) + uintptr_t(p->out_offset * 4);
  return (rhs % 16 == 0) && ((p->rhs_stride0 * es) % 16 == 0) && (lhs % (k0 * es) == 0) &&
         ((p->lhs_stride0 * es) % (k0 * es) == 0) && (out % 4 == 0);
}

namespace {
template <NarrowType T>
int launch_narrow_m0(const GenericArgs& a, int blocks, cudaStream_t stream) {
  // From which M0 on the tensor-core form runs. Measured per call at N = 28672, K = 8192 (M0 = 1,
  // 2, 4, 8; CUDA-core form / tensor-core form): bf16 76 / 69, 80 / 69, 96 / 70, 163 / 84 us;
  // f16 83 / 85, 80 / 87, 104 / 90, 183 / 87 us; s8 40 / 44, 48 / 45, 57 / 46, 105 / 44 us.
  const int mma_from_default = T == NarrowType::BF16 ? 1 : (T == NarrowType::S8 ? 2 : 4);
  const int mma_from = debug_int("IREE_UK_B200_DEBUG_NARROW_MMA_FROM", mma_from_default);
  if (a.M0 >= mma_from) {
    switch (a.M0) {
      case 1: mmt4d_narrow_mma_kernel<T, 1><<<blocks, 256, 0, stream>>>(a); break;
      case 2: mmt4d_narrow_mma_kernel<T, 2><<<blocks, 256, 0, stream>>>(a); break;
      case 4: mmt4d_narrow_mma_kernel<T, 4><<<blocks, 256, 0, stream>>>(a); break;
      default: mmt4d_narrow_mma_kernel<T, 8><<<blocks, 256, 0, stream>>>(a); break;
    }
    return cuda_status(cudaGetLastError());
  }
  switch (a.M0) {
    case 1: mmt4d_narrow_kernel<T, 1><<<blocks, 256, 0, stream>>>(a); break;
    case 2: mmt4d_narrow_kernel<T, 2><<<blocks, 256, 0, stream>>>(a); break;
    case 4: mmt4d_narrow_kernel<T, 4><<<blocks, 256, 0, stream>>>(a); break;
    default: mmt4d_narrow_kernel<T, 8><<<blocks, 256, 0, stream>>>(a); break;
  }
  return cuda_status(cudaGetLastError());
}
}  // namespace

int launch_mmt4d_narrow(const iree_uk_mmt4d_params_t* p, cudaStream_t stream) {
  GenericArgs a;
  if (!fill_args(p, &a)) return IREE_UK_B200_INVALID_ARGUMENT;
  const int64_t blocks = a.M * a.N;
  if (blocks <= 0) return IREE_UK_B200_OK;
  switch (p->flags & IREE_UK_FLAG_MMT4D_TYPE_MASK) {
    case IREE_UK_FLAG_MMT4D_TYPE_S8S8S32: return launch_narrow_m0<NarrowType::S8>(a, int(blocks), stream);
    case IREE_UK_FLAG_MMT4D_TYPE_F16F16F32: return launch_narrow_m0<NarrowType::F16>(a, int(blocks), stream);
    default: return launch_narrow_m0<NarrowType::BF16>(a, int(blocks), stream);
  }
}

bool mmt4d_gemv_s16u4_eligible(const iree_uk_mmt4d_params_t* p) {
  if ((p->flags & IREE_UK_FLAG_MMT4D_TYPE_MASK) != IREE_UK_FLAG_MMT4D_TYPE_S16U4S32) return false;
  if (p->M0 != 1 || p->N0 != 32 || p->K0 != 8 || p->K < 1) return false;
  if (p->M * p->N > 0x7FFFFFFF) return false;
  // 16-byte loads: LHS tile rows are K*16 bytes, RHS tile rows K*128 bytes.
  const uintptr_t lhs = reinterpret_cast<uintptr_t>(p->lhs_buffer) + uintptr_t(p->lhs_offset * 2);
  const uintptr_t rhs = reinterpret_cast<uintptr_t>(p->rhs_buffer) + uintptr_t(p->rhs_offset / 2);
  return (lhs % 16 == 0) && (rhs % 16 == 0) && ((p->lhs_stride0 * 2) % 16 == 0) &&
         ((p->rhs_stride0 / 2) % 16 == 0);
}

int launch_mmt4d_gemv_s16u4(const iree_uk_mmt4d_params_t* p, cudaStream_t stream) {
  GenericArgs a;
  if (!fill_args(p, &a)) return IREE_UK_B200_INVALID_ARGUMENT;
  if (a.M <= 0 || a.N <= 0) return IREE_UK_B200_OK;
  uint32_t* status = device_status_word();
  if (!status) return IREE_UK_B200_CUDA_ERROR;
  // One LHS row per block for the decode call; batches of rows share a pass over the weights
  // four rows at a time.
  if (a.M == 1) {
    mmt4d_gemv_s16u4_kernel<1><<<int(a.N), kGemvBulkWarps * 32, 0, stream>>>(a, status);
  } else {
    const int64_t blocks = (a.M + 3) / 4 * a.N;
    mmt4d_gemv_s16u4_kernel<4><<<int(blocks), kGemvBulkWarps * 32, 0, stream>>>(a, status);
  }
  return cuda_status(cudaGetLastError());
}

}  // namespace uk
