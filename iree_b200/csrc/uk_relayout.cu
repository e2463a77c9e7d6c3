// pack / unpack: bandwidth-bound relayouts between a strided 2-D matrix and the 4-D tiled
// layout [outer0][outer1][tile0][tile1].
//
// Two kernel families:
//  * "generic": one thread per tiled element, any parameters the reference accepts.
//  * "staged":  a block moves a rectangle of R0 x R1 tiles through shared memory so that
//    both the matrix side (row segments) and the tiled side (runs of whole tiles) are
//    accessed as long contiguous runs with 16-byte vector instructions where alignment
//    allows. The rectangle is kept in shared memory in matrix form [R0*T0 rows][R1*T1 cols]
//    with a 16-byte-aligned row pitch of 4 (mod 8) words. The tile shapes that carry real
//    traffic get constant-shape instantiations whose index arithmetic folds to shifts.
//
// Semantics follow iree_uk_pack_p / iree_uk_unpack_p (ukernel/pack.c:254-322,
// ukernel/unpack.c:190-257): opaque elements of 1, 2 or 4 bytes; padding writes the low
// element-size bytes of padding_value; unpack never writes outside out_size0 x out_size1.
#include <algorithm>
#include "uk_common.h"

namespace uk {
namespace {

// One description serves pack and unpack: `mat` is the 2-D side, `tiled` the 4-D side.
struct RelayoutArgs {
  const char* src;  // pack: matrix, unpack: tiled
  char* dst;        // pack: tiled,  unpack: matrix
  int64_t mat_stride0, mat_stride1;  // elements
  int64_t mat_size0, mat_size1;      // valid extent of the matrix
  int64_t outer0, outer1;            // tile counts along matrix dim 0 / dim 1
  int64_t tiled_stride_o0, tiled_stride_o1;  // element strides of those two tile indices
  int32_t T0, T1;                    // tile extent along matrix dim 0 / dim 1
  int32_t inner_s0, inner_s1;        // element strides of t0 / t1 inside a tile
  uint32_t pad;                      // pack only: low bytes are the fill pattern
  // staged kernels only
  int32_t R0, R1;        // tiles per block along dim 0 / dim 1
  int32_t pitch_words;   // shared-memory row pitch in 32-bit words
  int32_t tile_fast_r0;  // 1: consecutive tiles of the tiled side walk dim 0 (outer transposed)
  int32_t vec_mat;       // 1: 16-byte vector access to the matrix side is legal
  int32_t vec_tiled;     // 1: 16-byte vector access to the tiled side is legal
  int64_t nblk1;         // blocks along dim 1
  int32_t use_bulk;      // constant-shape kernels: move whole matrix rows with bulk async copies
  uint32_t* status;      // per-device status word; bit kStatusRelayoutTimeout on an expired wait
};

constexpr uint32_t kStatusRelayoutTimeout = 1u << 5;

template <int ES> struct ElemT;
template <> struct ElemT<1> { using type = uint8_t; };
template <> struct ElemT<2> { using type = uint16_t; };
template <> struct ElemT<4> { using type = uint32_t; };

// ---------------------------------------------------------------------------------------
// generic kernels
// ---------------------------------------------------------------------------------------

template <int ES, bool IS_PACK>
__global__ void __launch_bounds__(256) relayout_generic_kernel(RelayoutArgs a) {
  using E = typename ElemT<ES>::type;
  const int64_t tile_elems = int64_t(a.T0) * a.T1;
  const int64_t total = a.outer0 * a.outer1 * tile_elems;
  const E padv = E(a.pad);
  for (int64_t idx = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; idx < total;
       idx += int64_t(gridDim.x) * blockDim.x) {
    const int64_t tile = idx / tile_elems;
    const int32_t e = int32_t(idx - tile * tile_elems);
    const int64_t o0 = tile / a.outer1, o1 = tile - o0 * a.outer1;
    const int32_t t0 = e / a.T1, t1 = e - t0 * a.T1;
    const int64_t i0 = o0 * a.T0 + t0, i1 = o1 * a.T1 + t1;
    const int64_t te = o0 * a.tiled_stride_o0 + o1 * a.tiled_stride_o1 +
                       int64_t(t0) * a.inner_s0 + int64_t(t1) * a.inner_s1;
    const bool inside = i0 < a.mat_size0 && i1 < a.mat_size1;
    const int64_t me = i0 * a.mat_stride0 + i1 * a.mat_stride1;
    if (IS_PACK) {
      reinterpret_cast<E*>(a.dst)[te] = inside ? reinterpret_cast<const E*>(a.src)[me] : padv;
    } else if (inside) {
      reinterpret_cast<E*>(a.dst)[me] = reinterpret_cast<const E*>(a.src)[te];
    }
  }
}

// ---------------------------------------------------------------------------------------
// staged kernels
// ---------------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t splat_pad(uint32_t pad, int es) {
  if (es == 1) { pad &= 0xFFu; return pad * 0x01010101u; }
  if (es == 2) { pad &= 0xFFFFu; return pad | (pad << 16); }
  return pad;
}

// Shared-memory row pitch in 32-bit words for `cols_bytes` of payload: a multiple of 4 words
// (rows stay 16-byte aligned for 128-bit shared-memory accesses) that is 4 modulo 8, so that
// walking down a column touches 8 different bank groups before wrapping.
__host__ __device__ constexpr int staged_pitch_words(int cols_bytes) {
  int p = ((cols_bytes + 15) / 16) * 4;
  return (p % 8 == 0) ? p + 4 : p;
}

// Compile-time shape of a staged kernel. kSpec = false: every quantity is read from the
// arguments (any shape). kSpec = true: the tile and block shape are constants, the host has
// checked that every block is full and that both sides allow 16-byte vectors, and index
// arithmetic folds to shifts.
struct RuntimeShape {
  static constexpr bool kSpec = false;
  static constexpr int T0 = 0, T1 = 0, R0 = 0, R1 = 0;
  static constexpr bool kFastT1 = false, kTileFastR0 = false;
};
template <int T0_, int T1_, int R0_, int R1_, bool FAST_T1, bool TILE_FAST_R0>
struct FixedShape {
  static constexpr bool kSpec = true;
  static constexpr int T0 = T0_, T1 = T1_, R0 = R0_, R1 = R1_;
  static constexpr bool kFastT1 = FAST_T1, kTileFastR0 = TILE_FAST_R0;
};

template <int ES, bool IS_PACK, class Shape>
__global__ void __launch_bounds__(256) relayout_staged_kernel(RelayoutArgs a) {
  using E = typename ElemT<ES>::type;
  extern __shared__ __align__(16) uint32_t smem_w[];
  char* smem_b = reinterpret_cast<char*>(smem_w);
  constexpr int NV = 16 / ES;  // elements per 16-byte vector
  constexpr bool kSpec = Shape::kSpec;

  const int T0 = kSpec ? Shape::T0 : a.T0, T1 = kSpec ? Shape::T1 : a.T1;
  const int R0 = kSpec ? Shape::R0 : a.R0, R1 = kSpec ? Shape::R1 : a.R1;
  const bool fast_is_t1 = kSpec ? Shape::kFastT1 : (a.inner_s1 == 1);
  const bool tile_fast_r0 = kSpec ? Shape::kTileFastR0 : (a.tile_fast_r0 != 0);
  const unsigned nblk1 = unsigned(a.nblk1);
  const unsigned b0 = blockIdx.x / nblk1, b1 = blockIdx.x - b0 * nblk1;
  const int64_t tile0_base = int64_t(b0) * R0, tile1_base = int64_t(b1) * R1;
  const int r0n = kSpec ? R0 : int(min(int64_t(R0), a.outer0 - tile0_base));  // tiles here
  const int r1n = kSpec ? R1 : int(min(int64_t(R1), a.outer1 - tile1_base));
  const int rows = r0n * T0, cols = r1n * T1;
  const int64_t row_base = tile0_base * T0, col_base = tile1_base * T1;
  const int pitch_words = kSpec ? staged_pitch_words(Shape::R1 * Shape::T1 * ES) : a.pitch_words;
  const int pitch_b = pitch_words * 4;
  const int tile_elems = T0 * T1;
  const int ntiles = r0n * r1n;
  const int fastN = fast_is_t1 ? T1 : T0;  // extent of the unit-stride index inside a tile
  const bool vec_mat = kSpec || (a.vec_mat && (cols % NV) == 0);
  const bool vec_tiled = kSpec || (a.vec_tiled && (tile_elems % NV) == 0);
  // A 16-byte vector of a tile is also contiguous in the staged (matrix-form) rectangle when
  // the tile's unit-stride index runs along the matrix row and a run is whole vectors.
  const bool row_vectors = fast_is_t1 && ((T1 * ES) % 16 == 0);
  const E padv = E(a.pad);

  const char* mat_src = a.src;  // used when IS_PACK
  char* mat_dst = a.dst;        // used when !IS_PACK
  const char* tiled_src = a.src;
  char* tiled_dst = a.dst;

  // tile index inside the block -> (r0, r1); consecutive tiles are adjacent on the tiled side
  auto tile_rc = [&](unsigned tl, int* r0, int* r1) {
    if (tile_fast_r0) { *r1 = int(tl / unsigned(r0n)); *r0 = int(tl - unsigned(*r1) * unsigned(r0n)); }
    else { *r0 = int(tl / unsigned(r1n)); *r1 = int(tl - unsigned(*r0) * unsigned(r1n)); }
  };
  auto smem_at = [&](int r0, int r1, int slow, int fast) -> char* {
    const int t0 = fast_is_t1 ? slow : fast, t1 = fast_is_t1 ? fast : slow;
    return smem_b + (r0 * T0 + t0) * pitch_b + (r1 * T1 + t1) * ES;
  };

  // ---- matrix side <-> shared memory: row segments ----
  auto matrix_phase = [&]() {
    if (vec_mat) {
      const unsigned vpr = unsigned(cols) / NV;
      const unsigned nvec = unsigned(rows) * vpr;
      const uint32_t padw = splat_pad(a.pad, ES);
      for (unsigned vi = threadIdx.x; vi < nvec; vi += blockDim.x) {
        const unsigned r = vi / vpr, cv = vi - r * vpr;
        const int64_t gi0 = row_base + r, gi1 = col_base + int64_t(cv) * NV;
        uint4* sv = reinterpret_cast<uint4*>(smem_w + r * pitch_words + cv * 4);
        if (IS_PACK) {
          if (gi0 < a.mat_size0 && gi1 + NV <= a.mat_size1) {
            *sv = __ldg(reinterpret_cast<const uint4*>(mat_src + (gi0 * a.mat_stride0 + gi1) * ES));
          } else if (gi0 >= a.mat_size0 || gi1 >= a.mat_size1) {
            *sv = make_uint4(padw, padw, padw, padw);
          } else {  // vector straddles the right edge
            E* se = reinterpret_cast<E*>(sv);
            for (int j = 0; j < NV; ++j)
              se[j] = (gi1 + j < a.mat_size1)
                          ? reinterpret_cast<const E*>(mat_src)[gi0 * a.mat_stride0 + gi1 + j]
                          : padv;
          }
        } else {
          if (gi0 >= a.mat_size0 || gi1 >= a.mat_size1) continue;
          if (gi1 + NV <= a.mat_size1) {
            *reinterpret_cast<uint4*>(mat_dst + (gi0 * a.mat_stride0 + gi1) * ES) = *sv;
          } else {
            const E* se = reinterpret_cast<const E*>(sv);
            for (int j = 0; j < NV && gi1 + j < a.mat_size1; ++j)
              reinterpret_cast<E*>(mat_dst)[gi0 * a.mat_stride0 + gi1 + j] = se[j];
          }
        }
      }
    } else {
      const unsigned nel = unsigned(rows) * unsigned(cols);
      for (unsigned ei = threadIdx.x; ei < nel; ei += blockDim.x) {
        const unsigned r = ei / unsigned(cols), c = ei - r * unsigned(cols);
        const int64_t gi0 = row_base + r, gi1 = col_base + c;
        E* sp = reinterpret_cast<E*>(smem_b + r * pitch_b + c * ES);
        const bool inside = gi0 < a.mat_size0 && gi1 < a.mat_size1;
        const int64_t me = gi0 * a.mat_stride0 + gi1 * a.mat_stride1;
        if (IS_PACK) *sp = inside ? reinterpret_cast<const E*>(mat_src)[me] : padv;
        else if (inside) reinterpret_cast<E*>(mat_dst)[me] = *sp;
      }
    }
  };

  // ---- tiled side <-> shared memory: runs of whole tiles ----
  auto tiled_phase = [&]() {
    if (vec_tiled) {
      const unsigned tvec = unsigned(tile_elems) / NV;
      const unsigned nvec = unsigned(ntiles) * tvec;
      for (unsigned vi = threadIdx.x; vi < nvec; vi += blockDim.x) {
        const unsigned tl = vi / tvec, v = vi - tl * tvec;
        int r0, r1;
        tile_rc(tl, &r0, &r1);
        const int e = int(v) * NV;
        int slow = int(unsigned(e) / unsigned(fastN)), fast = e - slow * fastN;
        const int64_t te = (tile0_base + r0) * a.tiled_stride_o0 +
                           (tile1_base + r1) * a.tiled_stride_o1 + e;
        if (row_vectors) {
          uint4* sv = reinterpret_cast<uint4*>(smem_at(r0, r1, slow, fast));
          if (IS_PACK) *reinterpret_cast<uint4*>(tiled_dst + te * ES) = *sv;
          else *sv = __ldg(reinterpret_cast<const uint4*>(tiled_src + te * ES));
        } else if (IS_PACK) {
          uint32_t w[4] = {0u, 0u, 0u, 0u};
#pragma unroll
          for (int j = 0; j < NV; ++j) {
            const uint32_t val = *reinterpret_cast<const E*>(smem_at(r0, r1, slow, fast));
            w[(j * ES) / 4] |= val << (8 * ((j * ES) % 4));
            if (++fast == fastN) { fast = 0; ++slow; }
          }
          *reinterpret_cast<uint4*>(tiled_dst + te * ES) = make_uint4(w[0], w[1], w[2], w[3]);
        } else {
          const uint4 in = __ldg(reinterpret_cast<const uint4*>(tiled_src + te * ES));
          const uint32_t w[4] = {in.x, in.y, in.z, in.w};
#pragma unroll
          for (int j = 0; j < NV; ++j) {
            *reinterpret_cast<E*>(smem_at(r0, r1, slow, fast)) =
                E(w[(j * ES) / 4] >> (8 * ((j * ES) % 4)));
            if (++fast == fastN) { fast = 0; ++slow; }
          }
        }
      }
    } else {
      const unsigned nel = unsigned(ntiles) * unsigned(tile_elems);
      for (unsigned ei = threadIdx.x; ei < nel; ei += blockDim.x) {
        const unsigned tl = ei / unsigned(tile_elems), e = ei - tl * unsigned(tile_elems);
        int r0, r1;
        tile_rc(tl, &r0, &r1);
        const int slow = int(e / unsigned(fastN)), fast = int(e) - slow * fastN;
        const int64_t te = (tile0_base + r0) * a.tiled_stride_o0 +
                           (tile1_base + r1) * a.tiled_stride_o1 + e;
        E* sp = reinterpret_cast<E*>(smem_at(r0, r1, slow, fast));
        if (IS_PACK) reinterpret_cast<E*>(tiled_dst)[te] = *sp;
        else *sp = reinterpret_cast<const E*>(tiled_src)[te];
      }
    }
  };

  // Constant-shape blocks that lie wholly inside the matrix move their matrix-side rows (one
  // contiguous, 16-byte aligned segment per row) with bulk asynchronous copies: no registers,
  // no per-vector instructions, every row of the block in flight at once.
  __shared__ __align__(8) uint64_t row_bar;
  const bool bulk = kSpec && a.use_bulk && row_base + rows <= a.mat_size0 &&
                    col_base + cols <= a.mat_size1;
  const uint32_t row_bytes = uint32_t(cols) * ES;
  if (IS_PACK && bulk) {
    const uint32_t bar = static_cast<uint32_t>(__cvta_generic_to_shared(&row_bar));
    if (threadIdx.x == 0) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(rows) : "memory");
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    for (int r = threadIdx.x; r < rows; r += blockDim.x) {
      const char* g = mat_src + ((row_base + r) * a.mat_stride0 + col_base) * ES;
      const uint32_t sdst = static_cast<uint32_t>(__cvta_generic_to_shared(smem_b + r * pitch_b));
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(row_bytes) : "memory");
      asm volatile(
          "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
          :: "r"(sdst), "l"(g), "r"(row_bytes), "r"(bar) : "memory");
    }
    // Bounded wait for all rows of the block. If it runs out, the block records that in the
    // status word, writes nothing (its tiles would hold whatever had landed), gives its copies
    // a second bounded wait so that none is still in flight into shared memory that is about
    // to be released, and returns.
    auto wait_rows = [&]() {
      const long long deadline = clock64() + (1ll << 31);
      uint32_t done = 0;
      while (!done && clock64() < deadline) {
        asm volatile(
            "{\n.reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n"
            "selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(done) : "r"(bar) : "memory");
      }
      return done != 0;
    };
    const bool landed = __syncthreads_and(wait_rows() ? 1 : 0) != 0;
    if (!landed) {
      if (threadIdx.x == 0) {
        atomicOr(a.status, kStatusRelayoutTimeout);
        wait_rows();
      }
      __syncthreads();
      return;
    }
    tiled_phase();
    return;
  }
  if (!IS_PACK && bulk) {
    tiled_phase();   // whole tiles -> shared memory (generic-proxy stores)
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    for (int r = threadIdx.x; r < rows; r += blockDim.x) {
      char* g = mat_dst + ((row_base + r) * a.mat_stride0 + col_base) * ES;
      const uint32_t ssrc = static_cast<uint32_t>(__cvta_generic_to_shared(smem_b + r * pitch_b));
      asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                   :: "l"(g), "r"(ssrc), "r"(row_bytes) : "memory");
    }
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // shared memory is released at exit
    return;
  }

  if (IS_PACK) {
    matrix_phase();  // matrix rows -> shared memory, padding filled in
    __syncthreads();
    tiled_phase();   // shared memory -> whole tiles
  } else {
    tiled_phase();   // whole tiles -> shared memory
    __syncthreads();
    matrix_phase();  // shared memory -> matrix rows; nothing outside mat_size0 x mat_size1
  }
}

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------

// Fills the fields common to the generic and staged kernels. Outer / inner transposition
// is expressed as strides (ukernel/pack.c:260-272, unpack.c:196-210).
void describe_tiled(int64_t size0, int64_t size1, int64_t size2, int64_t size3, int64_t stride0,
                    bool transpose_outer, bool transpose_inner, RelayoutArgs* a) {
  // Physical tiled array: [size0][size1][size2][size3], strides (stride0, size2*size3, size3, 1).
  int64_t outer0 = size0, outer1 = size1;
  int64_t so0 = stride0, so1 = size2 * size3;
  int64_t T0 = size2, T1 = size3, s0 = size3, s1 = 1;
  if (transpose_outer) { std::swap(outer0, outer1); std::swap(so0, so1); }
  if (transpose_inner) { std::swap(T0, T1); std::swap(s0, s1); }
  // A one-element extent has no stride of its own: make the other index the unit-stride one.
  if (T0 == 1) s1 = 1;
  if (T1 == 1 && T0 != 1) { s0 = 1; s1 = T0; }
  a->outer0 = outer0; a->outer1 = outer1;
  a->tiled_stride_o0 = so0; a->tiled_stride_o1 = so1;
  a->T0 = int32_t(T0); a->T1 = int32_t(T1);
  a->inner_s0 = int32_t(s0); a->inner_s1 = int32_t(s1);
  a->tile_fast_r0 = transpose_outer ? 1 : 0;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Chooses the block rectangle and the vector flags. Returns the dynamic shared-memory
// bytes, or 0 when the staged kernel should not be used.
size_t plan_staged(RelayoutArgs* a, int es, const char* mat_base, const char* tiled_base) {
  if (a->outer0 <= 0 || a->outer1 <= 0 || a->T0 <= 0 || a->T1 <= 0) return 0;
  if (a->inner_s1 != 1 && a->inner_s0 != 1) return 0;
  const int64_t tile_bytes = int64_t(a->T0) * a->T1 * es;
  const int64_t kTarget = 16 * 1024;
  int64_t R0 = 1, R1 = 1;
  const int nv = 16 / es;
  // R1 multiple that keeps block column offsets 16-byte aligned on the matrix side.
  int64_t r1_quantum = 1;
  while ((r1_quantum * a->T1) % nv) r1_quantum *= 2;
  if (!a->tile_fast_r0) {
    R1 = std::max<int64_t>(1, kTarget / tile_bytes);
  } else {
    R1 = std::max<int64_t>(1, (256 + int64_t(a->T1) * es - 1) / (int64_t(a->T1) * es));
  }
  R1 = (R1 + r1_quantum - 1) / r1_quantum * r1_quantum;
  if (R1 > a->outer1) R1 = a->outer1;
  R0 = std::max<int64_t>(1, kTarget / (tile_bytes * R1));
  if (!a->tile_fast_r0) R0 = 1;
  if (R0 > a->outer0) R0 = a->outer0;
  const int64_t rows = R0 * a->T0, cols = R1 * a->T1;
  const int64_t pitch_words = staged_pitch_words(int(cols * es));
  const int64_t smem = rows * pitch_words * 4;
  if (smem > 46 * 1024) return 0;
  a->R0 = int32_t(R0); a->R1 = int32_t(R1);
  a->pitch_words = int32_t(pitch_words);
  a->nblk1 = (a->outer1 + R1 - 1) / R1;
  const int64_t nblk0 = (a->outer0 + R0 - 1) / R0;
  if (a->nblk1 * nblk0 > 0x7FFFFFFF) return 0;
  a->vec_mat = (a->mat_stride1 == 1 && aligned16(mat_base) && (a->mat_stride0 * es) % 16 == 0 &&
                (cols * es) % 16 == 0)
                   ? 1 : 0;
  a->vec_tiled = (aligned16(tiled_base) && tile_bytes % 16 == 0 &&
                  (a->tiled_stride_o0 * es) % 16 == 0 && (a->tiled_stride_o1 * es) % 16 == 0)
                     ? 1 : 0;
  return size_t(smem);
}

template <bool IS_PACK>
int launch_generic(const RelayoutArgs& a, int es, cudaStream_t stream) {
  const int64_t total = a.outer0 * a.outer1 * a.T0 * a.T1;
  if (total <= 0) return IREE_UK_B200_OK;
  const int threads = 256;
  const int64_t blocks = std::min<int64_t>((total + threads - 1) / threads, 148 * 32);
  switch (es) {
    case 1: relayout_generic_kernel<1, IS_PACK><<<int(blocks), threads, 0, stream>>>(a); break;
    case 2: relayout_generic_kernel<2, IS_PACK><<<int(blocks), threads, 0, stream>>>(a); break;
    default: relayout_generic_kernel<4, IS_PACK><<<int(blocks), threads, 0, stream>>>(a); break;
  }
  return cuda_status(cudaGetLastError());
}

void pack_args(const iree_uk_pack_params_t* p, int es, RelayoutArgs* a) {
  *a = RelayoutArgs{};
  a->src = static_cast<const char*>(p->in_buffer) + p->in_offset * es;
  a->dst = static_cast<char*>(p->out_buffer) + p->out_offset * es;
  a->mat_stride0 = p->in_stride0; a->mat_stride1 = p->in_stride1;
  a->mat_size0 = p->in_size0; a->mat_size1 = p->in_size1;
  a->pad = uint32_t(p->padding_value);
  describe_tiled(p->out_size0, p->out_size1, p->out_size2, p->out_size3, p->out_stride0,
                 (p->flags & IREE_UK_FLAG_PACK_TRANSPOSE_OUTER) != 0,
                 (p->flags & IREE_UK_FLAG_PACK_TRANSPOSE_INNER) != 0, a);
}

void unpack_args(const iree_uk_unpack_params_t* p, int es, RelayoutArgs* a) {
  *a = RelayoutArgs{};
  a->src = static_cast<const char*>(p->in_buffer) + p->in_offset * es;
  a->dst = static_cast<char*>(p->out_buffer) + p->out_offset * es;
  a->mat_stride0 = p->out_stride0; a->mat_stride1 = p->out_stride1;
  a->mat_size0 = p->out_size0; a->mat_size1 = p->out_size1;
  describe_tiled(p->in_size0, p->in_size1, p->in_size2, p->in_size3, p->in_stride0,
                 (p->flags & IREE_UK_FLAG_UNPACK_TRANSPOSE_OUTER) != 0,
                 (p->flags & IREE_UK_FLAG_UNPACK_TRANSPOSE_INNER) != 0, a);
}

}  // namespace

int launch_pack_generic(const iree_uk_pack_params_t* p, cudaStream_t stream) {
  const int es = pack_elem_size(p->flags);
  RelayoutArgs a;
  pack_args(p, es, &a);
  return launch_generic<true>(a, es, stream);
}

int launch_unpack_generic(const iree_uk_unpack_params_t* p, cudaStream_t stream) {
  const int es = unpack_elem_size(p->flags);
  RelayoutArgs a;
  unpack_args(p, es, &a);
  return launch_generic<false>(a, es, stream);
}

bool pack_staged_eligible(const iree_uk_pack_params_t* p) {
  const int es = pack_elem_size(p->flags);
  RelayoutArgs a;
  pack_args(p, es, &a);
  return plan_staged(&a, es, a.src, a.dst) != 0;
}

bool unpack_staged_eligible(const iree_uk_unpack_params_t* p) {
  const int es = unpack_elem_size(p->flags);
  RelayoutArgs a;
  unpack_args(p, es, &a);
  return plan_staged(&a, es, a.dst, a.src) != 0;
}

namespace {

// True when a launch with constant shape (T0, T1, R0, R1) is legal for the planned problem:
// same tile, block shape overridden to the constants, all blocks full, vectors on both sides.
template <class Shape>
bool fits_fixed_shape(const RelayoutArgs& a, int es, const char* mat_base, const char* tiled_base) {
  if (a.T0 != Shape::T0 || a.T1 != Shape::T1) return false;
  if ((a.inner_s1 == 1) != Shape::kFastT1 && !(a.T0 == 1 || a.T1 == 1)) return false;
  if ((a.tile_fast_r0 != 0) != Shape::kTileFastR0) return false;
  if (a.outer0 % Shape::R0 || a.outer1 % Shape::R1) return false;
  const int64_t tile_bytes = int64_t(a.T0) * a.T1 * es;
  const bool vec_mat = a.mat_stride1 == 1 && aligned16(mat_base) && (a.mat_stride0 * es) % 16 == 0 &&
                       (int64_t(Shape::R1) * Shape::T1 * es) % 16 == 0;
  const bool vec_tiled = aligned16(tiled_base) && tile_bytes % 16 == 0 &&
                         (a.tiled_stride_o0 * es) % 16 == 0 && (a.tiled_stride_o1 * es) % 16 == 0;
  return vec_mat && vec_tiled &&
         (a.outer0 / Shape::R0) * (a.outer1 / Shape::R1) <= 0x7FFFFFFF;
}

template <int ES, bool IS_PACK, class Shape>
int launch_fixed(RelayoutArgs a, cudaStream_t stream) {
  a.R0 = Shape::R0; a.R1 = Shape::R1;
  a.nblk1 = a.outer1 / Shape::R1;
  a.status = device_status_word();
  a.use_bulk = a.status ? 1 : 0;  // the bulk-row path reports an expired wait through the status word
  const int64_t blocks = a.nblk1 * (a.outer0 / Shape::R0);
  constexpr int pitch = staged_pitch_words(Shape::R1 * Shape::T1 * ES);
  constexpr size_t smem = size_t(Shape::R0) * Shape::T0 * pitch * 4;
  static_assert(smem <= 48 * 1024, "fixed shape exceeds the default shared-memory limit");
  relayout_staged_kernel<ES, IS_PACK, Shape><<<int(blocks), 256, smem, stream>>>(a);
  return cuda_status(cudaGetLastError());
}

// Constant-shape instantiations for the tile shapes that carry real traffic (the tiles the
// reference's x86-64 encoder picks, Codegen/ExternalInterfaces/CPUEncodingExternalModels.cpp:
// 479-585): LHS-style 16xK0 tiles, RHS-style tiles packed with both transposes, and 16x16
// accumulator tiles. (T0, T1) are extents along matrix rows / columns.
using Pack16x1   = FixedShape<16, 1, 1, 256, false, false>;  // f32 [M][K] -> [M1][K1][16][1]
using Pack16x2   = FixedShape<16, 2, 1, 256, true, false>;   // bf16/i8 [M][K] -> [M1][K1][16][2]
// RHS-style packs read a block of matrix rows whose segments go to different tile rows. Blocks
// of few, long row segments (8 rows x 2 KB) keep their rate when the memory system is slow (a
// GPU warmed up by a long GEMM: 0.98-1.03 of a same-size copy, where 64 rows x 256 bytes fell to
// 0.79); the many-short-rows shapes remain for matrices the long ones do not divide.
using PackT1x16  = FixedShape<1, 16, 8, 32, true, true>;     // [K][N] -> [N1][K1][16][1], 0x300
using PackT1x16Small = FixedShape<1, 16, 64, 4, true, true>;
using PackT2x16  = FixedShape<2, 16, 4, 64, false, true>;    // [K][N] -> [N1][K1][16][2], 0x300
using PackT2x16Small = FixedShape<2, 16, 32, 8, false, true>;
using Tile16x16  = FixedShape<16, 16, 1, 16, true, false>;   // accumulator tiles

template <int ES, bool IS_PACK>
int launch_staged(RelayoutArgs& a, const char* mat_base, const char* tiled_base,
                  cudaStream_t stream) {
#define UK_TRY_FIXED(SHAPE)                                         \
  if (fits_fixed_shape<SHAPE>(a, ES, mat_base, tiled_base))         \
    return launch_fixed<ES, IS_PACK, SHAPE>(a, stream);
  UK_TRY_FIXED(Pack16x1)
  UK_TRY_FIXED(Pack16x2)
  UK_TRY_FIXED(PackT1x16)
  UK_TRY_FIXED(PackT1x16Small)
  UK_TRY_FIXED(PackT2x16)
  UK_TRY_FIXED(PackT2x16Small)
  UK_TRY_FIXED(Tile16x16)
#undef UK_TRY_FIXED
  const size_t smem = plan_staged(&a, ES, mat_base, tiled_base);
  if (!smem) return IREE_UK_B200_UNSUPPORTED;
  const int64_t blocks = a.nblk1 * ((a.outer0 + a.R0 - 1) / a.R0);
  relayout_staged_kernel<ES, IS_PACK, RuntimeShape><<<int(blocks), 256, smem, stream>>>(a);
  return cuda_status(cudaGetLastError());
}

}  // namespace

int launch_pack_staged(const iree_uk_pack_params_t* p, cudaStream_t stream) {
  const int es = pack_elem_size(p->flags);
  RelayoutArgs a;
  pack_args(p, es, &a);
  switch (es) {
    case 1: return launch_staged<1, true>(a, a.src, a.dst, stream);
    case 2: return launch_staged<2, true>(a, a.src, a.dst, stream);
    default: return launch_staged<4, true>(a, a.src, a.dst, stream);
  }
}

int launch_unpack_staged(const iree_uk_unpack_params_t* p, cudaStream_t stream) {
  const int es = unpack_elem_size(p->flags);
  RelayoutArgs a;
  unpack_args(p, es, &a);
  switch (es) {
    case 2: return launch_staged<2, false>(a, a.dst, a.src, stream);
    default: return launch_staged<4, false>(a, a.dst, a.src, stream);
  }
}

// ---------------------------------------------------------------------------------------
// slab interleave for the sharded output (no reference counterpart)
// ---------------------------------------------------------------------------------------
namespace {
__global__ void __launch_bounds__(256) interleave_slabs_kernel(const uint4* __restrict__ in,
                                                               uint4* __restrict__ out, int64_t M,
                                                               int64_t n_per, int64_t tile_vecs,
                                                               int world) {
  // in: [world][M][n_per][tile_vecs], out: [M][world*n_per][tile_vecs]
  const int64_t row_vecs = n_per * tile_vecs;
  const int64_t total = int64_t(world) * M * row_vecs;
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < total;
       i += int64_t(gridDim.x) * blockDim.x) {
    const int64_t r = i / (M * row_vecs);
    const int64_t rem = i - r * (M * row_vecs);
    const int64_t m = rem / row_vecs, c = rem - m * row_vecs;
    out[(m * world + r) * row_vecs + c] = in[i];
  }
}
}  // namespace

int launch_interleave_slabs(const void* gathered, void* out, int64_t M, int64_t N,
                            int64_t tile_elems, int elem_size, int world, cudaStream_t stream) {
  if (world <= 0 || N % world || (tile_elems * elem_size) % 16 || !aligned16(gathered) ||
      !aligned16(out))
    return IREE_UK_B200_INVALID_ARGUMENT;
  const int64_t tile_vecs = tile_elems * elem_size / 16;
  const int64_t total = M * N * tile_vecs;
  if (total == 0) return IREE_UK_B200_OK;
  const int64_t blocks = std::min<int64_t>((total + 255) / 256, 148 * 16);
  interleave_slabs_kernel<<<int(blocks), 256, 0, stream>>>(
      static_cast<const uint4*>(gathered), static_cast<uint4*>(out), M, N / world, tile_vecs,
      world);
  return cuda_status(cudaGetLastError());
}

}  // namespace uk
