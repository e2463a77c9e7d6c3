// pack / unpack: bandwidth-bound relayouts between a strided 2-D matrix and the 4-D tiled
// layout [outer0][outer1][tile0][tile1].
//
// Two kernel families:
//  * "generic": one thread per tiled element, any parameters the reference accepts.
//  * "staged":  a block moves a rectangle of R0 x R1 tiles through shared memory so that
//    both the matrix side (row segments) and the tiled side (runs of whole tiles) are
//    accessed as long contiguous runs with 16-byte vector instructions where alignment
//    allows. The rectangle is kept in shared memory in matrix form [R0*T0 rows][R1*T1 cols]
//    with an odd pitch (in 32-bit words) so that walking a column is bank-conflict free.
//
// Semantics follow iree_uk_pack_p / iree_uk_unpack_p (ukernel/pack.c:254-322,
// ukernel/unpack.c:190-257): opaque elements of 1, 2 or 4 bytes; padding writes the low
// element-size bytes of padding_value; unpack never writes outside out_size0 x out_size1.
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
  int32_t pitch_words;   // shared-memory row pitch in 32-bit words (odd)
  int32_t tile_fast_r0;  // 1: consecutive tiles of the tiled side walk dim 0 (outer transposed)
  int32_t vec_mat;       // 1: 16-byte vector access to the matrix side is legal
  int32_t vec_tiled;     // 1: 16-byte vector access to the tiled side is legal
  int64_t nblk1;         // blocks along dim 1
};

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

template <int ES>
__global__ void __launch_bounds__(256) pack_staged_kernel(RelayoutArgs a) {
  using E = typename ElemT<ES>::type;
  extern __shared__ uint32_t smem_w[];
  char* smem_b = reinterpret_cast<char*>(smem_w);
  constexpr int NV = 16 / ES;  // elements per 16-byte vector

  const int64_t b0 = blockIdx.x / a.nblk1, b1 = blockIdx.x - b0 * a.nblk1;
  const int64_t tile0_base = b0 * a.R0, tile1_base = b1 * a.R1;
  const int r0n = int(min(int64_t(a.R0), a.outer0 - tile0_base));  // tiles in this block
  const int r1n = int(min(int64_t(a.R1), a.outer1 - tile1_base));
  const int rows = r0n * a.T0, cols = r1n * a.T1;
  const int64_t row_base = tile0_base * a.T0, col_base = tile1_base * a.T1;
  const int pitch_b = a.pitch_words * 4;
  const E padv = E(a.pad);

  // ---- phase 1: matrix rows -> shared memory, padding filled in ----
  if (a.vec_mat && (cols % NV) == 0) {
    const int vpr = cols / NV;
    const int nvec = rows * vpr;
    const uint32_t padw = splat_pad(a.pad, ES);
    for (int vi = threadIdx.x; vi < nvec; vi += blockDim.x) {
      const int r = vi / vpr, cv = vi - r * vpr;
      const int64_t gi0 = row_base + r, gi1 = col_base + int64_t(cv) * NV;
      uint32_t* sw = smem_w + r * a.pitch_words + cv * 4;
      if (gi0 < a.mat_size0 && gi1 + NV <= a.mat_size1) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(
            a.src + (gi0 * a.mat_stride0 + gi1) * ES));
        sw[0] = v.x; sw[1] = v.y; sw[2] = v.z; sw[3] = v.w;
      } else if (gi0 >= a.mat_size0 || gi1 >= a.mat_size1) {
        sw[0] = padw; sw[1] = padw; sw[2] = padw; sw[3] = padw;
      } else {  // vector straddles the right edge
        E* se = reinterpret_cast<E*>(sw);
        for (int j = 0; j < NV; ++j)
          se[j] = (gi1 + j < a.mat_size1)
                      ? reinterpret_cast<const E*>(a.src)[gi0 * a.mat_stride0 + gi1 + j]
                      : padv;
      }
    }
  } else {
    const int nel = rows * cols;
    for (int ei = threadIdx.x; ei < nel; ei += blockDim.x) {
      const int r = ei / cols, c = ei - r * cols;
      const int64_t gi0 = row_base + r, gi1 = col_base + c;
      E v = padv;
      if (gi0 < a.mat_size0 && gi1 < a.mat_size1)
        v = reinterpret_cast<const E*>(a.src)[gi0 * a.mat_stride0 + gi1 * a.mat_stride1];
      *reinterpret_cast<E*>(smem_b + r * pitch_b + c * ES) = v;
    }
  }
  __syncthreads();

  // ---- phase 2: shared memory -> whole tiles, consecutive threads on consecutive bytes ----
  const int tile_elems = a.T0 * a.T1;
  const int ntiles = r0n * r1n;
  // Inside a tile, the element with the unit stride is the "fast" one.
  const bool fast_is_t1 = (a.inner_s1 == 1);
  const int fastN = fast_is_t1 ? a.T1 : a.T0;  // extent of the unit-stride index
  if (a.vec_tiled && (tile_elems % NV) == 0) {
    const int tvec = tile_elems / NV;
    const int nvec = ntiles * tvec;
    for (int vi = threadIdx.x; vi < nvec; vi += blockDim.x) {
      const int tl = vi / tvec, v = vi - tl * tvec;
      int r0, r1;
      if (a.tile_fast_r0) { r1 = tl / r0n; r0 = tl - r1 * r0n; }
      else { r0 = tl / r1n; r1 = tl - r0 * r1n; }
      int e = v * NV;
      int slow = e / fastN, fast = e - slow * fastN;
      E vals[NV];
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        const int t0 = fast_is_t1 ? slow : fast, t1 = fast_is_t1 ? fast : slow;
        vals[j] = *reinterpret_cast<const E*>(smem_b + (r0 * a.T0 + t0) * pitch_b +
                                              (r1 * a.T1 + t1) * ES);
        if (++fast == fastN) { fast = 0; ++slow; }
      }
      const int64_t te = (tile0_base + r0) * a.tiled_stride_o0 +
                         (tile1_base + r1) * a.tiled_stride_o1 + e;
      uint4 out;
      if (ES == 4) {
        out = make_uint4(vals[0], vals[1], vals[2], vals[3]);
      } else {
        uint32_t w[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint32_t x = 0;
#pragma unroll
          for (int j = 0; j < 4 / ES; ++j) x |= uint32_t(vals[q * (4 / ES) + j]) << (8 * ES * j);
          w[q] = x;
        }
        out = make_uint4(w[0], w[1], w[2], w[3]);
      }
      *reinterpret_cast<uint4*>(a.dst + te * ES) = out;
    }
  } else {
    const int nel = ntiles * tile_elems;
    for (int ei = threadIdx.x; ei < nel; ei += blockDim.x) {
      const int tl = ei / tile_elems, e = ei - tl * tile_elems;
      int r0, r1;
      if (a.tile_fast_r0) { r1 = tl / r0n; r0 = tl - r1 * r0n; }
      else { r0 = tl / r1n; r1 = tl - r0 * r1n; }
      const int slow = e / fastN, fast = e - slow * fastN;
      const int t0 = fast_is_t1 ? slow : fast, t1 = fast_is_t1 ? fast : slow;
      const E v = *reinterpret_cast<const E*>(smem_b + (r0 * a.T0 + t0) * pitch_b +
                                              (r1 * a.T1 + t1) * ES);
      const int64_t te = (tile0_base + r0) * a.tiled_stride_o0 +
                         (tile1_base + r1) * a.tiled_stride_o1 + e;
      reinterpret_cast<E*>(a.dst)[te] = v;
    }
  }
}

template <int ES>
__global__ void __launch_bounds__(256) unpack_staged_kernel(RelayoutArgs a) {
  using E = typename ElemT<ES>::type;
  extern __shared__ uint32_t smem_w[];
  char* smem_b = reinterpret_cast<char*>(smem_w);
  constexpr int NV = 16 / ES;

  const int64_t b0 = blockIdx.x / a.nblk1, b1 = blockIdx.x - b0 * a.nblk1;
  const int64_t tile0_base = b0 * a.R0, tile1_base = b1 * a.R1;
  const int r0n = int(min(int64_t(a.R0), a.outer0 - tile0_base));
  const int r1n = int(min(int64_t(a.R1), a.outer1 - tile1_base));
  const int rows = r0n * a.T0, cols = r1n * a.T1;
  const int64_t row_base = tile0_base * a.T0, col_base = tile1_base * a.T1;
  const int pitch_b = a.pitch_words * 4;

  // ---- phase 1: whole tiles -> shared memory (matrix form) ----
  const int tile_elems = a.T0 * a.T1;
  const int ntiles = r0n * r1n;
  const bool fast_is_t1 = (a.inner_s1 == 1);
  const int fastN = fast_is_t1 ? a.T1 : a.T0;
  if (a.vec_tiled && (tile_elems % NV) == 0) {
    const int tvec = tile_elems / NV;
    const int nvec = ntiles * tvec;
    for (int vi = threadIdx.x; vi < nvec; vi += blockDim.x) {
      const int tl = vi / tvec, v = vi - tl * tvec;
      int r0, r1;
      if (a.tile_fast_r0) { r1 = tl / r0n; r0 = tl - r1 * r0n; }
      else { r0 = tl / r1n; r1 = tl - r0 * r1n; }
      const int e = v * NV;
      const int64_t te = (tile0_base + r0) * a.tiled_stride_o0 +
                         (tile1_base + r1) * a.tiled_stride_o1 + e;
      const uint4 in = __ldg(reinterpret_cast<const uint4*>(a.src + te * ES));
      const uint32_t w[4] = {in.x, in.y, in.z, in.w};
      int slow = e / fastN, fast = e - slow * fastN;
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        const int t0 = fast_is_t1 ? slow : fast, t1 = fast_is_t1 ? fast : slow;
        const E val = E(w[(j * ES) / 4] >> (8 * ((j * ES) % 4)));
        *reinterpret_cast<E*>(smem_b + (r0 * a.T0 + t0) * pitch_b + (r1 * a.T1 + t1) * ES) = val;
        if (++fast == fastN) { fast = 0; ++slow; }
      }
    }
  } else {
    const int nel = ntiles * tile_elems;
    for (int ei = threadIdx.x; ei < nel; ei += blockDim.x) {
      const int tl = ei / tile_elems, e = ei - tl * tile_elems;
      int r0, r1;
      if (a.tile_fast_r0) { r1 = tl / r0n; r0 = tl - r1 * r0n; }
      else { r0 = tl / r1n; r1 = tl - r0 * r1n; }
      const int slow = e / fastN, fast = e - slow * fastN;
      const int t0 = fast_is_t1 ? slow : fast, t1 = fast_is_t1 ? fast : slow;
      const int64_t te = (tile0_base + r0) * a.tiled_stride_o0 +
                         (tile1_base + r1) * a.tiled_stride_o1 + e;
      *reinterpret_cast<E*>(smem_b + (r0 * a.T0 + t0) * pitch_b + (r1 * a.T1 + t1) * ES) =
          reinterpret_cast<const E*>(a.src)[te];
    }
  }
  __syncthreads();

  // ---- phase 2: shared memory -> matrix rows; nothing outside mat_size0 x mat_size1 ----
  if (a.vec_mat && (cols % NV) == 0) {
    const int vpr = cols / NV;
    const int nvec = rows * vpr;
    for (int vi = threadIdx.x; vi < nvec; vi += blockDim.x) {
      const int r = vi / vpr, cv = vi - r * vpr;
      const int64_t gi0 = row_base + r, gi1 = col_base + int64_t(cv) * NV;
      if (gi0 >= a.mat_size0 || gi1 >= a.mat_size1) continue;
      const uint32_t* sw = smem_w + r * a.pitch_words + cv * 4;
      if (gi1 + NV <= a.mat_size1) {
        *reinterpret_cast<uint4*>(a.dst + (gi0 * a.mat_stride0 + gi1) * ES) =
            make_uint4(sw[0], sw[1], sw[2], sw[3]);
      } else {
        const E* se = reinterpret_cast<const E*>(sw);
        for (int j = 0; j < NV && gi1 + j < a.mat_size1; ++j)
          reinterpret_cast<E*>(a.dst)[gi0 * a.mat_stride0 + gi1 + j] = se[j];
      }
    }
  } else {
    const int nel = rows * cols;
    for (int ei = threadIdx.x; ei < nel; ei += blockDim.x) {
      const int r = ei / cols, c = ei - r * cols;
      const int64_t gi0 = row_base + r, gi1 = col_base + c;
      if (gi0 < a.mat_size0 && gi1 < a.mat_size1)
        reinterpret_cast<E*>(a.dst)[gi0 * a.mat_stride0 + gi1 * a.mat_stride1] =
            *reinterpret_cast<const E*>(smem_b + r * pitch_b + c * ES);
    }
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
  int64_t pitch_words = (cols * es + 3) / 4;
  if ((pitch_words & 1) == 0) pitch_words += 1;
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

int launch_pack_staged(const iree_uk_pack_params_t* p, cudaStream_t stream) {
  const int es = pack_elem_size(p->flags);
  RelayoutArgs a;
  pack_args(p, es, &a);
  const size_t smem = plan_staged(&a, es, a.src, a.dst);
  if (!smem) return IREE_UK_B200_UNSUPPORTED;
  const int64_t blocks = a.nblk1 * ((a.outer0 + a.R0 - 1) / a.R0);
  switch (es) {
    case 1: pack_staged_kernel<1><<<int(blocks), 256, smem, stream>>>(a); break;
    case 2: pack_staged_kernel<2><<<int(blocks), 256, smem, stream>>>(a); break;
    default: pack_staged_kernel<4><<<int(blocks), 256, smem, stream>>>(a); break;
  }
  return cuda_status(cudaGetLastError());
}

int launch_unpack_staged(const iree_uk_unpack_params_t* p, cudaStream_t stream) {
  const int es = unpack_elem_size(p->flags);
  RelayoutArgs a;
  unpack_args(p, es, &a);
  const size_t smem = plan_staged(&a, es, a.dst, a.src);
  if (!smem) return IREE_UK_B200_UNSUPPORTED;
  const int64_t blocks = a.nblk1 * ((a.outer0 + a.R0 - 1) / a.R0);
  switch (es) {
    case 2: unpack_staged_kernel<2><<<int(blocks), 256, smem, stream>>>(a); break;
    default: unpack_staged_kernel<4><<<int(blocks), 256, smem, stream>>>(a); break;
  }
  return cuda_status(cudaGetLastError());
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
