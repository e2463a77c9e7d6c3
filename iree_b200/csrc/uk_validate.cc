// Host-side argument checks. The reference asserts these conditions in debug builds and
// treats the rest of each ukernel as infallible; here a violated condition is reported to
// the caller and nothing is launched.
#include <cstdlib>
#include <cstring>

#include "uk_common.h"

namespace uk {

bool env_flag(const char* name) {
  const char* v = std::getenv(name);
  return v && v[0] && std::strcmp(v, "0") != 0;
}

#ifdef IREE_UK_B200_EXPERIMENTS
int debug_int(const char* name, int fallback) {
  const char* v = std::getenv(name);
  return v ? std::atoi(v) : fallback;
}
#endif

bool mmt4d_types(uint32_t flags, Mmt4dTypes* t) {
  switch (flags & IREE_UK_FLAG_MMT4D_TYPE_MASK) {
    case IREE_UK_FLAG_MMT4D_TYPE_F32F32F32: *t = {Elem::F32, Elem::F32, Elem::F32}; return true;
    case IREE_UK_FLAG_MMT4D_TYPE_S8S8S32: *t = {Elem::S8, Elem::S8, Elem::S32}; return true;
    case IREE_UK_FLAG_MMT4D_TYPE_F16F16F32: *t = {Elem::F16, Elem::F16, Elem::F32}; return true;
    case IREE_UK_FLAG_MMT4D_TYPE_F16F16F16: *t = {Elem::F16, Elem::F16, Elem::F16}; return true;
    case IREE_UK_FLAG_MMT4D_TYPE_BF16BF16F32: *t = {Elem::BF16, Elem::BF16, Elem::F32}; return true;
    case IREE_UK_FLAG_MMT4D_TYPE_BF16BF16BF16: *t = {Elem::BF16, Elem::BF16, Elem::BF16}; return true;
    case IREE_UK_FLAG_MMT4D_TYPE_S16S16S32: *t = {Elem::S16, Elem::S16, Elem::S32}; return true;
    case IREE_UK_FLAG_MMT4D_TYPE_S16U4S32: *t = {Elem::S16, Elem::U4, Elem::S32}; return true;
    case IREE_UK_FLAG_MMT4D_TYPE_S16S8S32: *t = {Elem::S16, Elem::S8, Elem::S32}; return true;
    case IREE_UK_FLAG_MMT4D_TYPE_S8S4S32: *t = {Elem::S8, Elem::S4, Elem::S32}; return true;
    default: return false;
  }
}

int pack_elem_size(uint32_t flags) {
  switch (flags & IREE_UK_FLAG_PACK_TYPE_MASK) {
    case IREE_UK_FLAG_PACK_TYPE_F32F32: return 4;
    case IREE_UK_FLAG_PACK_TYPE_I8I8: return 1;
    case IREE_UK_FLAG_PACK_TYPE_I32I32: return 4;
    case IREE_UK_FLAG_PACK_TYPE_F16F16: return 2;
    case IREE_UK_FLAG_PACK_TYPE_BF16BF16: return 2;
    default: return 0;
  }
}

int unpack_elem_size(uint32_t flags) {
  switch (flags & IREE_UK_FLAG_UNPACK_TYPE_MASK) {
    case IREE_UK_FLAG_UNPACK_TYPE_F32F32: return 4;
    case IREE_UK_FLAG_UNPACK_TYPE_I32I32: return 4;
    case IREE_UK_FLAG_UNPACK_TYPE_F16F16: return 2;
    case IREE_UK_FLAG_UNPACK_TYPE_BF16BF16: return 2;
    default: return 0;
  }
}

static bool in_unsigned_range(int64_t v, int bits) { return v >= 0 && v < (int64_t(1) << bits); }

// ukernel/mmt4d.c:12-48. Two deliberate differences, both stricter: type id 0 (NONE) is
// rejected (the reference lets it through the assert and then misbehaves), and the
// whole-byte rules for the right-hand side use the RHS element width (the reference
// computes `rhs_bits` from the LHS type, mmt4d.c:41, and relies on the exact-bytes
// assertions of mmt4d.c:72-80 instead).
int validate_mmt4d(const iree_uk_mmt4d_params_t* p) {
  if (!p) return IREE_UK_B200_INVALID_ARGUMENT;
  const uint32_t allflags = IREE_UK_FLAG_MMT4D_TYPE_MASK | IREE_UK_FLAG_MMT4D_ACCUMULATE |
                            IREE_UK_FLAG_MMT4D_SKIP_INTERMEDIATE_ROUNDINGS |
                            IREE_UK_FLAG_MMT4D_ALLOW_GENERIC_FALLBACK_TILE_FUNCTION;
  if (p->flags & ~allflags) return IREE_UK_B200_INVALID_ARGUMENT;
  Mmt4dTypes t;
  if (!mmt4d_types(p->flags, &t)) return IREE_UK_B200_INVALID_ARGUMENT;
  if (!in_unsigned_range(p->M, 31) || !in_unsigned_range(p->N, 31) ||
      !in_unsigned_range(p->K, 31))
    return IREE_UK_B200_INVALID_ARGUMENT;
  if (!in_unsigned_range(p->M0, 15) || !in_unsigned_range(p->N0, 15) ||
      !in_unsigned_range(p->K0, 15))
    return IREE_UK_B200_INVALID_ARGUMENT;
  if (elem_bits(t.out) < 8) return IREE_UK_B200_INVALID_ARGUMENT;
  const int lb = elem_bits(t.lhs), rb = elem_bits(t.rhs);
  if ((int64_t(p->K0) * lb) % 8 || (int64_t(p->K0) * rb) % 8) return IREE_UK_B200_INVALID_ARGUMENT;
  if ((p->lhs_stride0 * lb) % 8 || (p->rhs_stride0 * rb) % 8) return IREE_UK_B200_INVALID_ARGUMENT;
  if ((p->lhs_offset * lb) % 8 || (p->rhs_offset * rb) % 8) return IREE_UK_B200_INVALID_ARGUMENT;
  return IREE_UK_B200_OK;
}

static int ceil_log2_u32(uint32_t n) {
  if (n <= 1) return 0;
  int l = 0;
  uint32_t v = n - 1;
  while (v) { v >>= 1; ++l; }
  return l;
}

// The reference pads through a 4096-byte temporary and asserts that one tile, rounded up
// to a power of two, fits (ukernel/pack.c:9,37-48, unpack.c:9-29). This library has no such
// buffer but accepts exactly the same tiles.
static bool tile_fits_reference_tmpbuf(int64_t t0, int64_t t1, int64_t elem_size) {
  const int64_t bytes = t0 * t1 * elem_size;
  if (bytes < 0 || bytes > 4096) return false;
  return (4096 >> ceil_log2_u32(uint32_t(bytes))) > 0;
}

// ukernel/pack.c:51-104
int validate_pack(const iree_uk_pack_params_t* p) {
  if (!p) return IREE_UK_B200_INVALID_ARGUMENT;
  const uint32_t allflags = IREE_UK_FLAG_PACK_TRANSPOSE_INNER |
                            IREE_UK_FLAG_PACK_TRANSPOSE_OUTER | IREE_UK_FLAG_PACK_TYPE_MASK;
  if (p->flags & ~allflags) return IREE_UK_B200_INVALID_ARGUMENT;
  const int es = pack_elem_size(p->flags);
  if (!es) return IREE_UK_B200_INVALID_ARGUMENT;
  if (p->in_size0 < 0 || p->in_size1 < 0 || p->out_size0 < 0 || p->out_size1 < 0 ||
      p->out_size2 < 0 || p->out_size3 < 0 || p->in_stride0 < 0 || p->in_stride1 < 0 ||
      p->out_stride0 < 0)
    return IREE_UK_B200_INVALID_ARGUMENT;
  if (p->out_stride1 != p->out_size2 * p->out_size3) return IREE_UK_B200_INVALID_ARGUMENT;
  int64_t outer0 = p->out_size0, outer1 = p->out_size1;
  int64_t tile0 = p->out_size2, tile1 = p->out_size3;
  if (p->flags & IREE_UK_FLAG_PACK_TRANSPOSE_OUTER) { int64_t t = outer0; outer0 = outer1; outer1 = t; }
  if (p->flags & IREE_UK_FLAG_PACK_TRANSPOSE_INNER) { int64_t t = tile0; tile0 = tile1; tile1 = t; }
  if (outer0 * tile0 < p->in_size0 || outer1 * tile1 < p->in_size1)
    return IREE_UK_B200_INVALID_ARGUMENT;
  if (!tile_fits_reference_tmpbuf(tile0, tile1, es)) return IREE_UK_B200_INVALID_ARGUMENT;
  return IREE_UK_B200_OK;
}

// ukernel/unpack.c:31-82
int validate_unpack(const iree_uk_unpack_params_t* p) {
  if (!p) return IREE_UK_B200_INVALID_ARGUMENT;
  const uint32_t allflags = IREE_UK_FLAG_UNPACK_TRANSPOSE_INNER |
                            IREE_UK_FLAG_UNPACK_TRANSPOSE_OUTER | IREE_UK_FLAG_UNPACK_TYPE_MASK;
  if (p->flags & ~allflags) return IREE_UK_B200_INVALID_ARGUMENT;
  const int es = unpack_elem_size(p->flags);
  if (!es) return IREE_UK_B200_INVALID_ARGUMENT;
  if (p->out_size0 < 0 || p->out_size1 < 0 || p->in_size0 < 0 || p->in_size1 < 0 ||
      p->in_size2 < 0 || p->in_size3 < 0 || p->in_stride0 < 0 || p->out_stride0 < 0 ||
      p->out_stride1 < 0)
    return IREE_UK_B200_INVALID_ARGUMENT;
  if (p->in_stride1 != p->in_size2 * p->in_size3) return IREE_UK_B200_INVALID_ARGUMENT;
  int64_t outer0 = p->in_size0, outer1 = p->in_size1;
  int64_t tile0 = p->in_size2, tile1 = p->in_size3;
  if (p->flags & IREE_UK_FLAG_UNPACK_TRANSPOSE_OUTER) { int64_t t = outer0; outer0 = outer1; outer1 = t; }
  if (p->flags & IREE_UK_FLAG_UNPACK_TRANSPOSE_INNER) { int64_t t = tile0; tile0 = tile1; tile1 = t; }
  if (outer0 * tile0 < p->out_size0 || outer1 * tile1 < p->out_size1)
    return IREE_UK_B200_INVALID_ARGUMENT;
  if (!tile_fits_reference_tmpbuf(tile0, tile1, es)) return IREE_UK_B200_INVALID_ARGUMENT;
  return IREE_UK_B200_OK;
}

}  // namespace uk
