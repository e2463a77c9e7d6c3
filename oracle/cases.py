"""Test-case builders for mmt4d / pack / unpack. TEST INFRASTRUCTURE ONLY.

Restates, in numpy, how the reference's own unit tests build their cases, so that the
parity tests here read like them:

* shape lists, tile lists, narrowed M0, with/without ACCUMULATE:
  runtime/src/iree/builtins/ukernel/tools/mmt4d_test.c:459-603
* pack / unpack outer shapes x transposes x padding modes, tile lists:
  tools/pack_test.c:137-241, tools/unpack_test.c:118-216
* randomly non-tight strides and non-zero offsets: mmt4d_test.c:352-402,
  pack_test.c:80-93
* value ranges chosen so float sums are exact (small integers): tools/util.c:105-170
* the deterministic minstd generator seeded with 1: tools/util.h:22-29, util.c:77-103

A case owns host byte buffers; ``params(...)`` binds them (or device copies of them) to a
ctypes params struct. Buffers are allocated as offset + addressed extent, so the whole
allocation — stride gaps and the offset prefix included — can be compared byte for byte,
which is the reference's "no stray writes" check (mmt4d_test.c:430-440).
"""
import ctypes as C

import numpy as np

from iree_b200 import abi


class Minstd:
    """std::minstd_rand, state 1 (tools/util.h:22-29, util.c:77-103)."""

    def __init__(self, state=1):
        self.state = state

    def u32(self):
        self.state = (self.state * 48271) % 2147483647
        return self.state

    def u64(self):
        hi = self.u32()
        return ((hi << 32) + self.u32()) & 0xFFFFFFFFFFFFFFFF

    def r16(self):
        return (self.u32() >> 8) & 0xFFFF

    def bit(self):
        return self.r16() & 1


# ------------------------------------------------------------------------------------
# values
# ------------------------------------------------------------------------------------

def _f32_to_bf16_bits(x):
    """Round-to-nearest-even f32 -> bf16 bit patterns (uint16)."""
    u = np.asarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    rounded = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return rounded.astype(np.uint16)


def bf16_bits_to_f32(b):
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def random_elements(kind, count, rng, mode="exact"):
    """``count`` elements of ``kind`` as raw bytes (uint8 array).

    mode="exact": the reference tests' small-integer ranges (tools/util.c:136-168):
      f32 {-2..1}, f16 {-8..7}, bf16 {-2..1}, s32/s16 [-512,1535], s8 full range,
      4-bit: uniformly random bytes.
    mode="normal": N(0,1) floats / full-range integers, the distributions the headline
      configurations use."""
    if kind in ("u4", "s4"):
        return rng.integers(0, 256, size=(count + 1) // 2, dtype=np.uint8)
    if kind == "s8":
        return rng.integers(-128, 128, size=count, dtype=np.int8).view(np.uint8)
    if kind == "s16":
        if mode == "exact":
            v = rng.integers(-512, 1536, size=count, dtype=np.int16)
        else:
            v = rng.integers(-32768, 32768, size=count, dtype=np.int16)
        return v.view(np.uint8)
    if kind == "s32":
        if mode == "exact":
            v = rng.integers(-512, 1536, size=count, dtype=np.int32)
        else:
            v = rng.integers(-2**31, 2**31, size=count, dtype=np.int64).astype(np.int32)
        return v.view(np.uint8)
    if kind == "f32":
        if mode == "exact":
            v = rng.integers(-2, 2, size=count).astype(np.float32)
        else:
            v = rng.standard_normal(count, dtype=np.float32)
        return v.view(np.uint8)
    if kind == "f16":
        if mode == "exact":
            v = rng.integers(-8, 8, size=count).astype(np.float16)
        else:
            v = rng.standard_normal(count, dtype=np.float32).astype(np.float16)
        return v.view(np.uint8)
    if kind == "bf16":
        if mode == "exact":
            v = rng.integers(-2, 2, size=count).astype(np.float32)
        else:
            v = rng.standard_normal(count, dtype=np.float32)
        return _f32_to_bf16_bits(v).view(np.uint8)
    raise ValueError(kind)


MMT4D_KINDS = {
    abi.MMT4D_F32F32F32: ("f32", "f32", "f32"),
    abi.MMT4D_S8S8S32: ("s8", "s8", "s32"),
    abi.MMT4D_F16F16F32: ("f16", "f16", "f32"),
    abi.MMT4D_BF16BF16F32: ("bf16", "bf16", "f32"),
    abi.MMT4D_F16F16F16: ("f16", "f16", "f16"),
    abi.MMT4D_BF16BF16BF16: ("bf16", "bf16", "bf16"),
    abi.MMT4D_S16S16S32: ("s16", "s16", "s32"),
    abi.MMT4D_S16U4S32: ("s16", "u4", "s32"),
    abi.MMT4D_S16S8S32: ("s16", "s8", "s32"),
    abi.MMT4D_S8S4S32: ("s8", "s4", "s32"),
}
KIND_BITS = {"f32": 32, "s32": 32, "f16": 16, "bf16": 16, "s16": 16, "s8": 8, "u4": 4,
             "s4": 4}

# (M, N, K) outer shapes, tools/mmt4d_test.c:459-479 (max reduction 1000 for 32-bit out).
MMT4D_SHAPES = [(0, 1, 1), (0, 5, 7), (1, 0, 1), (5, 0, 7), (1, 1, 0), (5, 7, 0),
                (1, 1, 1), (1, 1, 2), (1, 1, 10), (1, 1, 1000), (2, 1, 1), (1, 2, 1),
                (2, 2, 2), (5, 7, 13)]

# (type, M0, N0, K0): the odd generic shapes of mmt4d_test.c:545-554 and the x86-64 shapes
# of :578-603, for the type triples this library serves.
MMT4D_TILES = [
    (abi.MMT4D_S8S8S32, 9, 6, 3), (abi.MMT4D_S16U4S32, 5, 3, 2),
    (abi.MMT4D_F16F16F32, 4, 6, 5), (abi.MMT4D_BF16BF16F32, 11, 4, 1),
    (abi.MMT4D_S8S8S32, 8, 8, 2), (abi.MMT4D_F16F16F32, 8, 8, 1),
    (abi.MMT4D_S8S8S32, 16, 16, 2), (abi.MMT4D_F16F16F32, 16, 16, 1),
    (abi.MMT4D_BF16BF16F32, 16, 16, 2), (abi.MMT4D_S16U4S32, 1, 32, 8),
]
# 16-bit-output triples: (type | extra flags, M0, N0, K0), mmt4d_test.c:552-554,583-596; the
# x86 paths exist only with SKIP_INTERMEDIATE_ROUNDINGS.
MMT4D_TILES_16BIT_OUT = [
    (abi.MMT4D_F16F16F16, 3, 5, 8), (abi.MMT4D_BF16BF16BF16, 2, 9, 3),
    (abi.MMT4D_F16F16F16 | abi.MMT4D_SKIP_INTERMEDIATE_ROUNDINGS, 8, 8, 1),
    (abi.MMT4D_F16F16F16 | abi.MMT4D_SKIP_INTERMEDIATE_ROUNDINGS, 16, 16, 1),
    (abi.MMT4D_BF16BF16BF16 | abi.MMT4D_SKIP_INTERMEDIATE_ROUNDINGS, 16, 16, 2),
]
# Further triples the generic kernel serves (mmt4d_test.c:545-551).
MMT4D_TILES_EXTRA = [
    (abi.MMT4D_F32F32F32, 3, 5, 7), (abi.MMT4D_S8S4S32, 9, 12, 2),
    (abi.MMT4D_S16S16S32, 7, 3, 6), (abi.MMT4D_S16S8S32, 7, 5, 6),
    (abi.MMT4D_F32F32F32, 16, 16, 1), (abi.MMT4D_S16S16S32, 16, 16, 2),
]


def narrowed_m0(m0):
    """M0 itself plus every power of two below it (mmt4d_test.c:535-538)."""
    out, n = [], 1
    while n < m0:
        out.append(n)
        n *= 2
    return out + [m0]


def _round_up_whole_bytes(index, bits):
    while (index * bits) & 7:
        index += 1
    return index


def _addr(buf):
    return buf.ctypes.data if isinstance(buf, np.ndarray) else int(buf)


class Mmt4dCase:
    """One mmt4d problem with host inputs and a host initial output."""

    def __init__(self, type_flag, M0, N0, K0, M, N, K, accumulate, seed=0, mode="exact",
                 loose=True, extra_flags=0):
        extra_flags |= type_flag & ~0xFF
        type_flag &= 0xFF
        self.kinds = MMT4D_KINDS[type_flag]
        lb, rb, ob = (KIND_BITS[k] for k in self.kinds)
        self.bits = (lb, rb, ob)
        eng = Minstd(1 + seed)
        rng = np.random.default_rng(1000 + seed)
        rnd = (lambda: eng.bit()) if loose else (lambda: 0)
        self.M, self.N, self.K, self.M0, self.N0, self.K0 = M, N, K, M0, N0, K0
        self.flags = type_flag | (abi.MMT4D_ACCUMULATE if accumulate else 0) | extra_flags
        # strides: tight or tight+1, rounded up to whole bytes (mmt4d_test.c:352-358)
        self.lhs_stride0 = _round_up_whole_bytes(K * M0 * K0 + rnd(), lb)
        self.rhs_stride0 = _round_up_whole_bytes(K * N0 * K0 + rnd(), rb)
        self.out_stride0 = _round_up_whole_bytes(N * M0 * N0 + rnd(), ob)
        self.lhs_offset = _round_up_whole_bytes(rnd(), lb)
        self.rhs_offset = _round_up_whole_bytes(rnd(), rb)
        self.out_offset = _round_up_whole_bytes(rnd(), ob)
        lhs_elems = self.lhs_offset + M * self.lhs_stride0
        rhs_elems = self.rhs_offset + N * self.rhs_stride0
        out_elems = self.out_offset + M * self.out_stride0
        self.lhs = random_elements(self.kinds[0], max(lhs_elems, 1), rng, mode)
        self.rhs = random_elements(self.kinds[1], max(rhs_elems, 1), rng, mode)
        self.out_init = random_elements(self.kinds[2], max(out_elems, 1), rng, mode)

    def params(self, lhs, rhs, out):
        """Bind buffers (numpy arrays or raw addresses) to an ``abi.Mmt4dParams``."""
        p = abi.Mmt4dParams()
        p.lhs_buffer, p.rhs_buffer, p.out_buffer = _addr(lhs), _addr(rhs), _addr(out)
        p.lhs_offset, p.lhs_stride0 = self.lhs_offset, self.lhs_stride0
        p.rhs_offset, p.rhs_stride0 = self.rhs_offset, self.rhs_stride0
        p.out_offset, p.out_stride0 = self.out_offset, self.out_stride0
        p.M, p.N, p.K, p.M0, p.N0, p.K0 = self.M, self.N, self.K, self.M0, self.N0, self.K0
        p.flags = self.flags
        p.cpu_data = None
        return p

    def label(self):
        return "t%x_%dx%dx%d_%dx%dx%d_f%x" % (self.flags & 0xFF, self.M0, self.N0, self.K0,
                                             self.M, self.N, self.K, self.flags)


PACK_KINDS = {abi.PACK_F32F32: 4, abi.PACK_I8I8: 1, abi.PACK_I32I32: 4, abi.PACK_F16F16: 2,
              abi.PACK_BF16BF16: 2}
# tools/pack_test.c:137-145
OUTER_SHAPES = [(0, 1), (1, 0), (1, 1), (3, 2), (9, 33)]
PAD_MODES = ["none", "one_incomplete_tile", "a_lot"]
# tools/pack_test.c:215-241 (generic + x86-64 tile shapes)
PACK_TILES = [(abi.PACK_F32F32, 3, 5), (abi.PACK_I8I8, 4, 2), (abi.PACK_I32I32, 3, 4),
              (abi.PACK_F16F16, 6, 7), (abi.PACK_BF16BF16, 9, 2), (abi.PACK_F32F32, 8, 1),
              (abi.PACK_I8I8, 8, 2), (abi.PACK_F32F32, 8, 8), (abi.PACK_I32I32, 8, 8),
              (abi.PACK_F32F32, 16, 1), (abi.PACK_BF16BF16, 16, 2), (abi.PACK_I8I8, 16, 2),
              (abi.PACK_F32F32, 16, 16), (abi.PACK_I32I32, 16, 16)]
# tools/unpack_test.c:198-216
UNPACK_TILES = [(abi.UNPACK_F32F32, 3, 5), (abi.UNPACK_I32I32, 3, 4),
                (abi.UNPACK_F16F16, 6, 7), (abi.UNPACK_BF16BF16, 9, 2),
                (abi.UNPACK_F32F32, 8, 8), (abi.UNPACK_I32I32, 8, 8),
                (abi.UNPACK_F32F32, 16, 16), (abi.UNPACK_I32I32, 16, 16)]


class PackCase:
    """One pack problem built the way tools/pack_test.c:73-193 builds it."""

    def __init__(self, type_flag, tile0, tile1, outer, transpose_inner, transpose_outer,
                 pad, seed=0, loose=True, max_offset=65535):
        eng = Minstd(1 + seed)
        rng = np.random.default_rng(2000 + seed)
        es = PACK_KINDS[type_flag]
        self.elem_size = es
        o0, o1 = outer
        if pad == "a_lot":
            o0, o1 = o0 + 16, o1 + 16
        self.flags = type_flag
        self.out_size0, self.out_size1 = o0, o1
        self.out_size2, self.out_size3 = tile0, tile1
        if transpose_outer:
            self.flags |= abi.PACK_TRANSPOSE_OUTER
            self.out_size0, self.out_size1 = o1, o0
        t0, t1 = tile0, tile1
        if transpose_inner:
            self.flags |= abi.PACK_TRANSPOSE_INNER
            t0, t1 = tile1, tile0
        self.in_size0, self.in_size1 = o0 * t0, o1 * t1
        if pad == "one_incomplete_tile":
            self.in_size0 = max(0, self.in_size0 - eng.r16() % t0)
            self.in_size1 = max(0, self.in_size1 - eng.r16() % t1)
        if pad == "a_lot":
            # Stricter than pack_test.c:160-175, which enlarges the source as well: here the
            # source keeps the un-enlarged extent, so 16 tiles each way are pure padding.
            self.in_size0, self.in_size1 = outer[0] * t0, outer[1] * t1
        self.padding_value = eng.u64()
        rnd = (lambda: eng.bit()) if loose else (lambda: 0)
        self.in_stride1 = 1 + rnd()
        self.in_stride0 = self.in_size1 * self.in_stride1 + rnd()
        self.out_stride1 = self.out_size2 * self.out_size3
        self.out_stride0 = self.out_size1 * self.out_stride1 + rnd()
        self.in_offset = eng.r16() % (max_offset + 1) if loose else 0
        self.out_offset = eng.r16() % (max_offset + 1) if loose else 0
        in_elems = self.in_offset + self.in_size0 * self.in_stride0 + 1
        out_elems = self.out_offset + self.out_size0 * self.out_stride0 + 1
        self.inp = rng.integers(0, 256, size=in_elems * es, dtype=np.uint8)
        self.out_init = rng.integers(0, 256, size=out_elems * es, dtype=np.uint8)

    def params(self, inp, out):
        p = abi.PackParams()
        p.in_buffer, p.out_buffer = _addr(inp), _addr(out)
        for f in ("in_offset", "in_stride0", "in_stride1", "out_offset", "out_stride0",
                  "out_stride1", "in_size0", "in_size1", "out_size0", "out_size1",
                  "out_size2", "out_size3", "padding_value", "flags"):
            setattr(p, f, getattr(self, f))
        p.cpu_data = None
        return p


class UnpackCase:
    """One unpack problem built the way tools/unpack_test.c:60-182 builds it."""

    def __init__(self, type_flag, tile0, tile1, outer, transpose_inner, transpose_outer,
                 pad, seed=0, loose=True, max_offset=65535):
        eng = Minstd(1 + seed)
        rng = np.random.default_rng(3000 + seed)
        es = abi.UNPACK_ELEM_SIZE[type_flag]
        self.elem_size = es
        s0, s1 = outer
        self.flags = type_flag
        self.in_size0, self.in_size1 = s0, s1
        if pad == "a_lot":
            self.in_size0 += 16
            self.in_size1 += 16
        self.in_size2, self.in_size3 = tile0, tile1
        t0, t1 = tile0, tile1
        if transpose_outer:
            self.flags |= abi.UNPACK_TRANSPOSE_OUTER
            s0, s1 = s1, s0
        if transpose_inner:
            self.flags |= abi.UNPACK_TRANSPOSE_INNER
            t0, t1 = t1, t0
        self.out_size0, self.out_size1 = s0 * t0, s1 * t1
        if pad == "one_incomplete_tile":
            self.out_size0 = max(0, self.out_size0 - eng.r16() % t0)
            self.out_size1 = max(0, self.out_size1 - eng.r16() % t1)
        rnd = (lambda: eng.bit()) if loose else (lambda: 0)
        self.in_stride1 = self.in_size2 * self.in_size3
        self.in_stride0 = self.in_size1 * self.in_stride1 + rnd()
        self.out_stride1 = 1 + rnd()
        self.out_stride0 = self.out_size1 * self.out_stride1 + rnd()
        self.in_offset = eng.r16() % (max_offset + 1) if loose else 0
        self.out_offset = eng.r16() % (max_offset + 1) if loose else 0
        in_elems = self.in_offset + self.in_size0 * self.in_stride0 + 1
        out_elems = self.out_offset + self.out_size0 * self.out_stride0 + 1
        self.inp = rng.integers(0, 256, size=in_elems * es, dtype=np.uint8)
        self.out_init = rng.integers(0, 256, size=out_elems * es, dtype=np.uint8)

    def params(self, inp, out):
        p = abi.UnpackParams()
        p.in_buffer, p.out_buffer = _addr(inp), _addr(out)
        for f in ("in_offset", "in_stride0", "in_stride1", "out_offset", "out_stride0",
                  "out_stride1", "in_size0", "in_size1", "in_size2", "in_size3",
                  "out_size0", "out_size1", "flags"):
            setattr(p, f, getattr(self, f))
        p.cpu_data = None
        return p


def all_pack_cases(tiles=None, max_offset=65535):
    seed = 0
    for type_flag, t0, t1 in (tiles or PACK_TILES):
        for outer in OUTER_SHAPES:
            for ti in (0, 1):
                for to in (0, 1):
                    for pad in PAD_MODES:
                        seed += 1
                        yield PackCase(type_flag, t0, t1, outer, ti, to, pad, seed,
                                       max_offset=max_offset)


def all_unpack_cases(tiles=None, max_offset=65535):
    seed = 0
    for type_flag, t0, t1 in (tiles or UNPACK_TILES):
        for outer in OUTER_SHAPES:
            for ti in (0, 1):
                for to in (0, 1):
                    for pad in PAD_MODES:
                        seed += 1
                        yield UnpackCase(type_flag, t0, t1, outer, ti, to, pad, seed,
                                         max_offset=max_offset)


def all_mmt4d_cases(tiles=None, shapes=None, mode="exact"):
    seed = 0
    for type_flag, M0, N0, K0 in (tiles or MMT4D_TILES):
        for m0 in narrowed_m0(M0):
            for (M, N, K) in (shapes or MMT4D_SHAPES):
                if (type_flag & 0xFF) == abi.MMT4D_BF16BF16BF16 and K == 1000:
                    K = 100  # max_reduction_size for bf16 outputs, mmt4d_test.c:453-454
                for acc in (0, 1):
                    seed += 1
                    yield Mmt4dCase(type_flag, m0, N0, K0, M, N, K, acc, seed, mode)


def rel_frobenius(a, b):
    """||a - b||_F / ||b||_F in float64 (0 when both are empty or b is all zero and a==b)."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    den = np.linalg.norm(b)
    num = np.linalg.norm(a - b)
    return 0.0 if num == 0.0 else num / max(den, 1e-300)
