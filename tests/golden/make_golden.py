"""Generates the golden vectors in this directory from the reference ukernels themselves.

Run where a reference checkout is available (it is compiled in place by
``make -C oracle ref``):   python tests/golden/make_golden.py

For a selection of the reference tests' cases (tools/mmt4d_test.c, pack_test.c,
unpack_test.c shape lists) it stores the case parameters, the input bytes, the initial
output bytes and the output bytes the compiled reference produced, one ``.npz`` per
operation. Inputs are stored, not regenerated, so the fixtures do not depend on a random
generator's stream. The integer / pack / unpack outputs are exact by definition; the float
cases use small-integer values (tools/util.c:136-168) and are exact as well.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import oracle  # noqa: E402
from iree_b200 import abi  # noqa: E402
from oracle import cases  # noqa: E402

MMT4D_FIELDS = ["lhs_offset", "lhs_stride0", "rhs_offset", "rhs_stride0", "out_offset",
                "out_stride0", "M", "N", "K", "M0", "N0", "K0", "flags"]
PACK_FIELDS = ["in_offset", "in_stride0", "in_stride1", "out_offset", "out_stride0",
               "out_stride1", "in_size0", "in_size1", "out_size0", "out_size1", "out_size2",
               "out_size3", "padding_value", "flags"]
UNPACK_FIELDS = ["in_offset", "in_stride0", "in_stride1", "out_offset", "out_stride0",
                 "out_stride1", "in_size0", "in_size1", "in_size2", "in_size3", "out_size0",
                 "out_size1", "flags"]


def main():
    oracle.build()
    assert oracle.ref_available(), "reference checkout not found; cannot generate goldens"
    store = {}
    n = 0
    shapes = [(1, 1, 0), (5, 7, 0), (1, 1, 1), (1, 1, 10), (2, 2, 2), (5, 7, 13)]
    for c in cases.all_mmt4d_cases(cases.MMT4D_TILES, shapes):
        if c.M0 not in (1, 4, 5, 9, 11, 16) or c.lhs.size + c.rhs.size + 2 * c.out_init.size > 12000:
            continue
        out = c.out_init.copy()
        oracle.mmt4d(c.params(c.lhs, c.rhs, out), "ref")
        k = "m%03d_" % n
        store[k + "fields"] = np.array([getattr(c, f) for f in MMT4D_FIELDS], dtype=np.int64)
        store[k + "lhs"], store[k + "rhs"] = c.lhs, c.rhs
        store[k + "init"], store[k + "out"] = c.out_init, out
        n += 1
    np.savez_compressed(os.path.join(HERE, "mmt4d_golden.npz"), count=n, **store)
    print("mmt4d cases:", n)

    store, n = {}, 0
    tiles = [(abi.PACK_F32F32, 3, 5), (abi.PACK_I8I8, 4, 2), (abi.PACK_BF16BF16, 16, 2),
             (abi.PACK_F32F32, 16, 1), (abi.PACK_I32I32, 16, 16)]
    for c in cases.all_pack_cases(tiles, max_offset=15):
        if c.inp.size + 2 * c.out_init.size > 9000 or c.out_size0 * c.out_size1 == 0:
            continue
        out = c.out_init.copy()
        oracle.pack(c.params(c.inp, out), "ref")
        k = "p%03d_" % n
        store[k + "fields"] = np.array([getattr(c, f) for f in PACK_FIELDS], dtype=np.uint64)
        store[k + "in"], store[k + "init"], store[k + "out"] = c.inp, c.out_init, out
        n += 1
    np.savez_compressed(os.path.join(HERE, "pack_golden.npz"), count=n, **store)
    print("pack cases:", n)

    store, n = {}, 0
    tiles = [(abi.UNPACK_F32F32, 3, 5), (abi.UNPACK_BF16BF16, 9, 2), (abi.UNPACK_I32I32, 16, 16)]
    for c in cases.all_unpack_cases(tiles, max_offset=15):
        if c.inp.size + 2 * c.out_init.size > 9000 or c.out_size0 * c.out_size1 == 0:
            continue
        out = c.out_init.copy()
        oracle.unpack(c.params(c.inp, out), "ref")
        k = "u%03d_" % n
        store[k + "fields"] = np.array([getattr(c, f) for f in UNPACK_FIELDS], dtype=np.int64)
        store[k + "in"], store[k + "init"], store[k + "out"] = c.inp, c.out_init, out
        n += 1
    np.savez_compressed(os.path.join(HERE, "unpack_golden.npz"), count=n, **store)
    print("unpack cases:", n)


if __name__ == "__main__":
    main()
