"""Loads the committed golden vectors (tests/golden/*.npz, written by make_golden.py from the
compiled reference ukernels) as lightweight case objects with a ``params`` binder."""
import os

import numpy as np

from iree_b200 import abi

HERE = os.path.dirname(os.path.abspath(__file__))
MMT4D_FIELDS = ["lhs_offset", "lhs_stride0", "rhs_offset", "rhs_stride0", "out_offset",
                "out_stride0", "M", "N", "K", "M0", "N0", "K0", "flags"]
PACK_FIELDS = ["in_offset", "in_stride0", "in_stride1", "out_offset", "out_stride0",
               "out_stride1", "in_size0", "in_size1", "out_size0", "out_size1", "out_size2",
               "out_size3", "padding_value", "flags"]
UNPACK_FIELDS = ["in_offset", "in_stride0", "in_stride1", "out_offset", "out_stride0",
                 "out_stride1", "in_size0", "in_size1", "in_size2", "in_size3", "out_size0",
                 "out_size1", "flags"]


def _addr(b):
    return b.ctypes.data if isinstance(b, np.ndarray) else int(b)


class Golden:
    def __init__(self, kind, fields, values, bufs):
        self.kind, self.bufs = kind, bufs
        self.values = dict(zip(fields, (int(v) for v in values)))

    def params(self, *ptrs):
        if self.kind == "mmt4d":
            p = abi.Mmt4dParams()
            p.lhs_buffer, p.rhs_buffer, p.out_buffer = (_addr(x) for x in ptrs)
        elif self.kind == "pack":
            p = abi.PackParams()
            p.in_buffer, p.out_buffer = (_addr(x) for x in ptrs)
        else:
            p = abi.UnpackParams()
            p.in_buffer, p.out_buffer = (_addr(x) for x in ptrs)
        for k, v in self.values.items():
            setattr(p, k, v)
        p.cpu_data = None
        return p


def load(kind):
    z = np.load(os.path.join(HERE, "golden", "%s_golden.npz" % kind))
    n = int(z["count"])
    prefix = {"mmt4d": "m", "pack": "p", "unpack": "u"}[kind]
    fields = {"mmt4d": MMT4D_FIELDS, "pack": PACK_FIELDS, "unpack": UNPACK_FIELDS}[kind]
    out = []
    for i in range(n):
        k = "%s%03d_" % (prefix, i)
        if kind == "mmt4d":
            bufs = {"lhs": z[k + "lhs"], "rhs": z[k + "rhs"], "init": z[k + "init"],
                    "out": z[k + "out"]}
        else:
            bufs = {"in": z[k + "in"], "init": z[k + "init"], "out": z[k + "out"]}
        out.append(Golden(kind, fields, z[k + "fields"], bufs))
    return out
