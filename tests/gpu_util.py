"""Helpers for the GPU parity tests: run a case through the C ABI on device copies of its
host buffers and hand back the whole output allocation as bytes. The expected bytes come from
the reference ukernels themselves (the library compiled in place under oracle/_ref) wherever
that library is present, and from the C restatement otherwise."""
import numpy as np
import torch

import oracle
from iree_b200 import ukernel as uk


def to_device(arr):
    return torch.from_numpy(np.ascontiguousarray(arr)).cuda()


def run_mmt4d_case(case, use_workspace=True):
    """Returns (gpu_out_bytes, path)."""
    lhs, rhs, out = to_device(case.lhs), to_device(case.rhs), to_device(case.out_init)
    p = case.params(lhs.data_ptr(), rhs.data_ptr(), out.data_ptr())
    ws = None
    if use_workspace:
        n = uk.mmt4d_workspace_size(p)
        if n:
            ws = torch.empty(n, dtype=torch.uint8, device="cuda")
    path = uk.mmt4d_path(p, ws is not None)
    uk.mmt4d(p, workspace=ws)
    torch.cuda.synchronize()
    return out.cpu().numpy(), path


def checker():
    """"ref" (the compiled reference ukernels) when present, else "oracle" (the restatement)."""
    return "ref" if oracle.ref_available() else "oracle"


def oracle_mmt4d(case, impl=None):
    out = case.out_init.copy()
    oracle.mmt4d(case.params(case.lhs, case.rhs, out), impl or checker())
    return out


def run_pack_case(case):
    inp, out = to_device(case.inp), to_device(case.out_init)
    p = case.params(inp.data_ptr(), out.data_ptr())
    path = uk.pack_path(p)
    uk.pack(p)
    torch.cuda.synchronize()
    return out.cpu().numpy(), path


def oracle_pack(case, impl=None):
    out = case.out_init.copy()
    oracle.pack(case.params(case.inp, out), impl or checker())
    return out


def run_unpack_case(case):
    inp, out = to_device(case.inp), to_device(case.out_init)
    p = case.params(inp.data_ptr(), out.data_ptr())
    path = uk.unpack_path(p)
    uk.unpack(p)
    torch.cuda.synchronize()
    return out.cpu().numpy(), path


def oracle_unpack(case, impl=None):
    out = case.out_init.copy()
    oracle.unpack(case.params(case.inp, out), impl or checker())
    return out


def check_device_status():
    st, detail = uk.device_status()
    assert st == 0, "device-side bounded wait ran out: status %d detail 0x%x" % (st, detail)


import contextlib


@contextlib.contextmanager
def f32_tensor_cores(type_flag):
    """Switches f32f32f32 to the tensor-core (three tf32 products) mode for the duration, when
    ``type_flag`` is that triple; other triples are unaffected."""
    from iree_b200 import abi
    if (type_flag & 0xFF) != abi.MMT4D_F32F32F32:
        yield
        return
    prev = uk.set_f32_mode(uk.F32_MODE_TF32X3)
    try:
        yield
    finally:
        uk.set_f32_mode(prev)
