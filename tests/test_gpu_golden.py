"""The committed golden vectors (tests/golden/*.npz: inputs and the outputs that the compiled
reference ukernels produced for them) run on the GPU through the C ABI. Every case is compared
over its whole output allocation, stride gaps and offset prefix included, which is the
reference's own "no stray writes" check (tools/mmt4d_test.c:430-440). All cases are exact:
integers, opaque pack / unpack bytes, and floats on the reference tests' small-integer values."""
import numpy as np
import pytest
import torch

from iree_b200 import ukernel as uk

import golden_util
import gpu_util as G

pytestmark = pytest.mark.gpu


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("with_workspace", [True, False], ids=["workspace", "no_workspace"])
def test_mmt4d_golden_vectors(with_workspace):
    gs = golden_util.load("mmt4d")
    assert len(gs) > 100
    for g in gs:
        lhs, rhs, out = _dev(g.bufs["lhs"]), _dev(g.bufs["rhs"]), _dev(g.bufs["init"])
        p = g.params(lhs.data_ptr(), rhs.data_ptr(), out.data_ptr())
        ws = None
        if with_workspace:
            n = uk.mmt4d_workspace_size(p)
            ws = torch.empty(n, dtype=torch.uint8, device="cuda") if n else None
        uk.mmt4d(p, workspace=ws)
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy(), g.bufs["out"]), g.values
    G.check_device_status()


def test_pack_golden_vectors():
    gs = golden_util.load("pack")
    assert len(gs) > 50
    for g in gs:
        inp, out = _dev(g.bufs["in"]), _dev(g.bufs["init"])
        uk.pack(g.params(inp.data_ptr(), out.data_ptr()))
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy(), g.bufs["out"]), g.values
    G.check_device_status()


def test_unpack_golden_vectors():
    gs = golden_util.load("unpack")
    assert len(gs) > 20
    for g in gs:
        inp, out = _dev(g.bufs["in"]), _dev(g.bufs["init"])
        uk.unpack(g.params(inp.data_ptr(), out.data_ptr()))
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy(), g.bufs["out"]), g.values
    G.check_device_status()
