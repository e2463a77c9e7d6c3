"""The IREE executable plugin (plugin/iree_uk_b200_plugin.c -> libiree_uk_b200_plugin.so): the
test plays the runtime's loader - query, load with parameters, resolve the ukernel imports, call
them the way compiled code does (int fn(void* params_ptr, void* context, void* reserved) with the
packed operands of the ukernel op), unload - following the reference's own sample
(samples/custom_dispatch/cpu/plugin/system_plugin.c:62-97, :147-209)."""
import ctypes as C

import numpy as np
import pytest

from iree_b200 import abi

import plugin_util as P

pytestmark = pytest.mark.skipif(not P.available(), reason="plugin not built (needs an IREE checkout)")


def test_query_reports_version_name_and_sanitizer():
    ld = P.Loader()
    assert ld.load_status == P.STATUS_OK
    h = ld.plugin.contents.header.contents
    assert h.version == P.VERSION_0_1
    assert h.name == b"iree_uk_b200" and b"B200" in h.description
    assert h.features == 0          # not standalone: it calls into the CUDA runtime
    assert h.sanitizer == 0         # built without a sanitizer
    assert all(x == 0 for x in h.reserved)
    assert not ld.query(0)          # a runtime that supports no version this plugin offers
    ld.unload()


def test_resolve_required_optional_and_preset_symbols():
    ld = P.Loader()
    st, bits, fns, ctxs = ld.resolve(["iree_uk_mmt4d", "iree_uk_pack", "iree_uk_unpack"])
    assert st == P.STATUS_OK and bits == 0
    assert all(fns) and all(c == ld.self_ptr.value for c in ctxs)
    assert len(set(fns)) == 3
    # a missing optional import is not an error, only a resolution bit
    st, bits, fns, _ = ld.resolve(["?iree_uk_mmt4d", "?no_such_import"])
    assert st == P.STATUS_OK and bits == P.RESOLUTION_MISSING_OPTIONAL
    assert fns[0] and not fns[1]
    # a missing required import: NOT_FOUND, and what could be resolved still is
    st, bits, fns, _ = ld.resolve(["iree_uk_pack", "no_such_import"])
    assert st == P.STATUS_NOT_FOUND and fns[0] and not fns[1]
    # entries another provider already resolved are left alone
    st, _, fns, _ = ld.resolve(["iree_uk_unpack"], preset=[0x1234])
    assert st == P.STATUS_OK and fns[0] == 0x1234
    ld.unload()


def test_load_parameters_are_parsed_and_bad_ones_rejected():
    ld = P.Loader([("stream", "0x0"), ("workspace", "0"), ("workspace_bytes", "0"),
                   ("some_other_plugins_key", "whatever")])
    assert ld.load_status == P.STATUS_OK
    ld.unload()
    bad = P.Loader([("workspace_bytes", "12 MiB")])
    assert (bad.load_status & 0x1F) == P.STATUS_INVALID_ARGUMENT
    assert not bad.live  # the state allocated before the bad parameter was freed again


def test_import_thunks_report_library_status_without_a_gpu():
    """Rejected parameters never reach a launch, so this runs anywhere: the thunk returns
    non-zero and the library's status is kept for the runtime to ask."""
    ld = P.Loader()
    _, _, fns, ctxs = ld.resolve(["iree_uk_mmt4d"])
    p = abi.Mmt4dParams()
    p.M, p.N, p.K, p.M0, p.N0, p.K0, p.flags = 1, 1, 1, 16, 16, 2, 0x0B  # type id out of range
    rc = P.IMPORT_FN(fns[0])(C.addressof(p), ctxs[0], None)
    assert rc == abi.INVALID_ARGUMENT
    assert ld.last_status() == abi.INVALID_ARGUMENT and ld.last_status() == 0
    ld.unload()


@pytest.mark.gpu
@pytest.mark.parametrize("with_workspace", [False, True], ids=["static_scratch", "workspace"])
def test_imports_compute_what_the_reference_ukernels_compute(with_workspace):
    import torch
    from oracle import cases
    from iree_b200 import ukernel as uk
    import gpu_util as G
    ld = P.Loader()
    st, _, fns, ctxs = ld.resolve(["iree_uk_mmt4d", "iree_uk_pack", "iree_uk_unpack"])
    assert st == P.STATUS_OK
    mmt4d, pack, unpack = (P.IMPORT_FN(f) for f in fns)
    stream = torch.cuda.current_stream().cuda_stream
    ws = torch.empty(64 << 20, dtype=torch.uint8, device="cuda") if with_workspace else None
    assert ld.configure(stream, ws.data_ptr() if ws is not None else None,
                        ws.numel() if ws is not None else 0) == 0

    # mmt4d: a tensor-core problem, a generic one, the s16u4 GEMV
    for spec in [(abi.MMT4D_S8S8S32, 16, 16, 2, 24, 40, 64, 1, "exact"),
                 (abi.MMT4D_BF16BF16F32, 16, 16, 2, 9, 17, 33, 0, "exact"),
                 (abi.MMT4D_S8S8S32, 9, 6, 3, 5, 7, 13, 1, "exact"),
                 (abi.MMT4D_S16U4S32, 1, 32, 8, 1, 12, 40, 0, "normal")]:
        t, M0, N0, K0, M, N, K, acc, mode = spec
        case = cases.Mmt4dCase(t, M0, N0, K0, M, N, K, acc, seed=51, mode=mode, loose=False)
        lhs, rhs, out = G.to_device(case.lhs), G.to_device(case.rhs), G.to_device(case.out_init)
        p = case.params(lhs.data_ptr(), rhs.data_ptr(), out.data_ptr())
        # compiled code always sets the fallback flag (CPULowerToUKernels.cpp:235)
        p.flags |= abi.MMT4D_ALLOW_GENERIC_FALLBACK
        assert mmt4d(C.addressof(p), ctxs[0], None) == 0
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy(), G.oracle_mmt4d(case)), case.label()

    pc = cases.PackCase(abi.PACK_F32F32, 16, 1, (9, 33), 0, 0, "one_incomplete_tile", seed=3)
    inp, out = G.to_device(pc.inp), G.to_device(pc.out_init)
    pp = pc.params(inp.data_ptr(), out.data_ptr())
    assert pack(C.addressof(pp), ctxs[1], None) == 0
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), G.oracle_pack(pc))

    uc = cases.UnpackCase(abi.UNPACK_I32I32, 16, 16, (9, 33), 1, 1, "one_incomplete_tile", seed=4)
    inp, out = G.to_device(uc.inp), G.to_device(uc.out_init)
    up = uc.params(inp.data_ptr(), out.data_ptr())
    assert unpack(C.addressof(up), ctxs[2], None) == 0
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), G.oracle_unpack(uc))
    assert ld.last_status() == 0
    assert uk.device_status() == (0, 0)
    ld.unload()


@pytest.mark.gpu
def test_mmt4d_beyond_the_static_scratch_uses_the_pool_when_allowed():
    """A problem whose scratch need exceeds the 32 MiB array: with "scratch_pool" = 1 the import
    runs the pre-pass kernels on memory of the library's stream-ordered pool; without it the
    scratch-free kernel. Both give the reference's result."""
    import torch
    from oracle import cases
    from iree_b200 import ukernel as uk
    import gpu_util as G
    case = cases.Mmt4dCase(abi.MMT4D_S8S8S32, 16, 16, 2, 40, 72, 10000, 1, seed=5, mode="exact",
                           loose=False)
    want = G.oracle_mmt4d(case)
    for allow in ("0", "1"):
        ld = P.Loader(params=[("scratch_pool", allow)])
        _, _, fns, ctxs = ld.resolve(["iree_uk_mmt4d"])
        assert ld.configure(torch.cuda.current_stream().cuda_stream, None, 0) == 0
        lhs, rhs, out = G.to_device(case.lhs), G.to_device(case.rhs), G.to_device(case.out_init)
        p = case.params(lhs.data_ptr(), rhs.data_ptr(), out.data_ptr())
        assert uk.mmt4d_workspace_size(p) > uk.STATIC_SCRATCH_BYTES
        assert P.IMPORT_FN(fns[0])(C.addressof(p), ctxs[0], None) == 0
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy(), want)
        assert ld.last_status() == 0
        ld.unload()
    assert uk.device_status() == (0, 0)
