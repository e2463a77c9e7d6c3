"""Benchmark harness, not part of the library: device-timed figures for the other
configurations of the path (single GPU): the small
s8s8s32 GEMM, an s8s8s32 GEMM at the prefill dimensions, the f16 GEMM with ACCUMULATE, the
s16u4s32 decode GEMV, and the pack / unpack relayouts. Used by ``bench.py`` to report them
beside the headline line; every figure is CUDA-event time per call. Configurations whose
working set would fit in L2 are timed as a sweep over several independent buffer sets whose
total footprint exceeds L2.

Bytes for pack / unpack count what is read plus what is written.
"""
import os
import sys

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from iree_b200 import abi  # noqa: E402
from iree_b200 import ukernel as uk  # noqa: E402


ITERS, WARMUP = 10, 3


def _time(fn, iters=None, warmup=None, flush=None):
    iters = ITERS if iters is None else iters
    warmup = WARMUP if warmup is None else warmup
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush is not None:
            flush.sum()  # read-only sweep: evicts L2 without leaving dirty lines to write back
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    return times[len(times) // 2], times[0]


def _time_rotating(fns, iters=None, warmup=None):
    """Per-call time of a small operation: one event pair around a sweep over ``fns`` —
    the same call on different buffer sets whose total footprint exceeds L2 — so that launch
    latency overlaps as it does in a real stream of calls and no call finds its operands in
    L2."""
    iters = ITERS if iters is None else iters
    warmup = WARMUP if warmup is None else warmup
    for _ in range(max(1, warmup)):
        for fn in fns:
            fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for fn in fns:
            fn()
        e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1) / len(fns))
    times.sort()
    return times[len(times) // 2], times[0]


SETTLE_SECONDS = 0.0  # set by run() when the whole list is measured


def _settle():
    """Every case of the whole list starts from an idle GPU: seconds of tensor-core work just
    before leave the part power-capped and its memory system slower for a second or two (a
    same-size device copy then measures 5.4 instead of 5.9 TB/s, a 7 us GEMV 9.7 us), and these
    figures are about the kernels, not about what ran before them."""
    if SETTLE_SECONDS > 0:
        import time
        torch.cuda.synchronize()
        time.sleep(SETTLE_SECONDS)


def _mmt4d_params(flags, M, N, K, M0, N0, K0, lhs, rhs, out):
    p = abi.Mmt4dParams()
    p.lhs_buffer, p.rhs_buffer, p.out_buffer = lhs.data_ptr(), rhs.data_ptr(), out.data_ptr()
    p.M, p.N, p.K, p.M0, p.N0, p.K0, p.flags = M, N, K, M0, N0, K0, flags
    p.lhs_stride0, p.rhs_stride0, p.out_stride0 = K * M0 * K0, K * N0 * K0, N * M0 * N0
    return p


def _rand_bytes(n):
    return torch.randint(0, 256, (n,), dtype=torch.uint8, device="cuda")


def _mmt4d_case(name, flags, M, N, K, M0, N0, K0, peaks, flush, float_dtype=None, copies=1,
                graph_calls=0, use_ws=True, pooled=False):
    """``copies`` > 1: the call is timed as a sweep over that many independent buffer sets
    (see _time_rotating); otherwise one call per event pair, with ``flush`` read in between."""
    lb, rb, _ = abi.MMT4D_BITS[flags & 0xFF]
    nl, nr = M * K * M0 * K0, N * K * N0 * K0
    keep, fns, path = [], [], None
    for _ in range(copies):
        if float_dtype is not None:
            lhs = torch.randn(nl, device="cuda").to(float_dtype)
            rhs = torch.randn(nr, device="cuda").to(float_dtype)
        else:
            lhs, rhs = _rand_bytes(nl * lb // 8), _rand_bytes(nr * rb // 8)
        out = torch.randn(M * N * M0 * N0, device="cuda") if float_dtype is not None else \
            torch.zeros(M * N * M0 * N0, dtype=torch.int32, device="cuda")
        p = _mmt4d_params(flags, M, N, K, M0, N0, K0, lhs, rhs, out)
        nws = uk.mmt4d_workspace_size(p) if use_ws else 0
        ws = torch.empty(nws, dtype=torch.uint8, device="cuda") if nws else None
        path = uk.mmt4d_path(p, ws is not None)
        keep.append((lhs, rhs, out, ws, p))
        if pooled:  # the plain signature, scratch from the library's stream-ordered pool
            fns.append(lambda p=p: uk.mmt4d_pooled(p))
        else:
            fns.append(lambda p=p, ws=ws: uk.mmt4d(p, workspace=ws))
    _settle()
    if copies > 1:
        med, best = _time_rotating(fns)
    else:
        med, best = _time(fns[0], flush=flush)
    ops = 2.0 * M * M0 * N * N0 * K * K0
    res = {"ms": med, "ms_best": best, "path": path, "tops": ops / med / 1e9}
    if copies > 1:
        res["timing"] = "sweep over %d buffer sets (footprint > L2), one event pair" % copies
    if graph_calls:
        _settle()
        res["graph_replay"] = _graph_replay(fns, graph_calls, ops)
    return name, res


def _graph_replay(fns, calls, ops_per_call):
    """``calls`` launches (cycling over the buffer sets) captured once in a CUDA graph and
    replayed: per-call time without the host's launch path."""
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fns[0]()  # anything lazily created on first use happens outside the capture
        torch.cuda.synchronize()
        with torch.cuda.graph(g, stream=side):
            for i in range(calls):
                fns[i % len(fns)]()
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(2):
        g.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(5):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1) / calls)
    times.sort()
    med = times[len(times) // 2]
    return {"calls_per_graph": calls, "ms_per_call": med, "tops": ops_per_call / med / 1e9}


def _matmul_rowmajor_case(M, N, K, bf16_peak):
    """bf16 x bf16 -> f32, lhs [M][K], rhs [K][N], out [M][N], all row-major."""
    lhs = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    rhs = torch.randn(K, N, device="cuda").to(torch.bfloat16)
    out = torch.empty(M, N, device="cuda")
    ops = 2.0 * M * N * K
    # fused
    mp = abi.MatmulParams()
    mp.lhs_buffer, mp.rhs_buffer, mp.out_buffer = lhs.data_ptr(), rhs.data_ptr(), out.data_ptr()
    mp.lhs_stride0, mp.rhs_stride0, mp.out_stride0 = K, N, N
    mp.M, mp.N, mp.K, mp.flags = M, N, K, abi.MMT4D_BF16BF16F32
    ws = torch.empty(uk.matmul_workspace_size(mp), dtype=torch.uint8, device="cuda")
    fused, fused_best = _time(lambda: uk.matmul(mp, ws))
    del ws
    # chain, tiles 16x16x2
    M1, N1, K1 = M // 16, N // 16, K // 2
    plhs = torch.empty(M * K, dtype=torch.bfloat16, device="cuda")
    prhs = torch.empty(N * K, dtype=torch.bfloat16, device="cuda")
    pout = torch.empty(M * N, device="cuda")

    def pack_params(src, dst, flags, s0, s1, o0, o1, t0, t1):
        p = abi.PackParams()
        p.in_buffer, p.out_buffer = src.data_ptr(), dst.data_ptr()
        p.in_size0, p.in_size1, p.in_stride0, p.in_stride1 = s0, s1, s1, 1
        p.out_size0, p.out_size1, p.out_size2, p.out_size3 = o0, o1, t0, t1
        p.out_stride1, p.out_stride0, p.flags = t0 * t1, o1 * t0 * t1, flags
        return p

    pl = pack_params(lhs, plhs, abi.PACK_BF16BF16, M, K, M1, K1, 16, 2)
    pr = pack_params(rhs, prhs, abi.PACK_BF16BF16 | abi.PACK_TRANSPOSE_INNER |
                     abi.PACK_TRANSPOSE_OUTER, K, N, N1, K1, 16, 2)
    q = _mmt4d_params(abi.MMT4D_BF16BF16F32, M1, N1, K1, 16, 16, 2, plhs, prhs, pout)
    ws = torch.empty(uk.mmt4d_workspace_size(q), dtype=torch.uint8, device="cuda")
    u = abi.UnpackParams()
    u.in_buffer, u.out_buffer = pout.data_ptr(), out.data_ptr()
    u.in_size0, u.in_size1, u.in_size2, u.in_size3 = M1, N1, 16, 16
    u.in_stride1, u.in_stride0 = 256, N1 * 256
    u.out_size0, u.out_size1, u.out_stride0, u.out_stride1 = M, N, N, 1
    u.flags = abi.UNPACK_F32F32

    def chain():
        uk.pack(pl)
        uk.pack(pr)
        uk.mmt4d(q, workspace=ws)
        uk.unpack(u)

    chain_ms, chain_best = _time(chain)
    # the halfway form: packed operands in, row-major result out (unpack folded into the epilogue)
    qu = _mmt4d_params(abi.MMT4D_BF16BF16F32, M1, N1, K1, 16, 16, 2, plhs, prhs, out)
    qu.out_stride0 = N
    unpacked_ms, _ = _time(lambda: uk.mmt4d_unpacked(qu, M, N, ws))
    parts = {}
    for name, fn in [("pack_lhs", lambda: uk.pack(pl)), ("pack_rhs", lambda: uk.pack(pr)),
                     ("mmt4d", lambda: uk.mmt4d(q, workspace=ws)), ("unpack", lambda: uk.unpack(u))]:
        parts[name] = _time(fn)[0]
    return {"fused_ms": fused, "fused_ms_best": fused_best, "fused_tflops": ops / fused / 1e9,
            "fused_frac_of_bf16_burst": ops / fused / 1e9 / bf16_peak,
            "chain_ms": chain_ms, "chain_ms_best": chain_best, "chain_tflops": ops / chain_ms / 1e9,
            "chain_parts_ms": parts, "chain_tiles": "16x16x2",
            "mmt4d_with_unpack_folded_ms": unpacked_ms}


def run(peaks, only=None, custom=None, custom_ws=True, custom_matmul=None):
    """All supplementary configurations, or those whose name contains ``only``. ``custom`` =
    (type name, M1, N1, K1) adds one tensor-core mmt4d of that size (used for profiling)."""
    res = {}
    global SETTLE_SECONDS
    SETTLE_SECONDS = 1.0 if only is None else 0.0

    def want(name):
        return only is None or only in name

    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    hbm = float(peaks.get("hbm_gbs", 6650.0))
    bf16_peak = float(peaks.get("bf16_tflops", 1590.0))

    # mmt4d s8s8s32 1024^3 (latency-bound by size) and at the prefill dimensions
    for name, args in [
        ("mmt4d_s8s8s32_1024x1024x1024", (abi.MMT4D_S8S8S32, 64, 64, 512, 16, 16, 2)),
        ("mmt4d_s8s8s32_8192x28672x8192", (abi.MMT4D_S8S8S32, 512, 1792, 4096, 16, 16, 2)),
    ]:
        if not want(name):
            continue
        small = args[1] < 512
        k, r = _mmt4d_case(name, *args, peaks, None, copies=24 if small else 1,
                           graph_calls=100 if small else 0)
        r["frac_of_2x_bf16_burst"] = r["tops"] / (2 * bf16_peak)
        r["frac_of_spec_4500"] = r["tops"] / 4500.0
        res[k] = r
    if custom is not None:
        tname, cm, cn, ck = custom
        flags, k0, dt = {"bf16": (abi.MMT4D_BF16BF16F32, 2, torch.bfloat16),
                         "f16": (abi.MMT4D_F16F16F32, 1, torch.float16),
                         "f32": (abi.MMT4D_F32F32F32, 1, torch.float32),
                         "s8": (abi.MMT4D_S8S8S32, 2, None)}[tname]
        prev = uk.set_f32_mode(uk.F32_MODE_TF32X3) if tname == "f32" else None
        small = cm * cn * ck < (1 << 24)
        k, r = _mmt4d_case("mmt4d_%s_custom_%dx%dx%d%s" % (tname, cm, cn, ck, "" if custom_ws else "_no_ws"),
                           flags, cm, cn, ck, 16, 16, k0, peaks, None, dt, use_ws=custom_ws,
                           copies=24 if small else 1, graph_calls=100 if small else 0)
        if prev is not None:
            uk.set_f32_mode(prev)
        res[k] = r
    if want("mmt4d_f16f16f32_acc_4096x4096x4096"):
        k, r = _mmt4d_case("mmt4d_f16f16f32_acc_4096x4096x4096",
                           abi.MMT4D_F16F16F32 | abi.MMT4D_ACCUMULATE, 256, 256, 4096, 16, 16, 1,
                           peaks, None, torch.float16)
        r["frac_of_bf16_burst"] = r["tops"] / bf16_peak
        r["frac_of_spec_2250"] = r["tops"] / 2250.0
        res[k] = r
    # s16u4s32 with many rows (prefill-shaped): two 8-bit tensor-core products per s16 x u4
    if want("mmt4d_s16u4s32_prefill_8192x14336x4096"):
        k, r = _mmt4d_case("mmt4d_s16u4s32_prefill_8192x14336x4096", abi.MMT4D_S16U4S32, 8192,
                           448, 512, 1, 32, 8, peaks, None)
        r["frac_of_2x_bf16_burst_counting_both_byte_products"] = 2 * r["tops"] / (2 * bf16_peak)
        res[k] = r
    # the headline problem through the plain three-pointer signature: scratch-free kernel, and
    # the pre-pass kernels on scratch from the library's memory pool
    for name, kw in [("mmt4d_bf16_headline_plain_call_scratch_free", {"use_ws": False}),
                     ("mmt4d_bf16_headline_plain_call_pooled_scratch", {"use_ws": False, "pooled": True})]:
        if want(name):
            k, r = _mmt4d_case(name, abi.MMT4D_BF16BF16F32, 512, 1792, 4096, 16, 16, 2, peaks,
                               None, torch.bfloat16, **kw)
            r["frac_of_bf16_burst"] = r["tops"] / bf16_peak
            res[k] = r
    # s16s16s32 16x16x2: four 8-bit tensor-core products per s16 x s16 term
    if want("mmt4d_s16s16s32_8192x14336x4096"):
        k, r = _mmt4d_case("mmt4d_s16s16s32_8192x14336x4096", abi.MMT4D_S16S16S32, 512, 896, 2048,
                           16, 16, 2, peaks, None)
        r["frac_of_2x_bf16_burst_counting_all_four_byte_products"] = 4 * r["tops"] / (2 * bf16_peak)
        res[k] = r
    # s16s8s32 16x16x2 (two products per term) and s8s4s32 16x16x2 (nibbles widened by the pre-pass)
    for name, flags, products in [("mmt4d_s16s8s32_8192x14336x4096", abi.MMT4D_S16S8S32, 2),
                                  ("mmt4d_s8s4s32_8192x14336x4096", abi.MMT4D_S8S4S32, 1)]:
        if want(name):
            k, r = _mmt4d_case(name, flags, 512, 896, 2048, 16, 16, 2, peaks, None)
            r["frac_of_2x_bf16_burst_counting_every_byte_product"] = products * r["tops"] / (2 * bf16_peak)
            res[k] = r
    # decode GEMV s16u4s32: bytes are the algorithmic figure (weights + vector + output)
    if want("mmt4d_s16u4s32_gemv_1x14336x4096"):
        k, r = _mmt4d_case("mmt4d_s16u4s32_gemv_1x14336x4096", abi.MMT4D_S16U4S32, 1, 448, 512,
                           1, 32, 8, peaks, None, copies=10, graph_calls=100)
        gemv_bytes = 448 * 512 * 128 + 512 * 16 + 448 * 32 * 4
        r["gbs"] = gemv_bytes / r["ms"] / 1e6
        r["frac_hbm"] = r["gbs"] / hbm
        r["graph_replay"]["gbs"] = gemv_bytes / r["graph_replay"]["ms_per_call"] / 1e6
        res[k] = r

    # decode-shaped GEMV on a narrowed tile: bf16 1x16x2, one token against the headline weights
    if want("mmt4d_bf16_gemv_1x28672x8192"):
        # two sets of weights used in turn: a call finds none of its 470 MB in the 126 MB L2
        k, r = _mmt4d_case("mmt4d_bf16_gemv_1x28672x8192", abi.MMT4D_BF16BF16F32, 1, 1792, 4096,
                           1, 16, 2, peaks, None, torch.bfloat16, copies=2, graph_calls=20)
        nbytes_gemv = 1792 * 4096 * 64 + 4096 * 4 + 1792 * 64
        r["gbs"] = nbytes_gemv / r["ms"] / 1e6
        r["frac_hbm"] = r["gbs"] / hbm
        r["graph_replay"]["gbs"] = nbytes_gemv / r["graph_replay"]["ms_per_call"] / 1e6
        res[k] = r
    # the same weights against 8 tokens (M0 = 8): bf16, and s8 at the same N and K
    for name, flags, dt, es in [("mmt4d_bf16_gemv_8x28672x8192", abi.MMT4D_BF16BF16F32, torch.bfloat16, 2),
                                ("mmt4d_s8_gemv_8x28672x8192", abi.MMT4D_S8S8S32, None, 1)]:
        if want(name):
            k, r = _mmt4d_case(name, flags, 1, 1792, 4096, 8, 16, 2, peaks, None, dt, copies=2,
                               graph_calls=20)
            nb = 1792 * 4096 * 32 * es + 4096 * 16 * es + 1792 * 8 * 16 * 4
            r["gbs"] = nb / r["ms"] / 1e6
            r["frac_hbm"] = r["gbs"] / hbm
            r["graph_replay"]["gbs"] = nb / r["graph_replay"]["ms_per_call"] / 1e6
            res[k] = r

    if custom_matmul is not None:
        mm, mn, mk = custom_matmul
        res["matmul_rowmajor_bf16_custom_%dx%dx%d" % (mm, mn, mk)] = _matmul_rowmajor_case(
            mm, mn, mk, bf16_peak)
    # the headline problem with the weights prepared once (RHS re-tiled outside the call)
    if want("mmt4d_bf16_prepared_rhs_8192x28672x8192"):
        M1, N1, K1 = 512, 1792, 4096
        lhs = torch.randn(M1 * K1 * 32, device="cuda").to(torch.bfloat16)
        rhs = (torch.randn(N1 * K1 * 32, device="cuda") * 0.02).to(torch.bfloat16)
        out = torch.empty(M1 * N1 * 256, device="cuda")
        p = _mmt4d_params(abi.MMT4D_BF16BF16F32, M1, N1, K1, 16, 16, 2, lhs, rhs, out)
        prepared = torch.empty(uk.mmt4d_prepared_rhs_size(p), dtype=torch.uint8, device="cuda")
        ws = torch.empty(uk.mmt4d_prepared_workspace_size(p), dtype=torch.uint8, device="cuda")
        prep_ms, _ = _time(lambda: uk.mmt4d_prepare_rhs(p, prepared))
        med, best = _time(lambda: uk.mmt4d_prepared(p, prepared, ws))
        ops = 2.0 * 8192 * 28672 * 8192
        res["mmt4d_bf16_prepared_rhs_8192x28672x8192"] = {
            "ms": med, "ms_best": best, "tops": ops / med / 1e9, "prepare_rhs_once_ms": prep_ms,
            "frac_of_bf16_burst": ops / med / 1e9 / bf16_peak}
        del lhs, rhs, out, prepared, ws

    # row-major matmul at the headline dimensions: the fused entry point beside the chain
    # pack LHS, pack RHS (TRANSPOSE_INNER | TRANSPOSE_OUTER), mmt4d, unpack run on this library
    if want("matmul_rowmajor_bf16_8192x28672x8192"):
        res["matmul_rowmajor_bf16_8192x28672x8192"] = _matmul_rowmajor_case(
            8192, 28672, 8192, bf16_peak)

    # pack f32 8192x8192 -> [512][8192][16][1]; TRANSPOSE_INNER variant; RHS-style 0x301.
    # The bandwidth-bound group, too, starts from an idle GPU (see _settle).
    _settle()
    _settle()
    n = 8192
    src = torch.randn(n * n, device="cuda")
    dst = torch.empty(n * n, device="cuda")
    nbytes = 2.0 * n * n * 4

    def pack_params(flags, o0, o1, t0, t1):
        p = abi.PackParams()
        p.in_buffer, p.out_buffer = src.data_ptr(), dst.data_ptr()
        p.in_size0, p.in_size1, p.in_stride0, p.in_stride1 = n, n, n, 1
        p.out_size0, p.out_size1, p.out_size2, p.out_size3 = o0, o1, t0, t1
        p.out_stride1 = t0 * t1
        p.out_stride0 = o1 * p.out_stride1
        p.flags = flags
        return p

    # a plain device copy of the same 256 MiB, timed the same way on this GPU: what the memory
    # system gives a kernel that reads and writes each byte once at this size
    copy_gbs = None
    if only is None or "pack" in only:
        med, _ = _time(lambda: dst.copy_(src))
        copy_gbs = nbytes / med / 1e6
        res["device_copy_256MiB_same_timing"] = {"ms": med, "gbs": copy_gbs, "frac_hbm": copy_gbs / hbm}

    for name, p in [
        ("pack_f32_8192x8192_to_512x8192x16x1", pack_params(abi.PACK_F32F32, 512, 8192, 16, 1)),
        ("pack_f32_transpose_inner_512x8192x1x16",
         pack_params(abi.PACK_F32F32 | abi.PACK_TRANSPOSE_INNER, 512, 8192, 1, 16)),
        ("pack_f32_rhs_0x301_512x8192x16x1",
         pack_params(abi.PACK_F32F32 | abi.PACK_TRANSPOSE_INNER | abi.PACK_TRANSPOSE_OUTER, 512,
                     8192, 16, 1)),
    ]:
        if not want(name):
            continue
        med, best = _time(lambda: uk.pack(p))
        res[name] = {"ms": med, "ms_best": best, "gbs": nbytes / med / 1e6,
                     "frac_hbm": nbytes / med / 1e6 / hbm,
                     "frac_of_same_size_copy": (nbytes / med / 1e6 / copy_gbs) if copy_gbs else None,
                     "path": uk.pack_path(p)}

    # unpack i32 [512][512][16][16] -> 8192x8192
    q = abi.UnpackParams()
    q.in_buffer, q.out_buffer = src.data_ptr(), dst.data_ptr()
    q.in_size0, q.in_size1, q.in_size2, q.in_size3 = 512, 512, 16, 16
    q.in_stride1, q.in_stride0 = 256, 512 * 256
    q.out_size0, q.out_size1, q.out_stride0, q.out_stride1 = n, n, n, 1
    q.flags = abi.UNPACK_I32I32
    if want("unpack_i32_512x512x16x16_to_8192x8192"):
        med, best = _time(lambda: uk.unpack(q))
        res["unpack_i32_512x512x16x16_to_8192x8192"] = {
            "ms": med, "ms_best": best, "gbs": nbytes / med / 1e6,
            "frac_hbm": nbytes / med / 1e6 / hbm,
            "frac_of_same_size_copy": (nbytes / med / 1e6 / copy_gbs) if copy_gbs else None,
            "path": uk.unpack_path(q)}
    return res


def main():
    """``python bench_supplementary.py [--only SUBSTR] [--mmt4d bf16,M1,N1,K1 [--no-ws]]
    [--matmul M,N,K] [--iters N] [--warmup N]``: prints one JSON object. With ``--only`` and one
    iteration it is a small single-kernel run, suitable for a profiler capture."""
    import argparse
    import json
    import os
    global ITERS, WARMUP
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default=None)
    ap.add_argument("--mmt4d", default=None)
    ap.add_argument("--no-ws", action="store_true")
    ap.add_argument("--matmul", default=None, help="M,N,K of a bf16 row-major matmul (elements)")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    ITERS, WARMUP = a.iters, a.warmup
    custom = None
    if a.mmt4d:
        t, m, n, k = a.mmt4d.split(",")
        custom = (t, int(m), int(n), int(k))
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        peaks = json.load(open(peaks_path))
    except OSError:
        peaks = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
    mm = tuple(int(x) for x in a.matmul.split(",")) if a.matmul else None
    only = a.only if a.only is not None else ("\0" if (custom or mm) else None)
    print(json.dumps(run(peaks, only=only, custom=custom, custom_ws=not a.no_ws, custom_matmul=mm)))


if __name__ == "__main__":
    main()
