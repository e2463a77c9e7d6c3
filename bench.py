#!/usr/bin/env python
"""Headline benchmark: the N-sharded prefill GEMM as one mmt4d call per GPU.

Workload (one "step" = one mmt4d call over the whole problem): mmt4d bf16bf16f32, logical
M = 8192 tokens x K = 8192 x N = 28672 (a Llama-3-70B-shaped FFN up-projection), tiles
16x16x2, i.e. LHS [512][4096][16][2], RHS [1792][4096][16][2], out f32 [512][1792][16][16].
With G GPUs (one process per GPU, launched by torch.distributed.run) rank r owns RHS tile
rows [r*N1/G, (r+1)*N1/G) and writes its own [512][N1/G][16][16] slab: no collective on the
data path, the LHS is replicated. Inputs are synthetic (seeded N(0,1) activations, N(0,0.02)
weights) and much larger than L2.

One JSON line is printed by rank 0. `value` is whole-job TFLOP/s with inputs resident in
HBM, timed with CUDA events on the launching stream, max over ranks. `e2e` is the same
metric through the host-buffer entry point (`iree_uk_b200_mmt4d_host`: pinned host LHS/RHS in,
host output out, copies pipelined against the kernels), all inside the timed region.

`--impl reference` times the reference's own CPU ukernel (compiled under oracle/_ref, all
host cores, M split over threads) on a bounded sample of the same workload.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

M1, K1, N1 = 512, 4096, 1792
M0, N0, K0 = 16, 16, 2
WORKLOAD = "mmt4d_bf16bf16f32_8192x8192x28672_tiles16x16x2_llama3_70b_ffn_up_prefill"


def read_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return json.load(f), "measured"
    except OSError:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.QUERY,
                 "--format=csv,noheader,nounits", "-lms", "10"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [x.strip() for x in line.split(",")]))

    def wait_first_sample(self, timeout=5.0):
        t0 = time.time()
        while self.proc and not self.rows and time.time() - t0 < timeout:
            time.sleep(0.01)

    def mark(self):
        """Host time stamp; samples between two marks belong to the timed region."""
        return time.time()

    def stop(self, t_begin=None, t_end=None):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, maxc, reasons = [], None, set()
        inside = [r for (t, r) in self.rows
                  if (t_begin is None or t >= t_begin) and (t_end is None or t <= t_end + 0.03)]
        if not inside:  # region shorter than the sampling period: take the nearest sample
            inside = [r for (_, r) in self.rows[-1:]]
        for r in inside:
            try:
                clocks.append(float(r[0]))
                maxc = float(r[1])
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        # keep the samples taken under load (upper half of the observed clocks)
        clocks.sort()
        med = clocks[len(clocks) // 2] if clocks else None
        return {"sm_mhz": med, "sm_max_mhz": maxc, "reasons": sorted(reasons),
                "samples": len(clocks)}


class CpuReference:
    """The CPU reference (oracle/_ref when built, else the C port) on a bounded sample of the
    workload: `rows` LHS tile rows, all N and K, tile rows split over all host threads."""

    def __init__(self, max_rows):
        import numpy as np

        import oracle
        from iree_b200 import abi
        self.oracle, self.abi = oracle, abi
        self.kind = "reference" if oracle.ref_available() else "port"
        self.impl = "ref" if self.kind == "reference" else "oracle"
        rng = np.random.default_rng(1234)

        def bf16(n, scale):
            out = np.empty(n, dtype=np.uint16)
            step = 1 << 24
            for i in range(0, n, step):
                x = rng.standard_normal(min(step, n - i), dtype=np.float32) * np.float32(scale)
                out[i:i + step] = (x.view(np.uint32) >> 16).astype(np.uint16)
            return out

        self.max_rows = max_rows
        self.lhs = bf16(max_rows * K1 * M0 * K0, 1.0)
        self.rhs = bf16(N1 * K1 * N0 * K0, 0.02)
        self.out = np.zeros(max_rows * N1 * M0 * N0, dtype=np.float32)
        self.threads = os.cpu_count() or 1

    def run(self, rows):
        """Seconds for one mmt4d over `rows` tile rows; also returns the threads used."""
        abi = self.abi
        rows = min(rows, self.max_rows)
        p = abi.Mmt4dParams()
        p.lhs_buffer, p.rhs_buffer = self.lhs.ctypes.data, self.rhs.ctypes.data
        p.out_buffer = self.out.ctypes.data
        p.M, p.N, p.K, p.M0, p.N0, p.K0 = rows, N1, K1, M0, N0, K0
        p.lhs_stride0, p.rhs_stride0, p.out_stride0 = K1 * M0 * K0, K1 * N0 * K0, N1 * M0 * N0
        p.flags = abi.MMT4D_BF16BF16F32
        t0 = time.perf_counter()
        used = self.oracle.mmt4d_threaded(p, self.threads, self.impl)
        return time.perf_counter() - t0, used

    def sized_rows(self, seconds):
        """Tile rows (a multiple of the thread count) that take about `seconds`."""
        dt, _ = self.run(self.threads)
        rate_rows = self.threads / dt
        rows = int(max(self.threads, min(self.max_rows, round(seconds * rate_rows))))
        return max(self.threads, rows // self.threads * self.threads)


def cpu_supplementary():
    """The CPU reference on the other configurations of the path (or bounded samples of them),
    all host threads, best of a few runs: the small s8 GEMM, the f16 GEMM with ACCUMULATE
    (M reduced), the s16u4 GEMV, and the f32 pack / i32 unpack of an 8192 x 8192 matrix."""
    from concurrent.futures import ThreadPoolExecutor

    import numpy as np

    import oracle
    from iree_b200 import abi
    impl = "ref" if oracle.ref_available() else "oracle"
    kind = "reference" if impl == "ref" else "port"
    threads = os.cpu_count() or 1
    rng = np.random.default_rng(7)
    res = {}

    def best(fn, runs=3):
        times = []
        for _ in range(runs):
            t0 = time.perf_counter()
            fn()
            times.append(time.perf_counter() - t0)
        return min(times)

    def mmt4d_case(name, flags, M, N, K, m0, n0, k0, lhs, rhs, out, sample):
        p = abi.Mmt4dParams()
        p.lhs_buffer, p.rhs_buffer, p.out_buffer = lhs.ctypes.data, rhs.ctypes.data, out.ctypes.data
        p.M, p.N, p.K, p.M0, p.N0, p.K0, p.flags = M, N, K, m0, n0, k0, flags
        lb, rb, _ = abi.MMT4D_BITS[flags & 0xFF]
        p.lhs_stride0, p.rhs_stride0, p.out_stride0 = K * m0 * k0, K * n0 * k0, N * m0 * n0
        used = [0]

        def run():
            used[0] = oracle.mmt4d_threaded(p, threads, impl)
        sec = best(run)
        ops = 2.0 * M * m0 * N * n0 * K * k0
        res[name] = {"ms": sec * 1e3, "tops": ops / sec / 1e12, "threads": used[0], "kind": kind,
                     "sample": sample}

    i8 = lambda n: rng.integers(-128, 128, n, dtype=np.int8)
    mmt4d_case("mmt4d_s8s8s32_1024x1024x1024", abi.MMT4D_S8S8S32, 64, 64, 512, 16, 16, 2,
               i8(1 << 20), i8(1 << 20), np.zeros(1 << 20, dtype=np.int32), "whole problem")
    f16 = lambda n: rng.standard_normal(n, dtype=np.float32).astype(np.float16)
    rows = 64
    mmt4d_case("mmt4d_f16f16f32_acc_4096x4096x4096", abi.MMT4D_F16F16F32 | abi.MMT4D_ACCUMULATE,
               rows, 256, 4096, 16, 16, 1, f16(rows * 4096 * 16), f16(256 * 4096 * 16),
               rng.standard_normal(rows * 256 * 256, dtype=np.float32),
               "M reduced to %d of 256 LHS tile rows" % rows)
    mmt4d_case("mmt4d_s16u4s32_gemv_1x14336x4096", abi.MMT4D_S16U4S32, 1, 448, 512, 1, 32, 8,
               rng.integers(-32768, 32768, 4096, dtype=np.int16),
               rng.integers(0, 256, 448 * 512 * 128, dtype=np.uint8),
               np.zeros(448 * 32, dtype=np.int32), "whole problem, N split over threads")
    res["mmt4d_s16u4s32_gemv_1x14336x4096"]["gbs"] = \
        29425664 / res["mmt4d_s16u4s32_gemv_1x14336x4096"]["ms"] / 1e6

    # pack f32 8192 x 8192 -> [512][8192][16][1] and unpack i32 [512][512][16][16] -> 8192 x 8192,
    # outer tile rows split over threads (callers slice the work, ukernel/README.md:26)
    n = 8192
    src = rng.standard_normal(n * n, dtype=np.float32)
    dst = np.empty(n * n, dtype=np.float32)

    def slices(total):
        per = -(-total // threads)
        return [(b, min(per, total - b)) for b in range(0, total, per)]

    def pack_job(b, c):
        q = abi.PackParams()
        q.in_buffer, q.out_buffer = src.ctypes.data, dst.ctypes.data
        q.in_offset, q.out_offset = b * 16 * n, b * n * 16
        q.in_size0, q.in_size1, q.in_stride0, q.in_stride1 = c * 16, n, n, 1
        q.out_size0, q.out_size1, q.out_size2, q.out_size3 = c, n, 16, 1
        q.out_stride1, q.out_stride0, q.flags = 16, n * 16, abi.PACK_F32F32
        return q

    def unpack_job(b, c):
        q = abi.UnpackParams()
        q.in_buffer, q.out_buffer = src.ctypes.data, dst.ctypes.data
        q.in_offset, q.out_offset = b * 512 * 256, b * 16 * n
        q.in_size0, q.in_size1, q.in_size2, q.in_size3 = c, 512, 16, 16
        q.in_stride1, q.in_stride0 = 256, 512 * 256
        q.out_size0, q.out_size1, q.out_stride0, q.out_stride1 = c * 16, n, n, 1
        q.flags = abi.UNPACK_I32I32
        return q

    for name, make, call in [("pack_f32_8192x8192_to_512x8192x16x1", pack_job, oracle.pack),
                             ("unpack_i32_512x512x16x16_to_8192x8192", unpack_job, oracle.unpack)]:
        jobs = [make(b, c) for b, c in slices(512)]
        with ThreadPoolExecutor(len(jobs)) as ex:
            sec = best(lambda: list(ex.map(lambda q: call(q, impl), jobs)))
        res[name] = {"ms": sec * 1e3, "gbs": 2.0 * n * n * 4 / sec / 1e9, "threads": len(jobs),
                     "kind": kind, "sample": "whole problem, bytes = read + written"}
    return res


def dram_traffic(kernel, workload):
    """dram__bytes_read.sum + dram__bytes_write.sum of one launch of `kernel` on `workload`,
    as recorded from an ncu capture in the tracked table beside the profile summaries; None
    when the table holds no such entry."""
    try:
        with open(os.path.join(ROOT, "profiles", "dram_traffic.json")) as f:
            table = json.load(f)
    except (OSError, ValueError):
        return None
    for row in table.get("captures", []):
        if row.get("kernel") == kernel and row.get("workload") == workload:
            return int(row["dram_bytes_read"]) + int(row["dram_bytes_write"])
    return None


def per_config_rooflines(supp, peaks):
    """One compact roofline entry per configuration of the path that has a target: the kernel,
    its CUDA-event time, what it achieved and the measured peak that bounds it. Tensor-bound
    int8 work is held against twice the measured bf16 burst figure (kind::i8 runs at twice the
    kind::f16 rate; no int8 figure is measured on this pool); HBM-bound work against the
    measured copy rate, bytes = read + written."""
    burst = float(peaks.get("bf16_tflops", 1590.0))
    hbm = float(peaks.get("hbm_gbs", 6650.0))
    out = {}

    def tensor(name, key, kernel, peak, scale=1.0, spec=None):
        r = supp.get(key)
        if not r:
            return
        a = scale * r["tops"]
        out[name] = {"kernel": kernel, "bound": "tensor", "ms": r["ms"], "achieved": a, "peak": peak,
                     "unit": "TOP/s", "frac": a / peak}
        if spec:
            out[name]["frac_of_spec"] = a / spec

    def memory(name, key, kernel, sub=None):
        r = supp.get(key)
        if r and sub:
            r = r.get(sub)
        if not r:
            return
        gbs = r["gbs"]
        out[name] = {"kernel": kernel, "bound": "hbm", "ms": r.get("ms", r.get("ms_per_call")),
                     "achieved": gbs, "peak": hbm, "unit": "GB/s", "frac": gbs / hbm}
        if r.get("ms_best") and r.get("ms"):  # the peak itself is a best-of-10 figure
            out[name]["frac_best_of_runs"] = gbs * r["ms"] / r["ms_best"] / hbm

    tensor("mmt4d_s8s8s32_8192x28672x8192", "mmt4d_s8s8s32_8192x28672x8192",
           "retile_kernel<2> + mmt4d_tc2_kernel<int>", 2 * burst, spec=4500.0)
    tensor("mmt4d_f16f16f32_acc_4096x4096x4096", "mmt4d_f16f16f32_acc_4096x4096x4096",
           "retile_kernel<2> + mmt4d_tc2_kernel<float>", burst, spec=2250.0)
    tensor("mmt4d_s16u4s32_prefill_8192x14336x4096_as_8bit_tensor_work",
           "mmt4d_s16u4s32_prefill_8192x14336x4096",
           "split_s16 + unpack_u4 + mmt4d_tc2_kernel<int> (two i8 products per term)", 2 * burst,
           scale=2.0)
    tensor("mmt4d_bf16_headline_plain_call_pooled_scratch", "mmt4d_bf16_headline_plain_call_pooled_scratch",
           "iree_uk_b200_mmt4d_pooled: retile_kernel<4> + mmt4d_tc2_kernel<float>", burst, spec=2250.0)
    tensor("mmt4d_bf16_headline_plain_call_scratch_free", "mmt4d_bf16_headline_plain_call_scratch_free",
           "iree_uk_b200_mmt4d: mmt4d_tc_sw_kernel", burst, spec=2250.0)
    tensor("mmt4d_s16s16s32_8192x14336x4096_as_8bit_tensor_work", "mmt4d_s16s16s32_8192x14336x4096",
           "retile_split_s16 + mmt4d_tc2_kernel<int> (four i8 products per term)", 2 * burst,
           scale=4.0)
    tensor("mmt4d_s16s8s32_8192x14336x4096_as_8bit_tensor_work", "mmt4d_s16s8s32_8192x14336x4096",
           "retile_split_s16 + retile_kernel<2> + mmt4d_tc2_kernel<int> (two i8 products per term)",
           2 * burst, scale=2.0)
    tensor("mmt4d_s8s4s32_8192x14336x4096", "mmt4d_s8s4s32_8192x14336x4096",
           "widen_s4_kernel + retile_kernel<2> + mmt4d_tc2_kernel<int>", 2 * burst)
    memory("mmt4d_s16u4s32_gemv_1x14336x4096_per_call", "mmt4d_s16u4s32_gemv_1x14336x4096",
           "mmt4d_gemv_s16u4_kernel")
    memory("mmt4d_s16u4s32_gemv_1x14336x4096_graph_replay", "mmt4d_s16u4s32_gemv_1x14336x4096",
           "mmt4d_gemv_s16u4_kernel", sub="graph_replay")
    memory("mmt4d_bf16_gemv_1x28672x8192_narrowed_m0_graph_replay", "mmt4d_bf16_gemv_1x28672x8192",
           "mmt4d_narrow_mma_kernel<bf16, M0=1>", sub="graph_replay")
    memory("mmt4d_bf16_gemv_8x28672x8192_narrowed_m0_graph_replay", "mmt4d_bf16_gemv_8x28672x8192",
           "mmt4d_narrow_mma_kernel<bf16, M0=8>", sub="graph_replay")
    memory("mmt4d_s8_gemv_8x28672x8192_narrowed_m0_graph_replay", "mmt4d_s8_gemv_8x28672x8192",
           "mmt4d_narrow_mma_kernel<s8, M0=8>", sub="graph_replay")
    memory("pack_f32_8192x8192_16x1", "pack_f32_8192x8192_to_512x8192x16x1",
           "relayout_staged_kernel<pack, 16x1>")
    memory("pack_f32_8192x8192_rhs_0x301", "pack_f32_rhs_0x301_512x8192x16x1",
           "relayout_staged_kernel<pack, 1x16 transposed>")
    memory("unpack_i32_8192x8192_16x16", "unpack_i32_512x512x16x16_to_8192x8192",
           "relayout_staged_kernel<unpack, 16x16>")
    return out


def sample_flops(rows):
    return 2.0 * (rows * M0) * (N1 * N0) * (K1 * K0)


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    ref = CpuReference(M1)
    rows = ref.sized_rows(1.5)  # about 1.5 s of host work per step
    kind, used = ref.kind, ref.threads
    times = []
    for i in range(args.warmup + args.steps):
        dt, used = ref.run(rows)
        if i >= args.warmup:
            times.append(dt)
    sec = sum(times) / len(times)
    value = sample_flops(rows) / sec / 1e12
    sample = "M reduced to %d of %d LHS tile rows (all N, all K) per step" % (rows, M1)
    line = {
        "impl": "reference", "metric": "mmt4d_tflops", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": used, "kind": kind,
                         "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--no-supplementary", action="store_true")
    ap.add_argument("--no-replicated", action="store_true",
                    help="skip the replicated-output routes measured at N > 1")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    if args.impl == "reference":
        run_reference_arm(args)
        return

    import numpy as np
    import torch
    import torch.distributed as dist

    from iree_b200 import abi
    from iree_b200 import ukernel as uk

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device; there is no CPU fallback"
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    assert N1 % world == 0, "N1 must divide across ranks"

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- synthetic inputs, generated directly in the tiled layouts ----
    n_local = N1 // world
    gen = torch.Generator(device="cuda").manual_seed(1234 + 4)
    lhs = torch.randn(M1 * K1 * M0 * K0, generator=gen, device="cuda").to(torch.bfloat16)
    gen_w = torch.Generator(device="cuda").manual_seed(99 + rank)
    rhs = (torch.randn(n_local * K1 * N0 * K0, generator=gen_w, device="cuda") * 0.02).to(
        torch.bfloat16)
    out = torch.empty(M1 * n_local * M0 * N0, dtype=torch.float32, device="cuda")

    full = abi.Mmt4dParams()
    full.M, full.N, full.K, full.M0, full.N0, full.K0 = M1, N1, K1, M0, N0, K0
    full.flags = abi.MMT4D_BF16BF16F32
    full.lhs_buffer, full.rhs_buffer, full.out_buffer = lhs.data_ptr(), rhs.data_ptr(), out.data_ptr()
    full.lhs_stride0, full.rhs_stride0 = K1 * M0 * K0, K1 * N0 * K0
    full.out_stride0 = N1 * M0 * N0
    p, n_begin = uk.shard_params(full, rank, world, rhs_is_local=True, out_is_local=True)
    ws = torch.empty(max(uk.mmt4d_workspace_size(p), 1), dtype=torch.uint8, device="cuda")
    path = uk.mmt4d_path(p, True)
    assert path in (abi.PATH_TCGEN05, abi.PATH_TCGEN05_RETILE), "tensor-core path not selected"
    stream = torch.cuda.current_stream()
    launches_per_step = 2 if path == abi.PATH_TCGEN05_RETILE else 1

    # ---- warm-up ----
    for _ in range(args.warmup):
        uk.mmt4d(p, stream, ws)
    barrier()

    # ---- spot check of the result against a plain fp32 matmul of the same tiles ----
    def tile_rows(buf, i, count):
        t = buf.view(-1, K1, 16, K0)[i:i + count].float()          # [c][K1][16][K0]
        return t.permute(0, 2, 1, 3).reshape(count * 16, K1 * K0)  # [c*16][K]
    a = tile_rows(lhs, M1 - 2, 2)
    b = tile_rows(rhs, n_local - 2, 2)
    want = a @ b.t()
    got = out.view(M1, n_local, 16, 16)[M1 - 2:, n_local - 2:].permute(0, 2, 1, 3).reshape(32, 32)
    spot_err = float((got - want).norm() / want.norm())
    assert spot_err < 1e-3, "result check failed: relative error %g" % spot_err

    # ---- timed region: resident inputs ----
    sampler = ClockSampler(local_rank)
    # the library records CUDA events around the pre-pass and the main kernel of every 4th
    # timed step (recording all of them would put three event records into every step)
    uk.kernel_timing(4)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    kernel_ms, prepass_ms = [], []
    barrier()
    if rank == 0:
        sampler.start()
        sampler.wait_first_sample()
    barrier()
    t_begin = sampler.mark()
    ev0.record(stream)
    for _ in range(args.steps):
        uk.mmt4d(p, stream, ws)
    ev1.record(stream)
    barrier()
    t_end = sampler.mark()
    clocks = sampler.stop(t_begin, t_end) if rank == 0 else None
    ms_total = ev0.elapsed_time(ev1)
    # per-kernel durations of the timed steps themselves: the library recorded CUDA events
    # around the pre-pass and the main kernel of every call (the last 64 are kept)
    a_ms, b_ms, n_calls = uk.kernel_timing_mean_ms()
    prepass_ms.append(a_ms)
    kernel_ms.append(b_ms)
    uk.kernel_timing(0)
    st, detail = uk.device_status(stream)
    assert st == 0, "device status %d (0x%x)" % (st, detail)

    t = torch.tensor([ms_total], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / args.steps
    total_flops = 2.0 * (M1 * M0) * (N1 * N0) * (K1 * K0)
    value = total_flops / (ms_step * 1e-3) / 1e12

    # ---- end to end: pinned host buffers, H2D + call + D2H inside the timed region ----
    h_lhs = torch.empty(lhs.numel(), dtype=torch.bfloat16).pin_memory()
    h_rhs = torch.empty(rhs.numel(), dtype=torch.bfloat16).pin_memory()
    h_out = torch.empty(out.numel(), dtype=torch.float32).pin_memory()
    h_lhs.copy_(lhs)
    h_rhs.copy_(rhs)
    h2d = (h_lhs.numel() + h_rhs.numel()) * 2
    d2h = h_out.numel() * 4

    # The host-buffer entry point: params hold HOST pointers, as in the reference's own call;
    # the library copies in, computes and copies back, pipelined over chunks of RHS tile rows.
    hp = abi.Mmt4dParams()
    hp.M, hp.N, hp.K, hp.M0, hp.N0, hp.K0 = M1, n_local, K1, M0, N0, K0
    hp.flags = abi.MMT4D_BF16BF16F32
    hp.lhs_buffer, hp.rhs_buffer, hp.out_buffer = h_lhs.data_ptr(), h_rhs.data_ptr(), h_out.data_ptr()
    hp.lhs_stride0, hp.rhs_stride0, hp.out_stride0 = K1 * M0 * K0, K1 * N0 * K0, n_local * M0 * N0
    # Two routes. (1) every rank makes the plain host-buffer call on its shard (the whole LHS
    # goes up once per rank). (2) N > 1 only: the LHS crosses PCIe once - each rank uploads 1/N
    # of its tile rows, an NVLink all-gather completes it on every GPU - and the call takes the
    # device-resident LHS. Which is faster depends on what the ranks' PCIe links share on the
    # host side, so at N > 1 both are timed and the faster one is the e2e figure (both are kept).
    arena = torch.empty(uk.mmt4d_host_arena_size(hp), dtype=torch.uint8, device="cuda")
    routes = {"iree_uk_b200_mmt4d_host": (lambda: uk.mmt4d_host(hp, arena, stream), h2d)}
    if world > 1:
        from iree_b200 import sharding
        sharded_host = sharding.HostShardedMmt4d(hp, h_lhs)
        routes["LHS 1/N per rank over PCIe + NCCL all-gather; iree_uk_b200_mmt4d_host_resident_lhs"] = (
            lambda: sharded_host.run(stream), sharded_host.h2d_bytes_lhs + h_rhs.numel() * 2)

    def time_route(step):
        step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.e2e_steps):
            step()
        e1.record(stream)
        barrier()
        t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) / args.e2e_steps

    e2e_routes, same = {}, 1
    for name, (step, _) in routes.items():
        h_out.zero_()
        e2e_routes[name] = time_route(step)
        same = min(same, 1 if torch.equal(h_out, out.cpu()) else 0)
    e2e_route = min(e2e_routes, key=e2e_routes.get)
    e2e_ms, h2d = e2e_routes[e2e_route], routes[e2e_route][1]
    if world > 1:  # every rank learns the verdict, so none is left waiting in a collective
        flag = torch.tensor([same], device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        same = int(flag.item())
    assert same == 1, "host-buffer path and device-buffer path disagree"
    e2e_value = total_flops / (e2e_ms * 1e-3) / 1e12

    # ---- replicated output (N > 1): all-gather + interleave beside the fused route, where
    # the kernel's epilogue stores every tile into all ranks' buffers over NVLink ----
    replicated = None
    if world > 1 and not args.no_replicated:
        try:
            from iree_b200 import sharding
            rep_steps = max(3, min(10, args.steps))
            tile = M0 * N0

            def timed(fn):
                fn()
                barrier()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                for _ in range(rep_steps):
                    fn()
                b.record(stream)
                barrier()
                tt = torch.tensor([a.elapsed_time(b)], dtype=torch.float64, device="cuda")
                dist.all_reduce(tt, op=dist.ReduceOp.MAX)
                return float(tt.item()) / rep_steps

            gathered_full = [None]

            def gather_route():
                uk.mmt4d(p, stream, ws)
                gathered_full[0] = sharding.gather_output(out, M1, N1, tile, stream=stream)

            gather_ms = timed(gather_route)
            full_out = torch.zeros(M1 * N1 * tile, dtype=torch.float32, device="cuda")
            full.out_buffer = full_out.data_ptr()
            pr, _ = uk.shard_params(full, rank, world, rhs_is_local=True, out_is_local=False)
            peers = sharding.PeerOutputs(full_out)
            fused_ms = timed(lambda: uk.mmt4d_peers(pr, peers.ptrs, ws, stream))
            same = bool(torch.equal(full_out, gathered_full[0]))
            flag = torch.tensor([1 if same else 0], device="cuda")
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            assert int(flag.item()) == 1, "fused replication and all-gather route disagree"
            barrier()
            peers.close()
            # third route: one multimem.st per tile through an NVLink multicast mapping
            mc_ms, mc_note, mc, mc_same = None, None, None, 1
            try:
                mc = sharding.MulticastOutput(M1 * N1 * tile, torch.float32)
                if mc.multicast_ptr:
                    full.out_buffer = mc.tensor.data_ptr()
                    pm, _ = uk.shard_params(full, rank, world, rhs_is_local=True, out_is_local=False)
                    mc_ms = timed(lambda: uk.mmt4d_multicast(pm, mc.multicast_ptr, ws, stream))
                    ok = torch.tensor([1 if torch.equal(mc.tensor, gathered_full[0]) else 0], device="cuda")
                    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
                    mc_same = int(ok.item())  # asserted below, after the orderly release
                else:
                    mc_note = "no multicast support reported"
            except Exception as e:  # symmetric memory unavailable: the other two routes stand
                mc_note = repr(e)[:200]
            # The buffer stays bound to the multicast object until every rank is done with it:
            # all ranks meet here, release it, and meet again before anyone moves on.
            barrier()
            mc = None
            barrier()
            assert mc_same == 1, "multicast route and all-gather route disagree"
            nvlink_bytes = (world - 1) * out.numel() * 4  # leaves each GPU per step
            replicated = {
                "gather_route_ms": gather_ms, "fused_peer_store_ms": fused_ms,
                "fused_tflops": total_flops / (fused_ms * 1e-3) / 1e12,
                "gather_route_tflops": total_flops / (gather_ms * 1e-3) / 1e12,
                "nvlink_bytes_out_per_gpu": nvlink_bytes,
                "fused_nvlink_gbs_per_gpu": nvlink_bytes / fused_ms / 1e6,
                "fused_multicast_ms": mc_ms, "fused_multicast_note": mc_note,
                "fused_multicast_tflops": (total_flops / (mc_ms * 1e-3) / 1e12) if mc_ms else None,
                "results_identical_on_all_ranks": True, "steps": rep_steps,
            }
            del gathered_full, full_out
        except AssertionError:
            raise  # a wrong result is never swallowed
        except Exception as e:  # an unavailable extra never blocks the headline line
            replicated = {"error": repr(e)[:300]}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks, peak_kind = read_peaks()
    k_ms = sorted(kernel_ms)[len(kernel_ms) // 2]
    local_flops = total_flops / world
    achieved = local_flops / (k_ms * 1e-3) / 1e12
    # Which measured cuBLAS figure the kernel is held against depends on what was timed: the
    # burst figure when the timed region is short (under a second) or the SM clock sampled during
    # it stayed within 5 % of its maximum, the sustained (power-capped) figure otherwise.
    burst = float(peaks.get("bf16_tflops", 1590.0))
    sustained = float(peaks.get("bf16_tflops_sustained", burst))
    region_s = ms_total * 1e-3
    sm, sm_max = (clocks or {}).get("sm_mhz"), (clocks or {}).get("sm_max_mhz")
    at_full_clock = bool(sm and sm_max and sm >= 0.95 * sm_max)
    use_burst = region_s < 1.0 or at_full_clock
    peak = burst if use_burst else sustained
    supp = None
    if world == 1 and not args.no_supplementary:
        try:
            import bench_supplementary
            supp = bench_supplementary.run(peaks)
        except Exception as e:  # supplementary figures never block the headline line
            supp = {"error": repr(e)}
    roofline = {
        "bound": "tensor", "kernel": "mmt4d_tc2_kernel (two-CTA tcgen05)", "achieved": achieved,
        "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
        "peak_kind": "%s, cuBLAS bf16 %s (timed region %.3f s, median SM clock %s of %s MHz)" % (
            peak_kind, "burst" if use_burst else "sustained", region_s, sm, sm_max),
        "frac_of_burst": achieved / burst, "frac_of_sustained": achieved / sustained,
        "frac_of_spec_2250": achieved / 2250.0,
        "traffic": dram_traffic("mmt4d_tc2_kernel", WORKLOAD) if world == 1 else None,
        "kernel_ms": k_ms, "prepass_ms": sorted(prepass_ms)[len(prepass_ms) // 2],
        "kernel_ms_from": "mean over %d of the timed steps (every 4th), CUDA events around the kernel" % n_calls,
    }
    if supp and "error" not in supp:
        roofline["per_config"] = per_config_rooflines(supp, peaks)

    cpu = None
    if world == 1:
        ref = CpuReference(256)
        rows = ref.sized_rows(15.0)  # about 15 s of host work
        dt, used = ref.run(rows)
        kind = ref.kind
        cpu = {"value": sample_flops(rows) / dt / 1e12, "unit": "TFLOP/s", "cores": used,
               "kind": kind,
               "sample": "M reduced to %d of %d LHS tile rows (all N, all K), one run" % (rows, M1)}

    line = {
        "metric": "mmt4d_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "tiles": "M0=16,N0=16,K0=2",
                   "sharding": "N1 split over %d rank(s), no data-path collective" % world,
                   "l2": "inputs_larger_than_l2", "path": "tcgen05+retile" if launches_per_step == 2 else "tcgen05",
                   "spot_check_rel_err": spot_err},
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "steps": args.e2e_steps,
                "bytes_are": "per rank" if world > 1 else "whole job",
                "route": e2e_route, "ms_per_step_by_route": e2e_routes},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu,
    }
    if replicated is not None:
        line["replicated_output"] = replicated
    if supp is not None:
        line["supplementary"] = supp
        try:
            line["supplementary_cpu_reference"] = cpu_supplementary()
        except Exception as e:
            line["supplementary_cpu_reference"] = {"error": repr(e)}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
