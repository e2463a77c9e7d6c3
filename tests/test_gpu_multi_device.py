"""iree_uk_b200_mmt4d_sharded: the N-sharded mmt4d driven from one process. With one visible
GPU both "devices" are device 0 (the sharding, the per-device dispatch and the peer-store
kernel still run); with two or more GPUs the shards really live on different devices and the
replicated output crosses NVLink."""
import numpy as np
import pytest

import oracle
from iree_b200 import abi
from oracle import cases

import gpu_util as G

pytestmark = pytest.mark.gpu


def _run(device_ids, replicate, t=abi.MMT4D_S8S8S32, K0=2, dims=(20, 24, 40)):
    import torch
    from iree_b200 import ukernel as uk
    M, N, K = dims
    case = cases.Mmt4dCase(t, 16, 16, K0, M, N, K, 0, seed=21, mode="normal", loose=False)
    want = G.oracle_mmt4d(case)
    world = len(device_ids)
    params, keep, outs, ws, streams = [], [], [], [], []
    for r, dev in enumerate(device_ids):
        with torch.cuda.device(dev):
            lhs = torch.from_numpy(case.lhs).cuda()
            rhs = torch.from_numpy(case.rhs).cuda()
            out = torch.from_numpy(case.out_init.copy()).cuda()
            full = case.params(lhs.data_ptr(), rhs.data_ptr(), out.data_ptr())
            p, _ = uk.shard_params(full, r, world, rhs_is_local=False, out_is_local=False)
            w = torch.empty(max(uk.mmt4d_workspace_size(p), 256), dtype=torch.uint8, device="cuda")
            params.append(p); keep.append((lhs, rhs)); outs.append(out); ws.append(w)
            streams.append(torch.cuda.current_stream())
    uk.mmt4d_sharded(device_ids, params, ws, streams, replicate_output=replicate)
    for dev in set(device_ids):
        torch.cuda.synchronize(dev)
    assert torch.cuda.current_device() == 0
    return case, want, [o.cpu().numpy() for o in outs]


def _devices(n):
    import torch
    have = torch.cuda.device_count()
    return [i % have for i in range(n)]


@pytest.mark.parametrize("world", [1, 2, 3])
def test_sharded_without_replication_each_buffer_holds_its_columns(world):
    from iree_b200 import sharding
    case, want, outs = _run(_devices(world), replicate=False)
    tile = 256 * 4  # bytes of one 16 x 16 x 32-bit output tile (buffers are byte arrays)
    w = want.reshape(case.M, case.N, tile)
    init = case.out_init.reshape(case.M, case.N, tile)
    for r, o in enumerate(outs):
        o = o.reshape(case.M, case.N, tile)
        b, c = sharding.shard_bounds(case.N, r, world)
        assert np.array_equal(o[:, b:b + c], w[:, b:b + c])
        if len(set(_devices(world))) == world:   # distinct buffers: the rest is untouched
            mask = np.ones(case.N, dtype=bool)
            mask[b:b + c] = False
            assert np.array_equal(o[:, mask], init[:, mask])


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("t,K0", [(abi.MMT4D_S8S8S32, 2), (abi.MMT4D_BF16BF16F32, 2)],
                         ids=["s8", "bf16"])
def test_sharded_with_replication_every_buffer_holds_everything(world, t, K0):
    case, want, outs = _run(_devices(world), replicate=True, t=t, K0=K0, dims=(20, 24, 40))
    for o in outs:
        if t == abi.MMT4D_S8S8S32:
            assert np.array_equal(o, want)
        else:
            assert cases.rel_frobenius(o.view(np.float32), want.view(np.float32)) <= 1e-3


def _multicast_worker(rank, world, port):
    """One rank of the multicast test. No rank raises, leaves or tears the process group down
    while any rank's buffer is still bound to the multicast object or any kernel may still be
    storing through it: each rank computes a local verdict without raising, the verdicts are
    combined with an all-reduce so that every rank takes the same path, the multicast object
    is released after a last barrier, and only then does a failed rank assert."""
    import os
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    from iree_b200 import sharding, ukernel as uk
    ok, why, mc = True, "", None
    try:
        case = cases.Mmt4dCase(abi.MMT4D_S8S8S32, 16, 16, 2, 20, 24, 40, 0, seed=21, mode="normal",
                               loose=False)
        want = G.oracle_mmt4d(case)
        mc = sharding.MulticastOutput(case.out_init.nbytes, torch.uint8)
        have_mc = torch.tensor([1 if mc.multicast_ptr else 0], device="cuda")
        dist.all_reduce(have_mc, op=dist.ReduceOp.MIN)
        if int(have_mc.item()) == 0:
            ok, why = False, "no multicast mapping on this system"
        else:
            mc.tensor.copy_(torch.from_numpy(case.out_init.view(np.uint8)))
            lhs, rhs = G.to_device(case.lhs), G.to_device(case.rhs)
            torch.cuda.synchronize()
            dist.barrier()
            full = case.params(lhs.data_ptr(), rhs.data_ptr(), mc.tensor.data_ptr())
            p, _ = uk.shard_params(full, rank, world, rhs_is_local=False, out_is_local=False)
            ws = torch.empty(max(uk.mmt4d_workspace_size(p), 256), dtype=torch.uint8, device="cuda")
            try:
                uk.mmt4d_multicast(p, mc.multicast_ptr, ws)
            except uk.UkernelError as e:
                ok, why = False, repr(e)
            torch.cuda.synchronize()
            dist.barrier()   # every rank's tiles have landed in every buffer
            if ok and uk.device_status() != (0, 0):
                ok, why = False, "device status"
            if ok and not np.array_equal(mc.tensor.cpu().numpy(), want.view(np.uint8)):
                ok, why = False, "rank %d: buffer differs from the reference result" % rank
    except Exception as e:  # reported after the orderly teardown below
        ok, why = False, repr(e)
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    torch.cuda.synchronize()
    dist.barrier()
    mc = None  # released only now: no rank is still storing through the mapping
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()
    assert ok, why
    assert int(flag.item()) == 1, "another rank failed"


def test_multicast_replication_two_processes():
    """Two ranks on two GPUs: each computes its tile columns and stores them once through the
    NVLink multicast mapping; both buffers then hold the oracle's whole result."""
    import socket
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mp.spawn(_multicast_worker, args=(2, port), nprocs=2, join=True)


def _host_sharded_worker(rank, world, port):
    """One rank of the sharded host-buffer call: its own RHS tile rows and output slab in pinned
    host memory, 1/world of the LHS uploaded, the rest received by an NCCL all-gather. Every rank
    reaches the final barrier whatever it found (verdicts are exchanged first)."""
    import os
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    from iree_b200 import sharding, ukernel as uk
    ok, why = True, ""
    try:
        M, N, K = 8, 6, 40
        case = cases.Mmt4dCase(abi.MMT4D_S8S8S32, 16, 16, 2, M, N, K, 0, seed=33, mode="normal",
                               loose=False)
        want = G.oracle_mmt4d(case).view(np.int32).reshape(M, N, 256)
        b, c = sharding.shard_bounds(N, rank, world)
        h_lhs = torch.from_numpy(case.lhs.copy()).pin_memory()
        rhs_rows = case.rhs.reshape(N, -1)[b:b + c].copy()
        h_rhs = torch.from_numpy(rhs_rows).pin_memory()
        h_out = torch.full((M * c * 256,), 7, dtype=torch.int32).pin_memory()
        p = abi.Mmt4dParams()
        p.M, p.N, p.K, p.M0, p.N0, p.K0, p.flags = M, c, K, 16, 16, 2, abi.MMT4D_S8S8S32
        p.lhs_buffer, p.rhs_buffer, p.out_buffer = h_lhs.data_ptr(), h_rhs.data_ptr(), h_out.data_ptr()
        p.lhs_stride0, p.rhs_stride0, p.out_stride0 = K * 32, K * 32, c * 256
        call = sharding.HostShardedMmt4d(p, h_lhs)
        for _ in range(2):  # twice: the second call reuses the arena and the gathered LHS buffer
            h_out.fill_(7)
            call.run()
            torch.cuda.synchronize()
            if not np.array_equal(h_out.numpy().reshape(M, c, 256), want[:, b:b + c]):
                ok, why = False, "rank %d: slab differs from the reference result" % rank
        if ok and uk.device_status() != (0, 0):
            ok, why = False, "device status"
    except Exception as e:
        ok, why = False, repr(e)
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()
    assert ok, why
    assert int(flag.item()) == 1, "another rank failed"


def test_host_buffers_sharded_over_two_processes():
    """Two ranks on two GPUs: the LHS crosses PCIe once (half per rank, completed by an
    all-gather), each rank's host output slab equals the reference's columns."""
    import socket
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mp.spawn(_host_sharded_worker, args=(2, port), nprocs=2, join=True)
