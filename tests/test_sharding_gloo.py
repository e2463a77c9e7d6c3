"""N-sharding across ranks, exercised with two gloo ranks on CPU: each rank takes its
parameters from the C ABI's ``iree_uk_b200_mmt4d_shard_params``, computes its slab (here with
the CPU oracle standing in for the device kernel), and the gathered, interleaved slabs must
equal the unsharded result bit for bit. Covers both addressing modes: a local slab and a slab
addressed inside the full output through out_offset."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from iree_b200 import abi, sharding
from iree_b200 import ukernel as uk
from oracle import cases


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, type_flag, M0, N0, K0, M, N, K):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        case = cases.Mmt4dCase(type_flag, M0, N0, K0, M, N, K, 0, seed=31, mode="normal",
                               loose=False)
        full_out = case.out_init.copy()
        full = case.params(case.lhs, case.rhs, full_out)
        oracle.mmt4d(full)
        want = full_out.view(np.int32).reshape(M, N, M0 * N0)

        # (1) slab inside a full-size output through out_offset, RHS addressed inside the full RHS
        out_a = case.out_init.copy()
        pa, begin = sharding.local_params(case.params(case.lhs, case.rhs, out_a), rank, world,
                                          rhs_is_local=False, out_is_local=False)
        assert (begin, pa.N) == sharding.shard_bounds(N, rank, world)
        oracle.mmt4d(pa)
        got_a = out_a.view(np.int32).reshape(M, N, M0 * N0)
        assert np.array_equal(got_a[:, begin:begin + pa.N], want[:, begin:begin + pa.N])
        untouched = np.ones(N, dtype=bool)
        untouched[begin:begin + pa.N] = False
        init = case.out_init.view(np.int32).reshape(M, N, M0 * N0)
        assert np.array_equal(got_a[:, untouched], init[:, untouched])

        # (2) local RHS rows and a local slab, then all-gather + interleave
        n_local = pa.N
        rb = case.bits[1]
        row_bytes = case.rhs_stride0 * rb // 8
        rhs_local = case.rhs[begin * row_bytes:(begin + n_local) * row_bytes].copy()
        slab = np.zeros(M * n_local * M0 * N0, dtype=np.int32)
        pb, _ = sharding.local_params(case.params(case.lhs, rhs_local, slab), rank, world,
                                      rhs_is_local=True, out_is_local=True)
        assert pb.out_stride0 == n_local * M0 * N0
        oracle.mmt4d(pb)
        gathered = [torch.empty(slab.size, dtype=torch.int32) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(slab))
        # host statement of iree_uk_b200_interleave_slabs: [r][M][N/w][tile] -> [M][N][tile]
        stacked = torch.stack(gathered).numpy().reshape(world, M, n_local, M0 * N0)
        inter = stacked.transpose(1, 0, 2, 3).reshape(M, N, M0 * N0)
        assert np.array_equal(inter, want)
    finally:
        dist.destroy_process_group()


def _run(world, *args):
    mp.spawn(_worker, args=(world, _free_port()) + args, nprocs=world, join=True)


def test_n_sharding_two_ranks_s8():
    _run(2, abi.MMT4D_S8S8S32, 16, 16, 2, 5, 8, 9)


def test_n_sharding_two_ranks_s16u4_gemv_shape():
    _run(2, abi.MMT4D_S16U4S32, 1, 32, 8, 1, 6, 16)


def test_shard_bounds_cover_every_tile_row():
    for n in (1, 7, 8, 30, 1792):
        for world in (1, 2, 4, 8):
            rows = []
            for r in range(world):
                b, c = sharding.shard_bounds(n, r, world)
                rows += list(range(b, b + c))
            assert rows == list(range(n))


def _peer_worker(rank, world, port):
    """Replicated output without an all-gather, on CPU: shared host memory stands in for peer
    device memory. Each rank computes its tile columns with the oracle and stores them into
    every rank's copy, as the device kernel does through the addresses PeerOutputs hands out."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M0 = N0 = 16
        case = cases.Mmt4dCase(abi.MMT4D_S8S8S32, M0, N0, 2, 3, 8, 5, 0, seed=7, mode="normal",
                               loose=False)
        want = case.out_init.copy()
        oracle.mmt4d(case.params(case.lhs, case.rhs, want))
        nbytes = case.out_init.nbytes
        from multiprocessing import shared_memory
        mine = shared_memory.SharedMemory(create=True, size=nbytes)
        opened = []

        def open_(name):
            shm = shared_memory.SharedMemory(name=name)
            opened.append(shm)
            return shm

        peers = sharding.PeerOutputs(mine, export=lambda buf: buf.name, open_=open_,
                                     close=lambda shm: shm.close())
        assert peers.rank == rank and len(peers.ptrs) == world - 1
        local = case.out_init.copy()
        p, begin = sharding.local_params(case.params(case.lhs, case.rhs, local), rank, world,
                                         rhs_is_local=False, out_is_local=False)
        oracle.mmt4d(p)
        tiles = local.view(np.int32).reshape(case.M, case.N, M0 * N0)[:, begin:begin + p.N]
        for shm in [mine] + peers.ptrs:
            dst = np.ndarray((case.M, case.N, M0 * N0), dtype=np.int32, buffer=shm.buf)
            dst[:, begin:begin + p.N] = tiles
            del dst
        dist.barrier()  # every rank's stores have landed in every copy
        got = np.ndarray(want.view(np.int32).shape, dtype=np.int32, buffer=mine.buf).copy()
        assert np.array_equal(got, want.view(np.int32))
        dist.barrier()
        peers.close()
        mine.close()
        mine.unlink()
    finally:
        dist.destroy_process_group()


def test_peer_outputs_replicate_without_a_gather_two_ranks():
    mp.spawn(_peer_worker, args=(2, _free_port()), nprocs=2, join=True)
