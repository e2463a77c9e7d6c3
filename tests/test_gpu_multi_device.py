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
