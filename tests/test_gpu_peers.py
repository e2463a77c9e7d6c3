"""mmt4d with peer copies of the output (iree_uk_b200_mmt4d_ws_peers): every output tile is
stored by the same kernel to further buffers. On one GPU the "peers" are other buffers of the
same device, first in this process and then in another process through the IPC handle
helpers; no kernel waits on another one, so a single GPU can run both cases."""
import os
import subprocess
import sys

import numpy as np
import pytest

from iree_b200 import abi
from oracle import cases

import gpu_util as G

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("spec", [
    (abi.MMT4D_S8S8S32, 16, 16, 2, 9, 17, 65, 0, False),
    (abi.MMT4D_S8S8S32, 16, 16, 2, 9, 17, 65, 1, True),     # gap between tile rows: 16-byte stores
    (abi.MMT4D_BF16BF16F32, 16, 16, 2, 32, 40, 70, 1, False),
    (abi.MMT4D_F16F16F32, 16, 16, 1, 160, 64, 33, 0, False),  # two-CTA kernel
], ids=["s8", "s8_acc_loose", "bf16_acc", "f16_pair"])
def test_peer_copies_on_the_same_device(spec):
    import torch
    from iree_b200 import ukernel as uk
    t, M0, N0, K0, M, N, K, acc, loose = spec
    case = cases.Mmt4dCase(t, M0, N0, K0, M, N, K, acc, seed=5, mode="normal", loose=False)
    if loose:  # a gap of 16 bytes between tile rows: the 16-byte store path
        case.out_stride0 += 4
        case.out_init = cases.random_elements(
            "s32", case.out_offset + case.M * case.out_stride0, np.random.default_rng(5))
    want = G.oracle_mmt4d(case)
    lhs, rhs, out = G.to_device(case.lhs), G.to_device(case.rhs), G.to_device(case.out_init)
    # peers start from a different content: only the tiles may change, and ACCUMULATE must
    # take the old values from the local buffer
    init_bytes = case.out_init.view(np.uint8)
    peers = [G.to_device(np.full(init_bytes.size, 0x5A, dtype=np.uint8)) for _ in range(3)]
    p = case.params(lhs.data_ptr(), rhs.data_ptr(), out.data_ptr())
    ws = torch.empty(uk.mmt4d_workspace_size(p), dtype=torch.uint8, device="cuda")
    uk.mmt4d_peers(p, [x.data_ptr() for x in peers], ws)
    torch.cuda.synchronize()
    G.check_device_status()
    got = out.cpu().numpy()
    if t == abi.MMT4D_S8S8S32:
        assert np.array_equal(got, want)
    else:
        assert cases.rel_frobenius(got.view(np.float32), want.view(np.float32)) <= 1e-3
    got_bytes = got.view(np.uint8)
    tile_mask = _tile_mask(case)
    assert np.array_equal(got_bytes[~tile_mask], init_bytes[~tile_mask])
    for x in peers:
        pg = x.cpu().numpy()
        # every tile byte equals the local result; everything between tiles keeps its fill
        assert np.array_equal(pg[tile_mask], got_bytes[tile_mask])
        assert np.all(pg[~tile_mask] == 0x5A)


def _tile_mask(case):
    """Bytes of the output allocation that belong to output tiles."""
    mask = np.zeros(case.out_init.nbytes, dtype=bool)
    tile_bytes = case.M0 * case.N0 * 4
    for i in range(case.M):
        start = (case.out_offset + i * case.out_stride0) * 4
        mask[start:start + case.N * tile_bytes] = True
    return mask


def test_unsupported_problems_launch_nothing():
    import torch
    from iree_b200 import ukernel as uk
    case = cases.Mmt4dCase(abi.MMT4D_F32F32F32, 8, 8, 1, 2, 2, 4, 0, seed=1, mode="normal",
                           loose=False)
    lhs, rhs, out = G.to_device(case.lhs), G.to_device(case.rhs), G.to_device(case.out_init)
    peer = G.to_device(case.out_init)
    p = case.params(lhs.data_ptr(), rhs.data_ptr(), out.data_ptr())
    ws = torch.empty(1 << 20, dtype=torch.uint8, device="cuda")
    with pytest.raises(uk.UkernelError) as e:
        uk.mmt4d_peers(p, [peer.data_ptr()], ws)
    assert e.value.status == abi.UNSUPPORTED
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy().view(np.uint8), case.out_init.view(np.uint8))
    assert np.array_equal(peer.cpu().numpy().view(np.uint8), case.out_init.view(np.uint8))


CHILD = r"""
import sys
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, sys.argv[1] + "/tests")
import torch
import gpu_util as G
from iree_b200 import abi, ukernel as uk
from oracle import cases
case = cases.Mmt4dCase(abi.MMT4D_S8S8S32, 16, 16, 2, 12, 20, 40, 0, seed=9, mode="normal",
                       loose=False)
lhs, rhs, out = G.to_device(case.lhs), G.to_device(case.rhs), G.to_device(case.out_init)
peer = uk.peer_open(bytes.fromhex(sys.argv[2]))
p = case.params(lhs.data_ptr(), rhs.data_ptr(), out.data_ptr())
ws = torch.empty(uk.mmt4d_workspace_size(p), dtype=torch.uint8, device="cuda")
uk.mmt4d_peers(p, [peer], ws)
torch.cuda.synchronize()
assert uk.device_status() == (0, 0)
uk.peer_close(peer)
print("CHILD_DONE")
"""


def test_peer_buffer_of_another_process():
    """The parent exports its buffer, a child process opens it and runs the mmt4d with that
    buffer as its peer; the parent then finds the oracle's result in its own memory."""
    import torch
    from iree_b200 import ukernel as uk
    case = cases.Mmt4dCase(abi.MMT4D_S8S8S32, 16, 16, 2, 12, 20, 40, 0, seed=9, mode="normal",
                           loose=False)
    want = G.oracle_mmt4d(case)
    # a buffer inside a larger allocation, so that the handle carries a non-zero offset
    nbytes = case.out_init.nbytes
    pool = torch.zeros(nbytes + 4096, dtype=torch.uint8, device="cuda")
    mine = pool[1024:1024 + nbytes]
    mine.copy_(torch.from_numpy(case.out_init.view(np.uint8)))
    torch.cuda.synchronize()
    handle = uk.peer_export(mine)
    r = subprocess.run([sys.executable, "-c", CHILD, ROOT, handle.hex()], capture_output=True,
                       text=True, timeout=300)
    assert r.returncode == 0 and "CHILD_DONE" in r.stdout, r.stdout + r.stderr
    torch.cuda.synchronize()
    assert np.array_equal(mine.cpu().numpy(), want.view(np.uint8))
    assert int(pool[:1024].sum()) == 0 and int(pool[1024 + nbytes:].sum()) == 0
