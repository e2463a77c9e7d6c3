"""N-sharding of mmt4d across GPUs: one process per GPU, no data-path collective.

mmt4d output tile columns j depend only on RHS tile row j (the j loop of
runtime/src/iree/builtins/ukernel/mmt4d.c:84-98 only advances ``rhs_panel`` and
``out_tile``), so GPU r of G owns RHS tile rows [r*N/G, (r+1)*N/G), receives the full LHS and
writes its own [M][N/G][M0][N0] slab. The arithmetic lives in the C ABI
(``iree_uk_b200_mmt4d_shard_params``); this module adds the optional replication of the output
through ``torch.distributed`` (NCCL all-gather of the slabs, then the library's interleave
kernel).
"""
from . import ukernel as uk


def shard_bounds(n_tiles, rank, world):
    """(first tile row, count) owned by ``rank``: contiguous, remainder on the first ranks —
    the same split ``iree_uk_b200_mmt4d_shard_params`` computes."""
    base, rem = divmod(n_tiles, world)
    begin = rank * base + min(rank, rem)
    return begin, base + (1 if rank < rem else 0)


def local_params(full, rank, world, rhs_is_local=True, out_is_local=True):
    """This rank's ``Mmt4dParams`` and its first owned tile row."""
    return uk.shard_params(full, rank, world, rhs_is_local, out_is_local)


def gather_output(slab, M, N, tile_elems, group=None, stream=None):
    """Replicate the output: all-gather equal per-rank slabs [M][N/world][tile] (a CUDA
    tensor) and interleave them into [M][N][tile]. Returns the full tensor."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    if N % world:
        raise ValueError("gather_output needs N divisible by the world size")
    gathered = torch.empty(world * slab.numel(), dtype=slab.dtype, device=slab.device)
    dist.all_gather_into_tensor(gathered, slab.contiguous().view(-1), group=group)
    full = torch.empty_like(gathered)
    uk.interleave_slabs(gathered, full, M, N, tile_elems, slab.element_size(), world, stream)
    return full


class HostShardedMmt4d:
    """The N-sharded mmt4d on HOST buffers: every rank holds the same LHS and its own RHS tile
    rows in (pinned) host memory and wants its own output slab in host memory.

    Uploading the whole LHS to every GPU sends it over PCIe ``world`` times, and the ranks of one
    machine share the host side of those links. Here the LHS crosses PCIe once: rank r uploads
    tile rows [r*M/world, (r+1)*M/world) into its place in a device buffer of the whole LHS, an
    all-gather over NVLink (NCCL, in place) completes that buffer on every GPU, and
    ``iree_uk_b200_mmt4d_host_resident_lhs`` runs the rest (RHS chunks in, kernels, output slabs
    out, pipelined). M must be divisible by the world size. ``params`` is this rank's
    ``Mmt4dParams`` with host pointers (as for ``ukernel.mmt4d_host``); ``host_lhs`` a pinned
    CPU tensor holding the whole LHS with tight tile rows."""

    def __init__(self, params, host_lhs, group=None):
        import torch
        import torch.distributed as dist
        self.dist, self.group, self.torch = dist, group, torch
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if params.M % self.world:
            raise ValueError("HostShardedMmt4d needs M divisible by the world size")
        self.params, self.host_lhs = params, host_lhs
        self.lhs_dev = torch.empty_like(host_lhs, device="cuda")
        self.row_elems = host_lhs.numel() // params.M
        per = (params.M // self.world) * self.row_elems
        self.my_dev = self.lhs_dev.view(-1)[self.rank * per:(self.rank + 1) * per]
        self.my_host = host_lhs.view(-1)[self.rank * per:(self.rank + 1) * per]
        self.arena = torch.empty(uk.mmt4d_host_arena_size(params), dtype=torch.uint8, device="cuda")
        self.h2d_bytes_lhs = per * host_lhs.element_size()

    def run(self, stream=None):
        """Enqueues one call on ``stream`` (a torch stream; default: the current one); the host
        output is complete once that stream has been synchronised."""
        torch = self.torch
        stream = stream if stream is not None else torch.cuda.current_stream()
        with torch.cuda.stream(stream):  # the copy and the collective are ordered on `stream`
            self.my_dev.copy_(self.my_host, non_blocking=True)
            self.dist.all_gather_into_tensor(self.lhs_dev.view(-1), self.my_dev, group=self.group)
            uk.mmt4d_host_resident_lhs(self.params, self.lhs_dev, self.row_elems, self.arena, stream)


class PeerOutputs:
    """The other ranks' copies of a replicated output buffer, addressable from this GPU.

    Every rank allocates a full [M][N][M0][N0] buffer and calls ``PeerOutputs(buffer, group)``
    (a collective: handles travel through ``all_gather_object``). ``ptrs`` then lists the
    addresses of the other ranks' buffers for ``ukernel.mmt4d_peers``, so that each rank's
    kernel stores its tile columns into all copies and no all-gather is needed. ``exchange``,
    ``export`` and ``open_`` are injectable for tests that run without GPUs."""

    def __init__(self, buffer, group=None, export=None, open_=None, close=None, exchange=None):
        export = export or uk.peer_export
        self._close = close or uk.peer_close
        open_ = open_ or uk.peer_open
        if exchange is None:
            import torch.distributed as dist

            def exchange(mine):
                got = [None] * dist.get_world_size(group)
                dist.all_gather_object(got, mine, group=group)
                return got, dist.get_rank(group)
        handles, rank = exchange(export(buffer))
        self.rank = rank
        self.ptrs = [open_(h) for r, h in enumerate(handles) if r != rank]

    def close(self):
        for ptr in self.ptrs:
            self._close(ptr)
        self.ptrs = []


class MulticastOutput:
    """A replicated output buffer reachable through an NVLink multicast mapping.

    A collective over ``group``: every rank gets ``tensor`` (its own full-size buffer, 1-D, of
    ``numel`` elements of ``dtype``) and ``multicast_ptr``, the address of the mapping that
    writes into all ranks' buffers at once (for ``ukernel.mmt4d_multicast``). The buffers and
    the mapping come from ``torch.distributed._symmetric_memory``; ``multicast_ptr`` is 0 where
    the system has no multicast support (no NVSwitch), and callers then use ``PeerOutputs``."""

    def __init__(self, numel, dtype, group=None):
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        group = group if group is not None else dist.group.WORLD
        self.tensor = symm_mem.empty(numel, dtype=dtype, device=torch.device("cuda", torch.cuda.current_device()))
        self.handle = symm_mem.rendezvous(self.tensor, group)
        base = int(self.handle.multicast_ptr)
        offset = int(getattr(self.handle, "offset", 0) or 0)
        self.multicast_ptr = base + offset if base else 0  # stands for tensor.data_ptr()
        self.peer_ptrs = [int(p) for r, p in enumerate(self.handle.buffer_ptrs)
                          if r != dist.get_rank(group)]
