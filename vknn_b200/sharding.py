"""Multi-GPU host logic: the path shards into independent (batch, head) units, so ranks never exchange data inside
a step. One process per GPU (torch.distributed; NCCL on GPUs, gloo in the CPU tests). The only collective is the
optional all-gather of the attention output for a consumer that needs every head on every rank (the boundary
where a head-sharded attention meets a replicated output projection).

The reference has no multi-device code at all (single device, batch-1 planning, docs/LIMITATIONS.md:15-32)."""
from __future__ import annotations

import os


def shard_range(n_units, rank, world):
    """Contiguous, balanced split of n_units over `world` ranks: the first n_units % world ranks get one extra."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("bad rank %d of %d" % (rank, world))
    base, extra = divmod(n_units, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_dim(t, dim, rank, world):
    """The rank's slice of tensor `t` along `dim` (a view, no copy)."""
    lo, hi = shard_range(t.shape[dim], rank, world)
    return t.narrow(dim, lo, hi - lo)


def gather_dim(local, dim, n_total, group=None):
    """All-gather ragged shards along `dim` back into the full tensor on every rank. Shards may differ by one unit,
    so they are padded to the largest shard for the collective and trimmed afterwards."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    if world == 1:
        return local
    sizes = [shard_range(n_total, r, world) for r in range(world)]
    biggest = max(hi - lo for lo, hi in sizes)
    moved = local.movedim(dim, 0).contiguous()
    if moved.shape[0] < biggest:
        pad = torch.zeros((biggest - moved.shape[0],) + tuple(moved.shape[1:]), dtype=moved.dtype, device=moved.device)
        moved = torch.cat([moved, pad], 0)
    out = [torch.empty_like(moved) for _ in range(world)]
    dist.all_gather(out, moved, group=group)
    full = torch.cat([o[: hi - lo] for o, (lo, hi) in zip(out, sizes)], 0)
    return full.movedim(0, dim).contiguous()


def qkv_head_slice(wqkv, bqkv, heads, rank, world):
    """This rank's heads of a packed QKV projection: Wqkv [d, 3*d] is read as [d, 3, heads, D] and bqkv [3*d] as
    [3, heads, D]; the slice keeps heads [rank*heads/world, (rank+1)*heads/world) of each of Q, K and V, packed the same way
    ([d, 3*Hl*D] and [3*Hl*D]). Torch tensors on any device."""
    if heads % world:
        raise ValueError("%d heads do not divide over %d ranks" % (heads, world))
    d = wqkv.shape[0]
    D, Hl = d // heads, heads // world
    wq = wqkv.view(d, 3, heads, D)[:, :, rank * Hl:(rank + 1) * Hl].reshape(d, 3 * Hl * D).contiguous()
    bq = bqkv.view(3, heads, D)[:, rank * Hl:(rank + 1) * Hl].reshape(3 * Hl * D).contiguous()
    return wq, bq


class _RawCuda:
    """Zero-copy torch view of a raw device pointer (through __cuda_array_interface__)."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (int(ptr), False), "version": 2}


def tensor_at(ptr, nbytes, dtype, shape, device):
    import torch
    return torch.as_tensor(_RawCuda(ptr, nbytes), device=device).view(dtype).view(*shape)


class PeerGather:
    """The gather buffers of a head-sharded encoder, shared between the ranks of one node so that the attention kernel
    itself can store its output tiles into every rank's buffer (vkc_attn_prefill_fanout) instead of an all-gather after it.

    Every rank allocates one block: two [rows, width] buffers (consecutive fan-outs alternate between them: a rank can be at
    most one fan-out ahead of a peer that still reads the other buffer) and one 32-bit flag per rank. The blocks are
    exchanged as 64-byte handles over the process group and mapped into every process; data then moves by plain peer stores
    over NVLink, and completion by one flag word per (writer, reader) pair. Waiting is bounded on the device
    (vkc_peer_wait): a rank that never arrives shows up as an error of the next sync, not as a hang."""

    FLAG_BYTES = 256

    def __init__(self, ctx, rows, width, dtype, group=None, multicast=True):
        import torch
        import torch.distributed as dist
        self.ctx, self.rows, self.width, self.dtype = ctx, rows, width, dtype
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world > 8:
            raise ValueError("PeerGather covers the GPUs of one node (at most 8 ranks)")
        esize = torch.empty((), dtype=dtype).element_size()
        self.buf_bytes = (rows * width * esize + 255) // 256 * 256
        self.block_bytes = 2 * self.buf_bytes + self.FLAG_BYTES
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.mcast_base, self._symm = 0, None
        # First choice: a symmetric-memory block with an NVSwitch multicast mapping (the allocation, the exchange of handles and
        # the multicast object are torch's; the stores are this library's kernels). One multimem store then reaches every rank,
        # so a producer pushes its rows through NVLink once instead of once per peer. Every rank must take the same route, so
        # the outcome is agreed on before anything is used; any failure falls back to plain peer mappings.
        if multicast and self.world > 1 and os.environ.get("VKNN_PEER_MULTICAST", "1") != "0":
            self._try_symmetric(group)
        if self._symm is not None:
            self.local = int(self.base[self.rank])
        else:
            self._plain_peer_mappings(ctx, group)
        self.state = torch.zeros(2, dtype=torch.int32, device=self.device)
        self.expected = torch.zeros(2, dtype=torch.int32, device=self.device)  # [0] fan-outs consumed so far, [1] CTA counter of a gated kernel
        self.calls = 0
        self.buffers = [tensor_at(self.local + k * self.buf_bytes, rows * width * esize, dtype, (rows, width), self.device) for k in range(2)]
        self._esize = esize

    def _try_symmetric(self, group):
        import torch
        import torch.distributed as dist

        def agreed(flag):
            oks = [None] * self.world
            dist.all_gather_object(oks, bool(flag), group=group)
            return all(oks)

        t, hdl, ok = None, None, False
        try:
            import torch.distributed._symmetric_memory as symm_mem
            from torch._C._distributed_c10d import _SymmetricMemory
            from torch._C._autograd import DeviceType
            ok = bool(_SymmetricMemory.has_multicast_support(DeviceType.CUDA, self.device.index))
            if ok:
                t = symm_mem.empty(self.block_bytes, dtype=torch.uint8, device=self.device)
                t.zero_()
                torch.cuda.synchronize()
        except Exception:  # noqa: BLE001 - no symmetric memory on this system
            ok = False
        if not agreed(ok):  # every rank allocates, or none goes into the collective below
            return
        try:
            hdl = symm_mem.rendezvous(t, group if group is not None else dist.group.WORLD)
            ok = int(hdl.multicast_ptr) != 0 and len(hdl.buffer_ptrs) == self.world
        except Exception:  # noqa: BLE001 - no multicast mapping could be made
            ok = False
        if agreed(ok):
            self._symm = (t, hdl)
            self.base = [int(p) for p in hdl.buffer_ptrs]
            self.mcast_base = int(hdl.multicast_ptr)

    def _plain_peer_mappings(self, ctx, group):
        import torch
        import torch.distributed as dist
        # Every rank takes part in both exchanges whatever happened locally, and all ranks then fail together: a rank that
        # raised on its own would leave the others waiting in a collective.
        self.local, self.base, handle, err = None, [], None, None
        try:
            self.local = ctx.raw_alloc(self.block_bytes)
            tensor_at(self.local, self.block_bytes, torch.uint8, (self.block_bytes,), self.device).zero_()
            torch.cuda.synchronize()
            handle = ctx.peer_export(self.local)
        except Exception as e:  # noqa: BLE001
            err = e
        handles = [None] * self.world
        dist.all_gather_object(handles, handle, group=group)
        if err is None and all(h is not None for h in handles):
            try:
                self.base = [self.local if r == self.rank else ctx.peer_open(handles[r]) for r in range(self.world)]
            except Exception as e:  # noqa: BLE001
                err = e
        oks = [None] * self.world
        dist.all_gather_object(oks, err is None and len(self.base) == self.world, group=group)  # also: every block is zeroed and mapped
        if not all(oks):
            if self.local is not None:
                ctx.raw_free(self.local)
            raise RuntimeError("PeerGather: sharing the gather buffers failed on rank(s) %s%s"
                               % ([r for r, ok in enumerate(oks) if not ok], (": %s" % err) if err is not None else ""))

    def mcast(self, k, col_offset):
        """Where this rank's columns start in buffer k of the multicast mapping (None without one)."""
        return self.mcast_base + k * self.buf_bytes + col_offset * self._esize if self.mcast_base else None

    def next_buffer(self):
        """Index of the buffer the next fan-out writes (and the next wait makes readable)."""
        k = self.calls % 2
        self.calls += 1
        return k

    def dests(self, k, col_offset):
        """Where this rank's columns start in buffer k of every rank."""
        return [b + k * self.buf_bytes + col_offset * self._esize for b in self.base]

    def flags(self):
        """The word this rank owns in every rank's flag array."""
        return [b + 2 * self.buf_bytes + 4 * self.rank for b in self.base]

    def wait(self, stream=None):
        self.ctx.peer_wait(self.local + 2 * self.buf_bytes, self.world, self.expected, stream=stream)

    def gate(self):
        """The same wait as a gate of the consuming GEMM (Context.gemm(..., gate=...)): flag array, flag count, state words."""
        return (self.local + 2 * self.buf_bytes, self.world, self.expected)

    def close(self):
        """Collective: every rank has finished using the buffers before any mapping goes away."""
        import torch
        import torch.distributed as dist
        torch.cuda.synchronize()
        if self._symm is not None:
            dist.barrier()
            torch.cuda.synchronize()
            self.buffers, self._symm, self.mcast_base = [], None, 0
            self.base = []
            return
        for r, b in enumerate(self.base):
            if r != self.rank:
                self.ctx.peer_close(b)
        self.ctx.raw_free(self.local)
        self.base = []
