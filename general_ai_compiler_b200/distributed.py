"""Query-block sharding of MSDA and camera/row sharding of DCNv2 across the GPUs of one node.

The reference is single-device (``src/gac/execution/cuda.py:132-138``); this
module adds the one thing the path needs to scale: every output element
depends on the read-only ``value`` (or image/weights) and on its own
locations/weights only, so ranks are independent once ``value`` is replicated.

* ``query_block`` / ``unit_block``: balanced contiguous partitions.
* ``broadcast_value``: one NCCL (or gloo) broadcast of the replicated tensor
  into each rank's OWN memory, timed on the device.  Kernels never read a
  peer's memory.
* ``sharded_msda``: each rank computes its query block with the local kernel;
  optionally all-gathers the blocks.  The concatenation equals the single-GPU
  output bit for bit (same per-row arithmetic).
* ``ShardedMsda``: the same sharding when ``value`` arrives S-sharded (each
  rank uploads 1/N of it): per batch entry an all-gather (or broadcast) over
  NVLink into each GPU's own memory, pipelined against the kernel.
* ``bind_host_near_gpu``: NUMA placement of a rank's pinned staging buffers.
* ``dcn_units``: (camera, output-row block) work units so that 6 cameras still
  keep 4 or 8 GPUs busy.

One process per GPU, ``torch.distributed`` for the plumbing.
"""

from __future__ import annotations

import math
import time
from typing import Callable, Sequence

import numpy as np


def unit_block(total: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous block [begin, end) of ``total`` units for ``rank``; sizes differ by at most one."""
    if world <= 0 or not 0 <= rank < world or total < 0:
        raise ValueError(f"bad partition request total={total} world={world} rank={rank}")
    base, extra = divmod(total, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def query_block(total_queries: int, world: int, rank: int) -> tuple[int, int]:
    return unit_block(total_queries, world, rank)


def dcn_units(cameras: int, out_rows: int, world: int, rows_per_unit: int | None = None) -> list[tuple[int, int, int]]:
    """(camera, row_begin, row_end) units: whole cameras when they divide the ranks evenly, else row blocks
    sized so every rank gets the same number of units."""
    if rows_per_unit is None:
        if cameras % world == 0:
            rows_per_unit = out_rows
        else:
            per_cam = world // math.gcd(int(cameras), int(world))
            rows_per_unit = -(-out_rows // per_cam)
    units = []
    for n in range(cameras):
        for r0 in range(0, out_rows, rows_per_unit):
            units.append((n, r0, min(out_rows, r0 + rows_per_unit)))
    return units


def dcn_rank_pieces(cameras: int, out_rows: int, world: int, rank: int) -> list[tuple[int, int, int, int]]:
    """The launches rank `rank` makes in the balanced split, as (n_begin, n_end, row_begin, row_end): its contiguous
    share of ``dcn_units`` with neighbouring row blocks of one camera merged, and neighbouring whole cameras merged
    into one image range (at most three launches for 6 cameras on 4 or 8 ranks)."""
    units = dcn_units(cameras, out_rows, world)
    u0, u1 = unit_block(len(units), world, rank)
    merged: list[list[int]] = []
    for n, r0, r1 in units[u0:u1]:
        if merged and merged[-1][0] == n and merged[-1][3] == r0:
            merged[-1][3] = r1                                    # next row block of the same camera
        else:
            merged.append([n, n + 1, r0, r1])
    pieces: list[list[int]] = []
    for piece in merged:
        whole = piece[2] == 0 and piece[3] == out_rows
        if whole and pieces and pieces[-1][2] == 0 and pieces[-1][3] == out_rows and pieces[-1][1] == piece[0]:
            pieces[-1][1] = piece[1]                              # next whole camera
        else:
            pieces.append(piece)
    return [tuple(int(v) for v in p) for p in pieces]


def dcn_pixel_block(cameras: int, plane: int, world: int, rank: int, tile: int = 128) -> tuple[int, int]:
    """Rank `rank`'s run [p0, p1) of the flattened (camera, row, column) output pixels: the 128-pixel tiles of the
    tensor-core kernel dealt out in contiguous, equally sized blocks, so a rank makes one launch whatever the
    camera count."""
    total = int(cameras) * int(plane)
    t0, t1 = unit_block(-(-total // tile), world, rank)
    return min(t0 * tile, total), min(t1 * tile, total)


def broadcast_value(tensor, src: int = 0, group=None) -> float:
    """Replicate ``tensor`` from ``src`` into every rank's own memory; returns the elapsed milliseconds
    (CUDA events on the current stream for device tensors, wall clock for host tensors)."""
    import torch
    import torch.distributed as dist

    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return 0.0
    if tensor.is_cuda:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(tensor.device)
        dist.barrier(group)
        a.record()
        dist.broadcast(tensor, src=src, group=group)
        b.record()
        torch.cuda.synchronize(tensor.device)
        return float(a.elapsed_time(b))
    t0 = time.perf_counter()
    dist.broadcast(tensor, src=src, group=group)
    return (time.perf_counter() - t0) * 1e3


def sharded_msda(value, locations, weights, spatial_shapes, *, gather: bool = False,
                 compute: Callable | None = None, group=None, total_queries: int | None = None):
    """Run MSDA on this rank's query block.

    ``value`` is the full (replicated) tensor.  ``locations``/``weights`` are either the FULL ``[B,Q,...]``
    tensors (the default: this rank's block is cut out of them) or, when ``total_queries`` is given, ALREADY this
    rank's block of a global set of ``total_queries`` queries (its length must then equal the block length;
    nothing is sliced).  Returns this rank's block ``[B, q_end-q_begin, H*D]``, or the gathered ``[B,Q,H*D]``
    when ``gather``.  ``compute`` defaults to the CUDA kernel; tests on CPU inject a stand-in.
    """
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    if compute is None:
        from . import ops

        compute = ops.msda_forward
    if total_queries is None:
        total_q = locations.shape[1]
        q0, q1 = query_block(total_q, world, rank)
        loc = locations[:, q0:q1].contiguous()
        att = weights[:, q0:q1].contiguous()
    else:
        total_q = int(total_queries)
        q0, q1 = query_block(total_q, world, rank)
        if locations.shape[1] != q1 - q0 or weights.shape[1] != q1 - q0:
            raise ValueError(f"rank {rank} owns queries [{q0},{q1}) of {total_q}; got a slice of {locations.shape[1]}")
        loc, att = locations, weights
    block = compute(value, loc, att, spatial_shapes)
    if not gather or world == 1:
        return block
    sizes = [query_block(total_q, world, r) for r in range(world)]
    longest = max(e - b for b, e in sizes)
    padded = torch.zeros((block.shape[0], longest, block.shape[2]), dtype=block.dtype, device=block.device)
    padded[:, : block.shape[1]] = block
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    return torch.cat([p[:, : e - b] for p, (b, e) in zip(parts, sizes)], dim=1)


def bind_host_near_gpu(device_index: int) -> list[int] | None:
    """Pin this process to the CPUs NVML reports as closest to GPU ``device_index`` (its NUMA node), so that the
    pinned staging buffers allocated afterwards are placed in that node's memory and the host->device copies of the
    ranks of one node do not all cross the socket interconnect.  Returns the CPU list, or None when NVML or the
    affinity call is unavailable (nothing is changed then).  Only this process's own affinity is touched."""
    import os

    try:
        import pynvml
        import torch

        pynvml.nvmlInit()
        uuid = str(torch.cuda.get_device_properties(device_index).uuid)
        if not uuid.startswith("GPU-"):
            uuid = "GPU-" + uuid
        handle = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(handle, words)
        cpus = [64 * i + b for i, word in enumerate(mask) for b in range(64) if (int(word) >> b) & 1]
        allowed = sorted(set(cpus) & os.sched_getaffinity(0))
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return allowed
    except Exception:
        return None


def head_shard(value, locations, weights, world: int, rank: int):
    """This rank's attention heads of an MSDA call: ``(value[:, :, h0:h1], locations[:, :, h0:h1], weights[:, :,
    h0:h1], (h0, h1))`` as dense arrays (NumPy in, NumPy out; torch in, torch out).

    Heads never share a texel line, a location or an output element, so a rank that holds only its heads runs the
    unchanged kernel on ``H/world`` heads and produces columns ``[h0*D, h1*D)`` of the output -- with NOTHING
    replicated: each rank stores, uploads and reads 1/world of ``value``.  It is the layout a head-wise
    (column-parallel) value / offset / weight projection leaves its results in; query blocks (``query_block``)
    need the whole ``value`` on every rank instead."""
    heads = int(value.shape[2])
    h0, h1 = unit_block(heads, world, rank)
    dense = (lambda t: t.contiguous()) if hasattr(value, "contiguous") else np.ascontiguousarray
    return dense(value[:, :, h0:h1]), dense(locations[:, :, h0:h1]), dense(weights[:, :, h0:h1]), (h0, h1)


def nccl_high_priority_options():
    """``pg_options`` for ``init_process_group("nccl", ...)`` that put NCCL's kernels on high-priority streams."""
    import torch.distributed as dist

    opts = dist.ProcessGroupNCCL.Options()
    opts.is_high_priority_stream = True
    return opts


class _DevicePointer:
    """Lets torch view device memory that the library allocated (``__cuda_array_interface__``)."""

    def __init__(self, ptr: int, shape, typestr: str) -> None:
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False), "version": 2}


class PeerBuffers:
    """One device buffer per rank that every other rank of the node can read with copy-engine peer copies.

    Each rank allocates ``nbytes`` through the library (``gacb_ipc_alloc``), the CUDA IPC handles travel over the
    process group, every rank maps the others' buffers, and ``barrier(stream)`` enqueues the library's bounded
    device-side barrier ("every rank's stream has got here").  ``pull(dst, rank, offset, nbytes, stream)`` is one
    ``cudaMemcpyAsync`` from rank ``rank``'s buffer into this GPU's own memory: NVLink traffic without a kernel.
    ``close()`` unmaps and frees; it is collective (ends with a barrier of the group)."""

    def __init__(self, nbytes: int, device, group=None) -> None:
        import ctypes

        import torch
        import torch.distributed as dist

        from . import native

        self.torch, self.dist, self.native, self.group = torch, dist, native, group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = torch.device(device)
        self.nbytes = int(nbytes)
        lib = native.load()
        self._lib = lib
        with torch.cuda.device(self.device):
            mine = []
            for size in (self.nbytes, 4096):              # payload, then flags (world uint32) + step counter
                ptr, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
                native.check(lib.gacb_ipc_alloc(size, ctypes.byref(ptr), handle), "gacb_ipc_alloc")
                mine.append((int(ptr.value), bytes(handle.raw)))
            self.local_ptr, self.local_flags = mine[0][0], mine[1][0]
            handles = [None] * self.world
            dist.all_gather_object(handles, (mine[0][1], mine[1][1]), group=group)
            self.ptrs, self.flag_ptrs, self._opened = [], [], []
            for r, (payload, flags) in enumerate(handles):
                if r == self.rank:
                    self.ptrs.append(self.local_ptr)
                    self.flag_ptrs.append(self.local_flags)
                    continue
                got = []
                for handle in (payload, flags):
                    ptr = ctypes.c_void_p()
                    native.check(lib.gacb_ipc_open(handle, ctypes.byref(ptr)), "gacb_ipc_open")
                    got.append(int(ptr.value))
                    self._opened.append(int(ptr.value))
                self.ptrs.append(got[0])
                self.flag_ptrs.append(got[1])
            self._flag_table = (ctypes.c_void_p * self.world)(*self.flag_ptrs)
            self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        dist.barrier(group)

    def local_tensor(self, shape, dtype):
        """This rank's buffer as a torch tensor (no copy)."""
        torch = self.torch
        typestr = {torch.float32: "<f4", torch.bfloat16: "<i2", torch.uint8: "|u1"}[dtype]
        t = torch.as_tensor(_DevicePointer(self.local_ptr, shape, typestr), device=self.device)
        return t.view(torch.bfloat16) if dtype == torch.bfloat16 else t

    def pull(self, dst, rank: int, offset: int, nbytes: int, stream) -> None:
        if offset < 0 or offset + nbytes > self.nbytes or nbytes > dst.numel() * dst.element_size():
            raise ValueError("peer copy outside the buffers")
        rc = self._lib.gacb_copy_async(dst.data_ptr(), self.ptrs[rank] + offset, nbytes, int(stream.cuda_stream))
        self.native.check(rc, "gacb_copy_async")

    def barrier(self, stream) -> None:
        rc = self._lib.gacb_peer_barrier(self._flag_table, self.local_flags, self.local_flags + 2048, self.world, self.rank,
                                         self.status.data_ptr(), int(stream.cuda_stream))
        self.native.check(rc, "gacb_peer_barrier")

    def check(self) -> None:
        """Raises ``BackendError`` if a device-side barrier gave up waiting for a peer."""
        self.native.check(self._lib.gacb_status_from_word(int(self.status.item())), "peer barrier")

    def close(self) -> None:
        if self._lib is None:
            return
        self.torch.cuda.synchronize(self.device)
        self.dist.barrier(self.group)                     # nobody still reads a buffer that is about to go away
        for ptr in self._opened:
            self._lib.gacb_ipc_close(ptr)
        self.dist.barrier(self.group)
        self._lib.gacb_ipc_free(self.local_ptr)
        self._lib.gacb_ipc_free(self.local_flags)
        self._lib = None


class _NoStream:
    """Stand-in for streams and events on a CPU-only box: everything runs in program order."""

    def wait_event(self, _):
        pass

    def wait_stream(self, _):
        pass

    def synchronize(self):
        pass


class ShardedMsda:
    """Query-sharded MSDA over the ranks of one node when ``value`` does NOT start out replicated.

    Rank r owns queries ``query_block(Q, world, r)`` of every batch entry (locations, weights and output are
    sliced, never replicated) and rows ``[r*Sp, (r+1)*Sp)`` of every batch entry's value slab, ``Sp =
    ceil(S / world)`` (the last rank's rows past S are padding).  One step, batch entry by batch entry:

        host shard b  --h2d stream-->  device shard b  --comm stream: all-gather-->  full slab b in this GPU's
        own memory  --compute stream: the MSDA kernel on slab b-->  output block b  --d2h stream-->  host

    so entry b+1 is on the wire while the kernel gathers from entry b.  The all-gather output is rank-major, i.e.
    the first S rows of the ``[world*Sp, H, D]`` buffer ARE the slab in order; the kernel reads only this GPU's
    own memory (no peer loads).  ``replicate="broadcast"`` instead has rank 0 hold the whole value and broadcast
    slab after slab.  ``replicate="peer_copy"`` (device-resident steps only) replaces the collective by copy-engine
    peer copies out of IPC-mapped shard buffers (``PeerBuffers``): no SM is taken from the gather kernel, so the
    copies of slab b+1 really run beside the kernel on slab b; two bounded device-side barriers per step order the
    ranks.  ``value_storage="bfloat16"`` casts the shard on the device before it travels, halving the
    bytes on the wire; the kernel then reads bf16 texels and accumulates in float32.

    The reference runs one device (``src/gac/execution/cuda.py:132-138``): there is no behaviour to match beyond
    "the concatenated blocks equal the single-device output", which holds bit for bit in float32.

    ``compute(value[1,S,H,D], loc[1,q,...], attn[1,q,...], spatial_shapes, out[1,q,H*D])`` defaults to the CUDA
    kernel; CPU tests inject a stand-in and run over gloo.  With NCCL, create the process group with
    high-priority streams (``nccl_high_priority_options()``), or the collective of entry b+1 queues up behind
    the thousands of CTAs of entry b's kernel instead of running beside them.
    """

    def __init__(self, *, batch: int, spatial_shapes, queries: int, heads: int, head_dim: int, points: int,
                 device, value_storage: str = "float32", replicate: str = "all_gather", group=None,
                 compute: Callable | None = None) -> None:
        import torch
        import torch.distributed as dist

        if replicate not in ("all_gather", "broadcast", "peer_copy"):
            raise ValueError("replicate must be 'all_gather', 'broadcast' or 'peer_copy'")
        if value_storage not in ("float32", "bfloat16"):
            raise ValueError("value_storage must be 'float32' or 'bfloat16'")
        self.torch, self.dist, self.group = torch, dist, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = torch.device(device)
        self.shapes = tuple((int(h), int(w)) for h, w in spatial_shapes)
        self.B, self.Q, self.H, self.D, self.P, self.L = batch, queries, heads, head_dim, points, len(self.shapes)
        self.S = sum(h * w for h, w in self.shapes)
        self.rows = -(-self.S // self.world)                    # Sp: value rows per rank and batch entry
        self.s0 = min(self.S, self.rank * self.rows)
        self.s1 = min(self.S, self.s0 + self.rows)
        self.q0, self.q1 = query_block(self.Q, self.world, self.rank)
        self.replicate = replicate
        self.storage = torch.float32 if value_storage == "float32" else torch.bfloat16
        self._compute = compute
        cuda = self.device.type == "cuda"
        qc = self.q1 - self.q0
        dev = dict(device=self.device)
        self.peers = None
        if replicate == "peer_copy":
            if not cuda or self.world == 1:
                raise ValueError("replicate='peer_copy' needs CUDA devices and more than one rank")
            # the shard every rank pulls from lives in a buffer the others can map; float32 shards are uploaded
            # straight into it, bf16 shards are cast into it
            item = 4 if self.storage == torch.float32 else 2
            self.peers = PeerBuffers(batch * self.rows * heads * head_dim * item, self.device, group)
            shared = self.peers.local_tensor((batch, self.rows, heads, head_dim), self.storage)
        if self.peers is not None and self.storage == torch.float32:
            self.shard32 = shared
        else:
            self.shard32 = torch.zeros((batch, self.rows, heads, head_dim), dtype=torch.float32, **dev)
        if self.storage == torch.float32:
            self.shard = self.shard32
        else:
            self.shard = shared if self.peers is not None else torch.zeros_like(self.shard32, dtype=self.storage)
        self.slabs = torch.zeros((batch, self.world * self.rows, heads, head_dim), dtype=self.storage, **dev)
        self.loc = torch.empty((batch, qc, heads, self.L, points, 2), dtype=torch.float32, **dev)
        self.attn = torch.empty((batch, qc, heads, self.L, points), dtype=torch.float32, **dev)
        self.out = torch.empty((batch, qc, heads * head_dim), dtype=torch.float32, **dev)
        pin = (lambda t: t.pin_memory()) if cuda else (lambda t: t)
        self.host = {"value_shard": pin(torch.zeros((batch, self.rows, heads, head_dim), dtype=torch.float32)),
                     "sampling_locations": pin(torch.empty(self.loc.shape, dtype=torch.float32)),
                     "attention_weights": pin(torch.empty(self.attn.shape, dtype=torch.float32)),
                     "output": pin(torch.empty(self.out.shape, dtype=torch.float32))}
        if cuda:
            with torch.cuda.device(self.device):
                # the collectives go first wherever they compete with a gather kernel for SMs: a kernel launched
                # later on a stream of equal priority would wait for the earlier kernel's whole grid
                self.s_comm = torch.cuda.Stream(priority=-1)
                self.s_h2d, self.s_compute, self.s_d2h = (torch.cuda.Stream() for _ in range(3))
        else:
            self.s_h2d = self.s_comm = self.s_compute = self.s_d2h = _NoStream()

    # ---- what moves per step (for the end-to-end byte counts)
    @property
    def h2d_bytes(self) -> int:
        return sum(int(self.host[k].numel()) * 4 for k in ("value_shard", "sampling_locations", "attention_weights"))

    @property
    def d2h_bytes(self) -> int:
        return int(self.host["output"].numel()) * 4

    @property
    def wire_bytes_in(self) -> int:
        """Bytes this rank receives over NVLink per step (all-gather: the other ranks' shards)."""
        item = 4 if self.storage == self.torch.float32 else 2
        slab = self.B * self.rows * self.H * self.D * item
        return slab * (self.world - 1)

    def close(self) -> None:
        """Collective: releases the peer-mapped buffers of ``replicate='peer_copy'`` (a no-op otherwise)."""
        if self.peers is not None:
            self.peers.close()
            self.peers = None

    def load_host(self, value, locations, weights) -> None:
        """Fill the pinned staging buffers with this rank's share of full host arrays (test / bench set-up)."""
        torch = self.torch
        v = torch.as_tensor(value)
        self.host["value_shard"].zero_()
        self.host["value_shard"][:, : self.s1 - self.s0].copy_(v[:, self.s0:self.s1])
        self.host["sampling_locations"].copy_(torch.as_tensor(locations)[:, self.q0:self.q1])
        self.host["attention_weights"].copy_(torch.as_tensor(weights)[:, self.q0:self.q1])

    def upload(self) -> None:
        """Host staging -> device, all at once (for the device-resident timing of ``step_resident``)."""
        self.shard32.copy_(self.host["value_shard"])
        self.loc.copy_(self.host["sampling_locations"])
        self.attn.copy_(self.host["attention_weights"])
        if self.device.type == "cuda":
            self.torch.cuda.synchronize(self.device)

    # ---- pieces of the pipeline
    def _ctx(self, stream):
        if self.device.type == "cuda":
            return self.torch.cuda.stream(stream)
        import contextlib

        return contextlib.nullcontext()

    def _event(self, stream):
        if self.device.type != "cuda":
            return None
        ev = self.torch.cuda.Event()
        ev.record(stream)
        return ev

    def set_broadcast_source(self, value) -> None:
        """``replicate="broadcast"``: rank 0 keeps the whole value in its slab buffer (in storage dtype)."""
        if self.rank == 0:
            self.slabs[:, : self.S].copy_(self.torch.as_tensor(value).to(self.device).to(self.storage))

    def _replicate_entry(self, b: int) -> None:
        """Enqueue on the comm stream: slab b of every rank's own memory <- the ranks' shards (or rank 0's slab)."""
        torch, dist = self.torch, self.dist
        with self._ctx(self.s_comm):
            if self.replicate == "broadcast":
                if self.world > 1:
                    dist.broadcast(self.slabs[b, : self.S], src=0, group=self.group)
                return
            if self.storage != torch.float32 and self.replicate != "peer_copy":
                self._cast_entry(b)
            if self.replicate == "peer_copy":
                # pull every rank's rows of slab b with the copy engines, the neighbours first so that the ranks
                # do not all read from the same GPU at once; this rank's own rows are a local copy
                entry = self.shard[b].numel() * self.shard.element_size()
                for k in range(self.world):
                    r = (self.rank + k) % self.world
                    self.peers.pull(self.slabs[b, r * self.rows:(r + 1) * self.rows], r, b * entry, entry, self.s_comm)
                return
            if self.world > 1:
                dist.all_gather_into_tensor(self.slabs[b], self.shard[b], group=self.group)
            else:
                self.slabs[b].copy_(self.shard[b], non_blocking=True)

    def _cast_entry(self, b: int) -> None:
        """float32 shard b -> storage dtype (bf16), on the comm stream."""
        if self.device.type == "cuda":
            from . import native

            rc = native.load().gacb_cast_f32_to_bf16(self.shard32[b].data_ptr(), self.shard[b].data_ptr(),
                                                     self.shard32[b].numel(), int(self.s_comm.cuda_stream))
            native.check(rc, "gacb_cast_f32_to_bf16")
        else:
            self.shard[b].copy_(self.shard32[b])

    def _peer_prologue(self) -> None:
        """peer_copy: before anybody pulls, every rank's shards of this step must be in place (and every pull of
        the previous step done, before a cast overwrites a shard): two device-side barriers around the casts."""
        with self._ctx(self.s_comm):
            self.peers.barrier(self.s_comm)              # all pulls of the previous step have been enqueued and run
            if self.storage != self.torch.float32:
                for b in range(self.B):
                    self._cast_entry(b)
            self.peers.barrier(self.s_comm)              # all shards of this step are ready

    def _compute_entry(self, b: int) -> None:
        value = self.slabs[b, : self.S].unsqueeze(0)
        loc, attn, out = self.loc[b:b + 1], self.attn[b:b + 1], self.out[b:b + 1]
        if loc.shape[1] == 0:
            return
        if self._compute is not None:
            self._compute(value, loc, attn, self.shapes, out)
            return
        from . import ops

        ops.msda_forward(value, loc, attn, self.shapes, out=out, stream=self.s_compute)

    def step_resident(self) -> None:
        """One step with the shards (or, for ``broadcast``, rank 0's whole value) already on the device:
        replication of entry b+1 overlaps the kernel of entry b.  Returns after enqueueing."""
        self.s_comm.wait_stream(self.s_compute)      # the previous step's kernels still read the slabs
        if self.replicate == "peer_copy":
            self._peer_prologue()
        for b in range(self.B):
            self._replicate_entry(b)
            self.s_compute.wait_event(self._event(self.s_comm))
            self._compute_entry(b)
        self.s_compute.wait_stream(self.s_comm)      # the step ends on the compute stream (and a capture can close)

    def capture_resident(self):
        """The device-resident step as ONE CUDA graph (collectives included), returned as a callable that replays
        it on the compute stream.  A step is six collectives and six kernel launches issued from Python; at eight
        GPUs each kernel is a few tens of microseconds, so launched one by one the step is paced by the host
        (about 0.1 ms per batch entry), not by NVLink or the kernel.  Every rank must capture and replay in step.
        Returns ``None`` when the capture fails (the caller keeps calling ``step_resident``)."""
        if self.device.type != "cuda":
            return None
        torch = self.torch
        try:
            for _ in range(2):
                self.step_resident()                 # warm: NCCL channels, kernel attributes
            torch.cuda.synchronize(self.device)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=self.s_compute, capture_error_mode="thread_local"):
                self.step_resident()
            torch.cuda.synchronize(self.device)
        except Exception:
            torch.cuda.synchronize(self.device)
            return None
        self._resident_graph = graph

        def replay():
            with torch.cuda.stream(self.s_compute):
                graph.replay()

        return replay

    def step(self):
        """One end-to-end step from the pinned host buffers ``self.host[...]`` to ``self.host['output']``
        (a torch tensor; valid until the next step).  Waits for the step to finish."""
        h = self.host
        self.s_h2d.wait_stream(self.s_comm)          # shard buffers are free once the previous gathers are done
        self.s_h2d.wait_stream(self.s_compute)
        self.s_comm.wait_stream(self.s_compute)
        if self.replicate == "peer_copy":
            raise NotImplementedError("the host-buffer step uses replicate='all_gather'; peer_copy is the "
                                      "device-resident form (step_resident)")
        for b in range(self.B):
            with self._ctx(self.s_h2d):
                self.shard32[b].copy_(h["value_shard"][b], non_blocking=True)
                self.loc[b].copy_(h["sampling_locations"][b], non_blocking=True)
                self.attn[b].copy_(h["attention_weights"][b], non_blocking=True)
            self.s_comm.wait_event(self._event(self.s_h2d))
            self._replicate_entry(b)
            self.s_compute.wait_event(self._event(self.s_comm))
            self.s_compute.wait_event(self._event(self.s_h2d))
            self._compute_entry(b)
            self.s_d2h.wait_event(self._event(self.s_compute))
            with self._ctx(self.s_d2h):
                h["output"][b].copy_(self.out[b], non_blocking=True)
        self.s_d2h.synchronize()
        return h["output"]
