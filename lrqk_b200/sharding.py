"""Sharding of a layer's (batch, KV head) units over the GPUs of one node, and the exchange of
the attention outputs between the shards.

Every (batch, query head) selection problem of the LRQK path is independent; the host K|V store
is shared by the G query heads of a KV head, so the unit of ownership is a (batch, KV head) pair.
``plan_shards`` cuts the units into one contiguous, equally sized run per rank.  Each rank then
runs the whole per-layer step for its units only; the output projection that follows needs the
attention rows of ALL heads, which ``HeadExchange`` delivers: the epilogue of the attention kernel
stores each finished row into every rank's exchange buffer over NVLink (plain peer stores into
CUDA-IPC mapped memory, one arrival word per source rank), and ``wait`` blocks the stream -- for a
bounded time -- until all ranks' rows of that push have arrived.  The reference is single-GPU and
has no counterpart of this file.

``torch.distributed`` is used for the rendezvous only (exchange of the 64-byte IPC handles);
with the ``gloo`` backend and no GPU the planning and bookkeeping parts still work, which is how
the CPU tests exercise them.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch

from . import _lib


def _parse_cpulist(text: str) -> List[int]:
    cpus: List[int] = []
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.extend(range(int(lo), int(hi or lo) + 1))
    return cpus


def gpu_numa_cpus(device_index: int, sysfs: str = "/sys") -> Optional[List[int]]:
    """CPUs of the NUMA node the GPU's PCIe slot hangs off, from sysfs; None when it cannot be told
    (no sysfs entry, node -1 on single-node machines)."""
    import os
    try:
        props = torch.cuda.get_device_properties(device_index)
        bus = "%04x:%02x:%02x.0" % (props.pci_domain_id, props.pci_bus_id, props.pci_device_id)
        with open(os.path.join(sysfs, "bus/pci/devices", bus, "numa_node")) as f:
            node = int(f.read().strip())
        if node < 0:
            return None
        with open(os.path.join(sysfs, "devices/system/node", f"node{node}", "cpulist")) as f:
            cpus = _parse_cpulist(f.read())
        return cpus or None
    except Exception:
        return None


def bind_host_to_gpu_numa(device_index: int) -> Optional[List[int]]:
    """Restrict this process to the CPUs next to the GPU, so that the page-locked K|V store it
    allocates afterwards (first touch) lands in the memory the GPU's host link reaches without
    crossing sockets -- the rows of every miss travel that path.  Returns the CPUs used, or None if
    the topology is not visible (nothing is changed then).  Call it before the first allocation."""
    import os
    cpus = gpu_numa_cpus(device_index)
    if not cpus:
        return None
    try:
        allowed = sorted(set(cpus) & set(os.sched_getaffinity(0)))
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return allowed
    except Exception:
        return None


@dataclass(frozen=True)
class Shard:
    """The units [unit_begin, unit_end) of the row-major (batch, KV head) grid owned by a rank."""
    rank: int
    unit_begin: int
    unit_end: int
    bsz: int        # batch entries the shard spans
    kv_heads: int   # KV heads per spanned batch entry
    b0: int         # first batch entry
    h0: int         # first KV head

    @property
    def units(self) -> int:
        return self.unit_end - self.unit_begin


def plan_shards(bsz: int, kv_heads: int, world: int) -> List[Shard]:
    """Equal contiguous shards of the B x Hkv unit grid.

    KV heads are split first (every rank keeps all batch entries); when there are more ranks than
    KV heads the batch is split too, so that a shard is ``bsz/b_parts`` batch entries by
    ``kv_heads/h_parts`` heads.  Raises ValueError when the grid does not divide evenly."""
    if world < 1 or bsz < 1 or kv_heads < 1:
        raise ValueError("bsz, kv_heads and world must be positive")
    if kv_heads % world == 0:
        h_parts, b_parts = world, 1
    elif world % kv_heads == 0 and bsz % (world // kv_heads) == 0:
        h_parts, b_parts = kv_heads, world // kv_heads
    else:
        raise ValueError(f"{bsz} x {kv_heads} (batch x KV heads) does not shard evenly over {world} ranks")
    hb, bb = kv_heads // h_parts, bsz // b_parts
    shards = []
    for rank in range(world):
        bp, hp = divmod(rank, h_parts)
        shards.append(Shard(rank=rank, unit_begin=rank * hb * bb, unit_end=(rank + 1) * hb * bb,
                            bsz=bb, kv_heads=hb, b0=bp * bb, h0=hp * hb))
    return shards


def slice_for_shard(x: torch.Tensor, shard: Shard, groups: int = 1) -> torch.Tensor:
    """The part of a [B, H, ...] tensor a shard owns (H = kv_heads * groups of the full model)."""
    return x[shard.b0:shard.b0 + shard.bsz, shard.h0 * groups:(shard.h0 + shard.kv_heads) * groups]


def assemble(gathered: torch.Tensor, shards: Sequence[Shard], bsz: int, q_heads: int, groups: int) -> torch.Tensor:
    """[world, b_local, hq_local, d] rows as the exchange delivers them -> [B, Hq, d] in model order."""
    out = gathered.new_empty((bsz, q_heads) + tuple(gathered.shape[3:]))
    for s in shards:
        slice_for_shard(out, s, groups).copy_(gathered[s.rank])
    return out


class HeadSharding:
    """Runs a whole decoder stack with every layer's (batch, KV head) units split over the ranks of a
    process group: the dense parts of the model are replicated, each rank keeps the LRQK state of its
    units only, and after the attention of a layer every rank receives the rows of all heads --
    through ``HeadExchange`` while decoding (one row per head, latency-bound), through the group's
    all-gather for the prompt pass (the prompt's rows of all heads, bandwidth-bound).

    ``DynamicLRQKCache.shard_heads`` attaches one of these to a cache; the patched attention forward
    then hands the cache full [B, H, L, d] tensors and this object cuts and reassembles them."""

    def __init__(self, group=None, rank: Optional[int] = None, world: Optional[int] = None):
        if rank is None or world is None:
            import torch.distributed as dist
            rank, world = dist.get_rank(group), dist.get_world_size(group)
        self.group, self.rank, self.world = group, rank, world
        self._plans = {}
        self._exchange: Optional[HeadExchange] = None

    def plan(self, bsz: int, kv_heads: int) -> List[Shard]:
        key = (bsz, kv_heads)
        if key not in self._plans:
            self._plans[key] = plan_shards(bsz, kv_heads, self.world)
        return self._plans[key]

    def shard(self, bsz: int, kv_heads: int) -> Shard:
        return self.plan(bsz, kv_heads)[self.rank]

    def local(self, x: torch.Tensor, kv_heads: int) -> torch.Tensor:
        """This rank's part of a [B, H, ...] tensor of query heads (H = kv_heads * groups) or KV heads."""
        return slice_for_shard(x, self.shard(x.shape[0], kv_heads), x.shape[1] // kv_heads)

    def local_rows(self, x: Optional[torch.Tensor], kv_heads: int) -> Optional[torch.Tensor]:
        """This rank's batch entries of a per-sequence tensor [B, ...] (a padding mask)."""
        if x is None:
            return None
        s = self.shard(x.shape[0], kv_heads)
        return x[s.b0:s.b0 + s.bsz]

    def _assemble(self, gathered: torch.Tensor, bsz: int, kv_heads: int, q_heads: int) -> torch.Tensor:
        """[world, b_local, hq_local, ...] -> [B, Hq, ...] in model order."""
        plan = self.plan(bsz, kv_heads)
        if plan[0].bsz == bsz:                                  # only heads are split: one permuting copy
            order = (1, 0, 2) + tuple(range(3, gathered.dim()))
            return gathered.permute(*order).reshape((bsz, q_heads) + tuple(gathered.shape[3:]))
        return assemble(gathered, plan, bsz, q_heads, q_heads // kv_heads)

    def gather_prompt(self, out_local: torch.Tensor, bsz: int, kv_heads: int, q_heads: int) -> torch.Tensor:
        """All ranks' prompt attention rows: [b_local, L, hq_local, d] -> [B, L, Hq, d]."""
        import torch.distributed as dist
        out_local = out_local.contiguous()
        gathered = out_local.new_empty((self.world,) + tuple(out_local.shape))
        dist.all_gather_into_tensor(gathered.view((-1,) + tuple(out_local.shape[1:])), out_local, group=self.group)
        plan = self.plan(bsz, kv_heads)
        seq_len, d = out_local.shape[1], out_local.shape[3]
        if plan[0].bsz == bsz:                                  # only heads are split: one permuting copy
            return gathered.permute(1, 2, 0, 3, 4).reshape(bsz, seq_len, q_heads, d)
        out = out_local.new_empty((bsz, seq_len, q_heads, d))
        g = q_heads // kv_heads
        for s in plan:
            out[s.b0:s.b0 + s.bsz, :, s.h0 * g:(s.h0 + s.kv_heads) * g].copy_(gathered[s.rank])
        return out

    def exchange(self, heads_per_rank: int, head_dim: int, dtype: torch.dtype) -> HeadExchange:
        """The exchange buffers of the decode steps (created collectively at the first step; every
        layer uses the same ones, a push being waited for before the next layer pushes)."""
        ex = self._exchange
        if ex is None:
            ex = self._exchange = HeadExchange(heads_per_rank, head_dim, dtype, group=self.group)
        elif (ex.heads_per_rank, ex.head_dim, ex.dtype) != (heads_per_rank, head_dim, dtype):
            raise ValueError("the layers of one cache must share head count, head size and dtype")
        return ex

    def gather_step(self, bsz: int, kv_heads: int, q_heads: int) -> torch.Tensor:
        """The rows of all heads [B, Hq, d] of this layer's push (the wait was enqueued with the step; it is
        enqueued here if the push came from the stage-by-stage path)."""
        ex = self._exchange
        rows = ex.rows()
        s = self.shard(bsz, kv_heads)
        return self._assemble(rows.view(self.world, s.bsz, -1, ex.head_dim), bsz, kv_heads, q_heads)

    def close(self):
        if self._exchange is not None:
            self._exchange.close()
            self._exchange = None


class PushSequence:
    """Sequence numbers of the pushes of one exchange buffer: 1, 2, 3, ...; push ``seq`` uses half
    ``seq & 1`` of the buffer, so a rank may issue push seq + 1 only after it has waited for push
    seq (that is what keeps a fast rank from overwriting rows a slow peer has not read yet)."""

    def __init__(self):
        self.issued = 0
        self.waited = 0

    def next_push(self) -> int:
        if self.issued != self.waited:
            raise RuntimeError("push %d has not been waited for; a second push would overwrite the half "
                               "a peer may still be reading" % self.issued)
        self.issued += 1
        return self.issued

    def next_wait(self) -> int:
        if self.waited >= self.issued:
            raise RuntimeError("nothing has been pushed since the last wait")
        self.waited += 1
        return self.waited


class HeadExchange:
    """Exchange buffers of all ranks, mapped into this process, plus the push/wait bookkeeping."""

    def __init__(self, heads_per_rank: int, head_dim: int, dtype: torch.dtype, group=None,
                 rank: Optional[int] = None, world: Optional[int] = None, local_ptrs: Optional[Sequence[int]] = None):
        """Collective over ``group`` (default process group): every rank creates its buffer and the
        IPC handles are all-gathered.  ``local_ptrs`` (with ``rank`` and ``world``) instead names
        buffers that already live in this process -- several emulated ranks on one device, see
        :meth:`local_group`."""
        from .state import _DTYPES
        self.lib = _lib.lib()
        self.heads_per_rank, self.head_dim, self.dtype = heads_per_rank, head_dim, dtype
        if local_ptrs is not None:
            self.rank, self.world = rank, world
            self.ptrs: List[int] = list(local_ptrs)
            self.own_ptr, self._owns = self.ptrs[rank], False
        else:
            import torch.distributed as dist
            self.rank = dist.get_rank(group) if rank is None else rank
            self.world = dist.get_world_size(group) if world is None else world
            if not 1 <= self.world <= _lib.MAX_PEERS:
                raise ValueError(f"1..{_lib.MAX_PEERS} ranks are supported, got {self.world}")
            nbytes = self.lib.lrqk_peer_buffer_bytes(self.world, heads_per_rank, head_dim, _DTYPES[dtype])
            own, handle = C.c_void_p(), C.create_string_buffer(64)
            _lib.check(self.lib.lrqk_peer_buffer_create(nbytes, C.byref(own), handle), "lrqk_peer_buffer_create")
            self.own_ptr, self._owns = own.value, True
            handles = [None] * self.world
            dist.all_gather_object(handles, handle.raw, group=group)
            self.ptrs = []
            for r in range(self.world):
                if r == self.rank:
                    self.ptrs.append(self.own_ptr)
                else:
                    p = C.c_void_p()
                    _lib.check(self.lib.lrqk_peer_buffer_open(handles[r], C.byref(p)), "lrqk_peer_buffer_open")
                    self.ptrs.append(p.value)
        self.counter = torch.zeros(1, dtype=torch.int32, device="cuda")
        self.status = torch.zeros(1, dtype=torch.int32, device="cuda")
        self.gathered = torch.empty((self.world, heads_per_rank, head_dim), dtype=dtype, device="cuda")
        g = _lib.PeerGroup()
        g.world, g.rank, g.heads_per_rank, g.head_dim, g.dtype = self.world, self.rank, heads_per_rank, head_dim, _DTYPES[dtype]
        for r in range(self.world):
            g.base[r] = self.ptrs[r]
        g.local_counter = self.counter.data_ptr()
        self.c = g
        self.seq = PushSequence()

    @classmethod
    def local_group(cls, world: int, heads_per_rank: int, head_dim: int, dtype: torch.dtype) -> List["HeadExchange"]:
        """``world`` emulated ranks inside this process, all buffers on the current device.  Pushes
        and waits of the emulated ranks must be issued in an order in which every wait finds its
        pushes already enqueued on the same stream (kernels that wait on one another must never
        share a GPU as separate launches)."""
        from .state import _DTYPES
        lib = _lib.lib()
        nbytes = lib.lrqk_peer_buffer_bytes(world, heads_per_rank, head_dim, _DTYPES[dtype])
        ptrs = []
        for _ in range(world):
            p, h = C.c_void_p(), C.create_string_buffer(64)
            _lib.check(lib.lrqk_peer_buffer_create(nbytes, C.byref(p), h), "lrqk_peer_buffer_create")
            ptrs.append(p.value)
        members = [cls(heads_per_rank, head_dim, dtype, rank=r, world=world, local_ptrs=ptrs) for r in range(world)]
        members[0]._local_all = ptrs  # member 0 frees all buffers on close
        return members

    def struct_ptr(self) -> int:
        return C.addressof(self.c)

    def wait(self, copy: bool = True) -> torch.Tensor:
        """Enqueue the bounded wait for the outstanding push; returns [world, heads_per_rank, d]."""
        seq = self.seq.next_wait()
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        out = C.c_void_p(self.gathered.data_ptr()) if copy else None
        _lib.check(self.lib.lrqk_allgather_wait(C.byref(self.c), seq, out, C.c_void_p(self.status.data_ptr()), stream),
                   "lrqk_allgather_wait")
        return self.gathered

    def rows(self) -> torch.Tensor:
        """All ranks' rows of the last push [world, heads_per_rank, d]; enqueues the wait if the push has not
        been waited for yet."""
        return self.gathered if self.seq.waited == self.seq.issued else self.wait()

    def check_status(self) -> None:
        """Synchronising check of the device status word (call it off the hot path)."""
        code = int(self.status.item())
        if code != 0:
            raise _lib.LrqkError(code, "lrqk_allgather_wait", self.lib.lrqk_strerror(code).decode())

    def close(self):
        if getattr(self, "ptrs", None):
            torch.cuda.synchronize()
            if self._owns:
                for r, p in enumerate(self.ptrs):
                    if r != self.rank:
                        self.lib.lrqk_peer_buffer_close(C.c_void_p(p))
                self.lib.lrqk_peer_buffer_destroy(C.c_void_p(self.own_ptr))
            for p in getattr(self, "_local_all", []):
                self.lib.lrqk_peer_buffer_destroy(C.c_void_p(p))
            self.ptrs = None
