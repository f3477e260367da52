"""Sequence-sharded decode over the GPUs of one box (include/mlops_fbla_shard.h): every rank keeps a contiguous run of
whole groups of ONE long sequence as an ordinary FBLA cache; a decode is two local passes of the CUDA library with
one tiny NCCL exchange after each (4 B per row, then 528 B per row). The reference has no multi-GPU path; this is
the natural split of its sum over sub-blocks, which only needs the rows' total mass R to be common to all shards.

    plan = plan_shards(tokens, world)                       # which tokens every rank holds
    shard = encode_shard(k_rank, v_rank, mode, plan[rank])  # k_rank / v_rank: the rank's tokens (+ 1, see plan)
    out = decode(q, shard, group)                           # q: the same [B, Hq, 128] BF16 on every rank
"""
import ctypes
from dataclasses import dataclass

import torch

from . import _C
from .fbla import FBLACache, encode

PARTIAL_STRIDE = 132


class Shard(ctypes.Structure):
    """mlops_fbla_shard"""
    _fields_ = [("group_first", ctypes.c_int), ("group_count", ctypes.c_int), ("windows", ctypes.c_int)]


_lib = _C.lib
_vp = ctypes.c_void_p
_lib.mlops_fbla_shard_mass.restype = ctypes.c_int
_lib.mlops_fbla_shard_mass.argtypes = [ctypes.POINTER(_C.Config), ctypes.POINTER(Shard), _vp, ctypes.POINTER(_C.Cache), _vp, _vp, ctypes.c_size_t, _vp]
_lib.mlops_fbla_shard_partial.restype = ctypes.c_int
_lib.mlops_fbla_shard_partial.argtypes = [ctypes.POINTER(_C.Config), ctypes.POINTER(Shard), _vp, ctypes.POINTER(_C.Cache), _vp, _vp, _vp, ctypes.c_size_t, _vp]
_lib.mlops_fbla_shard_total_mass.restype = ctypes.c_int
_lib.mlops_fbla_shard_total_mass.argtypes = [ctypes.c_int, ctypes.c_int, _vp, _vp, _vp]
_lib.mlops_fbla_shard_combine.restype = ctypes.c_int
_lib.mlops_fbla_shard_combine.argtypes = [ctypes.c_int, _vp, _vp, _vp]


class Link(ctypes.Structure):
    """mlops_fbla_shard_link"""
    _fields_ = [("rank", ctypes.c_int), ("world", ctypes.c_int), ("mailboxes", ctypes.POINTER(ctypes.c_void_p)), ("wait_polls", ctypes.c_uint)]


_lib.mlops_fbla_shard_mailbox_bytes.restype = ctypes.c_size_t
_lib.mlops_fbla_shard_mailbox_bytes.argtypes = [ctypes.c_int, ctypes.c_int]
_lib.mlops_fbla_shard_step.restype = ctypes.c_int
_lib.mlops_fbla_shard_step.argtypes = [ctypes.POINTER(_C.Config), ctypes.POINTER(Shard), ctypes.POINTER(Link), _vp, ctypes.POINTER(_C.Cache), _vp, _vp,
                                       ctypes.c_size_t, _vp]
_lib.mlops_fbla_shard_link_status.restype = ctypes.c_int
_lib.mlops_fbla_shard_link_status.argtypes = [ctypes.POINTER(Link), ctypes.c_int, _vp]


@dataclass
class ShardPlan:
    rank: int
    world: int
    token_first: int   # the rank's tokens [token_first, token_end) of the sequence
    token_end: int
    extra: int         # 1: the rank's cache also takes token `token_end` (the next rank's first), closing its last group
    group_first: int   # local closed groups [group_first, group_first + group_count)
    group_count: int
    windows: int       # bit 0: holds the sequence's sink group, bit 1: holds its open group


def plan_shards(tokens: int, world: int):
    """Splits ceil(tokens / 128) groups as evenly as possible into `world` contiguous runs (the last rank also gets the
    partly filled open group). Every rank gets at least one group; world is reduced if there are fewer groups."""
    groups = (tokens + 127) // 128
    world = max(1, min(world, groups))
    plans, g = [], 0
    for r in range(world):
        n = groups // world + (1 if r < groups % world else 0)
        first, end = g * 128, min(tokens, (g + n) * 128)
        last = r == world - 1
        windows = (1 if r == 0 else 0) | (2 if last else 0)
        gf = 1 if r == 0 else 0
        gc = n - gf - (1 if last else 0)   # the last rank's last group is the open one
        plans.append(ShardPlan(r, world, first, end, 0 if last else 1, gf, max(gc, 0), windows))
        g += n
    return plans


@dataclass
class SequenceShard:
    cache: FBLACache
    plan: ShardPlan
    scratch: torch.Tensor = None
    mass: torch.Tensor = None
    gathered: torch.Tensor = None
    total: torch.Tensor = None
    partial: torch.Tensor = None


def encode_shard(k: torch.Tensor, v: torch.Tensor, mode: str, plan: ShardPlan) -> SequenceShard:
    """k, v [B, Hkv, n, 128]: the rank's tokens token_first .. token_end - 1, followed by token `token_end` when
    plan.extra is 1."""
    n = plan.token_end - plan.token_first + plan.extra
    if k.shape[2] != n:
        raise ValueError(f"rank {plan.rank} needs {n} tokens (its {plan.token_end - plan.token_first} + {plan.extra}), got {k.shape[2]}")
    return SequenceShard(encode(k, v, mode), plan)


def _raise(st, what):
    if st == _C.INVALID_VALUE:
        raise ValueError(_C.last_error())
    if st != _C.OK:
        raise RuntimeError(f"{what} failed: {_C.last_error()}")


def _prepare(q, s: SequenceShard):
    c = s.cache
    B, Hq = q.shape[0], q.shape[1]
    kv_heads = c.meta.shape[1]
    cfg = _C.Config(B, Hq, kv_heads, c.tokens, 0.0, 0.0, c.format, c.capacity, 0, 0, 0, 0, 0)
    rows = B * Hq
    if s.scratch is None:
        n = _lib.mlops_fbla_decode_scratch_bytes(ctypes.byref(cfg))
        if n == 0:
            raise ValueError("invalid FBLA configuration for the shard")
        dev = q.device
        s.scratch = torch.empty(n, dtype=torch.uint8, device=dev)
        s.mass = torch.empty(rows, dtype=torch.float32, device=dev)
        s.gathered = torch.empty(s.plan.world * rows, dtype=torch.float32, device=dev)
        s.total = torch.empty(rows, dtype=torch.float32, device=dev)
        s.partial = torch.empty(rows * PARTIAL_STRIDE, dtype=torch.float32, device=dev)
    cache = _C.Cache(c.coarse.data_ptr(), c.fine.data_ptr(), c.meta.data_ptr(), c.sink_k.data_ptr(), c.sink_v.data_ptr(), c.open_k.data_ptr(),
                     c.open_v.data_ptr(), None)
    sh = Shard(s.plan.group_first, s.plan.group_count, s.plan.windows)
    return cfg, cache, sh, rows


def local_mass(q, s: SequenceShard, scale=0.0, tau=0.0):
    """Pass 1: the shard's coarse pass; returns the rows' local log2 mass (a view of the shard's buffer)."""
    cfg, cache, sh, rows = _prepare(q, s)
    cfg.scale, cfg.tau = scale, tau
    st = _lib.mlops_fbla_shard_mass(ctypes.byref(cfg), ctypes.byref(sh), q.data_ptr(), ctypes.byref(cache), s.mass.data_ptr(), s.scratch.data_ptr(),
                                    s.scratch.numel(), torch.cuda.current_stream(q.device).cuda_stream)
    _raise(st, "mlops_fbla_shard_mass")
    return s.mass


def total_mass(gathered, shards, rows, out):
    st = _lib.mlops_fbla_shard_total_mass(shards, rows, gathered.data_ptr(), out.data_ptr(), torch.cuda.current_stream(out.device).cuda_stream)
    _raise(st, "mlops_fbla_shard_total_mass")
    return out


def local_partial(q, s: SequenceShard, total, scale=0.0, tau=0.0):
    """Pass 2: select with the common mass, refine, and the shard's share of every row."""
    cfg, cache, sh, rows = _prepare(q, s)
    cfg.scale, cfg.tau = scale, tau
    st = _lib.mlops_fbla_shard_partial(ctypes.byref(cfg), ctypes.byref(sh), q.data_ptr(), ctypes.byref(cache), total.data_ptr(), s.partial.data_ptr(),
                                       s.scratch.data_ptr(), s.scratch.numel(), torch.cuda.current_stream(q.device).cuda_stream)
    _raise(st, "mlops_fbla_shard_partial")
    return s.partial


def combine(partial_sum, q):
    out = torch.empty_like(q)
    st = _lib.mlops_fbla_shard_combine(q.shape[0] * q.shape[1], partial_sum.data_ptr(), out.data_ptr(), torch.cuda.current_stream(q.device).cuda_stream)
    _raise(st, "mlops_fbla_shard_combine")
    return out


def exchange_mass(mass, gathered, group=None):
    """Exchange A: every rank's local row masses, concatenated rank-major into `gathered` [world * rows]."""
    import torch.distributed as dist
    dist.all_gather_into_tensor(gathered, mass, group=group)
    return gathered


def exchange_partial(partial, group=None):
    """Exchange B: the rows' shares summed over the ranks, in place."""
    import torch.distributed as dist
    dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=group)
    return partial


def decode(q: torch.Tensor, s: SequenceShard, group=None, *, scale: float = 0.0, tau: float = 0.0) -> torch.Tensor:
    """One decode step of the sharded sequence; call on every rank of `group` with the same q. Returns the full
    output [B, Hq, 128] BF16 on every rank."""
    rows = q.shape[0] * q.shape[1]
    local_mass(q, s, scale, tau)
    if s.plan.world > 1:
        exchange_mass(s.mass, s.gathered, group)                            # exchange A: 4 B per row and rank
        total_mass(s.gathered, s.plan.world, rows, s.total)
    else:
        total_mass(s.mass, 1, rows, s.total)
    local_partial(q, s, s.total, scale, tau)
    if s.plan.world > 1:
        exchange_partial(s.partial, group)                                  # exchange B: 528 B per row
    return combine(s.partial, q)


class GraphedDecode:
    """The same decode step with its three local segments (mass pass; total mass + partial pass; combine) replayed from
    CUDA graphs and the two exchanges launched between them as ordinary NCCL calls (collectives are never captured): at
    a few KB per exchange the step is bound by launches, and the graphs remove most of the host's share. q and the
    shard's buffers must stay where they are; the output tensor is reused by every call."""

    def __init__(self, q: torch.Tensor, s: SequenceShard, group=None, *, scale: float = 0.0, tau: float = 0.0):
        self.q, self.s, self.group, self.world = q, s, group, s.plan.world
        rows = q.shape[0] * q.shape[1]
        decode(q, s, group, scale=scale, tau=tau)  # eagerly once: per-device kernel configuration happens here, not under capture
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self.g_mass = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.g_mass, stream=side):
                local_mass(q, s, scale, tau)
                if self.world == 1:
                    total_mass(s.mass, 1, rows, s.total)
            self.g_partial = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.g_partial, stream=side):
                if self.world > 1:
                    total_mass(s.gathered, self.world, rows, s.total)
                local_partial(q, s, s.total, scale, tau)
            self.g_combine = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.g_combine, stream=side):
                self.out = combine(s.partial, q)
        torch.cuda.current_stream().wait_stream(side)

    def __call__(self) -> torch.Tensor:
        self.g_mass.replay()
        if self.world > 1:
            exchange_mass(self.s.mass, self.s.gathered, self.group)
        self.g_partial.replay()
        if self.world > 1:
            exchange_partial(self.s.partial, self.group)
        self.g_combine.replay()
        return self.out


class LinkedDecode:
    """The sharded decode step with both exchanges done by the GPUs themselves (mlops_fbla_shard_step): every rank stores
    its rows' masses and sums straight into the other ranks' mailboxes over NVLink and polls its own mailbox, with a
    bound, for theirs. No NCCL call is on the step's path, so the whole step -- nine small launches -- is captured in
    ONE CUDA graph and replayed. The mailboxes are torch symmetric memory (peer-mapped; multicast is not used).

        step = LinkedDecode(q, shard, group)      # collective: every rank of `group` constructs it
        out = step()                              # every rank calls it the same number of times

    mailboxes: give the list of the ranks' mailbox base addresses (ints) instead of a group to supply the memory yourself
    (a single process driving one GPU, tests)."""

    def __init__(self, q: torch.Tensor, s: SequenceShard, group=None, *, scale: float = 0.0, tau: float = 0.0, mailboxes=None, rank=None,
                 wait_polls: int = 0, graph: bool = True):
        self.q, self.s = q, s
        rows = q.shape[0] * q.shape[1]
        world = s.plan.world if mailboxes is None else len(mailboxes)
        rank = s.plan.rank if rank is None else rank
        nbytes = _lib.mlops_fbla_shard_mailbox_bytes(world, rows)
        if nbytes == 0:
            raise ValueError(f"no mailbox layout for {world} ranks and {rows} rows")
        self._keep = []
        if mailboxes is None:
            if world > 1:
                import os
                os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer mappings are all this path uses
                import torch.distributed as dist
                import torch.distributed._symmetric_memory as symm
                box = symm.empty(nbytes, dtype=torch.uint8, device=q.device)
                box.zero_()
                torch.cuda.synchronize(q.device)
                handle = symm.rendezvous(box, group if group is not None else dist.group.WORLD)
                mailboxes = [int(p) for p in handle.buffer_ptrs]
                self._keep += [box, handle]
                dist.barrier(group)  # every mailbox is zeroed before anybody's first store can land in it
            else:
                box = torch.zeros(nbytes, dtype=torch.uint8, device=q.device)
                mailboxes = [box.data_ptr()]
                self._keep.append(box)
        self._boxes = (ctypes.c_void_p * world)(*mailboxes)
        self.link = Link(rank, world, ctypes.cast(self._boxes, ctypes.POINTER(ctypes.c_void_p)), wait_polls)
        self.rows = rows
        self.out = torch.empty_like(q)
        self._cfg, self._cache, self._sh, _ = _prepare(q, s)
        self._cfg.scale, self._cfg.tau = scale, tau
        self.graph = None
        self._eager()  # once eagerly: per-device kernel configuration happens here, not under capture
        torch.cuda.synchronize(q.device)
        if graph:
            side = torch.cuda.Stream(q.device)
            side.wait_stream(torch.cuda.current_stream(q.device))
            with torch.cuda.stream(side):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    self._eager()
            torch.cuda.current_stream(q.device).wait_stream(side)
            self.graph = g

    def _eager(self):
        st = _lib.mlops_fbla_shard_step(ctypes.byref(self._cfg), ctypes.byref(self._sh), ctypes.byref(self.link), self.q.data_ptr(),
                                        ctypes.byref(self._cache), self.out.data_ptr(), self.s.scratch.data_ptr(), self.s.scratch.numel(),
                                        torch.cuda.current_stream(self.q.device).cuda_stream)
        _raise(st, "mlops_fbla_shard_step")

    def __call__(self) -> torch.Tensor:
        if self.graph is not None:
            self.graph.replay()
        else:
            self._eager()
        return self.out

    def status(self) -> int:
        """0, or which exchange gave up waiting (1 masses, 2 sums) + 16 * the rank that stayed silent; synchronises."""
        return _lib.mlops_fbla_shard_link_status(ctypes.byref(self.link), self.rows, torch.cuda.current_stream(self.q.device).cuda_stream)
