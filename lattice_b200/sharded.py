"""Column-parallel N-sharding of one Q4 linear over the ranks of a process group.

Output rows are independent and every row's blocks are contiguous, so rank r of G owns
rows ``[r*n/G, (r+1)*n/G)``: a byte range of the payload (the ``qw_extra_offset``
addressing of the reference's ``dispatch_gemm_q4_at``,
crates/inference/src/forward/metal_qwen35/inner/dispatch.rs:1037-1097) plus the same
rows of LoRA ``B``.  Activations, LoRA ``A`` and the rotation signs are replicated.  The
only exchange step is the all-gather of the output slices.
"""
from __future__ import annotations

import ctypes as C
from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist

from . import _lib


def shard_plan(n: int, k: int, world: int, rank: int) -> Tuple[int, int, int]:
    """(n0, n1, payload byte offset) of `rank`'s row range; validated by the library."""
    n0, n1, off = C.c_uint64(), C.c_uint64(), C.c_uint64()
    _lib.check(_lib.lib().lq4_shard_plan(n, k, world, rank, C.byref(n0), C.byref(n1), C.byref(off)))
    return int(n0.value), int(n1.value), int(off.value)


class ShardedLinear:
    """Runs ``compute(x) -> y_local[m, n1 - n0]`` on this rank and gathers ``y[m, n]`` on every rank."""

    def __init__(self, n: int, k: int, compute: Callable[[torch.Tensor], torch.Tensor],
                 group: Optional[dist.ProcessGroup] = None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.n, self.k = n, k
        self.n0, self.n1, self.byte_offset = shard_plan(n, k, self.world, self.rank)
        self.sizes: List[int] = []
        for r in range(self.world):
            a, b, _ = shard_plan(n, k, self.world, r)
            self.sizes.append(b - a)
        self.compute = compute
        self._gather_buf: Optional[torch.Tensor] = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y_local = self.compute(x)
        m = y_local.shape[0]
        assert y_local.shape[1] == self.n1 - self.n0
        if self.world == 1:
            return y_local
        if len(set(self.sizes)) == 1:
            # equal shards: one all_gather into a [world, m, n/world] buffer, then a strided view
            if self._gather_buf is None or self._gather_buf.shape[0] != self.world * m:
                self._gather_buf = torch.empty((self.world * m, self.sizes[0]), dtype=y_local.dtype, device=y_local.device)
            dist.all_gather_into_tensor(self._gather_buf, y_local.contiguous(), group=self.group)
            if m == 1:
                return self._gather_buf.view(1, self.n)
            return self._gather_buf.view(self.world, m, self.sizes[0]).permute(1, 0, 2).reshape(m, self.n)
        parts = [torch.empty((m, s), dtype=y_local.dtype, device=y_local.device) for s in self.sizes]
        dist.all_gather(parts, y_local.contiguous(), group=self.group)
        return torch.cat(parts, dim=1)


class _DeviceArray:
    """Exposes a raw device address range to torch through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, shape: Tuple[int, ...], owner):
        self.__cuda_array_interface__ = {"shape": shape, "typestr": "<f4", "data": (ptr, False), "version": 2}
        self._owner = owner


class PeerGather:
    """Output buffers for the all-gather that is fused into the decode kernels' epilogue.

    Every rank allocates one peer buffer (``lq4_peer_buf_create``), the 64-byte handles travel over the
    process group, and each rank maps the others' buffers.  ``full`` is this rank's ``[m, n_total]`` f32
    output as a torch tensor: a projection writes its column range of it (``out=full[:, c0:c1]``) with
    ``gather=self.desc`` and the kernel stores the same values into every peer's ``full``.  After
    ``backend.gather_wait(self.desc)`` the columns written by the peers are complete here as well.
    """

    def __init__(self, m: int, n_total: int, group: Optional[dist.ProcessGroup] = None, device: Optional[int] = None):
        L = _lib.lib()
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if self.world > _lib.MAX_PEERS:
            raise ValueError(f"at most {_lib.MAX_PEERS} ranks")
        if device is not None:
            torch.cuda.set_device(device)
        self.m, self.n_total = m, n_total
        h = C.c_void_p()
        _lib.check(L.lq4_peer_buf_create(m * n_total * 4, C.byref(h)))
        self._buf = h.value
        self._opened: List[int] = []
        own_base = L.lq4_peer_buf_base(self._buf)
        handle = (C.c_uint8 * _lib.PEER_HANDLE_BYTES)()
        _lib.check(L.lq4_peer_buf_export(self._buf, handle))
        bases = [0] * self.world
        bases[self.rank] = own_base
        if self.world > 1:
            handles: List[Optional[bytes]] = [None] * self.world
            dist.all_gather_object(handles, bytes(handle), group=group)
            for r in range(self.world):
                if r == self.rank:
                    continue
                raw = (C.c_uint8 * _lib.PEER_HANDLE_BYTES).from_buffer_copy(handles[r])
                p = C.c_void_p()
                _lib.check(L.lq4_peer_buf_open(raw, C.byref(p)))
                self._opened.append(p.value)
                bases[r] = p.value
        self.desc = _lib.GatherDesc(self.world, self.rank, (C.c_void_p * _lib.MAX_PEERS)(*bases))
        self.full = torch.as_tensor(_DeviceArray(L.lq4_peer_buf_payload(self._buf), (m, n_total), self), device="cuda")

    def close(self) -> None:
        L = _lib.lib()
        if dist.is_initialized() and self.world > 1:
            torch.cuda.synchronize()
            dist.barrier(group=self.group)       # nobody unmaps while a peer may still write
        for p in self._opened:
            L.lq4_peer_buf_close(p)
        self._opened = []
        if self._buf:
            self.full = None
            L.lq4_peer_buf_free(self._buf)
            self._buf = None


def merge_topk_candidates(vals: torch.Tensor, ids: torch.Tensor, top_k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """The best ``top_k`` of any number of candidate lists, in the reference's candidate order (higher logit
    first, ties to the lower token id; shaders/qwen35.metal:1697-1703).  ``vals`` f32 and ``ids`` (token ids as
    int64, or int32 holding u32 bit patterns) have the same shape; sentinel slots (-inf, 0xFFFFFFFF) lose to
    every real candidate.  Exact: every shard's list is an exact local top-k, so their union holds the
    global one (the merge-pass argument of shaders/qwen35.metal:1730-1770, across GPUs instead of tiles)."""
    v = vals.reshape(-1).to(torch.float32)
    i = ids.reshape(-1).to(torch.int64) & 0xFFFFFFFF
    by_id = torch.argsort(i, stable=True)
    v, i = v[by_id], i[by_id]
    by_logit = torch.argsort(v, descending=True, stable=True)      # stable: equal logits keep ascending ids
    v, i = v[by_logit][:top_k], i[by_logit][:top_k]
    return v, i


class ShardedLmHead:
    """Vocabulary rows sharded over the ranks (``shard_plan``): every rank selects the exact top-k of its own
    rows on the device (``lq4_lm_head_topk``), the candidates (k pairs per rank, not the logit row) are
    all-gathered, and every rank merges them to the same global top-k.  The exchange is ``world * k * 8`` bytes."""

    def __init__(self, vocab: int, k: int, local_topk: Callable[[torch.Tensor, int], Tuple[torch.Tensor, torch.Tensor]],
                 group: Optional[dist.ProcessGroup] = None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.vocab = vocab
        self.n0, self.n1, self.byte_offset = shard_plan(vocab, k, self.world, self.rank)
        self.local_topk = local_topk              # (x, top_k) -> (logits[top_k], shard-local row ids[top_k])

    def topk(self, x: torch.Tensor, top_k: int) -> Tuple[torch.Tensor, torch.Tensor]:
        vals, ids = self.local_topk(x, top_k)
        ids = ids.to(torch.int64) & 0xFFFFFFFF
        sentinel = ids == 0xFFFFFFFF
        ids = torch.where(sentinel, ids, ids + self.n0)                  # shard-local row -> token id
        if self.world == 1:
            return merge_topk_candidates(vals, ids, top_k)
        # one exchange: [logit bits | token id] as int64 pairs
        mine = torch.stack([vals.to(torch.float32).contiguous().view(torch.int32).to(torch.int64), ids], dim=1).contiguous()
        both = torch.empty((self.world * top_k, 2), dtype=torch.int64, device=mine.device)
        dist.all_gather_into_tensor(both, mine, group=self.group)
        all_vals = both[:, 0].to(torch.int32).view(torch.float32)
        return merge_topk_candidates(all_vals, both[:, 1], top_k)
