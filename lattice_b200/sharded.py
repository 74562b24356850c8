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


def exchange_nccl_id(group: Optional[dist.ProcessGroup] = None) -> bytes:
    """Rank 0 draws an NCCL unique id through the library and every rank of `group` receives its 128 bytes
    (over whatever backend the group runs on: the id is host data)."""
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    box: List[Optional[bytes]] = [None]
    if rank == 0:
        buf = (C.c_uint8 * _lib.NCCL_ID_BYTES)()
        _lib.check(_lib.lib().lq4_nccl_unique_id(buf))
        box[0] = bytes(buf)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
    assert box[0] is not None and len(box[0]) == _lib.NCCL_ID_BYTES
    return box[0]


def row_blocks(m: int, n_local: int, sm_count: int = 148) -> List[Tuple[int, int]]:
    """The tile-row blocks ``lq4_linear_sharded`` pipelines (row ranges ``[r0, r1)``): as many blocks as keep
    each block's product at about one wave of 256 x 256 tiles, at most four, in multiples of 256 rows."""
    blocks = 1
    if m > 256:
        tiles = ((n_local + 255) // 256) * ((m + 255) // 256)
        blocks = min(4, max(1, (tiles + sm_count // 2) // sm_count))
    rows_per = ((m + blocks - 1) // blocks + 255) // 256 * 256
    return [(r0, min(m, r0 + rows_per)) for r0 in range(0, m, rows_per)]


def place_slices_host(gathered, rows: int, n_total: int, world: int):
    """Host restatement of the placement pass (``lq4_place_slices``): ``gathered`` is the flat rank-major
    result of an all-gather of ``[rows, n_r]`` slices; returns the row-major ``[rows, n_total]`` array."""
    import numpy as np
    g = np.asarray(gathered, dtype=np.float32).reshape(-1)
    y = np.empty((rows, n_total), np.float32)
    for r in range(world):
        n0, n1 = n_total * r // world, n_total * (r + 1) // world
        y[:, n0:n1] = g[n0 * rows: n1 * rows].reshape(rows, n1 - n0)
    return y


class NcclShardedLinear:
    """One N-sharded Q4 linear through ``lq4_linear_sharded``: this rank's rows of the weight (and of LoRA B) on
    its GPU, the ``[m, n / world]`` slices gathered into a full ``[m, n]`` output on every rank over NCCL.

    ``qw_local`` holds rows ``[n0, n1)`` of the weight (``shard_plan``); ``lora`` is a descriptor whose ``b``
    already points at those rows.  The communicator is created by the library from an id exchanged over
    `group` (any backend), or passed in as a raw ``ncclComm_t`` address."""

    def __init__(self, backend, qw_local, n_total: int, lora=None, group: Optional[dist.ProcessGroup] = None,
                 nccl_comm: Optional[int] = None):
        self.be = backend
        self.qw = qw_local
        self.lora = lora
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.n_total, self.k = n_total, qw_local.k
        self.n0, self.n1, self.byte_offset = shard_plan(n_total, self.k, self.world, self.rank)
        if qw_local.n != self.n1 - self.n0:
            raise ValueError(f"rank {self.rank} must hold rows [{self.n0}, {self.n1}) of the weight, got {qw_local.n} rows")
        self._own_comm = False
        self.comm = nccl_comm
        if self.world > 1 and self.comm is None:
            ident = exchange_nccl_id(group)
            h = C.c_void_p()
            raw = (C.c_uint8 * _lib.NCCL_ID_BYTES).from_buffer_copy(ident)
            _lib.check(_lib.lib().lq4_nccl_comm_create(raw, self.world, self.rank, C.byref(h)))
            self.comm, self._own_comm = h.value, True

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        x = x.contiguous()
        m = x.shape[0]
        y = out if out is not None else torch.empty((m, self.n_total), dtype=torch.float32, device=x.device)
        assert y.is_cuda and y.dtype == torch.float32 and y.shape == (m, self.n_total) and y.stride(1) == 1
        args = _lib.LinearArgs(x.data_ptr(), self.be._dtype_of(x), m, self.qw.n, self.k, self.qw.payload_ptr, None, 0,
                               C.pointer(self.lora) if self.lora is not None else None, None, _lib.PATH_AUTO, None, None)
        desc = _lib.ShardDesc(self.comm, self.world, self.rank, self.n_total, y.data_ptr(), y.stride(0))
        _lib.check(_lib.lib().lq4_linear_sharded(self.be._ctx, C.byref(args), C.byref(desc),
                                                 torch.cuda.current_stream().cuda_stream))
        return y

    def close(self) -> None:
        if self._own_comm and self.comm:
            torch.cuda.synchronize()
            _lib.lib().lq4_nccl_comm_destroy(self.comm)
            self.comm, self._own_comm = None, False


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


class StepBuffer:
    """The buffer a decode step's activations travel through (``lq4_step_buf_create``): ``payload`` is a flat
    f32 device tensor; outputs whose ``y`` is a slice of it can feed later groups of the same
    ``lq4_decode_step`` call, on this GPU and - with a process group - on every rank (each rank creates a buffer
    of the same size, the handles travel over the group, every rank maps the others')."""

    def __init__(self, n_floats: int, group: Optional[dist.ProcessGroup] = None, device: Optional[int] = None):
        L = _lib.lib()
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if self.world > _lib.MAX_PEERS:
            raise ValueError(f"at most {_lib.MAX_PEERS} ranks")
        if device is not None:
            torch.cuda.set_device(device)
        h = C.c_void_p()
        _lib.check(L.lq4_step_buf_create(n_floats, C.byref(h)))
        self._buf = h.value
        self._opened: List[int] = []
        bases = [0] * self.world
        bases[self.rank] = L.lq4_peer_buf_base(self._buf)
        if self.world > 1:
            handle = (C.c_uint8 * _lib.PEER_HANDLE_BYTES)()
            _lib.check(L.lq4_peer_buf_export(self._buf, handle))
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
        self.payload = torch.as_tensor(_DeviceArray(L.lq4_peer_buf_payload(self._buf), (n_floats,), self), device="cuda")

    def close(self) -> None:
        L = _lib.lib()
        if dist.is_initialized() and self.world > 1:
            torch.cuda.synchronize()
            dist.barrier(group=self.group)       # nobody unmaps while a peer may still write
        for p in self._opened:
            L.lq4_peer_buf_close(p)
        self._opened = []
        if self._buf:
            self.payload = None
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
