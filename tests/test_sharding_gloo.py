"""N-sharded column-parallel path on CPU: two gloo ranks, each computes its row range with the
oracle (the GPU kernel is exercised elsewhere), the output slices are all-gathered."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, m, k, n, rank_lora, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle
    from lattice_b200.sharded import ShardedLinear, shard_plan
    from tests._cases import make_case

    case = make_case(3, m, k, n, rank=rank_lora, alpha=2.0 * rank_lora, extra=7)
    n0, n1, off = shard_plan(n, k, world, rank)
    assert off == n0 * (k // 32) * 20
    payload = case["payload"][off: off + (n1 - n0) * (k // 32) * 20]      # the shard is a byte range
    lora = None
    if rank_lora:
        a, b, s = case["lora"]
        lora = (a, b[n0:n1], s)                                           # A replicated, rows of B sharded

    def compute(x):
        return torch.from_numpy(oracle.q4_linear(x.numpy(), payload, m, n1 - n0, k, lora=lora))

    lin = ShardedLinear(n, k, compute)
    assert (lin.n0, lin.n1) == (n0, n1)
    y = lin.forward(torch.from_numpy(case["x"]))
    assert y.shape == (m, n)
    np.save(os.path.join(out_dir, f"y{rank}.npy"), y.numpy())
    if rank == 0:
        np.save(os.path.join(out_dir, "ref.npy"), case["y_ref"])
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("m,k,n,r", [(1, 256, 96, 4), (3, 128, 70, 0)])      # 70 rows: uneven shards of 35
def test_two_rank_sharded_linear_gathers_full_output(tmp_path, m, k, n, r):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), m, k, n, r, str(tmp_path)), nprocs=world, join=True)
    ref = np.load(tmp_path / "ref.npy")
    for rank in range(world):
        y = np.load(tmp_path / f"y{rank}.npy")
        # each shard is the same arithmetic as the matching rows of the full product
        assert np.max(np.abs(y - ref)) < 1e-5


def test_three_rank_uneven_plan():
    from lattice_b200.sharded import shard_plan
    sizes = [shard_plan(100, 64, 3, r) for r in range(3)]
    assert [s[0] for s in sizes] == [0, 33, 66] and sizes[-1][1] == 100


def _topk_worker(rank, world, port, vocab, k, top_k, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle
    from lattice_b200.sharded import ShardedLmHead

    rng = np.random.default_rng(99)
    logits = (rng.integers(-50, 50, vocab).astype(np.float32) * np.float32(0.5))      # many ties across the shards
    logits[[3, vocab // 2, vocab - 1]] = np.nan

    def local_topk(x, kk):
        vals, ids = oracle.topk(logits[head.n0:head.n1], kk)      # stands in for lq4_lm_head_topk on this rank's rows
        return torch.from_numpy(vals), torch.from_numpy(ids.view(np.int32).copy())

    head = ShardedLmHead(vocab, k, local_topk)
    vals, ids = head.topk(torch.zeros(1, k), top_k)
    np.save(os.path.join(out_dir, f"v{rank}.npy"), vals.numpy())
    np.save(os.path.join(out_dir, f"i{rank}.npy"), ids.numpy())
    if rank == 0:
        rv, ri = oracle.topk(logits, top_k)
        np.save(os.path.join(out_dir, "rv.npy"), rv)
        np.save(os.path.join(out_dir, "ri.npy"), ri.astype(np.int64))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("vocab,top_k", [(1000, 8), (37, 50)])      # 37 rows, 50 wanted: sentinels fill the tail
def test_two_rank_sharded_lm_head_topk_is_the_global_topk(tmp_path, vocab, top_k):
    world = 2
    mp.spawn(_topk_worker, args=(world, _free_port(), vocab, 64, top_k, str(tmp_path)), nprocs=world, join=True)
    rv, ri = np.load(tmp_path / "rv.npy"), np.load(tmp_path / "ri.npy")
    for rank in range(world):
        assert np.array_equal(np.load(tmp_path / f"i{rank}.npy"), ri)
        assert np.array_equal(np.load(tmp_path / f"v{rank}.npy"), rv)


def _nccl_host_logic_worker(rank, world, port, m, k, n, out_dir):
    """What lq4_linear_sharded does on the host side, with the oracle as each rank's product and gloo as the
    transport: the id exchange, the tile-row blocks, the rank-major gather and the placement."""
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle
    from lattice_b200 import _lib
    from lattice_b200.sharded import exchange_nccl_id, place_slices_host, row_blocks, shard_plan
    from tests._cases import make_case

    ident = exchange_nccl_id()                      # rank 0 draws it through the library, all ranks hold it
    assert len(ident) == _lib.NCCL_ID_BYTES
    ids = [None] * world
    dist.all_gather_object(ids, ident)
    assert all(i == ids[0] for i in ids)

    case = make_case(3, m, k, n, rank=4, alpha=8.0, extra=9)
    n0, n1, off = shard_plan(n, k, world, rank)
    payload = case["payload"][off: off + (n1 - n0) * (k // 32) * 20]
    a, b, s = case["lora"]
    sizes = [shard_plan(n, k, world, r)[1] - shard_plan(n, k, world, r)[0] for r in range(world)]
    y = np.empty((m, n), np.float32)
    blocks = row_blocks(m, n1 - n0, sm_count=2)     # a tiny "device" so that several blocks appear
    assert blocks[0][0] == 0 and blocks[-1][1] == m and all(b0[1] == b1[0] for b0, b1 in zip(blocks, blocks[1:]))
    for r0, r1 in blocks:
        mine = oracle.q4_linear(case["x"][r0:r1], payload, r1 - r0, n1 - n0, k, lora=(a, b[n0:n1], s))
        parts = [torch.empty((r1 - r0) * sz) for sz in sizes]
        dist.all_gather(parts, torch.from_numpy(mine.reshape(-1)))
        y[r0:r1] = place_slices_host(torch.cat(parts).numpy(), r1 - r0, n, world)
    np.save(os.path.join(out_dir, f"y{rank}.npy"), y)
    if rank == 0:
        np.save(os.path.join(out_dir, "ref.npy"), case["y_ref"])
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("m,k,n", [(600, 64, 70), (3, 128, 96)])      # 35-row slices (not a multiple of four); 600 tokens: 3 row blocks
def test_two_rank_nccl_sharded_host_logic(tmp_path, m, k, n):
    world = 2
    mp.spawn(_nccl_host_logic_worker, args=(world, _free_port(), m, k, n, str(tmp_path)), nprocs=world, join=True)
    ref = np.load(tmp_path / "ref.npy")
    for r in range(world):
        assert np.array_equal(np.load(tmp_path / f"y{r}.npy"), ref)


def test_row_blocks_follow_the_library_rule():
    from lattice_b200.sharded import row_blocks
    assert row_blocks(1, 2176) == [(0, 1)]
    assert row_blocks(256, 8704) == [(0, 256)]
    assert row_blocks(2048, 8704) == [(0, 1024), (1024, 2048)]         # two ranks: 272 tiles, two blocks of one wave
    assert row_blocks(2048, 4352) == [(0, 2048)]                       # four ranks: 136 tiles, one block
    assert row_blocks(2048, 2176) == [(0, 2048)]
    assert row_blocks(2048, 17408)[0] == (0, 512) and len(row_blocks(2048, 17408)) == 4
