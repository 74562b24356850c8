"""GPU checks of the N-sharded linear: the placement pass against its host restatement, the one-rank form of
lq4_linear_sharded, and - on a box with at least two GPUs - two ranks gathering over NCCL."""
import ctypes as C
import os
import socket
import sys

import numpy as np
import pytest

import oracle
from lattice_b200 import _lib
from tests._cases import make_case, tol_ratio

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("rows,n_total,world,pad", [(5, 64, 2, 0), (3, 70, 3, 0), (7, 17408, 8, 0), (4, 96, 4, 32),
                                                   (1, 10, 4, 0), (2, 1024, 1, 0)])
def test_placement_pass_matches_host_restatement(rows, n_total, world, pad):
    from lattice_b200.sharded import place_slices_host
    rng = np.random.default_rng(rows * n_total + world)
    g = rng.standard_normal(rows * n_total).astype(np.float32)
    y = torch.full((rows, n_total + pad), float("nan"), device="cuda")
    _lib.check(_lib.lib().lq4_place_slices(dev(g).data_ptr(), y.data_ptr(), n_total + pad, rows, n_total, world,
                                           torch.cuda.current_stream().cuda_stream))
    got = y.cpu().numpy()
    assert np.array_equal(got[:, :n_total], place_slices_host(g, rows, n_total, world))
    assert np.isnan(got[:, n_total:]).all()                      # the pitch padding is not touched


def test_sharded_entry_point_with_one_rank_is_the_plain_linear():
    from lattice_b200 import CudaQ4Backend, Q4WeightBuf
    from lattice_b200.sharded import NcclShardedLinear
    be = CudaQ4Backend(0)
    try:
        case = make_case(2, 3, 1024, 300, rank=16, alpha=32.0, extra=61)
        qw = Q4WeightBuf.from_host_payload(case["payload"], case["n"], case["k"])
        a, b, s = case["lora"]
        ad, bd = dev(a), dev(b)
        lin = NcclShardedLinear(be, qw, case["n"], lora=_lib.LoraDesc(ad.data_ptr(), bd.data_ptr(), 16, s))
        y = lin.forward(dev(case["x"]))
        be.check_device_status()
        assert tol_ratio(y.cpu().numpy(), case["y_ref"]) <= 1.0
        # argument checks happen before any launch
        args = _lib.LinearArgs(0, 0, 1, 10, 64, 0, None, 0, None, None, 0, None, None)
        desc = _lib.ShardDesc(None, 2, 0, 30, y.data_ptr(), 0)
        assert _lib.lib().lq4_linear_sharded(be._ctx, C.byref(args), C.byref(desc), None) == _lib.ERR_SHAPE   # 10 != 15 rows
        desc = _lib.ShardDesc(None, 2, 5, 30, y.data_ptr(), 0)
        assert _lib.lib().lq4_linear_sharded(be._ctx, C.byref(args), C.byref(desc), None) == _lib.ERR_SHAPE   # rank >= world
        qw.free()
    finally:
        be.close()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _rank_worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)      # host transport for the NCCL id only
    from lattice_b200 import CudaQ4Backend, Q4WeightBuf
    from lattice_b200.sharded import NcclShardedLinear, shard_plan
    be = CudaQ4Backend(rank)
    ok = True
    # decode shape, prefill shape with several row blocks, slices that are not a multiple of four columns
    for ci, (m, k, n, r, bf16) in enumerate([(1, 1024, 1024, 16, False), (600, 512, 2048, 8, True), (40, 256, 70, 0, False)]):
        case = make_case(3, m, k, n, rank=r, alpha=2.0 * r, bf16_x=bf16, extra=70 + ci)
        n0, n1, off = shard_plan(n, k, world, rank)
        qw = Q4WeightBuf.from_host_payload(case["payload"][off: off + (n1 - n0) * (k // 32) * 20], n1 - n0, k)
        lora, keep = None, []
        if r:
            a, b, s = case["lora"]
            ad, bd = torch.from_numpy(a).cuda(), torch.from_numpy(np.ascontiguousarray(b[n0:n1])).cuda()
            keep = [ad, bd]
            lora = _lib.LoraDesc(ad.data_ptr(), bd.data_ptr(), r, s)
        lin = NcclShardedLinear(be, qw, n, lora=lora)
        x = torch.from_numpy(case["x"]).cuda()
        x = x.to(torch.bfloat16) if bf16 else x
        for _ in range(2):                           # twice: the staging buffers and events are reused
            y = lin.forward(x)
        torch.cuda.synchronize()
        be.check_device_status()
        ratio = tol_ratio(y.cpu().numpy(), case["y_ref"])
        ok = ok and ratio <= 1.0 and bool(torch.isfinite(y).all())
        lin.close()
        qw.free()
    open(os.path.join(out_dir, f"ok{rank}"), "w").write("1" if ok else "0")
    dist.barrier()
    be.close()
    dist.destroy_process_group()


def test_two_ranks_gather_over_nccl(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs on the box")
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_rank_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert (tmp_path / f"ok{r}").read_text() == "1"
