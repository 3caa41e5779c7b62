"""Two GPUs, one process each, NCCL: the (batch x head) partition of the path with the CUDA kernels, and the
all-gather of the layer output that follows it.  Heads never exchange data while they are computed; the only
collective is the plain `all_gather` AFTER the path (no in-switch reduction, no peer-memory kernel of this
library is involved).  Skipped where fewer than two GPUs are visible."""
import math
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _inputs(B, H, S, D):
    g = torch.Generator().manual_seed(123)
    return tuple(torch.randn(B, H, S, D, generator=g).to(torch.bfloat16) for _ in range(3))


def _worker(rank, world, port, out_dir):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    import quant_flash_attn_b200 as qfa
    B, H, S, D = 2, 5, 384, 128                      # 10 heads over 2 ranks; 5 over 2 (uneven) below
    q, k, v = _inputs(B, H, S, D)
    sm = 1.0 / math.sqrt(D)
    ql, kl, vl = (qfa.head_slice(t, world, rank).to(dev) for t in (q, k, v))
    o = qfa.quant_attention(ql, kl, vl, True, sm)
    qfa.check_kernel_status()
    # device-side timing protocol of the benchmark: events, barrier, max over ranks
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dist.barrier()
    a.record()
    o2 = qfa.quant_attention(ql, kl, vl, True, sm)
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b)], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    assert torch.equal(o, o2) and t.item() > 0
    full = qfa.all_gather_heads(o, B, H)
    assert full.shape == (B, H, S, D) and full.device == dev
    s, e = qfa.shard_bounds(B * H, world, rank)
    assert torch.equal(full.reshape(1, B * H, S, D)[:, s:e], o)
    # uneven slices (3 + 2 heads): padded for the collective, trimmed afterwards
    s5, e5 = qfa.shard_bounds(5, world, rank)
    got = qfa.all_gather_heads(torch.full((1, e5 - s5, 4, 8), float(rank), device=dev), 1, 5)
    assert got.shape == (1, 5, 4, 8) and got[0, :3].eq(0).all() and got[0, 3:].eq(1).all()
    torch.save({"span": (s, e), "o": o.cpu(), "gathered": full.cpu()}, os.path.join(out_dir, f"r{rank}.pt"))
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_partition_and_all_gather(tmp_path):
    import torch.multiprocessing as mp
    import quant_flash_attn_b200 as qfa
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    B, H, S, D = 2, 5, 384, 128
    q, k, v = _inputs(B, H, S, D)
    want = qfa.quant_attention(q.cuda(), k.cuda(), v.cuda(), True, 1.0 / math.sqrt(D)).cpu()
    parts = [torch.load(os.path.join(tmp_path, f"r{r}.pt")) for r in range(world)]
    assert parts[0]["span"][0] == 0 and parts[-1]["span"][1] == B * H
    # a head computed alone on another GPU gives the same bits as inside the full batch
    assert torch.equal(torch.cat([p["o"] for p in parts], dim=1).reshape(B, H, S, D), want)
    for p in parts:
        assert torch.equal(p["gathered"], want)
