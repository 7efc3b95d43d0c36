"""Multi-rank host logic on CPU (gloo, world_size 2): every (b,h) owns its state, so ranks take
disjoint batch shards with no data-path collective; the only communication is the barrier and the
max-over-ranks of the elapsed time, exactly what bench.py does under torchrun."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    sys.path[:0] = [str(root), str(root / "ram-net_b200")]
    import ramnet_ops
    g = torch.Generator().manual_seed(0)
    B = 4
    q, k = torch.randn(B, 12, 2, 2, 4, generator=g), torch.randn(B, 12, 2, 2, 4, generator=g)
    v = torch.randn(B, 12, 2, 6, generator=g)
    shard = slice(rank * B // world, (rank + 1) * B // world)
    dist.barrier()
    y, (slot, mass) = ramnet_ops.random_access_memory_attention(k[shard], q[shard], v[shard], embed_num=1, top_k=3,
                                                                impl_backend="torch")
    elapsed = torch.tensor([float(rank + 1)], dtype=torch.float64)
    dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
    gathered = [torch.empty_like(y) for _ in range(world)]
    dist.all_gather(gathered, y)
    if rank == 0:
        full, _ = ramnet_ops.random_access_memory_attention(k, q, v, embed_num=1, top_k=3, impl_backend="torch")
        out.put((float(elapsed.item()), bool(torch.allclose(torch.cat(gathered, 0), full, atol=1e-6))))
    dist.destroy_process_group()


def test_batch_sharding_over_two_gloo_ranks_reproduces_the_single_process_result():
    ctx = mp.get_context("spawn")
    out = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    slowest, same = out.get()
    assert slowest == 2.0 and same
