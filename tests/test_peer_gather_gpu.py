"""Copy-engine reassembly of shards between two GPUs of one node (CUDA IPC + asynchronous peer
copies, no collective kernel): the buffers of both ranks hold every rank's shard afterwards.
Needs two visible GPUs; skipped otherwise."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, ok):
    sys.path.insert(0, os.path.join(ROOT, "flash-attention_b200"))
    from flash_attn_b200 import parallel
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        dev = torch.device("cuda", rank)
        pg = parallel.PeerTokenGather((1000, 4, 64), torch.float16, dev)
        assert pg.uses_copy_engines
        side = torch.cuda.Stream(device=dev)
        for it in range(3):   # the slots are rewritten on every call
            shard = torch.full((1000, 4, 64), float(10 * it + rank + 1), dtype=torch.float16, device=dev)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                pg.gather(shard)
                pg.wait()
            for r in range(world):
                assert torch.all(pg.buffer[r] == float(10 * it + r + 1)), (it, r)
            dist.barrier()   # nobody overwrites a slot that a peer is still checking
        pg.close()
        # head shards arrive in their final (total, heads, d) layout through pitched copies
        g = torch.Generator().manual_seed(5)
        full = torch.randn(777, 8, 64, generator=g).to(torch.bfloat16)
        hg = parallel.PeerHeadGather(777, 8, 64, torch.bfloat16, dev)
        assert hg.uses_copy_engines
        with torch.cuda.stream(side):
            hg.gather(parallel.shard_heads(full, world, rank).to(dev))
            hg.wait()
        assert torch.equal(hg.buffer.cpu(), full)
        dist.barrier()
        hg.close()
        ok[rank] = 1
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_copies_fill_every_ranks_buffer():
    world = 2
    port = 29500 + (os.getpid() % 2000)
    ctx = mp.get_context("spawn")
    ok = ctx.Array("i", [0] * world)
    procs = [ctx.Process(target=_worker, args=(r, world, port, ok)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        assert p.exitcode == 0
    assert list(ok) == [1] * world
