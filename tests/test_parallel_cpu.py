"""Host-side sharding helpers with two gloo ranks on CPU: head shards gathered back equal the
unsharded tensor, token shards likewise, and shard_range covers every item once."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, ok):
    sys.path.insert(0, os.path.join(ROOT, "flash-attention_b200"))
    from flash_attn_b200 import parallel
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        full = torch.randn(37, 8, 16, generator=g)
        shard = parallel.shard_heads(full, world, rank)
        assert shard.shape == (37, 8 // world, 16) and shard.is_contiguous()
        gathered = parallel.all_gather_heads(shard)
        assert torch.equal(gathered, full)
        _, finish = parallel.all_gather_heads(shard, async_op=True)
        assert torch.equal(finish(), full)
        tok = full[rank * 10:(rank + 1) * 10].contiguous()
        assert torch.equal(parallel.all_gather_tokens(tok), full[:10 * world])
        # the copy-engine reassembly falls back to the collective without CUDA: same result
        pg = parallel.PeerTokenGather(tok.shape, tok.dtype, tok.device)
        assert not pg.uses_copy_engines
        pg.gather(tok)
        pg.wait()
        assert torch.equal(pg.buffer.view(-1, 8, 16), full[:10 * world])
        hg = parallel.PeerHeadGather(37, 8, 16, full.dtype, full.device)
        hg.gather(shard)
        hg.wait()
        assert torch.equal(hg.buffer, full)
        try:
            parallel.shard_heads(torch.zeros(3, 5, 4), world, rank)
            raise AssertionError("expected ValueError")
        except ValueError:
            pass
        ok[rank] = 1
    finally:
        dist.destroy_process_group()


def test_head_and_token_sharding_roundtrip_two_ranks():
    world = 2
    port = 29500 + (os.getpid() % 2000)
    ok = mp.get_context("spawn").Array("i", [0] * world)
    procs = [mp.get_context("spawn").Process(target=_worker, args=(r, world, port, ok)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert list(ok) == [1] * world


@pytest.mark.parametrize("n,world", [(32, 8), (10, 4), (3, 5), (0, 2)])
def test_shard_range_partitions(n, world):
    sys.path.insert(0, os.path.join(ROOT, "flash-attention_b200"))
    from flash_attn_b200 import parallel
    spans = [parallel.shard_range(n, world, r) for r in range(world)]
    assert spans[0][0] == 0 and spans[-1][1] == n
    for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
        assert a1 == b0 and a0 <= a1
    sizes = [e - s for s, e in spans]
    assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        parallel.shard_range(n, world, world)
