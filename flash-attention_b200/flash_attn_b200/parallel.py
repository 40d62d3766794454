"""Multi-GPU use of the attention path: shard batch x heads across ranks (no inter-GPU traffic while
the kernels run) and reassemble outputs with one NCCL all-gather over NVLink.

Every (batch, head) pair of attention is independent -- the reference launches one CTA per pair
(csrc/flash_attn/src/fmha_fprop_fp16_kernel.sm80.cu:77) -- so a rank needs only its own shard of
q, k, v.  These helpers are host-side plumbing over torch.distributed (NCCL on GPUs, gloo on CPU
in the tests); they take no part in the single-GPU path.
"""
import torch
import torch.distributed as dist


def shard_range(n_items, world_size, rank):
    """Contiguous [start, end) of `n_items` owned by `rank`; the first n_items % world_size ranks
    get one extra item."""
    if not 0 <= rank < world_size:
        raise ValueError("rank %d outside world of %d" % (rank, world_size))
    base, rem = divmod(n_items, world_size)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def shard_heads(x, world_size, rank, head_axis=-2):
    """Contiguous copy of this rank's heads of x (..., heads, head_dim)."""
    heads = x.shape[head_axis]
    if heads % world_size != 0:
        raise ValueError("heads (%d) must be divisible by the world size (%d)" % (heads, world_size))
    start, end = shard_range(heads, world_size, rank)
    return x.narrow(head_axis, start, end - start).contiguous()


def all_gather_heads(x_shard, group=None, async_op=False):
    """(total, heads / world, d) shards -> (total, heads, d) on every rank.

    Returns the full tensor, or (full tensor, finish) when async_op is set: call finish() to
    wait for the collective and complete the local re-layout."""
    world = dist.get_world_size(group)
    total, hs, d = x_shard.shape
    staging = torch.empty((world * total, hs, d), dtype=x_shard.dtype, device=x_shard.device)
    work = dist.all_gather_into_tensor(staging, x_shard.contiguous(), group=group, async_op=async_op)

    def finish():
        if work is not None:
            work.wait()
        return staging.view(world, total, hs, d).permute(1, 0, 2, 3).reshape(total, world * hs, d)

    if async_op:
        return None, finish
    return finish()


def all_gather_tokens(x_shard, group=None, async_op=False):
    """(tokens_per_rank, heads, d) shards with equal token counts -> (world * tokens, heads, d):
    reassembly for batch-sharded work."""
    world = dist.get_world_size(group)
    out = torch.empty((world * x_shard.shape[0],) + tuple(x_shard.shape[1:]), dtype=x_shard.dtype,
                      device=x_shard.device)
    work = dist.all_gather_into_tensor(out, x_shard.contiguous(), group=group, async_op=async_op)
    if async_op:
        return out, work
    return out
