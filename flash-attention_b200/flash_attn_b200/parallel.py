"""Multi-GPU use of the attention path: shard batch x heads across ranks (no inter-GPU traffic while
the kernels run) and reassemble outputs with one NCCL all-gather over NVLink.

Every (batch, head) pair of attention is independent -- the reference launches one CTA per pair
(csrc/flash_attn/src/fmha_fprop_fp16_kernel.sm80.cu:77) -- so a rank needs only its own shard of
q, k, v.  These helpers are host-side plumbing over torch.distributed (NCCL on GPUs, gloo on CPU
in the tests); they take no part in the single-GPU path.
"""
import ctypes

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


class PeerTokenGather:
    """Reassembly of equal-sized shards on the copy engines instead of a collective kernel.

    Attention kernels occupy every SM with one CTA each; an all-gather kernel running beside them
    takes SMs away, and one held to a few CTAs is too slow once the gathered volume grows with the
    world size.  Here every rank owns a receive buffer of `world` slots, the ranks open each other's
    buffers once through CUDA IPC, and a call writes the local shard into slot `rank` of every
    buffer with one asynchronous device-to-device copy per destination (NVLink peer writes issued
    by the copy engines, ordered on the caller's current stream; no kernel is launched).

    `buffer` (world, *shard_shape) is complete on every rank after `wait()`.  Without CUDA (the CPU
    tests) or when IPC is unavailable, `gather` falls back to `all_gather_into_tensor`.
    """

    _IPC_LAZY_PEER_ACCESS = 1

    def __init__(self, shard_shape, dtype, device, group=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.buffer = torch.empty((self.world,) + tuple(shard_shape), dtype=dtype, device=device)
        self.shard_bytes = self.buffer[0].numel() * self.buffer.element_size()
        self._cu = None
        self._peer_base = [None] * self.world   # mapped base of every rank's allocation
        self._peer_slot0 = [0] * self.world     # device address of slot 0 of every rank's buffer
        ok = False
        handle = (ctypes.c_ubyte * 64)()
        offset = 0
        if self.buffer.is_cuda and self.world > 1:
            try:
                cu = ctypes.CDLL("libcuda.so.1")
                base, size = ctypes.c_uint64(), ctypes.c_size_t()
                ptr = ctypes.c_uint64(self.buffer.data_ptr())
                rc = cu.cuMemGetAddressRange_v2(ctypes.byref(base), ctypes.byref(size), ptr)
                rc = rc or cu.cuIpcGetMemHandle(ctypes.byref(handle), ctypes.c_uint64(base.value))
                if rc == 0:
                    offset = ptr.value - base.value
                    self._cu = cu
                    ok = True
            except OSError:
                ok = False
        exported = [None] * self.world
        dist.all_gather_object(exported, (ok, bytes(handle), offset), group=group)
        if self._cu is not None and all(e[0] for e in exported):
            class _Handle(ctypes.Structure):
                _fields_ = [("reserved", ctypes.c_ubyte * 64)]
            self._cu.cuIpcOpenMemHandle_v2.argtypes = [ctypes.POINTER(ctypes.c_uint64), _Handle, ctypes.c_uint]
            self._cu.cuMemcpyAsync.argtypes = [ctypes.c_uint64, ctypes.c_uint64, ctypes.c_size_t, ctypes.c_void_p]
            self._cu.cuIpcCloseMemHandle.argtypes = [ctypes.c_uint64]
            opened = True
            for r, (_, raw, off) in enumerate(exported):
                if r == self.rank:
                    self._peer_slot0[r] = self.buffer.data_ptr()
                    continue
                h = _Handle()
                ctypes.memmove(ctypes.byref(h), raw, 64)
                mapped = ctypes.c_uint64()
                rc = self._cu.cuIpcOpenMemHandle_v2(ctypes.byref(mapped), h, self._IPC_LAZY_PEER_ACCESS)
                if rc != 0:
                    opened = False
                    break
                self._peer_base[r] = mapped.value
                self._peer_slot0[r] = mapped.value + off
            # all ranks use the same route: the copies of one rank fill only its own slot
            flags = [None] * self.world
            dist.all_gather_object(flags, opened, group=group)
            if not all(flags):
                self.close()
        else:
            self._cu = None
        self.uses_copy_engines = self._cu is not None

    def gather(self, shard):
        """Enqueue the reassembly of `shard` (this rank's slot) on the current stream."""
        shard = shard.contiguous()
        if shard.numel() * shard.element_size() != self.shard_bytes:
            raise ValueError("shard size does not match the buffer's slot size")
        if not self.uses_copy_engines:
            dist.all_gather_into_tensor(self.buffer.view(-1), shard.view(-1), group=self.group)
            return
        stream = ctypes.c_void_p(torch.cuda.current_stream(self.buffer.device).cuda_stream)
        src = ctypes.c_uint64(shard.data_ptr())
        shard.record_stream(torch.cuda.current_stream(self.buffer.device))
        for step in range(self.world):
            r = (self.rank + step) % self.world   # own slot first, then the ranks in ring order
            dst = ctypes.c_uint64(self._peer_slot0[r] + self.rank * self.shard_bytes)
            rc = self._cu.cuMemcpyAsync(dst, src, ctypes.c_size_t(self.shard_bytes), stream)
            if rc != 0:
                raise RuntimeError("cuMemcpyAsync to rank %d failed with CUDA error %d" % (r, rc))

    def wait(self):
        """The buffers of all ranks are complete after this returns (stream synchronisation, then
        a barrier of the group)."""
        if self.buffer.is_cuda:
            torch.cuda.current_stream(self.buffer.device).synchronize()
        dist.barrier(group=self.group)

    def close(self):
        if self._cu is not None:
            for r, base in enumerate(self._peer_base):
                if base is not None:
                    self._cu.cuIpcCloseMemHandle(ctypes.c_uint64(base))
                    self._peer_base[r] = None
        self._cu = None
        self.uses_copy_engines = False
