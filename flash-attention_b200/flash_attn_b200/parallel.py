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


class _PeerWindow:
    """A device buffer of this rank plus the same buffer of every other rank of the node, mapped into
    this process through CUDA IPC (driver API through ctypes; the buffers come from the framework's
    allocator, so the handle is taken on the base of the allocation and the offset travels with it).
    `addr[r]` is the device address of rank r's buffer, or the window is unusable (`cu is None`): no
    CUDA, a single rank, or an allocator / driver that cannot export the memory."""

    _IPC_LAZY_PEER_ACCESS = 1

    class _Handle(ctypes.Structure):
        _fields_ = [("reserved", ctypes.c_ubyte * 64)]

    def __init__(self, buffer, group):
        self.buffer = buffer
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.cu = None
        self._mapped = [None] * self.world
        self.addr = [0] * self.world
        ok, offset = False, 0
        handle = (ctypes.c_ubyte * 64)()
        cu = None
        if buffer.is_cuda and self.world > 1:
            try:
                cu = ctypes.CDLL("libcuda.so.1")
                base, size = ctypes.c_uint64(), ctypes.c_size_t()
                ptr = ctypes.c_uint64(buffer.data_ptr())
                rc = cu.cuMemGetAddressRange_v2(ctypes.byref(base), ctypes.byref(size), ptr)
                rc = rc or cu.cuIpcGetMemHandle(ctypes.byref(handle), ctypes.c_uint64(base.value))
                ok = rc == 0
                offset = ptr.value - base.value
            except OSError:
                ok = False
        exported = [None] * self.world
        dist.all_gather_object(exported, (ok, bytes(handle), offset), group=group)
        if not (ok and all(e[0] for e in exported)):
            return
        cu.cuIpcOpenMemHandle_v2.argtypes = [ctypes.POINTER(ctypes.c_uint64), self._Handle, ctypes.c_uint]
        cu.cuIpcCloseMemHandle.argtypes = [ctypes.c_uint64]
        cu.cuMemcpyAsync.argtypes = [ctypes.c_uint64, ctypes.c_uint64, ctypes.c_size_t, ctypes.c_void_p]
        self.cu = cu
        opened = True
        for r, (_, raw, off) in enumerate(exported):
            if r == self.rank:
                self.addr[r] = buffer.data_ptr()
                continue
            h = self._Handle()
            ctypes.memmove(ctypes.byref(h), raw, 64)
            mapped = ctypes.c_uint64()
            if cu.cuIpcOpenMemHandle_v2(ctypes.byref(mapped), h, self._IPC_LAZY_PEER_ACCESS) != 0:
                opened = False
                break
            self._mapped[r] = mapped.value
            self.addr[r] = mapped.value + off
        # every rank must use the same route: a rank fills only its own part of the others' buffers
        flags = [None] * self.world
        dist.all_gather_object(flags, opened, group=group)
        if not all(flags):
            self.close()

    def stream_handle(self):
        return ctypes.c_void_p(torch.cuda.current_stream(self.buffer.device).cuda_stream)

    def wait(self):
        """Every rank's buffer is complete after this returns: the copies enqueued on the current
        stream have been delivered (stream synchronisation), on all ranks (barrier of the group)."""
        if self.buffer.is_cuda:
            torch.cuda.current_stream(self.buffer.device).synchronize()
        dist.barrier(group=self.group)

    def close(self):
        if self.cu is not None:
            for r, base in enumerate(self._mapped):
                if base is not None:
                    self.cu.cuIpcCloseMemHandle(ctypes.c_uint64(base))
                    self._mapped[r] = None
        self.cu = None


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

    def __init__(self, shard_shape, dtype, device, group=None):
        world = dist.get_world_size(group)
        self.buffer = torch.empty((world,) + tuple(shard_shape), dtype=dtype, device=device)
        self.shard_bytes = self.buffer[0].numel() * self.buffer.element_size()
        self._win = _PeerWindow(self.buffer, group)

    @property
    def uses_copy_engines(self):
        return self._win.cu is not None

    def gather(self, shard):
        """Enqueue the reassembly of `shard` (this rank's slot) on the current stream."""
        w = self._win
        shard = shard.contiguous()
        if shard.numel() * shard.element_size() != self.shard_bytes:
            raise ValueError("shard size does not match the buffer's slot size")
        if w.cu is None:
            dist.all_gather_into_tensor(self.buffer.view(-1), shard.view(-1), group=w.group)
            return
        stream = w.stream_handle()
        shard.record_stream(torch.cuda.current_stream(self.buffer.device))
        for step in range(w.world):
            r = (w.rank + step) % w.world   # own slot first, then the ranks in ring order
            rc = w.cu.cuMemcpyAsync(w.addr[r] + w.rank * self.shard_bytes, shard.data_ptr(), self.shard_bytes, stream)
            if rc != 0:
                raise RuntimeError("cuMemcpyAsync to rank %d failed with CUDA error %d" % (r, rc))

    def wait(self):
        self._win.wait()

    def close(self):
        self._win.close()


class PeerHeadGather:
    """(total, heads / world, d) shards -> (total, heads, d) on every rank, on the copy engines: the
    head-sharded counterpart of PeerTokenGather.  Rank r writes its heads into columns
    [r * heads / world, (r + 1) * heads / world) of every rank's `buffer` with one asynchronous
    pitched (2-D) device-to-device copy per destination, so the result arrives in its final layout.
    Falls back to `all_gather_heads` without CUDA or IPC."""

    class _Memcpy2D(ctypes.Structure):   # CUDA_MEMCPY2D of the driver API
        _fields_ = [("srcXInBytes", ctypes.c_size_t), ("srcY", ctypes.c_size_t), ("srcMemoryType", ctypes.c_uint),
                    ("srcHost", ctypes.c_void_p), ("srcDevice", ctypes.c_uint64), ("srcArray", ctypes.c_void_p),
                    ("srcPitch", ctypes.c_size_t),
                    ("dstXInBytes", ctypes.c_size_t), ("dstY", ctypes.c_size_t), ("dstMemoryType", ctypes.c_uint),
                    ("dstHost", ctypes.c_void_p), ("dstDevice", ctypes.c_uint64), ("dstArray", ctypes.c_void_p),
                    ("dstPitch", ctypes.c_size_t),
                    ("WidthInBytes", ctypes.c_size_t), ("Height", ctypes.c_size_t)]

    _MEMORYTYPE_UNIFIED = 4

    def __init__(self, total, heads, d, dtype, device, group=None):
        world = dist.get_world_size(group)
        if heads % world != 0:
            raise ValueError("heads (%d) must be divisible by the world size (%d)" % (heads, world))
        self.buffer = torch.empty((total, heads, d), dtype=dtype, device=device)
        self.total, self.heads, self.d = total, heads, d
        self.row_bytes = heads * d * self.buffer.element_size()
        self.shard_row_bytes = self.row_bytes // world
        self._win = _PeerWindow(self.buffer, group)
        if self._win.cu is not None:
            self._win.cu.cuMemcpy2DAsync_v2.argtypes = [ctypes.POINTER(self._Memcpy2D), ctypes.c_void_p]

    @property
    def uses_copy_engines(self):
        return self._win.cu is not None

    def gather(self, shard):
        """Enqueue the reassembly of `shard` (this rank's heads) on the current stream."""
        w = self._win
        shard = shard.contiguous()
        if tuple(shard.shape) != (self.total, self.heads // w.world, self.d):
            raise ValueError("shard shape %s does not match (total, heads / world, d)" % (tuple(shard.shape),))
        if w.cu is None:
            self.buffer.copy_(all_gather_heads(shard, group=w.group))
            return
        stream = w.stream_handle()
        shard.record_stream(torch.cuda.current_stream(self.buffer.device))
        for step in range(w.world):
            r = (w.rank + step) % w.world
            c = self._Memcpy2D()
            c.srcMemoryType = c.dstMemoryType = self._MEMORYTYPE_UNIFIED
            c.srcDevice, c.srcPitch = shard.data_ptr(), self.shard_row_bytes
            c.dstDevice, c.dstPitch = w.addr[r] + w.rank * self.shard_row_bytes, self.row_bytes
            c.WidthInBytes, c.Height = self.shard_row_bytes, self.total
            rc = w.cu.cuMemcpy2DAsync_v2(ctypes.byref(c), stream)
            if rc != 0:
                raise RuntimeError("cuMemcpy2DAsync to rank %d failed with CUDA error %d" % (r, rc))

    def wait(self):
        self._win.wait()

    def close(self):
        self._win.close()
