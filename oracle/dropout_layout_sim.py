"""Literal simulation of how the reference kernels hand out dropout decisions -- TEST
INFRASTRUCTURE ONLY (imported by tests/, never by the product).

`oracle/attention_oracle.py:dropout_keep_mask` computes the keep mask from a closed form
(subsequence / counter / slot as functions of batch, head, row, column).  This file does not use
that formula.  It walks the reference's CUDA code the way the hardware would: it enumerates the
threads of one CTA, gives every thread its Philox streams, runs the kernels' loop nests in their
order, lets each stream hand out one 128-bit draw per call, and writes the eight 16-bit
decisions of a draw to the (row, column) positions that thread owns in its score fragment.  A
test then asserts that both routes give the same mask, which pins the closed form (and the CUDA
code derived from it) against the reference source rather than against one derivation.

Reference lines followed (paths inside csrc/flash_attn/src of lw921014/flash-attention):
  * generator: philox.cuh:7-136 (key = seed, counter = (offset / 4, subsequence), 6 rounds with
    a key bump + 1 final round, counter + 1 after every call);
  * 8 x uint16 view of a draw: fmha/utils.h:642-648;
  * streams and subsequences: forward fmha_fprop_kernel_1xN.h:643-656 (two streams per thread,
    subsequences tidx_global and tidx_global + blockDim.x with tidx_global = (b * H + h) *
    blockDim.x * 2 + tidx), backward fmha_dgrad_kernel_1xN_loop.h:669-681 (one stream,
    tidx_global = (b * H + h) * blockDim.x + tidx), the block-sparse kernels alike
    (fmha_block_fprop_kernel_1xN.h:497-503, fmha_block_dgrad_kernel_1xN_loop.h:727-741);
  * order of the calls inside one iteration: fmha/softmax.h:375-414 (forward, streams
    alternate over the 16 x 64 slabs) and :347-373 (backward, one stream);
  * which element of the fragment is which (row, column): fmha/mask.h:41-60 and the write
    `elt_[2 * mi + ii][4 * ni + jj]` of fmha/softmax.h:203-212;
  * loop nests: forward fmha_fprop_kernel_1xN.h:255 (a key block past the end of the keys is not
    entered), :270-272 (causal start row), :365-366 (row tiles, break past the last query),
    :657-670 (key-block loop); backward fmha_dgrad_kernel_1xN_loop.h:140, :187-188, :304-307,
    :683-699; block-sparse forward fmha_block_fprop_kernel_1xN.h:88-117, :205-232, :486-488 with
    fmha_blockmask.h:41-53, backward fmha_block_dgrad_kernel_1xN_loop.h:129-134, :315-321,
    :665-666;
  * tile shapes: forward FMHA_kernel_traits<N, d, 16, 1, 4> (fmha_fprop_fp16_kernel.sm80.cu:89-146),
    backward FMHA_kernel_traits<N, d, 16, 1, 8> (fmha_dgrad_fp16_kernel_loop.sm80.cu:58-101):
    16 query rows per iteration, 4 resp. 8 warps side by side over the N key columns.
"""
import numpy as np

_SA = 0xD2511F53
_SB = 0xCD9E8D57
_KA = 0x9E3779B9
_KB = 0xBB67AE85
_M32 = 0xFFFFFFFF


def _single_round(ctr, key):
    """philox.cuh:121-131 on arrays of uint64 holding 32-bit words; ctr = [x, y, z, w]."""
    x, y, z, w = ctr
    res0 = np.uint64(_SA) * x          # 32 x 32 -> 64, exact in uint64
    res1 = np.uint64(_SB) * z
    return [(res1 >> np.uint64(32)) ^ y ^ np.uint64(key[0]), res1 & np.uint64(_M32),
            (res0 >> np.uint64(32)) ^ w ^ np.uint64(key[1]), res0 & np.uint64(_M32)]


class _Stream:
    """One Philox object per thread (philox.cuh:7-28), vectorised over the threads of a CTA:
    they all make the same number of calls, so the low 64 bits of the counter are one number."""

    def __init__(self, seed, subsequence, offset):
        self.key = (seed & _M32, (seed >> 32) & _M32)
        self.sub = np.asarray(subsequence, dtype=np.uint64)
        self.lo = offset // 4

    def __call__(self):
        lo = self.lo & 0xFFFFFFFFFFFFFFFF
        carry = self.lo >> 64
        sub = self.sub + np.uint64(carry)
        ctr = [np.full_like(self.sub, lo & _M32), np.full_like(self.sub, (lo >> 32) & _M32),
               sub & np.uint64(_M32), sub >> np.uint64(32)]
        k0, k1 = self.key
        for _ in range(6):                       # philox.cuh:35-39
            ctr = _single_round(ctr, (k0, k1))
            k0 = (k0 + _KA) & _M32
            k1 = (k1 + _KB) & _M32
        out = _single_round(ctr, (k0, k1))       # :41
        self.lo += 1                             # incr(), :42
        # utils.h:642-648: eight little-endian uint16
        u16 = []
        for word in out:
            u16.append(word & np.uint64(0xFFFF))
            u16.append(word >> np.uint64(16))
        return u16                               # list of 8 arrays [threads]


def _thread_geometry(threads):
    """mask.h:41-55 with WARPS_M = 1: first row and first column a thread owns in a 16 x
    (16 * warps) slab."""
    tidx = np.arange(threads)
    warp, lane = tidx // 32, tidx % 32
    warp_n = warp          # warp / WARPS_M with WARPS_M = 1
    quad, tid = lane // 4, (lane % 4) * 2
    return tidx, quad, warp_n * 16 + tid


def _scatter(keep, u16, threshold, row0, quad, col_base, ni, n_per_mma_cta, col_offset):
    """softmax.h:389-394: tmp[ii * 4 + jj] decides elt_[mi * 2 + ii][4 * ni + jj], which mask.h:57-60
    places at row = row0 + quad + 8 * ii, column = ni * N_PER_MMA_PER_CTA + col + (jj & 2) * 4 + (jj & 1)."""
    for ii in range(2):
        for jj in range(4):
            rows = row0 + quad + 8 * ii
            cols = col_offset + ni * n_per_mma_cta + col_base + (jj & 2) * 4 + (jj & 1)
            ok = (rows < keep.shape[0]) & (cols < keep.shape[1])
            keep[rows[ok], cols[ok]] = (u16[ii * 4 + jj] <= np.uint64(threshold))[ok]


def simulate_keep_mask(seed, offset, batch_idx, head_idx, heads, seqlen_q, seqlen_k,
                       max_seqlen_q, max_seqlen_k_rounded, threshold, block_n, causal=False,
                       backward=False, blockmask=None):
    """Keep mask (ceil16(seqlen_q), ceil_N(seqlen_k)) uint8 (1 = kept, 255 = never drawn) produced
    by running the reference's loops for one (batch, head).

    seqlen_q / seqlen_k   actual lengths of this sequence (cu_seqlens differences)
    max_seqlen_q          params.seqlen_q before rounding; the kernels see it rounded up to 16
    max_seqlen_k_rounded  params.seqlen_k as the host entry rounds it (a multiple of block_n)
    threshold             params.p_dropout_in_uint16_t
    block_n               Cta_tile_p::N, 128 or 256
    backward              enumerate the backward kernel (256 threads, one stream) instead of the
                          forward kernel (128 threads, two streams)
    blockmask             converted block mask (key blocks, slots): run the block-sparse kernels
    """
    n = block_n
    threads = 256 if backward else 128
    warps_n = threads // 32
    n_per_mma_cta = 16 * warps_n                   # gemm.h:406-408
    mmas_n = n // n_per_mma_cta                    # :411-413
    tidx, quad, col_base = _thread_geometry(threads)
    bh = batch_idx * heads + head_idx
    if backward:
        streams = [_Stream(seed, bh * threads + tidx, offset)]
    else:
        tg = bh * threads * 2 + tidx
        streams = [_Stream(seed, tg, offset), _Stream(seed, tg + threads, offset)]

    sq_param = (max_seqlen_q + 15) // 16 * 16
    steps_total = (sq_param + 15) // 16
    rows_out = (seqlen_q + 15) // 16 * 16
    cols_out = (seqlen_k + n - 1) // n * n
    keep = np.full((rows_out, cols_out), 255, dtype=np.uint8)

    def draw(row0, loop_step_idx):
        col_offset = loop_step_idx * n
        if backward:                                # softmax.h:347-373
            for ni in range(mmas_n):
                _scatter(keep, streams[0](), threshold, row0, quad, col_base, ni, n_per_mma_cta, col_offset)
        else:                                       # softmax.h:375-414
            for ni in range(0, mmas_n, 2):
                _scatter(keep, streams[0](), threshold, row0, quad, col_base, ni, n_per_mma_cta, col_offset)
                _scatter(keep, streams[1](), threshold, row0, quad, col_base, ni + 1, n_per_mma_cta, col_offset)

    if max_seqlen_k_rounded == n:
        loop_steps = [0]
    else:
        loop_steps = range((max_seqlen_k_rounded + n - 1) // n)
    for loop_step_idx in loop_steps:
        if seqlen_k <= loop_step_idx * n:           # stop_early
            continue
        if blockmask is None:
            begin = loop_step_idx * n // 16 if causal else 0
            steps = steps_total - begin
            for l in range(steps):
                if (begin + l) * 16 >= seqlen_q:
                    break
                draw((begin + l) * 16, loop_step_idx)
        else:
            row = blockmask[loop_step_idx]
            mask_val = int(row[0])
            if mask_val == -1:
                continue
            block_row_idx = mask_val // 4
            for l in range(steps_total):
                if block_row_idx * 16 >= seqlen_q:
                    break
                mask_val_next = int(row[l + 1]) if l < steps_total - 1 else -1
                draw(block_row_idx * 16, loop_step_idx)
                if mask_val_next == -1:
                    break
                mask_val = mask_val_next
                block_row_idx = mask_val // 4
    return keep
