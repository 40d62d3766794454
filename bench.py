"""Benchmark of the attention hot path (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--seqlen S]

Workload (default): BERT-base-shaped varlen training attention -- batch 8, 12 heads, head_dim 64,
fp16, max_seqlen 4096, per-sequence lengths uniform in [max/2, max] from a seed, packed with
cu_seqlens, dropout 0.1, non-causal, Q/K/V/dO ~ N(0,1); synthetic data standing in for the
BERT-base attention shapes of the reference's speed-up chart.  One step = `passes_per_step`
forward + backward passes over that batch (so many that the timed region of K steps lasts about a
second and the clock samples fall inside it).  Metric: algorithmic TFLOP/s,
3.5 * 4 * d * heads * sum(s_i^2) per pass.

The printed JSON line follows the driver's contract: `value` is measured with inputs resident in
HBM, `e2e` through the public functional API with pinned host buffers copied in and results
copied out inside the timed region, `roofline` for the dominant kernel (backward main kernel)
against the measured tensor-core peak, `cpu_baseline` = the CPU oracle (standard attention in
fp32) timed on a bounded sample on this host.  With N > 1 (one process per GPU under torchrun)
every rank runs its own batch shard (weak scaling, no data-path collective) and the outputs are
re-assembled on every rank with asynchronous peer copies over NVLink (copy engines, no kernel: an
all-gather kernel would take SMs from attention kernels that want all of them), on a side stream;
`ms_per_step_no_gather` is the same loop without the re-assembly.  The line also
carries `long_context` (batch 2 x 32 heads x 65536, causal, bf16: this rank's 32 / N heads, forward +
backward, with and without the all-gather of the outputs over NVLink) and `causal_lm_d128_S4096`.
"""
import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "flash-attention_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import numpy as np  # noqa: E402
import torch  # noqa: E402

BATCH, HEADS, HEAD_DIM = 8, 12, 64
DROPOUT_P = 0.1
CPU_SAMPLE_HEADS = 4  # heads of the bounded sample the CPU legs run (a pass over all 12 takes ~10 s)
METRIC = "fwd+bwd attention TFLOP/s (algorithmic, 3.5 x forward)"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"tflops": float(d["bf16_tflops"]), "tflops_sustained": float(d["bf16_tflops_sustained"]),
                "hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
    return {"tflops": 1590.0, "tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


def workload_lengths(max_seqlen, seed, batch=BATCH):
    rng = np.random.RandomState(seed)
    return rng.randint(max_seqlen // 2, max_seqlen + 1, size=batch).tolist()


def fwd_flops(lengths, heads=HEADS, d=HEAD_DIM, causal=False):
    return 4.0 * d * heads * sum(float(s) * float(s) for s in lengths) * (0.5 if causal else 1.0)


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons of one GPU while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu_index), "--query-gpu=" + self.FIELDS,
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                smax.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": float(max(smax)) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def cpu_attention_sample(seqlens, heads, d, causal, dropout_p, threads, repeats=1, min_seconds=0.0):
    """fwd+bwd of the reference's standard attention (the oracle's restatement of `attention_ref`,
    fp32, dropout through the framework's own dropout as the reference does) over the sequences
    `seqlens`, one at a time; run `repeats` times after a warm-up pass and then until `min_seconds`
    of timed work have been done; returns (mean seconds per pass over all of them, flops per pass,
    passes timed)."""
    from oracle import attention_oracle as orc
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(0)
    data = []
    for n in seqlens:
        qkv = torch.randn(1, n, 3, heads, d, generator=g, requires_grad=True)
        data.append((qkv, torch.randn(1, n, heads, d, generator=g), torch.ones(1, n, dtype=torch.bool)))

    def one_pass():
        t0 = time.perf_counter()
        for qkv, dout, mask in data:
            qkv.grad = None
            out = orc.attention_ref(qkv, mask, dropout_p, upcast=True, causal=causal)
            out.backward(dout)
        return time.perf_counter() - t0

    one_pass()  # warm-up
    total, n = 0.0, 0
    while n < repeats or (total < min_seconds and n < 400):
        total += one_pass()
        n += 1
    return total / n, 3.5 * fwd_flops(seqlens, heads, d, causal), n


def cpu_sample_lengths(lengths):
    """The bounded sample of the workload the CPU legs run: its longest and its shortest sequence."""
    return [max(lengths), min(lengths)]


def run_reference(args):
    """--impl reference: the reference's CPU implementation of the path (its standard attention,
    restated in oracle/, since the reference tree is not present on the GPU box and its CUDA
    kernels target sm75/sm80 only) on all host threads, on a bounded sample of the workload: the
    longest and the shortest of its sequences, all heads, dropout on."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    lengths = workload_lengths(args.seqlen, args.seed)
    sample = cpu_sample_lengths(lengths)
    times = []
    flops = 0.0
    for i in range(args.warmup + args.steps):
        dt, flops, _ = cpu_attention_sample(sample, CPU_SAMPLE_HEADS, HEAD_DIM, False, DROPOUT_P, threads, repeats=1)
        if i >= args.warmup:
            times.append(dt)
    t = float(np.mean(times))
    value = flops / t / 1e12
    desc = ("sample of the workload: each step = 1 pass over its longest and its shortest sequence (%d and %d "
            "tokens) x %d of the %d heads, dropout %.1f, fp32 standard attention fwd+bwd"
            % (sample[0], sample[1], CPU_SAMPLE_HEADS, HEADS, DROPOUT_P))
    cfg = workload_config(args, lengths)
    cfg["workload"] = cfg["workload"] + " -- CPU arm runs a SAMPLE of it (see cpu_baseline.sample)"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": t * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": cfg,
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(args, lengths):
    return {"workload": "BERT-base varlen attention fwd+bwd: batch %d x %d heads x d %d, fp16, "
                        "max_seqlen %d, lengths U[max/2,max], dropout %.1f, non-causal"
                        % (BATCH, HEADS, HEAD_DIM, args.seqlen, DROPOUT_P),
            "batch_per_gpu": BATCH, "heads": HEADS, "head_dim": HEAD_DIM, "max_seqlen": args.seqlen,
            "total_tokens_per_gpu": int(sum(lengths)), "dropout_p": DROPOUT_P, "causal": False,
            "parallelism": "batch shards, one per GPU; outputs re-assembled on every rank by peer copies",
            "l2": "working set (qkv, dout, out, dqkv, fp32 dq accumulator) exceeds the 126 MB L2"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--seqlen", type=int, default=4096)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--no-long-context", action="store_true",
                    help="skip the head-sharded 65536-token block (for quick runs)")
    ap.add_argument("--passes", type=int, default=0,
                    help="forward+backward passes per step (0 = as many as make K steps last about 1 s)")
    ap.add_argument("--only-extra", default=None, metavar="NAME",
                    help="run just one entry of the extras sweep (e.g. causal_lm_bf16_d128_S4096) and "
                         "print it; for profiler captures of the other configurations")
    ap.add_argument("--kernels-only", action="store_true",
                    help="skip the host-buffer and CPU legs (for profiler runs)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    if args.impl == "reference":
        run_reference(args)
        return

    import torch.distributed as dist
    from flash_attn_b200 import flash_attn_cuda as fc
    from flash_attn_b200 import parallel
    from flash_attn_b200.bert_padding import unpad_input
    from flash_attn_b200.flash_attn_interface import flash_attn_unpadded_qkvpacked_func

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        # Collectives (the head-shard gather of the long-context block) run beside attention kernels
        # that want every SM: keep NCCL's kernels to a few CTAs.
        os.environ.setdefault("NCCL_MAX_CTAS", "4")
        dist.init_process_group("nccl", device_id=dev)

    if args.only_extra:
        print(json.dumps({"extras": extras(fc, dev, measured_peaks(), only=args.only_extra)}), flush=True)
        return

    # ------------------------------------------------------------------ synthetic workload
    lengths = workload_lengths(args.seqlen, args.seed)          # same lengths on every rank
    S = args.seqlen
    g = torch.Generator(device=dev).manual_seed(1000 + rank)    # different data per rank
    padded = torch.randn(BATCH, S, 3 * HEADS * HEAD_DIM, device=dev, dtype=torch.float16, generator=g)
    mask = torch.arange(S, device=dev)[None, :] < torch.tensor(lengths, device=dev)[:, None]
    x_unpad, _, cu, max_s = unpad_input(padded, mask)
    del padded
    qkv = x_unpad.reshape(-1, 3, HEADS, HEAD_DIM).contiguous()
    total = qkv.shape[0]
    dout = torch.randn(total, HEADS, HEAD_DIM, device=dev, dtype=torch.float16, generator=g)
    scale = HEAD_DIM ** -0.5
    q, k, v = qkv[:, 0], qkv[:, 1], qkv[:, 2]
    dqkv = torch.empty_like(qkv)
    gen = torch.cuda.default_generators[local_rank]
    torch.cuda.manual_seed(1234)
    side = torch.cuda.Stream(device=dev)

    # Re-assembly of the outputs of all ranks: every rank writes its shard into the receive buffers of
    # the others with asynchronous peer copies (copy engines over NVLink, no kernel), on a side stream.
    reassembly = parallel.PeerTokenGather((total, HEADS, HEAD_DIM), torch.float16, dev) if world > 1 else None

    def one_pass(gather):
        """forward + backward through the extension-module contract (C ABI), data in HBM."""
        out, lse, seed, offset = fc.fwd(q, k, v, cu, cu, max_s, max_s, DROPOUT_P, scale, False, False, False,
                                        None, return_philox=True)
        if gather:
            # ordered by streams only (no host wait); the copies of pass i may still run during pass i + 1
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                reassembly.gather(out)
        fc.bwd(dout, q, k, v, out, lse, dqkv[:, 0], dqkv[:, 1], dqkv[:, 2], cu, cu, max_s, max_s,
               DROPOUT_P, scale, False, False, None, philox=(seed, offset))
        return out

    state = {"passes": 1}

    def step_resident():
        for _ in range(state["passes"]):
            one_pass(world > 1)
        if world > 1:
            torch.cuda.current_stream().wait_stream(side)   # a step ends when its last shard has been delivered

    def step_no_gather():
        for _ in range(state["passes"]):
            one_pass(False)

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = t.item()
        return ms

    flops_fwd = fwd_flops(lengths)
    flops_step = 3.5 * flops_fwd
    peaks = measured_peaks()

    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.3)  # let the first samples arrive before the timed region starts
    # passes per step: enough that the K timed steps last about a second
    if args.passes > 0:
        state["passes"] = args.passes
    else:
        est = timed(step_resident, 3, 2)
        if world > 1:
            t = torch.tensor([est], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            est = t.item()
        state["passes"] = max(1, min(200, int(math.ceil(1000.0 / (args.steps * est)))))
    passes = state["passes"]
    ms_step = timed(step_resident, args.steps, args.warmup)
    fc.check_device_status(dev)
    value = world * passes * flops_step / (ms_step * 1e-3) / 1e12
    ms_step_no_gather = timed(step_no_gather, args.steps, 1) if world > 1 else None
    if reassembly is not None:
        reassembly.wait()    # no rank unmaps a buffer that a peer is still writing
        reassembly.close()

    # ------------------------------------------------------------------ end to end (host buffers)
    # Every step copies its inputs from pinned host memory, runs forward + backward through the
    # public functional API (autograd) and copies its results (out, dqkv) back to pinned host
    # memory.  Copies and compute of consecutive steps are pipelined over three streams with two
    # sets of buffers, as a serving / training loop that feeds the GPU from host memory would do.
    qkv_host = [qkv.cpu().pin_memory() for _ in range(2)]
    dout_host = [dout.cpu().pin_memory() for _ in range(2)]
    out_host = [torch.empty((total, HEADS, HEAD_DIM), dtype=torch.float16).pin_memory() for _ in range(2)]
    dqkv_host = [torch.empty_like(qkv_host[0]).pin_memory() for _ in range(2)]
    qkv_dev = [torch.empty_like(qkv) for _ in range(2)]
    dout_dev = [torch.empty_like(dout) for _ in range(2)]
    s_h2d, s_d2h = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    ev_in = [torch.cuda.Event() for _ in range(2)]     # inputs of buffer b are on the device
    ev_done = [torch.cuda.Event() for _ in range(2)]   # compute of buffer b finished
    ev_out = [torch.cuda.Event() for _ in range(2)]    # results of buffer b are on the host
    e2e_state = {"i": 0}

    def step_e2e():
        i = e2e_state["i"]
        e2e_state["i"] = i + 1
        bsel = i % 2
        main = torch.cuda.current_stream()
        with torch.cuda.stream(s_h2d):
            if i >= 2:
                s_h2d.wait_event(ev_done[bsel])       # the step that last used these buffers
            qkv_dev[bsel].copy_(qkv_host[bsel], non_blocking=True)
            dout_dev[bsel].copy_(dout_host[bsel], non_blocking=True)
            ev_in[bsel].record(s_h2d)
        main.wait_event(ev_in[bsel])
        x = qkv_dev[bsel].detach().requires_grad_()
        out = flash_attn_unpadded_qkvpacked_func(x, cu, max_s, DROPOUT_P, softmax_scale=scale, causal=False)
        out.backward(dout_dev[bsel])
        ev_done[bsel].record(main)
        with torch.cuda.stream(s_d2h):
            s_d2h.wait_event(ev_done[bsel])
            if i >= 2:
                s_d2h.wait_event(ev_out[bsel])
            out_d, grad_d = out.detach(), x.grad
            out_d.record_stream(s_d2h)
            grad_d.record_stream(s_d2h)
            out_host[bsel].copy_(out_d, non_blocking=True)
            dqkv_host[bsel].copy_(grad_d, non_blocking=True)
            ev_out[bsel].record(s_d2h)

    def timed_e2e(steps, warmup):
        for _ in range(warmup):
            step_e2e()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step_e2e()
        torch.cuda.current_stream().wait_stream(s_d2h)   # the last results must have reached the host
        torch.cuda.current_stream().wait_stream(s_h2d)
        e1.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        if world > 1:
            tt = torch.tensor([ms], device=dev)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            ms = tt.item()
        return ms

    state["passes"] = 1
    ms_e2e = timed_e2e(max(4, args.steps), 4) if not args.kernels_only else float("nan")
    e2e_value = world * flops_step / (ms_e2e * 1e-3) / 1e12
    h2d = qkv_host[0].numel() * 2 + dout_host[0].numel() * 2
    d2h = out_host[0].numel() * 2 + dqkv_host[0].numel() * 2

    # ------------------------------------------------------------------ kernel-level numbers
    out, lse = fc.fwd(q, k, v, cu, cu, max_s, max_s, DROPOUT_P, scale, False, False, False, None)

    def fwd_only():
        fc.fwd(q, k, v, cu, cu, max_s, max_s, DROPOUT_P, scale, False, False, False, None)

    def bwd_main_only():
        fc.bwd(dout, q, k, v, out, lse, dqkv[:, 0], dqkv[:, 1], dqkv[:, 2], cu, cu, max_s, max_s,
               DROPOUT_P, scale, False, False, None, _stage_mask=2)

    def bwd_all():
        fc.bwd(dout, q, k, v, out, lse, dqkv[:, 0], dqkv[:, 1], dqkv[:, 2], cu, cu, max_s, max_s,
               DROPOUT_P, scale, False, False, None)

    ms_fwd = timed(fwd_only, args.steps, 3)
    ms_bwd = timed(bwd_all, args.steps, 3)
    ms_bwd_main = timed(bwd_main_only, args.steps, 3)
    clocks = sampler.stop()
    achieved = 2.5 * flops_fwd / (ms_bwd_main * 1e-3) / 1e12
    roofline = {"bound": "tensor", "kernel": "fa_bwd_kernel (backward main kernel)",
                "achieved": achieved, "peak": peaks["tflops"], "unit": "TFLOP/s",
                "frac": achieved / peaks["tflops"], "peak_source": peaks["source"] + " (burst cuBLAS bf16)",
                # dram__bytes_read.sum + dram__bytes_write.sum of one launch from the ncu capture in
                # profiles/fa_bwd_kernel_bert_varlen_fp16_S4096.txt (default workload only)
                "traffic": 365.7e6 if (args.seqlen == 4096 and args.seed == 0) else None,
                "traffic_unit": "bytes per launch",
                "fwd_kernel": {"achieved": flops_fwd / (ms_fwd * 1e-3) / 1e12,
                               "frac": flops_fwd / (ms_fwd * 1e-3) / 1e12 / peaks["tflops"]}}

    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp16", "data": "synthetic",
        "config": dict(workload_config(args, lengths), passes_per_step=passes),
        "ms_per_pass": ms_step / passes,
        "ms_per_step_no_gather": ms_step_no_gather,
        "pct_of_peak": 100.0 * value / world / peaks["tflops"],
        "fwd_tflops_per_gpu": flops_fwd / (ms_fwd * 1e-3) / 1e12,
        "bwd_tflops_per_gpu": 2.5 * flops_fwd / (ms_bwd * 1e-3) / 1e12,
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": 4 * passes * args.steps,
        "roofline": roofline,
    }

    # free the headline buffers before the other blocks
    del qkv_host, dout_host, out_host, dqkv_host, qkv_dev, dout_dev
    if world == 1 and not args.kernels_only:
        line["causal_lm_d128_S4096"] = causal_lm_block(fc, dev, peaks, 4096, iters=20)
    if not args.kernels_only and not args.no_long_context and HEADS_LONG % world == 0:
        line["long_context"] = long_context_block(fc, parallel, dist, dev, world, rank, peaks,
                                                  iters=20 if world > 1 else 10)
    if rank == 0 and world == 1 and not args.kernels_only:
        threads = os.cpu_count() or 1
        sample = cpu_sample_lengths(lengths)
        dt, fl, n_cpu = cpu_attention_sample(sample, CPU_SAMPLE_HEADS, HEAD_DIM, False, DROPOUT_P, threads,
                                             repeats=1, min_seconds=10.0)
        line["cpu_baseline"] = {
            "value": fl / dt / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
            "sample": "%d passes (about 10 s) over the longest and the shortest sequence of the workload (%d and "
                      "%d tokens) x %d of the %d heads, fp32 standard attention fwd+bwd, dropout %.1f"
                      % (n_cpu, sample[0], sample[1], CPU_SAMPLE_HEADS, HEADS, DROPOUT_P)}
        if not args.no_extras:
            line["extras"] = extras(fc, dev, peaks)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


HEADS_LONG = 32


def _time_passes(fn, iters, warmup=2):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def long_context_block(fc, parallel, dist, dev, world, rank, peaks, iters):
    """Long-context attention sharded by head: batch 2 x 32 heads x 65536 tokens x d 64, causal, bf16,
    dropout 0.  Rank r holds heads [r * 32 / N, (r + 1) * 32 / N); the data of a head does not
    depend on N (seeded per head).  Times this rank's forward + backward with and without the
    re-assembly of the output shards on every rank over NVLink (pitched peer copies on a side stream,
    ordered by streams); the slowest rank's time is reported.  FLOPs count half of the full problem
    (4 d H B S^2 / 2)."""
    B, H, d, S = 2, HEADS_LONG, 64, 65536
    hs = H // world
    h0 = rank * hs

    def head_stack(tag):
        cols = []
        for h in range(h0, h0 + hs):
            gh = torch.Generator(device=dev).manual_seed(9000 + 10 * h + tag)
            cols.append(torch.randn(B * S, d, device=dev, dtype=torch.bfloat16, generator=gh))
        return torch.stack(cols, dim=1).contiguous()

    q, k, v, dout = head_stack(0), head_stack(1), head_stack(2), head_stack(3)
    cu = torch.arange(0, (B + 1) * S, S, dtype=torch.int32, device=dev)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    side = torch.cuda.Stream(device=dev)
    # (B * S, 32, d) on every rank, filled by pitched peer copies on the copy engines
    full = parallel.PeerHeadGather(B * S, H, d, torch.bfloat16, dev) if world > 1 else None

    def one_pass(gather):
        out, lse = fc.fwd(q, k, v, cu, cu, S, S, 0.0, 0.125, False, True, False, None)
        if gather:
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                full.gather(out)
        fc.bwd(dout, q, k, v, out, lse, dq, dk, dv, cu, cu, S, S, 0.0, 0.125, False, True, None)
        if gather:
            torch.cuda.current_stream().wait_stream(side)

    def fwd_only():
        fc.fwd(q, k, v, cu, cu, S, S, 0.0, 0.125, False, True, False, None)

    def slowest(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev)
        dist.barrier()
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    if world > 1:
        dist.barrier()
    ms_fwd = slowest(_time_passes(fwd_only, iters, warmup=1))
    ms_plain = slowest(_time_passes(lambda: one_pass(False), iters, warmup=1))
    ms_gather = slowest(_time_passes(lambda: one_pass(True), iters, warmup=1)) if world > 1 else None
    fc.check_device_status(dev)
    fl = fwd_flops([S] * B, hs, d, causal=True)
    res = {"workload": "batch 2 x 32 heads x 65536 tokens x d 64, causal, bf16, dropout 0; %d heads per GPU" % hs,
           "heads_per_gpu": hs, "iters": iters, "fwd_ms": ms_fwd, "fwd_bwd_ms": ms_plain,
           "fwd_tflops_per_gpu": fl / ms_fwd / 1e9, "fwd_pct_peak": 100 * fl / ms_fwd / 1e9 / peaks["tflops"],
           "fwd_bwd_tflops_per_gpu": 3.5 * fl / ms_plain / 1e9,
           "fwd_bwd_pct_peak": 100 * 3.5 * fl / ms_plain / 1e9 / peaks["tflops"],
           "fwd_bwd_tflops_all_gpus": world * 3.5 * fl / ms_plain / 1e9}
    if ms_gather is not None:
        res["fwd_bwd_ms_with_gather"] = ms_gather
        res["fwd_bwd_tflops_per_gpu_with_gather"] = 3.5 * fl / ms_gather / 1e9
        res["gathered_bytes_per_gpu"] = int(B * S * H * d * 2)
        res["gather"] = "peer copies (copy engines)" if full.uses_copy_engines else "NCCL all-gather"
    if full is not None:
        full.close()
    del q, k, v, dout, dq, dk, dv, full
    return res


def causal_lm_block(fc, dev, peaks, S, iters):
    """Causal LM attention, bf16: batch 16 x 12 heads x d 128 x S tokens, dropout 0 (FLOPs: half of the
    full problem)."""
    B, H, d = 16, 12, 128
    g = torch.Generator(device=dev).manual_seed(11)
    mk = lambda: torch.randn(B * S, H, d, device=dev, dtype=torch.bfloat16, generator=g)
    q, k, v, dout = mk(), mk(), mk(), mk()
    cu = torch.arange(0, (B + 1) * S, S, dtype=torch.int32, device=dev)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    sc = d ** -0.5
    out, lse = fc.fwd(q, k, v, cu, cu, S, S, 0.0, sc, False, True, False, None)
    f = _time_passes(lambda: fc.fwd(q, k, v, cu, cu, S, S, 0.0, sc, False, True, False, None), iters)
    b = _time_passes(lambda: fc.bwd(dout, q, k, v, out, lse, dq, dk, dv, cu, cu, S, S, 0.0, sc, False, True, None),
                     iters)
    fl = fwd_flops([S] * B, H, d, causal=True)
    return {"iters": iters, "fwd_ms": f, "bwd_ms": b, "fwd_tflops": fl / f / 1e9,
            "fwd_pct_peak": 100 * fl / f / 1e9 / peaks["tflops"], "fwd_bwd_tflops": 3.5 * fl / (f + b) / 1e9,
            "fwd_bwd_pct_peak": 100 * 3.5 * fl / (f + b) / 1e9 / peaks["tflops"]}


def extras(fc, dev, peaks, only=None):
    """Sweeps over the other benchmark configurations (20 iterations each after warm-up, kernel time
    only, data resident): reported for context, not part of the headline value.  `only` limits
    the sweep to one named entry."""
    res = {}

    def wanted(name):
        return only is None or only == name

    def time_fwd_bwd(q, k, v, dout, cu, S, p, causal, scale, iters=20):
        out, lse = fc.fwd(q, k, v, cu, cu, S, S, p, scale, False, causal, False, None)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        for _ in range(2):
            fc.fwd(q, k, v, cu, cu, S, S, p, scale, False, causal, False, None)
            fc.bwd(dout, q, k, v, out, lse, dq, dk, dv, cu, cu, S, S, p, scale, False, causal, None)
        torch.cuda.synchronize()
        ev[0].record()
        for _ in range(iters):
            fc.fwd(q, k, v, cu, cu, S, S, p, scale, False, causal, False, None)
        ev[1].record()
        for _ in range(iters):
            fc.bwd(dout, q, k, v, out, lse, dq, dk, dv, cu, cu, S, S, p, scale, False, causal, None)
        ev[2].record()
        torch.cuda.synchronize()
        return ev[0].elapsed_time(ev[1]) / iters, ev[1].elapsed_time(ev[2]) / iters

    def graph_times(q, k, v, dout, cu, S, p, causal, scale, reps=10):
        """GPU time per call without the host in the loop: `reps` forward (then backward) calls of
        the C ABI captured in a CUDA graph and replayed.  Short sequences are otherwise timed at
        the speed of the Python binding (tens of microseconds per call)."""
        import ctypes
        from flash_attn_b200 import _lib
        out, lse = fc.fwd(q, k, v, cu, cu, S, S, p, scale, False, causal, False, None)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        softmax_d = torch.empty_like(lse)
        dims = fc._check_qkv(q, k, v, cu, cu)
        pf = _lib.FwdParams()
        fc._fill_fwd(pf, dims, q, k, v, out, lse, cu, cu, S, S, p, scale, causal, 1234, 0)
        pb = _lib.BwdParams()
        fc._fill_fwd(pb.fwd, dims, q, k, v, out, lse, cu, cu, S, S, p, scale, causal, 1234, 0)
        pb.dout, pb.softmax_d = dout.data_ptr(), softmax_d.data_ptr()
        pb.dq, pb.dk, pb.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
        pb.dq_row_stride, pb.dq_head_stride = dq.stride(0), dq.stride(1)
        pb.dk_row_stride, pb.dk_head_stride = dk.stride(0), dk.stride(1)
        pb.dv_row_stride, pb.dv_head_stride = dv.stride(0), dv.stride(1)
        ws = torch.empty(_lib.lib.fa_bwd_workspace_bytes(dims[1], dims[3], dims[4]), dtype=torch.uint8, device=q.device)
        pb.workspace, pb.workspace_bytes = ws.data_ptr(), ws.numel()
        times = []
        side_stream = torch.cuda.Stream(device=q.device)
        for call, params in ((_lib.lib.fa_fwd, pf), (_lib.lib.fa_bwd, pb)):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side_stream):
                _lib.check(call(ctypes.byref(params), fc._raw_stream()))   # first use outside capture
                torch.cuda.synchronize()
                with torch.cuda.graph(graph, stream=side_stream):
                    for _ in range(reps):
                        _lib.check(call(ctypes.byref(params), fc._raw_stream()))
            graph.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            graph.replay()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1) / reps)
        return times[0], times[1]

    g = torch.Generator(device=dev).manual_seed(5)
    # BERT-base varlen sweep (fp16, dropout 0.1)
    for S in (128, 256, 512, 1024, 2048, 4096):
        if not wanted("bert_varlen_fp16_dropout_S%d" % S):
            continue
        lengths = workload_lengths(S, 0)
        total = sum(lengths)
        cu = torch.tensor(np.concatenate([[0], np.cumsum(lengths)]), dtype=torch.int32, device=dev)
        qkv = torch.randn(total, 3, HEADS, HEAD_DIM, device=dev, dtype=torch.float16, generator=g)
        dout = torch.randn(total, HEADS, HEAD_DIM, device=dev, dtype=torch.float16, generator=g)
        f, b = time_fwd_bwd(qkv[:, 0], qkv[:, 1], qkv[:, 2], dout, cu, S, DROPOUT_P, False, 0.125)
        fl = fwd_flops(lengths)
        entry = {"fwd_ms": f, "bwd_ms": b, "fwd_tflops": fl / f / 1e9, "fwd_bwd_tflops": 3.5 * fl / (f + b) / 1e9,
                 "fwd_bwd_pct_peak": 100 * 3.5 * fl / (f + b) / 1e9 / peaks["tflops"]}
        if S <= 512:
            # short sequences: also the GPU time alone (graph replay), and HBM GB/s from it
            fg, bg = graph_times(qkv[:, 0], qkv[:, 1], qkv[:, 2], dout, cu, S, DROPOUT_P, False, 0.125)
            hd = HEADS * HEAD_DIM
            fwd_bytes = 2 * 3 * total * hd + 2 * total * hd + 4 * BATCH * HEADS * S
            bwd_bytes = 2 * hd * 5 * total + 2 * hd * 3 * total + 8 * BATCH * HEADS * S
            entry["fwd_gpu_ms"], entry["bwd_gpu_ms"] = fg, bg
            entry["fwd_bwd_gpu_tflops"] = 3.5 * fl / (fg + bg) / 1e9
            entry["fwd_gbs"] = fwd_bytes / fg / 1e6
            entry["bwd_gbs"] = bwd_bytes / bg / 1e6
            entry["fwd_pct_hbm_peak"] = 100 * fwd_bytes / fg / 1e6 / peaks["hbm_gbs"]
        res["bert_varlen_fp16_dropout_S%d" % S] = entry
    # causal LM (bf16, d = 128)
    for S in (512, 1024, 2048, 4096, 8192):
        if not wanted("causal_lm_bf16_d128_S%d" % S):
            continue
        B, H, d = 16, 12, 128
        cu = torch.arange(0, (B + 1) * S, S, dtype=torch.int32, device=dev)
        q = torch.randn(B * S, H, d, device=dev, dtype=torch.bfloat16, generator=g)
        k = torch.randn(B * S, H, d, device=dev, dtype=torch.bfloat16, generator=g)
        v = torch.randn(B * S, H, d, device=dev, dtype=torch.bfloat16, generator=g)
        dout = torch.randn(B * S, H, d, device=dev, dtype=torch.bfloat16, generator=g)
        f, b = time_fwd_bwd(q, k, v, dout, cu, S, 0.0, True, d ** -0.5)
        fl = fwd_flops([S] * B, H, d, causal=True)
        res["causal_lm_bf16_d128_S%d" % S] = {
            "fwd_ms": f, "bwd_ms": b, "fwd_tflops": fl / f / 1e9, "fwd_bwd_tflops": 3.5 * fl / (f + b) / 1e9,
            "fwd_pct_peak": 100 * fl / f / 1e9 / peaks["tflops"],
            "fwd_bwd_pct_peak": 100 * 3.5 * fl / (f + b) / 1e9 / peaks["tflops"]}
        del q, k, v, dout
    # block-sparse (fp16, d = 64, 256 x 256 blocks at 25 % density + diagonal, dropout 0.1)
    if wanted("blocksparse_fp16_d64_S4096"):
        from flash_attn_b200.flash_blocksparse_attn_interface import convert_blockmask
        B, H, d, S = 4, 16, 64, 4096
        nb = S // 256
        gl = torch.Generator().manual_seed(7)
        blocks = (torch.rand(nb, nb, generator=gl) < 0.25) | torch.eye(nb, dtype=torch.bool)
        layout = blocks.repeat_interleave(16, dim=0).to(torch.int32).to(dev)   # (16-row blocks, key blocks)
        conv = convert_blockmask(layout, False)
        cu = torch.arange(0, (B + 1) * S, S, dtype=torch.int32, device=dev)
        q = torch.randn(B * S, H, d, device=dev, dtype=torch.float16, generator=g)
        k = torch.randn(B * S, H, d, device=dev, dtype=torch.float16, generator=g)
        v = torch.randn(B * S, H, d, device=dev, dtype=torch.float16, generator=g)
        dout = torch.randn(B * S, H, d, device=dev, dtype=torch.float16, generator=g)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        out, lse = fc.fwd_block(q, k, v, cu, cu, conv, S, S, DROPOUT_P, 0.125, False, False, None)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        for it in range(2):
            if it == 1:
                torch.cuda.synchronize()
                ev[0].record()
            for _ in range(20):
                fc.fwd_block(q, k, v, cu, cu, conv, S, S, DROPOUT_P, 0.125, False, False, None)
            if it == 1:
                ev[1].record()
            for _ in range(20):
                fc.bwd_block(dout, q, k, v, out, lse, dq, dk, dv, cu, cu, conv, S, S, DROPOUT_P, 0.125,
                             False, None)
        ev[2].record()
        torch.cuda.synchronize()
        f, b = ev[0].elapsed_time(ev[1]) / 20, ev[1].elapsed_time(ev[2]) / 20
        density = float(blocks.float().mean())
        fl = 4.0 * d * H * B * float(S) * float(S) * density   # work of the blocks in the layout
        res["blocksparse_fp16_d64_S4096"] = {
            "fwd_ms": f, "bwd_ms": b, "layout_density": density, "fwd_tflops": fl / f / 1e9,
            "fwd_bwd_tflops": 3.5 * fl / (f + b) / 1e9,
            "fwd_bwd_pct_peak": 100 * 3.5 * fl / (f + b) / 1e9 / peaks["tflops"]}
        del q, k, v, dout, dq, dk, dv
    # padding helpers (HBM bound): unpad = row gather, pad = row scatter over zeros
    if wanted("unpad_pad_fp16_B64_S512_D2304"):
        from flash_attn_b200 import bert_padding as bp
        B, S, D = 64, 512, 2304
        lengths = torch.tensor(workload_lengths(S, 0, batch=B), device=dev)
        mask = torch.arange(S, device=dev)[None, :] < lengths[:, None]
        idx = torch.nonzero(mask.flatten(), as_tuple=False).flatten()
        x = torch.randn(B * S, D, device=dev, dtype=torch.float16, generator=g)
        packed = bp.gather_rows(x, idx)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(5)]
        for it in range(2):
            if it == 1:
                torch.cuda.synchronize()
                ev[0].record()
            for _ in range(20):
                bp.gather_rows(x, idx)
            if it == 1:
                ev[1].record()
            for _ in range(20):
                bp.scatter_rows(packed, idx, B * S)
            if it == 1:
                ev[2].record()
            for _ in range(20):
                x.index_select(0, idx)
            if it == 1:
                ev[3].record()
            for _ in range(20):
                x.new_zeros((B * S, D)).index_copy_(0, idx, packed)
        ev[4].record()
        torch.cuda.synchronize()
        row = D * 2
        n = idx.numel()
        t = [ev[i].elapsed_time(ev[i + 1]) / 20 for i in range(4)]
        gather_bytes = 2 * n * row + 8 * n                 # rows read + written, indices
        scatter_bytes = n * row + B * S * row + 8 * n + 8 * B * S   # rows read, output written once, index maps
        res["unpad_pad_fp16_B64_S512_D2304"] = {
            "tokens": n, "gather_ms": t[0], "scatter_ms": t[1],
            "gather_gbs": gather_bytes / t[0] / 1e6, "scatter_gbs": scatter_bytes / t[1] / 1e6,
            "gather_frac_hbm_peak": gather_bytes / t[0] / 1e6 / peaks["hbm_gbs"],
            "scatter_frac_hbm_peak": scatter_bytes / t[1] / 1e6 / peaks["hbm_gbs"],
            "torch_index_select_ms": t[2], "torch_zeros_index_copy_ms": t[3]}
        del x, packed
    # rotary embedding on packed qkv (HBM bound): one pass, qkv read once and written once
    if wanted("rotary_qkv_fp16_B64_S512_H12_D64"):
        from flash_attn_b200.rotary import RotaryEmbedding
        B, S, H, D = 64, 512, 12, 64
        qkv = torch.randn(B, S, 3, H, D, device=dev, dtype=torch.float16, generator=g)
        rope = RotaryEmbedding(D).to(dev)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        for it in range(2):
            if it == 1:
                torch.cuda.synchronize()
                ev[0].record()
            for _ in range(20):
                rope.apply_qkv(qkv)
            if it == 1:
                ev[1].record()
            for _ in range(20):
                q_, k_ = rope(qkv[:, :, 0], qkv[:, :, 1], seq_dimension=-3)
                torch.stack([q_, k_, qkv[:, :, 2]], dim=2)
        ev[2].record()
        torch.cuda.synchronize()
        t_fused, t_ops = ev[0].elapsed_time(ev[1]) / 20, ev[1].elapsed_time(ev[2]) / 20
        nbytes = 2 * qkv.numel() * 2
        res["rotary_qkv_fp16_B64_S512_H12_D64"] = {
            "fused_ms": t_fused, "fused_gbs": nbytes / t_fused / 1e6,
            "fused_frac_hbm_peak": nbytes / t_fused / 1e6 / peaks["hbm_gbs"], "framework_ops_ms": t_ops}
        del qkv
    # long context, one GPU's share of an 8-way head shard (batch 2, 32 / 8 = 4 heads, d = 64, causal, bf16)
    if wanted("long_context_bf16_d64_S65536_4heads"):
        B, H, d, S = 2, 4, 64, 65536
        cu = torch.arange(0, (B + 1) * S, S, dtype=torch.int32, device=dev)
        q = torch.randn(B * S, H, d, device=dev, dtype=torch.bfloat16, generator=g)
        k = torch.randn(B * S, H, d, device=dev, dtype=torch.bfloat16, generator=g)
        v = torch.randn(B * S, H, d, device=dev, dtype=torch.bfloat16, generator=g)
        dout = torch.randn(B * S, H, d, device=dev, dtype=torch.bfloat16, generator=g)
        f, b = time_fwd_bwd(q, k, v, dout, cu, S, 0.0, True, 0.125, iters=10)
        fl = fwd_flops([S] * B, H, d, causal=True)
        res["long_context_bf16_d64_S65536_4heads"] = {
            "fwd_ms": f, "bwd_ms": b, "fwd_tflops": fl / f / 1e9, "fwd_bwd_tflops": 3.5 * fl / (f + b) / 1e9,
            "fwd_pct_peak": 100 * fl / f / 1e9 / peaks["tflops"],
            "fwd_bwd_pct_peak": 100 * 3.5 * fl / (f + b) / 1e9 / peaks["tflops"]}
        del q, k, v, dout
    # reduced cases for profiler captures (a few launches, a few hundred MB): only run when asked for by name
    if only in ("reduced_blocksparse_fp16_d64_S4096_B1H4", "reduced_causal_bf16_d64_S16384_B1H4"):
        B, H, d = 1, 4, 64
        sparse = only.startswith("reduced_blocksparse")
        S = 4096 if sparse else 16384
        dt = torch.float16 if sparse else torch.bfloat16
        cu = torch.arange(0, (B + 1) * S, S, dtype=torch.int32, device=dev)
        mk = lambda: torch.randn(B * S, H, d, device=dev, dtype=dt, generator=g)
        q, k, v, dout = mk(), mk(), mk(), mk()
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        if sparse:
            from flash_attn_b200.flash_blocksparse_attn_interface import convert_blockmask
            from flash_attn_b200.sparsity_layouts import RandomLayout
            conv = convert_blockmask(RandomLayout(0.25, seed=7).make_layout(S).to(dev), False)
            fwd = lambda: fc.fwd_block(q, k, v, cu, cu, conv, S, S, DROPOUT_P, 0.125, False, False, None)
            out, lse = fwd()
            bwd = lambda: fc.bwd_block(dout, q, k, v, out, lse, dq, dk, dv, cu, cu, conv, S, S, DROPOUT_P, 0.125,
                                       False, None)
        else:
            fwd = lambda: fc.fwd(q, k, v, cu, cu, S, S, 0.0, 0.125, False, True, False, None)
            out, lse = fwd()
            bwd = lambda: fc.bwd(dout, q, k, v, out, lse, dq, dk, dv, cu, cu, S, S, 0.0, 0.125, False, True, None)
        f = _time_passes(fwd, 3, warmup=1)
        b = _time_passes(bwd, 3, warmup=1)
        res[only] = {"fwd_ms": f, "bwd_ms": b}
        return res
    # dense attention without dropout / without the causal mask, and the cost of the deterministic dQ mode
    dense = {"dense_fp16_d64_nodropout_S4096": (8, 12, 64, 4096, torch.float16, False, 0.0),
             "dense_bf16_d128_noncausal_S4096": (16, 12, 128, 4096, torch.bfloat16, False, 0.0),
             "dense_bf16_d64_causal_S16384": (2, 16, 64, 16384, torch.bfloat16, True, 0.0),
             "dense_fp16_d64_dropout_S4096": (8, 12, 64, 4096, torch.float16, False, DROPOUT_P)}
    for name, (B, H, d, S, dt, causal, p) in dense.items():
        if not wanted(name):
            continue
        cu = torch.arange(0, (B + 1) * S, S, dtype=torch.int32, device=dev)
        q = torch.randn(B * S, H, d, device=dev, dtype=dt, generator=g)
        k = torch.randn(B * S, H, d, device=dev, dtype=dt, generator=g)
        v = torch.randn(B * S, H, d, device=dev, dtype=dt, generator=g)
        dout = torch.randn(B * S, H, d, device=dev, dtype=dt, generator=g)
        f, b = time_fwd_bwd(q, k, v, dout, cu, S, p, causal, d ** -0.5)
        fc.options.deterministic = True
        try:
            _, b_det = time_fwd_bwd(q, k, v, dout, cu, S, p, causal, d ** -0.5)
        finally:
            fc.options.deterministic = False
        fl = fwd_flops([S] * B, H, d, causal=causal)
        res[name] = {"fwd_ms": f, "bwd_ms": b, "fwd_tflops": fl / f / 1e9, "bwd_tflops": 2.5 * fl / b / 1e9,
                     "fwd_pct_peak": 100 * fl / f / 1e9 / peaks["tflops"],
                     "bwd_pct_peak": 100 * 2.5 * fl / b / 1e9 / peaks["tflops"],
                     "fwd_bwd_tflops": 3.5 * fl / (f + b) / 1e9,
                     "fwd_bwd_pct_peak": 100 * 3.5 * fl / (f + b) / 1e9 / peaks["tflops"],
                     "bwd_deterministic_ms": b_det, "deterministic_bwd_slowdown": b_det / b}
        del q, k, v, dout
    return res


if __name__ == "__main__":
    main()
