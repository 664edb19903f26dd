#!/usr/bin/env python
"""Benchmark of the double-backward flash attention operator.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl fhob|reference]

One "step" is one call of the operator (pre-pass + three sweeps) over one batch
of synthetic heads resident in HBM.  Work is sharded over batch x heads with no
collective (weak scaling: every GPU gets the same number of heads), so under
torchrun each rank runs its own shard and the only communication is the
barrier/max-reduction around the timed region.  Rank 0 prints ONE JSON line.

Flop accounting: F_alg = 24*BH*pairs*D (the 12 distinct contractions of the
maths) is what `value`, `e2e` and `cpu_baseline` use; F_exec = 44*BH*pairs*D
(22 contractions issued: 5 by the sweep that yields dd and b, 9 by the dQ2/ddO
pass, 8 by the dK2/dV2 pass) is reported beside it.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
for _p in (ROOT, ROOT / "flash-hob_b200"):
    if str(_p) not in sys.path:
        sys.path.insert(0, str(_p))

# name -> per-GPU shape.  "cfg5-shard" is 1/8 of the cross-attention scaling configuration
# (B=16 H=32 -> 512 heads, 64 per GPU), so --gpus 8 is exactly that configuration.
WORKLOADS = {
    "cfg5-shard": dict(bh=64, n_q=4096, n_k=8192, d=128, causal=False, cot=1.0,
                       desc="bf16 non-causal cross-attention N_Q=4096 N_K=8192 D=128, 64 heads per GPU "
                            "(B=16 H=32 sharded 8 ways)"),
    "cfg2": dict(bh=64, n_q=2048, n_k=2048, d=64, causal=False, cot=1.0,
                 desc="bf16 non-causal B=4 H=16 N=2048 D=64"),
    "cfg3": dict(bh=128, n_q=4096, n_k=4096, d=128, causal=True, cot=0.1,
                 desc="bf16 causal B=8 H=16 N=4096 D=128, cotangents 0.1*N(0,1)"),
    "cfg4-shard": dict(bh=4, n_q=32768, n_k=32768, d=128, causal=True, cot=1.0,
                       desc="bf16 causal N=32768 D=128, 4 heads per GPU (B=1 H=32 sharded 8 ways)"),
    "n8192": dict(bh=32, n_q=8192, n_k=8192, d=128, causal=False, cot=1.0,
                  desc="bf16 non-causal B=1 H=32 N=8192 D=128"),
}
GEMM_UNITS = {"pass12": 5, "pass3": 9, "pass4": 8}
EXEC_OVER_ALG = sum(GEMM_UNITS.values()) / 12.0
# dram__bytes_read.sum + dram__bytes_write.sum per head of one launch of each pass on the default
# workload's shape (N_Q=4096, N_K=8192, D=128), from the ncu capture summarised in
# profiles/tc_pass_kernels_cfg5_16heads.md (captured with 16 heads; traffic grows in proportion to
# the heads, every head having its own tensors).  None for shapes that were not captured.
DRAM_BYTES_PER_HEAD = {("cfg5-shard", "pass12"): 191.01e6 / 16,
                       ("cfg5-shard", "pass3"): 207.72e6 / 16, ("cfg5-shard", "pass4"): 229.56e6 / 16}
KERNEL_NAMES = {"pass12": "tc_pass_kernel<2, {d}, 64, 1, 0>",
                "pass3": "tc_pass_kernel<3, {d}, 64, 0, 0>", "pass4": "tc_pass_kernel<4, {d}, 64, 0, 0>"}


_JSON_FD = None


def claim_stdout():
    """stdout must carry exactly one JSON line, but native libraries write there too (NCCL prints
    its version banner to file descriptor 1).  Keep a private copy of the real stdout for the JSON
    line and point descriptor 1, and with it everything else, at stderr."""
    global _JSON_FD
    if _JSON_FD is None:
        sys.stdout.flush()
        _JSON_FD = os.dup(1)
        os.dup2(2, 1)


def emit(line: dict):
    data = (json.dumps(line) + "\n").encode()
    if _JSON_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_JSON_FD, data)


def pairs(w):
    if w["causal"]:
        assert w["n_q"] == w["n_k"]
        return w["n_q"] * (w["n_q"] + 1) // 2
    return w["n_q"] * w["n_k"]


def f_alg(w, heads=None):
    return 24.0 * (w["bh"] if heads is None else heads) * pairs(w) * w["d"]


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        j = json.loads(p.read_text())
        return dict(burst=j["bf16_tflops"], sustained=j["bf16_tflops_sustained"], hbm=j["hbm_gbs"], src="measured")
    return dict(burst=1590.0, sustained=1400.0, hbm=6650.0, src="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi.

    The process is started well before the timed region (its start-up touches the driver) and
    keeps sampling every 50 ms; `window(t0, t1)` then summarises only the samples whose
    timestamps fall inside the timed region."""
    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            pass

    def window(self, t0, t1):
        """Stops sampling; t0/t1 are time.time() stamps bracketing the timed region."""
        import datetime
        if self.proc is None:
            return None
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        clocks, powers, max_clk, reasons, total = [], [], None, set(), 0
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in out.strip().splitlines():
            f = [s.strip() for s in line.split(",")]
            if len(f) < 8:
                continue
            total += 1
            try:
                ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                clk, mx, pw = float(f[1]), float(f[2]), float(f[3])
            except ValueError:
                continue
            if not (t0 - 0.03 <= ts <= t1 + 0.03):
                continue
            clocks.append(clk)
            powers.append(pw)
            max_clk = mx
            for n, v in zip(names, f[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not clocks:
            return dict(sm_mhz=None, sm_max_mhz=max_clk, reasons=[], samples=0, samples_total=total)
        return dict(sm_mhz=statistics.median(clocks), sm_max_mhz=max_clk, power_w_median=statistics.median(powers),
                    reasons=sorted(reasons), samples=len(clocks), samples_total=total)


def make_batch(w, device, seed):
    g = torch.Generator(device=device).manual_seed(seed)
    def rnd(n, s=1.0):
        return (torch.randn(w["bh"], n, w["d"], generator=g, device=device, dtype=torch.float32) * s).bfloat16()
    x = dict(q=rnd(w["n_q"]), k=rnd(w["n_k"]), v=rnd(w["n_k"]), do=rnd(w["n_q"], w["cot"]),
             ddq=rnd(w["n_q"], w["cot"]), ddk=rnd(w["n_k"], w["cot"]), ddv=rnd(w["n_k"], w["cot"]))
    return x


def cpu_reference_sample(w, reps, warmup):
    """The oracle's grad-of-grad (restatement of jax.vjp(attn_bwd)) on the host cores, one head per step."""
    from oracle import attn_oracle as O
    torch.set_num_threads(os.cpu_count() or 1)
    g = torch.Generator().manual_seed(99)
    x = [torch.randn(n, w["d"], generator=g).bfloat16().float()
         for n in (w["n_q"], w["n_k"], w["n_k"], w["n_q"], w["n_q"], w["n_k"], w["n_k"])]
    scale = w["d"] ** -0.5
    times = []
    for i in range(warmup + reps):
        t0 = time.perf_counter()
        O.bwdbwd_autograd(*x, scale, w["causal"])
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    sec = statistics.median(times)
    return dict(value=f_alg(w, heads=1) / sec / 1e12, unit="TFLOP/s", cores=torch.get_num_threads(), kind="port",
                sample=f"1 head of the workload per step (fp32 torch autograd-of-autograd of the first backward, "
                       f"{reps} steps after {warmup} warm-up, median {sec*1e3:.0f} ms)"), sec


def run_reference(args, w, rank):
    if rank != 0:
        return
    reps = max(1, args.steps)
    cb, sec = cpu_reference_sample(w, reps, max(1, min(args.warmup, 2)))
    line = dict(metric="double_backward_attention_tflops", value=cb["value"], unit="TFLOP/s", impl="reference",
                n_gpus=args.gpus, steps=reps, warmup=max(1, min(args.warmup, 2)), ms_per_step=sec * 1e3,
                higher_is_better=True, scaling="weak", vs_baseline=None, dtype="f32", data="synthetic",
                config=dict(workload=args.workload, description=w["desc"], bh_per_gpu=w["bh"], n_q=w["n_q"],
                            n_k=w["n_k"], d=w["d"], causal=w["causal"],
                            sample="each step is a bounded sample of the workload: 1 head on the host CPU"),
                cpu_baseline=cb,
                e2e=dict(value=cb["value"], unit="TFLOP/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0),
                note="reference XLA double-backward cannot run (jax is not installed); this is the CPU oracle "
                     "port of jax.vjp(attn_bwd) on the box's host cores")
    emit(line)


def mem_sweep():
    """Peak memory of one operator call against sequence length (bf16 causal, 2 heads, D=128).

    Prints one JSON line: per length the bytes of the nine inputs, of the four outputs, the extra
    bytes the call allocated beyond its outputs (the workspace) and what a dense fp32 score
    matrix per head pair would have taken."""
    import fhob
    from fhob import ops
    dev = torch.device("cuda", 0)
    rows = []
    for n in (2048, 4096, 8192, 16384, 32768, 65536):
        w = dict(bh=2, n_q=n, n_k=n, d=128, causal=True, cot=1.0)
        x = make_batch(w, dev, 7)
        o, lse = fhob.attention_forward(x["q"], x["k"], x["v"], 128 ** -0.5, is_causal=True)
        torch.cuda.synchronize()
        ops._workspaces.clear()
        torch.cuda.empty_cache()
        torch.cuda.reset_peak_memory_stats(dev)
        base = torch.cuda.memory_allocated(dev)
        outs = fhob.flash_bwdbwd(x["q"], x["k"], x["v"], o, x["do"], x["ddq"], x["ddk"], x["ddv"], lse, 128 ** -0.5,
                                 is_causal=True, check=True)
        peak = torch.cuda.max_memory_allocated(dev) - base
        out_bytes = sum(t.numel() * t.element_size() for t in outs)
        in_bytes = sum(t.numel() * t.element_size() for t in list(x.values()) + [o, lse])
        rows.append(dict(n=n, input_bytes=in_bytes, output_bytes=out_bytes, extra_bytes=peak - out_bytes,
                         dense_fp32_scores_bytes=2 * n * n * 4))
        del x, o, lse, outs
    print(json.dumps(dict(mem_sweep=rows, note="extra_bytes = workspace (status word + 4 fp32 row vectors, "
                          "1 MiB minimum block); grows linearly with n")), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="cfg5-shard", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="fhob", choices=["fhob", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-producers", action="store_true", help="do not time the forward / first-backward kernels")
    ap.add_argument("--no-clocks", action="store_true", help="do not sample clocks with nvidia-smi")
    ap.add_argument("--heads", type=int, default=0, help="heads per GPU (default: the workload's); "
                    "smaller values give the small cases profiler captures need")
    ap.add_argument("--mem-sweep", action="store_true",
                    help="instead of the benchmark: peak device memory of one call vs sequence length")
    args = ap.parse_args()
    if args.mem_sweep:
        mem_sweep()
        return
    claim_stdout()
    w = dict(WORKLOADS[args.workload])
    if args.heads > 0:
        w["bh"] = args.heads
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, w, rank)
        return

    import torch.distributed as dist
    import fhob
    from fhob import _lib
    from fhob.ops import _Problem

    warmup = max(3, args.warmup)
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    from fhob.sharding import head_shard, max_over_ranks as _max_over_ranks

    def max_over_ranks(ms):
        return _max_over_ranks(ms, device=dev)

    # weak scaling: the job has bh*world heads and every rank owns a contiguous shard of bh of them
    shard_start, shard_heads = head_shard(w["bh"] * world, world, rank)
    assert shard_heads == w["bh"]
    x = make_batch(w, dev, 1234 + shard_start)
    scale = w["d"] ** -0.5
    o, lse = fhob.attention_forward(x["q"], x["k"], x["v"], scale, is_causal=w["causal"])
    args_dev = (x["q"], x["k"], x["v"], o, x["do"], x["ddq"], x["ddk"], x["ddv"], lse, scale)
    in_bytes = sum(t.numel() * t.element_size() for t in args_dev[:9])
    out_bytes = 2 * (x["q"].numel() + x["k"].numel()) * 2

    def step():
        return fhob.flash_bwdbwd(*args_dev, is_causal=w["causal"])

    # ---- device-resident timing
    sampler = ClockSampler(local) if rank == 0 and not args.no_clocks else None
    if sampler:
        time.sleep(0.5)   # let the sampler finish starting up outside the timed region
    barrier()
    # warm-up: at least `warmup` steps and at least 0.3 s of work, so that the timed region starts
    # with the clocks already up (an idle GPU needs tens of milliseconds to leave its idle clocks)
    t_w = time.time()
    done_w = 0
    outs = None
    while done_w < warmup or time.time() - t_w < 0.3:
        outs = step()   # same allocation pattern as the timed loop: no cudaMalloc is left for it
        done_w += 1
        if done_w % 4 == 0:
            torch.cuda.synchronize()
    warmup = done_w
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_start = time.time()
    e0.record()
    for _ in range(args.steps):
        outs = step()
    e1.record()
    barrier()
    t_end = time.time()
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    clocks = sampler.window(t_start, t_end) if sampler else None
    ms_step = ms_total / args.steps
    prob = _Problem(*args_dev, w["causal"], "auto")
    status = prob.status()
    if status != 0:
        raise RuntimeError(f"device status {status} after the timed region")

    # ---- per-pass timing (same stream, CUDA events between the stages)
    lib = _lib.load()
    stages = ["prepass", "pass12", "pass3", "pass4"]
    acc = {s: 0.0 for s in stages}
    s_ptr = C.c_void_p(prob.stream)
    for it in range(2 + args.steps):
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(len(stages) + 1)]
        evs[0].record()
        for i, s in enumerate(stages):
            _lib.check(getattr(lib, f"fhob_{s}")(C.byref(prob.p), s_ptr), s)
            evs[i + 1].record()
        torch.cuda.synchronize()
        if it >= 2:
            for i, s in enumerate(stages):
                acc[s] += evs[i].elapsed_time(evs[i + 1])
    peaks = measured_peaks()
    unit_flops = 2.0 * w["bh"] * pairs(w) * w["d"]
    passes = {}
    for s in stages:
        ms = acc[s] / args.steps
        passes[s] = dict(ms=round(ms, 4))
        if s in GEMM_UNITS:
            tf = GEMM_UNITS[s] * unit_flops / (ms * 1e-3) / 1e12
            passes[s].update(tflops=round(tf, 1), frac_of_sustained_peak=round(tf / peaks["sustained"], 4))
    dom = max(GEMM_UNITS, key=lambda s: passes[s]["ms"])
    per_head = DRAM_BYTES_PER_HEAD.get((args.workload, dom))
    for s in GEMM_UNITS:
        ph = DRAM_BYTES_PER_HEAD.get((args.workload, s))
        passes[s]["dram_traffic_bytes"] = ph * w["bh"] if ph else None
    roofline = dict(bound="tensor", kernel=KERNEL_NAMES[dom].format(d=w["d"]), achieved=passes[dom]["tflops"],
                    peak=peaks["sustained"], unit="TFLOP/s",
                    frac=round(passes[dom]["tflops"] / peaks["sustained"], 4),
                    frac_of_burst_peak=round(passes[dom]["tflops"] / peaks["burst"], 4),
                    peak_source=f"{peaks['src']} cuBLAS bf16 (sustained, kernel timed inside a long step)",
                    flops_basis=f"{GEMM_UNITS[dom]} contractions of 2*BH*pairs*D flop issued by this pass",
                    traffic=per_head * w["bh"] if per_head else None)

    # ---- the producers either side of the operator (forward: O and L; first backward: dQ, dK, dV),
    # outside the timed region; algorithmic counts: 2 and 5 contractions of 2*BH*pairs*D flop
    producers = None
    if not args.no_producers:
        from fhob.autograd import attention_backward
        def timed(fn, reps=5):
            fn()
            torch.cuda.synchronize()
            e0.record()
            for _ in range(reps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / reps
        ms_f = timed(lambda: fhob.attention_forward(x["q"], x["k"], x["v"], scale, is_causal=w["causal"]))
        ms_b = timed(lambda: attention_backward(x["q"], x["k"], x["v"], o, x["do"], lse, scale,
                                                is_causal=w["causal"]))
        producers = dict(
            forward=dict(ms=round(ms_f, 4), tflops_alg=round(2 * unit_flops / (ms_f * 1e-3) / 1e12, 1),
                         executed_contractions=2, kernels="fo_kernel<4,..> (single sweep, online softmax)"),
            first_backward=dict(ms=round(ms_b, 4), tflops_alg=round(5 * unit_flops / (ms_b * 1e-3) / 1e12, 1),
                                executed_contractions=7, kernels="prepass + fo_kernel<2,..> (dQ) + fo_kernel<3,..> (dK, dV)"))

    # ---- end to end through the public entry point with host buffers
    e2e = None
    if not args.no_e2e:
        host = [t.cpu().pin_memory() for t in args_dev[:9]]
        for _ in range(2):
            fhob.flash_bwdbwd(*host, scale, is_causal=w["causal"], device=dev)
        barrier()
        n_e2e = max(2, min(args.steps, 5))
        e0.record()
        for _ in range(n_e2e):
            fhob.flash_bwdbwd(*host, scale, is_causal=w["causal"], device=dev)
        e1.record()
        barrier()
        ms_e2e = max_over_ranks(e0.elapsed_time(e1)) / n_e2e
        e2e = dict(value=f_alg(w) * world / (ms_e2e * 1e-3) / 1e12, unit="TFLOP/s", ms_per_step=ms_e2e,
                   h2d_bytes_per_step=in_bytes, d2h_bytes_per_step=out_bytes, steps=n_e2e)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline:
        cpu_baseline, _ = cpu_reference_sample(w, reps=3, warmup=1)

    value = f_alg(w) * world / (ms_step * 1e-3) / 1e12
    line = dict(
        metric="double_backward_attention_tflops", value=value, unit="TFLOP/s", n_gpus=world, steps=args.steps,
        warmup=warmup, ms_per_step=ms_step, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="bf16",
        data="synthetic",
        config=dict(workload=args.workload, description=w["desc"], bh_per_gpu=w["bh"], n_q=w["n_q"], n_k=w["n_k"],
                    d=w["d"], causal=w["causal"], parallelism=f"batch*heads sharded over {world} GPU(s), no collective",
                    l2="inputs larger than L2: %.0f MB read per step" % (in_bytes / 1e6)),
        per_gpu=dict(tflops_alg=value / world, tflops_exec=value / world * EXEC_OVER_ALG,
                     frac_bf16_peak_alg=value / world / peaks["burst"],
                     frac_bf16_peak_exec=value / world * EXEC_OVER_ALG / peaks["burst"],
                     frac_bf16_sustained_exec=value / world * EXEC_OVER_ALG / peaks["sustained"]),
        flops=dict(f_alg_per_step=f_alg(w) * world, f_exec_per_step=f_alg(w) * world * EXEC_OVER_ALG),
        passes=passes, roofline=roofline, producers=producers, cpu_baseline=cpu_baseline, e2e=e2e, clocks=clocks,
        gpu_launches=4 * args.steps, peak_mem_bytes=torch.cuda.max_memory_allocated(dev))
    emit(line)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
