#!/usr/bin/env python
"""Benchmark of the double-backward flash attention operator.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl fhob|reference|reference-triton]

One "step" is one call of the operator (pre-pass + three sweeps) over this
rank's heads of the job, resident in HBM.  The default job is the multi-GPU
scaling configuration, bf16 non-causal cross-attention B=16 H=32 N_Q=4096
N_K=8192 D=128 = 512 heads: one GPU runs all 512, N GPUs run 512/N each
(strong scaling; heads are independent, so there is no collective on the data
path - the only communication is the barrier and the max-reduction around the
timed region).  Rank 0 prints ONE JSON line.  At one GPU the same line also
carries short runs of the other configurations, the peak-memory sweep over the
sequence length, a check of the timed outputs against the fp64 oracle, the
CPU baseline and the reference project's own Triton operator timed on the
same GPU.

Flop accounting: F_alg = 24*BH*pairs*D (the 12 distinct contractions of the
maths) is what `value`, `e2e`, `roofline.achieved` and `cpu_baseline` use;
F_exec = 44*BH*pairs*D (22 contractions issued: 5 by the sweep that yields dd
and b, 9 by the dQ2/ddO pass, 8 by the dK2/dV2 pass) is reported beside it.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import math
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

# name -> the whole job (heads = batch * heads of the configuration)
WORKLOADS = {
    "cfg5": dict(bh=512, n_q=4096, n_k=8192, d=128, causal=False, cot=1.0,
                 desc="bf16 non-causal cross-attention B=16 H=32 N_Q=4096 N_K=8192 D=128 (512 heads)"),
    "cfg2": dict(bh=64, n_q=2048, n_k=2048, d=64, causal=False, cot=1.0,
                 desc="bf16 non-causal B=4 H=16 N=2048 D=64"),
    "cfg3": dict(bh=128, n_q=4096, n_k=4096, d=128, causal=True, cot=0.1,
                 desc="bf16 causal B=8 H=16 N=4096 D=128, cotangents 0.1*N(0,1)"),
    "cfg4": dict(bh=32, n_q=32768, n_k=32768, d=128, causal=True, cot=1.0,
                 desc="bf16 causal B=1 H=32 N=32768 D=128"),
    "n8192": dict(bh=32, n_q=8192, n_k=8192, d=128, causal=False, cot=1.0,
                  desc="bf16 non-causal B=1 H=32 N=8192 D=128"),
    "cfg1": dict(bh=2, n_q=256, n_k=256, d=64, causal=False, cot=1.0, dtype="f32",
                 desc="fp32 non-causal B=1 H=2 N=256 D=64 (the reference's CPU-runnable case; launch-latency-bound)"),
    "f32-n2048": dict(bh=64, n_q=2048, n_k=2048, d=64, causal=False, cot=1.0, dtype="f32",
                      desc="fp32 non-causal 64 heads N=2048 D=64 (cfg2's shape in fp32: tensor cores with split "
                           "bf16 operands, three products per contraction)"),
}
# the other configurations carried by the one-GPU line: (workload, heads, steps)
EXTRAS = (("cfg2", 64, 20), ("cfg3", 128, 8), ("cfg4", 32, 5), ("n8192", 32, 5), ("cfg1", 2, 20), ("f32-n2048", 64, 5))
GEMM_UNITS = {"pass12": 5, "pass3": 9, "pass4": 8}
EXEC_OVER_ALG = sum(GEMM_UNITS.values()) / 12.0
# dram__bytes_read.sum + dram__bytes_write.sum per head of one launch of each pass at N_Q=4096,
# N_K=8192, D=128, from an ncu capture of a 16-head case (every head has its own tensors, so the
# traffic of a launch grows in proportion to its heads).
DRAM_BYTES_PER_HEAD = {("cfg5", "pass12"): 190.32e6 / 16, ("cfg5", "pass3"): 213.21e6 / 16,
                       ("cfg5", "pass4"): 229.11e6 / 16}
# template arguments: pass, head dim of q/k, head dim of v, streamed rows, fused dd+b sweep, fp16 storage,
# split fp32 operands
KERNEL_NAMES = {"pass12": "tc_pass_kernel<2, {d}, {d}, 64, 1, 0, 0>",
                "pass3": "tc_pass_kernel<3, {d}, {d}, 64, 0, 0, 0>", "pass4": "tc_pass_kernel<4, {d}, {d}, 64, 0, 0, 0>"}
METRIC = "double_backward_attention_tflops"

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


def make_batch(w, heads, device, seed):
    g = torch.Generator(device=device).manual_seed(seed)
    def rnd(n, s=1.0):
        t = (torch.randn(heads, n, w["d"], generator=g, device=device, dtype=torch.float32) * s).bfloat16()
        return t.float() if w.get("dtype") == "f32" else t   # fp32 workloads: bf16-representable fp32 values
    return dict(q=rnd(w["n_q"]), k=rnd(w["n_k"]), v=rnd(w["n_k"]), do=rnd(w["n_q"], w["cot"]),
                ddq=rnd(w["n_q"], w["cot"]), ddk=rnd(w["n_k"], w["cot"]), ddv=rnd(w["n_k"], w["cot"]))


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


def config_block(name, w, heads, world):
    return dict(workload=name, description=w["desc"], heads=w["bh"], heads_per_gpu=heads, n_q=w["n_q"], n_k=w["n_k"],
                d=w["d"], causal=w["causal"],
                parallelism=f"batch*heads split over {world} GPU(s) (strong scaling), no collective")


def run_reference(args, w, rank):
    """The reference arm: the reference's CPU path.  Its own double backward is JAX/XLA, which is
    not installed (and cannot be, offline), so the arm times the oracle's restatement of
    jax.vjp(attn_bwd) on all host cores, one head of the workload per step."""
    if rank != 0:
        return
    reps = max(1, args.steps)
    warm = max(1, min(args.warmup, 2))
    cb, sec = cpu_reference_sample(w, reps, warm)
    cfg = config_block(args.workload, w, w["bh"] // max(1, args.gpus), args.gpus)
    cfg["sample"] = "each step is a bounded sample of the workload: 1 head on the host CPU"
    emit(dict(metric=METRIC, value=cb["value"], unit="TFLOP/s", impl="reference", n_gpus=args.gpus, steps=reps,
              warmup=warm, ms_per_step=sec * 1e3, higher_is_better=True, scaling="strong", vs_baseline=None,
              dtype="f32", data="synthetic", config=cfg, cpu_baseline=cb,
              e2e=dict(value=cb["value"], unit="TFLOP/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0),
              note="reference XLA double-backward cannot run (jax is not installed); this is the CPU oracle "
                   "port of jax.vjp(attn_bwd) on the box's host cores"))


class Case:
    """One workload resident on one GPU: inputs, saved forward results, the operator call."""

    def __init__(self, w, heads, dev, seed):
        import fhob
        self.w, self.heads, self.dev = w, heads, dev
        self.x = make_batch(w, heads, dev, seed)
        self.scale = w["d"] ** -0.5
        x = self.x
        self.o, self.lse = fhob.attention_forward(x["q"], x["k"], x["v"], self.scale, is_causal=w["causal"])
        self.args = (x["q"], x["k"], x["v"], self.o, x["do"], x["ddq"], x["ddk"], x["ddv"], self.lse, self.scale)
        self.in_bytes = sum(t.numel() * t.element_size() for t in self.args[:9])
        self.out_bytes = 2 * (x["q"].numel() + x["k"].numel()) * x["q"].element_size()
        self.unit_flops = 2.0 * heads * pairs(w) * w["d"]

    def step(self, impl="auto"):
        import fhob
        return fhob.flash_bwdbwd(*self.args, is_causal=self.w["causal"], impl=impl)

    def status(self):
        from fhob.ops import _Problem
        return _Problem(*self.args, self.w["causal"], "auto").status()

    def time_passes(self, iters):
        """Average CUDA-event time of each stage over `iters` runs of the four stages (after two untimed)."""
        from fhob import _lib
        from fhob.ops import _Problem
        prob = _Problem(*self.args, self.w["causal"], "auto")
        lib = _lib.load()
        stages = ["prepass", "pass12", "pass3", "pass4"]
        acc = {s: 0.0 for s in stages}
        s_ptr = C.c_void_p(prob.stream)
        recorded = []
        for it in range(2 + iters):
            evs = [torch.cuda.Event(enable_timing=True) for _ in range(len(stages) + 1)]
            evs[0].record()
            for i, s in enumerate(stages):
                _lib.check(getattr(lib, f"fhob_{s}")(C.byref(prob.p), s_ptr), s)
                evs[i + 1].record()
            if it % 8 == 7:
                torch.cuda.synchronize()   # keeps the launch queue short
            if it >= 2:
                recorded.append(evs)
        torch.cuda.synchronize()
        for evs in recorded:
            for i, s in enumerate(stages):
                acc[s] += evs[i].elapsed_time(evs[i + 1])
        peaks = measured_peaks()
        out = {}
        for s in stages:
            ms = acc[s] / iters
            out[s] = dict(ms=round(ms, 4))
            if s in GEMM_UNITS:
                tf = GEMM_UNITS[s] * self.unit_flops / (ms * 1e-3) / 1e12
                out[s].update(contractions=GEMM_UNITS[s], tflops_exec=round(tf, 1),
                              frac_of_sustained_peak=round(tf / peaks["sustained"], 4),
                              frac_of_burst_peak=round(tf / peaks["burst"], 4))
        return out

    def check_head(self, outs, head):
        """Max relative error of one head of `outs` against the chunked fp64 oracle (run on the GPU)."""
        from oracle import attn_oracle as O
        x = self.x
        ref = O.bwdbwd_closed_form_chunked(*(x[n][head].double() for n in ("q", "k", "v", "do", "ddq", "ddk", "ddv")),
                                           self.scale, self.w["causal"], chunk=1024)
        return {n: O.rel_err(g[head], r) for n, g, r in zip(("dq2", "dk2", "dv2", "ddo"), outs, ref[:4])}


def summarise(w, heads, ms_step, world=1):
    """value and fractions of the measured cuBLAS bf16 peaks for `world` ranks of `heads` heads each."""
    peaks = measured_peaks()
    per_gpu = f_alg(w, heads) / (ms_step * 1e-3) / 1e12
    return dict(tflops_alg=per_gpu, tflops_exec=per_gpu * EXEC_OVER_ALG,
                frac_bf16_burst_alg=per_gpu / peaks["burst"], frac_bf16_sustained_alg=per_gpu / peaks["sustained"],
                frac_bf16_burst_exec=per_gpu * EXEC_OVER_ALG / peaks["burst"],
                frac_bf16_sustained_exec=per_gpu * EXEC_OVER_ALG / peaks["sustained"])


def run_extra(name, heads, steps, dev):
    """A short device-resident run of another configuration (one GPU): warm-up, `steps` timed
    steps, per-pass times, one head checked against the oracle."""
    w = dict(WORKLOADS[name])
    case = Case(w, heads, dev, seed=4321)
    for _ in range(3):
        outs = case.step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        outs = case.step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    status = case.status()
    res = dict(description=w["desc"], heads=heads, steps=steps, ms_per_step=round(ms, 4), device_status=status,
               inputs_mb=round(case.in_bytes / 1e6, 1))
    res.update({k: round(v, 4) for k, v in summarise(w, heads, ms).items()})
    res["passes"] = case.time_passes(max(3, steps // 2))
    res["max_rel_err_vs_fp64_oracle"] = case.check_head(outs, heads - 1)
    if w.get("dtype") == "f32":
        # every contraction is issued as three bf16 products (hi.hi + hi.lo + lo.hi): the executed-flop
        # figures above count each contraction once, the tensor pipe does three times that
        res["dtype"] = "f32"
        res["tolerance"] = 1e-4
        res["products_per_contraction"] = 3
        case.step("simt")
        torch.cuda.synchronize()
        e0.record()
        outs = case.step("simt")
        e1.record()
        torch.cuda.synchronize()
        res["cuda_core_kernels"] = dict(ms_per_step=round(e0.elapsed_time(e1), 4),
                                        tflops_alg=round(f_alg(w, heads) / e0.elapsed_time(e1) / 1e9, 2),
                                        max_rel_err_vs_fp64_oracle=case.check_head(outs, heads - 1))
    return res


def mem_sweep(dev):
    """Peak memory of one operator call against sequence length (bf16 causal, 2 heads, D=128): per
    length the bytes of the nine inputs, of the four outputs, the extra bytes the call allocated
    beyond its outputs (the workspace, 1 MiB minimum block) and what dense fp32 score matrices
    would have taken."""
    import fhob
    from fhob import ops
    rows = []
    for n in (2048, 4096, 8192, 16384, 32768, 65536):
        w = dict(bh=2, n_q=n, n_k=n, d=128, causal=True, cot=1.0)
        x = make_batch(w, 2, dev, 7)
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
    ops._workspaces.clear()
    torch.cuda.empty_cache()
    return rows


# ---------------------------------------------------------------- the reference's Triton operator

def competitor_child(args):
    """Times the reference project's own operator (fhog.flash_bwdbwd, Triton, installed unmodified
    under baseline/_ref) on this GPU and compares its results with this library's.  Prints one
    JSON object.  Non-causal shapes with lengths that are multiples of its tiles only: it has no
    causal mask and no bounds checks."""
    ref_dir = ROOT / "baseline" / "_ref"
    if not (ref_dir / "fhog" / "triton_bwdbwd.py").exists():
        print(json.dumps(dict(error=f"{ref_dir.relative_to(ROOT)} is missing (baseline/install_reference.sh "
                                    "installs the reference there)")))
        return
    cache = ROOT / "baseline" / "_triton_cache"
    if cache.is_dir():
        os.environ.setdefault("TRITON_CACHE_DIR", str(cache))
    sys.path.insert(0, str(ref_dir))
    import fhob
    from oracle import attn_oracle as O
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    w = dict(WORKLOADS[args.workload])
    heads = args.heads or w["bh"]
    if w["causal"] or w.get("dtype") == "f32":
        print(json.dumps(dict(error="the reference operator has no causal mask and is benchmarked in 16-bit only")))
        return
    # its autotune key holds the sequence lengths and the head dim, not the number of heads, so the
    # (slow) tuning runs are made on a 16-head case
    tune_heads = min(heads, 16)
    case = Case(w, tune_heads, dev, seed=777)
    t0 = time.time()
    from fhog.triton_bwdbwd import bwdbwd_kernel_stage1, bwdbwd_kernel_stage2, flash_bwdbwd as ref_bwdbwd
    how = "as shipped: fhog.flash_bwdbwd, a torch.compile(fullgraph=True) wrapper around two autotuned Triton kernels"
    as_shipped_error = None
    try:
        theirs = ref_bwdbwd(*case.args)      # first call: torch.compile + Triton autotune over its config list
    except Exception as e:  # noqa: BLE001
        # The compiled wrapper can fail with this image's torch/triton pair.  The function under
        # the wrapper is the same unmodified reference code; calling it directly only skips
        # torch.compile (the Triton kernels and their autotuning are untouched).
        eager = getattr(ref_bwdbwd, "_torchdynamo_orig_callable", None) or getattr(ref_bwdbwd, "__wrapped__", None)
        lines = [l for l in str(e).strip().splitlines() if l.strip()]
        as_shipped_error = f"{type(e).__name__}: " + " | ".join(lines[-3:])[:500]
        if eager is None:
            print(json.dumps(dict(error=as_shipped_error)))
            return
        import importlib
        importlib.import_module("torch._dynamo").reset()
        ref_bwdbwd = eager
        how = "the function under the reference's torch.compile wrapper, called directly (the wrapper itself failed)"
        theirs = ref_bwdbwd(*case.args)
    torch.cuda.synchronize()
    setup_s = time.time() - t0
    if tune_heads < heads:
        del theirs, case
        torch.cuda.empty_cache()
        case = Case(w, heads, dev, seed=777)
    for _ in range(2):
        theirs = ref_bwdbwd(*case.args)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        theirs = ref_bwdbwd(*case.args)
    e1.record()
    torch.cuda.synchronize()
    ms_ref = e0.elapsed_time(e1) / args.steps
    for _ in range(3):
        ours = case.step()
    e0.record()
    for _ in range(args.steps):
        ours = case.step()
    e1.record()
    torch.cuda.synchronize()
    ms_ours = e0.elapsed_time(e1) / args.steps
    def cfg(k):
        b = getattr(k, "best_config", None)
        return str(b) if b is not None else None
    names = ("dq2", "dk2", "dv2", "ddo")
    oracle_err_theirs = case.check_head(theirs, heads - 1)
    oracle_err_ours = case.check_head(ours, heads - 1)
    print(json.dumps(dict(
        workload=args.workload, heads=heads, steps=args.steps, setup_s=round(setup_s, 1), how=how,
        as_shipped_error=as_shipped_error,
        reference_triton=dict(ms_per_step=round(ms_ref, 4), tflops_alg=round(f_alg(w, heads) / ms_ref / 1e9, 1),
                              autotuned_stage1=cfg(bwdbwd_kernel_stage1), autotuned_stage2=cfg(bwdbwd_kernel_stage2),
                              max_rel_err_vs_fp64_oracle=oracle_err_theirs),
        this_library=dict(ms_per_step=round(ms_ours, 4), tflops_alg=round(f_alg(w, heads) / ms_ours / 1e9, 1),
                          max_rel_err_vs_fp64_oracle=oracle_err_ours),
        speedup=round(ms_ref / ms_ours, 2),
        max_rel_diff_between_the_two={n: O.rel_err(a, b.float()) for n, a, b in zip(names, ours, theirs)})))


def competitor_triton(cases, steps, timeout_s):
    """Runs `competitor_child` once per (workload, heads) in a child process with a time limit, so
    that a slow autotune or a failure of the reference's code cannot take the benchmark line down."""
    out = {}
    for name, heads in cases:
        cmd = [sys.executable, str(ROOT / "bench.py"), "--competitor-child", "--workload", name, "--heads", str(heads),
               "--steps", str(steps)]
        try:
            r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout_s)
            lines = [l for l in r.stdout.strip().splitlines() if l.startswith("{")]
            out[name] = json.loads(lines[-1]) if lines else dict(
                error=f"exit code {r.returncode}: " + (r.stderr.strip().splitlines() or ["no output"])[-1][:300])
        except subprocess.TimeoutExpired:
            out[name] = dict(error=f"no result within {timeout_s} s (Triton compiles and times every configuration "
                                   "of the reference's autotune list on the first call)")
        except Exception as e:  # noqa: BLE001
            out[name] = dict(error=f"{type(e).__name__}: {e}"[:300])
    return out


# ---------------------------------------------------------------- main

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="cfg5", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="fhob", choices=["fhob", "reference", "reference-triton"],
                    help="reference: the CPU arm (oracle port on the host cores); reference-triton: the reference's "
                         "own Triton operator on one GPU, same workload (non-causal 16-bit workloads only)")
    ap.add_argument("--heads", type=int, default=0, help="heads of the whole job (default: the workload's); "
                    "smaller values give the small cases profiler captures need")
    ap.add_argument("--min-timed-s", type=float, default=1.0,
                    help="rounds of --steps steps are repeated until at least this much device time is covered")
    ap.add_argument("--min-rounds", type=int, default=3, help="at least this many rounds (the median round is reported)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-producers", action="store_true", help="do not time the forward / first-backward kernels")
    ap.add_argument("--no-clocks", action="store_true", help="do not sample clocks with nvidia-smi")
    ap.add_argument("--no-extras", action="store_true",
                    help="one GPU: skip the other configurations, the memory sweep and the Triton comparison")
    ap.add_argument("--no-competitor", action="store_true", help="skip only the reference's Triton operator")
    ap.add_argument("--competitor-timeout", type=int, default=240)
    ap.add_argument("--competitor-child", action="store_true", help=argparse.SUPPRESS)
    args = ap.parse_args()
    if args.competitor_child:
        competitor_child(args)
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
    if args.impl == "reference-triton":
        if rank == 0:
            heads = w["bh"] // max(1, args.gpus)
            res = competitor_triton(((args.workload, heads),), steps=max(2, min(args.steps, 10)),
                                    timeout_s=max(args.competitor_timeout, 600))[args.workload]
            cfg = config_block(args.workload, w, heads, 1)
            cfg["sample"] = f"{heads} heads on one GPU (one rank's share when --gpus > 1)"
            if "error" in res:
                emit(dict(impl="reference-triton", unavailable=res["error"], config=cfg))
            else:
                t = res["reference_triton"]
                emit(dict(metric=METRIC, value=t["tflops_alg"], unit="TFLOP/s", impl="reference-triton", n_gpus=1,
                          steps=res["steps"], warmup=2, ms_per_step=t["ms_per_step"], higher_is_better=True,
                          scaling="strong", vs_baseline=None, dtype="bf16", data="synthetic", config=cfg, detail=res))
        return

    import torch.distributed as dist
    import fhob
    from fhob.hostmem import near_device
    from fhob.sharding import head_shard, max_over_ranks as _max_over_ranks

    warmup = max(3, args.warmup)
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        return _max_over_ranks(ms, device=dev)

    # strong scaling: the job's heads are split into contiguous shards, one per rank
    shard_start, shard_heads = head_shard(w["bh"], world, rank)
    if shard_heads == 0:
        raise SystemExit(f"rank {rank}: the job has fewer heads ({w['bh']}) than ranks ({world})")
    case = Case(w, shard_heads, dev, seed=1234 + shard_start)

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
        outs = case.step()   # same allocation pattern as the timed loop: no cudaMalloc is left for it
        done_w += 1
        if done_w % 4 == 0:
            torch.cuda.synchronize()
    torch.cuda.synchronize()
    warmup = done_w
    est_ms = (time.time() - t_w) * 1e3 / done_w
    # rounds of exactly `steps` steps; enough of them to cover --min-timed-s of device time
    rounds = max(1, args.min_rounds, min(50, math.ceil(args.min_timed_s * 1e3 / max(est_ms * args.steps, 1e-3))))
    if world > 1:
        t = torch.tensor([rounds], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        rounds = int(t.item())
    barrier()
    round_ms = []
    t_start = time.time()
    for _ in range(rounds):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            outs = case.step()
        e1.record()
        barrier()
        round_ms.append(max_over_ranks(e0.elapsed_time(e1)))
    t_end = time.time()
    clocks = sampler.window(t_start, t_end) if sampler else None
    ms_step = statistics.median(round_ms) / args.steps
    status = case.status()
    if status != 0:
        raise RuntimeError(f"device status {status} after the timed region")

    # ---- the timed outputs against the fp64 oracle (one head, outside the timed region)
    parity = case.check_head(outs, shard_heads - 1) if rank == 0 else None

    # ---- per-pass timing (same stream, CUDA events between the stages)
    peaks = measured_peaks()
    passes = case.time_passes(max(args.steps, 10) * (2 if est_ms < 30 else 1))
    dom = max(GEMM_UNITS, key=lambda s: passes[s]["ms"])
    for s in GEMM_UNITS:
        ph = DRAM_BYTES_PER_HEAD.get((args.workload, s))
        passes[s]["dram_traffic_bytes"] = ph * shard_heads if ph else None
        passes[s]["share_of_step"] = round(passes[s]["ms"] / sum(passes[k]["ms"] for k in passes), 4)
    per_head = DRAM_BYTES_PER_HEAD.get((args.workload, dom))
    per_gpu = summarise(w, shard_heads, ms_step)
    roofline = dict(
        bound="tensor", unit="TFLOP/s",
        achieved=round(per_gpu["tflops_alg"], 1), peak=peaks["sustained"], frac=round(per_gpu["frac_bf16_sustained_alg"], 4),
        basis="whole operator on one GPU, algorithmic flops (12 contractions: F_alg = 24*BH*pairs*D) / step time; "
              "the operator issues 22 contractions (recomputation in three sweeps), so 12/22 = 0.545 is the "
              "ceiling of this figure",
        frac_of_burst_peak=round(per_gpu["frac_bf16_burst_alg"], 4), peak_burst=peaks["burst"],
        peak_source=f"{peaks['src']} cuBLAS bf16: sustained (seconds-long loop under the power cap; the timed "
                    f"region here is {sum(round_ms) / 1e3:.1f} s) and burst",
        executed=dict(achieved=round(per_gpu["tflops_exec"], 1), frac=round(per_gpu["frac_bf16_sustained_exec"], 4),
                      frac_of_burst_peak=round(per_gpu["frac_bf16_burst_exec"], 4),
                      basis="the same with the 22 issued contractions (what the tensor pipe executes)"),
        dominant_kernel=dict(kernel=KERNEL_NAMES[dom].format(d=w["d"]), ms=passes[dom]["ms"],
                             share_of_step=passes[dom]["share_of_step"], achieved_exec=passes[dom]["tflops_exec"],
                             frac_exec=passes[dom]["frac_of_sustained_peak"],
                             frac_exec_of_burst_peak=passes[dom]["frac_of_burst_peak"],
                             basis=f"{GEMM_UNITS[dom]} contractions of 2*BH*pairs*D flop issued by this launch / its "
                                   "average CUDA-event time"),
        traffic=per_head * shard_heads if per_head else None,
        traffic_note="dominant kernel, per launch: ncu dram bytes of a 16-head capture scaled by the heads")

    # ---- the producers either side of the operator (forward: O and L; first backward: dQ, dK, dV),
    # outside the timed region; algorithmic counts: 2 and 5 contractions of 2*BH*pairs*D flop
    producers = None
    x = case.x
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
        ms_f = timed(lambda: fhob.attention_forward(x["q"], x["k"], x["v"], case.scale, is_causal=w["causal"]))
        ms_b = timed(lambda: attention_backward(x["q"], x["k"], x["v"], case.o, x["do"], case.lse, case.scale,
                                                is_causal=w["causal"]))
        producers = dict(
            forward=dict(ms=round(ms_f, 4), tflops_alg=round(2 * case.unit_flops / (ms_f * 1e-3) / 1e12, 1),
                         executed_contractions=2, kernels="fo_kernel<4,..> (single sweep, online softmax)"),
            first_backward=dict(ms=round(ms_b, 4), tflops_alg=round(5 * case.unit_flops / (ms_b * 1e-3) / 1e12, 1),
                                executed_contractions=7, kernels="prepass + fo_kernel<2,..> (dQ) + fo_kernel<3,..> (dK, dV)"))

    # ---- end to end through the public entry point with host buffers
    e2e = None
    if not args.no_e2e:
        with near_device(dev) as placement:
            host = [t.cpu().pin_memory() for t in case.args[:9]]
            host_out = tuple(torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
                             for t in (x["q"], x["k"], x["k"], x["q"]))
        # what the link gives one direction at a time (pinned memory, one large copy each way)
        big = max(host[:8], key=lambda t: t.numel())
        dst = torch.empty_like(big, device=dev)
        link = {}
        for name, fn in (("h2d", lambda: dst.copy_(big, non_blocking=True)),
                         ("d2h", lambda: host_out[1].copy_(x["k"], non_blocking=True))):
            fn()
            torch.cuda.synchronize()
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            nbytes = (big if name == "h2d" else x["k"]).numel() * 2
            link[name] = nbytes / (e0.elapsed_time(e1) * 1e-3) / 1e9
        # every input tensor alone: pinned buffers that landed on a remote memory node show up here
        per_tensor = []
        for t in host[:8]:
            d_t = dst[: t.shape[0]] if t.shape == big.shape else torch.empty_like(t, device=dev)
            d_t.copy_(t, non_blocking=True)
            torch.cuda.synchronize()
            e0.record()
            d_t.copy_(t, non_blocking=True)
            e1.record()
            torch.cuda.synchronize()
            per_tensor.append(round(t.numel() * t.element_size() / (e0.elapsed_time(e1) * 1e-3) / 1e9, 1))
            del d_t
        link["h2d_per_tensor"] = per_tensor
        # and with both directions busy in the step's own proportion (two parts up, one part down),
        # which is what the pipelined path asks of the link
        up, down = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        up.wait_stream(torch.cuda.current_stream(dev))
        down.wait_stream(torch.cuda.current_stream(dev))
        u0, u1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(up):
            u0.record()
            for _ in range(2):
                dst.copy_(big, non_blocking=True)
            u1.record()
        with torch.cuda.stream(down):
            host_out[1].copy_(x["k"], non_blocking=True)
        torch.cuda.synchronize()
        link["h2d_duplex"] = 2 * big.numel() * 2 / (u0.elapsed_time(u1) * 1e-3) / 1e9
        if world > 1:
            # all ranks upload at the same moment (the slowest rank counts): what the host gives
            # every link when each GPU of the job pulls from it at once
            barrier()
            e0.record()
            for _ in range(2):
                dst.copy_(big, non_blocking=True)
            e1.record()
            torch.cuda.synchronize()
            link["h2d_all_ranks"] = 2 * big.numel() * 2 / (max_over_ranks(e0.elapsed_time(e1)) * 1e-3) / 1e9
            # the same with every rank also downloading (two parts up, one part down, like the step)
            barrier()
            up.wait_stream(torch.cuda.current_stream(dev))
            down.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(up):
                u0.record()
                for _ in range(2):
                    dst.copy_(big, non_blocking=True)
                u1.record()
            with torch.cuda.stream(down):
                host_out[1].copy_(x["k"], non_blocking=True)
            torch.cuda.synchronize()
            link["h2d_all_ranks_duplex"] = 2 * big.numel() * 2 / (max_over_ranks(u0.elapsed_time(u1)) * 1e-3) / 1e9
        del dst
        def e2e_step():
            return fhob.flash_bwdbwd(*host, case.scale, is_causal=w["causal"], device=dev, out=host_out)
        for _ in range(2):
            e2e_step()
        barrier()
        n_e2e = max(2, min(args.steps, 5))
        e0.record()
        for _ in range(n_e2e):
            e2e_step()
        e1.record()
        barrier()
        ms_e2e = max_over_ranks(e0.elapsed_time(e1)) / n_e2e
        e2e = dict(value=f_alg(w) / (ms_e2e * 1e-3) / 1e12, unit="TFLOP/s", ms_per_step=ms_e2e,
                   h2d_bytes_per_step=case.in_bytes, d2h_bytes_per_step=case.out_bytes, steps=n_e2e,
                   note="bytes are this rank's (rank 0); inputs in pinned host memory, results into pinned host "
                        "tensors passed as out=, uploads, kernels and downloads of head ranges overlapped",
                   h2d_gbs=round(case.in_bytes / (ms_e2e * 1e-3) / 1e9, 1),
                   d2h_gbs=round(case.out_bytes / (ms_e2e * 1e-3) / 1e9, 1),
                   link_alone_h2d_gbs=round(link["h2d"], 1), link_alone_d2h_gbs=round(link["d2h"], 1),
                   frac_of_link_h2d=round(case.in_bytes / (ms_e2e * 1e-3) / 1e9 / link["h2d"], 3),
                   link_alone_h2d_gbs_per_input=link["h2d_per_tensor"],
                   link_all_ranks_at_once_h2d_gbs=round(link["h2d_all_ranks"], 1) if "h2d_all_ranks" in link else None,
                   link_all_ranks_at_once_duplex_h2d_gbs=(round(link["h2d_all_ranks_duplex"], 1)
                                                          if "h2d_all_ranks_duplex" in link else None),
                   link_duplex_h2d_gbs=round(link["h2d_duplex"], 1),
                   frac_of_duplex_link_h2d=round(case.in_bytes / (ms_e2e * 1e-3) / 1e9 / link["h2d_duplex"], 3),
                   host_placement=placement)
        del host, host_out

    peak_mem = torch.cuda.max_memory_allocated(dev)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- one GPU only: the other configurations, memory against sequence length, the
    # reference's Triton operator on the same GPU, the CPU baseline
    extras = sweep = competitor = cpu_baseline = None
    if world == 1:
        del case, outs, x
        torch.cuda.empty_cache()
        if not args.no_extras:
            extras = {}
            for name, heads, steps in EXTRAS:
                key = name if heads == WORKLOADS[name]["bh"] else f"{name}-shard"
                try:
                    extras[key] = run_extra(name, heads, steps, dev)
                except Exception as e:  # noqa: BLE001
                    extras[key] = dict(error=f"{type(e).__name__}: {e}"[:300])
                torch.cuda.empty_cache()
            sweep = mem_sweep(dev)
            if not args.no_competitor:
                torch.cuda.empty_cache()
                competitor = competitor_triton((("cfg2", 64), ("cfg5", 16)), steps=10, timeout_s=args.competitor_timeout)
        if not args.no_cpu_baseline:
            cpu_baseline, _ = cpu_reference_sample(w, reps=3, warmup=1)

    value = f_alg(w) / (ms_step * 1e-3) / 1e12
    cfg = config_block(args.workload, w, shard_heads, world)
    cfg["l2"] = "inputs larger than L2: %.0f MB read per step and GPU" % (case_in_mb(w, shard_heads))
    line = dict(
        metric=METRIC, value=value, unit="TFLOP/s", n_gpus=world, steps=args.steps, warmup=warmup,
        rounds=rounds, ms_per_step=ms_step, ms_per_round=[round(m, 3) for m in round_ms],
        timing="median over `rounds` rounds of exactly `steps` steps each (CUDA events, max over ranks per round)",
        higher_is_better=True, scaling="strong", vs_baseline=None, dtype="bf16", data="synthetic", config=cfg,
        per_gpu=per_gpu, flops=dict(f_alg_per_step=f_alg(w), f_exec_per_step=f_alg(w) * EXEC_OVER_ALG),
        passes=passes, roofline=roofline, parity_of_timed_outputs=dict(
            max_rel_err_vs_fp64_oracle=parity, head="last head of rank 0's shard", tolerance=2e-2),
        producers=producers, cpu_baseline=cpu_baseline, e2e=e2e, clocks=clocks,
        gpu_launches=4 * args.steps * rounds, peak_mem_bytes=peak_mem,
        other_configs=extras, mem_sweep=sweep, competitor_triton=competitor)
    emit(line)
    if world > 1:
        dist.destroy_process_group()


def case_in_mb(w, heads):
    es = 2
    return heads * ((4 * w["n_q"] + 4 * w["n_k"]) * w["d"] * es + 4 * w["n_q"]) / 1e6


if __name__ == "__main__":
    main()
