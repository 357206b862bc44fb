#!/usr/bin/env python
"""FLCE forward+backward throughput on B200s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c3|c4|c5|small]

One step = one fused-linear-cross-entropy forward + backward over one batch of synthetic tokens
(default workload: the Llama-3-8B head, N=32768 tokens, H=4096, V=128256, bf16, 5 % ignored targets,
mean reduction, returning grad_input and grad_weight).  With N GPUs (launched under torchrun, one rank
per GPU) every rank processes its own N tokens against a replicated weight and the weight gradient is
all-reduced over NCCL inside the step: weak scaling, `value` is the sum over ranks.

Rank 0 prints one JSON line.  `--impl reference` times the torch
Linear+CrossEntropy ground truth of the reference's tests on the host cores instead.
"""

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "liger-kernel_b200"))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

WORKLOADS = {
    # name: N, H, V, ignored fraction, kwargs
    "small": dict(N=4096, H=1024, V=32000, ign=0.10, kw=dict()),
    "profile": dict(N=10880, H=4096, V=32768, ign=0.05, kw=dict()),  # small case for ncu captures: one token chunk of the
    # C2 size (so the weight-gradient GEMM has its real K), a quarter of the vocabulary; W = 268 MB > L2, 0.7 GB copy
    "c2": dict(N=32768, H=4096, V=128256, ign=0.05, kw=dict()),
    "c3": dict(N=32768, H=3584, V=152064, ign=0.20, kw=dict(label_smoothing=0.1, lse_square_scale=1e-4, return_z_loss=True)),
    "c4": dict(N=16384, H=3584, V=256000, ign=0.05, zipf=1.1, kw=dict(softcap=30.0, reduction="sum")),
    "c5": dict(N=65536, H=8192, V=128256, ign=0.05, kw=dict()),
}
NAMES = {
    "small": "FLCE small head N=4096 H=1024 V=32000 bf16",
    "profile": "FLCE profiling case N=10880 H=4096 V=32768 bf16 (one token chunk)",
    "c2": "Llama-3-8B LM head FLCE bf16: N=32768 (B=8,T=4096) H=4096 V=128256, 5% ignored, mean, fwd+bwd",
    "c3": "Qwen2.5-7B-style head FLCE bf16: N=32768 H=3584 V=152064, label_smoothing 0.1, z-loss 1e-4, 20% ignored",
    "c4": "Gemma-2-9B-style head FLCE bf16: N=16384 H=3584 V=256000, softcap 30, sum, Zipf(1.1) targets, 5% ignored",
    "c5": "Llama-3-70B LM head FLCE bf16: N=65536 H=8192 V=128256, 5% ignored, mean",
}


# DRAM bytes per (live token row x vocabulary column) of one launch, from an ncu capture of the profiling case with the DRAM
# counters alone (dram__bytes_read.sum + dram__bytes_write.sum over 10336 live rows x 32768 columns, one token chunk of the C2
# height; summary under profiles/).  Traffic of a full-size launch is this figure times the units that launch covers: the
# store of the chunk and the streamed operand grow with the units for a fixed raster.
_PROFILE_UNITS = 10336 * 32768
NCU_DRAM_BYTES_PER_UNIT = {"stats": (1.373e9 + 0.684e9) / _PROFILE_UNITS, "dz": 0.0,
                           "dw": (2.033e9 + 0.264e9) / _PROFILE_UNITS, "dx": (2.173e9 + 0.081e9) / _PROFILE_UNITS}


BESIDE_GEMM_GROUP = None   # set in main() at N > 1: the NCCL group for collectives that run beside a GEMM


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(burst=float(d["bf16_tflops"]), sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                    hbm=float(d["hbm_gbs"]), source="measured")
    return dict(burst=1590.0, sustained=1400.0, hbm=6650.0, source="fallback")


def make_inputs(spec, device, seed):
    g = torch.Generator(device=device).manual_seed(seed)
    N, H, V = spec["N"], spec["H"], spec["V"]
    x = torch.randn(N, H, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    w = (torch.randn(V, H, generator=g, device=device, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    if spec.get("zipf"):
        # class frequencies of natural text: rank r drawn with probability proportional to r^-s (inverse-CDF sampling)
        cdf = torch.cumsum(torch.arange(1, V + 1, device=device, dtype=torch.float64).pow(-float(spec["zipf"])), 0)
        u = torch.rand(N, generator=g, device=device, dtype=torch.float64) * cdf[-1]
        t = torch.searchsorted(cdf, u).clamp_(max=V - 1)
    else:
        t = torch.randint(0, V, (N,), generator=g, device=device)
    drop = torch.rand(N, generator=g, device=device) < spec["ign"]
    t = torch.where(drop, torch.full_like(t, -100), t)
    return x, w, t


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled every 200 ms while a timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.path = None

    def __enter__(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=self.out, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.out.close()

    def summary(self):
        res = dict(sm_mhz=None, sm_max_mhz=None, reasons=[], samples=0)
        if self.path is None or not os.path.exists(self.path):
            return res
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 7:
                    continue
                try:
                    sm.append(float(parts[0]))
                    mx.append(float(parts[1]))
                except ValueError:
                    continue
                for name, val in zip(names, parts[3:7]):
                    if val.lower() == "active":
                        reasons.add(name)
        os.unlink(self.path)
        if sm:
            busy = [v for v in sm if v > 0.5 * max(sm)] or sm
            res.update(sm_mhz=statistics.median(busy), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return res


class CpuReference:
    """The torch Linear+CrossEntropy ground truth of the reference's tests (fp32, autograd backward) on the host cores,
    fed with rows of the workload's shape at the full H and V.  The weight is built once, outside any timing."""

    def __init__(self, spec, seed=99):
        # torchrun pins OMP_NUM_THREADS=1 for its workers: take all host cores back for the CPU arm
        torch.set_num_threads(max(1, os.cpu_count() or 1))
        self.g = torch.Generator().manual_seed(seed)
        self.H, self.V = spec["H"], spec["V"]
        self.w = torch.randn(self.V, self.H, generator=self.g) * 0.02
        self.kw = {k: v for k, v in spec["kw"].items() if k in ("label_smoothing", "lse_square_scale", "softcap", "reduction")}

    def run_rows(self, rows):
        from oracle.flce_oracle import torch_linear_ce_reference

        x = torch.randn(rows, self.H, generator=self.g)
        t = torch.randint(0, self.V, (rows,), generator=self.g)
        t[::20] = -100
        t0 = time.perf_counter()
        torch_linear_ce_reference(x, self.w, t, **self.kw)
        return time.perf_counter() - t0


def cpu_reference_rate(spec, seconds_budget, rows_per_chunk=256, max_rows=1024):
    """tokens/s over up to max_rows rows in chunks, stopping early once the time budget is spent."""
    ref = CpuReference(spec)
    ref.run_rows(32)  # warm the thread pool
    done, busy = 0, 0.0
    while done < max_rows and busy < seconds_budget:
        busy += ref.run_rows(rows_per_chunk)
        done += rows_per_chunk
    return done / busy, done, busy


def run_reference(args, spec, rank, world):
    if rank != 0:
        return
    rows = 256
    ref = CpuReference(spec)
    for _ in range(args.warmup):
        ref.run_rows(rows)
    busy = 0.0
    for _ in range(args.steps):
        busy += ref.run_rows(rows)
    value = rows * args.steps / busy
    cores = torch.get_num_threads()
    sample = f"{rows} rows per step with the full H={spec['H']} and V={spec['V']} (fp32 torch Linear+CrossEntropy, autograd backward)"
    print(json.dumps({
        "impl": "reference", "metric": "flce_fwd_bwd_tokens_per_s", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * busy / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": NAMES[args.workload], "sample": sample},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "host_cpus": os.cpu_count(),
    }))


def run_liger(args, spec, rank, world, local_rank):
    """The reference's own GPU operator (installed unmodified under baseline/_ref) on the same workload and
    timing, for the side-by-side number.  `--impl liger_triton`: its default Triton path; `--impl liger_cutedsl`:
    its CuTe-DSL sm_100 path (LIGER_KERNEL_IMPL=cutedsl), which needs a newer nvidia-cutlass-dsl than some images have;
    `--impl torch_gpu`: plain torch Linear + cross-entropy on the GPU with materialised fp32 logits."""
    if rank != 0:
        return
    if args.impl == "torch_gpu":
        def ref_flce(xin, w, t, softcap=None, lse_square_scale=0.0, return_z_loss=False, accum_dtype=None, **ce_kw):
            # the plain path the fused operator replaces: fp32 logits [N, V] materialised, torch cross-entropy
            logits = (xin @ w.t()).float()
            if softcap is not None:
                logits = softcap * torch.tanh(logits / softcap)
            loss = torch.nn.functional.cross_entropy(logits, t, ignore_index=-100, **ce_kw)
            if lse_square_scale:
                lse = torch.logsumexp(logits, dim=-1)
                loss = loss + lse_square_scale * (lse[t != -100] ** 2).mean()
            return loss
    else:
        ref_dir = os.path.join(ROOT, "baseline", "_ref")
        if not os.path.isdir(os.path.join(ref_dir, "liger_kernel")):
            print(json.dumps({"impl": args.impl, "unavailable": "baseline/_ref/liger_kernel is not installed"}))
            return
        if args.impl == "liger_cutedsl":
            os.environ["LIGER_KERNEL_IMPL"] = "cutedsl"
        sys.path.insert(0, ref_dir)
        try:
            from liger_kernel.transformers.functional import liger_fused_linear_cross_entropy as ref_flce
        except Exception as e:  # noqa: BLE001
            print(json.dumps({"impl": args.impl, "unavailable": f"import failed: {type(e).__name__}: {e}"[:300]}))
            return
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    x, w, t = make_inputs(spec, device, 1234)
    w.requires_grad_(True)
    kw = dict(spec["kw"])
    if args.accum_fp32:
        kw["accum_dtype"] = torch.float32
    N, H, V = spec["N"], spec["H"], spec["V"]

    def step():
        xin = x.detach().requires_grad_(True)
        w.grad = None
        out = ref_flce(xin, w, t, **kw)
        loss = out if torch.is_tensor(out) else out.loss
        loss.backward()
        return loss

    try:
        for _ in range(args.warmup):
            step()
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats()
        with ClockSampler(local_rank) as clocks:
            marks = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
            marks[0].record()
            for i in range(args.steps):
                step()
                marks[i + 1].record()
            torch.cuda.synchronize()
    except Exception as e:  # noqa: BLE001
        print(json.dumps({"impl": args.impl, "unavailable": f"run failed: {type(e).__name__}: {e}"[:300]}))
        return
    ms = marks[0].elapsed_time(marks[-1]) / args.steps
    per_step = sorted(marks[i].elapsed_time(marks[i + 1]) for i in range(args.steps))
    quantiles = {f"p{q}": per_step[min(len(per_step) - 1, int(q / 100 * len(per_step)))] for q in (20, 50, 80)}
    clock_info = clocks.summary()
    peaks = load_peaks()
    tflops = 8.0 * N * H * V / (ms * 1e-3) / 1e12
    print(json.dumps({
        "impl": args.impl, "metric": "flce_fwd_bwd_tokens_per_s", "value": N / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "dtype": "bf16",
        "data": "synthetic", "config": {"workload": NAMES[args.workload], "accum_dtype": "fp32" if args.accum_fp32 else None},
        "tflops_credited_8NHV": tflops, "frac_of_burst": tflops / peaks["burst"],
        "peak_mem_gb": torch.cuda.max_memory_allocated() / 1e9,
        "ms_per_step_quantiles": quantiles,
        "clocks": {"sm_mhz": clock_info["sm_mhz"], "sm_max_mhz": clock_info["sm_max_mhz"], "reasons": clock_info["reasons"]},
    }))


COMPARATORS = [
    # name in the bench line, extra command-line arguments
    ("liger_triton", ["--impl", "liger_triton"]),
    ("liger_triton_accum_fp32", ["--impl", "liger_triton", "--accum-fp32"]),
    ("liger_cutedsl", ["--impl", "liger_cutedsl"]),
    ("torch_gpu", ["--impl", "torch_gpu"]),
]


def run_comparators(args, timeout_s):
    """The reference's own GPU operators and plain torch on the same box, same inputs (same seed), same steps and the same
    CUDA-event timing, each in a child process of its own (a fresh CUDA context, nothing of this library loaded)."""
    out = {}
    for name, extra in COMPARATORS:
        cmd = [sys.executable, os.path.abspath(__file__), "--workload", args.workload, "--steps", str(args.steps),
               "--warmup", str(args.warmup)] + extra
        t0 = time.perf_counter()
        try:
            proc = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout_s, stdin=subprocess.DEVNULL)
        except subprocess.TimeoutExpired:
            out[name] = {"unavailable": f"no result within {timeout_s} s"}
            continue
        rec = None
        for line in reversed(proc.stdout.strip().splitlines()):
            if line.startswith("{"):
                try:
                    rec = json.loads(line)
                    break
                except ValueError:
                    continue
        if rec is None:
            tail = (proc.stderr or proc.stdout or "").strip().splitlines()[-1:] or [""]
            out[name] = {"unavailable": f"exit code {proc.returncode}: {tail[0][:200]}"}
        elif "unavailable" in rec:
            out[name] = {"unavailable": rec["unavailable"]}
        else:
            out[name] = {"ms_per_step": rec["ms_per_step"], "tokens_per_s": rec["value"], "peak_mem_gb": rec.get("peak_mem_gb"),
                         "ms_per_step_quantiles": rec.get("ms_per_step_quantiles"), "clocks": rec.get("clocks"),
                         "wall_s": round(time.perf_counter() - t0, 1)}
    return out


def multi_gpu_extras(args, rank, world, device, peaks):
    """At N > 1 GPUs, after the weak-scaling line: the fixed-problem (strong scaling) configurations the workload list
    names as multi-GPU, each timed on all ranks and, for the efficiency, on rank 0 alone in the same invocation;
    the collectives' own device time; the spread of the ranks' kernel time; and a bare all-reduce of a grad_weight-sized
    buffer.  Returns a dict of extra keys for the JSON line (rank 0) or None."""
    import torch.distributed as dist

    import liger_kernel_b200.sharded as sharded
    from liger_kernel_b200 import _lib
    from liger_kernel_b200.transformers.functional import liger_fused_linear_cross_entropy

    steps, warmup = 3, 2

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    def timed(step_fn, participate=True):
        ms = 0.0
        if participate:
            for _ in range(warmup):
                step_fn()
            torch.cuda.synchronize()
        barrier()
        if participate:
            _lib.profile_enable(True)
            sharded.COLLECTIVE_EVENTS = []
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                step_fn()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / steps
        barrier()
        out = dict(ms=ms, kernels_ms=0.0, collectives={})
        if participate:
            prof = _lib.profile_read(reset=True)
            _lib.profile_enable(False)
            out["kernels_ms"] = sum(v[0] for v in prof.values()) / steps
            for name, a, b in sharded.COLLECTIVE_EVENTS:
                out["collectives"][name] = out["collectives"].get(name, 0.0) + a.elapsed_time(b) / steps
            sharded.COLLECTIVE_EVENTS = None
        return out

    def gather_max(v):
        t = torch.tensor([v], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def gather_min(v):
        t = torch.tensor([v], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return float(t.item())

    extras = {}
    # ---- a bare all-reduce of a grad_weight-sized bf16 buffer (C2: 1.05 GB)
    spec = WORKLOADS[args.workload]
    buf = torch.zeros(spec["V"], spec["H"], device=device, dtype=torch.bfloat16)
    r = timed(lambda: dist.all_reduce(buf))
    ms = gather_max(r["ms"])
    nbytes = buf.numel() * 2
    extras["allreduce_alone"] = {"bytes": nbytes, "ms": ms, "algbw_gbs": nbytes / ms / 1e6,
                                 "busbw_gbs": nbytes / ms / 1e6 * 2 * (world - 1) / world}
    del buf
    single_gpu_ms = {}
    for key, wl, mode in (("c5_strong_token", "c5", "token"), ("c5_vocab", "c5", "vocab"), ("c4_vocab", "c4", "vocab")):
        try:
            spec = WORKLOADS[wl]
            N, H, V = spec["N"], spec["H"], spec["V"]
            kw = {k: v for k, v in spec["kw"].items() if k != "return_z_loss"}
            x, w, t = make_inputs(spec, device, 4321)        # the same full problem on every rank
            if wl not in single_gpu_ms:
                w1 = w.clone().requires_grad_(True)

                def one_gpu():
                    xin = x.detach().requires_grad_(True)
                    w1.grad = None
                    out = liger_fused_linear_cross_entropy(xin, w1, t, **kw)
                    (out if torch.is_tensor(out) else out.loss).backward()

                r1 = timed(one_gpu, participate=(rank == 0))
                single_gpu_ms[wl] = gather_max(r1["ms"])
                del w1
            if mode == "token":
                n_loc = N // world
                xs, ts = x[rank * n_loc:(rank + 1) * n_loc].clone(), t[rank * n_loc:(rank + 1) * n_loc].clone()
                ws = w.clone().requires_grad_(True)

                def step():
                    xin = xs.detach().requires_grad_(True)
                    ws.grad = None
                    sharded.token_sharded_fused_linear_cross_entropy(
                        xin, ws, ts, group=BESIDE_GEMM_GROUP if sharded.OVERLAP_GRAD_WEIGHT else None, **kw).backward()
            else:
                per = (V + world - 1) // world
                lo = rank * per
                ws = w[lo:min(V, lo + per)].clone().requires_grad_(True)

                def step():
                    xin = x.detach().requires_grad_(True)
                    ws.grad = None
                    sharded.vocab_sharded_fused_linear_cross_entropy(
                        xin, ws, t, lo, V, group=BESIDE_GEMM_GROUP if sharded.OVERLAP_COLLECTIVES else None,
                        **kw).backward()
            del w
            r = timed(step)
            ms = gather_max(r["ms"])
            colls = {}
            for name in sorted(r["collectives"]):
                colls[name] = gather_max(r["collectives"][name])
            extras[key] = {
                "workload": NAMES[wl], "sharding": mode, "scaling": "strong", "ms_per_step": ms,
                "tokens_per_s": N / (ms * 1e-3), "single_gpu_ms_per_step": single_gpu_ms[wl],
                "efficiency_vs_n1": single_gpu_ms[wl] / (world * ms),
                "collective_ms_max_over_ranks": colls,
                "rank_kernel_ms": {"min": gather_min(r["kernels_ms"]), "max": gather_max(r["kernels_ms"])},
                "steps": steps, "warmup": warmup,
            }
            del x, t, ws
            torch.cuda.empty_cache()
        except Exception as e:  # noqa: BLE001
            extras[key] = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
            barrier()
    return extras if rank == 0 else None


def run_ours(args, spec, rank, world, local_rank):
    import torch.distributed as dist

    from liger_kernel_b200 import _lib
    from liger_kernel_b200.sharded import token_sharded_fused_linear_cross_entropy
    from liger_kernel_b200.transformers.functional import liger_fused_linear_cross_entropy

    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        import liger_kernel_b200.sharded as sharded_mod
        if args.comm_overlap is not None:      # 0: nothing overlapped; 1: also grad_weight of the token-sharded main line
            sharded_mod.OVERLAP_COLLECTIVES = bool(args.comm_overlap)
            sharded_mod.OVERLAP_GRAD_WEIGHT = bool(args.comm_overlap)
        import datetime
        dist.init_process_group("nccl", device_id=device, timeout=datetime.timedelta(seconds=180))
        # calls whose collectives run beside a GEMM (which leaves them RESERVE_SMS_FOR_COLLECTIVE SMs) go through a
        # second group limited to 16 thread blocks; a collective with the GPU to itself uses the default group
        global BESIDE_GEMM_GROUP
        BESIDE_GEMM_GROUP = None
        if sharded_mod.OVERLAP_COLLECTIVES or sharded_mod.OVERLAP_GRAD_WEIGHT:
            BESIDE_GEMM_GROUP = sharded_mod.new_group_for_collectives_beside_gemm(
                max_ctas=16, timeout=datetime.timedelta(seconds=180), device_id=device)
    if args.cta_pair is not None:
        _lib.set_option("cta_pair", args.cta_pair)
    if args.raster_mb is not None:
        _lib.set_option("raster_group_bytes", args.raster_mb << 20)
    import liger_kernel_b200.ops.fused_linear_cross_entropy as flce_op
    if args.mode is not None:
        flce_op.MODE = args.mode
    if args.store is not None:
        flce_op.STORE_MODE = args.store
    if args.wide_tiles is not None:
        _lib.set_option("wide_tiles", args.wide_tiles)
    if args.poll_sleep_ns is not None:
        _lib.set_option("poll_sleep_ns", args.poll_sleep_ns)
    if args.n_group is not None:
        _lib.set_option("raster_n_group", args.n_group)
    for item in args.option:
        name, value = item.split("=", 1)
        _lib.set_option(name, int(value))
    if args.chunk_gib is not None:
        flce_op.CHUNK_BUDGET_BYTES = int(args.chunk_gib * (1 << 30))
    peaks = load_peaks()
    from liger_kernel_b200.sharded import vocab_sharded_fused_linear_cross_entropy

    vocab_lo = 0
    if args.sharding == "vocab" and world > 1:
        # replicated tokens, each rank owns a slice of the vocabulary (strong scaling of one problem)
        x, w, t = make_inputs(spec, device, 1234)
        per = (spec["V"] + world - 1) // world
        vocab_lo = rank * per
        w = w[vocab_lo:min(spec["V"], vocab_lo + per)].clone()
    elif args.strong and world > 1:
        # one global batch split by rows
        x, w, t = make_inputs(spec, device, 1234)
        n_loc = spec["N"] // world
        x, t = x[rank * n_loc:(rank + 1) * n_loc].clone(), t[rank * n_loc:(rank + 1) * n_loc].clone()
    else:
        x, w, t = make_inputs(spec, device, 1234 + rank)
        if world > 1:
            dist.broadcast(w, 0)
    w.requires_grad_(True)
    x_host = x.cpu().pin_memory()
    t_host = t.cpu().pin_memory()
    x_dev = torch.empty_like(x)
    t_dev = torch.empty_like(t)
    kw = dict(spec["kw"])
    N, H, V = spec["N"], spec["H"], spec["V"]

    def step(xin, tin):
        xin = xin.detach().requires_grad_(True)
        w.grad = None
        if world > 1 and args.sharding == "vocab":
            skw = {k: v for k, v in kw.items() if k != "return_z_loss"}
            loss = vocab_sharded_fused_linear_cross_entropy(xin, w, tin, vocab_lo, spec["V"], **skw)
        elif world > 1:
            # global-batch loss; grad_weight is all-reduced over NCCL inside backward
            skw = {k: v for k, v in kw.items() if k != "return_z_loss"}
            loss = token_sharded_fused_linear_cross_entropy(
                xin, w, tin, overlap_grad_weight=args.overlap,
                group=BESIDE_GEMM_GROUP if sharded_mod.OVERLAP_GRAD_WEIGHT else None, **skw)
        else:
            out = liger_fused_linear_cross_entropy(xin, w, tin, **kw)
            loss = out if torch.is_tensor(out) else out.loss
        loss.backward()
        return loss, xin.grad

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        v = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(v, op=dist.ReduceOp.MAX)
        return float(v.item())

    for _ in range(args.warmup):
        step(x, t)
    torch.cuda.reset_peak_memory_stats()
    launches0 = _lib.lib.flce_b200_kernel_launches()
    _lib.profile_enable(True)
    import liger_kernel_b200.sharded as sharded_timing
    if world > 1:
        sharded_timing.COLLECTIVE_EVENTS = []
    barrier()
    with ClockSampler(local_rank) as clocks:
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
        marks[0].record()
        for i in range(args.steps):
            step(x, t)
            marks[i + 1].record()
        e0, e1 = marks[0], marks[-1]
        barrier()
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    per_step = sorted(marks[i].elapsed_time(marks[i + 1]) for i in range(args.steps))      # this rank's steps
    step_quantiles = {f"p{q}": per_step[min(len(per_step) - 1, int(q / 100 * len(per_step)))] for q in (20, 50, 80)}
    prof = _lib.profile_read(reset=True)
    _lib.profile_enable(False)
    collective_ms = None
    if world > 1:
        collective_ms = {}
        for name, a, b in sharded_timing.COLLECTIVE_EVENTS:
            collective_ms[name] = collective_ms.get(name, 0.0) + a.elapsed_time(b) / args.steps
        sharded_timing.COLLECTIVE_EVENTS = None
        collective_ms = {name: max_over_ranks(v) for name, v in sorted(collective_ms.items())}
        kernel_sum = sum(v[0] for v in prof.values()) / args.steps
        rank_kernel_ms = {"max": max_over_ranks(kernel_sum), "min": -max_over_ranks(-kernel_sum)}
    launches = _lib.lib.flce_b200_kernel_launches() - launches0
    peak_mem = torch.cuda.max_memory_allocated()
    clock_info = clocks.summary()

    # End to end: host buffers in, loss out, every step.  Every step's inputs cross PCIe from pinned host memory inside the
    # timed region, on a copy stream and into the other of two device buffers, so that step i+1's copy runs beside step
    # i's kernels (what a data loader with a prefetching device iterator does); the loss is read back every step.
    copy_stream = torch.cuda.Stream(device=device)
    bufs = [(x_dev, t_dev), (torch.empty_like(x), torch.empty_like(t))]
    ready = [torch.cuda.Event(), torch.cuda.Event()]
    consumed = [torch.cuda.Event(), torch.cuda.Event()]

    def start_copy(slot):
        copy_stream.wait_event(consumed[slot])             # the step that last read this buffer is done with it
        with torch.cuda.stream(copy_stream):
            bufs[slot][0].copy_(x_host, non_blocking=True)
            bufs[slot][1].copy_(t_host, non_blocking=True)
            ready[slot].record()

    def e2e_run(n_steps):
        for slot in (0, 1):
            consumed[slot].record()
        start_copy(0)
        last = 0.0
        for i in range(n_steps):
            slot = i & 1
            if i + 1 < n_steps:
                start_copy(slot ^ 1)
            torch.cuda.current_stream().wait_event(ready[slot])
            loss, _ = step(*bufs[slot])
            consumed[slot].record()
            last = float(loss.item())
        return last

    e2e_run(max(2, args.warmup // 2))
    barrier()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record()
    e2e_run(args.steps)
    e3.record()
    barrier()
    ms_e2e = max_over_ranks(e2.elapsed_time(e3))

    extras = None
    if world > 1 and not args.no_variants and args.sharding == "token" and not args.strong:
        extras = multi_gpu_extras(args, rank, world, device, peaks)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    ms_step = ms_total / args.steps
    strong = world > 1 and (args.strong or args.sharding == "vocab")
    tokens = N if strong else N * world
    value = tokens / (ms_step * 1e-3)
    flops_step = 8.0 * N * H * V / (world if strong else 1)  # per rank, as the metric credits them
    tflops = flops_step / (ms_step * 1e-3) / 1e12
    # Each tensor-core kernel kind multiplies this rank's live rows (targets that are not ignore_index: the others are
    # moved out of the way and skipped) by H x V (its share of the vocabulary) once: 2 * rows * H * V executed FLOPs.
    rows_here = x.shape[0]
    live_here = int((t != -100).sum().item()) if flce_op.SKIP_IGNORED else rows_here
    kind_flops = 2.0 * live_here * H * w.shape[0] * args.steps
    kinds = [k for k in ("stats", "dz", "dw", "dx") if prof[k][0] > 0]
    dom = max(kinds, key=lambda k: prof[k][0])
    dom_ms, dom_launches = prof[dom]
    achieved = kind_flops / (dom_ms * 1e-3) / 1e12 if dom_ms > 0 else 0.0
    per_kind = {k: {"ms_per_step": prof[k][0] / args.steps, "launches_per_step": prof[k][1] / args.steps,
                    "tflops_executed": (kind_flops / (prof[k][0] * 1e-3) / 1e12) if prof[k][0] > 0 else None}
                for k in ("stats", "dz", "dw", "dx")}
    per_kind["row_passes"] = {"ms_per_step": prof["gemm"][0] / args.steps, "launches_per_step": prof["gemm"][1] / args.steps}
    executed_step = sum(2.0 * live_here * H * w.shape[0] for k in kinds)
    result = {
        "metric": "flce_fwd_bwd_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "strong" if strong else "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": NAMES[args.workload], "tokens_per_gpu": x.shape[0], "hidden": H, "vocab_per_gpu": w.shape[0],
                   "parallelism": "single GPU" if world == 1 else (
                       f"vocab-sharded x{world}: all-gather of row statistics, all-reduce of grad_input" if args.sharding == "vocab"
                       else f"token-sharded x{world}, NCCL all-reduce of grad_weight"),
                   "l2_policy": "inputs larger than L2 (weight alone is %.2f GB)" % (V * H * 2 / 1e9),
                   "cta_pair": args.cta_pair, "raster_mb": args.raster_mb, "mode": flce_op.MODE,
                   "store": flce_op.STORE_MODE, "skip_ignored_rows": flce_op.SKIP_IGNORED},
        "tflops_per_gpu": tflops,
        "tflops_per_gpu_executed": executed_step / (ms_step * 1e-3) / 1e12,
        "flops_note": "tflops_per_gpu credits 8.N.H.V per step as the metric defines it; executed = 2.rows.H.V per tensor-core "
                      "sweep actually run (3 sweeps when gradients are formed in forward, 4 with recompute), rows = targets "
                      "that are not ignore_index",
        "live_rows_per_gpu": live_here,
        "frac_of_bf16_peak": {"burst": tflops / peaks["burst"], "sustained": tflops / peaks["sustained"], "peaks": peaks["source"]},
        "roofline": {"bound": "tensor", "kernel": dom, "achieved": achieved, "peak": peaks["sustained"], "unit": "TFLOP/s",
                     "frac": achieved / peaks["sustained"], "frac_of_burst": achieved / peaks["burst"],
                     "launches": dom_launches, "avg_launch_ms": dom_ms / max(1, dom_launches),
                     "peak_kind": f"sustained bf16 GEMM, {peaks['source']}",
                     "flops_basis": "executed: 2 x live rows x H x V per step for this kernel kind",
                     "traffic": NCU_DRAM_BYTES_PER_UNIT[dom] * live_here * w.shape[0] * args.steps / max(1, dom_launches),
                     "traffic_note": "ncu capture of the N=10880 (10336 live), V=32768 case scaled by live rows x columns per launch"},
        "kernels": per_kind,
        "e2e": {"value": tokens / (ms_e2e / args.steps * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
                "h2d_bytes_per_step": x_host.numel() * 2 + t_host.numel() * 8, "d2h_bytes_per_step": 4},
        "global_tokens_per_step": tokens,
        "collective_ms_max_over_ranks": collective_ms,
        "rank_kernel_ms": rank_kernel_ms if world > 1 else None,
        "comm_overlap": ({"grad_input_of_vocab_shards": sharded_timing.OVERLAP_COLLECTIVES,
                          "grad_weight_of_token_shards": sharded_timing.OVERLAP_GRAD_WEIGHT} if world > 1 else None),
        "gpu_launches": int(launches),
        "peak_mem_gb": peak_mem / 1e9,
        "ms_per_step_quantiles": step_quantiles,
        "clocks": {"sm_mhz": clock_info["sm_mhz"], "sm_max_mhz": clock_info["sm_max_mhz"], "reasons": clock_info["reasons"],
                   "samples": clock_info["samples"]},
    }
    if world == 1 and args.mode is None and not args.no_variants:
        # the same workload on the two-sweep path (logits recomputed in backward: 8.N.H.V executed, least memory)
        default_mode = flce_op.MODE
        flce_op.MODE = "recompute"
        for _ in range(args.warmup):
            step(x, t)
        torch.cuda.reset_peak_memory_stats()
        _lib.profile_enable(True)
        barrier()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(args.steps):
            step(x, t)
        s1.record()
        barrier()
        ms_ss = s0.elapsed_time(s1) / args.steps
        prof_ss = _lib.profile_read(reset=True)
        _lib.profile_enable(False)
        flce_op.MODE = default_mode
        result["recompute_mode"] = {
            "ms_per_step": ms_ss, "value": tokens / (ms_ss * 1e-3), "unit": "tokens/s",
            "tflops_credited_8NHV": 8.0 * N * H * V / (ms_ss * 1e-3) / 1e12,
            "peak_mem_gb": torch.cuda.max_memory_allocated() / 1e9,
            "kernels_ms_per_step": {k: prof_ss[k][0] / args.steps for k in prof_ss},
            "note": "LIGER_B200_FLCE_MODE=recompute: forward keeps nothing of size N x V, backward recomputes the logit tiles; "
                    "the headline value above is the default mode (gradients formed in forward from a bounded 16-bit copy)",
        }
    if world == 1 and not args.no_cpu_baseline:
        rate, rows, secs = cpu_reference_rate(spec, seconds_budget=12.0)
        result["cpu_baseline"] = {
            "value": rate, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"first {rows} rows with the full H and V, fp32 torch Linear+CrossEntropy with autograd, {secs:.1f} s",
        }
    if extras:
        result.update(extras)
    if world == 1 and not args.no_comparators:
        comps = run_comparators(args, args.comparator_timeout)
        result["comparators"] = comps
        liger_ms = [c["ms_per_step"] for n, c in comps.items() if n.startswith("liger") and "ms_per_step" in c]
        # below 1 means this library's step is shorter than the fastest of the reference's own GPU paths on this box
        result["vs_liger_best"] = (ms_step / min(liger_ms)) if liger_ms else None
    print(json.dumps(result))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "liger_triton", "liger_cutedsl", "torch_gpu"])
    ap.add_argument("--accum-fp32", action="store_true", dest="accum_fp32")
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--cta-pair", type=int, default=None, dest="cta_pair")
    ap.add_argument("--raster-mb", type=int, default=None, dest="raster_mb")
    ap.add_argument("--mode", default=None, choices=["recompute", "single_sweep", "auto"])
    ap.add_argument("--store", default=None, choices=["auto", "logits", "exp"], help="what the single-sweep mode keeps of a chunk")
    ap.add_argument("--wide-tiles", type=int, default=None, dest="wide_tiles")
    ap.add_argument("--poll-sleep-ns", type=int, default=None, dest="poll_sleep_ns")
    ap.add_argument("--option", action="append", default=[], metavar="NAME=VALUE",
                    help="library tuning option (flce_b200_set_option); may be repeated")
    ap.add_argument("--n-group", type=int, default=None, dest="n_group",
                    help="gradient GEMMs: n-tiles per raster group (0 = all: the re-read operand is the whole of B)")
    ap.add_argument("--comm-overlap", type=int, default=None, dest="comm_overlap",
                    help="multi-GPU: 1 = start every big collective beside the GEMM that follows (side stream, SMs reserved, NCCL "
                         "capped at 16 CTAs), 0 = issue them after the sweep with every SM to themselves; default: only the "
                         "partial grad_input of vocabulary shards is overlapped")
    ap.add_argument("--chunk-gib", type=float, default=None, dest="chunk_gib",
                    help="bytes (GiB) of the bounded 16-bit copy of a token chunk in the single-sweep mode (default 2.5)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-variants", action="store_true", dest="no_variants")
    ap.add_argument("--no-comparators", action="store_true", dest="no_comparators",
                    help="skip the reference's GPU operators and plain torch (timed after the main measurement at --gpus 1)")
    ap.add_argument("--comparator-timeout", type=int, default=180, dest="comparator_timeout", help="seconds per comparator")
    ap.add_argument("--sharding", default="token", choices=["token", "vocab"])
    ap.add_argument("--overlap", action="store_true", help="all-reduce grad_weight slab by slab on a side stream")
    ap.add_argument("--strong", action="store_true", help="fixed global batch split over the ranks (token sharding)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    spec = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, spec, rank, world)
    elif args.impl in ("liger_triton", "liger_cutedsl", "torch_gpu"):
        run_liger(args, spec, rank, world, local_rank)
    else:
        run_ours(args, spec, rank, world, local_rank)


if __name__ == "__main__":
    main()
