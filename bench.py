#!/usr/bin/env python
"""Benchmark of the triangle-attention hot path (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one forward + backward pass of the pair-biased masked attention over one batch of
synthetic input with the AF3 crop-384 shapes (q, k, v [1, 384, 384, 4, 32] bf16, pair_bias
[1, 1, 4, 384, 384], last 32 tokens padded).  With N > 1 (launched under torch.distributed.run, one
rank per GPU) every rank holds its own 384 rows that share the pair bias; the bias gradient is
all-reduced over NCCL inside the timed region ("weak" scaling: per-GPU work is fixed).

Prints ONE JSON line (rank 0).  `value` is algorithmic TFLOP/s (14*B*N*H*L^2*D per step) of the whole
job with inputs resident in HBM; `e2e` is the same metric through the public operator with pinned
HOST buffers, host<->device copies inside the timed region.  Each of the K timed steps repeats the
forward + backward pass often enough for the timed region to last about a second (`config.inner_repeats`;
`ms_per_step` stays the time of ONE pass), so that the clocks are those of sustained load.
`config.strong_L768` is the strong-scaling case (768 rows of L = 768 split over the ranks) and
`config.block_L768_ms` the long-crop block, both measured in the same run.  `--impl reference` times the
reference's PyTorch path (restated in oracle/) on the host cores on a bounded sample of the rows.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

L, H, D, ROWS = 384, 4, 32, 384
METRIC, UNIT = "triangle_attention_fwd_bwd_throughput", "TFLOP/s"


def profiled_dram_bytes(kernel):
    """dram__bytes_read.sum + dram__bytes_write.sum of one launch of `kernel` at the benchmark size, parsed from the
    ncu summary committed under profiles/ (None when there is none): measured by ncu, not in this run."""
    import glob
    import re
    for path in sorted(glob.glob(os.path.join(ROOT, "profiles", f"{kernel}_cfg2_L384.md"))):
        m = re.search(r"dram__bytes_read\.sum \+ dram__bytes_write\.sum\D+([0-9.]+)\s*MB", open(path).read())
        if m:
            return float(m.group(1)) * 1e6
    return None


def flops_per_step(rows):
    return 14.0 * rows * H * L * L * D          # 2 matmuls forward + 5 backward, 2*rows*H*L*L*D each


def algorithmic_bytes(rows, es=2):
    """Each tensor touched once per pass: fwd reads q,k,v,bias,mask and writes o,lse; bwd reads
    q,k,v,o,dO,lse,bias,mask and writes dq,dk,dv,dbias."""
    t = rows * L * H * D * es
    bias = H * L * L * es
    lse = rows * H * L * 4
    return (3 * t + bias + t + lse) + (5 * t + lse + bias + 3 * t + H * L * L * 4)


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(tflops=d["bf16_tflops"], tflops_sustained=d.get("bf16_tflops_sustained"), hbm=d["hbm_gbs"], src="measured")
    return dict(tflops=1590.0, tflops_sustained=1400.0, hbm=6650.0, src="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i] == "Active" for r in self.rows)]
        mx = max(int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit())
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": mx, "reasons": reasons, "samples": len(sm)}


def cpu_baseline(sample_rows=32, reps=2):
    """The reference's PyTorch attention (oracle restatement, fp32) on the host cores, forward+backward,
    on `sample_rows` of the 384 rows (rows are independent, so time scales linearly in rows)."""
    from megafold_b200 import workloads
    from oracle import pairformer_oracle as orc
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    c = workloads.triangle_attention(L=L, N=sample_rows, H=H, D=D)
    f = {k: (v.float() if v.is_floating_point() else v) for k, v in c.items()}
    orc.evo_attention_fwd_bwd(f["q"], f["k"], f["v"], f["mask"], f["bias"], f["d_out"])      # warm-up
    t0 = time.perf_counter()
    for _ in range(reps):
        orc.evo_attention_fwd_bwd(f["q"], f["k"], f["v"], f["mask"], f["bias"], f["d_out"])
    dt = (time.perf_counter() - t0) / reps
    return {"value": flops_per_step(sample_rows) / dt / 1e12, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"{sample_rows} of {ROWS} rows at L={L}, fp32 torch on CPU, fwd+bwd, {reps} reps",
            "seconds_per_sample": dt}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rows = 16
    from megafold_b200 import workloads
    from oracle import pairformer_oracle as orc
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    c = workloads.triangle_attention(L=L, N=rows, H=H, D=D)
    f = {k: (v.float() if v.is_floating_point() else v) for k, v in c.items()}
    step = lambda: orc.evo_attention_fwd_bwd(f["q"], f["k"], f["v"], f["mask"], f["bias"], f["d_out"])  # noqa: E731
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    val = flops_per_step(rows) / dt / 1e12
    sample = f"each step = {rows} of {ROWS} rows at L={L} (rows are independent), fp32 torch on {cores} host threads"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3 * ROWS / rows, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "cfg2_triangle_L384 (reference PyTorch attention path on CPU)", "rows_per_step": rows,
                   "L": L, "H": H, "D": D, "note": "ms_per_step is extrapolated linearly to the full 384 rows"},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_ours(args):
    import torch.distributed as dist
    import megafold_b200 as mfb
    from megafold_b200 import _lib, workloads
    from megafold_b200.sharded import evo_attention_backward_sharded, row_shard

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the operators have no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    host = workloads.triangle_attention(L=L, N=ROWS, H=H, D=D, seed=rank)      # the metric's workload: always 384 rows per GPU
    host["bias"] = workloads.triangle_attention(L=L, N=1, H=H, D=D, seed=0)["bias"]     # shared by all ranks
    pinned = {k: v.pin_memory() for k, v in host.items()}
    c = {k: v.to(dev) for k, v in host.items()}

    def fwd_bwd(t):
        """One pass on device-resident tensors; with several ranks dBias is all-reduced on a side stream while dQ / dK / dV
        are computed (the collective is inside the timed region)."""
        o, lse = mfb.evo_attention_forward(t["q"], t["k"], t["v"], t["mask"], t["bias"])
        dq, dk, dv, db = evo_attention_backward_sharded(t["d_out"], t["q"], t["k"], t["v"], t["mask"], t["bias"], o, lse)
        return o, dq, dk, dv, db

    out_host = None

    def step_e2e():
        """The public call for host-resident operands: pinned inputs in, pinned results out."""
        nonlocal out_host
        out = mfb.evoformer_fwd_bwd_host(pinned["q"], pinned["k"], pinned["v"], pinned["mask"], pinned["bias"], pinned["d_out"],
                                         device=dev, group=dist.group.WORLD if world > 1 else None)
        out_host = list(out.values())
        return out

    def timed(fn, steps, warmup, sampler=None, inner=1):
        """`steps` timed steps of `inner` calls each, CUDA events on the launching stream, max over ranks; ms per call."""
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ctx = sampler if sampler is not None else _Null()
        with ctx:
            e0.record()
            for _ in range(steps * inner):
                fn()
            e1.record()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
        ms = e0.elapsed_time(e1) / (steps * inner)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    # how many passes per step make the timed region last about a second (same number on every rank)
    probe_ms = timed(lambda: fwd_bwd(c), 5, 3)
    inner = max(1, min(400, int(round(1000.0 / (args.steps * probe_ms)))))
    sampler = ClockSampler(local) if rank == 0 else None
    launches0 = _lib.launch_count()
    ms = timed(lambda: fwd_bwd(c), args.steps, args.warmup, sampler, inner)
    launches = (_lib.launch_count() - launches0) * args.steps * inner // (args.steps * inner + args.warmup)
    path_bwd = _lib.last_path()
    status = _lib.lib().mf_async_status()
    ms_e2e = timed(step_e2e, max(2, min(args.steps, 5)), 2)

    # per-kernel-family timing on the launching stream: forward call and backward call separately
    o, lse = mfb.evo_attention_forward(c["q"], c["k"], c["v"], c["mask"], c["bias"])
    path_fwd = _lib.last_path()
    ms_fwd = timed(lambda: mfb.evo_attention_forward(c["q"], c["k"], c["v"], c["mask"], c["bias"]), args.steps, 3, None, inner)
    ms_bwd = timed(lambda: mfb.evo_attention_backward(c["d_out"], c["q"], c["k"], c["v"], c["mask"], c["bias"], o, lse),
                   args.steps, 3, None, inner)
    del o, lse

    # strong scaling: 768 rows of L = 768 (H 4, D 32) split over the ranks, dBias all-reduced
    L2 = 768
    a, b = row_shard(L2, rank, world)
    big = workloads.triangle_attention(L=L2, N=L2, H=H, D=D, pad=38, seed=1)
    s = {k: (v[:, a:b].to(dev) if k != "bias" else v.to(dev)) for k, v in big.items()}
    del big
    ms_strong = timed(lambda: fwd_bwd(s), 5, 3)
    strong = {"ms": ms_strong, "tflops": 14.0 * L2 * H * L2 * L2 * D / (ms_strong * 1e-3) / 1e12, "rows_per_gpu": b - a,
              "note": "triangle attention fwd+bwd, N = L = 768, H = 4, D = 32, rows split over the ranks, dBias all-reduce inside"}
    del s
    torch.cuda.empty_cache()
    # the long-crop block (benchmark configuration 5) at L = 768, rows sharded the same way
    ms_block = block_bench(dev, 768, group=dist.group.WORLD if world > 1 else None)
    if world > 1:
        t = torch.tensor([ms_block], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_block = float(t.item())

    if rank != 0:
        _teardown(world)
        return
    peaks = measured_peaks()
    total_rows = ROWS * world
    value = flops_per_step(total_rows) / (ms * 1e-3) / 1e12
    e2e_value = flops_per_step(total_rows) / (ms_e2e * 1e-3) / 1e12
    h2d = sum(v.numel() * v.element_size() for v in pinned.values())
    d2h = sum(t.numel() * t.element_size() for t in out_host)
    clocks = sampler.summary() if sampler else None
    # dominant kernel family = the slower of the two calls; the roofline that bounds it: the tensor pipe by the
    # benchmark's FLOP convention.  The timed region lasts about a second, so the sustained peak is the denominator.
    dom = "backward" if ms_bwd >= ms_fwd else "forward"
    dom_ms = max(ms_bwd, ms_fwd)
    dom_flops = (10.0 if dom == "backward" else 4.0) * ROWS * H * L * L * D
    achieved = dom_flops / (dom_ms * 1e-3) / 1e12
    peak = peaks["tflops_sustained"] or peaks["tflops"]
    cfg = {"workload": "cfg2_triangle_L384", "B": 1, "rows_per_gpu": ROWS, "L": L, "H": H, "D": D,
           "pad_tokens": 32, "l2": "inputs+outputs of one pass (~490 MB) exceed the 126 MB L2",
           "inner_repeats": inner, "timed_region_s": ms * args.steps * inner * 1e-3,
           "parallelism": f"rows sharded over {world} GPU(s); dBias all-reduced (NCCL) on a side stream while dQ/dK/dV are computed" if world > 1 else "single GPU",
           "kernel_path": {"forward": path_fwd, "backward": path_bwd}, "ms_forward": ms_fwd, "ms_backward": ms_bwd,
           "ms_times_sm_mhz": (ms * clocks["sm_mhz"] if clocks and clocks.get("sm_mhz") else None),
           "hbm_gbs_algorithmic": algorithmic_bytes(ROWS) / (ms * 1e-3) / 1e9, "peaks": peaks["src"],
           "strong_L768": strong, "block_L768_ms": ms_block, "block_L768_tflops": block_flops(768) / (ms_block * 1e-3) / 1e12,
           "async_status": status}
    kern = "evo_bwd_ws_kernel" if dom == "backward" else "evo_fwd_ws_kernel"
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": cfg,
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": ms_e2e, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": int(launches),
        "roofline": {"bound": "tensor", "kernel": f"attention {dom} call ({path_bwd if dom == 'backward' else path_fwd}); largest kernel {kern}",
                     "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                     # dram__bytes_read.sum + dram__bytes_write.sum of one launch of the call's largest kernel at this size,
                     # from the ncu capture summarised under profiles/ (measured by ncu, not in this run)
                     "traffic": (profiled_dram_bytes(kern) if ROWS == 384 else None), "traffic_unit": "bytes per launch",
                     "peak_source": peaks["src"] + " bf16 sustained (the timed region lasts ~1 s)"},
        "cpu_baseline": cpu_baseline() if world == 1 else None,
    }
    if world == 1 and not args.no_extras:
        line["parity"] = parity_cfg2(c, dev)
        del c
        torch.cuda.empty_cache()
        line["extras"] = extras(dev)
    print(json.dumps(line), flush=True)
    _teardown(world)


def _teardown(world):
    """Leave the process group in an orderly way: CUDA graphs that captured NCCL collectives (host pipeline, block) must
    be gone before the communicator is destroyed.  A timer ends the process if the teardown itself blocks."""
    if world <= 1:
        return
    import gc
    from megafold_b200 import host_pipeline
    timer = threading.Timer(60.0, lambda: os._exit(0))
    timer.daemon = True
    timer.start()
    host_pipeline._cache.clear()
    gc.collect()
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()
    timer.cancel()


def parity_cfg2(c, dev):
    """Largest absolute / relative error of every output of the benchmark pass against the fp32 oracle evaluated on the
    GPU (TF32 off) on the same bf16 inputs: the oracle is the checker here, nothing of it is timed."""
    import megafold_b200 as mfb
    from oracle import pairformer_oracle as orc
    tf32 = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        o, lse = mfb.evo_attention_forward(c["q"], c["k"], c["v"], c["mask"], c["bias"])
        got = (o,) + tuple(mfb.evo_attention_backward(c["d_out"], c["q"], c["k"], c["v"], c["mask"], c["bias"], o, lse))
        ref = orc.evo_attention_fwd_bwd(c["q"].float(), c["k"].float(), c["v"].float(), c["mask"], c["bias"].float(), c["d_out"].float())
        out = {"tolerance": "rtol = atol = 2e-2 (atol x sqrt(384) for d_pair_bias, a sum over the 384 rows)"}
        for n, g_, r_ in zip(("o", "dq", "dk", "dv", "d_pair_bias"), got, ref):
            err = (g_.float() - r_).abs()
            big = r_.abs() > 0.1 * r_.abs().max()
            atol = 2e-2 * (384 ** 0.5 if n == "d_pair_bias" else 1.0)
            out[n] = {"max_abs_err": float(err.max()), "max_rel_err_large": float((err[big] / r_.abs()[big]).max()),
                      "within_tolerance": bool((err <= atol + 2e-2 * r_.abs()).all())}
        return out
    finally:
        torch.backends.cuda.matmul.allow_tf32 = tf32


def _time_cuda(fn, steps, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def run_only(args):
    """One kernel family in a loop on a (small) case: the command ncu captures are taken from."""
    import megafold_b200 as mfb
    from megafold_b200 import workloads
    from megafold_b200.fused_layernorm_linear import layernorm_linear_backward, layernorm_linear_forward
    from megafold_b200.fused_transition import transition_backward, transition_forward
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    if args.only in ("fwd", "bwd", "step", "single_step"):
        # single_step: configuration 3 (single-representation attention: one row, sixteen heads of 24, L = 768)
        c = {k: v.to(dev) for k, v in (workloads.single_attention() if args.only == "single_step"
                                       else workloads.triangle_attention(L=L, N=args.rows, H=H, D=D)).items()}
        o, lse = mfb.evo_attention_forward(c["q"], c["k"], c["v"], c["mask"], c["bias"])
        if args.only == "fwd":
            fn = lambda: mfb.evo_attention_forward(c["q"], c["k"], c["v"], c["mask"], c["bias"])            # noqa: E731
        elif args.only in ("step", "single_step"):
            def fn():
                o2, lse2 = mfb.evo_attention_forward(c["q"], c["k"], c["v"], c["mask"], c["bias"])
                mfb.evo_attention_backward(c["d_out"], c["q"], c["k"], c["v"], c["mask"], c["bias"], o2, lse2)
        else:
            fn = lambda: mfb.evo_attention_backward(c["d_out"], c["q"], c["k"], c["v"], c["mask"], c["bias"], o, lse)  # noqa: E731
    elif args.only in ("lnl", "lnl_bwd"):
        c = {k: (v.to(dev) if v is not None else None) for k, v in workloads.layernorm_linear(M=args.rows * L).items()}
        fn = lambda: layernorm_linear_forward(c["x"], c["w"], c["b"], c["ln_w"], c["ln_b"])                   # noqa: E731
        if args.only == "lnl_bwd":
            _, mean, rstd = fn()
            fn = lambda: layernorm_linear_backward(c["d_out"], c["x"], c["w"], c["ln_w"], c["ln_b"], mean, rstd, True)  # noqa: E731
    elif args.only == "block":
        # strong scaling of the long-crop block: rows of the pair representation sharded over the ranks
        world = int(os.environ.get("WORLD_SIZE", "1"))
        if world > 1:
            dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
            torch.cuda.set_device(dev)
            dist.init_process_group("nccl", device_id=dev)
        ms = block_bench(dev, args.L, args.steps, args.warmup, graphed=not args.no_graph)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t)
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"workload": f"cfg5_pairformer_block_L{args.L}", "n_gpus": world, "scaling": "strong",
                              "ms_fwd_bwd": ms, "tflops": block_flops(args.L) / (ms * 1e-3) / 1e12,
                              "cuda_graph": bool(getattr(block_bench, "graphed", False))}))
        _teardown(world)
        return
    else:
        c = {k: v.to(dev) for k, v in workloads.transition(M=args.rows * L).items()}
        fn = lambda: transition_forward(c["x"], c["ln_w"], c["ln_b"], c["w1"], c["w2"])                       # noqa: E731
        if args.only == "transition_bwd":
            _, mean, rstd = fn()
            fn = lambda: transition_backward(c["d_out"], c["x"], c["ln_w"], c["ln_b"], c["w1"], c["w2"], mean, rstd)  # noqa: E731
    ms = _time_cuda(fn, args.steps, args.warmup)
    print(f"{args.only}: rows={args.rows} {ms * 1e3:.1f} us per call")


def extras(dev, steps=5):
    """Secondary workloads of the path (benchmark configurations 3 and 4 and the LayernormLinear around configuration 2):
    CUDA-event timings with inputs resident in HBM, a few repetitions each."""
    import megafold_b200 as mfb
    from megafold_b200 import _lib, workloads
    from megafold_b200.fused_layernorm_linear import layernorm_linear_backward, layernorm_linear_forward
    from megafold_b200.fused_transition import transition_backward, transition_forward
    peaks = measured_peaks()
    out = {}
    # same-box comparator: the reference's PyTorch attention path (oracle restatement) in bf16 on this GPU, torch eager
    try:
        from oracle import pairformer_oracle as orc
        c = {k: v.to(dev) for k, v in workloads.triangle_attention().items()}
        eager = lambda: orc.evo_attention_fwd_bwd(c["q"], c["k"], c["v"], c["mask"], c["bias"], c["d_out"], compute_dtype=torch.bfloat16)  # noqa: E731
        ms_e = _time_cuda(eager, 3, 2)
        out["torch_eager_gpu_cfg2"] = {"ms_fwd_bwd": ms_e, "tflops": flops_per_step(ROWS) / (ms_e * 1e-3) / 1e12,
                                       "note": "PyTorch eager bf16 on the same GPU: einsum, masked_fill, softmax, einsum + autograd"}
        del c
        torch.cuda.empty_cache()
    except Exception as e:      # noqa: BLE001
        out["torch_eager_gpu_cfg2"] = {"error": f"{type(e).__name__}: {e}"}
    # config 3: single-representation attention with pair bias, D = 24
    c = {k: v.to(dev) for k, v in workloads.single_attention().items()}
    o, lse = mfb.evo_attention_forward(c["q"], c["k"], c["v"], c["mask"], c["bias"])
    pf = _lib.last_path()
    ms_f = _time_cuda(lambda: mfb.evo_attention_forward(c["q"], c["k"], c["v"], c["mask"], c["bias"]), steps, 2)
    ms_b = _time_cuda(lambda: mfb.evo_attention_backward(c["d_out"], c["q"], c["k"], c["v"], c["mask"], c["bias"], o, lse), steps, 2)
    B3, _, L3, H3, D3 = c["q"].shape
    bytes3 = 2 * c["bias"].numel() * 2 + c["bias"].numel() * 2 + 8 * c["q"].numel() * 2      # bias read twice, dBias written, q/k/v/o/dO/dq/dk/dv
    out["cfg3_single_attention_L768_D24"] = {
        "ms_forward": ms_f, "ms_backward": ms_b, "path_forward": pf, "path_backward": _lib.last_path(),
        "tflops": 14.0 * B3 * H3 * L3 * L3 * D3 / ((ms_f + ms_b) * 1e-3) / 1e12,
        "hbm_gbs_algorithmic": bytes3 / ((ms_f + ms_b) * 1e-3) / 1e9, "hbm_frac_of_measured": bytes3 / ((ms_f + ms_b) * 1e-3) / 1e9 / peaks["hbm"]}
    del c, o, lse
    # the shape of the reference's own kernel benchmark (B = 4, H = 32, D = 64, one row, L = 384, 16-bit): forward on the
    # general tensor-core kernel, backward on the warp-specialised kernels with the head size taken as two halves of 32
    c = {k: v.to(dev) for k, v in workloads.single_attention(L=384, H=32, D=64, B=4, drop=0.0).items()}
    o, lse = mfb.evo_attention_forward(c["q"], c["k"], c["v"], c["mask"], c["bias"])
    pf = _lib.last_path()
    ms_f = _time_cuda(lambda: mfb.evo_attention_forward(c["q"], c["k"], c["v"], c["mask"], c["bias"]), steps, 2)
    ms_b = _time_cuda(lambda: mfb.evo_attention_backward(c["d_out"], c["q"], c["k"], c["v"], c["mask"], c["bias"], o, lse), 3, 1)
    fl = 4.0 * 4 * 32 * 384 * 384 * 64
    out["reference_benchmark_shape_B4_H32_D64_L384"] = {
        "ms_forward": ms_f, "ms_backward": ms_b, "path_forward": pf, "path_backward": _lib.last_path(),
        "tflops_forward": fl / (ms_f * 1e-3) / 1e12, "tflops_backward": 2.5 * fl / (ms_b * 1e-3) / 1e12,
        "tflops_fwd_bwd": 3.5 * fl / ((ms_f + ms_b) * 1e-3) / 1e12,
        "reference_comment_block": "Triton fp16 at L=384: 40.7 fwd / 11.2 bwd / 14.0 fwd+bwd TFLOP/s, hardware not stated "
                                   "(benchmarks/evoattention_speed.py:123-153)"}
    del c, o, lse
    # LayernormLinear 128 -> 512 on the [384*384, 128] pair representation (the projection around config 2)
    c = {k: (v.to(dev) if v is not None else None) for k, v in workloads.layernorm_linear().items()}
    y, mean, rstd = layernorm_linear_forward(c["x"], c["w"], c["b"], c["ln_w"], c["ln_b"])
    pf = _lib.last_path()
    ms_f = _time_cuda(lambda: layernorm_linear_forward(c["x"], c["w"], c["b"], c["ln_w"], c["ln_b"]), steps, 2)
    ms_b = _time_cuda(lambda: layernorm_linear_backward(c["d_out"], c["x"], c["w"], c["ln_w"], c["ln_b"], mean, rstd, True), 2, 1)
    M, K = c["x"].shape
    N = c["w"].shape[1]
    fwd_bytes = (M * K + M * N + K * N) * 2
    out["layernorm_linear_147456x128x512"] = {
        "ms_forward": ms_f, "ms_backward": ms_b, "path_forward": pf, "path_backward": _lib.last_path(),
        "forward_hbm_gbs": fwd_bytes / (ms_f * 1e-3) / 1e9, "forward_hbm_frac_of_measured": fwd_bytes / (ms_f * 1e-3) / 1e9 / peaks["hbm"],
        "forward_tflops": 2.0 * M * K * N / (ms_f * 1e-3) / 1e12}
    del c, y, mean, rstd
    # config 4: Transition on [512*512, 128], expansion 4
    torch.cuda.empty_cache()
    c = {k: v.to(dev) for k, v in workloads.transition().items()}
    torch.cuda.reset_peak_memory_stats(dev)
    base = torch.cuda.memory_allocated(dev)
    y, mean, rstd = transition_forward(c["x"], c["ln_w"], c["ln_b"], c["w1"], c["w2"])
    pf = _lib.last_path()
    transition_backward(c["d_out"], c["x"], c["ln_w"], c["ln_b"], c["w1"], c["w2"], mean, rstd)
    torch.cuda.synchronize()
    peak = torch.cuda.max_memory_allocated(dev) - base
    ms_f = _time_cuda(lambda: transition_forward(c["x"], c["ln_w"], c["ln_b"], c["w1"], c["w2"]), steps, 2)
    ms_b = _time_cuda(lambda: transition_backward(c["d_out"], c["x"], c["ln_w"], c["ln_b"], c["w1"], c["w2"], mean, rstd), 2, 1)
    M, dim = c["x"].shape
    inner = c["w2"].shape[1]
    f_fwd = 2.0 * M * dim * 2 * inner + 2.0 * M * inner * dim
    out["cfg4_transition_512x512x128"] = {
        "ms_forward": ms_f, "ms_backward": ms_b, "path_forward": pf, "path_backward": _lib.last_path(),
        "forward_tflops": f_fwd / (ms_f * 1e-3) / 1e12, "forward_frac_of_measured_bf16_peak": f_fwd / (ms_f * 1e-3) / 1e12 / peaks["tflops"],
        "fwd_bwd_tflops": 3.0 * f_fwd / ((ms_f + ms_b) * 1e-3) / 1e12,
        "peak_extra_memory_mb_fwd_bwd": peak / 2 ** 20,
        "note": "forward keeps the hidden activation on chip; backward recomputes it (workspace counted in the peak)"}
    del c, y, mean, rstd
    torch.cuda.empty_cache()
    return out


def block_flops(Lb):
    """Algorithmic fwd+bwd FLOPs of the long-crop block: attention 14*N*H*L^2*D, GEMMs 3 * 2*M*K*N."""
    M = Lb * Lb
    tri = 14.0 * Lb * 4 * Lb * Lb * 32 + 6.0 * M * 128 * (512 + 4 + 128)
    single = 14.0 * 16 * Lb * Lb * 24 + 6.0 * M * 128 * 16 + 6.0 * Lb * 384 * (4 * 384 + 384)
    return 2 * tri + 6.0 * M * 128 * (1024 + 512) + single


def block_bench(dev, Lb=768, steps=3, warmup=2, group=None, graphed=True):
    """Benchmark configuration 5: one Pairformer block (two triangle attentions, pair transition, single attention with
    pair bias) forward + backward in bf16 on this rank's rows of a [L, L, 128] pair representation (rows sharded
    over the process group, 5 % padding at the tail).  Returns ms per step (max over ranks is the caller's job)."""
    from megafold_b200 import row_shard
    from megafold_b200.pairformer_block import PairformerBlock
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    torch.manual_seed(0)
    m = PairformerBlock(device=dev, dtype=torch.bfloat16, group=group)
    g = torch.Generator().manual_seed(1)
    a, b = row_shard(Lb, rank, world)
    pair = torch.randn(Lb, Lb, 128, generator=g)[a:b].to(dev, torch.bfloat16).requires_grad_(True)
    single = torch.randn(Lb, 384, generator=g).to(dev, torch.bfloat16).requires_grad_(True)
    mask = torch.ones(Lb, dtype=torch.bool, device=dev)
    mask[Lb - (Lb + 19) // 20:] = False
    d_pair = torch.randn(b - a, Lb, 128, device=dev, dtype=torch.bfloat16)
    d_single = torch.randn(Lb, 384, device=dev, dtype=torch.bfloat16)

    def step():
        for t in (pair, single, *m.parameters()):
            t.grad = None
        x, s2 = m(pair, single, mask)
        torch.autograd.backward([x, s2], [d_pair, d_single])

    # A block is a few hundred launches and a handful of collectives; with the rows spread over 8 GPUs the host
    # issues them more slowly than the GPUs run them.  So the step is recorded once into a CUDA graph (kernels of the
    # library, torch glue and NCCL collectives alike) and the timed steps replay it; if the capture is refused the
    # step is issued directly.
    graph = None
    if graphed:
        try:
            side = torch.cuda.Stream(dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                for _ in range(2):
                    step()
            torch.cuda.current_stream(dev).wait_stream(side)
            torch.cuda.synchronize(dev)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step()
        except Exception as e:          # noqa: BLE001
            graph = None
            torch.cuda.synchronize(dev)
            print(f"[bench] CUDA graph capture of the block failed ({type(e).__name__}: {e}); issuing the step directly", file=sys.stderr)
    ok = torch.tensor([1 if graph is not None else 0], device=dev)
    if world > 1:
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)         # every rank replays, or none
    if not int(ok):
        graph = None
    block_bench.graphed = graph is not None
    return _time_cuda(graph.replay if graph is not None else step, steps, warmup)


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--rows", type=int, default=ROWS, help="rows (N) per GPU; smaller values give profiler-sized cases")
    ap.add_argument("--only", default="all", choices=["all", "fwd", "bwd", "step", "single_step", "lnl", "lnl_bwd", "transition", "transition_bwd", "block"],
                    help="run just one kernel family in the timed loop (for ncu captures); prints no JSON line")
    ap.add_argument("--L", type=int, default=768, help="crop length of --only block")
    ap.add_argument("--no-graph", action="store_true", help="--only block: issue the step directly instead of replaying a CUDA graph")
    ap.add_argument("--no-extras", action="store_true", help="skip the secondary workloads (cfg 3, cfg 4, LayernormLinear)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else max(args.warmup, 1)
    if args.impl == "reference":
        run_reference(args)
    elif args.only != "all":
        run_only(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
