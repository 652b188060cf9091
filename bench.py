#!/usr/bin/env python
"""Benchmark of the DP-Linear backward hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl native|reference] [--workload NAME]

A step is one DP backward of one Linear layer on one batch of synthetic input:
    dW = (1/B) sum_b clip(G_b^T X_b) + N(0, (sigma/sqrt(B))^2)      (fdp_linear_wgrad)
    dX = G W                                                        (fdp_linear_dgrad)
and, on N > 1 GPUs (one process per GPU, the batch sharded, B samples per rank), an NCCL all-reduce
of the clipped sums.  The metric is algorithmic TFLOP/s: 4*B*T*in*out per rank and step.
Rank 0 prints one JSON line.  On the default workload the same run then times the GPT-2-medium DP
training step on the same ranks and adds it to the line as "gpt2_medium", and an untimed check that
the N-rank result equals a single-rank evaluation of the concatenated batch ("parity_check").
`--impl reference` times the CPU port of the reference's pure-PyTorch per-sample path on the host
cores instead (rank 0 only), a step being the whole batch of the workload.
`--workload llama7b_shaped` runs a Llama-2-7B-shaped decoder with every Linear but lm_head wrapped.
"""
import argparse
import contextlib
import ctypes
import datetime
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (B per GPU, T, in, out, dtype, g_scale)
    "linear_bf16_b32_t1024_4096x4096": (32, 1024, 4096, 4096, "bf16", 1e-3),
    "conv1d_bf16_b16_t1024_1024x3072": (16, 1024, 1024, 3072, "bf16", 1e-3),
    "linear_bf16_b8_t1024_1024x3072": (8, 1024, 1024, 3072, "bf16", 1e-3),     # a GPT-2-medium c_attn call
    "linear_bf16_b4_t2048_4096x4096": (4, 2048, 4096, 4096, "bf16", 1e-3),     # a Llama-2-7B attention projection
    "linear_fp32_b4_t128_768x768": (4, 128, 768, 768, "f32", 1e-2),
    "linear_fp32_b8_t1024_4096x4096": (8, 1024, 4096, 4096, "f32", 1e-2),      # fp32 weights at the config-2 layer size
    "small_bf16_b4_t256_512x512": (4, 256, 512, 512, "bf16", 1e-3),
}
DEFAULT_WORKLOAD = "linear_bf16_b32_t1024_4096x4096"
METRIC, UNIT = "dp_linear_bwd_tflops", "TFLOP/s"
# dram__bytes_read.sum + dram__bytes_write.sum of one clipped-sum GEMM launch, from an ncu capture of
# this workload (bytes per launch)
TRAFFIC = {"linear_bf16_b32_t1024_4096x4096": 1.429e9}
NOMINAL_BF16_TFLOPS = 2250.0


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(bf16=p["bf16_tflops"], bf16_sustained=p.get("bf16_tflops_sustained", p["bf16_tflops"]),
                    hbm=p["hbm_gbs"], source="measured")
    return dict(bf16=1590.0, bf16_sustained=1400.0, hbm=6650.0, source="fallback")


def flops_bwd(B, T, n_in, n_out):
    return 4.0 * B * T * n_in * n_out


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples (20 ms period) with their wall-clock stamps, so the
    ones that fall inside a timed region can be picked out afterwards."""
    Q = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, gpu_index):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                       "-lms", "20", "-i", str(gpu_index)], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.p = None

    def wait_first_sample(self, limit_s=5.0):
        t0 = time.time()
        while self.p is not None and time.time() - t0 < limit_s:
            if os.path.getsize(self.f.name) > 0:
                return True
            time.sleep(0.02)
        return False

    def stop(self, windows):
        """windows: list of (t_start, t_end) wall-clock pairs; samples inside any of them count."""
        import datetime
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.p is None:
            return out
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except Exception:
            self.p.kill()
        self.f.flush()
        self.f.seek(0)
        sm, mx, reasons, power = [], [], set(), []
        for line in self.f.read().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                ts = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                clk, clk_max = float(parts[1]), float(parts[2])
            except ValueError:
                continue
            if not any(a <= ts <= b for a, b in windows):
                continue
            sm.append(clk)
            mx.append(clk_max)
            try:
                power.append(float(parts[3]))
            except ValueError:
                pass
            for name, val in zip(self.NAMES, parts[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.f.name)
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm),
                       power_w_max=max(power) if power else None)
        return out


def cpu_port_rate(T, n_in, n_out, dtype_name, budget_s, sample_b=2, steps=None, warmup=1):
    """TFLOP/s of the reference's per-sample path (CPU port in oracle/) on a bounded sample."""
    import torch
    from oracle import dp_oracle as O
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    dt = torch.bfloat16 if dtype_name == "bf16" else torch.float32
    X, G, W = O.make_linear_inputs(sample_b, T, n_in, n_out, 1e-3, seed=0, dtype=dt)
    for _ in range(warmup):
        O.torch_port_linear_backward(G, X, W, 1.0, 1.0, 1.0, False)
    times = []
    t_start = time.perf_counter()
    while True:
        t0 = time.perf_counter()
        O.torch_port_linear_backward(G, X, W, 1.0, 1.0, 1.0, False)
        times.append(time.perf_counter() - t0)
        if steps is not None:
            if len(times) >= steps:
                break
        elif time.perf_counter() - t_start > budget_s and len(times) >= 3:
            break
    med = statistics.median(times)
    return dict(value=flops_bwd(sample_b, T, n_in, n_out) / med / 1e12, unit=UNIT, cores=cores, kind="port",
                sample=f"{sample_b} of the workload's samples per step (T={T}, {n_in}->{n_out}, {dtype_name}), "
                       f"median of {len(times)} steps, torch CPU ops as the reference issues them",
                ms_per_step=med * 1e3, steps=len(times))


def workload_config(args, wl, world, l2_note):
    B, T, n_in, n_out, dtn, _ = wl
    return {"workload": args.workload, "B_per_gpu": B, "T": T, "in": n_in, "out": n_out,
            "C": 1.0, "noise_multiplier": args.sigma, "bias": False, "grad_dtype": "f32",
            "flops_per_step_per_gpu": flops_bwd(B, T, n_in, n_out), "l2": l2_note,
            "parallelism": f"dp{world}" + (" + NCCL all-reduce of dW" if world > 1 else "")}


def run_reference(args, wl):
    """The reference arm: the per-sample path on the host cores, one step = the workload's whole batch
    (all B samples of one rank), all host threads.  Rank 0 alone works."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    B, T, n_in, n_out, dtn, _ = wl
    base = cpu_port_rate(T, n_in, n_out, dtn, budget_s=0, sample_b=B, steps=max(1, args.steps),
                         warmup=max(1, args.warmup))
    line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": base["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dtn, "data": "synthetic",
            "config": workload_config(args, wl, 1, "host memory"),
            "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def dist_setup():
    """(rank, local_rank, world, device); one NCCL process group per process when launched by torchrun."""
    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1 and not dist.is_initialized():
        # a short collective timeout: a rank that falls out of step ends the job in minutes, not hours
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
    return rank, local_rank, world, dev


def parity_check(dev, rank, world):
    """Untimed: does the N-rank job reproduce the single-rank gradient of the concatenated batch?

    Every rank generates all the shards (seed = shard index), runs its own through the library with
    divisor world*B and its share of the noise, and the results are all-reduced (SUM).  Rank 0 then
    evaluates the concatenated batch alone and compares: sigma = 0 -> max|a-b| / max|b| (the sums
    differ only in fp32 association); zero gradient with sigma = 1 -> the noise tensors must be
    bit-equal (each element is drawn by exactly one rank and the others add exact zeros)."""
    import torch
    import torch.distributed as dist
    from flashdp4review_b200.core import ops
    B, T, n_in, n_out = 4, 512, 1024, 768
    shards = []
    for r in range(world):
        gen = torch.Generator().manual_seed(1000 + r)
        shards.append((torch.randn(B, T, n_in, generator=gen).to(torch.bfloat16),
                       (torch.randn(B, T, n_out, generator=gen) * 1e-3).to(torch.bfloat16)))
    X, G = (t.to(dev) for t in shards[rank])
    out = {}

    def sharded(Xs, Gs, sigma):
        noise = ops.NoiseSpec(std=ops.noise_std(sigma, B * world), seed=77, param_id=5, step=3, rank=rank, world=world)
        dW = ops.dp_linear_weight_grad(Xs, Gs, 1.0, 1.0, batch_divisor=B * world, noise=noise, out_dtype=torch.float32)
        if world > 1:
            dist.all_reduce(dW, op=dist.ReduceOp.SUM)
        return dW

    def single(Xa, Ga, sigma):
        noise = ops.NoiseSpec(std=ops.noise_std(sigma, B * world), seed=77, param_id=5, step=3)
        return ops.dp_linear_weight_grad(Xa, Ga, 1.0, 1.0, batch_divisor=B * world, noise=noise, out_dtype=torch.float32)

    got0 = sharded(X, G, 0.0)
    gotz = sharded(torch.zeros_like(X), torch.zeros_like(G), 1.0)
    got1 = sharded(X, G, 1.0)
    if rank == 0:
        Xa = torch.cat([x for x, _ in shards]).to(dev)
        Ga = torch.cat([g for _, g in shards]).to(dev)
        want0 = single(Xa, Ga, 0.0)
        wantz = single(torch.zeros_like(Xa), torch.zeros_like(Ga), 1.0)
        want1 = single(Xa, Ga, 1.0)
        rel = lambda a, b: float((a - b).abs().max() / b.abs().max())
        out = {"shape": f"B={B}/rank T={T} {n_in}->{n_out} bf16", "ranks": world,
               "max_rel": rel(got0, want0), "max_rel_with_noise": rel(got1, want1),
               "noise_bit_equal": bool(torch.equal(gotz, wantz)), "tolerance": 1e-2}
        out["ok"] = out["max_rel"] < 1e-2 and out["max_rel_with_noise"] < 1e-2 and out["noise_bit_equal"]
    return out


def reference_gpu_leg(args):
    """Runs `reference_gpu_child` in a process of its own and returns its JSON object: whatever the
    reference's code or its JIT compiler does on this GPU -- a compile error (caught there), a crash, a
    stall -- cannot take the bench with it."""
    cmd = [sys.executable, os.path.abspath(__file__), "--workload", args.workload, "--sigma", str(args.sigma),
           "--ref-gpu-child"]
    try:
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    except subprocess.TimeoutExpired:
        return {"unavailable": "the child process that runs the reference did not finish within 600 s"}
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    if r.returncode != 0 or not lines:
        tail = (r.stderr.strip().splitlines() or [""])[-1][:200]
        return {"unavailable": "child process exited with %d: %s" % (r.returncode, tail)}
    return json.loads(lines[-1])


def reference_gpu_child(args, wl):
    """Child of `reference_gpu_leg`: the bench's inputs (rank 0's), this library's sigma = 0 result for
    the comparison, then the reference's code; prints one JSON object."""
    import torch
    from flashdp4review_b200.core import ops
    B, T, n_in, n_out, dtn, g_scale = wl
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    dt = torch.bfloat16 if dtn == "bf16" else torch.float32
    gen = torch.Generator().manual_seed(0)
    X = torch.randn(B, T, n_in, generator=gen).to(dt).to(dev)
    G = (torch.randn(B, T, n_out, generator=gen) * g_scale).to(dt).to(dev)
    W = (torch.randn(n_out, n_in, generator=gen) * 0.02).to(dt).to(dev)
    own = ops.dp_linear_weight_grad(X, G, 1.0, 1.0, batch_divisor=B, noise=None, out_dtype=torch.float32)

    def timed(fn, steps):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)
    print(json.dumps(reference_gpu_run(X, G, W, args.sigma, timed, own)), flush=True)


def reference_gpu_run(X, G, W, sigma, timed, own_dw):
    """The UNMODIFIED reference package on this GPU, where `__graft_entry__.build()` installed it
    (`baseline/_ref`, outside the history), run on the bench's own X and G.  Context for the headline
    only: none of this library's code runs inside these timings.  Three entries, each on its own:
      stock   its `DPLinear` autograd function (flashdp/layers/linear.py:40-104) run backward -- dX product,
              `linear_weight_flashdp`, `.div_(B)`, `torch.normal` noise -- with the layer's default
              `auto_tune=True`: the runtime tuner times the Triton per-sample loop
              (flashdp/core/bmtm_clip_loop.py:162-173) against the `torch.jit.script` einsum loop
              (flashdp/core/linear_clip.py:94-104) on the first backward and keeps the faster;
      triton  the same with `auto_tune=False`, which always takes the Triton loop;
      torch_candidate  the tuner's second candidate, `_weight_grad_block_clip`, called directly and
              followed by the remaining operations of that backward, for the case that the Triton
              kernels do not compile for this GPU (then `stock` fails too: the tuner runs them first)."""
    import torch
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "flashdp")):
        return {"unavailable": "no installed reference under baseline/_ref"}
    B, T, n_in = X.shape
    n_out = G.shape[-1]
    out = {"what": "unmodified reference code for the DPLinear backward (dX + clipped dW + noise) on the same GPU",
           "unit": UNIT}

    def failure(e):
        msg = str(e).splitlines()[0][:200] if str(e) else ""
        return {"unavailable": "%s: %s" % (type(e).__name__, msg)}

    def record(ms):
        return {"value": flops_bwd(B, T, n_in, n_out) / (ms * 1e-3) / 1e12, "ms_per_step": ms}
    try:
        if ref_dir not in sys.path:
            sys.path.insert(0, ref_dir)
        import flashdp as ref
        from flashdp.core.linear_clip import _weight_grad_block_clip
    except Exception as e:
        out.update(failure(e))
        return out
    for key, auto in (("stock", True), ("triton", False)):
        try:
            layer = ref.DPLinear(n_in, n_out, bias=None, device=X.device, dtype=X.dtype, C=1.0, clamp_value=1.0,
                                 noise_multiplier=sigma, auto_tune=auto)
            xr = X.detach().requires_grad_(True)
            y = layer(xr)

            def bwd():
                return torch.autograd.grad(y, [xr, layer.weight], G, retain_graph=True)
            for _ in range(3):          # the first call runs the layer's tuner (2 x 110 loops) when it is on
                bwd()
            out[key] = record(timed(bwd, 5) / 5)
            if auto:
                fn = layer.runtime_tuner.chosen_func
                out[key]["tuner_chose"] = getattr(fn, "__name__", None) or getattr(fn, "name", None) or str(fn)
            else:
                # how far the Triton loop's clipped mean is from this library's on the same inputs; its
                # per-sample norm accumulator starts from uninitialised memory (bmtm_clip_loop.py:146), so
                # a difference is reported, not asserted (the noise differs too: compare at sigma = 0)
                layer.noise_multiplier = 0.0
                dw_ref = torch.autograd.grad(layer(xr), [layer.weight], G)[0].float()
                out[key]["max_rel_diff_vs_this_library_sigma0"] = float((dw_ref - own_dw).abs().max() / own_dw.abs().max())
            del layer, xr, y
        except Exception as e:              # e.g. Triton cannot compile the reference's kernel for this GPU
            out[key] = failure(e)
            torch.cuda.synchronize()
    try:
        clip_args = torch.tensor([1.0, 1.0], device=X.device)

        def candidate():
            dx = G @ W                                                  # flashdp/layers/linear.py:62-64
            dw = _weight_grad_block_clip(G, X, clip_args=clip_args).div_(B)
            dw.add_(torch.normal(mean=0, std=sigma / math.sqrt(B), size=dw.shape, device=dw.device, dtype=dw.dtype))
            return dx, dw
        for _ in range(3):
            candidate()
        out["torch_candidate"] = record(timed(candidate, 5) / 5)
        dw0 = _weight_grad_block_clip(G, X, clip_args=clip_args).div_(B).float()
        out["torch_candidate"]["max_rel_diff_vs_this_library_sigma0"] = float((dw0 - own_dw).abs().max() / own_dw.abs().max())
    except Exception as e:
        out["torch_candidate"] = failure(e)
    torch.cuda.synchronize()
    return out


def run_native(args, wl):
    import torch
    import torch.distributed as dist
    import flashdp4review_b200 as fdp
    from flashdp4review_b200 import _lib
    from flashdp4review_b200.core import ops

    B, T, n_in, n_out, dtn, g_scale = wl
    rank, local_rank, world, dev = dist_setup()
    if world != args.gpus and world > 1:
        args.gpus = world
    lib = _lib.load()
    _lib.check(lib.fdp_check_device(local_rank), "fdp_check_device")
    fdp.manual_seed(1234)
    fdp.set_data_parallel(rank, world)
    dt = torch.bfloat16 if dtn == "bf16" else torch.float32

    # synthetic inputs: X~N(0,1), G~N(0,g_scale^2), W~N(0,0.02^2); a different seed per rank (its shard)
    gen = torch.Generator().manual_seed(rank)
    Xh = torch.randn(B, T, n_in, generator=gen).to(dt)
    Gh = (torch.randn(B, T, n_out, generator=gen) * g_scale).to(dt)
    Wh = (torch.randn(n_out, n_in, generator=gen) * 0.02).to(dt)
    Xh, Gh = Xh.pin_memory(), Gh.pin_memory()
    X, G, W = Xh.to(dev), Gh.to(dev), Wh.to(dev)
    step_no = [0]

    # input gradient: this library's GEMM for 16-bit layers; fp32 layers keep the package default for
    # that product, cuBLAS through torch, as the reference does (flashdp/layers/linear.py:62-64)
    if dtn == "f32":
        def input_grad(Gd):
            return (Gd.reshape(-1, n_out) @ W).view(B, T, n_in)
    else:
        def input_grad(Gd):
            return ops.linear_input_grad(Gd, W, "out_in")

    def step(Xd, Gd):
        step_no[0] += 1
        noise = ops.NoiseSpec(std=ops.noise_std(args.sigma, B * world), seed=1234, param_id=1, step=step_no[0],
                              rank=rank, world=world)
        dW = ops.dp_linear_weight_grad(Xd, Gd, 1.0, 1.0, batch_divisor=B * world, noise=noise,
                                       out_dtype=torch.float32, norm_algo=args.norm_algo)
        if world == 1:
            return dW, input_grad(Gd)
        # the all-reduce of this layer's gradient runs beside the input-gradient GEMM, which leaves a few
        # SMs free for it; the norm pass and the clipped-sum GEMM above had the whole GPU
        work = dist.all_reduce(dW, op=dist.ReduceOp.SUM, async_op=True)
        with fdp.sm_reservation(args.reserve_sms):
            dX = input_grad(Gd)
        work.wait()
        return dW, dX

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    # L2 hygiene: the default workload's inputs (0.5 GB) exceed the 126 MB L2; smaller workloads
    # get the L2 overwritten by a 256 MB fill between steps, each step timed by its own event pair
    in_bytes = (X.numel() + G.numel()) * X.element_size()
    flush = None if in_bytes > 2 * 126e6 else torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed_steps(steps):
        if flush is None:
            return timed(lambda: step(X, G), steps)
        barrier()
        evs = []
        for _ in range(steps):
            flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            step(X, G)
            e1.record()
            evs.append((e0, e1))
        barrier()
        ms = torch.tensor([sum(a.elapsed_time(b) for a, b in evs)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    sampler = ClockSampler(local_rank) if rank == 0 else None
    for _ in range(max(args.warmup, 3)):
        step(X, G)
    if sampler:
        sampler.wait_first_sample()
    launches0 = lib.fdp_launch_count()
    w0 = time.time()
    total_ms = timed_steps(args.steps)
    windows = [(w0, time.time())]
    launches = lib.fdp_launch_count() - launches0
    ms_per_step = total_ms / args.steps
    value = world * flops_bwd(B, T, n_in, n_out) / (ms_per_step * 1e-3) / 1e12
    # a short timed region may see too few 20 ms clock samples: keep the same load running (untimed)
    # until about 0.6 s of it has been observed.  Every rank runs the same number of extra steps
    # (ms_per_step is the all-reduced maximum), because each step holds a collective.
    extra = 0
    if total_ms < 600.0:
        extra = int(600.0 / max(ms_per_step, 1e-3)) + 1
        w1 = time.time()
        for _ in range(extra):
            step(X, G)
        torch.cuda.synchronize()
        windows.append((w1, time.time()))
    clocks = None
    if sampler:
        clocks = sampler.stop(windows)
        clocks["window"] = "timed region" + (f" + {extra} more identical steps" if extra else "")
    # end to end: every step copies its inputs from pinned host memory and its gradient back.  The
    # copies of step i+1 run on a second stream into a second pair of device buffers while step i
    # computes (the copy engine and the SMs overlap; the PCIe transfer is the longer of the two).
    dW_host = torch.empty(n_out, n_in, dtype=torch.float32).pin_memory()
    bufs = [(X, G), (torch.empty_like(X), torch.empty_like(G))]
    copy_stream = torch.cuda.Stream(dev)
    h2d_done = [torch.cuda.Event(), torch.cuda.Event()]
    free = [torch.cuda.Event(), torch.cuda.Event()]

    def h2d(slot):
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(free[slot])
            bufs[slot][0].copy_(Xh, non_blocking=True)
            bufs[slot][1].copy_(Gh, non_blocking=True)
            h2d_done[slot].record(copy_stream)

    def e2e_run(steps):
        cur = torch.cuda.current_stream(dev)
        for f in free:
            f.record(cur)
        h2d(0)
        for i in range(steps):
            slot = i % 2
            if i + 1 < steps:
                h2d(1 - slot)
            cur.wait_event(h2d_done[slot])
            dW, dX = step(*bufs[slot])
            free[slot].record(cur)
            dW_host.copy_(dW, non_blocking=True)

    e2e_steps = max(2, min(args.steps, 10))
    e2e_run(2)
    e2e_ms = timed(lambda: e2e_run(e2e_steps), 1) / e2e_steps
    e2e_value = world * flops_bwd(B, T, n_in, n_out) / (e2e_ms * 1e-3) / 1e12
    h2d = Xh.numel() * Xh.element_size() + Gh.numel() * Gh.element_size()
    d2h = dW_host.numel() * 4

    # dominant kernel (clipped-sum GEMM) timed alone with CUDA events recorded inside the call
    pk = peaks()
    roof = None
    phases = None
    # (every rank runs these steps: each holds a collective; only rank 0 reads the phase times)
    if rank == 0:
        lib.fdp_profile_enable(1)
    # five back-to-back steps, phase times of the last one (read after the loop, so the measured step
    # ran in the same steady clock/power state as the timed region)
    acc = [[], [], [], []]
    for rep in range(3):
        for _ in range(5):
            step(X, G)
        if rank == 0:
            ms = (ctypes.c_float * 4)()
            if lib.fdp_profile_read(ms, 4) == 4:
                for i in range(4):
                    acc[i].append(ms[i])
    if rank == 0:
        lib.fdp_profile_enable(0)
        if acc[3]:
            phases = {n: statistics.mean(v) for n, v in zip(("norm_pass_ms", "clip_factors_ms", "prescale_ms",
                                                             "clipped_gemm_ms"), acc)}
            gemm_flops = 2.0 * B * T * n_in * n_out
            achieved = gemm_flops / (phases["clipped_gemm_ms"] * 1e-3) / 1e12
            # against the BURST cuBLAS figure: the phase events are read right after five back-to-back
            # steps that follow the mostly idle end-to-end leg, a burst-like window
            roof = {"kernel": "clipped-sum GEMM (tcgen05)" if dtn != "f32" else
                    ("clipped-sum GEMM (tcgen05, three bf16 products)" if fdp.fp32_mode() == "tensor"
                     else "clipped-sum GEMM (fp32 FMA)"),
                    "bound": "tensor", "achieved": achieved, "peak": pk["bf16"], "unit": "TFLOP/s",
                    "frac": achieved / pk["bf16"], "frac_of_sustained_peak": achieved / pk["bf16_sustained"],
                    "frac_of_nominal": achieved / NOMINAL_BF16_TFLOPS,
                    "peak_source": pk["source"] + " (burst cuBLAS bf16, torch.matmul 8192^3)",
                    "traffic": TRAFFIC.get(args.workload), "phases_ms": phases,
                    "wgrad_path_tflops": gemm_flops / (sum(phases.values()) * 1e-3) / 1e12}
    barrier()

    # Context: the reference's per-sample ALGORITHM (one product, norm, scale and add per sample, then
    # /B and torch.normal noise -- flashdp/core/linear_clip.py:94-104, flashdp/layers/linear.py:62-80)
    # issued as plain torch ops on this same GPU, i.e. cuBLAS and elementwise library kernels.
    gpu_loop = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        def loop_step():
            accw = torch.zeros(n_out, n_in, device=dev, dtype=X.dtype)
            for b in range(B):
                g = G[b].t() @ X[b]
                accw += g * torch.clamp(1.0 / (torch.linalg.norm(g.float()) + 1e-10), max=1.0).to(g.dtype)
            accw = accw / B + torch.randn_like(accw) * (args.sigma / math.sqrt(B))
            return accw, G.reshape(B * T, n_out) @ W
        for _ in range(3):
            loop_step()
        loop_ms = timed(loop_step, 5) / 5
        gpu_loop = {"value": flops_bwd(B, T, n_in, n_out) / (loop_ms * 1e-3) / 1e12, "unit": UNIT,
                    "ms_per_step": loop_ms, "what": "per-sample loop of torch ops (cuBLAS) on the same GPU"}

    ref_gpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline and not args.no_ref_gpu and dtn == "bf16":
        torch.cuda.synchronize()
        ref_gpu = reference_gpu_leg(args)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        full = cpu_port_rate(T, n_in, n_out, dtn, budget_s=0, sample_b=B, steps=2, warmup=1) if args.cpu_full else None
        cpu = cpu_port_rate(T, n_in, n_out, dtn, budget_s=args.cpu_budget)
        cpu = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}
        if full is not None:
            # the same path on the workload's whole batch (the per-sample loop is linear in B)
            cpu["whole_batch"] = {"value": full["value"], "ms_per_step": full["ms_per_step"], "steps": full["steps"],
                                  "samples": B}

    check = None
    if not args.no_check and dtn == "bf16":
        check = parity_check(dev, rank, world)

    line = None
    if rank == 0:
        l2_note = ("inputs (X, G: %.0f MB) larger than the 126 MB L2" % (h2d / 1e6)) if flush is None \
            else "L2 overwritten by a 256 MB fill between steps"
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": dtn, "data": "synthetic",
                "config": workload_config(args, wl, world, l2_note),
                "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                        "ms_per_step": e2e_ms, "steps": e2e_steps},
                "gpu_launches": int(launches), "clocks": clocks, "roofline": roof, "cpu_baseline": cpu,
                "step_frac_nominal": value / world / NOMINAL_BF16_TFLOPS, "step_frac_burst": value / world / pk["bf16"],
                "parity_check": check, "gpu_loop_baseline": gpu_loop, "reference_on_gpu": ref_gpu}
    # the second headline metric on the same ranks: GPT-2-medium DP training tokens/s
    if args.workload == DEFAULT_WORKLOAD and not args.no_gpt2:
        del X, G, W, bufs, flush
        torch.cuda.empty_cache()
        g = gpt2_measure(args, steps=max(args.steps, 20), with_no_dp=True)
        if rank == 0:
            line["gpt2_medium"] = g
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_hbm(args):
    """The HBM-bound kernels at the GPT-2 c_attn / LayerNorm shapes (bf16, B=16, T=1024): LayerNorm
    forward, LayerNorm backward (dx + per-sample dgamma/dbeta + clip + noise) and the bias gradient.
    Calls run back to back over rotating inputs larger than the L2; achieved GB/s = algorithmic bytes /
    time per call against the measured copy bandwidth."""
    import torch
    from flashdp4review_b200 import _lib
    from flashdp4review_b200.core import ops
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    B, T, d, n_out = 16, 1024, 1024, 3072
    dt = torch.bfloat16
    gen = torch.Generator().manual_seed(0)
    # ROT independent input sets, visited in turn: 6 x 67..134 MB per operator, so a call never finds its
    # inputs in the 126 MB L2 and no flush (whose dirty lines the timed kernel would have to evict) is needed
    ROT = 6
    xs = [torch.randn(B, T, d, generator=gen).to(dt).to(dev) for _ in range(ROT)]
    dys = [(torch.randn(B, T, d, generator=gen) * 1e-3).to(dt).to(dev) for _ in range(ROT)]
    Gs = [(torch.randn(B, T, n_out, generator=gen) * 1e-3).to(dt).to(dev) for _ in range(ROT)]
    gamma = torch.ones(d, device=dev)
    beta = torch.zeros(d, device=dev)
    # 1 GiB fill: overwrites the L2 (isolated timing) and keeps the GPU busy while the host queues calls
    flush = torch.empty(1 << 30, dtype=torch.uint8, device=dev)
    noise = ops.NoiseSpec(std=0.25, seed=1, param_id=1, param_id2=2, step=1)
    bufs = [ops.layernorm_fwd_fused(x, gamma, beta, 1e-5)[1] for x in xs]
    cases = {
        "layernorm_fwd": (lambda i: ops.layernorm_fwd_fused(xs[i], gamma, beta, 1e-5), 2 * xs[0].numel() * 2 + 8 * B * T),
        "layernorm_bwd": (lambda i: ops.dp_layernorm_backward(dys[i], xs[i], gamma, bufs[i]["mean"], bufs[i]["rstd"],
                                                              1.0, 1.0, noise=noise), 3 * xs[0].numel() * 2 + 8 * B * T),
        "bias_grad": (lambda i: ops.dp_bias_grad(Gs[i], 1.0, 1.0, noise=noise), Gs[0].numel() * 2),
    }
    pk = peaks()
    res = {}
    for name, (fn, nbytes) in cases.items():
        for i in range(max(args.warmup, 3)):
            fn(i % ROT)
        # (1) streamed: steps x ROT calls queued back to back behind a few ms of fills (so the host runs
        # ahead of the GPU), one event pair around all of them
        torch.cuda.synchronize()
        for _ in range(24):
            flush.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            for i in range(ROT):
                fn(i)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / (args.steps * ROT)
        # (2) isolated: one call per event pair, L2 overwritten before it
        times = []
        for it in range(args.steps):
            flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn(it % ROT)
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        res[name] = {"ms": ms, "ms_isolated": statistics.median(times), "ms_isolated_min": min(times),
                     "algorithmic_bytes": nbytes, "achieved_gbs": nbytes / ms / 1e6,
                     "frac_of_measured_hbm": nbytes / ms / 1e6 / pk["hbm"]}
    k = res["layernorm_bwd"]
    line = {"metric": "layernorm_bwd_gbs", "value": k["achieved_gbs"], "unit": "GB/s", "n_gpus": 1,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": k["ms"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": args.workload, "B": B, "T": T, "d": d, "n_out": n_out,
                       "l2": "six rotating input sets per operator (400-800 MB), far larger than the 126 MB L2",
                       "timing": "ms: whole library calls (all their kernels) queued back to back over the rotating "
                                 "inputs, one CUDA-event pair around steps*6 calls; ms_isolated: one call per event "
                                 "pair right after a 1 GiB fill (the call then also evicts the fill's dirty lines)"},
            "roofline": {"bound": "hbm", "achieved": k["achieved_gbs"], "peak": pk["hbm"], "unit": "GB/s",
                         "frac": k["frac_of_measured_hbm"], "traffic": None, "peak_source": pk["source"]},
            "kernels": res, "gpu_launches": int(lib.fdp_launch_count())}
    print(json.dumps(line), flush=True)


def gpt2_measure(args, steps, with_no_dp=False, no_dp=False):
    """GPT-2-medium DP training step (24 layers, d=1024, 16 heads, ctx 1024, vocab 50257; random init,
    uniform random tokens, micro-batch 8 per GPU, bf16 autocast, Adam lr 1e-4, C=1, sigma=1): the
    transformers GPT2LMHeadModel with every Conv1D / LayerNorm wrapped, lm_head skipped
    (the loop of example/gpt2/train.py:71-86).  Returns tokens/s over all ranks and the pieces of the
    JSON line; `with_no_dp` also times the same model unwrapped for context."""
    import torch
    import torch.distributed as dist
    import flashdp4review_b200 as fdp
    from flashdp4review_b200 import _lib
    from flashdp4review_b200.distributed import DPGradReducer
    from flashdp4review_b200.layers import Conv1D
    from transformers import GPT2Config, GPT2LMHeadModel

    rank, local_rank, world, dev = dist_setup()
    lib = _lib.load()
    fdp.manual_seed(1234)
    fdp.set_data_parallel(rank, world)
    # fp32 run (--fp32: no autocast, the reference's own default, example/gpt2/train.py:34)
    fdp.set_input_grad_impl(args.gemm_impl)
    if args.fp32:
        fdp.set_fp32_mode(args.fp32_mode)
    micro_batch, seq = args.micro_batch, 1024
    cfg = GPT2Config(n_layer=args.layers, n_embd=1024, n_head=16, n_positions=1024, vocab_size=50257,
                     resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
    gen = torch.Generator().manual_seed(42 + rank)
    tokens_h = torch.randint(0, cfg.vocab_size, (micro_batch, seq + 1), generator=gen).pin_memory()
    tokens = tokens_h.to(dev)
    loss_h = torch.zeros((), dtype=torch.float32).pin_memory()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    def build(dp):
        torch.manual_seed(0)
        model = GPT2LMHeadModel(cfg).to(dev)
        if dp:
            with contextlib.redirect_stdout(sys.stderr):     # stdout carries the JSON line only
                fdp.wrap_with_flashdp_layers(model, target_modules=[Conv1D, torch.nn.Linear, torch.nn.LayerNorm],
                                             skip_layers=["lm_head"], C=1.0, noise_multiplier=1.0, feedback=False)
        # fused=True: one multi-tensor kernel; the default would fall back to ~300 per-parameter kernel chains
        # because DPParameter is a Parameter subclass (torch's foreach/fused auto-selection wants exact types)
        opt = torch.optim.Adam(model.parameters(), lr=1e-4, fused=True)
        # gradients live in the all-reduce buckets; the DP layers write their weight gradients straight into them
        reducer = DPGradReducer(model, grad_as_bucket_view=True) if world > 1 else None

        def step(tok):
            if reducer is not None:
                reducer.zero_grad()
            else:
                opt.zero_grad(set_to_none=True)
            with torch.autocast("cuda", dtype=torch.bfloat16, enabled=not args.fp32):
                out = model(input_ids=tok[:, :-1], labels=tok[:, :-1])
            out.loss.backward()
            if reducer is not None:
                reducer.finish()
            opt.step()
            return out.loss
        return step, reducer

    res = {}
    if with_no_dp and not no_dp:
        plain_step, plain_reducer = build(False)
        for _ in range(3):
            plain_step(tokens)
        res["no_dp_ms_per_step"] = timed(lambda: plain_step(tokens), 10) / 10
        if plain_reducer is not None:
            plain_reducer.remove()
        del plain_step, plain_reducer
        torch.cuda.empty_cache()

    step, reducer = build(not no_dp)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    for _ in range(max(args.warmup, 3)):
        step(tokens)
    if sampler:
        sampler.wait_first_sample()
    l0, w0 = lib.fdp_launch_count(), time.time()
    total_ms = timed(lambda: step(tokens), steps)
    windows = [(w0, time.time())]
    launches = lib.fdp_launch_count() - l0
    ms_per_step = total_ms / steps

    def e2e_step():
        tokens.copy_(tokens_h, non_blocking=True)
        loss_h.copy_(step(tokens).detach().float(), non_blocking=True)

    e2e_steps = max(2, min(steps, 10))
    e2e_step()
    e2e_ms = timed(e2e_step, e2e_steps) / e2e_steps
    clocks = sampler.stop(windows) if sampler else None
    peak_mem = torch.cuda.max_memory_allocated(dev)
    res.update({"tokens_per_s": world * micro_batch * seq / (ms_per_step * 1e-3), "ms_per_step": ms_per_step,
                "steps": steps, "n_gpus": world, "gpu_launches": int(launches), "clocks": clocks,
                "loss": float(loss_h), "peak_memory_bytes": int(peak_mem),
                "e2e": {"value": world * micro_batch * seq / (e2e_ms * 1e-3), "unit": "tokens/s",
                        "h2d_bytes_per_step": tokens_h.numel() * 8, "d2h_bytes_per_step": 4,
                        "ms_per_step": e2e_ms, "steps": e2e_steps},
                "config": {"layers": args.layers, "d_model": 1024, "heads": 16, "seq_len": seq,
                           "micro_batch_per_gpu": micro_batch, "global_batch": micro_batch * world,
                           "dp_wrapped": not no_dp, "gemm_impl": args.gemm_impl, "optimizer": "Adam lr 1e-4 (fused)",
                           "C": 1.0, "noise_multiplier": 1.0, "parallelism": f"dp{world}",
                           "grad_buckets": "fp32, 64 MB, gradients are views of the buckets" if world > 1 else None,
                           "l2": "activations and weights (GBs) far larger than the 126 MB L2"}})
    if reducer is not None:
        reducer.remove()
    return res


def run_gpt2(args):
    """`--workload gpt2_medium`: the GPT-2-medium DP step as a JSON line of its own (`--no-dp`: the
    same model unwrapped)."""
    import torch.distributed as dist
    g = gpt2_measure(args, steps=args.steps, no_dp=args.no_dp)
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    if rank == 0:
        cfg = dict(g["config"], workload=args.workload)
        line = {"metric": "gpt2_medium_dp_tokens_per_s", "value": g["tokens_per_s"], "unit": "tokens/s", "n_gpus": world,
                "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": g["ms_per_step"],
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "f32 (%s)" % args.fp32_mode if args.fp32 else "bf16",
                "data": "synthetic", "config": cfg, "e2e": g["e2e"], "gpu_launches": g["gpu_launches"],
                "clocks": g["clocks"], "loss": g["loss"], "peak_memory_bytes": g["peak_memory_bytes"]}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def build_llama(layers=32, d=4096, heads=32, ffn=11008, vocab=32000, dtype=None, device=None):
    """A Llama-2-7B-shaped decoder in plain PyTorch (pre-norm blocks with RMSNorm, rotary attention
    through scaled_dot_product_attention, SwiGLU MLP, untied lm_head); random init.  Every projection
    is an nn.Linear without bias, so wrap_with_flashdp_layers can swap them."""
    import torch
    import torch.nn as nn
    import torch.nn.functional as F

    class RMSNorm(nn.Module):
        def __init__(self, n, eps=1e-5):
            super().__init__()
            self.weight = nn.Parameter(torch.ones(n))
            self.eps = eps

        def forward(self, x):
            v = x.float()
            return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype) * self.weight

    def rope(x, cos, sin):          # x (B, H, T, hd)
        x1, x2 = x[..., ::2], x[..., 1::2]
        return torch.stack((x1 * cos - x2 * sin, x1 * sin + x2 * cos), dim=-1).flatten(-2)

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.attn_norm, self.mlp_norm = RMSNorm(d), RMSNorm(d)
            self.q_proj, self.k_proj, self.v_proj, self.o_proj = (nn.Linear(d, d, bias=False) for _ in range(4))
            self.gate_proj, self.up_proj = nn.Linear(d, ffn, bias=False), nn.Linear(d, ffn, bias=False)
            self.down_proj = nn.Linear(ffn, d, bias=False)

        def forward(self, x, cos, sin):
            B, T, _ = x.shape
            h = self.attn_norm(x)
            split = lambda t: t.view(B, T, heads, d // heads).transpose(1, 2)
            q, k, v = split(self.q_proj(h)), split(self.k_proj(h)), split(self.v_proj(h))
            a = F.scaled_dot_product_attention(rope(q, cos, sin), rope(k, cos, sin), v, is_causal=True)
            x = x + self.o_proj(a.transpose(1, 2).reshape(B, T, d))
            h = self.mlp_norm(x)
            return x + self.down_proj(F.silu(self.gate_proj(h)) * self.up_proj(h))

    class Decoder(nn.Module):
        def __init__(self):
            super().__init__()
            self.embed = nn.Embedding(vocab, d)
            self.blocks = nn.ModuleList(Block() for _ in range(layers))
            self.norm = RMSNorm(d)
            self.lm_head = nn.Linear(d, vocab, bias=False)

        def forward(self, tokens):
            T = tokens.shape[1]
            hd = d // heads
            inv = 1.0 / (10000.0 ** (torch.arange(0, hd, 2, device=tokens.device, dtype=torch.float32) / hd))
            ang = torch.arange(T, device=tokens.device, dtype=torch.float32)[:, None] * inv[None, :]
            x = self.embed(tokens)
            cos, sin = ang.cos().to(x.dtype), ang.sin().to(x.dtype)
            for blk in self.blocks:
                x = blk(x, cos, sin)
            return self.lm_head(self.norm(x))

    with torch.device(device if device is not None else "cpu"):
        model = Decoder()
    for name, prm in model.named_parameters():
        if prm.dim() == 2:
            torch.nn.init.normal_(prm, std=0.02)
    return model.to(dtype) if dtype is not None else model


def run_llama(args):
    """Llama-2-7B-shaped decoder (32 layers, d 4096, 32 heads, SwiGLU 11008, RMSNorm, vocab 32000), every
    nn.Linear but lm_head DP-wrapped, uniform random tokens, seq 2048, micro-batch 4 per GPU, parameters
    and activations in bf16 (no autocast), C = 1, sigma = 1; data-parallel with the clipped sums written
    straight into bf16 all-reduce buckets.  Optimizer: fused Adam on the bf16 parameters (bf16 moments).
    Metric: tokens/s over all ranks; the line also carries the memory high-water mark."""
    import torch
    import torch.distributed as dist
    import flashdp4review_b200 as fdp
    from flashdp4review_b200 import _lib
    from flashdp4review_b200.distributed import DPGradReducer

    rank, local_rank, world, dev = dist_setup()
    lib = _lib.load()
    fdp.manual_seed(1234)
    fdp.set_data_parallel(rank, world)
    fdp.set_input_grad_impl(args.gemm_impl)
    micro_batch, seq, vocab = args.llama_micro_batch, args.llama_seq, 32000
    torch.manual_seed(0)
    model = build_llama(layers=args.llama_layers, dtype=torch.bfloat16, device=dev)
    n_params = sum(p.numel() for p in model.parameters())
    if not args.no_dp:
        with contextlib.redirect_stdout(sys.stderr):         # stdout carries the JSON line only
            fdp.wrap_with_flashdp_layers(model, target_modules=[torch.nn.Linear], skip_layers=["lm_head"], C=1.0,
                                         noise_multiplier=1.0, feedback=False)
    n_dp = sum(p.numel() for p in model.parameters() if getattr(p, "requires_dp", False))
    opt = torch.optim.Adam(model.parameters(), lr=1e-4, fused=True)
    reducer = DPGradReducer(model, grad_as_bucket_view=True, bucket_bytes=256 << 20) if world > 1 else None
    gen = torch.Generator().manual_seed(42 + rank)
    tokens_h = torch.randint(0, vocab, (micro_batch, seq + 1), generator=gen).pin_memory()
    tokens = tokens_h.to(dev)
    loss_h = torch.zeros((), dtype=torch.float32).pin_memory()

    def step(tok):
        if reducer is not None:
            reducer.zero_grad()
        else:
            opt.zero_grad(set_to_none=True)
        logits = model(tok[:, :-1])
        loss = torch.nn.functional.cross_entropy(logits.float().view(-1, vocab), tok[:, 1:].reshape(-1))
        loss.backward()
        if reducer is not None:
            reducer.finish()
        opt.step()
        return loss

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    sampler = ClockSampler(local_rank) if rank == 0 else None
    for _ in range(max(args.warmup, 3)):
        step(tokens)
    if sampler:
        sampler.wait_first_sample()
    l0, w0 = lib.fdp_launch_count(), time.time()
    total_ms = timed(lambda: step(tokens), args.steps)
    windows = [(w0, time.time())]
    launches = lib.fdp_launch_count() - l0
    ms_per_step = total_ms / args.steps

    def e2e_step():
        tokens.copy_(tokens_h, non_blocking=True)
        loss_h.copy_(step(tokens).detach().float(), non_blocking=True)

    e2e_steps = max(2, min(args.steps, 5))
    e2e_step()
    e2e_ms = timed(e2e_step, e2e_steps) / e2e_steps
    clocks = sampler.stop(windows) if sampler else None
    # the all-reduce alone, on buffers of the buckets' sizes (context for the overlap)
    allreduce_ms = None
    if reducer is not None:
        allreduce_ms = timed(lambda: [dist.all_reduce(f) for f in reducer._flat], 3) / 3
        for f in reducer._flat:
            f.zero_()
    if rank == 0:
        tok_s = world * micro_batch * seq / (ms_per_step * 1e-3)
        line = {"metric": "llama7b_shaped_dp_tokens_per_s", "value": tok_s, "unit": "tokens/s", "n_gpus": world,
                "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": args.workload, "layers": args.llama_layers, "d_model": 4096, "heads": 32,
                           "ffn": 11008, "vocab": vocab, "seq_len": seq, "micro_batch_per_gpu": micro_batch,
                           "global_batch": micro_batch * world, "parameters": n_params, "dp_parameters": n_dp,
                           "dp_wrapped": not args.no_dp, "gemm_impl": args.gemm_impl,
                           "optimizer": "Adam lr 1e-4 (fused, bf16 moments)", "C": 1.0, "noise_multiplier": 1.0,
                           "parallelism": f"dp{world}",
                           "grad_buckets": "bf16, 256 MB, gradients are views of the buckets" if world > 1 else None,
                           "allreduce_bytes_per_step": 2 * sum(p.numel() for p in model.parameters()) if world > 1 else 0,
                           "l2": "activations and weights (tens of GB) far larger than the 126 MB L2"},
                "e2e": {"value": world * micro_batch * seq / (e2e_ms * 1e-3), "unit": "tokens/s",
                        "h2d_bytes_per_step": tokens_h.numel() * 8, "d2h_bytes_per_step": 4, "ms_per_step": e2e_ms,
                        "steps": e2e_steps},
                "gpu_launches": int(launches), "clocks": clocks, "loss": float(loss_h),
                "peak_memory_bytes": int(torch.cuda.max_memory_allocated(dev)), "allreduce_alone_ms": allreduce_ms}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS) + ["gpt2_medium", "hbm_kernels_bf16_b16_t1024", "llama7b_shaped"])
    ap.add_argument("--llama-layers", type=int, default=32, help="llama7b_shaped: number of decoder blocks")
    ap.add_argument("--llama-seq", type=int, default=2048)
    ap.add_argument("--llama-micro-batch", type=int, default=4)
    ap.add_argument("--layers", type=int, default=24, help="gpt2_medium: number of transformer blocks")
    ap.add_argument("--micro-batch", type=int, default=8, help="gpt2_medium: samples per GPU and step")
    ap.add_argument("--gemm-impl", default="native", choices=["native", "library", "auto"],
                    help="gpt2_medium: forward / input-gradient GEMMs of the DP layers by this library or by cuBLAS")
    ap.add_argument("--no-dp", action="store_true", help="gpt2_medium: leave the model unwrapped (context only)")
    ap.add_argument("--fp32", action="store_true", help="gpt2_medium: fp32 throughout, no autocast (context only)")
    ap.add_argument("--fp32-mode", default="tensor", choices=["tensor", "exact"],
                    help="gpt2_medium --fp32: DP weight gradients as three bf16 tensor-core products, or on fp32-FMA kernels")
    ap.add_argument("--norm-algo", default="auto", choices=["auto", "direct", "gram"])
    ap.add_argument("--sigma", type=float, default=1.0, help="noise_multiplier of the DP-Linear workloads")
    ap.add_argument("--cpu-budget", type=float, default=12.0, help="seconds of CPU work for cpu_baseline")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-full", action="store_true", default=True,
                    help="cpu_baseline also times the workload's whole batch (two steps)")
    ap.add_argument("--no-cpu-full", dest="cpu_full", action="store_false")
    ap.add_argument("--no-gpt2", action="store_true", help="default workload: skip the GPT-2-medium leg")
    ap.add_argument("--no-check", action="store_true", help="skip the untimed N-rank == single-rank check")
    ap.add_argument("--reserve-sms", type=int, default=12,
                    help="N > 1: SMs the input-gradient GEMM leaves to the all-reduce that runs beside it")
    ap.add_argument("--ref-gpu-child", action="store_true", help=argparse.SUPPRESS)
    ap.add_argument("--no-ref-gpu", action="store_true",
                    help="skip the context leg that runs the installed reference package on the same GPU")
    args = ap.parse_args()
    if args.workload == "hbm_kernels_bf16_b16_t1024":
        return run_hbm(args)
    if args.workload == "llama7b_shaped":
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "the reference's per-sample path has no CPU-"
                              "feasible whole-model run; the per-layer CPU baseline is the default workload's"}))
            return
        return run_llama(args)
    if args.workload == "gpt2_medium":
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "the reference's per-sample path has no CPU-"
                              "feasible whole-model run; the per-layer CPU baseline is the default workload's"}))
            return
        return run_gpt2(args)
    wl = WORKLOADS[args.workload]
    if args.ref_gpu_child:
        return reference_gpu_child(args, wl)
    if args.impl == "reference":
        run_reference(args, wl)
    else:
        run_native(args, wl)


if __name__ == "__main__":
    main()
