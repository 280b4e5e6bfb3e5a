#!/usr/bin/env python
"""Benchmark of the training hot path: CIFAR-10-style network, batch 256 per GPU,
cross-entropy after softmax, Adam (lr 1e-3), fp32 -- training samples/s.

    python bench.py --gpus 1 --steps 50 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference ...     # the reference's own CPU path on the host cores

One JSON line is printed by rank 0.  `value` is measured with inputs resident in
HBM; `e2e` goes through the HOST-buffer entry point (host->device copy of the
batch and device->host copy of the network output inside the timed region).
Data are synthetic with CIFAR-10's shapes (3x32x32 inputs ~ N(0,1), 10 classes).

A block of `--steps` steps is timed with CUDA events between barriers, and the
block is repeated until at least one second has been timed; the line reports the
median block (`ms_per_step`) with the fastest and slowest beside it.  With more
than one rank the line also carries `parity`: the replicas' parameters compared
bit for bit after the timed steps, and two data-parallel steps compared with the
same two steps of ONE GPU on the concatenated mini-batch.
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

ROOT = Path(__file__).resolve().parent
for p in (ROOT, ROOT / "tests"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))

BATCH = 256
NB = 8  # distinct mini-batches rotated through the step
IN_DIM, OUT_DIM = 3 * 32 * 32, 10
MIN_TIMED_MS = 1000.0  # the block of --steps steps is repeated until this much has been timed
MAX_BLOCKS = 400
WORKLOAD = "cifar10_net conv5x5(3->32,same)-relu-maxpool2 conv5x5(32->32)-relu-maxpool2 " \
           "conv5x5(32->64)-relu-maxpool2 fc1024->64-relu fc64->10-softmax; cross_entropy; adam lr=1e-3"
LOSS_CE, OPT_ADAM = 1, 1
SM_COUNT, FP32_LANES = 148, 128


def conv_flops(B, w, c, oc, k):
    return 2.0 * B * w * w * oc * c * k * k


# the three convolutions of the net: (name, width, in_c, out_c, k)
CONVS = [("conv1", 32, 3, 32, 5), ("conv2", 16, 32, 32, 5), ("conv3", 8, 32, 64, 5)]


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples while a region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.proc = None
        self.gpu = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                  "sw_power_cap"), f[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "samples": len(sm), "reasons": sorted(reasons)}


def make_specs():
    from cases import build_net_specs
    return build_net_specs("cifar")


def synthetic_batches(n_batches, seed):
    import numpy as np
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((n_batches, BATCH, IN_DIM)).astype(np.float32)
    labels = rng.integers(0, OUT_DIM, (n_batches, BATCH))
    t = np.zeros((n_batches, BATCH, OUT_DIM), np.float32)
    for i in range(n_batches):
        t[i, np.arange(BATCH), labels[i]] = 1.0
    return x, t


# --------------------------------------------------------------------------------------------
# reference arm: the unmodified reference's CPU path (OpenMP, backend_t::internal)
# --------------------------------------------------------------------------------------------
def host_cores():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def run_reference(args, rank, world):
    if rank != 0:
        return
    import numpy as np
    import oracle_lib as o
    from cases import hyper_for, xavier_params
    specs, keep = make_specs()
    arr = (type(specs[0]) * len(specs))(*specs)
    x, t = synthetic_batches(NB, 1000)
    hy = hyper_for(OPT_ADAM)
    ref = o.load_reference()
    count = [0]
    if ref is not None:
        # all host cores, whatever OMP_NUM_THREADS the launcher exported (torch.distributed.run sets 1)
        kind, cores = "reference", ref.ref_set_threads(host_cores())
        h = ref.ref_net_create(arr, len(specs), 42)
        p0 = xavier_params(specs, 42)
        ref.ref_net_set_params(h, o.p(p0))

        def one_step():
            i = count[0] % NB
            count[0] += 1
            s = ref.ref_net_fit(h, o.p(x[i]), o.p(t[i]), BATCH, 1, LOSS_CE, OPT_ADAM, C.byref(hy))
            assert s >= 0
            return s
        sample = f"one mini-batch of {BATCH} samples per step through network::fit, OpenMP {cores} threads"
        per_step = BATCH
    else:
        orc = o.load_oracle()
        kind, cores = "port", 1
        sub = 32
        net = orc.orc_net_create(arr, len(specs), sub)
        params = np.ctypeslib.as_array(orc.orc_net_params(net), shape=(orc.orc_net_param_count(net),))
        params[:] = xavier_params(specs, 42)

        def one_step():
            i = count[0] % NB
            count[0] += 1
            xs, ts = np.ascontiguousarray(x[i][:sub]), np.ascontiguousarray(t[i][:sub])
            t0 = time.perf_counter()
            orc.orc_net_train_step(net, o.p(xs), o.p(ts), sub, LOSS_CE, OPT_ADAM, C.byref(hy))
            return time.perf_counter() - t0
        sample = f"{sub} samples per step through the C restatement, 1 thread"
        per_step = sub
    for _ in range(args.warmup):
        one_step()
    secs = sum(one_step() for _ in range(args.steps))
    value = per_step * args.steps / secs
    line = {
        "impl": "reference", "metric": "train_samples_per_s", "value": value, "unit": "samples/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * secs / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
        "config": bench_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": "samples/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "the CPU reference runs one GPU's mini-batch per step on rank 0's host cores",
    }
    print(json.dumps(line), flush=True)


def bench_config(world):
    """The `config` object, identical in both arms."""
    return {"workload": WORKLOAD, "per_gpu_batch": BATCH, "global_batch": BATCH * world,
            "parallelism": f"dp{world}",
            "l2": f"{NB} distinct mini-batches rotate through the step; the activations and gradients a step "
                  "touches are about 130 MB, larger than the 126 MB L2, so no flush is needed"}


# --------------------------------------------------------------------------------------------
# own arm
# --------------------------------------------------------------------------------------------
def time_kernels(ctx, torch, ops, reps=20):
    """Per convolution pass of the net at batch 256 (forward, dX, dW): CUDA-event time of the
    pass's main kernel alone (b200_conv2d_time_pass: operand copies and filter matrices prepared
    outside the timed region) and of the whole operator call (every launch the pass needs).
    Returns {name: {"ms", "op_ms", "flops", "tensor"}}."""
    from tiny_cnn_b200._lib import check, ptr
    out = {}
    g = torch.Generator(device="cuda").manual_seed(3)
    lib, h = ctx.lib, ctx.handle
    for name, w, c, oc, k in CONVS:
        d = ops.conv_params(w, w, c, k, k, oc, True, True)
        x = torch.randn(BATCH, c * w * w, device="cuda", generator=g)
        W = (torch.rand(oc * c * k * k, device="cuda", generator=g) - 0.5) * 0.2
        b = torch.zeros(oc, device="cuda")
        dy = torch.randn(BATCH, oc * w * w, device="cuda", generator=g)
        y = torch.empty(BATCH, oc * w * w, device="cuda")
        dx = torch.empty_like(x)
        dW, db = torch.zeros_like(W), torch.zeros_like(b)

        def fwd():
            check(lib.b200_conv2d_fwd(h, C.byref(d), ptr(x), ptr(W), ptr(b), ptr(y), BATCH))

        def bwd():
            check(lib.b200_conv2d_bwd(h, C.byref(d), ptr(x), ptr(W), ptr(dy), ptr(dx), ptr(dW), ptr(db), 0, BATCH))

        def bwd_nodx():
            check(lib.b200_conv2d_bwd(h, C.byref(d), ptr(x), ptr(W), ptr(dy), None, ptr(dW), ptr(db), 0, BATCH))
        op = {}
        for key, fn in (("fwd", fwd), ("bwd", bwd), ("dw", bwd_nodx)):
            for _ in range(3):
                fn()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            for _ in range(reps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            op[key] = e0.elapsed_time(e1) / reps
        op["dx"] = max(op["bwd"] - op["dw"], 1e-6)
        fl = conv_flops(BATCH, w, c, oc, k)
        for pi, key in enumerate(("fwd", "dx", "dw")):
            ms, tc = C.c_float(0), C.c_int(0)
            check(lib.b200_conv2d_time_pass(h, C.byref(d), ptr(x), ptr(W), ptr(dy), BATCH, pi, reps,
                                            C.byref(ms), C.byref(tc)))
            out[f"{name}_{key}"] = {"ms": ms.value, "op_ms": op[key], "flops": fl, "tensor": bool(tc.value)}
    return out


# DRAM traffic per launch (dram__bytes_read.sum + dram__bytes_write.sum) from the ncu captures
# summarised under profiles/; None where no capture of that launch exists
# (profiles/conv_tc_kernel_conv2_fwd_b256_ncu_full.md; conv2's dX launch is the same kernel on
# tensors of the same sizes -- 32 -> 32 channels, the same 512 tiles -- so the figure stands for both)
NCU_DRAM_BYTES = {"conv2_fwd": 17.04e6, "conv2_dx": 17.04e6}


def conv_rooflines(kt, peaks):
    """Per-kernel table and the roofline object of the dominant kernel.  Tensor-core passes
    compute every fp32 product as three TF32 products, so their ceiling in algorithmic
    (fp32-equivalent) flop/s is the TF32 rate / 3 = the measured bf16 rate / 6."""
    peak_fp32 = SM_COUNT * FP32_LANES * 2 * 1.965e9 / 1e12
    bf16 = peaks.get("bf16_tflops")
    peak_tc = (bf16 if bf16 else 1590.0) / 6.0
    src = "of measured" if bf16 else "of fallback"
    kernels = {}
    for k, v in kt.items():
        tf = v["flops"] / (v["ms"] * 1e-3) / 1e12
        peak = peak_tc if v["tensor"] else peak_fp32
        kernels[k] = {"ms": round(v["ms"], 4), "op_ms": round(v["op_ms"], 4), "tflops": round(tf, 3),
                      "engine": "tcgen05 3xTF32" if v["tensor"] else "fp32 FFMA",
                      "frac_of_peak": round(tf / peak, 4)}
    # the kernel function with the largest share of the step: conv_tc_kernel runs the forward and
    # dX passes of every tensor-core layer; report its longest launch
    fam = [k for k, v in kt.items() if v["tensor"] and not k.endswith("_dw")]
    pool = fam if fam else list(kt)
    dom = max(pool, key=lambda k: (round(kt[k]["ms"], 3), k.endswith("_fwd")))
    v = kt[dom]
    tf = v["flops"] / (v["ms"] * 1e-3) / 1e12
    tensor = v["tensor"]
    peak = peak_tc if tensor else peak_fp32
    conv_ms = sum(x["ms"] for x in kt.values())
    conv_op_ms = sum(x["op_ms"] for x in kt.values())
    conv_fl = sum(x["flops"] for x in kt.values())
    op_tf = v["flops"] / (v["op_ms"] * 1e-3) / 1e12
    roofline = {
        "kernel": ("conv_tc_kernel" if tensor else "conv FFMA kernel") + f" ({dom})",
        "bound": "tensor" if tensor else "fp32",
        "achieved": round(tf, 3), "peak": round(peak, 2), "unit": "TFLOP/s", "frac": round(tf / peak, 4),
        # the same pass as the operator call issues it: the main kernel plus the layout kernels it needs
        # (tall hi/lo copies, filter matrices, partial-row merges)
        "achieved_op": round(op_tf, 3), "frac_op": round(op_tf / peak, 4),
        "traffic": NCU_DRAM_BYTES.get(dom),
        "peak_source": (f"algorithmic fp32 flop/s; ceiling = bf16 tensor peak {bf16} TFLOP/s {src} / 2 (TF32 rate) "
                        "/ 3 (three TF32 products per fp32 product)") if tensor else
                       "fp32 FFMA: 148 SMs x 128 lanes x 2 flop x clocks.max.sm 1965 MHz (no measured fp32 figure)",
        "tensor_pipe_tflops": round(3 * tf, 1) if tensor else None,
        "conv_main_kernels_all": {"ms": round(conv_ms, 4), "tflops": round(conv_fl / (conv_ms * 1e-3) / 1e12, 3)},
        "conv_operator_calls_all": {"ms": round(conv_op_ms, 4),
                                    "tflops": round(conv_fl / (conv_op_ms * 1e-3) / 1e12, 3)},
        "fp32_ffma_peak": round(peak_fp32, 2), "hbm_gbs": peaks.get("hbm_gbs"),
    }
    return kernels, roofline


def kernel_timeline(torch, path, rank, world, some_steps):
    """Start and duration of every kernel of one replayed step on rank 0, as text.  Not a bench
    number: the profiler's own overhead is in it; it shows which kernels overlap which."""
    import re

    from torch.profiler import ProfilerActivity, profile
    if rank != 0:
        some_steps()
        torch.cuda.synchronize()
        return
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        some_steps()
        torch.cuda.synchronize()
    evs = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA]
    evs.sort(key=lambda e: e.time_range.start)
    marks = [i for i, e in enumerate(evs) if "opt_advance_powers" in e.name]  # the last kernel of a step
    if len(marks) < 4:
        return
    a, b = marks[-3] + 1, marks[-2] + 1
    t0 = evs[a].time_range.start
    rows = [f"# one replayed step of {world} replica(s), rank 0: {len(evs[a:b])} kernels / copies, "
            f"{evs[b - 1].time_range.end - t0:.1f} us from the first start to the last end",
            "# start_us  duration_us  kernel"]
    for e in evs[a:b]:
        m = re.search(r"(\w+_kernel)", e.name)
        rows.append(f"{e.time_range.start - t0:9.1f} {e.time_range.end - e.time_range.start:11.1f}  "
                    f"{m.group(1) if m else e.name[:60]}")
    Path(path).parent.mkdir(parents=True, exist_ok=True)
    Path(path).write_text("\n".join(rows) + "\n")


def run_b200(args, rank, world, local_rank):
    import numpy as np
    import torch
    import torch.distributed as dist

    from tiny_cnn_b200 import network as nw
    from tiny_cnn_b200 import ops
    from tiny_cnn_b200._lib import check, load
    from tiny_cnn_b200.parallel import DataParallel

    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local_rank}"))
    lib = load()
    ctx = ops.Context(local_rank)
    net = nw.cifar10_net(local_rank).build(BATCH, ctx)
    p0 = net.init_weight(np.random.default_rng(42))  # same seed on every rank: identical replicas
    opt = nw.adam(1e-3)
    dp = DataParallel(net)
    # replicas: the bucket is summed over NVLink by the library's own kernels inside the step's graph;
    # NCCL only when the peer mapping is unavailable (or B200_DP_NCCL=1)
    peer = world > 1 and os.environ.get("B200_DP_NCCL") != "1" and dp.enable_peer_reduce()

    xh, th = synthetic_batches(NB, 1000 + rank)
    x_all = torch.from_numpy(xh).cuda()
    t_all = torch.from_numpy(th).cuda()
    x_cur = torch.empty(BATCH, IN_DIM, device="cuda")
    t_cur = torch.empty(BATCH, OUT_DIM, device="cuda")
    x_pin = torch.from_numpy(xh).pin_memory()
    t_pin = torch.from_numpy(th).pin_memory()
    out_pin = torch.empty(BATCH, OUT_DIM).pin_memory()
    out_dev = net.output_tensor(BATCH)

    def dp_step(x, t):
        if world == 1 or peer:
            net.train_onebatch(opt, x, t, LOSS_CE)
        else:
            net.forward_backward(x, t, LOSS_CE)
            dp.allreduce_grads()
            net.update(opt)

    def step(i):
        # the NB resident mini-batches are passed where they lie: the library keeps one captured graph
        # per input pointer (up to eight), so no copy runs between two steps
        dp_step(x_all[i % NB], t_all[i % NB])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world > 1:
            tms = torch.tensor([ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(tms, op=dist.ReduceOp.MAX)
            ms = float(tms[0])
        return ms

    def restart():
        """Every timed block starts from the initial weights with a fresh optimizer (outside the timed
        region): thousands of adam steps on eight fixed mini-batches of random labels memorise them
        until a softmax output rounds to exactly 1, where the reference's cross_entropy::df
        (y - t) / (y (1 - y)) is 0/0 -- on the CPU as much as here -- and the weights turn to NaN."""
        net.set_params(p0)
        check(lib.b200_net_opt_reset(net.handle, 1))

    def timed_block(run_steps, steps):
        """barrier, event, `steps` steps, event, barrier; device time, max over ranks."""
        restart()
        barrier()
        l0 = lib.b200_launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        run_steps(steps)
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1)), lib.b200_launch_count() - l0

    def repeat_blocks(run_steps, steps):
        """Repeat the block until MIN_TIMED_MS have been timed (every rank sees the same max-reduced
        times, so every rank stops after the same block)."""
        times, launches = [], 0
        min_ms, min_blocks = (0.0, 1) if args.profile else (MIN_TIMED_MS, 3)
        while (sum(times) < min_ms or len(times) < min_blocks) and len(times) < MAX_BLOCKS:
            ms, launches = timed_block(run_steps, steps)
            times.append(ms)
        return times, launches

    # ---- inputs resident in HBM ------------------------------------------------------------
    counter = [0]

    def run_device(steps):
        for _ in range(steps):
            step(counter[0])
            counter[0] += 1

    warmup = max(args.warmup, 3)
    run_device(max(warmup, 3 * NB))  # every mini-batch's graph is captured on its second use
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    blocks, launches = repeat_blocks(run_device, args.steps)
    clocks = sampler.stop() if rank == 0 else None
    ctx.sync()  # raises if a kernel gave up a bounded wait (a peer reduction that timed out)
    ms = statistics.median(blocks)

    # informational, never the reported value: the same step without the gradient with respect to the
    # input images, which the reference computes and network::fit never reads (weights bit-identical)
    ms_no_input_grad = None
    if world == 1 and not args.profile:
        check(lib.b200_net_set_input_grad(net.handle, 0))
        run_device(3 * NB)
        ms_no_input_grad = statistics.median(timed_block(run_device, args.steps)[0] for _ in range(5))
        check(lib.b200_net_set_input_grad(net.handle, 1))
        run_device(3 * NB)

    # ---- end to end: every step's inputs from pinned host memory, its output back to the host ----
    fit_ok = world == 1 or peer

    def run_e2e(steps):
        base = counter[0]
        counter[0] += steps
        if fit_ok:
            # network::fit's counterpart: one library call; the upload of mini-batch i+1 runs on a copy
            # stream beside step i (with several ranks the reduction over the replicas is inside the step)
            net.fit(opt, xs_fit[:steps * BATCH], ts_fit[:steps * BATCH], BATCH, 1, LOSS_CE, outs_fit[:steps * BATCH])
            return
        for i in range(base, base + steps):
            x_cur.copy_(x_pin[i % NB], non_blocking=True)
            t_cur.copy_(t_pin[i % NB], non_blocking=True)
            dp_step(x_cur, t_cur)
            out_pin.copy_(out_dev, non_blocking=True)
            torch.cuda.current_stream().synchronize()

    n_fit = max(args.steps, warmup)
    if fit_ok:
        idx = [i % NB for i in range(n_fit)]
        xs_fit = torch.cat([x_pin[j] for j in idx]).pin_memory()
        ts_fit = torch.cat([t_pin[j] for j in idx]).pin_memory()
        outs_fit = torch.empty(n_fit * BATCH, OUT_DIM).pin_memory()
    run_e2e(warmup)
    blocks_e2e, _ = repeat_blocks(run_e2e, args.steps)
    ctx.sync()
    ms_e2e = statistics.median(blocks_e2e)

    # ---- optional: kernel timeline of one replayed step (CUPTI through torch.profiler, rank 0) ----
    if args.timeline:
        restart()
        barrier()
        # every resident mini-batch has its own captured graph: each one replays under the profiler before the step that is kept
        kernel_timeline(torch, args.timeline, rank, world, lambda: run_device(3 * NB))
        barrier()

    # ---- replicas against each other and against one GPU on the concatenated mini-batch ----
    parity = None
    if world > 1:
        parity = dp_parity(torch, dist, np, nw, ops, net, opt, dp, dp_step, p0, rank, world, local_rank, ctx)

    global_batch = BATCH * world
    value = global_batch * args.steps / (ms * 1e-3)
    e2e_value = global_batch * args.steps / (ms_e2e * 1e-3)

    line = None
    if rank == 0:
        # per-kernel roofline of the convolution kernels, timed alone with CUDA events
        kt = time_kernels(ctx, torch, ops, reps=2 if args.profile else 20)
        peaks = {}
        mp = ROOT / "MEASURED_PEAKS.json"
        if mp.exists():
            peaks = json.loads(mp.read_text())
        kernels, roofline = conv_rooflines(kt, peaks)
        cpu = cpu_baseline() if world == 1 and not args.profile else None
        cpp = e2e_cpp(max(4 * args.steps, 200)) if world == 1 and not args.profile else None
        per = 1.0 / args.steps
        line = {
            "metric": "train_samples_per_s", "value": value, "unit": "samples/s", "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": ms * per,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32",
            "data": "synthetic",
            "config": bench_config(world),
            "timing": {"blocks": len(blocks), "timed_ms": round(sum(blocks), 2),
                       "ms_per_step_median": ms * per, "ms_per_step_min": min(blocks) * per,
                       "ms_per_step_max": max(blocks) * per,
                       "how": f"blocks of {args.steps} steps between barriers, CUDA events, max over ranks, "
                              f"repeated until {MIN_TIMED_MS:.0f} ms were timed; the median block is reported"},
            "notes": {
                "arithmetic": "fp32 results; conv2/conv3 passes on tcgen05 tensor cores as 3xTF32 (hi/lo split, fp32 "
                              "accumulation) -- also conv1 forward and dW; conv1 dX and the rest fp32 FFMA",
                "step": ("CUDA graph of forward+backward+update" if world == 1 else
                         "one CUDA graph: forward+backward with the gradients of all layers but the first pushed to the "
                         "peers over NVLink from a side branch as soon as they exist, then first-layer push + "
                         "rank-ordered sum (the library's peer-memory kernels), update" if peer else
                         "CUDA graph of forward+backward, NCCL sum all-reduce of the gradient bucket, update")
                        + "; inside the graph the weight-gradient kernels and the filter matrices run on a "
                          "side branch beside the forward / dX chain",
                "without_input_gradient": (None if ms_no_input_grad is None else {
                    "ms_per_step": ms_no_input_grad / args.steps,
                    "samples_per_s": BATCH * args.steps / (ms_no_input_grad * 1e-3),
                    "what": "informational: b200_net_set_input_grad(net, 0) drops the first layer's dX, a tensor the "
                            "reference computes and network::fit never reads; weights bit-identical; `value` keeps it"}),
                "peer_rendezvous": ({"ipc": "b200_peer_buffer_create/_open (the library's inter-process handles)",
                                     "symm": "torch symmetric memory"}.get(dp.rendezvous) if peer else None)},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "samples/s", "ms_per_step": ms_e2e * per,
                    "ms_per_step_min": min(blocks_e2e) * per, "ms_per_step_max": max(blocks_e2e) * per,
                    "blocks": len(blocks_e2e),
                    "api": ("Sequential.fit -> b200_net_fit_host on every rank: uploads of the next mini-batch overlap "
                            "the current step" + ("" if world == 1 else "; the reduction over the replicas is inside the step"))
                           if fit_ok else "per-step copies, forward_backward, NCCL all-reduce, update",
                    "h2d_bytes_per_step": BATCH * (IN_DIM + OUT_DIM) * 4,
                    "d2h_bytes_per_step": BATCH * OUT_DIM * 4},
            "gpu_launches": int(launches),
            "roofline": roofline,
            "kernels": kernels,
        }
        if parity is not None:
            line["parity"] = parity
        if cpu is not None:
            line["cpu_baseline"] = cpu
        if cpp is not None:
            line["e2e_cpp"] = cpp
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if line is not None:
        print(json.dumps(line), flush=True)


def dp_parity(torch, dist, np, nw, ops, net, opt, dp, dp_step, p0, rank, world, local_rank, ctx):
    """Outside any timed region.  (a) After the timed steps every replica must hold the same
    parameters, bit for bit.  (b) The gradient bucket of one data-parallel forward + backward, summed
    over the replicas, against forward + backward of a single GPU (rank 0) on the concatenated
    mini-batch of world x BATCH samples: gradients are sums over the batch with no 1/N, so sharding
    must change them by rounding only.  (c) Two data-parallel adam steps from the initial weights
    against the same two steps of that single GPU.  Adam divides every gradient by its own magnitude
    (step = alpha * g / sqrt(g^2 + 1e-8)), so a weight whose gradient is within rounding of zero can
    move by up to alpha in either run: (c) reports the worst difference, which that mechanism bounds
    by 2 * steps * alpha, and the share of the weights within 1e-3."""
    from tiny_cnn_b200._lib import check
    def replicas_differ():
        """number of parameters that are not bit-equal on every rank, and the largest difference"""
        mine = torch.from_numpy(net.get_params()).cuda()
        gathered = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        n_bad, worst_d = 0, 0.0
        for g in gathered[1:]:
            n_bad = max(n_bad, int((gathered[0].view(torch.int32) != g.view(torch.int32)).sum()))  # bit patterns
            worst_d = max(worst_d, float(torch.nan_to_num((gathered[0] - g).abs(), nan=float("inf")).max()))
        return n_bad, worst_d, bool(torch.isfinite(mine).all())

    bad_timed, diff_timed, finite_timed = replicas_differ()
    # (b) restart every replica from the initial weights with a fresh optimizer
    steps = 2
    net.set_params(p0)
    check(net.lib.b200_net_opt_reset(net.handle, 1))
    xs, ts = synthetic_batches(steps, 7000 + rank)
    x_d, t_d = torch.from_numpy(xs).cuda(), torch.from_numpy(ts).cuda()
    x_buf, t_buf = torch.empty(BATCH, IN_DIM, device="cuda"), torch.empty(BATCH, OUT_DIM, device="cuda")
    for s in range(steps):
        x_buf.copy_(x_d[s])
        t_buf.copy_(t_d[s])
        dp_step(x_buf, t_buf)
    ctx.sync()
    p_dp = net.get_params()
    bad_steps, diff_steps, finite_steps = replicas_differ()
    identical = bad_timed == 0 and bad_steps == 0
    # (b) one forward + backward from the initial weights, bucket summed over the replicas
    net.set_params(p0)
    net.forward_backward(x_d[0], t_d[0], LOSS_CE)
    dp.allreduce_grads()
    ctx.sync()
    g_dp = net.grads_tensor().cpu().numpy().copy()
    worst = worst_grad = share = worst_abs = None
    if rank == 0:
        big = nw.cifar10_net(local_rank).build(BATCH * world, ctx)
        big.set_params(p0)
        parts = [synthetic_batches(steps, 7000 + r) for r in range(world)]
        x = torch.from_numpy(np.concatenate([pr[0][0] for pr in parts])).cuda()
        t = torch.from_numpy(np.concatenate([pr[1][0] for pr in parts])).cuda()
        big.forward_backward(x, t, LOSS_CE)
        ctx.sync()
        g_one = big.grads_tensor().cpu().numpy().copy()
        worst_grad = 0.0
        for off, ln in big.tensors():
            a, b = g_dp[off:off + ln], g_one[off:off + ln]
            worst_grad = max(worst_grad, float(np.abs(a - b).max() / max(float(np.abs(b).max()), 1e-30)))
        for s in range(steps):
            x = torch.from_numpy(np.concatenate([pr[0][s] for pr in parts])).cuda()
            t = torch.from_numpy(np.concatenate([pr[1][s] for pr in parts])).cuda()
            big.train_onebatch(opt, x, t, LOSS_CE)
        ctx.sync()
        p_one = big.get_params()
        worst, within, total, worst_abs = 0.0, 0, 0, 0.0
        for off, ln in big.tensors():
            a, b = p_dp[off:off + ln], p_one[off:off + ln]
            d, mx = np.abs(a - b), max(float(np.abs(b).max()), 1e-30)
            worst = max(worst, float(d.max() / mx))
            worst_abs = max(worst_abs, float(d.max()))
            within += int((d <= 1e-3 * mx).sum())
            total += ln
        share = within / total
        big.close()
    dist.barrier()
    return {"replicas_identical": bool(identical),
            "replica_mismatches": {"after_timed_steps": [bad_timed, diff_timed], "after_parity_steps": [bad_steps, diff_steps],
                                   "what": "[parameters whose bit patterns differ between ranks, largest |difference|]"},
            "weights_finite": finite_timed and finite_steps,
            # the sum over the replicas against one GPU on the concatenated mini-batch: the gradient bucket
            "vs_single_gpu": worst_grad, "vs_single_gpu_tol": 1e-3,
            "grads_vs_single_gpu": worst_grad, "grads_tol": 1e-3,
            "weights_vs_single_gpu": {"worst": worst, "share_within_1e-3": share, "worst_abs": worst_abs,
                                      "adam_reach": 2 * steps * opt.alpha, "steps": steps},
            "how": f"gradient bucket of one data-parallel forward + backward on {world} x {BATCH} samples, summed over "
                   f"the replicas, against one GPU on the concatenated {world * BATCH}-sample mini-batch (largest "
                   "|difference| of a parameter tensor's gradient / its largest magnitude); then the weights after "
                   f"{steps} adam steps of both (adam moves a weight whose gradient is within rounding of zero by up "
                   "to alpha in either run: worst_abs is bounded by adam_reach = 2 * steps * alpha, not by 1e-3); "
                   "replicas compared bit pattern by bit pattern after the timed steps and after these"}


def e2e_cpp(steps):
    """network<sequential>::fit of the same net under engine backend_t::b200, timed inside a C++
    program around the fit call (tiny_cnn_b200/host/bench_fit.cpp, built by oracle/build_oracle.py
    where the tiny-dnn tree is present): std::vector<vec_t> in pageable memory in, trained weights in
    the layer objects out.  None when the binary was not built."""
    exe = ROOT / "oracle" / "_ref" / "bin" / "bench_fit_b200"
    if not exe.exists():
        return None
    try:
        res = subprocess.run([str(exe), str(steps), str(BATCH)], capture_output=True, text=True, timeout=300)
        line = [ln for ln in res.stdout.splitlines() if ln.startswith("{")][-1]
        d = json.loads(line)
    except Exception as e:  # a diagnostic figure: its absence must not cost the bench line
        return {"error": f"{type(e).__name__}: {e}"}
    return {"value": d["samples_per_s"], "unit": "samples/s", "ms_per_step": d["ms_per_step"], "steps": d["steps"],
            "device_fit": d["device_fit"],
            "api": "tiny_dnn::network<sequential>::fit<cross_entropy>(adam, std::vector<vec_t>, ...) with every "
                   "layer on core::backend_t::b200, wall clock around the call"}


def cpu_baseline():
    """The reference's CPU path on this box's host cores, on a bounded sample of the workload:
    backend_t::internal (the parity target) for about 10 s and, as an informational second column,
    the reference's AVX kernels (backend_t::avx: its fastest shipped path for 5x5 convolutions)."""
    import numpy as np
    import oracle_lib as o
    from cases import hyper_for, xavier_params
    specs, keep = make_specs()
    arr = (type(specs[0]) * len(specs))(*specs)
    x, t = synthetic_batches(NB, 1000)
    hy = hyper_for(OPT_ADAM)
    ref = o.load_reference()
    if ref is None:
        orc = o.load_oracle()
        sub = 32
        net = orc.orc_net_create(arr, len(specs), sub)
        params = np.ctypeslib.as_array(orc.orc_net_params(net), shape=(orc.orc_net_param_count(net),))
        params[:] = xavier_params(specs, 42)
        xs, ts = np.ascontiguousarray(x[0][:sub]), np.ascontiguousarray(t[0][:sub])
        t0 = time.perf_counter()
        n = 0
        while time.perf_counter() - t0 < 10.0:
            orc.orc_net_train_step(net, o.p(xs), o.p(ts), sub, LOSS_CE, OPT_ADAM, C.byref(hy))
            n += sub
        secs = time.perf_counter() - t0
        return {"value": n / secs, "unit": "samples/s", "cores": 1, "kind": "port",
                "sample": f"{n} samples in steps of {sub} through the C restatement"}

    def timed(lib, budget_s):
        cores = lib.ref_set_threads(host_cores())
        h = lib.ref_net_create(arr, len(specs), 42)
        lib.ref_net_set_params(h, o.p(xavier_params(specs, 42)))
        lib.ref_net_fit(h, o.p(x[0]), o.p(t[0]), BATCH, 1, LOSS_CE, OPT_ADAM, C.byref(hy))  # warm-up
        secs, steps = 0.0, 0
        while secs < budget_s and steps < 200:
            i = (steps + 1) % NB
            secs += lib.ref_net_fit(h, o.p(x[i]), o.p(t[i]), BATCH, 1, LOSS_CE, OPT_ADAM, C.byref(hy))
            steps += 1
        lib.ref_net_destroy(h)
        return BATCH * steps / secs, steps, cores
    value, steps, cores = timed(ref, 10.0)
    out = {"value": value, "unit": "samples/s", "cores": cores, "kind": "reference",
           "sample": f"{steps} mini-batches of {BATCH} through network::fit (backend_t::internal, "
                     f"OpenMP, {cores} threads)"}
    avx = o.load_reference_avx()
    if avx is not None:
        v, n, c = timed(avx, 5.0)
        out["avx"] = {"value": v, "unit": "samples/s", "cores": c,
                      "sample": f"{n} mini-batches of {BATCH} through network::fit, built -DCNN_USE_SSE -DCNN_USE_AVX "
                                "-mavx with backend_t::avx (informational: not the parity target)"}
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--profile", action="store_true",
                    help="short run for a profiler: one timed block per leg, no CPU baseline, no per-kernel timing")
    ap.add_argument("--timeline", default=None, metavar="FILE",
                    help="also write the kernel timeline of one replayed step (rank 0, torch.profiler) to FILE")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.steps is None:
        args.steps = 50 if args.impl == "b200" else 10
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if world != args.gpus:
        if args.gpus != 1 or world != 1:
            raise SystemExit(f"--gpus {args.gpus} needs {args.gpus} ranks (launch with torch.distributed.run); "
                             f"WORLD_SIZE is {world}")
    run_b200(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
