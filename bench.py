#!/usr/bin/env python
"""Benchmark of the mapped-convolution hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (one "step"): spherical mapped convolution forward + backward (input gradient, weight
gradient, bias gradient) on an equirectangular 512 x 1024 image, batch 8 per GPU, 64 -> 64
channels, bf16 activations with fp32 accumulation, 3 x 3 gnomonic kernel (K = 9), bilinear
interpolation, N(0,1) synthetic data, channels-last activations.

Metric: algorithmic TFLOP/s = 3 GEMMs x 2 * B*OH*OW*Cout*Cin*K per step (interpolation flops not
counted), whole job over all GPUs, device time (CUDA events, max over ranks).

  value        inputs resident in HBM when the timed region starts
  e2e          same step through the public layer API with HOST (pinned) buffers: x and the
               upstream gradient are copied in and y, grad_x, grad_w, grad_b are copied out inside
               the timed region
  roofline     the slowest kernel family of the step, timed alone with CUDA events
  cpu_baseline the reference's own CPU extension (or, if it is not built, the C port of it) on
               one batch element of the same workload, on the host's cores

With N > 1 (torchrun) every rank runs the same per-GPU batch (weak scaling) and the weight / bias
gradients are all-reduced over NCCL, the only exchange the path has.

--impl reference times the reference's CPU implementation alone (rank 0 only).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

H, W, KH, KW = 512, 1024, 3, 3
CIN = COUT = 64
K = KH * KW
BATCH = 8  # per GPU


# dram__bytes_read.sum + dram__bytes_write.sum of the family's main kernel per launch at batch 8,
# scaled from ncu captures of a batch-2 case: the activation terms grow with the batch (x 4), the
# effective weights (111 MB, forward / input gradient) and the per-slot partial sums (175 MB, weight
# gradient) do not
DRAM_TRAFFIC_BYTES = {"conv_fwd": 1.07e9, "conv_dgrad": 1.08e9, "conv_wgrad": 2.29e9}


def flops_per_step(batch):
    return 3 * 2.0 * batch * H * W * COUT * CIN * K


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm=d["hbm_gbs"], bf16=d["bf16_tflops"], bf16_sustained=d["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines, self.n0 = index, None, [], 0

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
            # nvidia-smi needs ~0.1 s before its first line: wait for it, so that the sampler is
            # live when the timed region starts; the samples of the region are those after n0
            t0 = time.time()
            while not self.lines and time.time() - t0 < 1.5:
                time.sleep(0.005)
            self.n0 = len(self.lines)
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.th.join(timeout=2)
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        # a region shorter than the sampling period: the last sample before it (the GPU is warm
        # from the warm-up steps by then)
        region = self.lines[self.n0:] or self.lines[-1:]
        for ln in region:
            f = [s.strip() for s in ln.split(",")]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[0]))
                mx = float(f[1])
            except ValueError:
                continue
            for n, v in zip(names, f[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx,
                "reasons": sorted(reasons), "samples": len(sm)}


def _map_builders():
    """The pure-torch sample-map builders, loaded by file path: importing the product package would
    load its CUDA libraries, which the CPU arm must not touch."""
    import importlib
    import types
    name = "_bench_map_builders"
    if name not in sys.modules:  # the util directory as a package of its own, without its __init__
        pkg = types.ModuleType(name)
        pkg.__path__ = [os.path.join(ROOT, "mappedconvolutions_b200", "util")]
        sys.modules[name] = pkg
    return importlib.import_module(name + ".spherical_projections")


def _all_host_threads():
    """torchrun pins OMP_NUM_THREADS=1 for its workers; the CPU legs are meant to use every host
    core this process may run on."""
    import torch
    if _FULL_AFFINITY is not None:  # (undo the NUMA binding of the end-to-end leg)
        os.sched_setaffinity(0, _FULL_AFFINITY)
    ncpu = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    os.environ["OMP_NUM_THREADS"] = str(ncpu)
    torch.set_num_threads(ncpu)
    return ncpu


_FULL_AFFINITY = None  # the CPUs this process could run on before bind_to_gpu_numa_node


def bind_to_gpu_numa_node(index):
    """Runs this process on the CPUs of the NUMA node its GPU hangs off, so that the pinned host
    buffers of the end-to-end leg (first touch) and the copy threads are local to the GPU's PCIe
    root.  Best effort: returns the node, or None where the platform does not tell."""
    try:
        import torch
        p = torch.cuda.get_device_properties(index)
        bdf = "%04x:%02x:%02x.0" % (p.pci_domain_id, p.pci_bus_id, p.pci_device_id)
        node = int(open("/sys/bus/pci/devices/%s/numa_node" % bdf).read())
        if node < 0:
            return None
        cpus = set()
        for part in open("/sys/devices/system/node/node%d/cpulist" % node).read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        global _FULL_AFFINITY
        full = os.sched_getaffinity(0)
        cpus &= full
        if cpus:
            _FULL_AFFINITY = full
            os.sched_setaffinity(0, cpus)
            return node
    except Exception:
        pass
    return None


def make_inputs(batch, seed):
    import torch
    get_projection_map = _map_builders().get_projection_map
    g = torch.Generator().manual_seed(seed)
    bf = torch.bfloat16
    x = torch.randn(batch, CIN, H, W, generator=g).to(bf).contiguous(memory_format=torch.channels_last)
    gy = torch.randn(batch, COUT, H, W, generator=g).to(bf).contiguous(memory_format=torch.channels_last)
    w = torch.randn(COUT, CIN, K, generator=g).to(bf)
    b = torch.randn(COUT, generator=g).to(bf)
    m = get_projection_map((H, W), (KH, KW), "gnomonic")
    return x, gy, w, b, m


# ---------------------------------------------------------------------------------------------
# reference / CPU arm
# ---------------------------------------------------------------------------------------------
def cpu_ops():
    """-> (ops namespace, kind).  The reference's own CPU build if present, else the C port."""
    from oracle import ref
    if ref.available():
        return ref.ops(), "reference"
    from oracle import oracle
    return oracle, "port"


def cpu_step(O, x, gy, w, b, m):
    y = O.mapped_conv_forward(x, m, w, b, K, 1)
    g = O.mapped_conv_backward(gy, m, x, w, b, K, 1)
    return y, g


def cpu_baseline(reps=1, warm=0):
    """fp32 forward + backward of ONE batch element of the workload on the host cores."""
    import torch
    _all_host_threads()
    O, kind = cpu_ops()
    x, gy, w, b, m = make_inputs(1, 1)
    x, gy, w, b = [t.float().contiguous() for t in (x, gy, w, b)]
    for _ in range(warm):
        cpu_step(O, x, gy, w, b, m)
    ts = []
    for _ in range(reps):
        t0 = time.perf_counter()
        cpu_step(O, x, gy, w, b, m)
        ts.append(time.perf_counter() - t0)
    t = statistics.median(ts)
    return dict(value=flops_per_step(1) / t / 1e12, unit="TFLOP/s", cores=torch.get_num_threads(),
                kind=kind, sample="1 of 8 batch elements, fp32 on bf16-rounded inputs, fwd+bwd, "
                "median of %d run(s), %.2f s per run" % (reps, t)), t


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    _all_host_threads()
    O, kind = cpu_ops()
    x, gy, w, b, m = make_inputs(1, 1)
    x, gy, w, b = [t.float().contiguous() for t in (x, gy, w, b)]
    for _ in range(args.warmup):
        cpu_step(O, x, gy, w, b, m)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_step(O, x, gy, w, b, m)
    dt = (time.perf_counter() - t0) / args.steps
    val = flops_per_step(1) / dt / 1e12
    sample = "each step = 1 of the 8 batch elements of the workload, fp32 on bf16-rounded inputs"
    print(json.dumps({
        "impl": "reference", "metric": "mapped-conv fwd+bwd TFLOP/s", "value": val, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": "config2: spherical mapped conv fwd+bwd 512x1024, 64->64, K=9 gnomonic, "
                               "bilinear; CPU sample of batch 1"},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": torch.get_num_threads(),
                         "kind": kind, "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0}))


# ---------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------
def run_ours(args):
    import torch
    import torch.distributed as dist
    from mappedconvolutions_b200 import _lib, ops
    from mappedconvolutions_b200.host import impl as host_ops  # the PyTorch C++ extension
    from mappedconvolutions_b200.dist import allreduce_gradients
    from mapped_convolution.nn import MappedConvolution

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    numa = bind_to_gpu_numa_node(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    L = _lib.lib()

    xh, gyh, w, b, m = make_inputs(BATCH, 1000 + rank)
    x, gy, w, b, m = [t.to(dev) for t in (xh, gyh, w, b, m)]
    x = x.contiguous(memory_format=torch.channels_last)
    gy = gy.contiguous(memory_format=torch.channels_last)

    def step():
        y = host_ops.mapped_conv_forward(x, m, w, b, K, 1)
        gx, gw, gb = host_ops.mapped_conv_backward(gy, m, x, w, b, K, 1)
        if world > 1:
            allreduce_gradients([gw, gb])
        return y, gx, gw, gb

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:  # (before the barrier: its start-up must not delay rank 0 inside the timed region)
        sampler.start()
    barrier()
    n0 = L.mc_kernel_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    launches = L.mc_kernel_launch_count() - n0
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if sampler else None
    # a bounded device-side wait that ran out makes a kernel return early: such a run is no result
    status = L.mc_device_status(torch.cuda.current_stream().cuda_stream, 1)
    assert status == 0, "device status word raised during the timed region: %d" % status
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = t.item()
    ms_step = ms / args.steps
    value = world * flops_per_step(BATCH) / (ms_step * 1e-3) / 1e12

    # ---- end to end through the layer API with host buffers -------------------------------
    layer = MappedConvolution(CIN, COUT, K, "bilinear").to(torch.bfloat16).to(dev)
    with torch.no_grad():
        layer.weight.copy_(w)
        layer.bias.copy_(b)
    xp, gyp = xh.pin_memory(), gyh.pin_memory()
    outs = dict(y=torch.empty_like(gyh).pin_memory(), gx=torch.empty_like(xh).pin_memory(),
                gw=torch.empty(COUT, CIN, K, dtype=torch.bfloat16).pin_memory(),
                gb=torch.empty(COUT, dtype=torch.bfloat16).pin_memory())
    h2d = xp.numel() * 2 + gyp.numel() * 2
    d2h = sum(t.numel() * t.element_size() for t in outs.values())

    # One batch element at a time, so that the upload of element i + 1 and the download of the
    # results of element i - 1 (separate copy engines, separate streams) run under the kernels of
    # element i; the weight / bias gradients accumulate across the elements in the layer.
    # Consecutive steps are pipelined the way a training loop prefetches its next batch: the
    # upload stream may start on step s + 1 while the results of step s are still on their way
    # back (every step still uploads all its inputs and downloads all its results; the timed
    # region ends only when the last download has landed).
    in_s, out_s = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)

    def e2e_step():
        main = torch.cuda.current_stream()
        layer.zero_grad(set_to_none=True)
        for i in range(BATCH):
            with torch.cuda.stream(in_s):
                xd = xp[i:i + 1].to(dev, non_blocking=True)
                gd = gyp[i:i + 1].to(dev, non_blocking=True)
            main.wait_stream(in_s)
            xd.record_stream(main)
            gd.record_stream(main)
            xd.requires_grad_(True)
            y = layer(xd, m)
            y.backward(gd)
            out_s.wait_stream(main)
            with torch.cuda.stream(out_s):
                y.record_stream(out_s)
                xd.grad.record_stream(out_s)
                outs["y"][i:i + 1].copy_(y.detach(), non_blocking=True)
                outs["gx"][i:i + 1].copy_(xd.grad, non_blocking=True)
        if world > 1:
            allreduce_gradients([layer.weight.grad, layer.bias.grad])
        outs["gw"].copy_(layer.weight.grad, non_blocking=True)
        outs["gb"].copy_(layer.bias.grad, non_blocking=True)

    def e2e_drain():
        main = torch.cuda.current_stream()
        main.wait_stream(out_s)
        main.wait_stream(in_s)

    e2e_steps = max(2, min(args.steps, 5))
    for _ in range(2):
        e2e_step()
    e2e_drain()
    barrier()
    in_s.wait_stream(torch.cuda.current_stream())
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e2e_drain()
    e1.record()
    barrier()
    ms_e = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms_e], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_e = t.item()
    e2e_val = world * flops_per_step(BATCH) / (ms_e / e2e_steps * 1e-3) / 1e12

    # ---- per-kernel timing for the roofline (rank 0, each family alone) ---------------------
    roof = cpu = None
    if rank == 0:
        def timed(fn, n=5):
            fn()
            torch.cuda.synchronize()
            a, c = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(n):
                fn()
            c.record()
            torch.cuda.synchronize()
            return a.elapsed_time(c) / n

        # each family through the extension, as the step runs it: forward; input gradient only;
        # weight + bias gradient only (each includes its few microseconds of helper kernels)
        fwd = lambda: host_ops.mapped_conv_forward(x, m, w, b, K, 1)
        dgrad = lambda: host_ops.mapped_conv_backward(gy, m, x, w, b, K, 1, True, False)
        wgrad = lambda: host_ops.mapped_conv_backward(gy, m, x, w, b, K, 1, False, True)
        fam = {"conv_fwd": fwd, "conv_dgrad": dgrad, "conv_wgrad": wgrad}
        times = {k: timed(f) for k, f in fam.items()}
        top = max(times, key=times.get)
        pk = peaks()
        gemm_flops = flops_per_step(BATCH) / 3
        ach = gemm_flops / (times[top] * 1e-3) / 1e12
        traffic = DRAM_TRAFFIC_BYTES.get(top)
        roof = {"bound": "tensor", "kernel": top, "achieved": ach, "peak": pk["bf16"],
                "unit": "TFLOP/s", "frac": ach / pk["bf16"], "traffic": traffic,
                "peak_source": pk["source"] + " burst bf16 (kernel timed alone)",
                "ms_per_launch": {k: round(v, 4) for k, v in times.items()},
                "tflops": {k: round(gemm_flops / (v * 1e-3) / 1e12, 2) for k, v in times.items()}}
        if not args.no_cpu:
            cpu, _ = cpu_baseline()

    # ---- the other configurations of the path, in the same JSON line --------------------------
    # config 5 (encoder training step, the fixed batch of 64 split over the ranks: strong scaling) at
    # every N; configs 3 / 4 (resample, pooling, k-NN: no exchange step, "replicas only") on one GPU.
    # Each timed region lasts at least a second so that the clock sampler sees it.
    secondary = []
    if not args.no_secondary:
        del x, gy, xp, gyp, outs
        torch.cuda.empty_cache()
        enc = encoder_record(10, 3, min_seconds=1.0)
        if rank == 0:
            secondary.append(enc)
            if world == 1:
                for wl in ("resample", "pool", "knn"):
                    torch.cuda.empty_cache()
                    secondary.append(secondary_record(wl, 10, 3, args.no_cpu, min_seconds=1.0))

    if rank == 0:
        print(json.dumps({
            "metric": "mapped-conv fwd+bwd TFLOP/s", "value": value, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "config2: spherical mapped conv fwd+bwd, equirect 512x1024, batch 8 "
                                   "per GPU, 64->64 ch, K=9 gnomonic map, bilinear, channels-last",
                       "l2": "inputs (537 MB per activation tensor) are larger than L2",
                       "parallelism": "batch-sharded dp%d, NCCL allreduce of grad_w/grad_b" % world,
                       "numa_node": numa},
            "clocks": clocks,
            "e2e": {"value": e2e_val, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": ms_e / e2e_steps},
            "gpu_launches": int(launches), "device_status": int(status),
            "roofline": roof, "cpu_baseline": cpu, "secondary": secondary}))
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------
# secondary workloads (--workload resample | pool | knn): the other configs of the path, same
# timing rules, one JSON line each.  The default run (conv) is the headline line.
# ---------------------------------------------------------------------------------------------
def secondary_record(wl, steps, warmup, no_cpu, min_seconds=0.0):
    """One record (a dict with the keys of the headline line) for a secondary workload: 'resample'
    (config 3), 'pool' (config 4) or 'knn' (config 4).  The timed region runs `steps` steps, or as
    many more as it takes to last `min_seconds`, so that the clock sampler sees it."""
    import torch
    from mappedconvolutions_b200 import _lib
    from mappedconvolutions_b200.host import impl as ops  # the PyTorch C++ extension
    from mappedconvolutions_b200 import util as mutil
    from mappedconvolutions_b200.util import icosphere as ico

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    L = _lib.lib()
    g = torch.Generator().manual_seed(0)
    cpu = None
    if wl == "resample":
        # config 3: equirect 512x1024x3 fp32 image (U[0,1]), batch 16, <-> icosphere level-7 vertices
        img_h = torch.rand(16, 3, 512, 1024, generator=g)
        m = mutil.image_to_sphere_resample_map((512, 1024), mutil.generate_icosphere(7))
        img, md = img_h.to(dev), m.to(dev)
        verts = ops.resample_from_map(img, md, 1)

        def step():
            v = ops.resample_from_map(img, md, 1)          # image -> vertices (gather, "Unresample")
            return ops.resample_to_map(v, md, 512, 1024, 1)  # vertices -> image (scatter, "Resample")
        algo_bytes = 2 * 133.4e6
        unit, metric = "GB/s", "resample gather+scatter GB/s"
        fam = {"gather": (lambda: ops.resample_from_map(img, md, 1), 133.4e6),
               "scatter": (lambda: ops.resample_to_map(verts, md, 512, 1024, 1), 133.4e6)}
        host_in, host_out = img_h.pin_memory(), torch.empty(16, 3, 512, 1024).pin_memory()

        def e2e_step():
            d_in = host_in.to(dev, non_blocking=True)
            v = ops.resample_from_map(d_in, md, 1)
            host_out.copy_(ops.resample_to_map(v, md, 512, 1024, 1), non_blocking=True)
        h2d, d2h = host_in.numel() * 4, host_out.numel() * 4
        workload = ("config3: resample equirect 512x1024x3 fp32 batch 16 -> icosphere-7 vertices "
                    "(bilinear gather) and back (weighted scatter-add)")

        def cpu_fn():
            O, kind = cpu_ops()
            a, mm = img_h[:4].contiguous(), m
            t0 = time.perf_counter()
            v = O.resample_from_map(a, mm, 1)
            O.resample_to_map(v, mm, 512, 1024, 1)
            dt = time.perf_counter() - t0
            return dict(value=algo_bytes / 4 / dt / 1e9, unit="GB/s", cores=torch.get_num_threads(),
                        kind=kind, sample="4 of 16 batch elements, gather + scatter, %.3f s" % dt)
    elif wl == "pool":
        # config 4: icosphere level 7 -> 6, 7-tap one-ring, nearest, batch 32, 128 ch, fp32
        x = torch.randn(32, 128, 1, ico.num_vertices(7), generator=g).to(dev)
        m = ico.pooling_map(7)
        md = m.to(dev)

        def step():
            return ops.mapped_avg_pool(x, md, 7, 0), ops.mapped_max_pool(x, md, 7, 0)
        algo_bytes = 3.358e9 + 4.700e9
        unit, metric = "GB/s", "mapped avg+max pool GB/s"
        x_cl = x.contiguous(memory_format=torch.channels_last)
        fam = {"avg_pool": (lambda: ops.mapped_avg_pool(x, md, 7, 0), 3.358e9),
               "max_pool": (lambda: ops.mapped_max_pool(x, md, 7, 0), 4.700e9),
               "avg_pool_channels_last": (lambda: ops.mapped_avg_pool(x_cl, md, 7, 0), 3.358e9),
               "max_pool_channels_last": (lambda: ops.mapped_max_pool(x_cl, md, 7, 0), 4.700e9)}
        xs_h = x[:4].cpu().pin_memory()
        out_h = torch.empty(4, 128, 1, ico.num_vertices(6)).pin_memory()

        def e2e_step():  # a 4-element slice of the batch keeps the pinned buffers modest
            xd = xs_h.to(dev, non_blocking=True)
            out_h.copy_(ops.mapped_avg_pool(xd, md, 7, 0), non_blocking=True)
            out_h.copy_(ops.mapped_max_pool(xd, md, 7, 0)[0], non_blocking=True)
        h2d, d2h = xs_h.numel() * 4, 2 * out_h.numel() * 4
        workload = ("config4: icosphere mapped avg + max pool level 7 -> 6, 7-tap one-ring, nearest, "
                    "batch 32, 128 ch, fp32 (NCHW)")

        def cpu_fn():
            O, kind = cpu_ops()
            a = xs_h[:2].contiguous()
            t0 = time.perf_counter()
            O.mapped_avg_pool(a, m, 7, 0)
            O.mapped_max_pool(a, m, 7, 0)
            dt = time.perf_counter() - t0
            return dict(value=algo_bytes / 16 / dt / 1e9, unit="GB/s", cores=torch.get_num_threads(),
                        kind=kind, sample="2 of 32 batch elements, avg + max pool, %.3f s" % dt)
    else:
        # config 4b: k = 9 nearest neighbours among the 163 842 unit-sphere vertices of level 7
        p_h = mutil.generate_icosphere(7).get_vertices().t().contiguous().unsqueeze(0)
        p = p_h.to(dev)
        n = p.shape[2]

        def step():
            return ops.knn_forward(p, p, 9)
        algo_bytes = float(n) * n  # pairs
        unit, metric = "Gpairs/s", "knn pairs/s (k=9, 163842 points)"
        fam = {"knn": (step, float(n) * n)}
        ph = p_h.pin_memory()
        idx_h = torch.empty(1, 9, n, dtype=torch.int64).pin_memory()

        def e2e_step():
            pd = ph.to(dev, non_blocking=True)
            idx_h.copy_(ops.knn_forward(pd, pd, 9)[0], non_blocking=True)
        h2d, d2h = ph.numel() * 4, idx_h.numel() * 8
        workload = "config4: KNN k=9 over 163842 level-7 icosphere vertices (3-D, fp32), ref = query"

        def cpu_fn():
            from oracle import oracle
            q = p_h[:, :, :2048].contiguous()
            t0 = time.perf_counter()
            oracle.knn_forward(p_h, q, 9)
            dt = time.perf_counter() - t0
            return dict(value=2048.0 * n / dt / 1e9, unit="Gpairs/s", cores=os.cpu_count(),
                        kind="port", sample="2048 of 163842 queries against all references (the "
                        "reference has no CPU KNN; C restatement), %.3f s" % dt)

    def timed(fn, n):
        a, c = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        for _ in range(n):
            fn()
        c.record()
        torch.cuda.synchronize()
        return a.elapsed_time(c) / n

    for _ in range(max(warmup, 3)):
        step()
    if min_seconds > 0:
        steps = max(steps, int(min_seconds * 1e3 / max(timed(step, 3), 1e-3)) + 1)
    sampler = ClockSampler(dev.index)
    sampler.start()
    n0 = L.mc_kernel_launch_count()
    ms = timed(step, steps)
    launches = L.mc_kernel_launch_count() - n0
    clocks = sampler.stop()
    status = L.mc_device_status(torch.cuda.current_stream().cuda_stream, 1)
    for _ in range(2):
        e2e_step()
    ms_e = timed(e2e_step, max(2, min(steps, 5)))
    times = {}
    for k, (fn, _) in fam.items():
        fn()
        times[k] = timed(fn, 10)
    top = max(times, key=times.get)
    pk = peaks()
    scale = 1e9
    ach = fam[top][1] / (times[top] * 1e-3) / scale
    if wl == "knn":
        roof = {"bound": "fp32 CUDA cores (no HBM or tensor roofline applies)", "kernel": top,
                "achieved": ach, "unit": unit, "peak": None, "frac": None, "traffic": None,
                "ms_per_launch": {k: round(v, 4) for k, v in times.items()}}
    else:
        roof = {"bound": "hbm", "kernel": top, "achieved": ach, "peak": pk["hbm"], "unit": "GB/s",
                "frac": ach / pk["hbm"], "traffic": None, "peak_source": pk["source"] + " copy bandwidth",
                "ms_per_launch": {k: round(v, 4) for k, v in times.items()},
                "gbs": {k: round(fam[k][1] / (v * 1e-3) / 1e9, 1) for k, v in times.items()}}
    if not no_cpu:
        _all_host_threads()
        cpu = cpu_fn()
    e2e_frac = {"resample": 1.0, "pool": 4.0 / 32.0, "knn": 1.0}[wl]
    return {
        "metric": metric, "value": algo_bytes / (ms * 1e-3) / scale, "unit": unit, "n_gpus": 1,
        "steps": steps, "warmup": max(warmup, 3), "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": workload}, "clocks": clocks,
        "e2e": {"value": algo_bytes * e2e_frac / (ms_e * 1e-3) / scale, "unit": unit,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": ms_e},
        "gpu_launches": int(launches), "device_status": int(status), "roofline": roof,
        "cpu_baseline": cpu}


def run_secondary(args):
    print(json.dumps(secondary_record(args.workload, args.steps, args.warmup, args.no_cpu)))


# ---------------------------------------------------------------------------------------------
# --workload encoder: config 5, an icosphere level-7 encoder training step.  Four mapped
# convolutions (3 -> 64 -> 128 -> 256 -> 256 channels, 7-tap one-ring maps, nearest) each followed
# by ReLU, mapped average pooling 7 -> 6 -> 5 between them; batch 64 in all, sharded over the
# ranks (strong scaling); weight gradients all-reduced over NCCL; plain SGD update.
# ---------------------------------------------------------------------------------------------
ENC_CH = (3, 64, 128, 256, 256)
ENC_LEVEL = (7, 6, 5, 5)  # mesh level each convolution runs at
ENC_BATCH = 64


def encoder_flops(batch):
    """fwd + dgrad + wgrad GEMM flops of the four convolutions (the first has no dgrad)."""
    from mappedconvolutions_b200 import util as mutil
    from mappedconvolutions_b200.util import icosphere as ico
    tot = 0.0
    for i in range(4):
        gemm = 2.0 * batch * ico.num_vertices(ENC_LEVEL[i]) * 7 * ENC_CH[i] * ENC_CH[i + 1]
        tot += gemm * (2 if i == 0 else 3)
    return tot


def encoder_record(steps, warmup, min_seconds=0.0):
    """The config-5 record (a dict; None on ranks other than 0).  Uses the process group the caller
    has set up; the fixed batch of 64 is split over the ranks."""
    import torch
    import torch.distributed as dist
    from mappedconvolutions_b200 import _lib, nn as mnn, dist as mdist
    from mappedconvolutions_b200.util import icosphere as ico

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    L = _lib.lib()
    lo, hi = mdist.shard_batch(ENC_BATCH, rank, world)
    nb = hi - lo
    torch.manual_seed(0)
    convs = torch.nn.ModuleList(
        [mnn.MappedConvolution(ENC_CH[i], ENC_CH[i + 1], 7, "nearest", activation="relu")
         for i in range(4)]).to(dev).to(torch.bfloat16)  # (ReLU in the conv kernel's epilogue)
    kmap = {l: ico.vertex_kernel_map(l).to(dev) for l in (7, 6, 5)}
    pmap = {l: ico.pooling_map(l).to(dev) for l in (7, 6)}
    pool = mnn.MappedAvgPool(7, "nearest")
    g = torch.Generator().manual_seed(1)
    x_h = torch.randn(ENC_BATCH, 3, 1, ico.num_vertices(7), generator=g).to(torch.bfloat16)[lo:hi]
    x_h = x_h.contiguous(memory_format=torch.channels_last).pin_memory()
    x = x_h.to(dev)
    params = [p for p in convs.parameters()]
    lr = 1e-3

    class MeanLoss(torch.autograd.Function):
        """loss = h.float().mean().  torch's own backward of mean() expands the scalar into a dense
        NCHW tensor; next to the channels-last activations of the layers that costs three strided
        passes per step (the expansion, a mixed-layout ReLU gradient, a copy back to channels-last).
        This backward writes the constant gradient once, in the activation's own layout."""

        @staticmethod
        def forward(ctx, h):
            ctx.save_for_backward(h)
            return h.mean(dtype=torch.float32)

        @staticmethod
        def backward(ctx, g):
            (h,) = ctx.saved_tensors
            return torch.empty_like(h).copy_((g / h.numel()).to(h.dtype))

    def step(xin):
        h = convs[0](xin, kmap[7])
        h = pool(h, pmap[7])
        h = convs[1](h, kmap[6])
        h = pool(h, pmap[6])
        h = convs[2](h, kmap[5])
        h = convs[3](h, kmap[5])
        loss = MeanLoss.apply(h)  # (float32 accumulation straight from the bf16 activation)
        loss.backward()
        grads = [p.grad for p in params]
        if world > 1:
            mdist.allreduce_gradients(grads)
        with torch.no_grad():
            torch._foreach_add_(params, grads, alpha=-lr)
        for p in params:
            p.grad = None
        return loss

    def sync():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(fn, n):
        a, c = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sync()
        a.record()
        for _ in range(n):
            fn()
        c.record()
        sync()
        t = torch.tensor([a.elapsed_time(c)], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for _ in range(max(warmup, 3)):
        step(x)
    if min_seconds > 0:  # (the same count on every rank: timed() takes the max over ranks)
        steps = max(steps, int(min_seconds * 1e3 / max(timed(lambda: step(x), 3) / 3, 1e-3)) + 1)
    sampler = ClockSampler(dev.index) if rank == 0 else None
    if sampler:
        sampler.start()
    n0 = L.mc_kernel_launch_count()
    ms = timed(lambda: step(x), steps) / steps
    launches = L.mc_kernel_launch_count() - n0
    clocks = sampler.stop() if sampler else None
    loss_h = torch.empty(1, dtype=torch.float32).pin_memory()

    def e2e_step():
        xd = x_h.to(dev, non_blocking=True)
        loss_h.copy_(step(xd).detach().reshape(1), non_blocking=True)
    for _ in range(2):
        e2e_step()
    ne = max(2, min(steps, 5))
    ms_e = timed(e2e_step, ne) / ne
    status = L.mc_device_status(torch.cuda.current_stream().cuda_stream, 1)
    fl = encoder_flops(ENC_BATCH)
    rec = None
    if rank == 0:
        pk = peaks()
        val = fl / (ms * 1e-3) / 1e12
        rec = ({
            "metric": "mapped-conv fwd+bwd TFLOP/s (encoder step)", "value": val, "unit": "TFLOP/s",
            "n_gpus": world, "steps": steps, "warmup": max(warmup, 3), "ms_per_step": ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": "config5: icosphere level-7 encoder training step, batch 64 in all, "
                                   "conv 3->64->128->256->256 (7-tap one-ring, nearest) + ReLU, avg pool "
                                   "7->6->5, SGD, channels-last bf16",
                       "l2": "activations of the first two levels (1.3 GB, 0.7 GB per rank at N=1) are larger than L2",
                       "parallelism": "batch-sharded dp%d, NCCL allreduce of weight gradients" % world,
                       "flops": "conv GEMM flops only (fwd + dgrad + wgrad; no dgrad for the first layer)"},
            "clocks": clocks,
            "e2e": {"value": fl / (ms_e * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": x_h.numel() * 2, "d2h_bytes_per_step": 4, "ms_per_step": ms_e},
            "gpu_launches": int(launches), "device_status": int(status),
            "roofline": {"bound": "tensor", "achieved": val / world, "peak": pk["bf16_sustained"],
                         "unit": "TFLOP/s", "frac": val / world / pk["bf16_sustained"],
                         "traffic": None, "note": "whole step (conv kernels, ReLU, pooling, update) per GPU against the bf16 GEMM peak"},
            "cpu_baseline": None})
    return rec


def run_encoder(args):
    import torch
    import torch.distributed as dist
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
    world = int(os.environ.get("WORLD_SIZE", "1"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    rec = encoder_record(args.steps, args.warmup)
    if rec is not None:
        print(json.dumps(rec))
    if world > 1:
        dist.destroy_process_group()


def run_profile_case(args):
    """Small case for profiler captures: the config-2 tensors at a reduced batch, three calls of the
    forward (or backward) op and nothing else, so that `-k <kernel> -s <skip> -c <count>` picks a
    warm launch.  Prints no bench line."""
    import torch
    from mappedconvolutions_b200 import ops
    from mappedconvolutions_b200.util import get_projection_map
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    B = args.batch
    if args.profile_case == "knn":  # config 4's k-NN on the 40 962 vertices of level 6
        from mappedconvolutions_b200 import util as mutil
        from mappedconvolutions_b200.util import icosphere as ico
        p = mutil.generate_icosphere(6).get_vertices().t().contiguous().unsqueeze(0).to(dev)
        for _ in range(3):
            ops.knn_forward(p, p, 9)
        torch.cuda.synchronize()
        print("profile case knn done")
        return
    if args.profile_case == "pool":  # config 4 at a reduced batch: avg pool, max pool, avg unpool
        from mappedconvolutions_b200 import util as mutil
        from mappedconvolutions_b200.util import icosphere as ico
        x = torch.randn(B, 128, 1, ico.num_vertices(7), device=dev)
        pm = ico.pooling_map(7).to(dev)
        for _ in range(3):
            y = ops.mapped_avg_pool(x, pm, 7, 0)
            ops.mapped_max_pool(x, pm, 7, 0)
            ops.mapped_avg_unpool(y, pm, 1, x.shape[3], 7, 0)
        torch.cuda.synchronize()
        print("profile case pool batch %d done" % B)
        return
    if args.profile_case == "first":  # config 5's first layer: 3 -> 64 channels on level-7 vertices
        from mappedconvolutions_b200 import util as mutil
        from mappedconvolutions_b200.util import icosphere as ico
        n = ico.num_vertices(7)
        cl = lambda t: t.to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        x1 = cl(torch.randn(B, 3, 1, n, device=dev))
        g1 = cl(torch.randn(B, 64, 1, n, device=dev))
        w1 = (torch.randn(64, 3, 7, device=dev) * 0.1).to(torch.bfloat16)
        b1 = torch.zeros(64, device=dev, dtype=torch.bfloat16)
        km = ico.vertex_kernel_map(7).to(dev).contiguous()
        for _ in range(3):
            ops.mapped_conv_forward(x1, km, w1, b1, 7, 0)
            ops.mapped_conv_backward(g1, km, x1, w1, b1, 7, 0, need_input_grad=False)
        torch.cuda.synchronize()
        print("profile case first batch %d done" % B)
        return
    if args.profile_case == "resample":  # config 3: gather to the level-7 vertices and scatter back
        from mappedconvolutions_b200 import util as mutil
        from mappedconvolutions_b200.util import icosphere as ico
        img = torch.rand(B, 3, 512, 1024, device=dev)
        rm = mutil.image_to_sphere_resample_map((512, 1024), mutil.generate_icosphere(7)).to(dev)
        for _ in range(3):
            v = ops.resample_from_map(img, rm, 1)
            ops.resample_to_map(v, rm, 512, 1024, 1)
        torch.cuda.synchronize()
        print("profile case resample batch %d done" % B)
        return
    bf = lambda *shape: torch.randn(*shape, device=dev).to(torch.bfloat16)
    x = bf(B, CIN, H, W).contiguous(memory_format=torch.channels_last)
    gy = bf(B, COUT, H, W).contiguous(memory_format=torch.channels_last)
    w, b = bf(COUT, CIN, K), bf(COUT)
    m = get_projection_map((H, W), (3, 3), "gnomonic").to(dev)
    # through the compiled binding, as the bench step runs it (row plans for this map);
    # --general-kernels: the kernels for maps without a row plan
    from mappedconvolutions_b200.host import impl as host_ops, COMPILED
    if args.general_kernels and COMPILED:
        host_ops.set_row_plans(False)
    for _ in range(3):
        if args.profile_case == "fwd":
            host_ops.mapped_conv_forward(x, m, w, b, K, 1)
        else:
            host_ops.mapped_conv_backward(gy, m, x, w, b, K, 1)
    torch.cuda.synchronize()
    print("profile case %s batch %d done" % (args.profile_case, B))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="conv", choices=["conv", "resample", "pool", "knn", "encoder"],
                    help="conv (default) is the headline config; the others are the remaining configs")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-secondary", action="store_true",
                    help="headline workload only: skip the records of configs 3, 4 and 5")
    ap.add_argument("--profile-case", choices=["fwd", "bwd", "pool", "knn", "resample", "first"],
                    help="run three calls of the config-2 forward / backward at --batch and exit "
                         "(small case for profiler captures)")
    ap.add_argument("--batch", type=int, default=2, help="batch of --profile-case")
    ap.add_argument("--general-kernels", action="store_true",
                    help="--profile-case fwd|bwd: the kernels for maps without a row plan")
    args = ap.parse_args()
    if args.profile_case:
        run_profile_case(args)
    elif args.impl == "reference":
        run_reference(args)
    elif args.workload == "encoder":
        run_encoder(args)
    elif args.workload != "conv":
        run_secondary(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
