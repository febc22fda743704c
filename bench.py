"""Benchmark of the block-sparse matmul path (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config config2] [--impl ours|reference]

One step = one forward product O = X·Y plus the two backward products dX = dO·Yᵀ, dY = Xᵀ·dO of
the workload (three launches of the native matmul kernel on pre-built plans; LUTs and plans
are built before the timed region, as the reference's warm ``layout_cache`` would be).

The default workload is the bf16 SDD case: X, Y (16, 2048, 2048), block 64, Bernoulli(0.25)
layouts from seed 1, exact inferred output layout, values N(0, 1/sqrt(K)), dO ~ N(0, 1).  Data is
synthetic (seeded); four input/output buffer sets are rotated so that no step finds its operands
in the 126 MB L2.

Prints ONE JSON line.  ``value`` is effective TFLOP/s (FLOPs of non-zero block pairs only) with
inputs resident in HBM; ``e2e`` is the same metric through ``blksprs_b200.ops.matmul`` + autograd
with pinned host buffers copied in and results copied out every step.  ``--impl reference`` times
the CPU oracle (dense masked matmul, all host threads) on the same workload instead.
With N > 1 (torchrun) every rank runs its own batch slice of an N-times larger batch (weak
scaling, no data-path collective); the timed region is bracketed by barriers and the maximum over
ranks is reported.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "block-sparse matmul effective TFLOP/s (nnz-block FLOPs), forward+backward"
N_BUFFER_SETS = 4

# DRAM bytes (read + write) of one forward launch of the default workload (config2), from the ncu
# capture summarised in profiles/matmul_umma_kernel_config2.md: 68.7 MB read + 73.5 MB written (the
# capture replays one launch on the same buffers, so part of the data is served from L2).
FWD_KERNEL_DRAM_TRAFFIC_BYTES = {"config2": 142.2e6}


# ---------------------------------------------------------------------------------------------
# workloads
# ---------------------------------------------------------------------------------------------

def _gen(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


def exact_output_layout(lx: torch.Tensor, ly: torch.Tensor) -> torch.Tensor:
    return torch.matmul(lx.float(), ly.float()) != 0


def workload_layouts(name: str, batch: int | None = None, seed_shift: int = 0):
    """CPU bool layouts (lx, ly, lo), block size and dtype of a named workload."""
    if name == "config1":
        g = _gen(0 + seed_shift)
        B = batch or 2
        lx = torch.rand((B, 8, 8), generator=g) < 0.5
        ly = torch.rand((B, 8, 8), generator=g) < 0.5
        for layout in (lx, ly):
            for b in range(B):
                if not layout[b].any():
                    layout[b, 0, 0] = True
        return lx, ly, torch.ones((B, 8, 8), dtype=torch.bool), 16, torch.float32
    if name == "config2":
        g = _gen(1 + seed_shift)
        B = batch or 16
        lx = torch.rand((B, 32, 32), generator=g) < 0.25
        ly = torch.rand((B, 32, 32), generator=g) < 0.25
        return lx, ly, exact_output_layout(lx, ly), 64, torch.bfloat16
    if name == "config3":
        B = batch or 512
        lx = torch.ones((B, 64, 2), dtype=torch.bool)
        ly = torch.ones((B, 2, 64), dtype=torch.bool)
        i = torch.arange(64)[:, None]
        j = torch.arange(64)[None, :]
        band = (j <= i) & ((i - j <= 7) | (j == 0))
        return lx, ly, band[None].expand(B, 64, 64).contiguous(), 64, torch.float16
    if name == "config4":
        g = _gen(2 + seed_shift)
        B = batch or 512
        lx = torch.rand((B, 64, 64), generator=g) < 0.25
        empty_rows = ~lx.any(-1)
        lx[..., 0] |= empty_rows
        ly = torch.ones((B, 64, 2), dtype=torch.bool)
        return lx, ly, torch.ones((B, 64, 2), dtype=torch.bool), 64, torch.bfloat16
    if name == "config5":
        g = _gen(3 + seed_shift)
        B = batch or 256
        lx = torch.rand((B, 32, 32), generator=g) < 0.10
        ly = torch.ones((B, 32, 8), dtype=torch.bool)
        return lx, ly, exact_output_layout(lx, ly), 128, torch.bfloat16
    raise ValueError(f"unknown workload {name}")


def workload_values(name: str, lx, ly, lo, bs, dtype, seed: int, device="cpu"):
    """Compressed x, y and grad-output tensors of a workload, generated on ``device``."""
    g = torch.Generator(device=device)
    g.manual_seed(1000 + seed)
    nx, ny, no = int(lx.sum()), int(ly.sum()), int(lo.sum())
    K = lx.size(2) * bs

    def randn(n, scale=1.0):
        return (torch.randn((n, bs, bs), generator=g, device=device, dtype=torch.float32) * scale).to(dtype)

    if name == "config2":
        x, y = randn(nx, 1 / math.sqrt(K)), randn(ny, 1 / math.sqrt(K))
    elif name == "config3":
        x, y = randn(nx, 1 / math.sqrt(128)), randn(ny, 1 / math.sqrt(128))
    elif name == "config4":
        # row-wise softmax over each row's active blocks (inactive = -inf), fp32, then cast
        logits = torch.randn((nx, bs, bs), generator=g, device=device, dtype=torch.float32)
        lut = torch.nonzero(lx).to(device)
        row_id = lut[:, 0] * lx.size(1) + lut[:, 1]
        n_rows = lx.size(0) * lx.size(1)
        e = torch.exp(logits - logits.amax())
        sums = torch.zeros((n_rows, bs), device=device).index_add_(0, row_id, e.sum(-1))
        x = (e / sums[row_id][:, :, None]).to(dtype)
        y = randn(ny)
    elif name == "config5":
        x, y = randn(nx, 0.02), randn(ny, 0.02)
    else:
        x, y = randn(nx), randn(ny)
    return x, y, randn(no)


def work_model(lx, ly, lo, bs, elem_bytes):
    """Pairs, FLOPs and compulsory bytes of the three products (each operand block that takes part
    in a pair read once, each output block written once)."""
    xf, yf, of = lx.float(), ly.float(), lo.float()
    fwd_pairs = (torch.matmul(xf, yf) * of).sum().item()
    dx_pairs = (torch.matmul(of, yf.transpose(-1, -2)) * xf).sum().item()
    dy_pairs = (torch.matmul(xf.transpose(-1, -2), of) * yf).sum().item()
    blk = bs * bs * elem_bytes
    x_used_f = ((torch.matmul(of, yf.transpose(-1, -2)) > 0) & lx).sum().item()   # x blocks with a partner
    y_used_f = ((torch.matmul(xf.transpose(-1, -2), of) > 0) & ly).sum().item()
    o_used_dx = ((torch.matmul(xf, yf) > 0) & lo).sum().item()                    # dO blocks with a partner
    fwd_bytes = (x_used_f + y_used_f + lo.sum().item()) * blk
    dx_bytes = (o_used_dx + y_used_f + lx.sum().item()) * blk
    dy_bytes = (x_used_f + o_used_dx + ly.sum().item()) * blk
    f = 2 * bs ** 3
    return {
        "pairs": {"fwd": int(fwd_pairs), "dx": int(dx_pairs), "dy": int(dy_pairs)},
        "flops": {"fwd": fwd_pairs * f, "dx": dx_pairs * f, "dy": dy_pairs * f},
        "bytes": {"fwd": fwd_bytes, "dx": dx_bytes, "dy": dy_bytes},
    }


# ---------------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------------

class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        names = {
            nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
            nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.005)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


def physical_gpu_index(local_index: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_index])
        except (ValueError, IndexError):
            pass
    return local_index


# ---------------------------------------------------------------------------------------------
# CPU arm (the oracle, timed): dense masked matmul forward + backward
# ---------------------------------------------------------------------------------------------

def cpu_step_time(name: str, sample_batch: int, steps: int, warmup: int):
    """Seconds per step of the CPU oracle on ``sample_batch`` batches of the workload, and the
    effective FLOPs of that sample."""
    from oracle import oracle
    lx, ly, lo, bs, dtype = workload_layouts(name, batch=sample_batch)
    x, y, g = workload_values(name, lx, ly, lo, bs, dtype, seed=0)
    wm = work_model(lx, ly, lo, bs, x.element_size())
    flops = sum(wm["flops"].values())
    torch.set_num_threads(os.cpu_count() or 1)

    def step():
        out = oracle.matmul_forward(x, lx, y, ly, lo, bs)
        gx, gy = oracle.matmul_backward(g, x, lx, y, ly, lo, bs)
        return out, gx, gy

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    return dt, flops


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    lx, _, _, _, _ = workload_layouts(args.config)
    full_batch = lx.size(0)
    sample = min(full_batch, args.cpu_batch)
    dt, flops = cpu_step_time(args.config, sample, max(args.steps, 1), max(args.warmup, 1))
    value = flops / dt / 1e12
    cores = torch.get_num_threads()
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3 * full_batch / sample,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32 (bf16 inputs upcast)",
        "data": "synthetic (seeded)",
        "config": {"workload": args.config, "note": "CPU dense masked-matmul oracle; blksprs has no CPU path"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                         "sample": f"{sample} of {full_batch} batches per step, fwd+bwd"},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------

def run_triton_arm(args):
    """Times the reference's own Triton op (installed under baseline/_ref) on the same workload:
    ``bs.ops.matmul`` forward + ``backward`` with a warm ``layout_cache``, DEFAULT autotune profile."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    line = {"impl": "triton-reference", "metric": METRIC, "unit": "TFLOP/s"}
    try:
        sys.path.insert(0, ref_dir)
        os.environ.setdefault("BLKSPRS_AUTOTUNE", "DEFAULT")
        import blksprs as ref
    except Exception as exc:  # not installed on this box
        line["unavailable"] = f"reference not importable from baseline/_ref: {exc!r}"[:200]
        print(json.dumps(line), flush=True)
        return
    dev = torch.device("cuda", 0)
    lx, ly, lo, bsz, dtype = workload_layouts(args.config)
    wm = work_model(lx, ly, lo, bsz, torch.empty((), dtype=dtype).element_size())
    lxd, lyd, lod = lx.to(dev), ly.to(dev), lo.to(dev)
    sets = [workload_values(args.config, lx, ly, lo, bsz, dtype, seed=s, device=dev) for s in range(N_BUFFER_SETS)]
    results = {}
    for label, validate in (("validation_on", True), ("validation_off", False)):
        (ref.utils.enable_validation if validate else ref.utils.disable_validation)()
        cache = {}

        def step(i, fwd_only=False):
            x, y, g = sets[i % N_BUFFER_SETS]
            x = x.detach().requires_grad_(not fwd_only)
            y = y.detach().requires_grad_(not fwd_only)
            out = ref.ops.matmul(x, lxd, y, lyd, lod, bsz, cache)
            if not fwd_only:
                out.backward(g)
            return out

        for mode, flops in (("fwd", wm["flops"]["fwd"]), ("fwd_bwd", sum(wm["flops"].values()))):
            for i in range(max(args.warmup, 3)):
                step(i, mode == "fwd")
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            for i in range(args.steps):
                step(i, mode == "fwd")
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / args.steps
            results[f"{label}/{mode}"] = {"ms_per_step": ms, "tflops": flops / (ms * 1e-3) / 1e12}
    ref.utils.enable_validation()
    line.update({"value": results["validation_off/fwd_bwd"]["tflops"], "results": results,
                 "config": {"workload": args.config}, "steps": args.steps, "warmup": args.warmup,
                 "triton": __import__("triton").__version__})
    print(json.dumps(line), flush=True)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def run_gpu_arm(args):
    import torch.distributed as dist
    import blksprs_b200 as bs
    from blksprs_b200 import _cabi
    from blksprs_b200.ops.matmul import matmul_build_layout_cache, _backward_plans, _PLANS
    from blksprs_b200.plan import check_device_status

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    # each rank owns its own batch slice (own seed) of a world-times larger batch: weak scaling
    lx, ly, lo, bsz, dtype = workload_layouts(args.config, seed_shift=100 * rank)
    wm = work_model(lx, ly, lo, bsz, torch.empty((), dtype=dtype).element_size())
    flops_step = sum(wm["flops"].values())
    lxd, lyd, lod = lx.to(dev), ly.to(dev), lo.to(dev)
    sets = []
    for s in range(N_BUFFER_SETS):
        x, y, g = workload_values(args.config, lx, ly, lo, bsz, dtype, seed=s + 10 * rank, device=dev)
        sets.append((x, y, g))

    cache = matmul_build_layout_cache({}, lxd, lyd, lod)
    plans = cache[_PLANS]
    _backward_plans(plans, cache["packed_indices_x"], cache["packed_indices_y"], sets[0][0].size(0),
                    sets[0][1].size(0))

    def kernel_step(i):
        x, y, g = sets[i % N_BUFFER_SETS]
        out = plans.forward.run(x, y, bsz)
        gx = plans.grad_x.run(g, y, bsz)
        gy = plans.grad_y.run(x, g, bsz)
        return out, gx, gy

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def forward_step(i):
        x, y, _ = sets[i % N_BUFFER_SETS]
        return plans.forward.run(x, y, bsz)

    def capture(step):
        """One CUDA graph of N_BUFFER_SETS consecutive steps (one per buffer set): the layouts are
        static, so the launches of a step never change and the host leaves the timed loop."""
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side, capture_error_mode="thread_local"):
                results = [step(i) for i in range(N_BUFFER_SETS)]
        torch.cuda.current_stream(dev).wait_stream(side)
        return graph, results

    def run_steps(graph, step, n):
        """Exactly n steps: whole graph replays, the remainder launched one by one."""
        for _ in range(n // N_BUFFER_SETS if graph is not None else 0):
            graph.replay()
        for i in range(n % N_BUFFER_SETS if graph is not None else n):
            step(i)

    for i in range(args.warmup):
        kernel_step(i)
    check_device_status(dev)
    step_graph = fwd_graph = None
    if not args.no_graph:
        step_graph, _step_results = capture(kernel_step)
        fwd_graph, _fwd_results = capture(forward_step)
        run_steps(step_graph, kernel_step, N_BUFFER_SETS)
        run_steps(fwd_graph, forward_step, N_BUFFER_SETS)
        check_device_status(dev)

    # ---- device-resident throughput -----------------------------------------------------
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(physical_gpu_index(local)) as clocks:
        barrier()
        e0.record()
        run_steps(step_graph, kernel_step, args.steps)
        e1.record()
        barrier()
    ms = e0.elapsed_time(e1)
    check_device_status(dev)

    # ---- per-kernel time of the forward launch (roofline) ---------------------------------
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    f0.record()
    run_steps(fwd_graph, forward_step, args.steps)
    f1.record()
    torch.cuda.synchronize()
    fwd_ms = f0.elapsed_time(f1) / args.steps

    # ---- the public op on device-resident tensors (what the reference's own timing measures) ----
    api_cache = {}

    def api_step(i):
        x, y, g = sets[i % N_BUFFER_SETS]
        x = x.detach().requires_grad_(True)
        y = y.detach().requires_grad_(True)
        bs.ops.matmul(x, lxd, y, lyd, lod, bsz, api_cache).backward(g)

    api_steps = 0 if args.kernel_only else args.steps
    for i in range(3 if api_steps else 0):
        api_step(i)
    a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a0.record()
    for i in range(api_steps):
        api_step(i)
    a1.record()
    torch.cuda.synchronize()
    api_ms = a0.elapsed_time(a1) / max(api_steps, 1)

    # ---- end to end through the public op, host buffers in and out -------------------------
    # Every step copies its three pinned host inputs to the device, runs ops.matmul + backward and
    # copies all three results back to pinned host memory.  The copies run on their own streams,
    # two buffer slots deep, so the upload of step i+1 and the download of step i-1 overlap step i
    # (the PCIe link is full duplex); nothing is skipped.
    host_sets = [tuple(t.cpu().pin_memory() for t in s) for s in sets[:2]]
    layout_cache = {}
    h2d = sum(t.numel() * t.element_size() for t in host_sets[0])
    dev_in = [tuple(torch.empty_like(t, device=dev) for t in host_sets[0]) for _ in range(2)]
    host_out = [None, None]
    keep = [None, None]
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_done = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]
    main = torch.cuda.current_stream(dev)
    d2h = 0
    issued = 0

    def e2e_step(i):
        nonlocal d2h, issued
        slot = i % 2
        with torch.cuda.stream(s_in):
            if issued >= 2:
                s_in.wait_event(ev_done[slot])       # step i-2 has finished reading this slot
            for dst, src in zip(dev_in[slot], host_sets[slot]):
                dst.copy_(src, non_blocking=True)
            ev_in[slot].record(s_in)
        main.wait_event(ev_in[slot])
        x = dev_in[slot][0].detach().requires_grad_(True)
        y = dev_in[slot][1].detach().requires_grad_(True)
        out = bs.ops.matmul(x, lxd, y, lyd, lod, bsz, layout_cache)
        out.backward(dev_in[slot][2])
        res = (out.detach(), x.grad, y.grad)
        ev_done[slot].record(main)
        if host_out[slot] is None:
            host_out[slot] = tuple(torch.empty(t.shape, dtype=t.dtype, pin_memory=True) for t in res)
            d2h = sum(t.numel() * t.element_size() for t in res)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_done[slot])
            for dst, src in zip(host_out[slot], res):
                dst.copy_(src, non_blocking=True)
                src.record_stream(s_out)
            ev_out[slot].record(s_out)
        keep[slot] = res
        issued += 1
        if issued >= 2:
            ev_out[1 - slot].synchronize()           # bound the host's run-ahead to two steps

    def e2e_drain():
        main.wait_stream(s_out)
        main.wait_stream(s_in)

    e2e_steps = 0 if args.kernel_only else args.steps
    for i in range(min(args.warmup, 3) if e2e_steps else 0):
        e2e_step(i)
    e2e_drain()
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    g0.record()
    for i in range(e2e_steps):
        e2e_step(i)
    e2e_drain()
    g1.record()
    barrier()
    e2e_s = g0.elapsed_time(g1) * 1e-3
    check_device_status(dev)
    if e2e_steps and rank == 0:
        # the last step's results really are on the host
        last = (e2e_steps - 1) % 2
        ref_out = plans.forward.run(sets[last][0], sets[last][1], bsz)
        assert torch.equal(host_out[last][0], ref_out.cpu()), "end-to-end result differs from the device-resident run"

    # ---- reduce over ranks -------------------------------------------------------------------
    stats = torch.tensor([ms, e2e_s * 1e3, fwd_ms], dtype=torch.float64, device=dev)
    total_flops = torch.tensor([flops_step], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        dist.all_reduce(total_flops, op=dist.ReduceOp.SUM)
    ms, e2e_ms, fwd_ms = stats.tolist()
    flops_all = total_flops.item()

    if rank == 0:
        peaks = measured_peaks()
        value = flops_all * args.steps / (ms * 1e-3) / 1e12
        e2e_value = flops_all * e2e_steps / (e2e_ms * 1e-3) / 1e12 if e2e_steps else None
        fwd_bytes = wm["bytes"]["fwd"]
        achieved = fwd_bytes / (fwd_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": str(dtype).replace("torch.", ""), "data": "synthetic (seeded)",
            "config": {
                "workload": args.config, "block_size": bsz, "batch_per_gpu": lx.size(0),
                "layout_x": list(lx.shape), "layout_y": list(ly.shape), "pairs": wm["pairs"],
                "l2": f"rotating {N_BUFFER_SETS} input/output buffer sets, larger than the 126 MB L2",
                "parallelism": f"batch-sharded x{world}, no collective",
                "launch": ("one launch per product" if args.no_graph else
                           f"CUDA graph of {N_BUFFER_SETS} steps ({3 * N_BUFFER_SETS} kernel nodes) replayed"),
            },
            "pct_of_tensor_peak": 100.0 * value / (peaks["bf16_tflops"] * world),
            "roofline": {
                "bound": "hbm", "kernel": "matmul_umma_kernel (forward launch)", "achieved": achieved,
                "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                "peak_source": peaks["source"], "algorithmic_bytes": fwd_bytes, "ms_per_launch": fwd_ms,
                "tensor_tflops": wm["flops"]["fwd"] / (fwd_ms * 1e-3) / 1e12,
                "traffic": FWD_KERNEL_DRAM_TRAFFIC_BYTES.get(args.config),
            },
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms / max(e2e_steps, 1)},
            "api": {"ms_per_step": api_ms if api_steps else None,
                    "what": "ops.matmul + backward on device tensors, warm layout cache, validation on"},
            "gpu_launches": 3 * args.steps,
            "clocks": clocks.summary(),
        }
        if world == 1 and not args.no_cpu_baseline and not args.kernel_only:
            sample = min(lx.size(0), args.cpu_batch)
            dt, cflops = cpu_step_time(args.config, sample, 2, 1)
            line["cpu_baseline"] = {"value": cflops / dt / 1e12, "unit": "TFLOP/s",
                                    "cores": torch.get_num_threads(), "kind": "port",
                                    "sample": f"{sample} of {lx.size(0)} batches, 2 steps of fwd+bwd, dense masked matmul"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--config", default="config2")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "triton"])
    ap.add_argument("--cpu-batch", type=int, default=16, help="batches of the workload the CPU arm times")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true",
                    help="launch the device-resident legs kernel by kernel instead of replaying a CUDA graph")
    ap.add_argument("--kernel-only", action="store_true",
                    help="skip the end-to-end and CPU legs (for short profiler runs)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.impl == "triton":
        run_triton_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
