"""Benchmark of the block-sparse matmul path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config config5] [--impl ours|reference|triton]
    python bench.py --probe softmax|conversion|matmul|attention|regular_attention|nocache [--small]       (side probes, see bench_probes.py)

Default workload = the multi-GPU sweep: bf16, block 128, X (256, 4096, 4096) with a Bernoulli(0.10)
layout from seed 3, Y (256, 4096, 1024) dense, exact inferred output layout, values N(0, 0.02).  ONE
seeded problem is batch-sharded evenly over the N ranks (strong scaling): every rank owns a contiguous
batch range, generates exactly the values of its batches (each batch has its own seed, so the data do
not depend on N), builds its own LUTs and plans and runs alone; there is no collective on the data
path.  One step = one forward product O = X*Y of the rank's shard (one launch of the tcgen05 kernel on
a pre-built plan; LUTs and plans are built before the timed region, as the reference's warm
``layout_cache`` would be).  Other workloads (``--config config1..config4``) time forward + backward
(three launches per step).

Prints ONE JSON line.  ``value`` is effective TFLOP/s (FLOPs of non-zero block pairs only) with the
inputs resident in HBM, through the public op ``blksprs_b200.ops.matmul`` (warm layout cache, validation
on); ``kernel_only`` is the same step launched from the pre-built plans and replayed from a CUDA graph
(with ``--kernel-only`` that form is timed as ``value`` and the other legs are skipped); ``e2e`` goes
through ``ops.matmul`` with pinned host buffers copied in and the results copied out every step.  R back-to-back regions of
exactly ``--steps`` steps are timed with CUDA events; the median region (maximum over ranks per
region) gives ``ms_per_step``.  ``parity`` holds a check of sampled output blocks against an fp32
product computed with torch from the same compressed operands, and a per-batch checksum of the whole
result gathered over NCCL (the only use of NCCL): rank 0 recomputes one batch of every other rank's
shard by itself and compares checksums bit for bit.  At N = 1 the line also carries ``also`` (the
other workloads at full size, each with its own sampled check), ``triton_reference`` (the reference's
own Triton op on the same GPU and tensors), ``cold_call`` (one forward call that builds all LUTs and
plans first; the reference's is in ``triton_reference``) and ``cpu_baseline`` (the CPU oracle on a
bounded sample).
``--impl reference`` times the CPU oracle (dense masked matmul, all host threads) instead.
"""
from __future__ import annotations

import argparse
import hashlib
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

N_BUFFER_SETS = 4
FORWARD_ONLY = ("config5",)  # workloads whose step is the forward product alone


def metric_name(config: str) -> str:
    what = "forward" if config in FORWARD_ONLY else "forward+backward"
    return f"block-sparse matmul effective TFLOP/s (nnz-block FLOPs), {what}"


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
        lut = torch.nonzero(lx).to(device)
        row_id = lut[:, 0] * lx.size(1) + lut[:, 1]
        n_rows = lx.size(0) * lx.size(1)
        x = torch.empty((nx, bs, bs), dtype=dtype, device=device)
        sums = torch.zeros((n_rows, bs), device=device)
        chunk = 1 << 15  # blocks per pass: bounds the fp32 temporaries at full size
        state = g.get_state()

        def exp_logits(first):  # exp(logit - 5) of blocks [first, first + chunk); logits ~ N(0, 1)
            return torch.exp(torch.randn((min(chunk, nx - first), bs, bs), generator=g, device=device,
                                         dtype=torch.float32) - 5.0)

        for first in range(0, nx, chunk):
            sums.index_add_(0, row_id[first:first + chunk], exp_logits(first).sum(-1))
        g.set_state(state)  # the second pass draws the same logits again
        for first in range(0, nx, chunk):
            x[first:first + chunk] = (exp_logits(first) / sums[row_id[first:first + chunk]][:, :, None]).to(dtype)
        y = randn(ny)
    elif name == "config5":
        x, y = randn(nx, 0.02), randn(ny, 0.02)
    else:
        x, y = randn(nx), randn(ny)
    return x, y, randn(no)


def batch_block_offsets(layout: torch.Tensor) -> torch.Tensor:
    """int64 (B + 1): index of the first compressed block of every batch."""
    per = layout.reshape(layout.size(0), -1).sum(1).to(torch.int64)
    out = torch.zeros(layout.size(0) + 1, dtype=torch.int64)
    out[1:] = torch.cumsum(per, 0)
    return out


def shard_values(name: str, lx, ly, lo, bs, dtype, seed: int, device, b0: int, b1: int):
    """Compressed x, y, grad-output of batches [b0, b1) of a workload whose values are seeded per
    batch: what a rank generates does not depend on how many ranks share the problem."""
    scale = {"config5": 0.02, "config2": 1 / math.sqrt(lx.size(2) * bs)}.get(name, 1.0)
    g = torch.Generator(device=device)
    outs = []
    for which, layout in enumerate((lx, ly, lo)):
        off = batch_block_offsets(layout)
        t = torch.empty((int(off[b1] - off[b0]), bs, bs), dtype=dtype, device=device)
        for b in range(b0, b1):
            n = int(off[b + 1] - off[b])
            if n == 0:
                continue
            g.manual_seed(((1000 + seed) * 4 + which) * 1_000_003 + b)
            s = scale if which < 2 else 1.0
            t[int(off[b] - off[b0]):int(off[b + 1] - off[b0])] = \
                (torch.randn((n, bs, bs), generator=g, device=device, dtype=torch.float32) * s).to(dtype)
        outs.append(t)
    return tuple(outs)


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


def step_flops(name: str, wm) -> float:
    return wm["flops"]["fwd"] if name in FORWARD_ONLY else sum(wm["flops"].values())


def buffer_sets(name: str) -> int:
    """Input/output buffer sets the GPU arm rotates.  One set of config5 (inputs + output of a rank's
    shard) is several times the 126 MB L2 at every N <= 8, two are rotated anyway; the small workloads
    rotate four; config3 / config4 (gigabytes per set) use one."""
    return 2 if name == "config5" else (N_BUFFER_SETS if name in ("config1", "config2") else 1)


def config_record(name: str, lx, ly, bs, wm, world: int, no_graph: bool = False, kernel_only: bool = False) -> dict:
    """The ``config`` object of a JSON line: the workload and the measurement protocol of the GPU arm;
    the same keys and values in every arm."""
    n_sets = buffer_sets(name)
    per_step = 1 if name in FORWARD_ONLY else 3
    return {
        "workload": name, "block_size": bs, "batch": lx.size(0), "batch_per_gpu": lx.size(0) // world,
        "layout_x": list(lx.shape), "layout_y": list(ly.shape), "pairs": wm["pairs"],
        "step": "forward" if name in FORWARD_ONLY else "forward + dX + dY",
        "parallelism": f"one problem batch-sharded evenly x{world}, per-shard LUTs, no collective",
        "l2": (f"{n_sets} input/output buffer sets rotated; the forward product of one set moves "
               f"{wm['bytes']['fwd'] / world / 1e6:.0f} MB per GPU against the 126 MB L2"),
        "launch": ((("value = kernel only: one launch per product from the pre-built plans" if no_graph else
                     f"value = kernel only: CUDA graph of {n_sets} steps ({per_step * n_sets} kernel nodes) replayed")
                    if kernel_only else
                    ("value = through the public op (ops.matmul on device tensors, warm layout cache, validation "
                     f"on); kernel_only = CUDA graph of {n_sets} steps ({per_step * n_sets} kernel nodes) replayed"))),
    }


# ---------------------------------------------------------------------------------------------
# checks that need no CPU oracle: sampled blocks against an fp32 torch product, checksums
# ---------------------------------------------------------------------------------------------

def sampled_block_check(a, la, b, lb, lo, out, bs, op: str, n_samples: int = 64, seed: int = 0):
    """Relative error (max|err| / max|ref| over the sampled blocks) of ``n_samples`` blocks of ``out``
    against an fp32 product of the same compressed operand blocks, computed with torch on the GPU.

    op "nn": out(b,i,j) = sum_k a(b,i,k) b(b,k,j);  "nt": out(b,i,k) = sum_j a(b,i,j) b(b,k,j)^T;
    "tn": out(b,k,j) = sum_i a(b,i,k)^T b(b,i,j).  Layouts are CPU bool tensors; the sampled blocks
    are spread over the whole output (first, last and random ones).
    """
    n_out = out.size(0)
    if n_out == 0:
        return {"sampled_blocks": 0, "max_rel_err": 0.0}
    lut = torch.nonzero(lo)
    pa = (torch.cumsum(la.reshape(-1).long(), 0) - 1).reshape(la.shape)
    pb = (torch.cumsum(lb.reshape(-1).long(), 0) - 1).reshape(lb.shape)
    g = _gen(4242 + seed)
    picks = torch.unique(torch.cat([torch.tensor([0, n_out - 1]),
                                    torch.randint(0, n_out, (max(n_samples - 2, 0),), generator=g)]))
    worst, ref_max = 0.0, 0.0
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        for p in picks.tolist():
            bb, r, c = lut[p].tolist()
            if op == "nn":
                ks = torch.nonzero(la[bb, r, :] & lb[bb, :, c]).flatten()
                ia, ib = pa[bb, r, ks], pb[bb, ks, c]
            elif op == "nt":
                ks = torch.nonzero(la[bb, r, :] & lb[bb, c, :]).flatten()
                ia, ib = pa[bb, r, ks], pb[bb, c, ks]
            else:
                ks = torch.nonzero(la[bb, :, r] & lb[bb, :, c]).flatten()
                ia, ib = pa[bb, ks, r], pb[bb, ks, c]
            if ks.numel():
                A = a[ia.to(a.device)].float()
                Bm = b[ib.to(b.device)].float()
                if op == "nt":
                    Bm = Bm.transpose(-1, -2)
                if op == "tn":
                    A = A.transpose(-1, -2)
                ref = torch.matmul(A, Bm).sum(0)
            else:
                ref = torch.zeros((bs, bs), device=out.device)
            err = float((out[p].float() - ref).abs().max())
            # a NaN compares false with everything and max() would silently drop it: anything that is not a
            # finite number counts as an error beyond every tolerance (1e30, which JSON can carry)
            worst = max(worst, err if math.isfinite(err) else 1e30)
            ref_max = max(ref_max, float(ref.abs().max()))
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    return {"sampled_blocks": int(picks.numel()), "max_rel_err": min(worst / max(ref_max, 1e-30), 1e30)}


def batch_checksums(t: torch.Tensor, layout: torch.Tensor) -> torch.Tensor:
    """int64 per batch: the sum of the raw bit patterns of the batch's blocks (exact, order-free)."""
    off = batch_block_offsets(layout).tolist()
    raw = t.view(torch.int16 if t.element_size() == 2 else torch.int32)
    sums = [raw[off[b]:off[b + 1]].sum(dtype=torch.int64) for b in range(layout.size(0))]
    return torch.stack(sums) if sums else torch.zeros(0, dtype=torch.int64, device=t.device)


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
            self._stop.wait(0.004)

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


def bind_to_gpu_numa_node(index: int) -> dict:
    """Best effort: restricts this process to the CPUs of the NUMA node the GPU hangs off, so that the
    pinned host buffers of the end-to-end leg (allocated afterwards, first touch) are local to it.
    Returns what was found and done; never raises."""
    info = {"bound": False}
    try:
        import pynvml
        pynvml.nvmlInit()
        bus = pynvml.nvmlDeviceGetPciInfo(pynvml.nvmlDeviceGetHandleByIndex(index)).busId
        bus = bus.decode() if isinstance(bus, bytes) else bus
        dom, rest = bus.split(":", 1)
        path = f"/sys/bus/pci/devices/{dom[-4:].lower()}:{rest.lower()}/numa_node"
        with open(path) as f:
            node = int(f.read().strip())
        nodes = [d for d in os.listdir("/sys/devices/system/node") if d.startswith("node") and d[4:].isdigit()]
        info.update({"gpu_numa_node": node, "host_numa_nodes": len(nodes)})
        if node >= 0 and len(nodes) > 1:
            with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
                cpus = set()
                for part in f.read().strip().split(","):
                    lo, _, hi = part.partition("-")
                    cpus.update(range(int(lo), int(hi or lo) + 1))
            allowed = cpus & os.sched_getaffinity(0)
            if allowed:
                os.sched_setaffinity(0, allowed)
                info["bound"] = True
                info["cpus"] = len(allowed)
    except Exception as exc:
        info["note"] = repr(exc)[:120]
    return info


def physical_gpu_index(local_index: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_index])
        except (ValueError, IndexError):
            pass
    return local_index


# ---------------------------------------------------------------------------------------------
# CPU arm (the oracle, timed): dense masked matmul
# ---------------------------------------------------------------------------------------------

def cpu_step_time(name: str, sample_batch: int, steps: int, warmup: int):
    """Seconds per step of the CPU oracle on ``sample_batch`` batches of the workload, and the
    effective FLOPs of that sample."""
    from oracle import oracle
    lx, ly, lo, bs, dtype = workload_layouts(name, batch=sample_batch)
    x, y, g = workload_values(name, lx, ly, lo, bs, dtype, seed=0)
    wm = work_model(lx, ly, lo, bs, x.element_size())
    flops = step_flops(name, wm)
    torch.set_num_threads(os.cpu_count() or 1)

    def step():
        out = oracle.matmul_forward(x, lx, y, ly, lo, bs)
        if name in FORWARD_ONLY:
            return out
        return out, oracle.matmul_backward(g, x, lx, y, ly, lo, bs)

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    return dt, flops


def run_reference_arm(args):
    """The CPU oracle on a bounded sample of the workload (blksprs has no CPU implementation of its
    own, so the oracle port stands in); rank 0 alone runs it."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    lx, ly, lo, bs, dtype = workload_layouts(args.config)
    wm = work_model(lx, ly, lo, bs, torch.empty((), dtype=dtype).element_size())
    full_batch = lx.size(0)
    sample = min(full_batch, args.cpu_batch)
    dt, flops = cpu_step_time(args.config, sample, max(args.steps, 1), max(min(args.warmup, 2), 1))
    value = flops / dt / 1e12
    cores = torch.get_num_threads()
    what = "forward" if args.config in FORWARD_ONLY else "forward + backward"
    line = {
        "impl": "reference", "metric": metric_name(args.config), "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt * 1e3 * full_batch / sample, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": str(dtype).replace("torch.", ""), "data": "synthetic (seeded)",
        "config": config_record(args.config, lx, ly, bs, wm, world),
        "note": "CPU dense masked-matmul oracle in fp32 (16-bit inputs upcast); blksprs has no CPU path",
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                         "sample": f"{sample} of {full_batch} batches per step, {what}, dense masked matmul"},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# the reference's Triton op on the same GPU
# ---------------------------------------------------------------------------------------------

def _import_reference():
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "blksprs")):
        raise RuntimeError("baseline/_ref holds no blksprs install")
    if ref_dir not in sys.path:
        sys.path.insert(0, ref_dir)
    os.environ.setdefault("BLKSPRS_AUTOTUNE", "DEFAULT")
    import blksprs as ref
    return ref


def cold_call_ms(call, repeats: int = 5) -> float:
    """Median wall-clock time (ms, device drained on both sides) of a forward call that has to build all
    of its metadata (no layout cache) and run the product."""
    times = []
    for _ in range(repeats + 1):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        call()
        torch.cuda.synchronize()
        times.append((time.perf_counter() - t0) * 1e3)
    return median(times[1:])


def our_cold_call_ms(p) -> float:
    """``cold_call_ms`` of the public op on buffer set 0 of problem ``p``, the library-owned layout caches
    switched off so that every call rebuilds LUTs and plans."""
    import blksprs_b200 as bs
    x, y, _ = p.sets[0]
    bs.utils.set_implicit_layout_caches(False)
    try:
        return cold_call_ms(lambda: bs.ops.matmul(x, p.lxd, y, p.lyd, p.lod, p.bs))
    finally:
        bs.utils.set_implicit_layout_caches(True)


def time_triton(ref, name: str, layouts_dev, sets, bsz, wm, steps: int, warmup: int) -> dict:
    """``bs.ops.matmul`` of the reference (forward, and forward + backward unless the workload is
    forward-only) with a warm ``layout_cache``, validation on and off; the autotuner runs in the warm-up."""
    lxd, lyd, lod = layouts_dev
    results = {}
    modes = [("fwd", wm["flops"]["fwd"])]
    if name not in FORWARD_ONLY:
        modes.append(("fwd_bwd", sum(wm["flops"].values())))
    for label, validate in (("validation_on", True), ("validation_off", False)):
        (ref.utils.enable_validation if validate else ref.utils.disable_validation)()
        cache = {}

        def step(i, fwd_only):
            x, y, g = sets[i % len(sets)]
            x = x.detach().requires_grad_(not fwd_only)
            y = y.detach().requires_grad_(not fwd_only)
            out = ref.ops.matmul(x, lxd, y, lyd, lod, bsz, cache)
            if not fwd_only:
                out.backward(g)

        for mode, flops in modes:
            for i in range(max(warmup, 3)):
                step(i, mode == "fwd")
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            for i in range(steps):
                step(i, mode == "fwd")
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / steps
            results[f"{label}/{mode}"] = {"ms_per_step": ms, "tflops": flops / (ms * 1e-3) / 1e12}
        # a call without layout_cache: the reference rebuilds its LUTs (the autotuner has run above)
        x0, y0, _ = sets[0]
        results[f"{label}/cold_fwd_ms"] = cold_call_ms(lambda: ref.ops.matmul(x0, lxd, y0, lyd, lod, bsz))
    ref.utils.enable_validation()
    return results


def run_triton_arm(args):
    """Stand-alone run of the reference's Triton op on one workload."""
    line = {"impl": "triton-reference", "metric": metric_name(args.config), "unit": "TFLOP/s"}
    try:
        ref = _import_reference()
    except Exception as exc:
        line["unavailable"] = f"reference not importable from baseline/_ref: {exc!r}"[:200]
        print(json.dumps(line), flush=True)
        return
    dev = torch.device("cuda", 0)
    lx, ly, lo, bsz, dtype = workload_layouts(args.config)
    wm = work_model(lx, ly, lo, bsz, torch.empty((), dtype=dtype).element_size())
    n_sets = buffer_sets(args.config)
    sets = [workload_values(args.config, lx, ly, lo, bsz, dtype, seed=s, device=dev) for s in range(n_sets)]
    results = time_triton(ref, args.config, (lx.to(dev), ly.to(dev), lo.to(dev)), sets, bsz, wm, args.steps,
                          args.warmup)
    key = "validation_off/fwd" if args.config in FORWARD_ONLY else "validation_off/fwd_bwd"
    line.update({"value": results[key]["tflops"], "results": results, "config": {"workload": args.config},
                 "steps": args.steps, "warmup": args.warmup, "triton": __import__("triton").__version__})
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------

def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def profiled_traffic(name: str, units: float):
    """DRAM bytes (read + write) of one forward launch from the kept profiler captures
    (profiles/dram_traffic.json: bytes per unit of a small capture), scaled to ``units`` of this
    launch; None for workloads without a capture."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.json")
    try:
        with open(path) as f:
            entry = json.load(f)[name]
        return entry["dram_bytes_per_unit"] * units
    except Exception:
        return None


class Problem:
    """A workload (or a batch shard of one) on a device: layouts, plans, buffer sets, launch closures."""

    def __init__(self, name, dev, b0=None, b1=None, n_sets=1, per_batch_seed=False, batch=None):
        from blksprs_b200.ops.matmul import matmul_build_layout_cache, _backward_plans, _PLANS
        self.name, self.dev = name, dev
        lx, ly, lo, bsz, dtype = workload_layouts(name, batch=batch)
        self.full = (lx, ly, lo)
        self.b0, self.b1 = (0, lx.size(0)) if b0 is None else (b0, b1)
        self.lx, self.ly, self.lo = (t[self.b0:self.b1].contiguous() for t in (lx, ly, lo))
        self.bs, self.dtype = bsz, dtype
        self.esize = torch.empty((), dtype=dtype).element_size()
        self.wm = work_model(self.lx, self.ly, self.lo, bsz, self.esize)
        self.lxd, self.lyd, self.lod = self.lx.to(dev), self.ly.to(dev), self.lo.to(dev)
        self.sets = []
        for s in range(n_sets):
            if per_batch_seed:
                self.sets.append(shard_values(name, lx, ly, lo, bsz, dtype, s, dev, self.b0, self.b1))
            else:
                self.sets.append(workload_values(name, self.lx, self.ly, self.lo, bsz, dtype, seed=s, device=dev))
        self.cache = matmul_build_layout_cache({}, self.lxd, self.lyd, self.lod)
        self.plans = self.cache[_PLANS]
        self.forward_only = name in FORWARD_ONLY
        if not self.forward_only:
            _backward_plans(self.plans, self.cache["packed_indices_x"], self.cache["packed_indices_y"],
                            self.sets[0][0].size(0), self.sets[0][1].size(0))
        self.flops = step_flops(name, self.wm)
        self.launches_per_step = 1 if self.forward_only else 3

    def forward(self, i):
        x, y, _ = self.sets[i % len(self.sets)]
        return self.plans.forward.run(x, y, self.bs)

    def step(self, i):
        x, y, g = self.sets[i % len(self.sets)]
        out = self.plans.forward.run(x, y, self.bs)
        if self.forward_only:
            return (out,)
        return out, self.plans.grad_x.run(g, y, self.bs), self.plans.grad_y.run(x, g, self.bs)

    def api_step(self, i, cache):
        import blksprs_b200 as bs
        x, y, g = self.sets[i % len(self.sets)]
        if self.forward_only:
            return (bs.ops.matmul(x, self.lxd, y, self.lyd, self.lod, self.bs, cache),)
        x = x.detach().requires_grad_(True)
        y = y.detach().requires_grad_(True)
        out = bs.ops.matmul(x, self.lxd, y, self.lyd, self.lod, self.bs, cache)
        out.backward(g)
        return out.detach(), x.grad, y.grad

    def parity(self, results, i=0, n_samples=64):
        """Sampled-block check of a step's results (computed from buffer set ``i``)."""
        x, y, g = self.sets[i % len(self.sets)]
        rec = sampled_block_check(x, self.lx, y, self.ly, self.lo, results[0], self.bs, "nn", n_samples)
        worst = rec["max_rel_err"]
        n = rec["sampled_blocks"]
        if len(results) == 3:
            rx = sampled_block_check(g, self.lo, y, self.ly, self.lx, results[1], self.bs, "nt", n_samples // 2)
            ry = sampled_block_check(x, self.lx, g, self.lo, self.ly, results[2], self.bs, "tn", n_samples // 2)
            worst = max(worst, rx["max_rel_err"], ry["max_rel_err"])
            n += rx["sampled_blocks"] + ry["sampled_blocks"]
        tol = 1e-3 if self.dtype == torch.float32 else 1e-2
        return {"sampled_blocks": n, "max_rel_err": worst, "tolerance": tol, "ok": bool(worst <= tol)}


def capture_graph(dev, step, n_sets):
    """One CUDA graph of ``n_sets`` consecutive steps (one per buffer set): the layouts are static, so
    the launches of a step never change and the host leaves the timed loop."""
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side, capture_error_mode="thread_local"):
            results = [step(i) for i in range(n_sets)]
    torch.cuda.current_stream(dev).wait_stream(side)
    return graph, results


def run_steps(graph, step, n, n_sets):
    """Exactly n steps: whole graph replays, the remainder launched one by one."""
    for _ in range(n // n_sets if graph is not None else 0):
        graph.replay()
    for i in range(n % n_sets if graph is not None else n):
        step(i)


def time_regions(graph, step, steps, n_sets, regions):
    """CUDA-event times (ms) of ``regions`` back-to-back regions of exactly ``steps`` steps each."""
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(regions + 1)]
    evs[0].record()
    for r in range(regions):
        run_steps(graph, step, steps, n_sets)
        evs[r + 1].record()
    torch.cuda.synchronize()
    return [evs[r].elapsed_time(evs[r + 1]) for r in range(regions)]


def median(v):
    s = sorted(v)
    return s[len(s) // 2]


def n_regions(est_ms_per_step: float, steps: int, want: int = 30, budget_s: float = 6.0) -> int:
    """R >= ``want`` regions and at least 1.5 s of timed work in all (a steady power and clock state, enough
    clock samples), within a budget."""
    region_s = max(est_ms_per_step * steps * 1e-3, 1e-6)
    r = max(want, int(1.5 / region_s) + 1)
    return max(5, min(r, int(budget_s / region_s), 4000))


def sub_record(name, dev, args, peaks):
    """Kernel-only record of another workload at full size with its own sampled check (N = 1 only)."""
    n_sets = buffer_sets(name)
    prob = Problem(name, dev, n_sets=n_sets)
    from blksprs_b200.plan import check_device_status
    for i in range(3):
        res = prob.step(i)
    check_device_status(dev)
    parity = prob.parity(prob.step(0), 0, 48)
    del res
    graph, _keep = capture_graph(dev, prob.step, n_sets)
    fgraph, _keepf = capture_graph(dev, prob.forward, n_sets)
    steps = max(n_sets, 8 if name in ("config3", "config4") else 20)
    steps -= steps % n_sets
    run_steps(graph, prob.step, n_sets, n_sets)
    run_steps(fgraph, prob.forward, n_sets, n_sets)
    torch.cuda.synchronize()
    t = median(time_regions(graph, prob.step, steps, n_sets, 7)) / steps
    tf = median(time_regions(fgraph, prob.forward, steps, n_sets, 7)) / steps
    check_device_status(dev)
    api_cache = {}
    for i in range(3):
        prob.api_step(i, api_cache)
    ta = median(time_regions(None, lambda i: prob.api_step(i, api_cache), steps, n_sets, 5)) / steps
    rec = {
        "dtype": str(prob.dtype).replace("torch.", ""), "block_size": prob.bs, "batch": prob.lx.size(0),
        "pairs": prob.wm["pairs"], "step": "forward" if prob.forward_only else "forward + dX + dY",
        "ms_per_step": t, "tflops": prob.flops / (t * 1e-3) / 1e12,
        "fwd_ms": tf, "fwd_tflops": prob.wm["flops"]["fwd"] / (tf * 1e-3) / 1e12,
        "fwd_hbm_gbs": prob.wm["bytes"]["fwd"] / (tf * 1e-3) / 1e9,
        "fwd_hbm_frac": prob.wm["bytes"]["fwd"] / (tf * 1e-3) / 1e9 / peaks["hbm_gbs"],
        "api_ms_per_step": ta, "launch": "CUDA graph replay (kernel only); api = ops.matmul (+ backward)",
        "parity": parity,
    }
    return rec, prob


def attention_chain_record(dev, peaks, batch=None):
    """Attention by parts at the size of the config3 -> config4 pair: P = softmax(scale * Q K^T) on the
    banded causal layout in bf16, then O = P V.  Times the part between the operands and P once as the
    chain of separate ops (matmul -> scale and cast to fp32 -> softmax -> cast to bf16) and once as the
    fused op (softmax in the matmul's epilogue plus one normalising pass), and the P V product."""
    import blksprs_b200 as bs
    lq, lkt, lo, bsz, dtype = workload_layouts("config3", batch=batch)
    q, kt, _ = workload_values("config3", lq, lkt, lo, bsz, dtype, seed=0, device=dev)
    B = lq.size(0)
    lv = torch.ones((B, 64, 2), dtype=torch.bool)
    g = torch.Generator(device=dev)
    g.manual_seed(5)
    v = torch.randn((int(lv.sum()), bsz, bsz), generator=g, device=dev).to(torch.bfloat16)
    lqd, lktd, lod, lvd = lq.to(dev), lkt.to(dev), lo.to(dev), lv.to(dev)
    scale = 128 ** -0.5
    caches = [{}, {}, {}]

    def chain():
        scores = bs.ops.matmul(q, lqd, kt, lktd, lod, bsz, caches[0])
        return bs.ops.softmax(scores.float() * scale, lod, bsz, layout_cache=caches[1]).to(torch.bfloat16)

    def fused():
        return bs.ops.matmul_softmax(q, lqd, kt, lktd, lod, bsz, scale=scale, out_dtype=torch.bfloat16,
                                     layout_cache=caches[0])

    def pv(p):
        return bs.ops.matmul(p, lod, v, lvd, lvd, bsz, caches[2])

    def timed(fn, n=5):
        for _ in range(2):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    p_chain, p_fused = chain(), fused()   # also builds the caches and plans
    pv(p_fused)
    torch.cuda.profiler.start()   # one warm pass of each form, for a profiler attached with "--profile-from-start off"
    chain()
    fused()
    pv(p_fused)
    torch.cuda.profiler.stop()
    diff = float((p_chain.float() - p_fused.float()).abs().max()) / max(float(p_chain.float().abs().max()), 1e-30)
    t_chain, t_fused = timed(chain), timed(fused)
    t_pv = timed(lambda: pv(p_fused))
    n_el = int(lo.sum()) * bsz * bsz
    return {
        "batch": B, "score_elements": n_el, "scores_to_probabilities_ms": {"separate_ops": t_chain, "fused": t_fused},
        "pv_ms": t_pv, "chain_ms": {"separate_ops": t_chain + t_pv, "fused": t_fused + t_pv},
        "bytes_moved_model": {"separate_ops": n_el * (2 + 2 + 4 + 4 + 4 + 4 + 2), "fused": n_el * (2 + 2 + 2),
                              "what": "score-sized tensors written and read between the matmul's accumulators and P"},
        "max_rel_diff_fused_vs_separate": diff,
    }


def run_gpu_arm(args):
    import torch.distributed as dist
    import blksprs_b200 as bs
    from blksprs_b200.plan import check_device_status
    from blksprs_b200.sharding import shard_bounds

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    numa = bind_to_gpu_numa_node(physical_gpu_index(local))
    if world > 1:
        # a short collective timeout: a rank that fails must end the job quickly, never leave the others waiting
        import datetime
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
    name = args.config
    peaks = measured_peaks()

    # ---- the rank's shard of ONE seeded problem --------------------------------------------------
    lx_full, ly_full, lo_full, bsz, dtype = workload_layouts(name, batch=args.batch)
    B = lx_full.size(0)
    b0, b1 = shard_bounds(B, world, rank)
    sharded = name in ("config5", "config2") and (world > 1 or name == "config5")
    if world > 1 and not sharded:
        raise SystemExit(f"--gpus > 1 is defined for the batch-sharded workloads (config5, config2), not {name}")
    n_sets = buffer_sets(name)
    prob = Problem(name, dev, b0 if sharded else None, b1 if sharded else None, n_sets=n_sets,
                   per_batch_seed=sharded, batch=args.batch)
    wm_full = work_model(lx_full, ly_full, lo_full, bsz, prob.esize)
    flops_all = step_flops(name, wm_full)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        results = prob.step(i)
    check_device_status(dev)
    graph = None
    if not args.no_graph:
        graph, _graph_results = capture_graph(dev, prob.step, n_sets)
        run_steps(graph, prob.step, n_sets, n_sets)
        check_device_status(dev)

    # ---- device-resident throughput: R regions of exactly --steps steps -------------------------
    # The main leg goes through the public op (what a caller runs, and what the reference's own timing of
    # its op measures); with --kernel-only it launches the pre-built plans instead (CUDA graph replay).
    api_cache = {}
    if args.kernel_only:
        main_graph, main_step = graph, prob.step
    else:
        main_graph, main_step = None, (lambda i: prob.api_step(i, api_cache))
        for i in range(max(3, args.warmup)):
            main_step(i)
    torch.cuda.synchronize()
    probe = time_regions(main_graph, main_step, args.steps, n_sets, 1)[0] / args.steps
    R = args.regions or n_regions(probe, args.steps)
    if world > 1:
        # every rank must time the same number of regions (the per-region times are reduced over ranks)
        r_all = torch.tensor([R], dtype=torch.int64, device=dev)
        dist.all_reduce(r_all, op=dist.ReduceOp.MAX)
        R = int(r_all.item())
    with ClockSampler(physical_gpu_index(local)) as clocks:
        barrier()
        torch.cuda.profiler.start()   # a profiler attached with "--profile-from-start off" sees the timed region only
        region_ms = time_regions(main_graph, main_step, args.steps, n_sets, R)
        torch.cuda.profiler.stop()
        barrier()
    check_device_status(dev)
    region_t = torch.tensor(region_ms, dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(region_t, op=dist.ReduceOp.MAX)   # a region ends when its slowest rank ends
    region_ms = region_t.tolist()
    ms_region = median(region_ms)

    # ---- the same steps launched from the pre-built plans (CUDA graph replay), kernel only ----------
    kernel_ms = None
    if not args.kernel_only and graph is not None:
        k_t = torch.tensor(time_regions(graph, prob.step, args.steps, n_sets, max(5, R // 4)), dtype=torch.float64,
                           device=dev)
        if world > 1:
            dist.all_reduce(k_t, op=dist.ReduceOp.MAX)
        kernel_ms = median(k_t.tolist()) / args.steps
        check_device_status(dev)

    # ---- parity: sampled blocks on every rank, per-batch checksums gathered over NCCL -------------
    results = prob.step(0)
    torch.cuda.synchronize()
    parity = prob.parity(results, 0, 64)
    sums = batch_checksums(results[0], prob.lo)
    counts = [shard_bounds(B, world, r)[1] - shard_bounds(B, world, r)[0] for r in range(world)]
    if world > 1:
        cap = max(counts)
        padded = torch.zeros(cap, dtype=torch.int64, device=dev)
        padded[:sums.numel()] = sums
        gathered = [torch.zeros_like(padded) for _ in range(world)]
        dist.all_gather(gathered, padded)
        all_sums = torch.cat([g[:c] for g, c in zip(gathered, counts)])
        stats = torch.tensor([parity["max_rel_err"], float(parity["sampled_blocks"])], dtype=torch.float64,
                             device=dev)
        worst = stats.clone()
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        dist.all_reduce(stats, op=dist.ReduceOp.SUM)
        parity["max_rel_err"] = float(worst[0])
        parity["sampled_blocks"] = int(stats[1])
        parity["ok"] = bool(parity["max_rel_err"] <= parity["tolerance"])
    else:
        all_sums = sums
    if sharded and rank == 0:
        # rank 0 recomputes, as a one-batch problem of its own, the first batch of every shard (its own
        # included) through the public op and compares with the owner's checksum, bit for bit
        equal = True
        for r in range(world):
            bb = shard_bounds(B, world, r)[0]
            x1, y1, _ = shard_values(name, lx_full, ly_full, lo_full, bsz, dtype, 0, dev, bb, bb + 1)
            o1 = bs.ops.matmul(x1, lx_full[bb:bb + 1].to(dev), y1, ly_full[bb:bb + 1].to(dev),
                               lo_full[bb:bb + 1].to(dev), bsz)
            equal &= bool(batch_checksums(o1, lo_full[bb:bb + 1])[0] == all_sums[bb])
        parity["checksums_equal_to_n1"] = equal
        parity["checksum_digest"] = hashlib.sha256(all_sums.cpu().numpy().tobytes()).hexdigest()[:16]
        parity["checksum_what"] = (f"{B} per-batch sums of the output's bit patterns; digest is the same at every N; "
                                   "rank 0 recomputed one batch per shard alone")
    del results

    # ---- end to end through the public op, host buffers in and out ------------------------------------
    e2e = None
    if not args.kernel_only:
        e2e = run_e2e(prob, dev, args, barrier, world, flops_all)

    line = None
    if rank == 0:
        ms_step = ms_region / args.steps
        value = flops_all / (ms_step * 1e-3) / 1e12
        fwd_bytes = wm_full["bytes"]["fwd"]
        line = {
            "metric": metric_name(name), "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong" if sharded else "weak", "vs_baseline": None,
            "dtype": str(dtype).replace("torch.", ""), "data": "synthetic (seeded per batch)" if sharded else
            "synthetic (seeded)",
            "config": config_record(name, lx_full, ly_full, bsz, wm_full, world, args.no_graph, args.kernel_only),
            "timing": {"regions": R, "steps_per_region": args.steps, "region_ms_median": ms_region,
                       "region_ms_min": min(region_ms), "region_ms_max": max(region_ms),
                       "what": "CUDA events around each region, maximum over ranks per region, median region"},
            "pct_of_tensor_peak": 100.0 * value / (peaks["bf16_tflops"] * world),
            "parity": parity,
            "e2e": e2e,
            "kernel_only": {"ms_per_step": kernel_ms,
                            "tflops": flops_all / (kernel_ms * 1e-3) / 1e12 if kernel_ms else None,
                            "what": "the same steps launched from the pre-built plans, CUDA graph replay"},
            "gpu_launches": prob.launches_per_step * args.steps * R,
            "host": {"numa": numa, "cpus": os.cpu_count()},
            "clocks": clocks.summary(),
        }
        if prob.forward_only:
            # the step is the forward launch: its duration is the step time of this rank's shard
            per_rank_bytes = fwd_bytes / world
            achieved = per_rank_bytes / (ms_step * 1e-3) / 1e9
            line["roofline"] = {
                "bound": "hbm", "kernel": "matmul_umma_kernel (forward launch, per GPU)", "achieved": achieved,
                "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                "peak_source": peaks["source"], "algorithmic_bytes": per_rank_bytes, "ms_per_launch": ms_step,
                "tensor_tflops": wm_full["flops"]["fwd"] / world / (ms_step * 1e-3) / 1e12,
                "traffic": profiled_traffic(name, wm_full["pairs"]["fwd"] / world),
            }
            # the fastest region (one of the first, before the power cap has settled the SM clock): what the
            # kernel reaches when it runs as a burst, as the copy that measured the peak did
            burst_ms = min(region_ms) / args.steps
            line["roofline"]["burst"] = {
                "ms_per_launch": burst_ms, "achieved": per_rank_bytes / (burst_ms * 1e-3) / 1e9,
                "frac": per_rank_bytes / (burst_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                "what": "fastest of the timed regions; frac / achieved above are the median region (sustained, "
                        "under the power cap the clocks record shows)"}
    if rank == 0 and not prob.forward_only:
        fgraph, _keepf = capture_graph(dev, prob.forward, n_sets)
        run_steps(fgraph, prob.forward, n_sets, n_sets)
        torch.cuda.synchronize()
        fwd_ms = median(time_regions(fgraph, prob.forward, args.steps, n_sets, max(5, R // 4))) / args.steps
        fb = prob.wm["bytes"]["fwd"]
        achieved = fb / (fwd_ms * 1e-3) / 1e9
        line["roofline"] = {
            "bound": "hbm", "kernel": "matmul kernel (forward launch)", "achieved": achieved,
            "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
            "peak_source": peaks["source"], "algorithmic_bytes": fb, "ms_per_launch": fwd_ms,
            "tensor_tflops": prob.wm["flops"]["fwd"] / (fwd_ms * 1e-3) / 1e12,
            "traffic": profiled_traffic(name, prob.wm["pairs"]["fwd"]),
        }
        del fgraph, _keepf

    # ---- N = 1 extras: the other workloads, the reference's Triton op, the CPU oracle ------------------
    if rank == 0 and world == 1 and not args.kernel_only and not args.quick:
        also, triton_rec = {}, {}
        try:
            ref = _import_reference()
        except Exception as exc:
            ref = None
            triton_rec = {"unavailable": f"reference not importable from baseline/_ref: {exc!r}"[:200]}

        def triton_on(p: Problem, label: str):
            if ref is None:
                return
            try:
                res = time_triton(ref, p.name, (p.lxd, p.lyd, p.lod), p.sets, p.bs, p.wm,
                                  5 if p.name == "config5" else 20, 3)
                triton_rec[label] = res
            except Exception as exc:  # the comparator must not take the bench line down
                triton_rec[label] = {"error": repr(exc)[:200]}

        triton_on(prob, name)
        ours_ms = {name: (line["kernel_only"]["ms_per_step"], line["ms_per_step"])}   # (kernel only, public op)
        ours_cold = {name: our_cold_call_ms(prob)}
        line["cold_call"] = {"ms": ours_cold[name], "what": "one forward call through the public op without any "
                             "layout cache (LUTs, plans, product; validation on), wall clock, median of 5"}
        del graph
        del prob
        torch.cuda.empty_cache()
        for other in [c for c in ("config2", "config1", "config3", "config4") if c != name]:
            try:
                rec, p = sub_record(other, dev, args, peaks)
                also[other] = rec
                ours_ms[other] = (rec["ms_per_step"], rec["api_ms_per_step"])
                if other in ("config1", "config2"):
                    triton_on(p, other)
                    ours_cold[other] = our_cold_call_ms(p)
                    rec["cold_call_ms"] = ours_cold[other]
                del p
            except Exception as exc:
                also[other] = {"error": repr(exc)[:300]}
            torch.cuda.empty_cache()
        for label, res in triton_rec.items():
            if isinstance(res, dict) and "validation_off/fwd" in res and label in ours_ms:
                key = "validation_off/fwd" if label in FORWARD_ONLY else "validation_off/fwd_bwd"
                if ours_ms[label][0]:
                    res["speedup_kernel_only"] = res[key]["ms_per_step"] / ours_ms[label][0]
                if ours_ms[label][1]:
                    res["speedup_public_op"] = res[key]["ms_per_step"] / ours_ms[label][1]
                if label in ours_cold and "validation_on/cold_fwd_ms" in res:
                    res["speedup_cold_call"] = res["validation_on/cold_fwd_ms"] / ours_cold[label]
        if ref is not None:
            triton_rec["what"] = ("reference bs.ops.matmul (Triton, BLKSPRS_AUTOTUNE=DEFAULT, autotune excluded) on the "
                                  "same GPU and tensors, warm layout_cache; speedup = reference validation_off time "
                                  "/ ours (kernel only, and through the public op with validation on); cold = one "
                                  "forward call without layout_cache, both with validation on")
        try:
            also["attention_chain"] = attention_chain_record(dev, peaks)
        except Exception as exc:
            also["attention_chain"] = {"error": repr(exc)[:300]}
        torch.cuda.empty_cache()
        line["also"] = also
        line["triton_reference"] = triton_rec
        if not args.no_cpu_baseline:
            sample = min(B, args.cpu_batch)
            dt, cflops = cpu_step_time(name, sample, 2, 1)
            what = "forward" if name in FORWARD_ONLY else "forward + backward"
            line["cpu_baseline"] = {"value": cflops / dt / 1e12, "unit": "TFLOP/s",
                                    "cores": torch.get_num_threads(), "kind": "port",
                                    "sample": f"{sample} of {B} batches, 2 steps of {what}, dense masked matmul"}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_e2e(prob: Problem, dev, args, barrier, world: int, flops_all: float):
    """Every step copies its pinned host inputs to the device, runs ops.matmul (+ backward) and copies
    all results back to pinned host memory.  The copies run on their own streams, two device slots
    deep, so the upload of step i+1 and the download of step i-1 overlap step i (the PCIe link is full
    duplex); nothing is skipped."""
    import torch.distributed as dist
    import blksprs_b200 as bs
    from blksprs_b200.plan import check_device_status
    n_in = 2 if prob.forward_only else 3
    host_in = tuple(t.cpu().pin_memory() for t in prob.sets[0][:n_in])
    layout_cache = {}
    h2d = sum(t.numel() * t.element_size() for t in host_in)
    dev_in = [tuple(torch.empty_like(t, device=dev) for t in host_in) for _ in range(2)]
    host_out = [None, None]
    keep = [None, None]
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_done = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]
    main = torch.cuda.current_stream(dev)
    state = {"d2h": 0, "issued": 0}

    def e2e_step(i):
        slot = i % 2
        with torch.cuda.stream(s_in):
            if state["issued"] >= 2:
                s_in.wait_event(ev_done[slot])       # step i-2 has finished reading this slot
            for dst, src in zip(dev_in[slot], host_in):
                dst.copy_(src, non_blocking=True)
            ev_in[slot].record(s_in)
        main.wait_event(ev_in[slot])
        if prob.forward_only:
            res = (bs.ops.matmul(dev_in[slot][0], prob.lxd, dev_in[slot][1], prob.lyd, prob.lod, prob.bs,
                                 layout_cache),)
        else:
            x = dev_in[slot][0].detach().requires_grad_(True)
            y = dev_in[slot][1].detach().requires_grad_(True)
            out = bs.ops.matmul(x, prob.lxd, y, prob.lyd, prob.lod, prob.bs, layout_cache)
            out.backward(dev_in[slot][2])
            res = (out.detach(), x.grad, y.grad)
        ev_done[slot].record(main)
        if host_out[slot] is None:
            host_out[slot] = tuple(torch.empty(t.shape, dtype=t.dtype, pin_memory=True) for t in res)
            state["d2h"] = sum(t.numel() * t.element_size() for t in res)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_done[slot])
            for dst, src in zip(host_out[slot], res):
                dst.copy_(src, non_blocking=True)
                src.record_stream(s_out)
            ev_out[slot].record(s_out)
        keep[slot] = res
        state["issued"] += 1
        if state["issued"] >= 2:
            ev_out[1 - slot].synchronize()           # bound the host's run-ahead to two steps

    def drain():
        main.wait_stream(s_out)
        main.wait_stream(s_in)

    steps = args.e2e_steps or args.steps
    for i in range(min(args.warmup, 3)):
        e2e_step(i)
    drain()
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    g0.record()
    for i in range(steps):
        e2e_step(i)
    drain()
    g1.record()
    barrier()
    ms = g0.elapsed_time(g1)
    check_device_status(dev)
    # the last step's results really are on the host
    last = (steps - 1) % 2
    ref_out = prob.plans.forward.run(prob.sets[0][0], prob.sets[0][1], prob.bs)
    assert torch.equal(host_out[last][0], ref_out.cpu()), "end-to-end result differs from the device-resident run"
    # plain copy rates of this rank (one direction at a time), to put the end-to-end figure in context
    c0, c1, c2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
    torch.cuda.synchronize()
    c0.record()
    for dst, src in zip(dev_in[0], host_in):
        dst.copy_(src, non_blocking=True)
    c1.record()
    for dst, src in zip(host_out[0], keep[0]):
        dst.copy_(src, non_blocking=True)
    c2.record()
    torch.cuda.synchronize()
    h2d_gbs = h2d / (c0.elapsed_time(c1) * 1e-3) / 1e9
    d2h_gbs = state["d2h"] / (c1.elapsed_time(c2) * 1e-3) / 1e9
    t = torch.tensor([ms, -h2d_gbs, -d2h_gbs], dtype=torch.float64, device=dev)
    tot = torch.tensor([float(h2d), float(state["d2h"])], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(tot, op=dist.ReduceOp.SUM)
    ms, h2d_min, d2h_min = t.tolist()
    return {"value": flops_all * steps / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
            "h2d_bytes_per_step": int(tot[0].item()), "d2h_bytes_per_step": int(tot[1].item()),
            "ms_per_step": ms / steps, "steps": steps,
            "copy_rate_gbs": {"h2d": -h2d_min, "d2h": -d2h_min,
                              "what": "slowest rank's plain pinned-memory copy rate, one direction at a time"}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--config", default="config5")
    ap.add_argument("--batch", type=int, default=None, help="batch size of the workload (default: its own)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "triton"])
    ap.add_argument("--regions", type=int, default=0, help="timed regions of --steps steps (default: >= 30)")
    ap.add_argument("--e2e-steps", type=int, default=0, help="steps of the end-to-end leg (default: --steps)")
    ap.add_argument("--cpu-batch", type=int, default=4, help="batches of the workload the CPU arm times")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true",
                    help="launch the device-resident legs kernel by kernel instead of replaying a CUDA graph")
    ap.add_argument("--kernel-only", action="store_true",
                    help="skip the public-op, end-to-end, comparator and CPU legs (for short profiler runs)")
    ap.add_argument("--quick", action="store_true", help="skip the other workloads, the Triton comparator and the CPU leg")
    ap.add_argument("--probe", choices=["softmax", "conversion", "matmul", "attention", "regular_attention", "nocache"], help="run a side probe instead")
    ap.add_argument("--small", action="store_true", help="with --probe: one small case")
    ap.add_argument("--iters", type=int, default=10, help="with --probe: timed iterations")
    args = ap.parse_args()
    if args.probe:
        import bench_probes
        bench_probes.run(args.probe, args.small, args.iters)
    elif args.impl == "reference":
        run_reference_arm(args)
    elif args.impl == "triton":
        run_triton_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
