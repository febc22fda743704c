"""Small timing probes of the kernels around the matmul (conversion, softmax) and of the public
matmul op over every dtype and block size; run through ``bench.py``.

``python bench.py --probe attention [--small]`` times the attention-score chain (separate ops against the
fused ``matmul_softmax``); ``--probe regular_attention`` the reference's own timing test of attention by parts
(fp32, block size 32).  ``python bench.py --probe softmax|conversion [--small]`` prints one line per case with the achieved
bandwidth (algorithmic bytes / CUDA-event time).  ``--small`` runs one case of a few hundred MB, the
size used for profiler captures.  ``python bench.py --probe matmul`` times the public matmul op
(forward, forward + backward) for every dtype and block size on a 16 x 2048^3 problem with 25 %
dense random layouts.
"""
from __future__ import annotations

import torch

import blksprs_b200 as bs


def _time(fn, iters: int) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def softmax(small: bool, iters: int) -> None:
    cases = [(32, 64, 64, 64, 0.25)] if small else [(128, 64, 64, 64, 0.25), (64, 64, 64, 64, 1.0),
                                                     (32, 32, 32, 128, 0.5), (256, 64, 64, 16, 0.25)]
    bs.utils.disable_validation()  # the checks read counts back from the device, which would serialise the launches
    for B, R, C, bsz, kept in cases:
        g = torch.Generator().manual_seed(1)
        layout = torch.rand((B, R, C), generator=g) < kept
        layout[:, :, 0] = True
        layout = layout.cuda()
        n = int(layout.sum())
        x = torch.randn((n, bsz, bsz), device="cuda")
        cache = {}
        xs = x.clone().requires_grad_(True)
        out = bs.ops.softmax(xs, layout, bsz, layout_cache=cache)
        grad = torch.randn_like(out)

        def backward():
            xs.grad = None
            out.backward(grad, retain_graph=True)

        fwd = _time(lambda: bs.ops.softmax(x, layout, bsz, layout_cache=cache), iters)
        bwd = _time(backward, iters)
        nbytes = n * bsz * bsz * 4
        print(f"softmax B={B} R={R} C={C} bs={bsz} kept={kept}: {nbytes / 2**20:.0f} MiB  "
              f"forward {fwd * 1e3:.0f} us = {2 * nbytes / fwd / 1e6:.0f} GB/s  "
              f"backward {bwd * 1e3:.0f} us = {3 * nbytes / bwd / 1e6:.0f} GB/s")
    bs.utils.enable_validation()


def conversion(small: bool, iters: int) -> None:
    cases = [(64, 8, 4096, 0.25)] if small else [(64, 32, 4096, 0.25), (64, 32, 4096, 1.0), (128, 32, 4096, 0.25),
                                                  (16, 8, 4096, 0.5)]
    bs.utils.disable_validation()  # the checks read counts back from the device, which would serialise the launches
    for bsz, B, n, kept in cases:
        g = torch.Generator(device="cuda")
        g.manual_seed(0)
        layout = torch.rand((B, n // bsz, n // bsz), generator=g, device="cuda") < kept
        dense = torch.randn((B, n, n), device="cuda", dtype=torch.bfloat16)
        c1, c2 = {}, {}
        comp = bs.ops.to_sparse(dense, layout, bsz, c1)
        for name, fn, nbytes in (
                ("to_sparse", lambda: bs.ops.to_sparse(dense, layout, bsz, c1), 2 * comp.numel() * 2),
                ("to_dense", lambda: bs.ops.to_dense(comp, layout, bsz, 0, c2), comp.numel() * 2 + dense.numel() * 2)):
            ms = _time(fn, iters)
            print(f"{name} bs={bsz} B={B} n={n} kept={kept}: {ms * 1e3:.0f} us  {nbytes / ms / 1e6:.0f} GB/s "
                  f"({nbytes / 1e6:.0f} MB moved)")
    bs.utils.enable_validation()


def matmul(small: bool, iters: int) -> None:
    bs.utils.disable_validation()
    B, n, kept = (4 if small else 16), 2048, 0.25
    for dtype in (torch.float32, torch.bfloat16, torch.float16):
        for bsz in (16, 32, 64, 128):
            g = torch.Generator().manual_seed(1)
            lx = (torch.rand((B, n // bsz, n // bsz), generator=g) < kept).cuda()
            ly = (torch.rand((B, n // bsz, n // bsz), generator=g) < kept).cuda()
            lo = bs.layouting.build_sparsity_layout_matmul(lx, ly)
            x = torch.randn((int(lx.sum()), bsz, bsz), device="cuda", dtype=dtype)
            y = torch.randn((int(ly.sum()), bsz, bsz), device="cuda", dtype=dtype)
            flops = 2.0 * float((lx.float() @ ly.float())[lo].sum()) * bsz ** 3
            cache = {}
            xs, ys = x.clone().requires_grad_(True), y.clone().requires_grad_(True)
            grad = torch.randn_like(bs.ops.matmul(xs, lx, ys, ly, lo, bsz, cache)).as_subclass(torch.Tensor)

            def step():
                xs.grad = ys.grad = None
                bs.ops.matmul(xs, lx, ys, ly, lo, bsz, cache).backward(grad)

            fwd = _time(lambda: bs.ops.matmul(x, lx, y, ly, lo, bsz, cache), iters)
            both = _time(step, iters)
            print(f"matmul {str(dtype)[6:]} bs={bsz}: forward {fwd * 1e3:.0f} us = {flops / fwd / 1e9:.0f} TFLOP/s  "
                  f"forward+backward {both * 1e3:.0f} us = {3 * flops / both / 1e9:.0f} TFLOP/s")
    bs.utils.enable_validation()


def attention(small: bool, iters: int) -> None:
    """softmax(scale * Q K^T) on the banded causal layout of the attention-score workload, as separate ops
    and as the fused op, then P V (``bench.attention_chain_record``); ``--small`` runs 32 of the 512 batches."""
    import json

    import bench
    rec = bench.attention_chain_record(torch.device("cuda", 0), bench.measured_peaks(), batch=32 if small else None)
    print(json.dumps(rec))


def nocache(small: bool, iters: int) -> None:
    """Calls WITHOUT a ``layout_cache`` (the reference's default): time per forward call on unchanged layout
    objects, with the library-owned caches on and off, and the reference's op called the same way."""
    import bench
    ref = None
    try:
        ref = bench._import_reference()
    except Exception as exc:
        print(f"reference not importable: {exc!r}")
    for name in ("config1", "config2") + (() if small else ("config5",)):
        lx, ly, lo, bsz, dtype = bench.workload_layouts(name, batch=8 if name == "config5" else None)
        x, y, _ = bench.workload_values(name, lx, ly, lo, bsz, dtype, seed=0, device="cuda")
        lxd, lyd, lod = lx.cuda(), ly.cuda(), lo.cuda()
        bs.utils.set_implicit_layout_caches(True)
        warm = _time(lambda: bs.ops.matmul(x, lxd, y, lyd, lod, bsz), iters)
        bs.utils.set_implicit_layout_caches(False)
        cold = _time(lambda: bs.ops.matmul(x, lxd, y, lyd, lod, bsz), iters)
        bs.utils.set_implicit_layout_caches(True)
        line = f"{name}: forward call without layout_cache: {warm * 1e3:.0f} us (library-owned cache), {cold * 1e3:.0f} us (rebuild every call)"
        if ref is not None:
            t = _time(lambda: ref.ops.matmul(x, lxd, y, lyd, lod, bsz), iters)
            line += f", reference {t * 1e3:.0f} us"
        print(line)


def regular_attention(small: bool, iters: int) -> None:
    """The one timing test the reference ships (test/cases/test_blocksparse.py:1481-1579): attention by
    parts, ``matmul(Q, K^T) -> * scale -> softmax -> matmul(P, V)``, with 8 heads, head dimension 64,
    fp32, block size 32, half of the attention blocks kept (no empty row), sequence length 512 / 1024 /
    2048; three warm-up runs, ten runs timed one by one with CUDA events, the median.  Timed here
    through this library's ops (the chain, with ``matmul_softmax`` in place of the first three steps,
    and that pair replayed from a CUDA graph) and, where the reference is importable, through the reference's ops on the same tensors,
    with both results compared."""
    import bench
    ref = None
    try:
        ref = bench._import_reference()
    except Exception as exc:
        print(f"reference not importable: {exc!r}")
    heads, d, bsz, kept = 8, 64, 32, 0.5
    for m in (512,) if small else (512, 1024, 2048):
        g = torch.Generator().manual_seed(m)
        rows = m // bsz
        layout = torch.ones((heads, rows, rows), dtype=torch.bool)
        for h in range(heads):
            drop = torch.randperm(rows * rows, generator=g)[:int(rows * rows * (1 - kept))]
            layout[h, drop // rows, drop % rows] = False
            for i in torch.nonzero(~layout[h].any(dim=1)).flatten().tolist():
                layout[h, i, int(torch.randint(0, rows, (1,), generator=g))] = True
        q, k, v = (torch.randn((heads, m, d), generator=g).cuda() for _ in range(3))
        l_qkv = torch.ones((heads, rows, d // bsz), dtype=torch.bool, device="cuda")
        l_attn = layout.cuda()
        scale = d ** -0.5

        def chain_of(lib):
            qs, ks, vs = (lib.ops.to_sparse(t, l_qkv, bsz) for t in (q, k, v))
            kt, l_kt = lib.ops.transpose(ks, l_qkv, bsz)
            l_out = lib.layouting.build_sparsity_layout_matmul(l_attn, l_qkv)
            caches = ({}, {}, {})

            def run():
                scores = lib.ops.matmul(qs, l_qkv, kt, l_kt, l_attn, bsz, layout_cache=caches[0]) * scale
                probs = lib.ops.softmax(scores, l_attn, bsz, layout_cache=caches[1])
                return lib.ops.matmul(probs, l_attn, vs, l_qkv, l_out, bsz, layout_cache=caches[2])
            return run, (qs, kt, l_kt, vs, l_out)

        def median_ms(fn):
            for _ in range(3):
                out = fn()
            torch.cuda.synchronize()
            times = []
            for _ in range(10):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                torch.cuda.synchronize()
                times.append(e0.elapsed_time(e1))
            return sorted(times)[5], out

        ours, (qs, kt, l_kt, vs, l_out) = chain_of(bs)
        fused_caches = ({}, {})

        def fused():
            probs = bs.ops.matmul_softmax(qs, l_qkv, kt, l_kt, l_attn, bsz, scale=scale, layout_cache=fused_caches[0])
            return bs.ops.matmul(probs, l_attn, vs, l_qkv, l_out, bsz, layout_cache=fused_caches[1])

        t_ours, out_ours = median_ms(ours)
        t_fused, out_fused = median_ms(fused)
        # the fused pair recorded into a CUDA graph: what is left when the host path is taken out
        side, graph = torch.cuda.Stream(), torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            fused()
            side.synchronize()
            with torch.cuda.graph(graph, stream=side, capture_error_mode="thread_local"):
                fused()
        t_graph, _ = median_ms(lambda: graph.replay())
        line = (f"regular attention seq={m}: {t_ours * 1e3:.0f} us (chain of four ops), "
                f"{t_fused * 1e3:.0f} us (matmul_softmax + matmul), {t_graph * 1e3:.0f} us (the latter replayed from a "
                f"CUDA graph)")
        plain = lambda t: t.as_subclass(torch.Tensor).float()
        err = float((plain(out_fused) - plain(out_ours)).abs().max())
        if ref is not None:
            theirs, _ = chain_of(ref)
            t_ref, out_ref = median_ms(theirs)
            err_ref = float((plain(out_ours) - plain(out_ref)).abs().max() / plain(out_ref).abs().max())
            line += f", reference {t_ref * 1e3:.0f} us; max |ours - reference| = {err_ref:.1e} of max |reference|"
        print(line + f"; max |fused - chain| = {err:.1e}")


PROBES = {"nocache": nocache, "softmax": softmax, "conversion": conversion, "matmul": matmul, "attention": attention,
          "regular_attention": regular_attention}


def run(what: str, small: bool, iters: int) -> None:
    PROBES[what](small, iters)
