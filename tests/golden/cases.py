"""Seeded inputs shared by ``make_golden.py`` (which feeds them to the reference) and the tests
(which feed the same inputs to the oracle and to the CUDA path).  CPU tensors only."""
import torch


def _gen(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


def bernoulli_layout(shape, p: float, seed: int) -> torch.Tensor:
    return torch.rand(shape, generator=_gen(seed)) < p


def lut_layouts():
    """(name, layout) pairs covering dtypes, empty / full / single-block layouts and sizes that
    cross the 2048-entry chunk boundary of the device scan."""
    probe = torch.tensor([[[1, 0], [0, 1]], [[0, 1], [1, 1]]], dtype=torch.bool)
    rnd = bernoulli_layout((3, 5, 7), 0.5, 10)
    big = bernoulli_layout((4, 33, 65), 0.25, 11)
    return [
        ("probe_bool", probe),
        ("random_bool", rnd),
        ("ones_float32", torch.ones((2, 4, 4), dtype=torch.float32)),
        ("random_int32", rnd.to(torch.int32)),
        ("random_int64", rnd.to(torch.int64)),
        ("random_uint8", rnd.to(torch.uint8)),
        ("random_float16", rnd.to(torch.float16)),
        ("random_float64", rnd.to(torch.float64)),
        ("all_zero", torch.zeros((2, 3, 4), dtype=torch.bool)),
        ("single_block", torch.ones((1, 1, 1), dtype=torch.bool)),
        ("last_only", torch.zeros((2, 9, 9), dtype=torch.bool).index_put_(
            (torch.tensor([1]), torch.tensor([8]), torch.tensor([8])), torch.tensor(True))),
        ("multi_chunk_bool", big),
        ("multi_chunk_float32", big.to(torch.float32)),
        ("dense_multi_chunk", torch.ones((3, 40, 40), dtype=torch.bool)),
    ]


def layout_pairs():
    """(name, layout_x, layout_y) for output-layout inference."""
    return [
        ("small", bernoulli_layout((2, 4, 6), 0.4, 20), bernoulli_layout((2, 6, 5), 0.4, 21)),
        ("sparse", bernoulli_layout((3, 16, 16), 0.1, 22), bernoulli_layout((3, 16, 8), 0.1, 23)),
        ("float_layouts", bernoulli_layout((2, 8, 8), 0.5, 24).float(), bernoulli_layout((2, 8, 8), 0.5, 25).float()),
        ("mixed_dtypes", bernoulli_layout((2, 8, 4), 0.5, 26).to(torch.int32), bernoulli_layout((2, 4, 8), 0.5, 27)),
        ("empty_inner", torch.zeros((1, 2, 0), dtype=torch.bool), torch.zeros((1, 0, 3), dtype=torch.bool)),
        ("empty_rows", torch.zeros((2, 5, 5), dtype=torch.bool), torch.ones((2, 5, 5), dtype=torch.bool)),
        ("tall", bernoulli_layout((2, 64, 2), 0.5, 28), bernoulli_layout((2, 2, 64), 0.5, 29)),
    ]


def config2_layouts(batch: int = 16):
    """Layouts of the bf16 SDD benchmark workload: (batch, 32, 32) Bernoulli(0.25) for x then y, seed 1."""
    g = _gen(1)
    lx = torch.rand((batch, 32, 32), generator=g) < 0.25
    ly = torch.rand((batch, 32, 32), generator=g) < 0.25
    return lx, ly


def big_layout_pairs():
    lx, ly = config2_layouts()
    return [("config2", lx, ly)]


def config1_case():
    """The plumbing workload: fp32, B=2, 128x128x128, bs=16, Bernoulli(0.5) layouts from seed 0 with
    one block forced per empty batch, all-ones output layout, N(0,1) values."""
    g = _gen(0)
    lx = torch.rand((2, 8, 8), generator=g) < 0.5
    ly = torch.rand((2, 8, 8), generator=g) < 0.5
    for layout in (lx, ly):
        for b in range(layout.size(0)):
            if not layout[b].any():
                layout[b, 0, 0] = True
    lo = torch.ones((2, 8, 8), dtype=torch.bool)
    return _values(lx, ly, lo, 16, torch.float32, g)


def _values(lx, ly, lo, bs, dtype, g):
    x = torch.randn((int(lx.sum()), bs, bs), generator=g).to(dtype)
    y = torch.randn((int(ly.sum()), bs, bs), generator=g).to(dtype)
    grad = torch.randn((int(lo.sum()), bs, bs), generator=g).to(dtype)
    return {"x": x, "lx": lx, "y": y, "ly": ly, "lo": lo, "bs": bs, "grad": grad}


def _random_case(seed, B, R, K, C, bs, p, dtype, out="exact"):
    g = _gen(seed)
    lx = torch.rand((B, R, K), generator=g) < p
    ly = torch.rand((B, K, C), generator=g) < p
    if out == "ones":
        lo = torch.ones((B, R, C), dtype=torch.bool)
    elif out == "exact":
        lo = torch.matmul(lx.float(), ly.float()) != 0
    else:  # a random output layout, unrelated to the structural product
        lo = torch.rand((B, R, C), generator=g) < 0.5
    return _values(lx, ly, lo, bs, dtype, g)


def matmul_cases():
    """(name, case) run through the reference's Triton kernels under the interpreter."""
    return [
        ("config1", config1_case()),
        ("rect_fp32_bs16", _random_case(30, 3, 3, 2, 4, 16, 0.6, torch.float32, "ones")),
        ("exact_fp32_bs16", _random_case(31, 2, 4, 4, 4, 16, 0.4, torch.float32, "exact")),
        ("random_out_fp32_bs32", _random_case(32, 2, 2, 3, 2, 32, 0.6, torch.float32, "random")),
        ("fp16_bs16", _random_case(33, 2, 3, 3, 3, 16, 0.6, torch.float16, "ones")),
        ("empty_x_fp32_bs16", _random_case(34, 1, 2, 2, 2, 16, 0.0, torch.float32, "ones")),
    ]
