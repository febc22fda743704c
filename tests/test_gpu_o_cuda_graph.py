"""Warm calls of the public ops read nothing from the device and allocate only through torch, so a chain
of them can be recorded into a CUDA graph and replayed on new values: attention by parts
(test/cases/test_blocksparse.py:1517-1529) as separate ops and with the fused op, block sizes 32 (mma.sync
kernels) and 64 (tcgen05 kernel, whose scheduling counters get a slot of their own per recorded launch)."""
import pytest
import torch

from gpu_util import DEV

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("bsz,dtype", [(32, torch.float32), (64, torch.bfloat16)], ids=["bs32-fp32", "bs64-bf16"])
@pytest.mark.parametrize("fused", [False, True], ids=["chain", "fused"])
def test_attention_by_parts_replays_from_a_graph(bsz, dtype, fused):
    import blksprs_b200 as bs
    heads, seq, d = 4, 8 * bsz, 2 * bsz
    g = torch.Generator().manual_seed(5)
    rows = seq // bsz
    layout = torch.rand((heads, rows, rows), generator=g) < 0.5
    layout[:, :, 0] = True
    l_attn = layout.to(DEV)
    l_qkv = torch.ones((heads, rows, d // bsz), dtype=torch.bool, device=DEV)
    q, k, v = (torch.randn((heads, seq, d), generator=g).to(DEV, dtype) for _ in range(3))
    qs, ks, vs = (bs.ops.to_sparse(t, l_qkv, bsz) for t in (q, k, v))
    kt, l_kt = bs.ops.transpose(ks, l_qkv, bsz)
    l_out = bs.layouting.build_sparsity_layout_matmul(l_attn, l_qkv)
    scale = d ** -0.5
    caches = ({}, {}, {})

    def chain():
        if fused:
            probs = bs.ops.matmul_softmax(qs, l_qkv, kt, l_kt, l_attn, bsz, scale=scale, layout_cache=caches[0])
        else:
            scores = bs.ops.matmul(qs, l_qkv, kt, l_kt, l_attn, bsz, layout_cache=caches[0])
            probs = bs.ops.softmax(scores.float() * scale, l_attn, bsz, layout_cache=caches[1]).to(dtype)
        return bs.ops.matmul(probs, l_attn, vs, l_qkv, l_out, bsz, layout_cache=caches[2])

    first = chain()                                   # builds LUTs and plans, validates the layouts
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        chain()                                        # once more on the capture stream before recording
        side.synchronize()
        with torch.cuda.graph(graph, stream=side, capture_error_mode="thread_local"):
            recorded = chain()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(recorded, first)
    # new values in the recorded operand buffers: the replay follows them
    for t in (qs, kt, vs):
        t.copy_(torch.randn(t.shape, generator=g).to(DEV, dtype))
    graph.replay()
    torch.cuda.synchronize()
    replayed = recorded.clone()
    assert torch.equal(replayed, chain())
    assert not torch.equal(replayed, first)
    from blksprs_b200.plan import check_device_status
    check_device_status()
