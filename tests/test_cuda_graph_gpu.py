"""The kernels of one call are chained by programmatic dependent launch; a CUDA graph captured
from the ops must replay to the same bits as the eager calls (decode forward, MLP forward,
quantiser), also when the inputs change between replays."""
import pytest
import torch

from helpers import ext

pytestmark = pytest.mark.gpu


def _decode_inputs(seed, B=2, H=4, S=2048, D=64):
    g = torch.Generator(device="cuda").manual_seed(seed)
    e = ext()
    Qi, sQ = e.quantize_per_token(torch.randn(B, H, D, device="cuda", generator=g))
    Ki, sK = e.quantize_per_token(torch.randn(B, H, S, D, device="cuda", generator=g))
    Vi, sV = e.quantize_per_token(torch.randn(B, H, S, D, device="cuda", generator=g))
    return [Qi, Ki, Vi, sQ.reshape(-1).contiguous(), sK.reshape(-1).contiguous(), sV.reshape(-1).contiguous()]


def test_decode_forward_replays_from_a_graph():
    e = ext()
    static = _decode_inputs(0)
    eager0 = e.int8_decode_attention_forward(*static).clone()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            e.int8_decode_attention_forward(*static)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = e.int8_decode_attention_forward(*static)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, eager0)
    fresh = _decode_inputs(1)
    for dst, src in zip(static, fresh):
        dst.copy_(src)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, e.int8_decode_attention_forward(*fresh))


def test_mlp_forward_replays_from_a_graph():
    e = ext()
    g = torch.Generator(device="cuda").manual_seed(3)
    M, dm, dff = 512, 256, 1024
    xi, sx = e.quantize_per_token(torch.randn(1, M, dm, device="cuda", dtype=torch.float16, generator=g))
    w1 = torch.randint(-127, 128, (dm, dff), dtype=torch.int8, device="cuda", generator=g)
    w2 = torch.randint(-127, 128, (dff, dm), dtype=torch.int8, device="cuda", generator=g)
    s1 = torch.rand(dff, device="cuda", generator=g) * 1e-3 + 1e-3
    s2 = torch.rand(dm, device="cuda", generator=g) * 1e-3 + 1e-3
    b1 = torch.randn(dff, device="cuda", generator=g) * 0.01
    sxf = sx.reshape(-1).contiguous()
    eager, eager_sc = e.int8_mlp_forward_per_channel_bias(xi, w1, w2, sxf, s1, s2, b1)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        e.int8_mlp_forward_per_channel_bias(xi, w1, w2, sxf, s1, s2, b1)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out, osc = e.int8_mlp_forward_per_channel_bias(xi, w1, w2, sxf, s1, s2, b1)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, eager) and torch.equal(osc, eager_sc)
