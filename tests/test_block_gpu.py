"""The pre-LN block around the INT8 ops (the caller either side of the hot path) against the
same block in fp16: the reference's own acceptance for its block bench is the cosine of the
two outputs (bench/bench_block.py:163-176)."""
import importlib

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _cos(a, b):
    return F.cosine_similarity(a.float().flatten(), b.float().flatten(), dim=0).item()


def _block(d, H, dff):
    return importlib.import_module("int8-transformer-kernels_b200").block.Int8Block(d, H, dff)


@pytest.mark.parametrize("B,H,Dh,dff,S", [(2, 8, 64, 2048, 256), (1, 4, 128, 1024, 384)])
def test_prefill_block_matches_fp16_block(B, H, Dh, dff, S):
    blk = _block(H * Dh, H, dff)
    x = torch.randn(B, S, H * Dh, device="cuda", dtype=torch.float16)
    i8 = blk.forward_prefill(x, True)
    f16 = blk.forward_prefill(x, False)
    assert i8.shape == f16.shape and not torch.isnan(i8).any()
    assert _cos(i8, f16) > 0.999
    mixed = blk.forward_prefill(x, True, fp16_attention=True)     # fp16 attention, INT8 feed-forward
    assert _cos(mixed, f16) > 0.999


@pytest.mark.parametrize("B,H,Dh,dff,Skv", [(128, 8, 64, 2048, 1024), (128, 4, 128, 1024, 777)])
def test_decode_block_matches_fp16_block(B, H, Dh, dff, Skv):
    blk = _block(H * Dh, H, dff)
    x = torch.randn(B, 1, H * Dh, device="cuda", dtype=torch.float16)
    K = torch.randn(B, H, Skv, Dh, device="cuda", dtype=torch.float16)
    V = torch.randn(B, H, Skv, Dh, device="cuda", dtype=torch.float16)
    i8 = blk.forward_decode(x, blk.quantize_kv(K, V), True)
    f16 = blk.forward_decode(x, (K, V), False)
    assert i8.shape == f16.shape and not torch.isnan(i8).any()
    assert _cos(i8, f16) > 0.999
