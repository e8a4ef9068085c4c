"""Decode attention over a paged INT8 KV cache with one length per request: against the
float64 oracle of each request, and against the contiguous op on the same data."""
import numpy as np
import pytest
import torch

from oracle import decode as odec
from helpers import ext, cosine

pytestmark = pytest.mark.gpu


def _paged_case(B, H, D, lens, page, seed, extra_pages=3):
    """Contiguous int8 K/V per request -> pools with a shuffled page assignment."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    e = ext()
    max_len = max(lens)
    max_pages = (max_len + page - 1) // page + 1
    need = sum((l + page - 1) // page for l in lens)
    num_pages = need + extra_pages
    perm = torch.randperm(num_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    K_pool = torch.randint(-127, 128, (num_pages, H, page, D), dtype=torch.int8, device="cuda", generator=g)
    V_pool = torch.randint(-127, 128, (num_pages, H, page, D), dtype=torch.int8, device="cuda", generator=g)
    sK_pool = torch.rand(num_pages, H, page, device="cuda", generator=g) + 7.0     # junk that must never be used
    sV_pool = torch.rand(num_pages, H, page, device="cuda", generator=g) + 7.0
    table = torch.full((B, max_pages), -1, dtype=torch.int32)
    Qi, sQ = e.quantize_per_token(torch.randn(B, H, D, device="cuda", generator=g))
    contig = []
    nxt = 0
    for b, L in enumerate(lens):
        Ki, sK = e.quantize_per_token(torch.randn(H, L, D, device="cuda", generator=g))
        Vi, sV = e.quantize_per_token(torch.randn(H, L, D, device="cuda", generator=g) * 2)
        contig.append((Ki, Vi, sK, sV))
        for p in range((L + page - 1) // page):
            pid = perm[nxt]; nxt += 1
            table[b, p] = pid
            n = min(page, L - p * page)
            K_pool[pid, :, :n] = Ki[:, p * page:p * page + n]
            V_pool[pid, :, :n] = Vi[:, p * page:p * page + n]
            sK_pool[pid, :, :n] = sK[:, p * page:p * page + n]
            sV_pool[pid, :, :n] = sV[:, p * page:p * page + n]
    table = table.clamp(min=0).cuda()          # unused entries point at page 0: they must not be read for data
    seq = torch.tensor(lens, dtype=torch.int32, device="cuda")
    return Qi, sQ, K_pool, V_pool, sK_pool, sV_pool, table, seq, contig


@pytest.mark.parametrize("B,H,D,page,lens", [
    (3, 2, 64, 16, [1, 130, 77]),
    (2, 4, 128, 16, [257, 16]),
    (4, 2, 64, 32, [500, 33, 1000, 128]),
    (2, 3, 128, 64, [640, 65]),
    (3, 2, 64, 128, [128, 129, 700]),
    (2, 12, 64, 16, [2048, 1500]),
])
def test_paged_matches_oracle_and_contiguous(B, H, D, page, lens):
    e = ext()
    Qi, sQ, Kp, Vp, sKp, sVp, table, seq, contig = _paged_case(B, H, D, lens, page, seed=sum(lens) + page)
    out = e.int8_decode_attention_paged(Qi, Kp, Vp, sQ.reshape(-1), sKp, sVp, table, seq, max(lens))
    assert out.shape == (B, H, D) and out.dtype == torch.float16 and not torch.isnan(out).any()
    for b, (Ki, Vi, sK, sV) in enumerate(contig):
        ref = odec.decode_attention(Qi[b:b + 1].cpu().numpy(), Ki[None].cpu().numpy(), Vi[None].cpu().numpy(),
                                    sQ[b:b + 1].cpu().numpy(), sK[None].cpu().numpy(), sV[None].cpu().numpy())
        got = out[b:b + 1].float().cpu().numpy()
        assert cosine(got, ref) > 0.9999
        assert np.abs(got - ref).max() < 2e-3 * max(1.0, float(np.abs(ref).max()))
        same = e.int8_decode_attention_forward(Qi[b:b + 1].contiguous(), Ki[None].contiguous(), Vi[None].contiguous(),
                                               sQ[b:b + 1].reshape(-1), sK.reshape(-1), sV.reshape(-1))
        assert (out[b:b + 1].float() - same.float()).abs().max().item() < 2e-3 * max(1.0, float(np.abs(ref).max()))


def test_paged_is_deterministic_and_rejects_bad_arguments():
    e = ext()
    Qi, sQ, Kp, Vp, sKp, sVp, table, seq, _ = _paged_case(2, 2, 64, [300, 40], 16, seed=9)
    a = e.int8_decode_attention_paged(Qi, Kp, Vp, sQ.reshape(-1), sKp, sVp, table, seq, 300)
    b = e.int8_decode_attention_paged(Qi, Kp, Vp, sQ.reshape(-1), sKp, sVp, table, seq, 304)   # looser bound, same result
    assert torch.equal(a, e.int8_decode_attention_paged(Qi, Kp, Vp, sQ.reshape(-1), sKp, sVp, table, seq, 300))
    assert (a.float() - b.float()).abs().max().item() < 2e-3
    with pytest.raises(RuntimeError):
        e.int8_decode_attention_paged(Qi, Kp, Vp, sQ.reshape(-1), sKp, sVp, table, seq, 10 ** 6)
    with pytest.raises(RuntimeError):
        e.int8_decode_attention_paged(Qi, Kp[:, :, :8].contiguous(), Vp[:, :, :8].contiguous(), sQ.reshape(-1),
                                      sKp[:, :, :8].contiguous(), sVp[:, :, :8].contiguous(), table, seq, 300)
