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


@pytest.mark.parametrize("B,H,D,page,seed", [(48, 3, 64, 16, 1), (40, 2, 128, 64, 2), (300, 1, 64, 128, 3)])
def test_paged_ragged_batch(B, H, D, page, seed):
    """One long request among many short ones, and more requests than the scan has CTAs per row:
    the runs of the CTAs are cut from the real lengths, every request must still come out as
    the contiguous op gives it."""
    e = ext()
    rng = np.random.default_rng(seed)
    lens = [int(v) for v in rng.integers(1, 700, size=B)]
    lens[B // 3] = 6000
    lens[0] = 1
    lens[-1] = 129
    Qi, sQ, Kp, Vp, sKp, sVp, table, seq, contig = _paged_case(B, H, D, lens, page, seed=seed)
    out = e.int8_decode_attention_paged(Qi, Kp, Vp, sQ.reshape(-1), sKp, sVp, table, seq, max(lens))
    assert not torch.isnan(out).any()
    for b, (Ki, Vi, sK, sV) in enumerate(contig):
        same = e.int8_decode_attention_forward(Qi[b:b + 1].contiguous(), Ki[None].contiguous(), Vi[None].contiguous(),
                                               sQ[b:b + 1].reshape(-1), sK.reshape(-1), sV.reshape(-1))
        tol = 2e-3 * max(1.0, float(same.float().abs().max()))
        assert (out[b:b + 1].float() - same.float()).abs().max().item() < tol, (b, lens[b])
    for b in (0, B // 3, B - 1):                  # and against the float64 oracle for the extremes
        Ki, Vi, sK, sV = contig[b]
        ref = odec.decode_attention(Qi[b:b + 1].cpu().numpy(), Ki[None].cpu().numpy(), Vi[None].cpu().numpy(),
                                    sQ[b:b + 1].cpu().numpy(), sK[None].cpu().numpy(), sV[None].cpu().numpy())
        assert cosine(out[b:b + 1].float().cpu().numpy(), ref) > 0.9999


def test_paged_request_without_positions_gives_zeros():
    e = ext()
    lens = [200, 5, 300, 140]
    Qi, sQ, Kp, Vp, sKp, sVp, table, seq, _ = _paged_case(4, 2, 64, lens, 32, seed=11)
    full = e.int8_decode_attention_paged(Qi, Kp, Vp, sQ.reshape(-1), sKp, sVp, table, seq, 300)
    for gone in (1, 3, 0):
        seq2 = seq.clone()
        seq2[gone] = 0
        out = e.int8_decode_attention_paged(Qi, Kp, Vp, sQ.reshape(-1), sKp, sVp, table, seq2, 300)
        assert torch.count_nonzero(out[gone]).item() == 0
        keep = [b for b in range(4) if b != gone]
        assert (out[keep].float() - full[keep].float()).abs().max().item() < 2e-3   # other runs, other merge order


def test_paged_more_requests_than_the_plan_keeps_in_shared_memory():
    """5000 requests: the plan kernel searches its prefix sums in global memory (it keeps up to
    4096 in shared memory).  Pages are shared between requests (the cache is only read), the
    result must match the same requests run in two batches of 2500 and, for a few of them, the
    contiguous op on the gathered pages."""
    e = ext()
    B, H, D, page, num_pages, max_pages = 5000, 2, 64, 16, 256, 20
    g = torch.Generator(device="cuda").manual_seed(5)
    Kp = torch.randint(-127, 128, (num_pages, H, page, D), dtype=torch.int8, device="cuda", generator=g)
    Vp = torch.randint(-127, 128, (num_pages, H, page, D), dtype=torch.int8, device="cuda", generator=g)
    sKp = torch.rand(num_pages, H, page, device="cuda", generator=g) * 0.02 + 0.005
    sVp = torch.rand(num_pages, H, page, device="cuda", generator=g) * 0.02 + 0.005
    table = torch.randint(0, num_pages, (B, max_pages), device="cuda", generator=g).to(torch.int32)
    seq = torch.randint(1, max_pages * page + 1, (B,), device="cuda", generator=g).to(torch.int32)
    Qi, sQ = e.quantize_per_token(torch.randn(B, H, D, device="cuda", generator=g))
    sq = sQ.reshape(-1).contiguous()
    S = max_pages * page
    out = e.int8_decode_attention_paged(Qi, Kp, Vp, sq, sKp, sVp, table, seq, S)
    assert not torch.isnan(out).any()
    for lo in (0, 2500):
        part = e.int8_decode_attention_paged(Qi[lo:lo + 2500].contiguous(), Kp, Vp, sq[lo * H:(lo + 2500) * H].contiguous(),
                                             sKp, sVp, table[lo:lo + 2500].contiguous(), seq[lo:lo + 2500].contiguous(), S)
        assert (out[lo:lo + 2500].float() - part.float()).abs().max().item() < 2e-3
    for b in (0, 1234, 4097, 4999):
        L = int(seq[b])
        n = (L + page - 1) // page
        ids = table[b, :n].long()
        Kc = Kp[ids].permute(1, 0, 2, 3).reshape(H, n * page, D)[:, :L].contiguous()
        Vc = Vp[ids].permute(1, 0, 2, 3).reshape(H, n * page, D)[:, :L].contiguous()
        sKc = sKp[ids].permute(1, 0, 2).reshape(H, n * page)[:, :L].contiguous()
        sVc = sVp[ids].permute(1, 0, 2).reshape(H, n * page)[:, :L].contiguous()
        same = e.int8_decode_attention_forward(Qi[b:b + 1].contiguous(), Kc[None], Vc[None], sQ[b:b + 1].reshape(-1),
                                               sKc.reshape(-1), sVc.reshape(-1))
        assert (out[b:b + 1].float() - same.float()).abs().max().item() < 2e-3


def test_page_id_outside_the_pool_is_not_followed():
    """With the pool size known (the op always passes it) a damaged page id is never used as an address:
    the kernel reads page 0 in its place, the other requests come out as before and check_status() reports
    the bad id; the call after that is clean again."""
    e = ext()
    lens = [300, 90, 257]
    Qi, sQ, Kp, Vp, sKp, sVp, table, seq, _ = _paged_case(3, 2, 64, lens, 16, seed=23)
    good = e.int8_decode_attention_paged(Qi, Kp, Vp, sQ.reshape(-1), sKp, sVp, table, seq, 300)
    torch.cuda.synchronize()
    e.check_status()
    bad = table.clone()
    bad[1, 2] = Kp.size(0) + 1000          # far outside the pool
    bad[1, 4] = -7
    out = e.int8_decode_attention_paged(Qi, Kp, Vp, sQ.reshape(-1), sKp, sVp, bad, seq, 300)
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all()
    assert (out[[0, 2]].float() - good[[0, 2]].float()).abs().max().item() < 2e-3
    with pytest.raises(RuntimeError, match="page id"):
        e.check_status()
    again = e.int8_decode_attention_paged(Qi, Kp, Vp, sQ.reshape(-1), sKp, sVp, table, seq, 300)
    torch.cuda.synchronize()
    e.check_status()
    assert (again.float() - good.float()).abs().max().item() < 2e-3
