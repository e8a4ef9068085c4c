"""Host-side logic of the multi-GPU paths, on CPU: partition arithmetic, and the
KV-sequence-sharded exchange run as 2 and 3 gloo ranks with numpy stand-ins
for the CUDA partial/merge ops."""
import math
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import decode as odec, quant
from helpers import pkg


def test_bh_ranges_cover_and_balance():
    sh = pkg().sharding
    for bh in (1, 7, 384, 2048, 2049):
        for world in (1, 2, 3, 4, 8):
            rs = [sh.bh_shard_range(bh, world, r) for r in range(world)]
            assert rs[0][0] == 0 and rs[-1][1] == bh
            assert all(a[1] == b[0] for a, b in zip(rs, rs[1:]))
            sizes = [b - a for a, b in rs]
            assert max(sizes) - min(sizes) <= 1


def test_seq_ranges_cover_and_align():
    sh = pkg().sharding
    for seq in (1, 100, 4096, 524288, 524289):
        for world in (1, 2, 4, 8):
            rs = [sh.seq_shard_range(seq, world, r) for r in range(world)]
            assert rs[0][0] == 0 and max(b for _, b in rs) == seq
            for (a, b), (c, d) in zip(rs, rs[1:]):
                assert b == c or (c == seq and d == seq)
            assert all(a % 128 == 0 or a == seq for a, _ in rs)


def _partial_np(Q, K, V, sQ, sK, sV):
    """numpy stand-in for int8_decode_attention_partial: rows (m in log2 units, l, 0, 0, acc)."""
    m, l, acc = odec.decode_partial(Q.numpy(), K.numpy(), V.numpy(), sQ.numpy(), sK.numpy(), sV.numpy(),
                                    0, K.shape[2])
    B, H, D = Q.shape
    row = np.zeros((B, H, D + 4), np.float32)
    row[..., 0] = m / math.log(2.0)
    row[..., 1] = l
    row[..., 4:] = acc
    return torch.from_numpy(row)


def _combine_np(parts):
    p = parts.numpy().astype(np.float64)
    _, _, _, out = odec.combine_partials(p[..., 0] * math.log(2.0), p[..., 1], p[..., 4:])
    return torch.from_numpy(out)


def _worker(rank, world, port, seq, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        sh = pkg().sharding
        rng = np.random.default_rng(0)           # every rank draws the same full problem
        B, H, D = 2, 3, 64
        q = rng.standard_normal((B, H, D)).astype(np.float16)
        K = rng.standard_normal((B, H, seq, D)).astype(np.float32)
        V = rng.standard_normal((B, H, seq, D)).astype(np.float32)
        Qi, sQ = quant.quantize_per_token(q)
        Ki, sK = quant.quantize_per_token(K)
        Vi, sV = quant.quantize_per_token(V)
        a, b = sh.seq_shard_range(seq, world, rank)
        t = lambda x: torch.from_numpy(np.ascontiguousarray(x))
        out = sh.decode_attention_seq_sharded(t(Qi), t(Ki[:, :, a:b]), t(Vi[:, :, a:b]), t(sQ), t(sK[:, :, a:b]),
                                              t(sV[:, :, a:b]), partial_fn=_partial_np, combine_fn=_combine_np)
        full = odec.decode_attention(Qi, Ki, Vi, sQ, sK, sV)
        err = float(np.abs(out.numpy() - full).max())
        with open(os.path.join(result_dir, f"r{rank}.txt"), "w") as f:
            f.write(repr(err))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,seq", [(2, 1000), (3, 200), (2, 100)])
def test_seq_sharded_exchange_over_gloo(world, seq, tmp_path):
    port = 29500 + (os.getpid() % 2000) + world * 7 + seq % 13
    mp.spawn(_worker, args=(world, port, seq, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        err = float(open(tmp_path / f"r{r}.txt").read())
        assert err < 1e-5, (r, err)


def _withholding_worker(rank, world, port, result_dir):
    """Step 1 runs on every rank; the last rank then leaves between steps, so step 2 is one
    partial short.  The ranks that stay must get an error from the exchange, not a wrong answer
    and not a hang (the process group carries a short timeout)."""
    import datetime
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    sh = pkg().sharding
    rng = np.random.default_rng(1)
    B, H, D, seq = 1, 2, 64, 256
    Qi, sQ = quant.quantize_per_token(rng.standard_normal((B, H, D)).astype(np.float16))
    Ki, sK = quant.quantize_per_token(rng.standard_normal((B, H, seq, D)).astype(np.float32))
    Vi, sV = quant.quantize_per_token(rng.standard_normal((B, H, seq, D)).astype(np.float32))
    a, b = sh.seq_shard_range(seq, world, rank)
    t = lambda x: torch.from_numpy(np.ascontiguousarray(x))
    args = (t(Qi), t(Ki[:, :, a:b]), t(Vi[:, :, a:b]), t(sQ), t(sK[:, :, a:b]), t(sV[:, :, a:b]))
    step = lambda: sh.decode_attention_seq_sharded(*args, partial_fn=_partial_np, combine_fn=_combine_np)
    out = step()
    ok1 = float(np.abs(out.numpy() - odec.decode_attention(Qi, Ki, Vi, sQ, sK, sV)).max()) < 1e-5
    verdict = "step1-bad"
    if ok1:
        if rank == world - 1:
            verdict = "left"                      # withholds its partial of step 2
        else:
            try:
                step()
                verdict = "step2-returned"        # must not happen: a partial is missing
            except Exception as e:                # noqa: BLE001  (gloo raises RuntimeError / DistBackendError)
                verdict = "error:" + type(e).__name__
    with open(os.path.join(result_dir, f"r{rank}.txt"), "w") as f:
        f.write(verdict)
    os._exit(0)                                   # no collective teardown with a rank gone


def test_rank_that_withholds_its_partial_surfaces_as_an_error(tmp_path):
    world = 2
    port = 29500 + (os.getpid() % 2000) + 911
    mp.spawn(_withholding_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert open(tmp_path / "r1.txt").read() == "left"
    assert open(tmp_path / "r0.txt").read().startswith("error:")
