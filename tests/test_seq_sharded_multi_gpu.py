"""KV-sequence-sharded decode on 2+ GPUs: the fused peer-memory exchange
(SeqShardedDecoder) against the NCCL all-gather path and the single-GPU forward.
Runs as child processes, one per GPU; skipped with fewer than two GPUs."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import pkg

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        p = pkg()
        ext, sh = p.int8_ext, p.sharding
        errs = []
        for (B, H, D, S) in [(2, 8, 128, 4096 * world + 300), (3, 4, 64, 1000)]:
            g = torch.Generator(device="cuda").manual_seed(5)        # same full problem on every rank
            Qi, sQ = ext.quantize_per_token(torch.randn(B, H, D, device="cuda", dtype=torch.float16, generator=g))
            Ki, sK = ext.quantize_per_token(torch.randn(B, H, S, D, device="cuda", generator=g))
            Vi, sV = ext.quantize_per_token(torch.randn(B, H, S, D, device="cuda", generator=g))
            full = ext.int8_decode_attention_forward(Qi, Ki, Vi, sQ, sK, sV)
            a, b = sh.seq_shard_range(S, world, rank)
            loc = [Qi, Ki[:, :, a:b].contiguous(), Vi[:, :, a:b].contiguous(), sQ,
                   sK[:, :, a:b].contiguous(), sV[:, :, a:b].contiguous()]
            via_nccl = sh.decode_attention_seq_sharded(*loc)
            dec = sh.SeqShardedDecoder(B, H, D, torch.device("cuda", rank))
            for _ in range(3):                                        # epochs 1..3 reuse the buffers
                fused = dec(*loc)
            dec.check()
            errs.append(float((fused.float() - full.float()).abs().max()))
            errs.append(float((fused.float() - via_nccl.float()).abs().max()))
        with open(os.path.join(result_dir, f"r{rank}.txt"), "w") as f:
            f.write(repr(max(errs)))
    finally:
        dist.destroy_process_group()


def test_fused_exchange_matches_nccl_path_and_single_gpu(tmp_path):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    port = 29600 + os.getpid() % 1000
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert float(open(tmp_path / f"r{r}.txt").read()) < 2e-3
