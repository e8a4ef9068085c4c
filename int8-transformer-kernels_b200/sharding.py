"""Multi-GPU decode attention: one process per GPU, torch.distributed for the plumbing.

Two ways to shard, both taken from how the reference's kernel is already
organised inside one GPU (``kernels/int8_decode_attention.cu:86-104``: every
(b,h) row is independent; ``:389-426``: split partials merge by log-sum-exp):

* by (batch, head): rank r owns a contiguous range of the flattened B*H rows
  and runs the ordinary forward on it -- no communication at all;
* by KV sequence: rank r holds positions [r*S/n, (r+1)*S/n) of every (b,h),
  computes ONE unnormalised (m, l, acc) row per (b,h) for its chunk
  (``int8_decode_attention_partial``), the rows are all-gathered (B*H*(D+4)
  floats per rank, tens of KB) and every rank merges them
  (``int8_decode_combine_partials``).

The partial/combine callables default to the CUDA ops; the CPU tests inject
numpy stand-ins to exercise the exchange logic over gloo.
"""
import torch
import torch.distributed as dist


def bh_shard_range(bh, world, rank):
    """Contiguous range of flattened (b,h) rows owned by ``rank``: sizes differ by at most one."""
    base, rem = divmod(bh, world)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def seq_shard_range(seq, world, rank, align=128):
    """Contiguous KV positions owned by ``rank``; chunk starts are multiples of ``align``
    (the kernel's stage size) so every rank but the last scans whole stages."""
    chunk = -(-seq // world)
    chunk = -(-chunk // align) * align
    start = min(seq, rank * chunk)
    return start, min(seq, start + chunk)


def _default_ops():
    from . import int8_ext
    return int8_ext.int8_decode_attention_partial, int8_ext.int8_decode_combine_partials


def decode_attention_bh_sharded(Q, K, V, sQ, sK, sV, forward=None):
    """(batch, head) sharding: the tensors ARE this rank's shard; no collective."""
    if forward is None:
        from . import int8_ext
        forward = int8_ext.int8_decode_attention_forward
    return forward(Q, K, V, sQ, sK, sV)


def decode_attention_seq_sharded(Q, K_local, V_local, sQ, sK_local, sV_local, group=None,
                                 partial_fn=None, combine_fn=None):
    """KV-sequence sharding: local partial, all-gather of the rows, merge on every rank.

    ``Q`` [B,H,D] and ``sQ`` are replicated; ``K_local``/``V_local`` [B,H,S_local,D]
    and their scales are this rank's chunk (``S_local`` may be 0 on trailing ranks).
    Returns fp16 [B,H,D] on every rank.
    """
    if partial_fn is None or combine_fn is None:
        partial_fn, combine_fn = _default_ops()
    world = dist.get_world_size(group)
    B, H, D = Q.shape
    if K_local.shape[2] > 0:
        part = partial_fn(Q, K_local, V_local, sQ, sK_local, sV_local)
    else:  # empty chunk: l == 0 rows are skipped by the merge
        part = torch.zeros(B, H, D + 4, dtype=torch.float32, device=Q.device)
        part[..., 0] = float("-inf")
    # concatenation along dim 0 (the form every backend accepts), viewed as [world, B, H, D+4]
    parts = torch.empty(world * B, H, D + 4, dtype=torch.float32, device=Q.device)
    dist.all_gather_into_tensor(parts, part.contiguous(), group=group)
    return combine_fn(parts.view(world, B, H, D + 4))
