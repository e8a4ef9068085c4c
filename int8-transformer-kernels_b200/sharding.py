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


class SeqShardedDecoder:
    """KV-sequence-sharded decode with the exchange fused into the merge kernel.

    Set up once per (B, H, D) and process group; every call runs, on each rank,
    the streaming kernel over the local KV chunk and then ONE kernel that merges
    the local partials, stores the merged rows into every rank's gather buffer
    through peer-mapped pointers (NVLink), signals, waits (bounded) for the other
    ranks and writes the fp16 result (``i8tk_decode_attention_seq_sharded``).
    The gather buffers and flags live in torch symmetric memory; no NCCL call is
    made on the data path.  All ranks must call in the same order.
    """

    def __init__(self, B, H, D, device, group=None, max_local_positions=None):
        import torch.distributed._symmetric_memory as symm_mem
        from . import cabi
        self._cabi = cabi
        self._lib = cabi.load()
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        self.B, self.H, self.D = B, H, D
        self.device = torch.device(device)
        BH = B * H
        ctas = self._lib.i8tk_decode_exchange_ctas(BH)
        self._parts = symm_mem.empty(2 * self.world * BH * (D + 4), dtype=torch.float32, device=self.device)
        self._flags = symm_mem.empty(self.world * ctas, dtype=torch.int32, device=self.device)
        self._parts.zero_()
        self._flags.zero_()
        self._parts_hdl = symm_mem.rendezvous(self._parts, self.group)
        self._flags_hdl = symm_mem.rendezvous(self._flags, self.group)
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)              # every rank's flags are zero before anyone signals
        self._epoch = 0
        self._ws = None
        self._ws_bytes = 0

    def _workspace(self, BH, S_local):
        need = max(256, self._lib.i8tk_decode_workspace_bytes(BH, S_local, self.D) if S_local > 0 else 256)
        if need > self._ws_bytes:
            # zeroed: the status block at its start is read back by check()
            self._ws = torch.zeros(need, dtype=torch.uint8, device=self.device)
            self._ws_bytes = need
        return self._ws

    def _checked(self, t, name, dtype):
        if t.dtype != dtype or t.device != self.device or not t.is_contiguous():
            raise ValueError("%s must be a contiguous %s tensor on %s (a slice of a larger cache has to be "
                             "copied first: the kernel reads S_local*D contiguous bytes per (b,h) row)"
                             % (name, dtype, self.device))
        return t

    def __call__(self, Q, K_local, V_local, sQ, sK_local, sV_local):
        B, H, D = Q.shape
        assert (B, H, D) == (self.B, self.H, self.D), "shape differs from the one set up"
        S_local = int(K_local.shape[2])
        BH = B * H
        self._checked(Q, "Q", torch.int8)
        self._checked(sQ, "sQ", torch.float32)
        if S_local:
            for t, nm, dt in ((K_local, "K_local", torch.int8), (V_local, "V_local", torch.int8),
                              (sK_local, "sK_local", torch.float32), (sV_local, "sV_local", torch.float32)):
                self._checked(t, nm, dt)
            if tuple(K_local.shape) != (B, H, S_local, D) or V_local.shape != K_local.shape:
                raise ValueError("K_local / V_local must be [B, H, S_local, D]")
            if sK_local.numel() != BH * S_local or sV_local.numel() != BH * S_local or sQ.numel() != BH:
                raise ValueError("scales must have one value per row")
        ws = self._workspace(BH, S_local)
        out = torch.empty(B, H, D, dtype=torch.float16, device=self.device)
        self._epoch += 1
        stream = torch.cuda.current_stream(self.device).cuda_stream
        rc = self._lib.i8tk_decode_attention_seq_sharded(
            Q.data_ptr(), K_local.data_ptr() if S_local else None, V_local.data_ptr() if S_local else None,
            out.data_ptr(), sQ.data_ptr(), sK_local.data_ptr() if S_local else None,
            sV_local.data_ptr() if S_local else None, BH, S_local, D, ws.data_ptr(), self._ws_bytes,
            self._parts_hdl.buffer_ptrs_dev, self._flags_hdl.buffer_ptrs_dev, self.rank, self.world,
            self._epoch, stream)
        self._cabi.check(rc, "i8tk_decode_attention_seq_sharded")
        return out

    def check(self):
        """Synchronises and raises if a bounded device-side wait gave up (a rank never arrived)."""
        stream = torch.cuda.current_stream(self.device).cuda_stream
        if self._ws is not None:
            rc = self._lib.i8tk_check_status_word(self._ws.data_ptr(), stream)
            if rc != self._cabi.OK:
                self._ws[:8].zero_()          # the record has been delivered
            self._cabi.check(rc, "seq-sharded decode")
