"""Oracle: INT8-KV decode attention (seq_q == 1) in numpy.

Test infrastructure only -- see ``oracle/__init__.py``.

The tolerance target is "the reference dequant computation": dequantise the
int8 operands with their per-token scales and run a plain softmax attention
in floating point (``validation/check_decode.py:65-68``).  The split-KV
partial / log-sum-exp combine algebra of the reference kernels
(``kernels/int8_decode_attention.cu:274-426``) is restated as well so the
multi-GPU sequence-sharded path can be checked on the CPU.
"""
import numpy as np


def dequantize(q_i8, scales):
    """``q.float() * scale[..., None]`` (``validation/check_decode.py:65-67``)."""
    return q_i8.astype(np.float32) * scales.astype(np.float32)[..., None]


def decode_attention(Qi, Ki, Vi, sQ, sK, sV, dtype=np.float64):
    """Reference decode attention on the dequantised values.

    ``Qi`` int8 [B,H,D]; ``Ki``,``Vi`` int8 [B,H,S,D]; ``sQ`` fp32 [B,H] (or
    flat B*H); ``sK``,``sV`` fp32 [B,H,S] (or flat).  Softmax scale is
    ``1/sqrt(D)`` (``kernels/int8_decode_attention.cu:448``; torch SDPA's
    default in ``validation/check_decode.py:68``).  Returns fp32 [B,H,D].

    ``dtype`` is the accumulation type; float64 gives the "exact" value the
    fp32 torch reference approximates.
    """
    B, H, D = Qi.shape
    S = Ki.shape[2]
    sQ = np.asarray(sQ, dtype=np.float32).reshape(B, H)
    sK = np.asarray(sK, dtype=np.float32).reshape(B, H, S)
    sV = np.asarray(sV, dtype=np.float32).reshape(B, H, S)
    qd = dequantize(Qi, sQ).astype(dtype)            # [B,H,D]
    out = np.empty((B, H, D), dtype=np.float32)
    inv_sqrt_d = dtype(1.0) / np.sqrt(dtype(D))
    for b in range(B):
        for h in range(H):
            kd = dequantize(Ki[b, h], sK[b, h]).astype(dtype)   # [S,D]
            vd = dequantize(Vi[b, h], sV[b, h]).astype(dtype)
            s = (kd @ qd[b, h]) * inv_sqrt_d                     # [S]
            s = s - s.max()
            p = np.exp(s)
            out[b, h] = ((p @ vd) / p.sum()).astype(np.float32)
    return out


def decode_partial(Qi, Ki, Vi, sQ, sK, sV, j0, j1):
    """Unnormalised online-softmax partial over KV positions ``[j0, j1)``.

    Restates what one split of ``int8_decode_partial_batch_kernel``
    (``kernels/int8_decode_attention.cu:274-386``) leaves in scratch:
    ``m = max_j score_j``, ``l = sum_j e^{score_j - m}``, ``acc[d] = sum_j
    e^{score_j - m} * sV_j * v_j[d]`` with ``score_j = (q.k_j) * sQ * sK_j /
    sqrt(D)`` in natural-log units.  An empty range gives ``(-inf, 0, 0)``.

    Shapes as :func:`decode_attention`.  Returns ``(m [B,H], l [B,H],
    acc [B,H,D])`` in float64.
    """
    B, H, D = Qi.shape
    S = Ki.shape[2]
    sQ = np.asarray(sQ, dtype=np.float32).reshape(B, H).astype(np.float64)
    sK = np.asarray(sK, dtype=np.float32).reshape(B, H, S).astype(np.float64)
    sV = np.asarray(sV, dtype=np.float32).reshape(B, H, S).astype(np.float64)
    m = np.full((B, H), -np.inf)
    l = np.zeros((B, H))
    acc = np.zeros((B, H, D))
    j1 = min(j1, S)
    if j1 <= j0:
        return m, l, acc
    inv_sqrt_d = 1.0 / np.sqrt(float(D))
    for b in range(B):
        for h in range(H):
            dots = Ki[b, h, j0:j1].astype(np.int64) @ Qi[b, h].astype(np.int64)
            score = dots.astype(np.float64) * sQ[b, h] * sK[b, h, j0:j1] * inv_sqrt_d
            mm = score.max()
            p = np.exp(score - mm)
            m[b, h] = mm
            l[b, h] = p.sum()
            acc[b, h] = (p * sV[b, h, j0:j1]) @ Vi[b, h, j0:j1].astype(np.float64)
    return m, l, acc


def combine_partials(ms, ls, accs):
    """Log-sum-exp merge of split partials.

    Restates ``int8_decode_combine_kernel``
    (``kernels/int8_decode_attention.cu:389-426``): ``gm = max_s m_s``;
    splits with ``l_s <= 0`` are skipped (``:414``); ``out = (sum_s acc_s
    e^{m_s-gm}) / (sum_s l_s e^{m_s-gm})``.

    ``ms``,``ls``: [nsplit, B, H]; ``accs``: [nsplit, B, H, D].  Returns the
    merged unnormalised ``(m, l, acc)`` and the normalised fp32 output.
    """
    ms = np.asarray(ms, dtype=np.float64)
    ls = np.asarray(ls, dtype=np.float64)
    accs = np.asarray(accs, dtype=np.float64)
    gm = ms.max(axis=0)
    with np.errstate(invalid="ignore"):
        w = np.where(ls > 0, np.exp(ms - gm[None]), 0.0)
    L = (ls * w).sum(axis=0)
    ACC = (accs * w[..., None]).sum(axis=0)
    out = (ACC / L[..., None]).astype(np.float32)
    return gm, L, ACC, out


def prefill_attention(Qi, Ki, Vi, sQ, sK, sV, dtype=np.float64):
    """Non-causal attention on the dequantised values, seq_q == seq_kv.

    Restates the reference check of its prefill kernel (``tests/test_int8.py:99-111``:
    dequantise per token, then ``common/baseline.py:7-22`` ``softmax(Q K^T / sqrt(D)) V``),
    in float64 instead of fp16.  ``Qi``,``Ki``,``Vi`` int8 [B,H,S,D]; scales fp32 [B,H,S]
    (or flat).  Returns fp32 [B,H,S,D].
    """
    B, H, S, D = Qi.shape
    sQ = np.asarray(sQ, dtype=np.float32).reshape(B, H, S)
    sK = np.asarray(sK, dtype=np.float32).reshape(B, H, S)
    sV = np.asarray(sV, dtype=np.float32).reshape(B, H, S)
    out = np.empty((B, H, S, D), dtype=np.float32)
    inv = dtype(1.0) / np.sqrt(dtype(D))
    for b in range(B):
        for h in range(H):
            q = dequantize(Qi[b, h], sQ[b, h]).astype(dtype)
            k = dequantize(Ki[b, h], sK[b, h]).astype(dtype)
            v = dequantize(Vi[b, h], sV[b, h]).astype(dtype)
            s = (q @ k.T) * inv
            s -= s.max(axis=1, keepdims=True)
            p = np.exp(s)
            out[b, h] = ((p @ v) / p.sum(axis=1, keepdims=True)).astype(np.float32)
    return out
