"""Oracle: symmetric INT8 quantisers (numpy, fp32 arithmetic, bit-exact target).

Test infrastructure only -- see ``oracle/__init__.py``.

All arithmetic is done in IEEE fp32 exactly as the reference's torch code
does it on a float tensor: a true fp32 division by the scale and
round-half-to-even (``np.rint``), then a clamp to [-128, 127].
"""
import numpy as np

_F127 = np.float32(127.0)
_EPS = np.float32(1e-8)


def _as_f32(x):
    """``t.float()`` of the reference: fp16/fp32 input widened to fp32."""
    return np.ascontiguousarray(x).astype(np.float32, copy=False)


def quantize_per_token(x):
    """Per-token (last-dim row) symmetric INT8 quantisation.

    Follows ``tests/test_int8.py:47-63`` (``quantize_per_token``) which is
    identical to ``validation/validate_int8.py:63-66`` (``q_per_token``):
    ``absmax = |x|.amax(-1).clamp(min=1e-8)``; ``scale = absmax / 127``;
    ``q = clamp(round_half_even(x / scale), -128, 127)``.

    Returns ``(q int8 [..., D], scales fp32 [...])``.
    """
    xf = _as_f32(x)
    absmax = np.maximum(np.abs(xf).max(axis=-1, keepdims=True), _EPS).astype(np.float32)
    scale = (absmax / _F127).astype(np.float32)
    q = np.rint((xf / scale).astype(np.float32))
    q = np.clip(q, -128.0, 127.0).astype(np.int8)
    return q, scale[..., 0].copy()


def quantize_per_tensor(x):
    """Per-tensor symmetric quantisation.

    Follows ``validation/validate_int8.py:58-60`` (``q_per_tensor``; the
    variant in ``tests/test_int8.py:39-44`` omits the 1e-8 clamp).
    Returns ``(q int8, scale fp32 scalar)``.
    """
    xf = _as_f32(x)
    s = (np.maximum(np.abs(xf).max(), _EPS) / _F127).astype(np.float32)
    q = np.clip(np.rint((xf / s).astype(np.float32)), -128.0, 127.0).astype(np.int8)
    return q, np.float32(s)


def quantize_per_channel_w(w):
    """Per-output-channel weight quantisation of ``w [in, out]``.

    Follows ``validation/validate_int8.py:75-81`` (``q_per_channel_w``): the
    scale reduces over the input dim and is indexed by output column.
    Returns ``(q int8 [in, out], scale fp32 [out])``.
    """
    wf = _as_f32(w)
    s = (np.maximum(np.abs(wf).max(axis=0), _EPS) / _F127).astype(np.float32)
    q = np.clip(np.rint((wf / s[None, :]).astype(np.float32)), -128.0, 127.0).astype(np.int8)
    return np.ascontiguousarray(q), s


def requant_rows_kernel_semantics(h_f16, row_absmax):
    """Row requantiser as the reference's MLP kernel does it.

    Follows ``kernels/int8_mlp.cu:768-795`` (``quantize_rows_kernel``) and
    ``kernels/int8_common.cuh:17-19`` (``f32_to_i8``): ``amax =
    max(absmax, 1e-8)``; ``inv = 127 / amax`` (fp32); the fp16-rounded value
    is widened to fp32 and MULTIPLIED by ``inv`` (no division), clamped to
    [-128, 127] and rounded half-to-even; the published scale is ``amax/127``.

    ``h_f16``: fp16 [M, N]; ``row_absmax``: fp32 [M] (taken on the fp32 value
    before the fp16 rounding, ``kernels/int8_mlp.cu:441-448``).
    """
    amax = np.maximum(row_absmax.astype(np.float32), _EPS)
    inv = (_F127 / amax).astype(np.float32)
    v = (h_f16.astype(np.float32) * inv[:, None]).astype(np.float32)
    q = np.rint(np.clip(v, -128.0, 127.0)).astype(np.int8)
    return q, (amax / _F127).astype(np.float32)


def layernorm_quantize(x_f16, eps=1e-5):
    """LayerNorm without affine parameters over the last dimension, stored as fp16, then
    :func:`quantize_per_token` of that fp16 tensor -- the two steps the reference's block runs
    as eager torch code before its INT8 MLP (``bench/bench_block.py:93-94`` then ``:59-63``).
    Mean and biased variance in float64, so this is the exactly rounded value the fp32
    implementations (torch's and the CUDA kernel's) approximate to within an fp16 ulp.
    Returns ``(y_f16, q_int8, scales_f32)``."""
    x = np.asarray(x_f16, dtype=np.float16).astype(np.float64)
    mean = x.mean(axis=-1, keepdims=True)
    var = ((x - mean) ** 2).mean(axis=-1, keepdims=True)
    y = ((x - mean) / np.sqrt(var + eps)).astype(np.float32).astype(np.float16)
    q, s = quantize_per_token(y)
    return y, q, s
