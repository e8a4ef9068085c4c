"""Oracle: fused INT8 MLP (int8 GEMM -> dequant -> [+bias] -> GELU(tanh) ->
per-token requant -> int8 GEMM -> requant) in numpy.

Test infrastructure only -- see ``oracle/__init__.py``.

Two restatements:

* :func:`sim_mlp` -- the reference's torch *simulation* on dequantised
  operands (``validation/validate_int8.py:174-225``), the tolerance target the
  reference itself validates its kernel against (max-abs 0.05,
  ``validation/validate_int8.py:54,511-514``).
* :func:`kernel_mlp` -- the arithmetic of the reference CUDA pipeline
  (``kernels/int8_mlp.cu:999-1191``) stage by stage, with exact int32
  accumulation, its epilogue order and its requantiser.  There is no torch
  oracle for this level; it is used to report int8-code mismatch rates.
"""
import numpy as np

from .quant import (quantize_per_token, quantize_per_tensor,
                    quantize_per_channel_w, requant_rows_kernel_semantics)

_KC = np.float32(0.7978845608028654)
_KA = np.float32(0.044715)


def gelu_tanh(x):
    """``0.5*x*(1+tanh(kC*(x+kA*x^3)))`` in fp32 (``kernels/int8_common.cuh:9-13``;
    ``F.gelu(approximate='tanh')`` in ``validation/validate_int8.py:208``)."""
    x = x.astype(np.float32)
    inner = (_KC * (x + _KA * x * x * x)).astype(np.float32)
    return (np.float32(0.5) * x * (np.float32(1.0) + np.tanh(inner).astype(np.float32))).astype(np.float32)


def mlp_use_wmma(T, d_model, d_ff):
    """Shape gate of the dynamic per-token/per-channel path
    (``kernels/int8_mlp.cu:1023-1026``; ``validation/validate_int8.py:84-89``)."""
    return T % 128 == 0 and d_model % 128 == 0 and d_ff % 128 == 0


def sim_mlp(x, W1, W2, b1=None):
    """Dequantised-operand simulation of the MLP.

    Follows ``validation/validate_int8.py:174-225`` (``sim_mlp``): on tile
    shapes per-token activation x per-channel weight, otherwise per-tensor;
    the hidden is always requantised per token; the output is requantised
    per token on tile shapes and per tensor otherwise.  ``b1`` (not in
    ``sim_mlp``) is added before GELU as ``validation/validate_int8.py:330-375``
    does for the real-model path.

    ``x`` [T, d_model] (or [B,S,d_model]), ``W1`` [d_model,d_ff], ``W2``
    [d_ff,d_model], floating point.  Returns a dict of fp32 stages.
    """
    d_model, d_ff = W1.shape
    x2 = np.asarray(x, dtype=np.float32).reshape(-1, d_model)
    T = x2.shape[0]
    tile = mlp_use_wmma(T, d_model, d_ff)
    if tile:
        xi, sx = quantize_per_token(x2)
        xd = xi.astype(np.float32) * sx[:, None]
        w1i, s1 = quantize_per_channel_w(W1)
        w2i, s2 = quantize_per_channel_w(W2)
        w1 = w1i.astype(np.float32) * s1[None, :]
        w2 = w2i.astype(np.float32) * s2[None, :]
    else:
        xi, sx = quantize_per_tensor(x2)
        xd = xi.astype(np.float32) * sx
        w1i, s1 = quantize_per_tensor(W1)
        w2i, s2 = quantize_per_tensor(W2)
        w1 = w1i.astype(np.float32) * s1
        w2 = w2i.astype(np.float32) * s2
    h_pre = (xd @ w1).astype(np.float32)
    if b1 is not None:
        h_pre = h_pre + np.asarray(b1, dtype=np.float32)[None, :]
    h = gelu_tanh(h_pre)
    hi, sh = quantize_per_token(h)
    hq = hi.astype(np.float32) * sh[:, None]
    out = (hq @ w2).astype(np.float32)
    if tile:
        oi, so = quantize_per_token(out)
        outq = oi.astype(np.float32) * so[:, None]
    else:
        oi, so = quantize_per_tensor(out)
        outq = oi.astype(np.float32) * so
    return {"x_dequant": xd, "h_pre_gelu": h_pre, "h_gelu": h,
            "h_requant": hq, "out_fp": out, "out": outq}


def _igemm(a_i8, b_i8):
    """Exact integer GEMM (float64 BLAS is exact here: |sum| < 2^53)."""
    return np.rint(a_i8.astype(np.float64) @ b_i8.astype(np.float64)).astype(np.int64)


def kernel_mlp(x_i8, W1_i8, W2_i8, sx, sw1, sw2, b1=None, per_token_out=True):
    """Stage-by-stage arithmetic of the reference's dynamic MLP pipeline.

    Follows ``kernels/int8_mlp.cu``: GEMM epilogue ``v = (float)acc * sa * sb
    [+ bias]`` then GELU (``:437-440``), fp16 store and row absmax of the fp32
    value (``:441-448``), ``quantize_rows_kernel`` (``:768-795``) for the hidden
    and (``per_token_out``) the output, ``quantize_tensor_kernel``
    (``:799-825``) for the legacy per-tensor output.

    ``x_i8`` [T,d_model]; ``W1_i8`` [d_model,d_ff]; ``W2_i8`` [d_ff,d_model];
    ``sx`` scalar or [T]; ``sw1`` scalar or [d_ff]; ``sw2`` scalar or
    [d_model]; ``b1`` None or [d_ff].

    Returns dict with ``hidden_f16``, ``hidden_i8``, ``hidden_scale``,
    ``out_f16``, ``out_i8``, ``out_scale`` ([T] or scalar).
    """
    T, d_model = x_i8.shape
    d_ff = W1_i8.shape[1]
    sx = np.broadcast_to(np.asarray(sx, dtype=np.float32).reshape(-1), (T,))
    sw1 = np.broadcast_to(np.asarray(sw1, dtype=np.float32).reshape(-1), (d_ff,))
    sw2 = np.broadcast_to(np.asarray(sw2, dtype=np.float32).reshape(-1), (d_model,))
    acc1 = _igemm(x_i8, W1_i8).astype(np.float32)
    v = ((acc1 * sx[:, None]).astype(np.float32) * sw1[None, :]).astype(np.float32)
    if b1 is not None:
        v = (v + np.asarray(b1, dtype=np.float32)[None, :]).astype(np.float32)
    v = gelu_tanh(v)
    h_absmax = np.abs(v).max(axis=1).astype(np.float32)
    h16 = v.astype(np.float16)
    hi, sh = requant_rows_kernel_semantics(h16, h_absmax)
    acc2 = _igemm(hi, W2_i8).astype(np.float32)
    o = ((acc2 * sh[:, None]).astype(np.float32) * sw2[None, :]).astype(np.float32)
    o16 = o.astype(np.float16)
    if per_token_out:
        o_absmax = np.abs(o).max(axis=1).astype(np.float32)
        oi, so = requant_rows_kernel_semantics(o16, o_absmax)
    else:
        g = np.full((T,), np.abs(o).max(), dtype=np.float32)
        oi, so_rows = requant_rows_kernel_semantics(o16, g)
        so = np.float32(so_rows[0])
    return {"hidden_f16": h16, "hidden_i8": hi, "hidden_scale": sh,
            "out_f16": o16, "out_i8": oi, "out_scale": so}


def static_mlp(x_i8, W1_i8, W2_i8, sx, sw1, sw2):
    """The reference's static-scale pipeline, the one it runs on shapes off its 128-tiles.

    Follows ``kernels/int8_mlp.cu:830-844`` (``compute_static_scales_kernel``: hidden scale
    ``sx*sw1*d_model``, output scale ``hidden_scale*sw2*d_ff``, and their reciprocals),
    ``:905-909`` / ``:946-949`` (epilogue ``v = acc * (sa*sb)``, GELU on GEMM1, then
    ``f32_to_i8(v, inv_scale)`` = ``rne(clamp(v * inv))``, ``kernels/int8_common.cuh:17-19``)
    and ``:1194-1225`` (the two launches).  Per-tensor scalar scales only.  Accumulation is
    exact here; the reference's scalar kernel accumulates in fp32, which is exact too while
    ``K * 127^2 < 2^24``.

    Returns dict with ``hidden_i8``, ``out_i8``, ``hidden_scale``, ``out_scale`` (fp32 scalars).
    """
    d_model, d_ff = W1_i8.shape
    sx, sw1, sw2 = np.float32(sx), np.float32(sw1), np.float32(sw2)
    sh = np.float32(np.float32(sx * sw1) * np.float32(d_model))
    so = np.float32(np.float32(sh * sw2) * np.float32(d_ff))
    inv_h = np.float32(np.float32(1.0) / sh)
    inv_o = np.float32(np.float32(1.0) / so)
    acc1 = _igemm(x_i8, W1_i8).astype(np.float32)
    v = gelu_tanh((acc1 * np.float32(sx * sw1)).astype(np.float32))
    hi = np.rint(np.clip((v * inv_h).astype(np.float32), -128.0, 127.0)).astype(np.int8)
    acc2 = _igemm(hi, W2_i8).astype(np.float32)
    o = (acc2 * np.float32(sh * sw2)).astype(np.float32)
    oi = np.rint(np.clip((o * inv_o).astype(np.float32), -128.0, 127.0)).astype(np.int8)
    return {"hidden_i8": hi, "out_i8": oi, "hidden_scale": sh, "out_scale": so}
