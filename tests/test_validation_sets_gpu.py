"""The reference's own validation inputs through the CUDA path: slices of its eight seeded
datasets (validation/generate_test_data.py:174-338 -- normal, outlier, boundary, stress,
short_seq, long_seq, zeros, constant) judged by its own gates with its own per-dataset
thresholds (validation/validate_int8.py:264-327, thresholds generate_test_data.py:169-171).

  gate 1  cosine / top-10 overlap / outlier ratio / no NaN against the fp reference
  gate 4  edge datasets: no NaN, zero in -> zero out, cosine floor
  and the check the reference runs before its stage traces: the kernel within 0.05 of its int8
  simulation (validate_int8.py:54,511-514) -- scaled by the output range where outputs reach
  tens (stress, outlier), since 0.05 absolute is then below fp16 resolution.

The attention kernel is expected to miss gate 1 on outlier / boundary / stress exactly as the
reference's does (generate_test_data.py marks them xfail: per-token scales cannot represent
those inputs); there the test requires agreement with the int8 simulation instead.
The fixture and the script that made it from the reference live in tests/golden/.
"""
import json

import numpy as np
import pytest
import torch

from oracle import quant, mlp as omlp
from helpers import ext, gold, cosine, gate1, gate4

pytestmark = pytest.mark.gpu

NAMES = ["normal", "outlier", "boundary", "stress", "short_seq", "long_seq", "zeros", "constant"]


def _meta(g):
    return json.loads(bytes(g["meta_json"]).decode())


def _cuda(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _sim_gap_limit(sim):
    return 0.05 * max(1.0, float(np.abs(sim).max()) / 4.0)


@pytest.mark.parametrize("name", NAMES)
def test_attention_on_validation_set(name):
    g = gold("validation_sets.npz")
    meta = _meta(g)[name]
    thr = meta["thresholds"]
    Q, K, V = (g[f"{name}__attn_{k}"] for k in ("Q", "K", "V"))
    (qi, sq), (ki, sk), (vi, sv) = (quant.quantize_per_token(t) for t in (Q, K, V))
    act = ext().int8_attention_forward(_cuda(qi), _cuda(ki), _cuda(vi), _cuda(sq), _cuda(sk), _cuda(sv))
    act = act.float().cpu().numpy()
    ref = g[f"{name}__attn_ref"].astype(np.float32)
    sim = g[f"{name}__attn_sim"]
    is_zero = bool(thr.get("zero_output"))
    res, fails = gate1(ref, act, thr, is_zero)
    gap = float(np.abs(act - sim).max())
    print(f"{name}: attention gate1 {res} sim gap {gap:.4f}")
    assert res["nan_inf"]
    if "attention" in meta["xfail"]:
        # quantisation-limited inputs: the int8 simulation misses gate 1 too; what the kernel
        # owes is the simulation's answer.  Near-tie argmax flips move whole rows, so compare
        # as the reference does for these sets: by cosine, and row by row for most rows.
        assert cosine(act, sim) > 0.995, cosine(act, sim)
        row_err = np.abs(act - sim).reshape(-1, act.shape[-1]).max(axis=1)
        assert float((row_err > _sim_gap_limit(sim)).mean()) < 0.10
    else:
        assert not fails, fails
        assert gap <= _sim_gap_limit(sim), gap
    if meta["edge"]:
        assert not gate4(ref, act, thr)


@pytest.mark.parametrize("name", NAMES)
def test_mlp_on_validation_set(name):
    g = gold("validation_sets.npz")
    meta = _meta(g)[name]
    thr = meta["thresholds"]
    x, W1, W2 = (g[f"{name}__mlp_{k}"] for k in ("x", "W1", "W2"))
    B, S, dm = x.shape
    T, dff = B * S, W1.shape[1]
    e = ext()
    if omlp.mlp_use_wmma(T, dm, dff):
        # per-token activation + per-channel weight overload (validate_int8.py:240-250)
        xi, sx = quant.quantize_per_token(x.reshape(T, dm))
        w1i, s1 = quant.quantize_per_channel_w(W1)
        w2i, s2 = quant.quantize_per_channel_w(W2)
        o8, osc = e.int8_mlp_forward(_cuda(xi.reshape(B, S, dm)), _cuda(w1i), _cuda(w2i), _cuda(sx), _cuda(s1), _cuda(s2))
        act = o8.float().cpu().numpy() * osc.cpu().numpy().reshape(B, S, 1)
    else:
        # per-tensor scales, scalar overload (validate_int8.py:251-258)
        xi, sx = quant.quantize_per_tensor(x)
        w1i, s1 = quant.quantize_per_tensor(W1)
        w2i, s2 = quant.quantize_per_tensor(W2)
        o8, osc = e.int8_mlp_forward(_cuda(xi), _cuda(w1i), _cuda(w2i), float(sx), float(s1), float(s2))
        act = o8.float().cpu().numpy() * osc
    ref = g[f"{name}__mlp_ref"].astype(np.float32)
    sim = g[f"{name}__mlp_sim"]
    is_zero = bool(thr.get("zero_output"))
    res, fails = gate1(ref, act, thr, is_zero)
    gap = float(np.abs(act - sim).max())
    print(f"{name}: mlp gate1 {res} sim gap {gap:.4f}")
    assert not fails, fails
    if not is_zero:
        assert gap <= _sim_gap_limit(sim), gap
    if meta["edge"]:
        assert not gate4(ref, act, thr)
