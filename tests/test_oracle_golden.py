"""The numpy oracle against the golden vectors produced by the reference's own
Python functions (tests/golden/make_golden.py).  CPU only."""
import os

import numpy as np
import pytest

from oracle import quant, decode, mlp

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _load(name):
    return np.load(os.path.join(GOLD, name))


def _names(npz, suffix="__x"):
    return sorted(k[: -len(suffix)] for k in npz.files if k.endswith(suffix))


def test_quantize_per_token_bit_exact():
    g = _load("quantize_per_token.npz")
    names = _names(g)
    assert len(names) >= 10
    for n in names:
        q, s = quant.quantize_per_token(g[n + "__x"])
        assert np.array_equal(q, g[n + "__q"]), n
        # scales must be bit-identical, not merely close
        assert np.array_equal(s.view(np.uint32), g[n + "__s"].view(np.uint32)), n


def test_weight_and_tensor_quantisers_bit_exact():
    g = _load("quantize_weights.npz")
    q, s = quant.quantize_per_channel_w(g["w__x"])
    assert np.array_equal(q, g["w__q"])
    assert np.array_equal(s.view(np.uint32), g["w__s"].view(np.uint32))
    q, s = quant.quantize_per_tensor(g["t__x"])
    assert np.array_equal(q, g["t__q"])
    assert np.float32(s) == np.float32(g["t__s"])


def _cos(a, b):
    a = a.astype(np.float64).ravel()
    b = b.astype(np.float64).ravel()
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b)))


def test_decode_attention_matches_reference_torch_path():
    g = _load("decode_attention.npz")
    keys = _names(g, "__ref")
    assert len(keys) == 13
    for k in keys:
        out = decode.decode_attention(g[k + "__Qi"], g[k + "__Ki"], g[k + "__Vi"],
                                      g[k + "__sQ"], g[k + "__sK"], g[k + "__sV"])
        ref = g[k + "__ref"]
        # fp32 torch SDPA vs float64 numpy on identical dequantised operands
        assert np.abs(out - ref).max() < 2e-5, k
        assert _cos(out, ref) > 0.999999, k


@pytest.mark.parametrize("nsplit", [1, 2, 3, 8])
def test_split_partials_combine_to_full_attention(nsplit):
    g = _load("decode_attention.npz")
    for k in ("B2_H2_D64_S33", "B1_H3_D128_S1000", "B1_H1_D64_S1"):
        args = [g[k + "__" + n] for n in ("Qi", "Ki", "Vi", "sQ", "sK", "sV")]
        S = args[1].shape[2]
        chunk = -(-S // nsplit)
        parts = [decode.decode_partial(*args, j0=i * chunk, j1=(i + 1) * chunk)
                 for i in range(nsplit)]      # trailing chunks may be empty
        ms, ls, accs = (np.stack(x) for x in zip(*parts))
        _, _, _, out = decode.combine_partials(ms, ls, accs)
        full = decode.decode_attention(*args)
        assert np.abs(out - full).max() < 1e-6, (k, nsplit)


def test_sim_mlp_matches_reference_simulation():
    g = _load("mlp_sim.npz")
    for tag in ("tile", "small"):
        st = mlp.sim_mlp(g[tag + "__x"], g[tag + "__W1"], g[tag + "__W2"])
        for stage in ("h_pre_gelu", "h_gelu", "h_requant", "out"):
            ref = g[f"{tag}__{stage}"]
            got = st[stage]
            scale = max(1e-6, float(np.abs(ref).max()))
            # fp32 BLAS summation order differs between numpy and torch; an
            # int8 code may flip by one step on a rounding tie after requant
            tol = 2e-5 * scale if stage in ("h_pre_gelu", "h_gelu") else 1.01 * scale / 127
            assert np.abs(got - ref).max() <= tol, (tag, stage)
            assert _cos(got, ref) > 0.9999, (tag, stage)


def test_kernel_mlp_close_to_simulation():
    g = _load("mlp_sim.npz")
    x, W1, W2 = g["tile__x"], g["tile__W1"], g["tile__W2"]
    T, dm = x.shape[-2], x.shape[-1]
    xi, sx = quant.quantize_per_token(x.reshape(T, dm))
    w1i, s1 = quant.quantize_per_channel_w(W1)
    w2i, s2 = quant.quantize_per_channel_w(W2)
    r = mlp.kernel_mlp(xi, w1i, w2i, sx, s1, s2)
    out = r["out_i8"].astype(np.float32) * r["out_scale"][:, None]
    ref = g["tile__out"]
    # the reference requires its kernel within 0.05 of the simulation
    assert np.abs(out - ref).max() < 0.05
    assert _cos(out, ref) > 0.9999


def test_layernorm_quantize_against_torch_cpu():
    """The float64 LayerNorm of the oracle and torch's fp32 one can differ by one fp16 ulp on a
    few elements (and then by one code): require near-identity, not bit-identity."""
    g = _load("layernorm_quantize.npz")
    names = _names(g)
    assert len(names) == 4
    for n in names:
        y, q, s = quant.layernorm_quantize(g[n + "__x"])
        ulp_off = np.mean(y.view(np.uint16) != g[n + "__y"].view(np.uint16))
        assert ulp_off < 2e-3, (n, ulp_off)
        dq = np.abs(q.astype(np.int32) - g[n + "__q"].astype(np.int32))
        assert dq.max() <= 1 and np.mean(dq != 0) < 2e-3, (n, dq.max(), np.mean(dq != 0))
        assert np.allclose(s, g[n + "__s"], rtol=1e-3, atol=0), n


VALIDATION_SETS = ["normal", "outlier", "boundary", "stress", "short_seq", "long_seq", "zeros", "constant"]


@pytest.mark.parametrize("name", VALIDATION_SETS)
def test_oracle_reproduces_the_reference_simulations_on_its_validation_sets(name):
    """Slices of the eight datasets of validation/generate_test_data.py:174-338 with the outputs
    of the reference's own int8 simulations on them (sim_attention / sim_mlp,
    validation/validate_int8.py:144-225): the numpy restatements must give the same numbers,
    up to fp32-vs-float64 accumulation and a one-step flip of an int8 code on a rounding tie."""
    g = _load("validation_sets.npz")
    Q, K, V = (g[f"{name}__attn_{k}"] for k in ("Q", "K", "V"))
    (qi, sq), (ki, sk), (vi, sv) = (quant.quantize_per_token(t) for t in (Q, K, V))
    got = decode.prefill_attention(qi, ki, vi, sq, sk, sv)
    sim = g[f"{name}__attn_sim"]
    assert np.abs(got - sim).max() <= 1e-4 * max(1.0, float(np.abs(sim).max())), name
    x, W1, W2 = (g[f"{name}__mlp_{k}"] for k in ("x", "W1", "W2"))
    got = mlp.sim_mlp(x, W1, W2)["out"].reshape(x.shape)
    sim = g[f"{name}__mlp_sim"]
    assert np.abs(got - sim).max() <= 1.01 * max(1e-6, float(np.abs(sim).max())) / 127, name
    assert _cos(got, sim) > 0.99999 or float(np.abs(sim).max()) == 0.0, name
