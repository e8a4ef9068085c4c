"""Generate the golden vectors that pin the oracle to the reference.

Run once, in a checkout that has the reference project next to it:

    python tests/golden/make_golden.py /path/to/int8-transformer-kernels

It imports the reference's own Python functions (no CUDA is touched) --
``tests/test_int8.py`` (``quantize_per_token``, ``quantize_to_int8``),
``validation/validate_int8.py`` (``q_per_token``, ``q_per_channel_w``,
``q_per_tensor``, ``sim_mlp``, ``cosine``) -- and the torch computation of
``validation/check_decode.py:65-68``, runs them on seeded CPU inputs and
stores inputs + outputs as small ``.npz`` files beside this script.  The
tests only read the ``.npz`` files; the reference is not needed to run them.

``validation_sets.npz`` holds slices of the reference's eight validation datasets
(``validation/generate_test_data.py:174-338``: normal, outlier, boundary, stress, short_seq,
long_seq, zeros, constant; CPU generator, seed 42), each with the outputs of the reference's
own fp reference (``common/baseline.py``) and int8 simulation (``sim_attention`` / ``sim_mlp``,
``validation/validate_int8.py:144-225``) ON THE SLICE, and the dataset's thresholds.
"""
import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))


def _import_reference(ref_root):
    for sub in ("common", "tests", "validation"):
        sys.path.insert(0, os.path.join(ref_root, sub))
    import test_int8            # noqa: E402
    import validate_int8        # noqa: E402
    return test_int8, validate_int8


def quantiser_cases(gen):
    """Seeded inputs that exercise ties, saturation, zero rows, outliers."""
    cases = {}
    cases["normal_f32_d64"] = torch.randn(2, 3, 17, 64, generator=gen)
    cases["normal_f16_d64"] = torch.randn(2, 3, 17, 64, generator=gen).half()
    cases["normal_f32_d128"] = torch.randn(1, 2, 33, 128, generator=gen)
    cases["normal_f16_d128"] = torch.randn(1, 2, 33, 128, generator=gen).half()
    cases["mlp_x_f16_d768"] = torch.randn(1, 5, 768, generator=gen).half()
    cases["mlp_x_f32_d1024"] = torch.randn(1, 3, 1024, generator=gen)
    z = torch.randn(4, 64, generator=gen)
    z[0] = 0.0                       # all-zero row: 1e-8 clamp
    z[1] = 1.0                       # constant row: every code 127
    z[2, :] = torch.arange(64) - 31.5   # exact .5 ties after scaling
    z[3] *= 1e-12                    # row under the clamp
    cases["edge_rows_f32"] = z
    big = torch.randn(3, 128, generator=gen)
    big[0, 5] = 6.0e4                # outlier (fp16 range)
    big[1] *= 1.2e4              # large but finite in fp16
    big[2, 7] = -20.0
    cases["outlier_f16"] = big.half()
    half_ties = (torch.arange(-127, 129).float() / 2.0).reshape(2, 128)
    half_ties[0, 0] = 63.5           # absmax 63.5 -> scale 0.5 -> codes x.5 ties
    half_ties[1, 0] = 63.5
    cases["half_ties_f32"] = half_ties
    cases["odd_width_f32"] = torch.randn(7, 37, generator=gen)
    return cases


def layernorm_quantize_cases(test_int8):
    """LayerNorm as the reference's block applies it (bench/bench_block.py:93-94:
    F.layer_norm(x, (d,)) on fp16) followed by the reference's per-token quantiser
    (bench/bench_block.py:59-63 == tests/test_int8.py:47-63), on the CPU."""
    gen = torch.Generator().manual_seed(777)
    out = {}
    for name, (rows, d, scale, shift) in {"d768": (9, 768, 1.0, 0.0), "d1024_shifted": (7, 1024, 3.0, 5.0),
                                          "d64": (12, 64, 0.1, -0.3), "d4096": (3, 4096, 2.0, 0.5)}.items():
        x = (torch.randn(rows, d, generator=gen) * scale + shift).half()
        y = F.layer_norm(x, (d,))
        q, sc = test_int8.quantize_per_token(y)
        out[name + "__x"], out[name + "__y"] = x.numpy(), y.numpy()
        out[name + "__q"], out[name + "__s"] = q.numpy(), sc.numpy()
    np.savez_compressed(os.path.join(HERE, "layernorm_quantize.npz"), **out)


def validation_sets(validate_int8):
    """Slices of the reference's eight validation datasets with its own references on them.

    The generator draws everything from one seeded CPU generator except the heavy-tailed
    "stress" attention tensors, which come from torch's global generator
    (``generate_test_data.py:137-139``): that one is seeded here (42) so the file is reproducible.
    Slices: attention keeps batch 0, two heads (one for long_seq) and the first 256 positions
    (1024 for long_seq, all 4 for short_seq); the MLP keeps batch 0's first 128 tokens (all of
    short_seq's) and every 2nd input channel / every 8th hidden channel, so log-spaced channel
    magnitudes keep their spread.  The reference outputs are computed on the slices, in fp32
    on the CPU (``attention_baseline`` / ``mlp_baseline`` run in fp16 on CUDA in the reference).
    """
    import json
    import generate_test_data as gtd
    import baseline
    torch.manual_seed(gtd.SEED)
    sets = gtd.build_datasets()
    out = {}
    meta = {}
    for name, d in sets.items():
        a = d["attention"]
        seq = a["Q"].shape[2]
        heads = 1 if name == "long_seq" else 2
        keep = {"long_seq": 1024, "short_seq": seq}.get(name, 256)
        Q, K, V = (a[k][:1, :heads, :keep].contiguous() for k in ("Q", "K", "V"))
        ref = baseline.attention_baseline(Q.float(), K.float(), V.float())
        sim = validate_int8.sim_attention(Q, K, V)["out"]
        for k, t in (("Q", Q), ("K", K), ("V", V)):
            out[f"{name}__attn_{k}"] = t.numpy()
        out[f"{name}__attn_ref"] = ref.half().numpy()        # the reference keeps this one in fp16
        out[f"{name}__attn_sim"] = sim.numpy()
        m = d["mlp"]
        x = m["x"][:1, :128, ::2].contiguous()
        W1 = m["W1"][::2, ::8].contiguous()
        W2 = m["W2"][::8, ::2].contiguous()
        ref = baseline.mlp_baseline(x.float(), W1.float(), W2.float())
        sim = validate_int8.sim_mlp(x, W1, W2)["out"]
        for k, t in (("x", x), ("W1", W1), ("W2", W2)):
            out[f"{name}__mlp_{k}"] = t.numpy()
        out[f"{name}__mlp_ref"] = ref.half().numpy()
        out[f"{name}__mlp_sim"] = sim.numpy()
        meta[name] = {"thresholds": d["thresholds"], "xfail": sorted(d.get("xfail", {})),
                      "edge": name in validate_int8.EDGE_DATASETS, "seq_len": d["seq_len"]}
    out["meta_json"] = np.frombuffer(json.dumps(meta, sort_keys=True).encode(), dtype=np.uint8)
    np.savez_compressed(os.path.join(HERE, "validation_sets.npz"), **out)


def main(ref_root, only=None):
    test_int8, validate_int8 = _import_reference(ref_root)
    if only == "layernorm":
        layernorm_quantize_cases(test_int8)
        return
    if only == "validation":
        validation_sets(validate_int8)
        return
    torch.manual_seed(0)
    gen = torch.Generator().manual_seed(20240607)

    # 1. per-token quantiser: both reference spellings must agree, store one.
    out = {}
    for name, t in quantiser_cases(gen).items():
        q1, s1 = test_int8.quantize_per_token(t)
        q2, s2 = validate_int8.q_per_token(t)
        assert torch.equal(q1, q2) and torch.equal(s1, s2), name
        out[name + "__x"] = t.numpy()
        out[name + "__q"] = q1.numpy()
        out[name + "__s"] = s1.numpy()
    np.savez_compressed(os.path.join(HERE, "quantize_per_token.npz"), **out)

    # 2. per-channel weight and per-tensor quantisers.
    out = {}
    w = torch.randn(96, 160, generator=gen) * 0.02
    qi, s = validate_int8.q_per_channel_w(w)
    out["w__x"], out["w__q"], out["w__s"] = w.numpy(), qi.numpy(), s.numpy()
    t = torch.randn(5, 64, generator=gen).half()
    qi, s = validate_int8.q_per_tensor(t)
    out["t__x"], out["t__q"], out["t__s"] = t.numpy(), qi.numpy(), np.float32(s)
    np.savez_compressed(os.path.join(HERE, "quantize_weights.npz"), **out)

    # 3. decode attention: the shapes of validation/check_decode.py:50-53 that
    #    are small enough to store (S <= 1000; the S=1000 case with B*H cut to 3),
    #    seeds 1234+S as there, inputs
    #    drawn on the CPU generator; reference = :65-68 on the CPU.
    out = {}
    cases = [(1, 1, 64, 1), (1, 1, 64, 31), (2, 2, 64, 33), (1, 2, 64, 127),
             (2, 2, 64, 128), (1, 3, 64, 1000),
             (1, 1, 128, 1), (1, 1, 128, 31), (2, 2, 128, 33), (1, 2, 128, 127),
             (2, 2, 128, 128), (1, 3, 128, 1000)]
    for B, H, D, S in cases:
        torch.manual_seed(1234 + S)
        Q = torch.randn(B, H, D, dtype=torch.float16)
        K = torch.randn(B, H, S, D, dtype=torch.float16)
        V = torch.randn(B, H, S, D, dtype=torch.float16)
        Qi, sQ = test_int8.quantize_per_token(Q)
        Ki, sK = test_int8.quantize_per_token(K)
        Vi, sV = test_int8.quantize_per_token(V)
        Qd = Qi.float() * sQ.unsqueeze(-1)
        Kd = Ki.float() * sK.unsqueeze(-1)
        Vd = Vi.float() * sV.unsqueeze(-1)
        ref = F.scaled_dot_product_attention(Qd.unsqueeze(2), Kd, Vd).squeeze(2)
        key = f"B{B}_H{H}_D{D}_S{S}"
        for nm, arr in (("Qi", Qi), ("Ki", Ki), ("Vi", Vi), ("sQ", sQ),
                        ("sK", sK), ("sV", sV), ("ref", ref)):
            out[f"{key}__{nm}"] = arr.numpy()
    # config 0 of the benchmark plan: B1 H12 D64 ctx1024, seed 0, q fp16, K/V fp32
    torch.manual_seed(0)
    q = torch.randn(1, 12, 1, 64).half()
    K = torch.randn(1, 12, 1024, 64)
    V = torch.randn(1, 12, 1024, 64)
    Qi, sQ = test_int8.quantize_per_token(q.squeeze(2))
    Ki, sK = test_int8.quantize_per_token(K)
    Vi, sV = test_int8.quantize_per_token(V)
    ref = F.scaled_dot_product_attention(
        (Qi.float() * sQ.unsqueeze(-1)).unsqueeze(2),
        Ki.float() * sK.unsqueeze(-1), Vi.float() * sV.unsqueeze(-1)).squeeze(2)
    for nm, arr in (("Qi", Qi), ("Ki", Ki), ("Vi", Vi), ("sQ", sQ),
                    ("sK", sK), ("sV", sV), ("ref", ref)):
        out[f"cfg0__{nm}"] = arr.numpy()
    np.savez_compressed(os.path.join(HERE, "decode_attention.npz"), **out)

    # 4. MLP simulation (tile shape -> per-token/per-channel/per-token-out path)
    #    and a non-tile shape (per-tensor path).
    out = {}
    for tag, (T, dm, dff) in {"tile": (128, 128, 256), "small": (4, 64, 96)}.items():
        x = torch.randn(1, T, dm, generator=gen).half()
        W1 = (torch.randn(dm, dff, generator=gen) * 0.02).half()
        W2 = (torch.randn(dff, dm, generator=gen) * 0.02).half()
        st = validate_int8.sim_mlp(x.float(), W1.float(), W2.float())
        out[f"{tag}__x"], out[f"{tag}__W1"], out[f"{tag}__W2"] = x.numpy(), W1.numpy(), W2.numpy()
        for k in ("h_pre_gelu", "h_gelu", "h_requant", "out"):
            out[f"{tag}__{k}"] = st[k].reshape(T, -1).numpy()
    np.savez_compressed(os.path.join(HERE, "mlp_sim.npz"), **out)
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    if len(sys.argv) not in (2, 3):
        sys.exit("usage: make_golden.py <path to the reference checkout> [layernorm|validation]")
    main(sys.argv[1], sys.argv[2] if len(sys.argv) == 3 else None)
    if len(sys.argv) == 2:
        main(sys.argv[1], "layernorm")
        main(sys.argv[1], "validation")
