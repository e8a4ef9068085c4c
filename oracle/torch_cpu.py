"""Oracle: the reference's CPU torch path, restated for timing and parity.

Test infrastructure only -- see ``oracle/__init__.py``.

The reference has no native CPU implementation of the hot path; what runs on
host cores is its torch reference computation.  These functions restate it in
CPU torch so it can be timed on a machine that has no copy of the reference.
"""
import torch
import torch.nn.functional as F


def decode_attention_cpu(Qi, Ki, Vi, sQ, sK, sV):
    """Dequantise + fp32 SDPA, seq_q == 1.

    Follows ``validation/check_decode.py:65-68``: ``Qd = Qi.float() *
    sQ[..., None]`` (likewise K, V), then
    ``F.scaled_dot_product_attention(Qd.unsqueeze(2), Kd, Vd).squeeze(2)``.
    ``Qi`` int8 [B,H,D]; ``Ki``,``Vi`` int8 [B,H,S,D]; scales fp32 [B,H] /
    [B,H,S].  Returns fp32 [B,H,D].
    """
    Qd = Qi.float() * sQ.unsqueeze(-1)
    Kd = Ki.float() * sK.unsqueeze(-1)
    Vd = Vi.float() * sV.unsqueeze(-1)
    return F.scaled_dot_product_attention(Qd.unsqueeze(2), Kd, Vd).squeeze(2)


def quantize_per_token_cpu(t):
    """``tests/test_int8.py:47-63`` restated in CPU torch."""
    t_f = t.float()
    abs_max = t_f.abs().amax(dim=-1, keepdim=True).clamp(min=1e-8)
    scales = abs_max / 127.0
    q = (t_f / scales).round().clamp(-128, 127).to(torch.int8)
    return q, scales.squeeze(-1)


def mlp_cpu(x, W1, W2):
    """``sim_mlp`` (``validation/validate_int8.py:174-225``) on tile shapes,
    restated in CPU torch: per-token x, per-channel W, tanh-GELU, per-token
    hidden and output requant.  Returns the dequantised fp32 output."""
    def q_ch(w):
        s = w.float().abs().amax(dim=0).clamp(min=1e-8) / 127.0
        return (w.float() / s).round().clamp(-128, 127) * s
    xi, sx = quantize_per_token_cpu(x)
    xd = xi.float() * sx.unsqueeze(-1)
    h = F.gelu(xd @ q_ch(W1), approximate="tanh")
    hi, sh = quantize_per_token_cpu(h)
    out = (hi.float() * sh.unsqueeze(-1)) @ q_ch(W2)
    oi, so = quantize_per_token_cpu(out)
    return oi.float() * so.unsqueeze(-1)
