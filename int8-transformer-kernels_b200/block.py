"""One pre-LN transformer block around the INT8 ops: the caller either side of the hot path.

Mirrors ``Block`` of the reference's end-to-end bench (``bench/bench_block.py:73-160``):
LayerNorm, QKV and output projections stay fp16 (cuBLAS through torch) and are shared by
both paths; the attention core and the MLP run either in fp16 (torch SDPA, fp16 GEMMs) or on
the INT8 kernels of this package.  Where the reference quantises with four or five eager
torch kernels per tensor (``bench/bench_block.py:59-63``), this block calls the fused
``quantize_per_token`` op (one pass, bit-identical codes for fp32 arithmetic on the fp16
input), which is the "quantisation glue" the reference names as its largest remaining cost.

Both regimes of the reference are covered: prefill (seq_q == seq_kv) and decode (one new
token over a prefilled INT8 KV cache).
"""
import importlib

import torch
import torch.nn.functional as F


def _ext():
    return importlib.import_module(__package__).int8_ext


def quantize_per_channel(w):
    """Per-output-channel weight quantisation, amax over the input dim (``bench/bench_block.py:66-70``)."""
    sc = w.float().abs().amax(0, keepdim=True).clamp(min=1e-8) / 127.0
    i8 = (w.float() / sc).round().clamp(-128, 127).to(torch.int8)
    return i8.contiguous(), sc.squeeze(0).contiguous().float()


class Int8Block:
    """Weights of one block; fp16 and INT8 forwards for prefill and decode."""

    def __init__(self, d_model, heads, d_ff, dtype=torch.float16, device="cuda", seed=0):
        self.d, self.H, self.dff = d_model, heads, d_ff
        self.Dh = d_model // heads
        g = torch.Generator(device=device).manual_seed(seed)
        rn = lambda *s: torch.randn(*s, generator=g, device=device, dtype=dtype)
        self.Wqkv = rn(d_model, 3 * d_model) * (d_model ** -0.5)
        self.Wo = rn(d_model, d_model) * (d_model ** -0.5)
        self.W1 = rn(d_model, d_ff) * (d_model ** -0.5)
        self.W2 = rn(d_ff, d_model) * (d_ff ** -0.5)
        self.W1i, self.sW1 = quantize_per_channel(self.W1)
        self.W2i, self.sW2 = quantize_per_channel(self.W2)
        self.ext = _ext()

    # ---- shared fp16 pieces ----
    def _ln(self, x):
        return F.layer_norm(x, (self.d,))

    def _project_qkv(self, h):
        B, S, _ = h.shape
        q, k, v = (h @ self.Wqkv).split(self.d, dim=-1)
        shp = lambda t: t.view(B, S, self.H, self.Dh).transpose(1, 2).contiguous()
        return shp(q), shp(k), shp(v)

    def _mlp_fp16(self, h):
        return F.gelu(h @ self.W1, approximate="tanh") @ self.W2

    def _mlp_int8(self, h, fused_ln=False):
        """h: the MLP input; with fused_ln, h is the residual stream and LayerNorm happens inside
        the quantiser kernel (``layernorm_quantize``)."""
        B, S, d = h.shape
        xi, sx = self.ext.layernorm_quantize(h) if fused_ln else self.ext.quantize_per_token(h)
        out_i8, out_sc = self.ext.int8_mlp_forward(xi, self.W1i, self.W2i, sx.reshape(-1), self.sW1, self.sW2)
        # dequantise and add the residual stream in one pass
        return self.ext.dequantize_per_token(out_i8, out_sc, h if fused_ln else None)

    def _tail(self, x, a, use_int8):
        h = x + a @ self.Wo
        if use_int8:
            return self._mlp_int8(h, fused_ln=True)        # LayerNorm, MLP, dequantise + residual
        return h + self._mlp_fp16(self._ln(h))

    # ---- prefill ----
    def forward_prefill(self, x, use_int8):
        B, S, _ = x.shape
        if use_int8:
            # projection -> int8 heads in one pass: no split / transpose / contiguous copies
            qkv_i, qkv_s = self.ext.quantize_qkv_heads(self._ln(x) @ self.Wqkv, self.H)
            a = self.ext.int8_attention_forward(qkv_i[0], qkv_i[1], qkv_i[2], qkv_s[0].reshape(-1),
                                                qkv_s[1].reshape(-1), qkv_s[2].reshape(-1))
        else:
            q, k, v = self._project_qkv(self._ln(x))
            a = F.scaled_dot_product_attention(q, k, v)
        return self._tail(x, a.transpose(1, 2).contiguous().view(B, S, self.d), use_int8)

    # ---- decode ----
    def quantize_kv(self, K, V):
        """fp16/fp32 [B,H,S,Dh] -> the INT8 cache tuple the decode path takes."""
        Ki, sK = self.ext.quantize_per_token(K)
        Vi, sV = self.ext.quantize_per_token(V)
        return Ki, Vi, sK.reshape(-1).contiguous(), sV.reshape(-1).contiguous()

    def append_kv(self, x, kv, pos):
        """Project the new token x [B,1,d], quantise its K and V rows and write them into the INT8
        cache (Ki, Vi, sK, sV) at position pos, in place (quantise on write)."""
        B = x.size(0)
        _, k, v = (self._ln(x) @ self.Wqkv).split(self.d, dim=-1)
        Ki, Vi, sK, sV = kv
        self.ext.kv_append_quantize(k.reshape(B, self.H, self.Dh), v.reshape(B, self.H, self.Dh), Ki, Vi, sK, sV, pos)

    def forward_decode(self, x, kv, use_int8):
        """x: [B,1,d] new token; kv: (Ki,Vi,sK,sV) for the INT8 path, (Kf,Vf) for fp16."""
        B = x.size(0)
        q, _, _ = (self._ln(x) @ self.Wqkv).split(self.d, dim=-1)
        if use_int8:
            Ki, Vi, sK, sV = kv
            qi, sq = self.ext.quantize_per_token(q.view(B, self.H, self.Dh).contiguous())
            a = self.ext.int8_decode_attention_forward(qi, Ki, Vi, sq.reshape(-1), sK, sV).view(B, 1, self.d)
        else:
            Kf, Vf = kv
            a = F.scaled_dot_product_attention(q.view(B, self.H, 1, self.Dh), Kf, Vf)
            a = a.transpose(1, 2).contiguous().view(B, 1, self.d)
        return self._tail(x, a, use_int8)
