"""A pre-LN transformer block built on the INT8 ops: what calls the hot path from either side.

The reference measures its kernels inside such a block (``bench/bench_block.py:73-231``): the
residual stream, LayerNorm and the QKV projection stay fp16; attention and the MLP run either
in fp16 (torch SDPA and fp16 GEMMs: the yardstick) or on the INT8 kernels.  Here the INT8 route
avoids the eager tensor-by-tensor glue that bench measured as its largest remaining cost
(``OPTIMIZATION.md:241-246``) by using the fused producers of this package:

  prefill   LayerNorm -> fp16 QKV GEMM -> ``quantize_qkv_heads`` (head-major INT8 in one pass)
            -> ``int8_attention_forward`` -> fp16 output projection
  decode    the new token's q quantised, attention over the INT8 KV cache with the result
            quantised per token inside the merge kernel
            (``int8_decode_attention_forward_quantized``), INT8 output projection (``int8_linear``)
  both      ``layernorm_quantize`` -> ``int8_mlp_forward`` -> ``dequantize_per_token`` with the
            residual added in the same pass

``BlockWeights`` holds one set of random weights in both precisions; ``Fp16Route`` and
``Int8Route`` are the two implementations of the same three steps (attend at prefill, attend at
decode, feed-forward); ``Int8Block`` keeps the entry points the tests and the benchmark use.
"""
import importlib
from dataclasses import dataclass

import torch
import torch.nn.functional as F


def _ops():
    return importlib.import_module(__package__).int8_ext


def per_channel_int8(weight):
    """[in, out] float weight -> (int8 codes, fp32 scale per output column), symmetric, the
    arithmetic of ``validation/validate_int8.py:75-81``."""
    w32 = weight.float()
    scale = w32.abs().amax(dim=0).clamp_min(1e-8).div(127.0)
    codes = torch.clamp(torch.round(w32 / scale), -128, 127).to(torch.int8)
    return codes.contiguous(), scale.float().contiguous()


@dataclass
class BlockWeights:
    d_model: int
    heads: int
    d_ff: int
    qkv: torch.Tensor      # [d_model, 3*d_model] fp16
    proj: torch.Tensor     # [d_model, d_model]   fp16
    up: torch.Tensor       # [d_model, d_ff]      fp16
    down: torch.Tensor     # [d_ff, d_model]      fp16
    proj_i8: torch.Tensor
    proj_scale: torch.Tensor
    up_i8: torch.Tensor
    up_scale: torch.Tensor
    down_i8: torch.Tensor
    down_scale: torch.Tensor

    @property
    def head_dim(self):
        return self.d_model // self.heads

    @classmethod
    def random(cls, d_model, heads, d_ff, device="cuda", seed=0):
        gen = torch.Generator(device=device).manual_seed(seed)

        def draw(rows, cols):          # variance-preserving initialisation
            w = torch.randn(rows, cols, generator=gen, device=device, dtype=torch.float16)
            return w * rows ** -0.5

        qkv, proj, up, down = draw(d_model, 3 * d_model), draw(d_model, d_model), draw(d_model, d_ff), draw(d_ff, d_model)
        return cls(d_model, heads, d_ff, qkv, proj, up, down, *per_channel_int8(proj), *per_channel_int8(up),
                   *per_channel_int8(down))


class Fp16Route:
    """The yardstick: torch SDPA and fp16 GEMMs."""

    def __init__(self, w):
        self.w = w

    def _heads(self, t, batch, seq):
        return t.view(batch, seq, self.w.heads, self.w.head_dim).transpose(1, 2)

    def attend_prefill(self, x):
        batch, seq, _ = x.shape
        q, k, v = (F.layer_norm(x, (self.w.d_model,)) @ self.w.qkv).chunk(3, dim=-1)
        ctx = F.scaled_dot_product_attention(self._heads(q, batch, seq), self._heads(k, batch, seq),
                                             self._heads(v, batch, seq))
        return x + ctx.transpose(1, 2).reshape(batch, seq, self.w.d_model) @ self.w.proj

    def attend_decode(self, x, cache):
        keys, values = cache
        batch = x.size(0)
        q = (F.layer_norm(x, (self.w.d_model,)) @ self.w.qkv)[..., : self.w.d_model]
        ctx = F.scaled_dot_product_attention(self._heads(q, batch, 1), keys, values)
        return x + ctx.transpose(1, 2).reshape(batch, 1, self.w.d_model) @ self.w.proj

    def feed_forward(self, h):
        y = F.layer_norm(h, (self.w.d_model,))
        return h + F.gelu(y @ self.w.up, approximate="tanh") @ self.w.down


class Int8Route:
    """The INT8 kernels of this package with their fused producers."""

    def __init__(self, w):
        self.w = w
        self.ops = _ops()

    def attend_prefill(self, x):
        batch, seq, _ = x.shape
        fused = F.layer_norm(x, (self.w.d_model,)) @ self.w.qkv
        codes, scales = self.ops.quantize_qkv_heads(fused, self.w.heads)       # [3,B,H,S,Dh], [3,B,H,S]
        ctx = self.ops.int8_attention_forward(codes[0], codes[1], codes[2], scales[0].reshape(-1),
                                              scales[1].reshape(-1), scales[2].reshape(-1))
        return x + ctx.transpose(1, 2).reshape(batch, seq, self.w.d_model) @ self.w.proj

    def attend_decode(self, x, cache):
        k_codes, v_codes, k_scales, v_scales = cache
        batch = x.size(0)
        q = (F.layer_norm(x, (self.w.d_model,)) @ self.w.qkv)[..., : self.w.d_model]
        q_codes, q_scales = self.ops.quantize_per_token(q.reshape(batch, self.w.heads, self.w.head_dim))
        if self.w.heads <= 32 and self.w.d_model % 128 == 0:
            # attention hands its result over as INT8 with one scale per token; INT8 projection
            ctx_codes, ctx_scales = self.ops.int8_decode_attention_forward_quantized(
                q_codes, k_codes, v_codes, q_scales.reshape(-1), k_scales, v_scales)
            return x + self.ops.int8_linear(ctx_codes, ctx_scales, self.w.proj_i8, self.w.proj_scale).view_as(x)
        ctx = self.ops.int8_decode_attention_forward(q_codes, k_codes, v_codes, q_scales.reshape(-1), k_scales, v_scales)
        return x + ctx.view(batch, 1, self.w.d_model) @ self.w.proj

    def feed_forward(self, h):
        codes, scales = self.ops.layernorm_quantize(h)                         # LayerNorm inside the quantiser
        out_codes, out_scales = self.ops.int8_mlp_forward(codes, self.w.up_i8, self.w.down_i8, scales.reshape(-1),
                                                          self.w.up_scale, self.w.down_scale)
        return self.ops.dequantize_per_token(out_codes, out_scales, h)         # dequantise + residual

    def quantize_cache(self, keys, values):
        k_codes, k_scales = self.ops.quantize_per_token(keys)
        v_codes, v_scales = self.ops.quantize_per_token(values)
        return k_codes, v_codes, k_scales.reshape(-1).contiguous(), v_scales.reshape(-1).contiguous()

    def append_to_cache(self, x, cache, position):
        """Quantise the new token's K and V rows straight into the INT8 cache at ``position``."""
        batch = x.size(0)
        fused = F.layer_norm(x, (self.w.d_model,)) @ self.w.qkv
        k_new = fused[..., self.w.d_model: 2 * self.w.d_model].reshape(batch, self.w.heads, self.w.head_dim)
        v_new = fused[..., 2 * self.w.d_model:].reshape(batch, self.w.heads, self.w.head_dim)
        k_codes, v_codes, k_scales, v_scales = cache
        self.ops.kv_append_quantize(k_new, v_new, k_codes, v_codes, k_scales, v_scales, position)


class Int8Block:
    """One block with both routes over the same weights.

    ``forward_prefill(x, use_int8)``: x fp16 [B, S, d_model].
    ``forward_decode(x, cache, use_int8)``: x fp16 [B, 1, d_model]; cache = ``quantize_kv(K, V)`` for
    the INT8 route, ``(K, V)`` fp16 [B, H, S, Dh] for the fp16 route.
    """

    def __init__(self, d_model, heads, d_ff, device="cuda", seed=0):
        self.weights = BlockWeights.random(d_model, heads, d_ff, device=device, seed=seed)
        self.routes = {False: Fp16Route(self.weights), True: Int8Route(self.weights)}

    def forward_prefill(self, x, use_int8, fp16_attention=False):
        """``fp16_attention`` with ``use_int8``: the mixed route -- attention through torch's fp16
        flash kernel, feed-forward on the INT8 MLP with its fused LayerNorm/quantise/dequantise."""
        route = self.routes[bool(use_int8)]
        attend = self.routes[False].attend_prefill if (use_int8 and fp16_attention) else route.attend_prefill
        return route.feed_forward(attend(x))

    def forward_decode(self, x, cache, use_int8):
        route = self.routes[bool(use_int8)]
        return route.feed_forward(route.attend_decode(x, cache))

    def quantize_kv(self, keys, values):
        return self.routes[True].quantize_cache(keys, values)

    def append_kv(self, x, cache, position):
        self.routes[True].append_to_cache(x, cache, position)
