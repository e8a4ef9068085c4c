// int8_ext -- PyTorch binding over the i8tk C ABI (include/i8tk.h).
//
// Mirrors the Python surface of the reference's torch extension
// (kernels/int8_ext.cu:458-479): the same six names / seven overloads with
// the same argument order, dtypes, shapes, scale layouts and return values,
// the same argument checks (TORCH_CHECK -> RuntimeError) with the same
// messages.  Differences, all additive:
//   * launches go to torch's current CUDA stream on the tensors' device and
//     scratch comes from torch's caching allocator (the reference uses the
//     legacy default stream and process-global static buffers);
//   * a non-zero status from the C ABI raises RuntimeError;
//   * extra ops the reference only has as Python code or inside its launcher:
//     quantize_per_token, int8_decode_attention_partial,
//     int8_decode_combine_partials, and check_status (the reference checks no
//     CUDA error; here every device-side wait is bounded and a wait that gave up
//     is recorded in the scratch block of the stream it ran on).
// This file contains no kernels and no arithmetic.
#include <torch/extension.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <c10/cuda/CUDAGraphsC10Utils.h>

#include <cuda_runtime.h>

#include <map>
#include <mutex>
#include <tuple>
#include <utility>
#include <vector>

#include "../../include/i8tk.h"

namespace {

void check_status(int rc, const char* what) {
    TORCH_CHECK(rc == I8TK_OK, what, " failed: ", i8tk_status_string(rc), " (", i8tk_last_error(), ")");
}

i8tk_stream_t current_stream() {
    return static_cast<i8tk_stream_t>(c10::cuda::getCurrentCUDAStream().stream());
}

// Scratch of the ops.  One grow-only block per (device, stream), kept for the life of the
// process: calls on one stream run one after the other, so they can share it, and calls on
// different streams never do.  Its first eight bytes are the status block of the C ABI: word 0
// is cleared by the first kernel of every call, word 1 counts bounded waits that gave up and
// is only ever reset by check_status() below -- so a caller may look rarely and still learn
// that a call in between failed.  While a CUDA graph is being captured the block comes from
// torch's allocator instead (the capture's private pool owns it), as it did before.
struct WsKey {
    int device;
    cudaStream_t stream;
    bool operator<(const WsKey& o) const { return device != o.device ? device < o.device : stream < o.stream; }
};
std::mutex g_ws_mutex;
std::map<WsKey, torch::Tensor> g_ws_cache;

torch::Tensor make_workspace(size_t bytes, const torch::Device& dev) {
    const int64_t need = static_cast<int64_t>(bytes > 256 ? bytes : 256);
    const auto opts = torch::TensorOptions().dtype(torch::kUInt8).device(dev);   // 512-byte aligned blocks
    const auto cur = c10::cuda::getCurrentCUDAStream(dev.index());
    if (c10::cuda::currentStreamCaptureStatusMayInitCtx() != c10::cuda::CaptureStatus::None)
        return torch::empty({need}, opts);
    std::lock_guard<std::mutex> lock(g_ws_mutex);
    torch::Tensor& slot = g_ws_cache[WsKey{static_cast<int>(dev.index()), cur.stream()}];
    if (!slot.defined() || slot.numel() < need) {
        // grow with headroom; the status block travels to the new block
        auto grown = torch::empty({need + need / 4}, opts);
        if (slot.defined()) grown.narrow(0, 0, 256).copy_(slot.narrow(0, 0, 256));
        else grown.narrow(0, 0, 256).zero_();
        slot = grown;
    }
    return slot;
}

// The fused MLP gets a scratch block of its own per (device, stream): nothing else writes to
// it, so from the second forward of a shape on it the library can be told that the block is as
// the previous forward left it (I8TK_MLP_WORKSPACE_KEPT: no preset kernel).  `tag` identifies
// shape and layout; *kept says whether the previous forward on this block had the same tag.
struct MlpWs {
    torch::Tensor buf;
    uint64_t tag = 0;
};
std::map<WsKey, MlpWs> g_mlp_ws_cache;

torch::Tensor make_mlp_workspace(size_t bytes, const torch::Device& dev, uint64_t tag, bool* kept) {
    const int64_t need = static_cast<int64_t>(bytes > 256 ? bytes : 256);
    const auto opts = torch::TensorOptions().dtype(torch::kUInt8).device(dev);
    *kept = false;
    const auto cur = c10::cuda::getCurrentCUDAStream(dev.index());
    if (c10::cuda::currentStreamCaptureStatusMayInitCtx() != c10::cuda::CaptureStatus::None)
        return torch::empty({need}, opts);
    std::lock_guard<std::mutex> lock(g_ws_mutex);
    MlpWs& slot = g_mlp_ws_cache[WsKey{static_cast<int>(dev.index()), cur.stream()}];
    if (!slot.buf.defined() || slot.buf.numel() < need) {
        auto grown = torch::empty({need + need / 4}, opts);
        if (slot.buf.defined()) grown.narrow(0, 0, 256).copy_(slot.buf.narrow(0, 0, 256));
        else grown.narrow(0, 0, 256).zero_();
        slot.buf = grown;
        slot.tag = 0;
    }
    *kept = slot.tag == tag && tag != 0;
    slot.tag = tag;
    return slot.buf;
}

// After a failed forward the block's state is unknown: the next call presets it again.
void forget_mlp_workspace(const torch::Device& dev) {
    const auto cur = c10::cuda::getCurrentCUDAStream(dev.index());
    std::lock_guard<std::mutex> lock(g_ws_mutex);
    auto it = g_mlp_ws_cache.find(WsKey{static_cast<int>(dev.index()), cur.stream()});
    if (it != g_mlp_ws_cache.end()) it->second.tag = 0;
}

// Synchronises every stream an op has run on, reads the status blocks back and raises if a
// bounded device-side wait gave up since the last check (the outputs of such a call are not
// valid).  Resets the counts.  Returns the number of blocks looked at.
int64_t check_status_torch() {
    std::vector<std::pair<WsKey, torch::Tensor>> blocks;
    {
        std::lock_guard<std::mutex> lock(g_ws_mutex);
        for (auto& kv : g_ws_cache) blocks.emplace_back(kv.first, kv.second);
        for (auto& kv : g_mlp_ws_cache) blocks.emplace_back(kv.first, kv.second.buf);
    }
    int64_t failures = 0;
    for (auto& kv : blocks) {
        c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(kv.first.device));
        uint32_t words[2] = {0u, 0u};
        TORCH_CHECK(cudaMemcpyAsync(words, kv.second.data_ptr(), sizeof(words), cudaMemcpyDeviceToHost,
                                    kv.first.stream) == cudaSuccess, "status read-back failed");
        TORCH_CHECK(cudaStreamSynchronize(kv.first.stream) == cudaSuccess, "stream synchronisation failed");
        if (words[1] != 0u) {
            failures += words[1];
            TORCH_CHECK(cudaMemsetAsync(kv.second.data_ptr(), 0, sizeof(words), kv.first.stream) == cudaSuccess,
                        "status reset failed");
        }
    }
    TORCH_CHECK(failures == 0, "int8_ext: ", failures,
                " device-side check(s) failed since the last look (a bounded wait that gave up, or a page id outside "
                "the pool); the outputs of those calls are not valid");
    return static_cast<int64_t>(blocks.size());
}

// ---- decode attention (kernels/int8_ext.cu:136-178) -------------------------
struct DecodeArgs {
    int BH, S, D;
    torch::Tensor sQ, sK, sV;
};

DecodeArgs check_decode(const torch::Tensor& Q, const torch::Tensor& K, const torch::Tensor& V,
                        const torch::Tensor& scale_Q, const torch::Tensor& scale_K,
                        const torch::Tensor& scale_V) {
    TORCH_CHECK(Q.device().is_cuda(), "Q must be a CUDA tensor");
    TORCH_CHECK(Q.dtype() == torch::kInt8, "Q must be int8");
    TORCH_CHECK(K.dtype() == torch::kInt8 && V.dtype() == torch::kInt8, "K, V must be int8");
    TORCH_CHECK(Q.is_contiguous() && K.is_contiguous() && V.is_contiguous(),
                "Q/K/V must be contiguous");
    TORCH_CHECK(Q.dim() == 3, "expected Q (batch, heads, head_dim) — seq_q == 1");
    TORCH_CHECK(K.dim() == 4, "expected K (batch, heads, seq_kv, head_dim)");
    TORCH_CHECK(K.sizes() == V.sizes(), "K/V shape mismatch");
    const int64_t batch = Q.size(0), heads = Q.size(1), head_dim = Q.size(2), seq_kv = K.size(2);
    TORCH_CHECK(K.size(0) == batch && K.size(1) == heads && K.size(3) == head_dim,
                "Q/K head/batch/dim mismatch");
    TORCH_CHECK(head_dim == 64 || head_dim == 128, "decode kernel v1 supports head_dim 64 or 128");
    TORCH_CHECK(K.device() == Q.device() && V.device() == Q.device(), "Q/K/V must be on one device");
    TORCH_CHECK(scale_Q.dtype() == torch::kFloat32 && scale_K.dtype() == torch::kFloat32 &&
                    scale_V.dtype() == torch::kFloat32, "scales must be float32");
    TORCH_CHECK(scale_Q.device() == Q.device() && scale_K.device() == Q.device() &&
                    scale_V.device() == Q.device(), "scales must be on the same CUDA device as Q");
    TORCH_CHECK(batch * heads < (1ll << 31) && seq_kv < (1ll << 31), "shape too large");
    DecodeArgs a;
    a.BH = static_cast<int>(batch * heads);
    a.S = static_cast<int>(seq_kv);
    a.D = static_cast<int>(head_dim);
    a.sQ = scale_Q.contiguous().view({a.BH});
    a.sK = scale_K.contiguous().view({static_cast<int64_t>(a.BH) * a.S});
    a.sV = scale_V.contiguous().view({static_cast<int64_t>(a.BH) * a.S});
    return a;
}

torch::Tensor int8_decode_attention_forward_torch(torch::Tensor Q, torch::Tensor K, torch::Tensor V,
                                                  torch::Tensor scale_Q, torch::Tensor scale_K,
                                                  torch::Tensor scale_V) {
    DecodeArgs a = check_decode(Q, K, V, scale_Q, scale_K, scale_V);
    c10::cuda::CUDAGuard guard(Q.device());
    auto out = torch::empty({Q.size(0), Q.size(1), Q.size(2)},
                            torch::TensorOptions().dtype(torch::kFloat16).device(Q.device()));
    const size_t wbytes = i8tk_decode_workspace_bytes(a.BH, a.S, a.D);
    auto ws = make_workspace(wbytes, Q.device());
    check_status(i8tk_decode_attention_forward(
                     Q.data_ptr<int8_t>(), K.data_ptr<int8_t>(), V.data_ptr<int8_t>(), out.data_ptr(),
                     a.sQ.data_ptr<float>(), a.sK.data_ptr<float>(), a.sV.data_ptr<float>(), a.BH, a.S,
                     a.D, ws.data_ptr(), wbytes, current_stream()),
                 "int8_decode_attention_forward");
    return out;
}

// Decode attention whose result leaves as INT8 for the output projection: (int8 [B, H*D], fp32 [B]).
std::tuple<torch::Tensor, torch::Tensor> int8_decode_attention_forward_quantized_torch(
    torch::Tensor Q, torch::Tensor K, torch::Tensor V, torch::Tensor scale_Q, torch::Tensor scale_K,
    torch::Tensor scale_V) {
    DecodeArgs a = check_decode(Q, K, V, scale_Q, scale_K, scale_V);
    TORCH_CHECK(Q.size(1) <= 32, "per-token output quantisation takes at most 32 heads");
    c10::cuda::CUDAGuard guard(Q.device());
    auto out = torch::empty({Q.size(0), Q.size(1) * Q.size(2)},
                            torch::TensorOptions().dtype(torch::kInt8).device(Q.device()));
    auto sc = torch::empty({Q.size(0)}, torch::TensorOptions().dtype(torch::kFloat32).device(Q.device()));
    const size_t wbytes = i8tk_decode_workspace_bytes(a.BH, a.S, a.D);
    auto ws = make_workspace(wbytes, Q.device());
    check_status(i8tk_decode_attention_forward_q8(
                     Q.data_ptr<int8_t>(), K.data_ptr<int8_t>(), V.data_ptr<int8_t>(), out.data_ptr<int8_t>(),
                     sc.data_ptr<float>(), nullptr, a.sQ.data_ptr<float>(), a.sK.data_ptr<float>(),
                     a.sV.data_ptr<float>(), static_cast<int>(Q.size(0)), static_cast<int>(Q.size(1)), a.S, a.D,
                     ws.data_ptr(), static_cast<size_t>(ws.numel()), current_stream()),
                 "int8_decode_attention_forward_quantized");
    return {out, sc};
}

// Paged INT8 KV cache, one length per request.  Pools int8 [num_pages, H, page, D] and fp32
// [num_pages, H, page]; page_table int32 [B, max_pages]; seq_lens int32 [B]; max_seq_len is the
// caller's host-side bound on seq_lens.
torch::Tensor int8_decode_attention_paged_torch(torch::Tensor Q, torch::Tensor K_pool, torch::Tensor V_pool,
                                                torch::Tensor scale_Q, torch::Tensor sK_pool,
                                                torch::Tensor sV_pool, torch::Tensor page_table,
                                                torch::Tensor seq_lens, int64_t max_seq_len) {
    TORCH_CHECK(Q.device().is_cuda() && Q.dtype() == torch::kInt8 && Q.dim() == 3 && Q.is_contiguous(),
                "Q must be a contiguous int8 CUDA tensor (batch, heads, head_dim)");
    TORCH_CHECK(K_pool.dtype() == torch::kInt8 && V_pool.dtype() == torch::kInt8 && K_pool.dim() == 4 &&
                    K_pool.sizes() == V_pool.sizes() && K_pool.is_contiguous() && V_pool.is_contiguous(),
                "K_pool, V_pool must be contiguous int8 (num_pages, heads, page_size, head_dim) of one shape");
    const int64_t B = Q.size(0), H = Q.size(1), D = Q.size(2);
    const int64_t pages = K_pool.size(0), page = K_pool.size(2);
    TORCH_CHECK(K_pool.size(1) == H && K_pool.size(3) == D, "Q / pool head or head_dim mismatch");
    TORCH_CHECK(D == 64 || D == 128, "decode kernel v1 supports head_dim 64 or 128");
    TORCH_CHECK(page == 16 || page == 32 || page == 64 || page == 128, "page_size must be 16, 32, 64 or 128");
    TORCH_CHECK(sK_pool.dtype() == torch::kFloat32 && sV_pool.dtype() == torch::kFloat32 &&
                    sK_pool.is_contiguous() && sV_pool.is_contiguous() && sK_pool.numel() == pages * H * page &&
                    sV_pool.numel() == pages * H * page,
                "sK_pool, sV_pool must be contiguous float32 with num_pages*heads*page_size elements");
    TORCH_CHECK(scale_Q.dtype() == torch::kFloat32 && scale_Q.numel() == B * H, "scale_Q must be float32, B*H elements");
    TORCH_CHECK(page_table.dtype() == torch::kInt32 && page_table.dim() == 2 && page_table.size(0) == B &&
                    page_table.is_contiguous(), "page_table must be contiguous int32 (batch, max_pages)");
    TORCH_CHECK(seq_lens.dtype() == torch::kInt32 && seq_lens.numel() == B && seq_lens.is_contiguous(),
                "seq_lens must be contiguous int32 with batch elements");
    TORCH_CHECK(page_table.device() == Q.device() && seq_lens.device() == Q.device() &&
                    K_pool.device() == Q.device() && V_pool.device() == Q.device() &&
                    sK_pool.device() == Q.device() && sV_pool.device() == Q.device() && scale_Q.device() == Q.device(),
                "all tensors must be on one CUDA device");
    TORCH_CHECK(max_seq_len >= 1 && max_seq_len <= page_table.size(1) * page, "max_seq_len does not fit the page table");
    c10::cuda::CUDAGuard guard(Q.device());
    auto sq = scale_Q.contiguous();
    auto out = torch::empty({B, H, D}, torch::TensorOptions().dtype(torch::kFloat16).device(Q.device()));
    const size_t wbytes = i8tk_decode_workspace_bytes(static_cast<int>(B * H), static_cast<int>(max_seq_len),
                                                      static_cast<int>(D));
    auto ws = make_workspace(wbytes, Q.device());
    // the pool size is known here, so page ids are checked on the device (check_status() reports a bad one)
    check_status(i8tk_decode_attention_paged_checked(
                     Q.data_ptr<int8_t>(), K_pool.data_ptr<int8_t>(), V_pool.data_ptr<int8_t>(), out.data_ptr(),
                     sq.data_ptr<float>(), sK_pool.data_ptr<float>(), sV_pool.data_ptr<float>(),
                     page_table.data_ptr<int32_t>(), seq_lens.data_ptr<int32_t>(), static_cast<int>(B),
                     static_cast<int>(H), static_cast<int>(max_seq_len), static_cast<int>(page),
                     static_cast<int>(page_table.size(1)), static_cast<int>(D), static_cast<int>(pages),
                     ws.data_ptr(), wbytes, current_stream()),
                 "int8_decode_attention_paged");
    return out;
}

// Unnormalised (m, l, acc) rows for a KV shard: fp32 [B, H, D+4].
torch::Tensor int8_decode_attention_partial_torch(torch::Tensor Q, torch::Tensor K, torch::Tensor V,
                                                  torch::Tensor scale_Q, torch::Tensor scale_K,
                                                  torch::Tensor scale_V) {
    DecodeArgs a = check_decode(Q, K, V, scale_Q, scale_K, scale_V);
    c10::cuda::CUDAGuard guard(Q.device());
    auto part = torch::empty({Q.size(0), Q.size(1), a.D + 4},
                             torch::TensorOptions().dtype(torch::kFloat32).device(Q.device()));
    const size_t wbytes = i8tk_decode_workspace_bytes(a.BH, a.S, a.D);
    auto ws = make_workspace(wbytes, Q.device());
    check_status(i8tk_decode_attention_partial(
                     Q.data_ptr<int8_t>(), K.data_ptr<int8_t>(), V.data_ptr<int8_t>(),
                     part.data_ptr<float>(), a.sQ.data_ptr<float>(), a.sK.data_ptr<float>(),
                     a.sV.data_ptr<float>(), a.BH, a.S, a.D, ws.data_ptr(), wbytes, current_stream()),
                 "int8_decode_attention_partial");
    return part;
}

// parts fp32 [nparts, B, H, D+4] -> fp16 [B, H, D]
torch::Tensor int8_decode_combine_partials_torch(torch::Tensor parts) {
    TORCH_CHECK(parts.device().is_cuda(), "parts must be a CUDA tensor");
    TORCH_CHECK(parts.dtype() == torch::kFloat32, "parts must be float32");
    TORCH_CHECK(parts.is_contiguous(), "parts must be contiguous");
    TORCH_CHECK(parts.dim() == 4, "expected parts (nparts, batch, heads, head_dim + 4)");
    const int64_t D = parts.size(3) - 4;
    TORCH_CHECK(D == 64 || D == 128, "decode kernel v1 supports head_dim 64 or 128");
    c10::cuda::CUDAGuard guard(parts.device());
    auto out = torch::empty({parts.size(1), parts.size(2), D},
                            torch::TensorOptions().dtype(torch::kFloat16).device(parts.device()));
    check_status(i8tk_decode_combine_partials(parts.data_ptr<float>(), static_cast<int>(parts.size(0)),
                                              static_cast<int>(parts.size(1) * parts.size(2)),
                                              static_cast<int>(D), out.data_ptr(), current_stream()),
                 "int8_decode_combine_partials");
    return out;
}

// ---- prefill attention (kernels/int8_ext.cu:83-129) -----------------------------
torch::Tensor int8_attention_forward_torch(torch::Tensor Q, torch::Tensor K, torch::Tensor V,
                                           torch::Tensor scale_Q, torch::Tensor scale_K,
                                           torch::Tensor scale_V) {
    TORCH_CHECK(Q.device().is_cuda(), "Q must be a CUDA tensor");
    TORCH_CHECK(Q.dtype() == torch::kInt8, "Q must be int8");
    TORCH_CHECK(K.dtype() == torch::kInt8, "K must be int8");
    TORCH_CHECK(V.dtype() == torch::kInt8, "V must be int8");
    TORCH_CHECK(Q.is_contiguous(), "Q must be contiguous");
    TORCH_CHECK(K.is_contiguous(), "K must be contiguous");
    TORCH_CHECK(V.is_contiguous(), "V must be contiguous");
    TORCH_CHECK(Q.dim() == 4, "expected (batch, heads, seq_len, head_dim)");
    TORCH_CHECK(Q.sizes() == K.sizes() && Q.sizes() == V.sizes(), "Q/K/V shape mismatch");
    TORCH_CHECK(scale_Q.dtype() == torch::kFloat32, "scale_Q must be float32");
    TORCH_CHECK(scale_K.dtype() == torch::kFloat32, "scale_K must be float32");
    TORCH_CHECK(scale_V.dtype() == torch::kFloat32, "scale_V must be float32");
    TORCH_CHECK(scale_Q.device().is_cuda(), "scale_Q must be CUDA");
    const int64_t batch = Q.size(0), heads = Q.size(1), seq_len = Q.size(2), head_dim = Q.size(3);
    const int64_t n_tokens = batch * heads * seq_len;
    TORCH_CHECK(n_tokens < (1ll << 31), "shape too large");
    auto sQ = scale_Q.contiguous().view({n_tokens});
    auto sK = scale_K.contiguous().view({n_tokens});
    auto sV = scale_V.contiguous().view({n_tokens});
    c10::cuda::CUDAGuard guard(Q.device());
    auto out = torch::empty({batch, heads, seq_len, head_dim},
                            torch::TensorOptions().dtype(torch::kFloat16).device(Q.device()));
    const size_t wbytes = i8tk_attention_workspace_bytes(static_cast<int>(batch), static_cast<int>(heads),
                                                         static_cast<int>(seq_len), static_cast<int>(head_dim));
    auto ws = make_workspace(wbytes, Q.device());
    check_status(i8tk_attention_forward(Q.data_ptr<int8_t>(), K.data_ptr<int8_t>(), V.data_ptr<int8_t>(),
                                        out.data_ptr(), sQ.data_ptr<float>(), sK.data_ptr<float>(),
                                        sV.data_ptr<float>(), static_cast<int>(batch), static_cast<int>(heads),
                                        static_cast<int>(seq_len), static_cast<int>(head_dim), ws.data_ptr(),
                                        wbytes, current_stream()),
                 "int8_attention_forward");
    return out;
}

// ---- per-token quantiser (tests/test_int8.py:47-63) ---------------------------
std::tuple<torch::Tensor, torch::Tensor> quantize_per_token_torch(torch::Tensor t) {
    TORCH_CHECK(t.device().is_cuda(), "t must be a CUDA tensor");
    TORCH_CHECK(t.dtype() == torch::kFloat32 || t.dtype() == torch::kFloat16,
                "t must be float32 or float16");
    TORCH_CHECK(t.dim() >= 1, "t must have at least one dimension");
    auto x = t.contiguous();
    const int64_t cols = x.size(-1);
    TORCH_CHECK(cols >= 1 && cols < (1ll << 31), "last dimension out of range");
    const int64_t rows = cols ? x.numel() / cols : 0;
    c10::cuda::CUDAGuard guard(x.device());
    auto q = torch::empty(x.sizes(), torch::TensorOptions().dtype(torch::kInt8).device(x.device()));
    auto sizes = x.sizes().vec();
    sizes.pop_back();
    auto s = torch::empty(sizes, torch::TensorOptions().dtype(torch::kFloat32).device(x.device()));
    if (rows == 0) return {q, s};
    int rc;
    if (x.dtype() == torch::kFloat32)
        rc = i8tk_quantize_per_token_f32(x.data_ptr<float>(), q.data_ptr<int8_t>(), s.data_ptr<float>(),
                                         rows, static_cast<int>(cols), current_stream());
    else
        rc = i8tk_quantize_per_token_f16(x.data_ptr(), q.data_ptr<int8_t>(), s.data_ptr<float>(), rows,
                                         static_cast<int>(cols), current_stream());
    check_status(rc, "quantize_per_token");
    return {q, s};
}

// ---- producer-side quantisation (the eager glue of bench/bench_block.py:59-63,93-94) ----
std::tuple<torch::Tensor, torch::Tensor> layernorm_quantize_torch(torch::Tensor t, double eps) {
    TORCH_CHECK(t.device().is_cuda(), "t must be a CUDA tensor");
    TORCH_CHECK(t.dtype() == torch::kFloat16, "t must be float16");
    TORCH_CHECK(t.dim() >= 1, "t must have at least one dimension");
    auto x = t.contiguous();
    const int64_t cols = x.size(-1);
    TORCH_CHECK(cols >= 8 && cols % 8 == 0 && cols <= 4096, "last dimension must be a multiple of 8, at most 4096");
    const int64_t rows = x.numel() / cols;
    c10::cuda::CUDAGuard guard(x.device());
    auto q = torch::empty(x.sizes(), torch::TensorOptions().dtype(torch::kInt8).device(x.device()));
    auto sizes = x.sizes().vec();
    sizes.pop_back();
    auto s = torch::empty(sizes, torch::TensorOptions().dtype(torch::kFloat32).device(x.device()));
    if (rows == 0) return {q, s};
    check_status(i8tk_layernorm_quantize_f16(x.data_ptr(), q.data_ptr<int8_t>(), s.data_ptr<float>(), rows,
                                             static_cast<int>(cols), static_cast<float>(eps), current_stream()),
                 "layernorm_quantize");
    return {q, s};
}

// qkv fp16 [B, S, 3*H*Dh] -> (int8 [3,B,H,S,Dh], fp32 [3,B,H,S]): index 0/1/2 = q/k/v.
std::tuple<torch::Tensor, torch::Tensor> quantize_qkv_heads_torch(torch::Tensor qkv, int64_t heads) {
    TORCH_CHECK(qkv.device().is_cuda() && qkv.dtype() == torch::kFloat16 && qkv.dim() == 3,
                "qkv must be a float16 CUDA tensor (batch, seq, 3*heads*head_dim)");
    auto x = qkv.contiguous();
    const int64_t B = x.size(0), S = x.size(1);
    TORCH_CHECK(heads > 0 && x.size(2) % (3 * heads) == 0, "last dimension must be 3*heads*head_dim");
    const int64_t Dh = x.size(2) / (3 * heads);
    TORCH_CHECK(Dh == 64 || Dh == 128, "head_dim must be 64 or 128");
    c10::cuda::CUDAGuard guard(x.device());
    auto q = torch::empty({3, B, heads, S, Dh}, torch::TensorOptions().dtype(torch::kInt8).device(x.device()));
    auto s = torch::empty({3, B, heads, S}, torch::TensorOptions().dtype(torch::kFloat32).device(x.device()));
    if (B * S == 0) return {q, s};
    check_status(i8tk_quantize_qkv_heads_f16(x.data_ptr(), q.data_ptr<int8_t>(), s.data_ptr<float>(),
                                             static_cast<int>(B), static_cast<int>(S), static_cast<int>(heads),
                                             static_cast<int>(Dh), current_stream()),
                 "quantize_qkv_heads");
    return {q, s};
}

// fp16(q * scales[row]) (+ residual): q int8 [..., cols], scales fp32 with one value per row.
torch::Tensor dequantize_per_token_torch(torch::Tensor q, torch::Tensor scales, c10::optional<torch::Tensor> residual) {
    TORCH_CHECK(q.device().is_cuda() && q.dtype() == torch::kInt8 && q.dim() >= 1 && q.is_contiguous(),
                "q must be a contiguous int8 CUDA tensor");
    const int64_t cols = q.size(-1);
    TORCH_CHECK(cols >= 16 && cols % 16 == 0, "last dimension must be a positive multiple of 16");
    const int64_t rows = q.numel() / cols;
    TORCH_CHECK(scales.dtype() == torch::kFloat32 && scales.numel() == rows && scales.device() == q.device(),
                "scales must be float32 with one value per row");
    auto sc = scales.contiguous();
    c10::cuda::CUDAGuard guard(q.device());
    auto out = torch::empty(q.sizes(), torch::TensorOptions().dtype(torch::kFloat16).device(q.device()));
    const void* res = nullptr;
    torch::Tensor r;
    if (residual.has_value()) {
        r = residual->contiguous();
        TORCH_CHECK(r.dtype() == torch::kFloat16 && r.sizes() == q.sizes() && r.device() == q.device(),
                    "residual must be float16 of q's shape");
        res = r.data_ptr();
    }
    if (rows == 0) return out;
    check_status(i8tk_dequantize_per_token_f16(q.data_ptr<int8_t>(), sc.data_ptr<float>(), res, out.data_ptr(), rows,
                                               static_cast<int>(cols), current_stream()),
                 "dequantize_per_token");
    return out;
}

// In place: K, V int8 [B,H,S_cap,D] and sK, sV fp32 (numel B*H*S_cap) receive the new token at `pos`.
void kv_append_quantize_torch(torch::Tensor k_new, torch::Tensor v_new, torch::Tensor K, torch::Tensor V,
                              torch::Tensor sK, torch::Tensor sV, int64_t pos) {
    TORCH_CHECK(K.device().is_cuda() && K.dtype() == torch::kInt8 && V.dtype() == torch::kInt8 &&
                K.dim() == 4 && V.sizes() == K.sizes() && K.is_contiguous() && V.is_contiguous(),
                "K, V must be contiguous int8 [B,H,S_cap,D] CUDA tensors of one shape");
    const int64_t B = K.size(0), H = K.size(1), S_cap = K.size(2), D = K.size(3);
    TORCH_CHECK(k_new.dtype() == torch::kFloat16 && v_new.dtype() == torch::kFloat16 &&
                k_new.numel() == B * H * D && v_new.numel() == B * H * D,
                "k_new, v_new must be float16 with B*H*D elements");
    TORCH_CHECK(sK.dtype() == torch::kFloat32 && sV.dtype() == torch::kFloat32 && sK.is_contiguous() &&
                sV.is_contiguous() && sK.numel() == B * H * S_cap && sV.numel() == B * H * S_cap,
                "sK, sV must be contiguous float32 with B*H*S_cap elements");
    TORCH_CHECK(pos >= 0 && pos < S_cap, "position outside the cache");
    auto kn = k_new.contiguous(), vn = v_new.contiguous();
    c10::cuda::CUDAGuard guard(K.device());
    check_status(i8tk_kv_append_quantize_f16(kn.data_ptr(), vn.data_ptr(), K.data_ptr<int8_t>(), V.data_ptr<int8_t>(),
                                             sK.data_ptr<float>(), sV.data_ptr<float>(), nullptr,
                                             static_cast<int>(pos), static_cast<int>(B * H), static_cast<int>(S_cap),
                                             static_cast<int>(D), current_stream()),
                 "kv_append_quantize");
}

}  // namespace

#include "int8_ext_mlp.inc"

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("int8_attention_forward", &int8_attention_forward_torch,
          "INT8 attention with per-token quantization (CUDA) — returns FP16");
    m.def("int8_decode_attention_forward", &int8_decode_attention_forward_torch,
          "INT8 flash-decoding attention (seq_q==1, INT8 KV cache) — returns FP16");
    m.def("int8_decode_attention_forward_quantized", &int8_decode_attention_forward_quantized_torch,
          "INT8 flash-decoding attention whose output is quantised per token for the next INT8 GEMM — "
          "returns (int8 [B, H*D], fp32 scales [B])");
    m.def("int8_decode_attention_paged", &int8_decode_attention_paged_torch,
          "INT8 flash-decoding attention over a paged INT8 KV cache with per-request lengths — returns FP16");
    m.def("int8_decode_attention_partial", &int8_decode_attention_partial_torch,
          "INT8 decode attention over a KV shard — returns unnormalised (m, l, 0, 0, acc[D]) rows");
    m.def("int8_decode_combine_partials", &int8_decode_combine_partials_torch,
          "Log-sum-exp merge of gathered decode partials — returns FP16");
    m.def("quantize_per_token", &quantize_per_token_torch,
          "Per-token symmetric INT8 quantisation — returns (int8, fp32 scales)");
    m.def("layernorm_quantize", &layernorm_quantize_torch, pybind11::arg("t"), pybind11::arg("eps") = 1e-5,
          "LayerNorm (no affine) + per-token INT8 quantisation of the fp16 result — returns (int8, fp32 scales)");
    m.def("quantize_qkv_heads", &quantize_qkv_heads_torch,
          "Fused QKV projection -> per-token INT8 in head-major layout — returns (int8 [3,B,H,S,Dh], fp32 [3,B,H,S])");
    m.def("dequantize_per_token", &dequantize_per_token_torch, pybind11::arg("q"), pybind11::arg("scales"),
          pybind11::arg("residual") = c10::nullopt, "fp16(q * scale[row]) (+ residual) — returns FP16");
    m.def("kv_append_quantize", &kv_append_quantize_torch,
          "Quantise the new token's K and V rows per token and write them into the INT8 cache at pos (in place)");
    m.def("check_status", &check_status_torch,
          "Synchronise the streams the ops ran on and raise if a bounded device-side wait gave up since the last check");
    register_mlp_ops(m);
}
