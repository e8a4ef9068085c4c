// Native launchers with the reference's own C++ signatures, over the i8tk C ABI.
//
// The reference's kernels are reached from C++ through free functions with C++ linkage that
// take raw device pointers and ints and return void (kernels/int8_ext.cu:27-70 declares them
// for the torch binding; tests/cuda/test_int8.cu:15-26 links them without torch;
// kernels/int8_common.cuh:54-59 declares the per-tensor quantiser pair).  This file defines
// the same functions -- same names, same parameter lists, same linkage -- so that code written
// against the reference's objects links against libi8tk_compat.so unchanged.
//
// Conventions kept from the reference: launches go to the legacy default stream; scratch is
// owned by the library, one grow-only block per device, never freed
// (kernels/int8_decode_attention.cu:430-440, kernels/int8_mlp.cu:954-977); nothing is
// returned; an unsupported head_dim does nothing (kernels/int8_decode_attention.cu:546).
// Not kept: the reference checks no CUDA error at all.  Here the status of the last call
// made by the calling thread is remembered and can be read with i8tk_compat_last_status()
// (0 = success, otherwise an i8tk_status code; i8tk_last_error() has the text).
//
// Differences in reach: int8_mlp_forward_per_channel on widths the tensor-core path does
// not take sets the status to I8TK_ERR_UNSUPPORTED where the reference silently runs its
// static-scale fallback and leaves out_row_scales unwritten
// (kernels/int8_mlp.cu:1023-1026,1194-1225).
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <mutex>

#include "../../include/i8tk.h"

namespace {

thread_local int g_last_status = I8TK_OK;

// One grow-only scratch block per device (index = CUDA device ordinal).
struct DeviceScratch {
    void* ptr = nullptr;
    size_t bytes = 0;
    float* mlp_out_scale = nullptr;   // device float[1]: output scale of the last per-tensor MLP call
    bool have_scale = false;
};
constexpr int kMaxDevices = 64;
DeviceScratch g_scratch[kMaxDevices];
std::mutex g_scratch_mutex;

DeviceScratch* scratch_for(size_t bytes) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    DeviceScratch& s = g_scratch[dev];
    if (s.mlp_out_scale == nullptr) {
        if (cudaMalloc(reinterpret_cast<void**>(&s.mlp_out_scale), 256) != cudaSuccess) return nullptr;
    }
    if (s.bytes < bytes) {
        // earlier work that uses the old block was queued on the same (legacy default) stream;
        // cudaFree waits for it
        if (s.ptr) cudaFree(s.ptr);
        s.ptr = nullptr;
        s.bytes = 0;
        const size_t want = bytes + bytes / 4 + 256;
        if (cudaMalloc(&s.ptr, want) != cudaSuccess) return nullptr;
        cudaMemset(s.ptr, 0, 256);                 // status block starts clean
        s.bytes = want;
    }
    return &s;
}

void mlp_call(const int8_t* x, const int8_t* W1, const int8_t* W2, int8_t* out, const float* scale_x,
              const float* scale_W1, const float* scale_W2, const float* bias1, float* out_row_scales,
              int batch, int seq_len, int d_model, int d_ff, int flags) {
    const long long T = (long long)batch * seq_len;
    if (batch <= 0 || seq_len <= 0 || T > 0x7fffffffll) {
        g_last_status = I8TK_ERR_INVALID_ARGUMENT;
        return;
    }
    const size_t need = i8tk_mlp_workspace_bytes((int)T, d_model, d_ff, flags);
    DeviceScratch* s = scratch_for(need);
    if (s == nullptr) {
        g_last_status = I8TK_ERR_CUDA;
        return;
    }
    g_last_status = i8tk_mlp_forward(x, W1, W2, out, scale_x, scale_W1, scale_W2, bias1, out_row_scales,
                                     out_row_scales ? nullptr : s->mlp_out_scale, (int)T, d_model, d_ff, flags,
                                     s->ptr, s->bytes, nullptr);
    if (!out_row_scales && g_last_status == I8TK_OK) s->have_scale = true;
}

}  // namespace

extern "C" int i8tk_compat_last_status(void) { return g_last_status; }

void int8_attention_forward(const int8_t* Q, const int8_t* K, const int8_t* V, half* out,
                            const float* scale_Q, const float* scale_K, const float* scale_V,
                            int batch, int heads, int seq_len, int head_dim) {
    const size_t need = i8tk_attention_workspace_bytes(batch, heads, seq_len, head_dim);
    if (need == 0) {                              // shape or head_dim the kernels do not take
        g_last_status = I8TK_ERR_UNSUPPORTED;
        return;
    }
    DeviceScratch* s = scratch_for(need);
    if (s == nullptr) {
        g_last_status = I8TK_ERR_CUDA;
        return;
    }
    g_last_status = i8tk_attention_forward(Q, K, V, out, scale_Q, scale_K, scale_V, batch, heads, seq_len,
                                           head_dim, s->ptr, s->bytes, nullptr);
}

void int8_decode_attention_forward(const int8_t* Q, const int8_t* K, const int8_t* V, half* out,
                                   const float* scale_Q, const float* scale_K, const float* scale_V,
                                   int BH, int S, int head_dim) {
    const size_t need = i8tk_decode_workspace_bytes(BH, S, head_dim);
    if (need == 0) {
        g_last_status = I8TK_ERR_UNSUPPORTED;
        return;
    }
    DeviceScratch* s = scratch_for(need);
    if (s == nullptr) {
        g_last_status = I8TK_ERR_CUDA;
        return;
    }
    g_last_status = i8tk_decode_attention_forward(Q, K, V, out, scale_Q, scale_K, scale_V, BH, S, head_dim,
                                                  s->ptr, s->bytes, nullptr);
}

void int8_mlp_forward(const int8_t* x, const int8_t* W1, const int8_t* W2, int8_t* out,
                      const float* scale_x, const float* scale_W1, const float* scale_W2,
                      int batch, int seq_len, int d_model, int d_ff) {
    mlp_call(x, W1, W2, out, scale_x, scale_W1, scale_W2, nullptr, nullptr, batch, seq_len, d_model, d_ff, 0);
}

void int8_mlp_forward_per_channel(const int8_t* x, const int8_t* W1, const int8_t* W2, int8_t* out,
                                  const float* scale_x, const float* scale_W1, const float* scale_W2,
                                  float* out_row_scales, int batch, int seq_len, int d_model, int d_ff) {
    mlp_call(x, W1, W2, out, scale_x, scale_W1, scale_W2, nullptr, out_row_scales, batch, seq_len, d_model, d_ff,
             I8TK_MLP_X_PER_TOKEN | I8TK_MLP_W_PER_CHANNEL);
}

void int8_mlp_forward_per_channel_bias(const int8_t* x, const int8_t* W1, const int8_t* W2, int8_t* out,
                                       const float* scale_x, const float* scale_W1, const float* scale_W2,
                                       const float* gemm1_bias, float* out_row_scales, int batch, int seq_len,
                                       int d_model, int d_ff) {
    mlp_call(x, W1, W2, out, scale_x, scale_W1, scale_W2, gemm1_bias, out_row_scales, batch, seq_len, d_model, d_ff,
             I8TK_MLP_X_PER_TOKEN | I8TK_MLP_W_PER_CHANNEL);
}

void transpose_int8_weights(const int8_t* W1, const int8_t* W2, int8_t* W1T, int8_t* W2T, int d_model, int d_ff) {
    g_last_status = i8tk_transpose_int8_weights(W1, W2, W1T, W2T, d_model, d_ff, nullptr);
}

void int8_mlp_forward_prepacked(const int8_t* x, const int8_t* W1T, const int8_t* W2T, int8_t* out,
                                const float* scale_x, const float* scale_W1, const float* scale_W2,
                                int batch, int seq_len, int d_model, int d_ff) {
    mlp_call(x, W1T, W2T, out, scale_x, scale_W1, scale_W2, nullptr, nullptr, batch, seq_len, d_model, d_ff,
             I8TK_MLP_PREPACKED);
}

// Output scale of the most recent per-tensor MLP call on the current device; 1.0 before any
// (kernels/int8_mlp.cu:1317-1322).  Blocks on a device-to-host copy, as the reference does.
void int8_mlp_get_output_scale(float* host_out) {
    int dev = 0;
    if (host_out == nullptr) return;
    *host_out = 1.f;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return;
    DeviceScratch& s = g_scratch[dev];
    if (s.have_scale && s.mlp_out_scale)
        g_last_status = cudaMemcpy(host_out, s.mlp_out_scale, sizeof(float), cudaMemcpyDeviceToHost) == cudaSuccess
                            ? I8TK_OK : I8TK_ERR_CUDA;
}

void quantize_fp16_to_int8(const half* input, int8_t* output, float* d_scale, int n) {
    g_last_status = i8tk_quantize_fp16_to_int8(input, output, d_scale, n, nullptr);
}

void dequantize_int8_to_fp16(const int8_t* input, half* output, float scale, int n) {
    g_last_status = i8tk_dequantize_int8_to_fp16(input, output, scale, n, nullptr);
}
