// extern "C" doors onto the reference project's own CUDA launchers, so that the
// GPU tests and the benchmark can run the UNMODIFIED reference kernels beside the
// new ones.  This file holds no kernel and no arithmetic; it is compiled together
// with the reference's kernels/*.cu where they lie (oracle/build_ref.py) into
// oracle/_ref/libref_kernels.so.  Test infrastructure only.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>

// declarations as in the reference's kernels/int8_ext.cu:27-70
void int8_decode_attention_forward(const int8_t* Q, const int8_t* K, const int8_t* V, half* out,
                                   const float* scale_Q, const float* scale_K, const float* scale_V,
                                   int BH, int S, int head_dim);
void int8_mlp_forward_per_channel_bias(const int8_t* x, const int8_t* W1, const int8_t* W2, int8_t* out,
                                       const float* scale_x, const float* scale_W1, const float* scale_W2,
                                       const float* gemm1_bias, float* out_row_scales,
                                       int batch, int seq_len, int d_model, int d_ff);
void int8_mlp_forward_prepacked(const int8_t* x, const int8_t* W1T, const int8_t* W2T, int8_t* out,
                                const float* scale_x, const float* scale_W1, const float* scale_W2,
                                int batch, int seq_len, int d_model, int d_ff);
void int8_mlp_get_output_scale(float* host_out);
void int8_attention_forward(const int8_t* Q, const int8_t* K, const int8_t* V, half* out,
                            const float* scale_Q, const float* scale_K, const float* scale_V,
                            int batch, int heads, int seq_len, int head_dim);

extern "C" int ref_decode_attention_forward(const int8_t* Q, const int8_t* K, const int8_t* V, void* out,
                                            const float* sQ, const float* sK, const float* sV,
                                            int BH, int S, int head_dim) {
    int8_decode_attention_forward(Q, K, V, static_cast<half*>(out), sQ, sK, sV, BH, S, head_dim);
    return (int)cudaGetLastError();
}

extern "C" int ref_mlp_forward_per_channel_bias(const int8_t* x, const int8_t* W1, const int8_t* W2,
                                                int8_t* out, const float* sx, const float* sW1,
                                                const float* sW2, const float* bias1, float* out_row_scales,
                                                int batch, int seq_len, int d_model, int d_ff) {
    int8_mlp_forward_per_channel_bias(x, W1, W2, out, sx, sW1, sW2, bias1, out_row_scales, batch, seq_len,
                                      d_model, d_ff);
    return (int)cudaGetLastError();
}

extern "C" int ref_mlp_forward_prepacked(const int8_t* x, const int8_t* W1T, const int8_t* W2T, int8_t* out,
                                         const float* sx, const float* sW1, const float* sW2, int batch,
                                         int seq_len, int d_model, int d_ff) {
    int8_mlp_forward_prepacked(x, W1T, W2T, out, sx, sW1, sW2, batch, seq_len, d_model, d_ff);
    return (int)cudaGetLastError();
}

extern "C" float ref_mlp_get_output_scale(void) {
    float s = 0.f;
    int8_mlp_get_output_scale(&s);
    return s;
}

extern "C" int ref_attention_forward(const int8_t* Q, const int8_t* K, const int8_t* V, void* out,
                                     const float* sQ, const float* sK, const float* sV, int batch, int heads,
                                     int seq_len, int head_dim) {
    int8_attention_forward(Q, K, V, static_cast<half*>(out), sQ, sK, sV, batch, heads, seq_len, head_dim);
    return (int)cudaGetLastError();
}
