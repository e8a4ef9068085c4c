/*
 * i8tk_compat.h -- the reference's own native launchers, provided by libi8tk_compat.so.
 *
 * C++ linkage, raw device pointers and ints, void return, legacy default stream,
 * library-owned scratch: exactly the functions kernels/int8_ext.cu:27-70 forward-declares
 * (and tests/cuda/test_int8.cu:15-26 links without torch), plus the per-tensor quantiser
 * pair of kernels/int8_common.cuh:54-59.  A translation unit written against the
 * reference's objects links against libi8tk_compat.so (which needs libi8tk.so) unchanged;
 * new code should prefer the C ABI in i8tk.h (explicit stream, caller-owned workspace,
 * status codes).
 *
 * The reference checks no error.  Here every launcher records the status of the call in a
 * thread-local that i8tk_compat_last_status() returns (0 = success, otherwise an
 * i8tk_status code; i8tk_last_error() has the text).
 */
#ifndef I8TK_COMPAT_H_
#define I8TK_COMPAT_H_

#include <cuda_fp16.h>
#include <stdint.h>

#ifndef __cplusplus
#error "the compat launchers have C++ linkage, as the reference's do"
#endif

/* kernels/int8_ext.cu:28-32 -- prefill attention, per-token scales [batch*heads*seq_len]. */
void int8_attention_forward(const int8_t* Q, const int8_t* K, const int8_t* V, half* out,
                            const float* scale_Q, const float* scale_K, const float* scale_V,
                            int batch, int heads, int seq_len, int head_dim);

/* kernels/int8_ext.cu:34-38 -- decode attention; head_dim outside {64,128} does nothing. */
void int8_decode_attention_forward(const int8_t* Q, const int8_t* K, const int8_t* V, half* out,
                                   const float* scale_Q, const float* scale_K, const float* scale_V,
                                   int BH, int S, int head_dim);

/* kernels/int8_ext.cu:40-44 -- per-tensor scales (device float[1] each), dynamic per-tensor
 * output scale kept by the library: read it with int8_mlp_get_output_scale. */
void int8_mlp_forward(const int8_t* x, const int8_t* W1, const int8_t* W2, int8_t* out,
                      const float* scale_x, const float* scale_W1, const float* scale_W2,
                      int batch, int seq_len, int d_model, int d_ff);

/* kernels/int8_ext.cu:46-51 -- scale_x [T], scale_W1 [d_ff], scale_W2 [d_model]; out_row_scales [T]. */
void int8_mlp_forward_per_channel(const int8_t* x, const int8_t* W1, const int8_t* W2, int8_t* out,
                                  const float* scale_x, const float* scale_W1, const float* scale_W2,
                                  float* out_row_scales, int batch, int seq_len, int d_model, int d_ff);

/* kernels/int8_ext.cu:53-58 -- the same with a pre-GELU bias [d_ff] (may be NULL). */
void int8_mlp_forward_per_channel_bias(const int8_t* x, const int8_t* W1, const int8_t* W2, int8_t* out,
                                       const float* scale_x, const float* scale_W1, const float* scale_W2,
                                       const float* gemm1_bias, float* out_row_scales, int batch, int seq_len,
                                       int d_model, int d_ff);

/* kernels/int8_ext.cu:60-63 -- W1 [d_model,d_ff] -> W1T [d_ff,d_model], W2 likewise. */
void transpose_int8_weights(const int8_t* W1, const int8_t* W2, int8_t* W1T, int8_t* W2T, int d_model, int d_ff);

/* kernels/int8_ext.cu:65-69 -- int8_mlp_forward on weights transposed once by the call above. */
void int8_mlp_forward_prepacked(const int8_t* x, const int8_t* W1T, const int8_t* W2T, int8_t* out,
                                const float* scale_x, const float* scale_W1, const float* scale_W2,
                                int batch, int seq_len, int d_model, int d_ff);

/* kernels/int8_ext.cu:71, kernels/int8_mlp.cu:1317-1322 -- output scale of the most recent
 * per-tensor MLP call on the current device (1.0 before any); blocks on a device-to-host copy. */
void int8_mlp_get_output_scale(float* host_out);

/* kernels/int8_common.cuh:54-59, kernels/quant_utils.cu:57-77 -- per-tensor FP16 <-> INT8. */
void quantize_fp16_to_int8(const half* input, int8_t* output, float* d_scale, int n);
void dequantize_int8_to_fp16(const int8_t* input, half* output, float scale, int n);

/* Status of the last launcher call made by this thread.  No counterpart in the reference. */
extern "C" int i8tk_compat_last_status(void);

#endif  /* I8TK_COMPAT_H_ */
