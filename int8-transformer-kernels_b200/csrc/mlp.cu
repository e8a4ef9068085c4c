// Fused INT8 MLP (placeholder while the tcgen05 GEMM is brought up).
#include "common.cuh"

namespace i8tk {
namespace {

// int8 [R][C] -> [C][R]; 64x64 tiles, 4-byte global accesses on both sides.
__global__ void __launch_bounds__(256)
transpose_i8_kernel(const int8_t* __restrict__ in, int8_t* __restrict__ out, int R, int C) {
    __shared__ int8_t tile[64][68];
    const int c0 = blockIdx.x * 64, r0 = blockIdx.y * 64;
    for (int i = threadIdx.x; i < 64 * 16; i += 256) {
        const int r = i / 16, c4 = (i % 16) * 4;
        if (r0 + r < R) {
            if (c0 + c4 + 3 < C && (C % 4) == 0) {
                const uint32_t w = *reinterpret_cast<const uint32_t*>(in + (size_t)(r0 + r) * C + c0 + c4);
                tile[r][c4] = (int8_t)(w & 0xff); tile[r][c4 + 1] = (int8_t)((w >> 8) & 0xff);
                tile[r][c4 + 2] = (int8_t)((w >> 16) & 0xff); tile[r][c4 + 3] = (int8_t)(w >> 24);
            } else {
                for (int e = 0; e < 4; ++e)
                    if (c0 + c4 + e < C) tile[r][c4 + e] = in[(size_t)(r0 + r) * C + c0 + c4 + e];
            }
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 64 * 16; i += 256) {
        const int c = i / 16, r4 = (i % 16) * 4;      // output row c0+c, cols r0+r4..
        if (c0 + c < C) {
            if (r0 + r4 + 3 < R && (R % 4) == 0) {
                const uint32_t w = (uint32_t)(uint8_t)tile[r4][c] | ((uint32_t)(uint8_t)tile[r4 + 1][c] << 8) |
                                   ((uint32_t)(uint8_t)tile[r4 + 2][c] << 16) | ((uint32_t)(uint8_t)tile[r4 + 3][c] << 24);
                *reinterpret_cast<uint32_t*>(out + (size_t)(c0 + c) * R + r0 + r4) = w;
            } else {
                for (int e = 0; e < 4; ++e)
                    if (r0 + r4 + e < R) out[(size_t)(c0 + c) * R + r0 + r4 + e] = tile[r4 + e][c];
            }
        }
    }
}

}  // namespace

int transpose_i8(const int8_t* in, int8_t* out, int R, int C, cudaStream_t st) {
    dim3 grid((C + 63) / 64, (R + 63) / 64);
    transpose_i8_kernel<<<grid, 256, 0, st>>>(in, out, R, C);
    I8TK_CUDA(cudaGetLastError());
    return I8TK_OK;
}

}  // namespace i8tk

using namespace i8tk;

extern "C" int i8tk_transpose_int8_weights(const int8_t* W1, const int8_t* W2, int8_t* W1T,
                                           int8_t* W2T, int d_model, int d_ff, i8tk_stream_t stream) {
    I8TK_REQUIRE(W1 && W2 && W1T && W2T, I8TK_ERR_INVALID_ARGUMENT, "null pointer argument");
    I8TK_REQUIRE(d_model > 0 && d_ff > 0, I8TK_ERR_INVALID_ARGUMENT, "d_model and d_ff must be positive");
    I8TK_REQUIRE(aligned_to(W1, 4) && aligned_to(W2, 4) && aligned_to(W1T, 4) && aligned_to(W2T, 4),
                 I8TK_ERR_ALIGNMENT, "weights must be 4-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int rc = transpose_i8(W1, W1T, d_model, d_ff, st);
    if (rc != I8TK_OK) return rc;
    return transpose_i8(W2, W2T, d_ff, d_model, st);
}

extern "C" size_t i8tk_mlp_workspace_bytes(int T, int d_model, int d_ff, int flags) {
    (void)T; (void)d_model; (void)d_ff; (void)flags;
    return 0;
}

extern "C" int i8tk_mlp_forward(const int8_t*, const int8_t*, const int8_t*, int8_t*, const float*,
                                const float*, const float*, const float*, float*, float*, int, int,
                                int, int, void*, size_t, i8tk_stream_t) {
    set_error("i8tk_mlp_forward is not built in this snapshot");
    return I8TK_ERR_UNSUPPORTED;
}
