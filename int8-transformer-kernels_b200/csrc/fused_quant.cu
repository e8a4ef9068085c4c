// Producer-side quantisation: the two steps either side of the INT8 path that the reference
// leaves to eager torch code and names as its largest remaining cost
// (OPTIMIZATION.md:241-246, bench/bench_block.py:107-151).
//
// * layernorm_quantize: LayerNorm (no affine, eps 1e-5, as F.layer_norm(x, (d,)) in
//   bench/bench_block.py:93-94) of an fp16 row, rounded to fp16 as torch stores it, then the
//   per-token quantiser's arithmetic (tests/test_int8.py:47-63) on that value -- one pass over
//   the row instead of LayerNorm + abs/amax/div/round/clamp/cast kernels.  Rows up to 2048 wide
//   take the code as round(x * (1/scale)) in one FMA (see quant4_fma2); wider rows divide.
// * kv_append_quantize: the new token's K and V rows ([B*H, D], fp16) quantised per token and
//   written straight into the INT8 cache at their position, with their scales -- quantise on
//   write, no intermediate tensors.
#include "common.cuh"

namespace i8tk {
namespace {

// packed fp32 pairs in their inline-PTX form here (see asm2 in common.cuh)
using f32x2 = asm2::f32x2;
using asm2::add2;
using asm2::fma2;
using asm2::mul2;
using asm2::pack2;
using asm2::unpack2;

__device__ __forceinline__ int quant_exact(float x, float scale) {
    // true division + round-half-even + clamp, exactly as torch does on fp32
    const float r = rintf(__fdiv_rn(x, scale));
    return (int)fminf(fmaxf(r, -128.f), 127.f);
}

constexpr int kLnThreads = 128;
constexpr int kLnMaxVec = 4;          // 16-byte vectors per thread: d_model <= 128 * 4 * 8 = 4096

__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int w = threadIdx.x >> 5;
    __syncthreads();                                  // red[] free again
    if ((threadIdx.x & 31) == 0) red[w] = v;
    __syncthreads();
    return red[0] + red[1] + red[2] + red[3];
}
__device__ __forceinline__ float block_max(float v, float* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    const int w = threadIdx.x >> 5;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[w] = v;
    __syncthreads();
    return fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
}

// Rows wider than 2048: one CTA per row; the row lives in registers between the three reductions.
__global__ void __launch_bounds__(kLnThreads)
layernorm_quantize_kernel(const __half* __restrict__ x, int8_t* __restrict__ q, float* __restrict__ scales,
                          int d, float eps) {
    __shared__ float red[4];
    const long long row = blockIdx.x;
    const int nvec = d / 8;
    const __half* xr = x + row * d;
    float v[kLnMaxVec][8];
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < kLnMaxVec; ++j) {
        const int vi = threadIdx.x + j * kLnThreads;
        if (vi < nvec) {
            const uint4 t = *reinterpret_cast<const uint4*>(xr + vi * 8);
            const __half2* h = reinterpret_cast<const __half2*>(&t);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __half22float2(h[i]);
                v[j][2 * i] = f.x;
                v[j][2 * i + 1] = f.y;
                sum += f.x + f.y;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[j][i] = 0.f;
        }
    }
    const float mean = block_sum(sum, red) / (float)d;
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < kLnMaxVec; ++j) {
        if (threadIdx.x + j * kLnThreads < nvec) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float c = v[j][i] - mean;
                ss = fmaf(c, c, ss);
            }
        }
    }
    const float rstd = rsqrtf(block_sum(ss, red) / (float)d + eps);
    // normalised value as torch stores it (fp16), which is what the quantiser sees
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < kLnMaxVec; ++j) {
        if (threadIdx.x + j * kLnThreads < nvec) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                v[j][i] = __half2float(__float2half_rn((v[j][i] - mean) * rstd));
                amax = fmaxf(amax, fabsf(v[j][i]));
            }
        }
    }
    amax = block_max(amax, red);
    const float scale = __fdiv_rn(fmaxf(amax, 1e-8f), 127.0f);
    if (threadIdx.x == 0) scales[row] = scale;
    int8_t* qr = q + row * d;
#pragma unroll
    for (int j = 0; j < kLnMaxVec; ++j) {
        const int vi = threadIdx.x + j * kLnThreads;
        if (vi < nvec) {
            uint32_t w[2];
#pragma unroll
            for (int k = 0; k < 2; ++k)
                w[k] = (uint32_t)(quant_exact(v[j][4 * k], scale) & 0xff) |
                       ((uint32_t)(quant_exact(v[j][4 * k + 1], scale) & 0xff) << 8) |
                       ((uint32_t)(quant_exact(v[j][4 * k + 2], scale) & 0xff) << 16) |
                       ((uint32_t)(quant_exact(v[j][4 * k + 3], scale) & 0xff) << 24);
            *reinterpret_cast<uint2*>(qr + vi * 8) = make_uint2(w[0], w[1]);
        }
    }
}

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max_f(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Four codes from two packed pairs: code = low byte of fma(x, 1/scale, 1.5 * 2^23), one rounding.
// No tie test here (the plain quantiser has one and is bit-exact): x * (1/scale) is within 1.6e-5
// of the exact quotient, so a code can differ from the divide-then-round result only for
// quotients that close to k + 0.5, about 3e-5 of all elements, while the normalised value itself
// differs from torch's in its last bit far more often than that.
__device__ __forceinline__ uint32_t quant4_fma2(f32x2 a, f32x2 b, f32x2 rcp2) {
    const f32x2 magic2 = pack2(12582912.f, 12582912.f);
    const float2 fa = unpack2(fma2(a, rcp2, magic2)), fb = unpack2(fma2(b, rcp2, magic2));
    return prmt(prmt(__float_as_uint(fa.x), __float_as_uint(fa.y), 0x0040u),
                prmt(__float_as_uint(fb.x), __float_as_uint(fb.y), 0x0040u), 0x5410u);
}

// One warp per row, the row in registers (NV 16-byte vectors per lane) as packed fp32 pairs, so
// the sums, the centring, the scaling and the quotient all run as fp32x2 instructions: d <= 256 * NV.
// No shared memory and no block-wide barrier; a block of eight warps walks rows grid-stride.
template <int NV>
__global__ void __launch_bounds__(256, (NV <= 4) ? 4 : 2)
layernorm_quantize_warp_kernel(const __half* __restrict__ x, int8_t* __restrict__ q, float* __restrict__ scales,
                               long long rows, int d, float eps) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int nvec = d / 8;
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    const float inv_d = 1.0f / (float)d;
    // the raw vectors of the warp's next row are requested as soon as those of the current row
    // have been unpacked, so a load is in flight during the three reductions of every row --
    // except at NV == 4, where the extra registers would cost a resident block per SM (measured:
    // no gain on long inputs, 15 % slower on short ones)
    constexpr bool kPrefetch = NV != 4;
    uint4 t[NV];
    auto fetch = [&](long long r) {
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const int vi = lane + j * 32;
            t[j] = make_uint4(0u, 0u, 0u, 0u);
            if (r < rows && vi < nvec) t[j] = *reinterpret_cast<const uint4*>(x + r * d + vi * 8);
        }
    };
    if constexpr (kPrefetch) fetch(warp);
    for (long long row = warp; row < rows; row += nwarps) {
        if constexpr (!kPrefetch) fetch(row);
        f32x2 v[NV][4];
        f32x2 sum2 = pack2(0.f, 0.f);
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const __half2* h = reinterpret_cast<const __half2*>(&t[j]);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __half22float2(h[i]);
                v[j][i] = pack2(f.x, f.y);
                sum2 = add2(sum2, v[j][i]);
            }
        }
        if constexpr (kPrefetch) fetch(row + nwarps);
        const float2 s2 = unpack2(sum2);
        const float mean = warp_sum_f(s2.x + s2.y) * inv_d;
        const f32x2 nmean2 = pack2(-mean, -mean);
        f32x2 ss2 = pack2(0.f, 0.f);
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            if (lane + j * 32 < nvec) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    v[j][i] = add2(v[j][i], nmean2);          // centred from here on
                    ss2 = fma2(v[j][i], v[j][i], ss2);
                }
            }
        }
        const float2 q2 = unpack2(ss2);
        const float rstd = rsqrtf(warp_sum_f(q2.x + q2.y) * inv_d + eps);
        // normalised value as torch stores it (fp16); its maximum is exact in fp16
        const f32x2 rstd2 = pack2(rstd, rstd);
        __half2 hmax = __floats2half2_rn(0.f, 0.f);
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            if (lane + j * 32 < nvec) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 n = unpack2(mul2(v[j][i], rstd2));
                    const __half2 hy = __floats2half2_rn(n.x, n.y);
                    hmax = __hmax2(hmax, __habs2(hy));
                    const float2 back = __half22float2(hy);
                    v[j][i] = pack2(back.x, back.y);
                }
            }
        }
        const float2 hm = __half22float2(hmax);
        const float amax = warp_max_f(fmaxf(hm.x, hm.y));
        const float scale = __fdiv_rn(fmaxf(amax, 1e-8f), 127.0f);
        const float rcp = __frcp_rn(scale);
        const f32x2 rcp2 = pack2(rcp, rcp);
        if (lane == 0) scales[row] = scale;
        int8_t* qr = q + row * d;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const int vi = lane + j * 32;
            if (vi < nvec)
                *reinterpret_cast<uint2*>(qr + vi * 8) = make_uint2(quant4_fma2(v[j][0], v[j][1], rcp2),
                                                                    quant4_fma2(v[j][2], v[j][3], rcp2));
        }
    }
}

// One warp per (tensor, b*h) row of D fp16 values (D a multiple of 32, <= 256).
__global__ void __launch_bounds__(128)
kv_append_quantize_kernel(const __half* __restrict__ k_new, const __half* __restrict__ v_new,
                          int8_t* __restrict__ K, int8_t* __restrict__ V, float* __restrict__ sK,
                          float* __restrict__ sV, const int* __restrict__ pos_per_row, int pos0, int BH,
                          int S_cap, int D) {
    const int warp = blockIdx.x * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (warp >= 2 * BH) return;
    const bool is_v = warp >= BH;
    const int bh = is_v ? warp - BH : warp;
    const __half* src = (is_v ? v_new : k_new) + (size_t)bh * D;
    const int pos = pos_per_row ? pos_per_row[bh] : pos0;
    if (pos < 0 || pos >= S_cap) return;                   // out of the cache: nothing is written
    constexpr int kMaxPerLane = 8;
    const int per_lane = D / 32;
    float x[kMaxPerLane];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
        x[i] = (i < per_lane) ? __half2float(src[lane * per_lane + i]) : 0.f;
        amax = fmaxf(amax, fabsf(x[i]));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float scale = __fdiv_rn(fmaxf(amax, 1e-8f), 127.0f);
    int8_t* dst = (is_v ? V : K) + ((size_t)bh * S_cap + pos) * D + lane * per_lane;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i)
        if (i < per_lane) dst[i] = (int8_t)quant_exact(x[i], scale);
    if (lane == 0) (is_v ? sV : sK)[(size_t)bh * S_cap + pos] = scale;
}

}  // namespace
}  // namespace i8tk

using namespace i8tk;

extern "C" int i8tk_layernorm_quantize_f16(const void* x_f16, int8_t* q, float* scales, int64_t rows,
                                           int d_model, float eps, i8tk_stream_t stream) {
    I8TK_REQUIRE(rows >= 0 && d_model >= 8, I8TK_ERR_INVALID_ARGUMENT, "rows must be >= 0 and d_model >= 8");
    if (rows == 0) return I8TK_OK;
    I8TK_REQUIRE(x_f16 && q && scales, I8TK_ERR_INVALID_ARGUMENT, "null pointer argument");
    I8TK_REQUIRE(d_model % 8 == 0 && d_model <= kLnThreads * kLnMaxVec * 8, I8TK_ERR_UNSUPPORTED,
                 "d_model must be a multiple of 8 and at most %d (got %d)", kLnThreads * kLnMaxVec * 8, d_model);
    I8TK_REQUIRE(rows < (1ll << 31), I8TK_ERR_UNSUPPORTED, "too many rows");
    I8TK_REQUIRE(aligned_to(x_f16, 16) && aligned_to(q, 8), I8TK_ERR_ALIGNMENT,
                 "x must be 16-byte and q 8-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const __half* xh = static_cast<const __half*>(x_f16);
    const int nvec = d_model / 8;
    long long blocks = (rows + 7) / 8;                    // eight warps (rows) per block
    if (blocks > 148ll * 16) blocks = 148ll * 16;
    if (nvec <= 32)
        I8TK_CUDA(launch_after(layernorm_quantize_warp_kernel<1>, dim3((unsigned)blocks), dim3(256), 0, st, xh, q, scales,
                               (long long)rows, d_model, eps));
    else if (nvec <= 64)
        I8TK_CUDA(launch_after(layernorm_quantize_warp_kernel<2>, dim3((unsigned)blocks), dim3(256), 0, st, xh, q, scales,
                               (long long)rows, d_model, eps));
    else if (nvec <= 128)
        I8TK_CUDA(launch_after(layernorm_quantize_warp_kernel<4>, dim3((unsigned)blocks), dim3(256), 0, st, xh, q, scales,
                               (long long)rows, d_model, eps));
    else if (nvec <= 256)
        I8TK_CUDA(launch_after(layernorm_quantize_warp_kernel<8>, dim3((unsigned)blocks), dim3(256), 0, st, xh, q, scales,
                               (long long)rows, d_model, eps));
    else                                                  // wider rows: one block per row
        layernorm_quantize_kernel<<<(unsigned)rows, kLnThreads, 0, st>>>(xh, q, scales, d_model, eps);
    I8TK_CUDA(cudaGetLastError());
    return I8TK_OK;
}

extern "C" int i8tk_kv_append_quantize_f16(const void* k_new_f16, const void* v_new_f16, int8_t* K, int8_t* V,
                                           float* sK, float* sV, const int32_t* pos_per_row, int pos,
                                           int BH, int S_cap, int head_dim, i8tk_stream_t stream) {
    I8TK_REQUIRE(k_new_f16 && v_new_f16 && K && V && sK && sV, I8TK_ERR_INVALID_ARGUMENT, "null pointer argument");
    I8TK_REQUIRE(BH > 0 && S_cap > 0, I8TK_ERR_INVALID_ARGUMENT, "sizes must be positive");
    I8TK_REQUIRE(head_dim % 32 == 0 && head_dim >= 32 && head_dim <= 256, I8TK_ERR_UNSUPPORTED,
                 "head_dim must be a multiple of 32 in [32, 256] (got %d)", head_dim);
    I8TK_REQUIRE(pos_per_row || (pos >= 0 && pos < S_cap), I8TK_ERR_INVALID_ARGUMENT,
                 "position %d outside the cache of %d positions", pos, S_cap);
    kv_append_quantize_kernel<<<(2 * BH + 3) / 4, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(k_new_f16), static_cast<const __half*>(v_new_f16), K, V, sK, sV, pos_per_row,
        pos, BH, S_cap, head_dim);
    I8TK_CUDA(cudaGetLastError());
    return I8TK_OK;
}
