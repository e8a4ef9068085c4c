// Per-token (row-wise) and per-tensor symmetric INT8 quantisers.
//
// Per token: bit-identical to the torch code the reference uses to feed its
// kernels (tests/test_int8.py:47-63 == validation/validate_int8.py:63-66):
//   absmax = max(|x|.amax(-1), 1e-8);  scale = absmax / 127   (fp32 IEEE division)
//   q = clamp(round_half_even(x / scale), -128, 127)          (fp32 IEEE division)
// Per tensor: kernels/quant_utils.cu:12-77 (absmax -> /127 -> rne(x/scale)).
//
// HBM-bound streaming kernels: 16-byte loads, several independent rows in
// flight per lane group, absmax by warp shuffles, no shared memory.
#include "common.cuh"

namespace i8tk {
namespace {

template <typename T> struct Vec16;          // 16 bytes of input elements, kept as loaded
template <> struct Vec16<float> {
    static constexpr int N = 4;
    __device__ static uint4 load(const float* p) { return *reinterpret_cast<const uint4*>(p); }
    __device__ static float absmax(const uint4& t) {
        return fmaxf(fmaxf(fabsf(__uint_as_float(t.x)), fabsf(__uint_as_float(t.y))),
                     fmaxf(fabsf(__uint_as_float(t.z)), fabsf(__uint_as_float(t.w))));
    }
    __device__ static void to_float(const uint4& t, float (&v)[4]) {
        v[0] = __uint_as_float(t.x); v[1] = __uint_as_float(t.y);
        v[2] = __uint_as_float(t.z); v[3] = __uint_as_float(t.w);
    }
};
template <> struct Vec16<__half> {
    static constexpr int N = 8;
    __device__ static uint4 load(const __half* p) { return *reinterpret_cast<const uint4*>(p); }
    // the maximum of fp16 values is exact in fp16: reduce as packed halves, convert once
    __device__ static float absmax(const uint4& t) {
        const __half2* h = reinterpret_cast<const __half2*>(&t);
        const __half2 m = __hmax2(__hmax2(__habs2(h[0]), __habs2(h[1])), __hmax2(__habs2(h[2]), __habs2(h[3])));
        const float2 f = __half22float2(m);
        return fmaxf(f.x, f.y);
    }
    __device__ static void to_float(const uint4& t, float (&v)[8]) {
        const __half2* h = reinterpret_cast<const __half2*>(&t);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(h[i]);
            v[2 * i] = f.x; v[2 * i + 1] = f.y;
        }
    }
};

__device__ __forceinline__ int quant1(float x, float scale) {
    // true division + round-half-even + clamp, exactly as torch does on fp32
    const float r = rintf(__fdiv_rn(x, scale));
    return (int)fminf(fmaxf(r, -128.f), 127.f);
}

__device__ __forceinline__ uint32_t pack4(int a, int b, int c, int d) {
    return (uint32_t)(a & 0xff) | ((uint32_t)(b & 0xff) << 8) | ((uint32_t)(c & 0xff) << 16) |
           ((uint32_t)(d & 0xff) << 24);
}

// Four codes with the division amortised over the row, bit-identical to quant1.
// `rcp` is the correctly rounded 1/scale, so x * rcp is within 2^-23 (relative) of the exact
// quotient, i.e. within 1.6e-5 of it for |quotient| <= 128, and the IEEE quotient is within
// 0.8e-5: the two can only round to different codes when x * rcp lies within 2.4e-5 of a
// rounding tie.  Quotients within 1e-4 of a tie (about 0.02 % of elements) are therefore redone
// with the IEEE division and the rest need nothing more than the multiply.  Rounding to nearest
// even is the addition of 1.5 * 2^23, which leaves the code in the low byte of the sum (product
// and addition are one FMA; the distance from a tie is a second FMA of the same product with
// minus the code);
// |x / scale| <= 127 by construction of the scale, so no clamp is needed.  Packed fp32x2
// arithmetic throughout: no conversion or rounding instruction (those run at a quarter of the
// FMA rate).
__device__ __forceinline__ uint32_t quant4(float x0, float x1, float x2, float x3, float scale, float rcp) {
    const f32x2 rcp2 = pack2(rcp, rcp);
    const f32x2 magic2 = pack2(12582912.f, 12582912.f);
    const f32x2 mone2 = pack2(-1.f, -1.f);
    const f32x2 xa = pack2(x0, x1), xb = pack2(x2, x3);
    const f32x2 ra = fma2(xa, rcp2, magic2), rb = fma2(xb, rcp2, magic2);     // low byte = code n
    // distance of the quotient from that code: x * rcp - n, with -n = magic - r (exact)
    const float2 da = unpack2(fma2(xa, rcp2, fma2(ra, mone2, magic2)));
    const float2 db = unpack2(fma2(xb, rcp2, fma2(rb, mone2, magic2)));
    const float2 fa = unpack2(ra), fb = unpack2(rb);
    uint32_t w = prmt(prmt(__float_as_uint(fa.x), __float_as_uint(fa.y), 0x0040u),
                      prmt(__float_as_uint(fb.x), __float_as_uint(fb.y), 0x0040u), 0x5410u);
    if (max3(max3(fabsf(da.x), fabsf(da.y), fabsf(db.x)), fabsf(db.y), 0.f) > 0.4999f)
        w = pack4(quant1(x0, scale), quant1(x1, scale), quant1(x2, scale), quant1(x3, scale));
    return w;
}

// Maxima of R rows, each spread over the G lanes of a group, reduced so that every lane ends
// up with the complete maximum of ONE row (*rsel): the first log2(R) butterfly steps halve the
// number of rows a lane carries instead of carrying all R through every step
// (3 + log2(G/4) shuffles for R = 4 instead of 4 * log2(G)).  Needs R <= G.
template <int G, int R>
__device__ __forceinline__ float reduce_rows(const float (&a)[R], int lane_in_group, int* rsel) {
    static_assert(R == 1 || R == 2 || R == 4, "row batch of 1, 2 or 4");
    static_assert(R <= G, "more rows than lanes in a group");
    float c;
    int sel = 0;
    int o = G / 2;
    if constexpr (R == 4) {
        const bool hi = (lane_in_group & o) != 0;
        const float r0 = __shfl_xor_sync(0xffffffffu, hi ? a[0] : a[2], o);
        const float r1 = __shfl_xor_sync(0xffffffffu, hi ? a[1] : a[3], o);
        const float b0 = fmaxf(hi ? a[2] : a[0], r0);
        const float b1 = fmaxf(hi ? a[3] : a[1], r1);
        sel = hi ? 2 : 0;
        o >>= 1;
        const bool hi2 = (lane_in_group & o) != 0;
        const float r2 = __shfl_xor_sync(0xffffffffu, hi2 ? b0 : b1, o);
        c = fmaxf(hi2 ? b1 : b0, r2);
        sel += hi2 ? 1 : 0;
        o >>= 1;
    } else if constexpr (R == 2) {
        const bool hi = (lane_in_group & o) != 0;
        const float r0 = __shfl_xor_sync(0xffffffffu, hi ? a[0] : a[1], o);
        c = fmaxf(hi ? a[1] : a[0], r0);
        sel = hi ? 1 : 0;
        o >>= 1;
    } else {
        c = a[0];
    }
#pragma unroll
    for (; o > 0; o >>= 1) c = fmaxf(c, __shfl_xor_sync(0xffffffffu, c, o));
    *rsel = sel;
    return c;
}
// Lane (within the group) that holds row r's result after reduce_rows.
template <int G, int R>
__device__ __forceinline__ int row_owner_lane(int r) {
    if constexpr (R == 4) return ((r >> 1) ? G / 2 : 0) + ((r & 1) ? G / 4 : 0);
    if constexpr (R == 2) return r ? G / 2 : 0;
    return 0;
}

// Where row r of the input goes in the output.  RowIdentity: to row r.  RowQkvHeads: the input
// is a fused projection [B*S, 3*H*Dh] read as rows of Dh elements, r = ((b*S + s)*3 + which)*H + h,
// and the output is [3][B][H][S] rows: the head-major layout the attention kernels take, so the
// split, view, transpose and contiguous copies of the eager path disappear into the quantiser.
struct RowIdentity {
    __device__ long long operator()(long long r) const { return r; }
};
struct RowQkvHeads {
    int B, S, H;
    __device__ long long operator()(long long r) const {
        const int h = (int)(r % H);
        const long long t3 = r / H;
        const int which = (int)(t3 % 3);
        const long long t = t3 / 3;
        const int s = (int)(t % S);
        const long long b = t / S;
        return (((long long)which * B + b) * H + h) * S + s;
    }
};

// Rows of `cols` elements, cols a multiple of Vec16<T>::N.  A row is handled by a
// group of G lanes (G a power of two <= 32); lane i of the group owns vectors
// i, i+G, ... (at most NV of them).  Each group keeps R rows in flight.
template <typename T, int G, int NV, int R, typename RowMap>
__global__ void __launch_bounds__(256, 4)
quantize_rows_vec_kernel(const T* __restrict__ x, int8_t* __restrict__ q,
                         float* __restrict__ scales, long long rows, int cols, RowMap out_row) {
    constexpr int N = Vec16<T>::N;
    pdl_wait();                                     // stream order towards the producer of x ...
    pdl_launch_dependents();                        // ... while the consumer of q may set itself up
    const int nvec = cols / N;
    constexpr int GPW = 32 / G;                     // groups per warp
    const int lane_in_group = threadIdx.x % G;
    const int group_in_warp = (threadIdx.x & 31) / G;
    const int group_lane0 = (threadIdx.x & 31) & ~(G - 1);
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;

    // The trip count is the same for every lane of a warp (the shuffles below
    // name all 32 lanes); rows past the end are predicated off.
    for (long long w0 = warp * GPW * R; w0 < rows; w0 += nwarps * GPW * R) {
        const long long r0 = w0 + (long long)group_in_warp * R;
        const int nrows = (int)(rows - r0 < R ? (rows - r0 > 0 ? rows - r0 : 0) : R);   // rows of this group that exist
        const T* xg = x + r0 * cols + lane_in_group * N;
        uint4 raw[R][NV];
        float amax[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                const int vi = lane_in_group + j * G;
                raw[r][j] = (r < nrows && vi < nvec) ? Vec16<T>::load(xg + r * cols + j * (G * N))
                                                     : make_uint4(0u, 0u, 0u, 0u);
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            amax[r] = 0.f;
#pragma unroll
            for (int j = 0; j < NV; ++j) amax[r] = fmaxf(amax[r], Vec16<T>::absmax(raw[r][j]));
        }
        float scale_r[R], rcp_r[R];
        if constexpr (R <= G) {
            // one division per lane serves R rows: each lane finishes one row's maximum, turns it
            // into scale and reciprocal, and the group reads them back by shuffle
            int rsel;
            const float am = reduce_rows<G, R>(amax, lane_in_group, &rsel);
            const float scale = __fdiv_rn(fmaxf(am, 1e-8f), 127.0f);
            const float rcp = __frcp_rn(scale);
            if (lane_in_group == row_owner_lane<G, R>(rsel) && rsel < nrows) scales[out_row(r0 + rsel)] = scale;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                scale_r[r] = __shfl_sync(0xffffffffu, scale, group_lane0 + row_owner_lane<G, R>(r));
                rcp_r[r] = __shfl_sync(0xffffffffu, rcp, group_lane0 + row_owner_lane<G, R>(r));
            }
        } else {
#pragma unroll
            for (int r = 0; r < R; ++r) {
#pragma unroll
                for (int o = G / 2; o > 0; o >>= 1)
                    amax[r] = fmaxf(amax[r], __shfl_xor_sync(0xffffffffu, amax[r], o));
                scale_r[r] = __fdiv_rn(fmaxf(amax[r], 1e-8f), 127.0f);
                rcp_r[r] = __frcp_rn(scale_r[r]);
                if (lane_in_group == 0 && r < nrows) scales[out_row(r0 + r)] = scale_r[r];
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            if (r >= nrows) continue;
            const float scale = scale_r[r], rcp = rcp_r[r];
            int8_t* qrow = q + out_row(r0 + r) * cols + lane_in_group * N;
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                const int vi = lane_in_group + j * G;
                if (vi >= nvec) continue;
                int8_t* dst = qrow + j * (G * N);
                float v[N];
                Vec16<T>::to_float(raw[r][j], v);
                if constexpr (N == 4) {
                    *reinterpret_cast<uint32_t*>(dst) = quant4(v[0], v[1], v[2], v[3], scale, rcp);
                } else {
                    uint2 pk;
                    pk.x = quant4(v[0], v[1], v[2], v[3], scale, rcp);
                    pk.y = quant4(v[4], v[5], v[6], v[7], scale, rcp);
                    *reinterpret_cast<uint2*>(dst) = pk;
                }
            }
        }
    }
}

// Any width / any alignment: one warp per row, two passes over the row (the
// second pass hits L1/L2).
template <typename T>
__global__ void __launch_bounds__(256)
quantize_rows_generic_kernel(const T* __restrict__ x, int8_t* __restrict__ q,
                             float* __restrict__ scales, long long rows, int cols) {
    const int lane = threadIdx.x & 31;
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long row = warp; row < rows; row += nwarps) {
        const T* xr = x + row * cols;
        float amax = 0.f;
        for (int i = lane; i < cols; i += 32) amax = fmaxf(amax, fabsf((float)xr[i]));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        const float scale = __fdiv_rn(fmaxf(amax, 1e-8f), 127.0f);
        if (lane == 0) scales[row] = scale;
        int8_t* qr = q + row * cols;
        for (int i = lane; i < cols; i += 32) qr[i] = (int8_t)quant1((float)xr[i], scale);
    }
}

template <typename T, int G, int NV, int R, typename RowMap = RowIdentity>
int launch_vec(const T* x, int8_t* q, float* scales, long long rows, int cols, cudaStream_t st,
               RowMap out_row = RowMap{}) {
    const long long groups = (rows + R - 1) / R;
    const long long threads = groups * G;
    long long blocks = (threads + 255) / 256;
    const long long cap = 148ll * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    I8TK_CUDA(launch_after(quantize_rows_vec_kernel<T, G, NV, R, RowMap>, dim3((unsigned)blocks), dim3(256), 0, st, x, q,
                           scales, rows, cols, out_row));
    return I8TK_OK;
}

template <typename T>
int quantize_per_token(const T* x, int8_t* q, float* scales, long long rows, int cols,
                       cudaStream_t st) {
    I8TK_REQUIRE(rows >= 0 && cols >= 1, I8TK_ERR_INVALID_ARGUMENT,
                 "rows must be >= 0 and cols >= 1 (rows=%lld cols=%d)", rows, cols);
    if (rows == 0) return I8TK_OK;                 // empty input: nothing to read or write
    I8TK_REQUIRE(x && q && scales, I8TK_ERR_INVALID_ARGUMENT, "null pointer argument");
    constexpr int N = Vec16<T>::N;
    const bool vec_ok = (cols % N == 0) && aligned_to(x, 16) && aligned_to(q, N);
    const int nvec = cols / N;
    if (vec_ok && nvec <= 256) {
        if (nvec <= 1) return launch_vec<T, 1, 1, 4>(x, q, scales, rows, cols, st);
        if (nvec <= 2) return launch_vec<T, 2, 1, 4>(x, q, scales, rows, cols, st);
        if (nvec <= 4) return launch_vec<T, 4, 1, 4>(x, q, scales, rows, cols, st);
        if (nvec <= 8) return launch_vec<T, 8, 1, 4>(x, q, scales, rows, cols, st);
        if (nvec <= 16) return launch_vec<T, 16, 1, 4>(x, q, scales, rows, cols, st);
        if (nvec <= 32) return launch_vec<T, 32, 1, 4>(x, q, scales, rows, cols, st);
        if (nvec <= 64) return launch_vec<T, 32, 2, 2>(x, q, scales, rows, cols, st);
        if (nvec <= 128) return launch_vec<T, 32, 4, 1>(x, q, scales, rows, cols, st);
        return launch_vec<T, 32, 8, 1>(x, q, scales, rows, cols, st);
    }
    long long blocks = (rows * 32 + 255) / 256;
    if (blocks > 148ll * 16) blocks = 148ll * 16;
    quantize_rows_generic_kernel<T><<<(int)blocks, 256, 0, st>>>(x, q, scales, rows, cols);
    I8TK_CUDA(cudaGetLastError());
    return I8TK_OK;
}

// ---- per-tensor (kernels/quant_utils.cu) ---------------------------------
__global__ void amax_f16_kernel(const __half* __restrict__ x, long long n, float* amax) {
    float v = 0.f;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x)
        v = fmaxf(v, fabsf(__half2float(x[i])));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    if ((threadIdx.x & 31) == 0) atomicMax(reinterpret_cast<unsigned int*>(amax), __float_as_uint(v));
}

__global__ void finalize_scale_kernel(float* s) { *s = *s / 127.f; }

__global__ void quant_tensor_f16_kernel(const __half* __restrict__ x, int8_t* __restrict__ q,
                                        long long n, const float* __restrict__ d_scale) {
    const float scale = *d_scale;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x) {
        const float v = __fdiv_rn(__half2float(x[i]), scale);
        q[i] = (int8_t)__float2int_rn(fmaxf(-128.f, fminf(127.f, v)));
    }
}

__global__ void dequant_tensor_kernel(const int8_t* __restrict__ q, __half* __restrict__ out,
                                      long long n, float scale) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x)
        out[i] = __float2half((float)q[i] * scale);
}

// out[r][c] = fp16(q[r][c] * scale[r]) (+ residual[r][c], added in fp32): the inverse step after the
// INT8 MLP, which the eager path spells as .float() * scale -> .half() (+ the residual add).
__global__ void __launch_bounds__(256)
dequant_rows_kernel(const int8_t* __restrict__ q, const float* __restrict__ scales,
                    const __half* __restrict__ residual, __half* __restrict__ out, long long vecs, int vecs_per_row) {
    pdl_wait();
    pdl_launch_dependents();
    for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < vecs;
         v += (long long)gridDim.x * blockDim.x) {
        const float sc = scales[v / vecs_per_row];
        const uint4 w = *reinterpret_cast<const uint4*>(q + v * 16);
        const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
        uint4 r0 = make_uint4(0u, 0u, 0u, 0u), r1 = r0;
        if (residual) {
            r0 = *reinterpret_cast<const uint4*>(residual + v * 16);
            r1 = *reinterpret_cast<const uint4*>(residual + v * 16 + 8);
        }
        const __half2* rh0 = reinterpret_cast<const __half2*>(&r0);
        const __half2* rh1 = reinterpret_cast<const __half2*>(&r1);
        uint32_t o[8];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int b0 = (int)(int8_t)(ww[k] & 0xff), b1 = (int)(int8_t)((ww[k] >> 8) & 0xff);
            const int b2 = (int)(int8_t)((ww[k] >> 16) & 0xff), b3 = (int)(int8_t)(ww[k] >> 24);
            const float2 ra = __half22float2(k < 2 ? rh0[2 * k] : rh1[2 * k - 4]);
            const float2 rb = __half22float2(k < 2 ? rh0[2 * k + 1] : rh1[2 * k - 3]);
            const __half2 ha = __floats2half2_rn(fmaf((float)b0, sc, ra.x), fmaf((float)b1, sc, ra.y));
            const __half2 hb = __floats2half2_rn(fmaf((float)b2, sc, rb.x), fmaf((float)b3, sc, rb.y));
            o[2 * k] = *reinterpret_cast<const uint32_t*>(&ha);
            o[2 * k + 1] = *reinterpret_cast<const uint32_t*>(&hb);
        }
        *reinterpret_cast<uint4*>(out + v * 16) = make_uint4(o[0], o[1], o[2], o[3]);
        *reinterpret_cast<uint4*>(out + v * 16 + 8) = make_uint4(o[4], o[5], o[6], o[7]);
    }
}

int grid_for(long long n) {
    long long b = (n + 255) / 256;
    if (b > 148ll * 16) b = 148ll * 16;
    if (b < 1) b = 1;
    return (int)b;
}

}  // namespace
}  // namespace i8tk

using namespace i8tk;

extern "C" int i8tk_quantize_qkv_heads_f16(const void* qkv_f16, int8_t* out, float* scales, int batch, int seq_len,
                                          int heads, int head_dim, i8tk_stream_t stream) {
    I8TK_REQUIRE(qkv_f16 && out && scales, I8TK_ERR_INVALID_ARGUMENT, "null pointer argument");
    I8TK_REQUIRE(batch > 0 && seq_len > 0 && heads > 0, I8TK_ERR_INVALID_ARGUMENT, "sizes must be positive");
    I8TK_REQUIRE(head_dim == 64 || head_dim == 128, I8TK_ERR_UNSUPPORTED, "head_dim must be 64 or 128 (got %d)",
                 head_dim);
    I8TK_REQUIRE(aligned_to(qkv_f16, 16) && aligned_to(out, 8), I8TK_ERR_ALIGNMENT,
                 "qkv must be 16-byte and out 8-byte aligned");
    const long long rows = (long long)batch * seq_len * 3 * heads;
    const RowQkvHeads map{batch, seq_len, heads};
    const __half* x = static_cast<const __half*>(qkv_f16);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (head_dim == 64) return launch_vec<__half, 8, 1, 4, RowQkvHeads>(x, out, scales, rows, 64, st, map);
    return launch_vec<__half, 16, 1, 4, RowQkvHeads>(x, out, scales, rows, 128, st, map);
}

extern "C" int i8tk_dequantize_per_token_f16(const int8_t* q, const float* scales, const void* residual_f16,
                                             void* out_f16, int64_t rows, int cols, i8tk_stream_t stream) {
    I8TK_REQUIRE(rows >= 0 && cols >= 16 && cols % 16 == 0, I8TK_ERR_INVALID_ARGUMENT,
                 "rows must be >= 0 and cols a positive multiple of 16");
    if (rows == 0) return I8TK_OK;
    I8TK_REQUIRE(q && scales && out_f16, I8TK_ERR_INVALID_ARGUMENT, "null pointer argument");
    I8TK_REQUIRE(aligned_to(q, 16) && aligned_to(out_f16, 16) && (!residual_f16 || aligned_to(residual_f16, 16)),
                 I8TK_ERR_ALIGNMENT, "q, out and residual must be 16-byte aligned");
    const long long vecs = rows * (cols / 16);
    long long blocks = (vecs + 255) / 256;
    if (blocks > 148ll * 16) blocks = 148ll * 16;
    I8TK_CUDA(launch_after(dequant_rows_kernel, dim3((unsigned)blocks), dim3(256), 0, static_cast<cudaStream_t>(stream),
                           q, scales, static_cast<const __half*>(residual_f16), static_cast<__half*>(out_f16), vecs,
                           cols / 16));
    return I8TK_OK;
}

extern "C" int i8tk_quantize_per_token_f32(const float* x, int8_t* q, float* scales, int64_t rows,
                                           int cols, i8tk_stream_t stream) {
    return quantize_per_token<float>(x, q, scales, rows, cols, static_cast<cudaStream_t>(stream));
}

extern "C" int i8tk_quantize_per_token_f16(const void* x, int8_t* q, float* scales, int64_t rows,
                                           int cols, i8tk_stream_t stream) {
    return quantize_per_token<__half>(static_cast<const __half*>(x), q, scales, rows, cols,
                                      static_cast<cudaStream_t>(stream));
}

extern "C" int i8tk_quantize_fp16_to_int8(const void* x, int8_t* q, float* d_scale, int64_t n,
                                          i8tk_stream_t stream) {
    I8TK_REQUIRE(x && q && d_scale && n > 0, I8TK_ERR_INVALID_ARGUMENT, "bad arguments");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const __half* xh = static_cast<const __half*>(x);
    I8TK_CUDA(cudaMemsetAsync(d_scale, 0, sizeof(float), st));
    amax_f16_kernel<<<grid_for(n), 256, 0, st>>>(xh, n, d_scale);
    finalize_scale_kernel<<<1, 1, 0, st>>>(d_scale);
    quant_tensor_f16_kernel<<<grid_for(n), 256, 0, st>>>(xh, q, n, d_scale);
    I8TK_CUDA(cudaGetLastError());
    return I8TK_OK;
}

extern "C" int i8tk_dequantize_int8_to_fp16(const int8_t* q, void* out, float scale, int64_t n,
                                            i8tk_stream_t stream) {
    I8TK_REQUIRE(q && out && n > 0, I8TK_ERR_INVALID_ARGUMENT, "bad arguments");
    dequant_tensor_kernel<<<grid_for(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        q, static_cast<__half*>(out), n, scale);
    I8TK_CUDA(cudaGetLastError());
    return I8TK_OK;
}
