// INT8-KV decode attention (seq_q == 1) for B200: split-KV flash decoding.
//
// Replaces int8_decode_attention_forward of the reference
// (kernels/int8_decode_attention.cu:443-547: launcher, :274-386 partial
// kernel, :389-426 combine kernel).  Same arithmetic contract --
//   score_j = (q . k_j) * sQ * sK_j / sqrt(D)        (int8 x int8 -> int32 dot)
//   out     = sum_j softmax(score)_j * sV_j * v_j    (fp32 accumulate, fp16 out)
// -- different machine mapping:
//
// * One warp owns one work unit (b*h, KV split) and a private ring of shared
//   memory stages.  K and V tiles of 32 positions are streamed HBM -> shared
//   memory by 1-D bulk async copies (the TMA engine) that complete on an
//   mbarrier; several tiles per warp are always in flight, so the bytes in
//   flight per SM (up to ~190 KB) cover HBM3e latency x bandwidth without
//   needing many resident warps.  No block-level barrier exists anywhere.
// * A tile row (64 or 128 int8) is split into 16-byte chunks; lane (g, c)
//   reads chunk c of rows g, g+R, g+2R, ... with 128-bit shared loads that are
//   bank-conflict free (a quarter-warp reads 128 contiguous bytes).
// * QK^T: four dp4a per 16-byte chunk, then a reduce-scatter over the lanes of
//   a row so that every lane ends up owning the full dot of ONE position:
//   the softmax arithmetic (scale, exp2, running sum) is done once per
//   position, not once per lane.
// * PV: the weight p_j*sV_j is broadcast back by shuffle; int8 -> fp32 uses a
//   byte-permute into the mantissa of 2^23 (full-rate ALU/FMA ops; no I2F).
// * Softmax runs in log2 units (log2(e) folded into the score scale) with a
//   running max per warp; the accumulator is rescaled only when the max moves.
// * Each unit leaves one unnormalised (m, l, acc[D]) row; a small second
//   kernel merges the rows of a (b,h) by log-sum-exp.  The same row format is
//   the exchange format of the multi-GPU sequence-sharded path.
#include "common.cuh"

#include <cmath>
#include <cstdlib>

namespace i8tk {
namespace {

constexpr int kTile = 32;             // KV positions per stage
constexpr int kWarps = 4;             // work units per CTA
constexpr float kLog2e = 1.4426950408889634f;

template <int D>
struct DecodeTraits {
    static constexpr int LPR = D / 16;                 // lanes per row (16 B each)
    static constexpr int RPP = 32 / LPR;               // rows per warp pass
    static constexpr int STAGES = (D == 64) ? 4 : 3;   // ring depth per warp
    static constexpr int TILE_BYTES = kTile * D;       // one of K or V
    static constexpr int STAGE_BYTES = 2 * TILE_BYTES; // K tile then V tile
    static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
    static constexpr int SMEM_BYTES = kWarps * RING_BYTES + kWarps * STAGES * 8;
    static constexpr int CTAS_PER_SM = (D == 64) ? 3 : 2;
    static constexpr int ROW_FLOATS = D + 4;           // m, l, 0, 0, acc[D]
};

enum EpilogueMode : int {
    kToScratchRows = 0,   // (m, l, acc) row per unit, merged by the combine kernel
    kToFinalF16 = 1,      // nsplit == 1: normalise and write fp16 directly
};

__device__ __forceinline__ int dot16(const int4& q, const int4& k) {
    int d = __dp4a(q.x, k.x, 0);
    d = __dp4a(q.y, k.y, d);
    d = __dp4a(q.z, k.z, d);
    d = __dp4a(q.w, k.w, d);
    return d;
}

// acc[0..3] += w * int8x4(word).  The word has been XORed with 0x80808080 so
// its bytes are u = v + 128 in [0, 255]; prmt drops byte j into the low
// mantissa of 0x4B000000 (= 2^23), and subtracting 2^23 + 128 recovers v
// exactly in fp32.
__device__ __forceinline__ void fma_i8x4(float* acc, uint32_t biased, float w) {
    constexpr float kMagic = 8388736.0f;  // 2^23 + 128
    const float f0 = __uint_as_float(prmt(biased, 0x4B000000u, 0x7650u)) - kMagic;
    const float f1 = __uint_as_float(prmt(biased, 0x4B000000u, 0x7651u)) - kMagic;
    const float f2 = __uint_as_float(prmt(biased, 0x4B000000u, 0x7652u)) - kMagic;
    const float f3 = __uint_as_float(prmt(biased, 0x4B000000u, 0x7653u)) - kMagic;
    acc[0] = fmaf(w, f0, acc[0]);
    acc[1] = fmaf(w, f1, acc[1]);
    acc[2] = fmaf(w, f2, acc[2]);
    acc[3] = fmaf(w, f3, acc[3]);
}

// Variant without the subtraction: byte j is moved into the low byte of an
// otherwise zero word, which read as fp32 is the denormal u * 2^-149.  FFMA
// takes denormal operands at full rate, the product with a weight pre-scaled
// by 2^kDenormShift is exact, and the +128 bias of u is removed once per unit
// from the running sum of weights.
constexpr int kDenormShift = 100;
__device__ __forceinline__ void fma_u8x4_denorm(float* acc, uint32_t biased, float w_scaled) {
    const float f0 = __uint_as_float(biased & 0xffu);
    const float f1 = __uint_as_float(prmt(biased, 0u, 0x4441u));
    const float f2 = __uint_as_float(prmt(biased, 0u, 0x4442u));
    const float f3 = __uint_as_float(biased >> 24);
    acc[0] = fmaf(w_scaled, f0, acc[0]);
    acc[1] = fmaf(w_scaled, f1, acc[1]);
    acc[2] = fmaf(w_scaled, f2, acc[2]);
    acc[3] = fmaf(w_scaled, f3, acc[3]);
}

// Reduce-scatter of LPR partial dots over the LPR lanes that share a row set:
// on return lane c of the group holds the full dot of position index k == c.
template <int LPR>
__device__ __forceinline__ int reduce_scatter(int (&d)[LPR], int c) {
    if constexpr (LPR == 8) {
        const bool hi = (c & 4) != 0;
        int r[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int keep = hi ? d[4 + i] : d[i];
            const int send = hi ? d[i] : d[4 + i];
            r[i] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
        }
        const bool hi2 = (c & 2) != 0;
        int s[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int keep = hi2 ? r[2 + i] : r[i];
            const int send = hi2 ? r[i] : r[2 + i];
            s[i] = keep + __shfl_xor_sync(0xffffffffu, send, 2);
        }
        const bool hi1 = (c & 1) != 0;
        const int keep = hi1 ? s[1] : s[0];
        const int send = hi1 ? s[0] : s[1];
        return keep + __shfl_xor_sync(0xffffffffu, send, 1);
    } else {
        static_assert(LPR == 4, "head_dim 64 or 128");
        const bool hi2 = (c & 2) != 0;
        int s[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int keep = hi2 ? d[2 + i] : d[i];
            const int send = hi2 ? d[i] : d[2 + i];
            s[i] = keep + __shfl_xor_sync(0xffffffffu, send, 2);
        }
        const bool hi1 = (c & 1) != 0;
        const int keep = hi1 ? s[1] : s[0];
        const int send = hi1 ? s[0] : s[1];
        return keep + __shfl_xor_sync(0xffffffffu, send, 1);
    }
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ---------------------------------------------------------------------------
// Pass 1: one warp scans KV positions [sp*chunk, min(S,(sp+1)*chunk)) of one
// (b,h) and leaves an unnormalised online-softmax row.
// ---------------------------------------------------------------------------
template <int D, int VMODE>
__global__ void __launch_bounds__(kWarps * 32)
decode_partial_kernel(const int8_t* __restrict__ Q, const int8_t* __restrict__ K,
                      const int8_t* __restrict__ V, const float* __restrict__ sQ,
                      const float* __restrict__ sK, const float* __restrict__ sV,
                      float* __restrict__ rows,     // [units, D+4] (mode 0)
                      __half* __restrict__ out,     // [BH, D]      (mode 1)
                      int S, int nsplit, int chunk, int units, float score_scale_log2,
                      int mode, uint32_t* __restrict__ status) {
    using T = DecodeTraits<D>;
    constexpr int LPR = T::LPR, RPP = T::RPP, STAGES = T::STAGES;

    extern __shared__ __align__(128) unsigned char smem[];
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int unit = blockIdx.x * kWarps + warp;
    if (unit >= units) return;

    unsigned char* ring = smem + warp * T::RING_BYTES;
    const uint32_t ring_s = smem_u32(ring);
    const uint32_t bar0 = smem_u32(smem + kWarps * T::RING_BYTES) + warp * STAGES * 8;

    const int bh = unit / nsplit;
    const int sp = unit - bh * nsplit;
    const int j0 = sp * chunk;
    const int n = min(S, j0 + chunk) - j0;          // positions of this unit
    const int ntiles = n > 0 ? (n + kTile - 1) / kTile : 0;

    const int c = lane % LPR;                       // 16-byte chunk of a row
    const int g = lane / LPR;                       // row within a pass
    const int own = g + RPP * c;                    // position in the tile whose softmax this lane runs

    const size_t row0 = (size_t)bh * S + j0;
    const int8_t* Kb = K + row0 * D;
    const int8_t* Vb = V + row0 * D;
    const float* sKb = sK + row0;
    const float* sVb = sV + row0;

    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; ++s) mbar_init(bar0 + 8 * s, 1);
        fence_mbar_init();
    }
    __syncwarp();

    auto issue = [&](int t) {
        // lane 0 only: start the K and V copies of tile t into stage t % STAGES
        const int st = t % STAGES;
        const int nrow = min(kTile, n - t * kTile);
        const uint32_t bytes = (uint32_t)nrow * D;
        const uint32_t bar = bar0 + 8 * st;
        const uint32_t dst = ring_s + st * T::STAGE_BYTES;
        mbar_expect_tx(bar, 2 * bytes);
        bulk_g2s(dst, Kb + (size_t)t * T::TILE_BYTES, bytes, bar);
        bulk_g2s(dst + T::TILE_BYTES, Vb + (size_t)t * T::TILE_BYTES, bytes, bar);
    };

    if (lane == 0) {
        const int pre = min(STAGES, ntiles);
        for (int t = 0; t < pre; ++t) issue(t);
    }

    const int4 q4 = *reinterpret_cast<const int4*>(Q + (size_t)bh * D + c * 16);
    const float qs = sQ[bh] * score_scale_log2;

    // per-position scales of the owned position, fetched two tiles ahead
    float sk0 = 0.f, sv0 = 0.f, sk1 = 0.f, sv1 = 0.f;
    if (own < n) { sk0 = sKb[own]; sv0 = sVb[own]; }
    if (kTile + own < n) { sk1 = sKb[kTile + own]; sv1 = sVb[kTile + own]; }

    float m = -INFINITY, l = 0.f;
    float wsum = 0.f;                               // VMODE 1: sum of weights of this lane's rows
    float acc[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i] = 0.f;

    bool ok = true;
    for (int t = 0; t < ntiles; ++t) {
        float sk2 = 0.f, sv2 = 0.f;
        {
            const int p2 = (t + 2) * kTile + own;
            if (p2 < n) { sk2 = sKb[p2]; sv2 = sVb[p2]; }
        }
        const int st = t % STAGES;
        const bool got = mbar_wait_bounded(bar0 + 8 * st, (t / STAGES) & 1);
        if (!__all_sync(0xffffffffu, got)) { ok = false; break; }

        const int4* Kt = reinterpret_cast<const int4*>(ring + st * T::STAGE_BYTES);
        const int4* Vt = reinterpret_cast<const int4*>(ring + st * T::STAGE_BYTES + T::TILE_BYTES);

        // ---- QK^T partial dots, then one full dot per lane ----------------
        int d[LPR];
#pragma unroll
        for (int k = 0; k < LPR; ++k) {
            const int4 kw = Kt[(g + RPP * k) * LPR + c];
            d[k] = dot16(q4, kw);
        }
        const int tot = reduce_scatter<LPR>(d, c);

        // ---- online softmax, log2 units, one position per lane -------------
        const bool valid = (t * kTile + own) < n;
        const float s = valid ? (float)tot * (qs * sk0) : -INFINITY;
        const float m_new = fmaxf(m, warp_max(s));
        if (m_new > m) {                            // warp-uniform
            const float corr = ex2_approx(m - m_new);
            l *= corr;
            wsum *= corr;
#pragma unroll
            for (int i = 0; i < 16; ++i) acc[i] *= corr;
            m = m_new;
        }
        const float p = ex2_approx(s - m);
        l += p;
        const float w = p * sv0;

        // ---- PV: acc[16 dims of chunk c] += w_row * v_row -------------------
#pragma unroll
        for (int k = 0; k < LPR; ++k) {
            const float wk = __shfl_sync(0xffffffffu, w, (lane & ~(LPR - 1)) | k);
            const int4 vw = Vt[(g + RPP * k) * LPR + c];
            if constexpr (VMODE == 0) {
                fma_i8x4(acc + 0, (uint32_t)vw.x ^ 0x80808080u, wk);
                fma_i8x4(acc + 4, (uint32_t)vw.y ^ 0x80808080u, wk);
                fma_i8x4(acc + 8, (uint32_t)vw.z ^ 0x80808080u, wk);
                fma_i8x4(acc + 12, (uint32_t)vw.w ^ 0x80808080u, wk);
            } else {
                wsum += wk;
                const float ws = wk * __uint_as_float((127u + kDenormShift) << 23);
                fma_u8x4_denorm(acc + 0, (uint32_t)vw.x ^ 0x80808080u, ws);
                fma_u8x4_denorm(acc + 4, (uint32_t)vw.y ^ 0x80808080u, ws);
                fma_u8x4_denorm(acc + 8, (uint32_t)vw.z ^ 0x80808080u, ws);
                fma_u8x4_denorm(acc + 12, (uint32_t)vw.w ^ 0x80808080u, ws);
            }
        }

        // every lane is done reading this stage: refill it
        __syncwarp();
        if (lane == 0 && t + STAGES < ntiles) {
            fence_proxy_async();
            issue(t + STAGES);
        }
        sk0 = sk1; sv0 = sv1; sk1 = sk2; sv1 = sv2;
    }

    if (!ok) {
        if (lane == 0) atomicExch(status, kDeviceTimeoutMagic);
        return;
    }

    // ---- fold the row groups; lanes g == 0 hold the chunk's 16 sums --------
#pragma unroll
    for (int o = LPR; o < 32; o <<= 1) {
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], o);
    }
    l = warp_sum(l);
    if constexpr (VMODE == 1) {
        // rows were spread over the row groups; lanes of one group saw the same weights
#pragma unroll
        for (int o = LPR; o < 32; o <<= 1) wsum += __shfl_xor_sync(0xffffffffu, wsum, o);
        const float unscale = __uint_as_float((127u + 149u - kDenormShift) << 23);
        const float bias = 128.0f * wsum;
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i] = fmaf(acc[i], unscale, -bias);
    }

    if (mode == kToFinalF16) {
        if (g == 0) {
            const float inv = 1.0f / l;
            __half2 h[8];
#pragma unroll
            for (int i = 0; i < 8; ++i)
                h[i] = __floats2half2_rn(acc[2 * i] * inv, acc[2 * i + 1] * inv);
            int4* dst = reinterpret_cast<int4*>(out + (size_t)bh * D + c * 16);
            dst[0] = *reinterpret_cast<int4*>(&h[0]);
            dst[1] = *reinterpret_cast<int4*>(&h[4]);
        }
    } else {
        float* row = rows + (size_t)unit * T::ROW_FLOATS;
        if (lane == 0) *reinterpret_cast<float4*>(row) = make_float4(m, l, 0.f, 0.f);
        if (g == 0) {
            float4* dst = reinterpret_cast<float4*>(row + 4 + c * 16);
#pragma unroll
            for (int i = 0; i < 4; ++i)
                dst[i] = make_float4(acc[4 * i], acc[4 * i + 1], acc[4 * i + 2], acc[4 * i + 3]);
        }
    }
}

// ---------------------------------------------------------------------------
// Pass 2: log-sum-exp merge of the rows of one (b,h).  One warp per (b,h);
// row (bh, s) lives at rows + (bh*stride_bh + s*stride_s) * (D+4).
// Writes either the normalised fp16 output or one merged row.
// ---------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(128)
decode_combine_kernel(const float* __restrict__ rows, int BH, int nsplit,
                      long long stride_bh, long long stride_s,
                      __half* __restrict__ out, float* __restrict__ row_out) {
    constexpr int ROW = D + 4;
    constexpr int DPL = D / 32;
    const int bh = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (bh >= BH) return;
    const int lane = threadIdx.x & 31;
    const float* base = rows + (size_t)bh * stride_bh * ROW;

    float gm = -INFINITY;
    for (int s = lane; s < nsplit; s += 32) {
        const float2 ml = *reinterpret_cast<const float2*>(base + (size_t)s * stride_s * ROW);
        if (ml.y > 0.f) gm = fmaxf(gm, ml.x);
    }
    gm = warp_max(gm);

    float L = 0.f;
    float a[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) a[i] = 0.f;
#pragma unroll 4
    for (int s = 0; s < nsplit; ++s) {
        const float* r = base + (size_t)s * stride_s * ROW;
        const float2 ml = *reinterpret_cast<const float2*>(r);
        if (ml.y <= 0.f) continue;                 // empty split
        const float w = ex2_approx(ml.x - gm);
        L = fmaf(ml.y, w, L);
        if constexpr (DPL == 4) {
            const float4 v = *reinterpret_cast<const float4*>(r + 4 + lane * 4);
            a[0] = fmaf(v.x, w, a[0]); a[1] = fmaf(v.y, w, a[1]);
            a[2] = fmaf(v.z, w, a[2]); a[3] = fmaf(v.w, w, a[3]);
        } else {
            const float2 v = *reinterpret_cast<const float2*>(r + 4 + lane * 2);
            a[0] = fmaf(v.x, w, a[0]); a[1] = fmaf(v.y, w, a[1]);
        }
    }

    if (out != nullptr) {
        const float inv = 1.0f / L;
        __half* o = out + (size_t)bh * D + lane * DPL;
        if constexpr (DPL == 4) {
            __half2 h0 = __floats2half2_rn(a[0] * inv, a[1] * inv);
            __half2 h1 = __floats2half2_rn(a[2] * inv, a[3] * inv);
            uint2 pk;
            pk.x = *reinterpret_cast<uint32_t*>(&h0);
            pk.y = *reinterpret_cast<uint32_t*>(&h1);
            *reinterpret_cast<uint2*>(o) = pk;
        } else {
            *reinterpret_cast<__half2*>(o) = __floats2half2_rn(a[0] * inv, a[1] * inv);
        }
    } else {
        float* r = row_out + (size_t)bh * ROW;
        if (lane == 0) *reinterpret_cast<float4*>(r) = make_float4(L > 0.f ? gm : -INFINITY, L, 0.f, 0.f);
        if constexpr (DPL == 4)
            *reinterpret_cast<float4*>(r + 4 + lane * 4) = make_float4(a[0], a[1], a[2], a[3]);
        else
            *reinterpret_cast<float2*>(r + 4 + lane * 2) = make_float2(a[0], a[1]);
    }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
struct Plan { int nsplit; int chunk; };

// Optional timing probe: events recorded on the launch stream immediately
// before and after the streaming (pass 1) kernel of the next calls made by
// this thread.
thread_local cudaEvent_t g_probe_start = nullptr;
thread_local cudaEvent_t g_probe_stop = nullptr;

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

// Pick the number of KV splits.  Units run one per warp, `slots` warps are
// resident on the device at once; a unit costs its tile count plus a fixed
// fill/drain overhead; the grid runs in ceil(units/slots) rounds.  Chunks are
// whole tiles so every bulk copy starts on a row boundary.
Plan make_plan(int BH, int S, int D, int sms) {
    const char* e = getenv("I8TK_DECODE_NSPLIT");
    const int forced = e ? atoi(e) : 0;
    const int ctas_per_sm = (D == 64) ? DecodeTraits<64>::CTAS_PER_SM : DecodeTraits<128>::CTAS_PER_SM;
    const long long slots = (long long)sms * ctas_per_sm * kWarps;
    const int tiles = (S + kTile - 1) / kTile;
    const int max_split = forced > 0 ? forced : (tiles / 4 > 1 ? tiles / 4 : 1);
    const double overhead = 6.0;                     // tile-times per unit (pipeline fill + epilogue)
    Plan best{1, tiles * kTile};
    double best_cost = 1e300;
    for (int ns = (forced > 0 ? forced : 1); ns <= max_split && ns <= 512; ++ns) {
        const int ctiles = (tiles + ns - 1) / ns;
        const int eff = (tiles + ctiles - 1) / ctiles;  // splits that are non-empty
        const long long units = (long long)BH * eff;
        const long long rounds = (units + slots - 1) / slots;
        const double cost = (double)rounds * (ctiles + overhead) + 0.02 * eff;
        if (cost < best_cost - 1e-9) {
            best_cost = cost;
            best = Plan{eff, ctiles * kTile};
        }
    }
    return best;
}

size_t workspace_bytes(int BH, int S, int D) {
    const Plan p = make_plan(BH, S, D, sm_count());
    return 256 + (size_t)BH * p.nsplit * (D + 4) * sizeof(float);
}

template <int D, int VMODE>
int launch_decode_v(const int8_t* Q, const int8_t* K, const int8_t* V, __half* out, float* part,
                  const float* sQ, const float* sK, const float* sV, int BH, int S,
                  void* workspace, size_t wbytes, cudaStream_t stream) {
    using T = DecodeTraits<D>;
    static bool attr_done[64] = {false};   // per template instance
    int dev = 0;
    I8TK_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        I8TK_CUDA(cudaFuncSetAttribute(decode_partial_kernel<D, VMODE>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, T::SMEM_BYTES));
        attr_done[dev] = true;
    }
    const Plan p = make_plan(BH, S, D, sm_count());
    const long long units_ll = (long long)BH * p.nsplit;
    I8TK_REQUIRE(units_ll < (1ll << 31) - 8, I8TK_ERR_UNSUPPORTED, "too many work units");
    const int units = (int)units_ll;
    const size_t need = 256 + (size_t)units * T::ROW_FLOATS * sizeof(float);
    I8TK_REQUIRE(workspace != nullptr && wbytes >= need, I8TK_ERR_WORKSPACE,
                 "decode workspace too small: need %zu bytes, got %zu", need, wbytes);
    I8TK_REQUIRE(aligned_to(workspace, 256), I8TK_ERR_ALIGNMENT, "workspace must be 256-byte aligned");

    uint32_t* status = reinterpret_cast<uint32_t*>(workspace);
    float* rows = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(workspace) + 256);
    const float score_scale_log2 = kLog2e / sqrtf((float)D);
    const int grid = (units + kWarps - 1) / kWarps;

    const bool direct = (p.nsplit == 1 && out != nullptr);
    if (g_probe_start) I8TK_CUDA(cudaEventRecord(g_probe_start, stream));
    decode_partial_kernel<D, VMODE><<<grid, kWarps * 32, T::SMEM_BYTES, stream>>>(
        Q, K, V, sQ, sK, sV, rows, out, S, p.nsplit, p.chunk, units, score_scale_log2,
        direct ? kToFinalF16 : kToScratchRows, status);
    I8TK_CUDA(cudaGetLastError());
    if (g_probe_stop) I8TK_CUDA(cudaEventRecord(g_probe_stop, stream));
    if (!direct) {
        decode_combine_kernel<D><<<(BH + 3) / 4, 128, 0, stream>>>(
            rows, BH, p.nsplit, (long long)p.nsplit, 1ll, out, part);
        I8TK_CUDA(cudaGetLastError());
    }
    return I8TK_OK;
}

int env_int(const char* name, int dflt) {
    const char* e = getenv(name);
    return e ? atoi(e) : dflt;
}

template <int D>
int launch_decode(const int8_t* Q, const int8_t* K, const int8_t* V, __half* out, float* part,
                  const float* sQ, const float* sK, const float* sV, int BH, int S,
                  void* workspace, size_t wbytes, cudaStream_t stream) {
    if (env_int("I8TK_DECODE_VMODE", 0) == 1)
        return launch_decode_v<D, 1>(Q, K, V, out, part, sQ, sK, sV, BH, S, workspace, wbytes, stream);
    return launch_decode_v<D, 0>(Q, K, V, out, part, sQ, sK, sV, BH, S, workspace, wbytes, stream);
}

int check_decode_args(const void* Q, const void* K, const void* V, const void* o,
                      const void* sQ, const void* sK, const void* sV, int BH, int S, int D) {
    I8TK_REQUIRE(Q && K && V && o && sQ && sK && sV, I8TK_ERR_INVALID_ARGUMENT, "null pointer argument");
    I8TK_REQUIRE(BH > 0 && S > 0, I8TK_ERR_INVALID_ARGUMENT, "BH and S must be positive (BH=%d S=%d)", BH, S);
    I8TK_REQUIRE(D == 64 || D == 128, I8TK_ERR_UNSUPPORTED,
                 "decode attention supports head_dim 64 or 128 (got %d)", D);
    I8TK_REQUIRE(aligned_to(Q, 16) && aligned_to(K, 16) && aligned_to(V, 16), I8TK_ERR_ALIGNMENT,
                 "Q, K, V must be 16-byte aligned");
    I8TK_REQUIRE(aligned_to(sQ, 4) && aligned_to(sK, 4) && aligned_to(sV, 4), I8TK_ERR_ALIGNMENT,
                 "scales must be 4-byte aligned");
    I8TK_REQUIRE(aligned_to(o, 16), I8TK_ERR_ALIGNMENT, "output must be 16-byte aligned");
    return I8TK_OK;
}

}  // namespace
}  // namespace i8tk

using namespace i8tk;

extern "C" size_t i8tk_decode_workspace_bytes(int BH, int S, int head_dim) {
    if (BH <= 0 || S <= 0 || (head_dim != 64 && head_dim != 128)) return 0;
    return workspace_bytes(BH, S, head_dim);
}

extern "C" int i8tk_decode_partial_stride(int head_dim) { return head_dim + 4; }

extern "C" int i8tk_decode_set_probe_events(void* start_event, void* stop_event) {
    g_probe_start = static_cast<cudaEvent_t>(start_event);
    g_probe_stop = static_cast<cudaEvent_t>(stop_event);
    return I8TK_OK;
}

extern "C" int i8tk_decode_plan(int BH, int S, int head_dim, int* nsplit, int* chunk) {
    I8TK_REQUIRE(BH > 0 && S > 0 && nsplit && chunk, I8TK_ERR_INVALID_ARGUMENT, "bad plan arguments");
    I8TK_REQUIRE(head_dim == 64 || head_dim == 128, I8TK_ERR_UNSUPPORTED, "head_dim must be 64 or 128");
    const Plan p = make_plan(BH, S, head_dim, sm_count());
    *nsplit = p.nsplit;
    *chunk = p.chunk;
    return I8TK_OK;
}

extern "C" int i8tk_decode_attention_forward(const int8_t* Q, const int8_t* K, const int8_t* V,
                                             void* out_f16, const float* sQ, const float* sK,
                                             const float* sV, int BH, int S, int head_dim,
                                             void* workspace, size_t workspace_bytes,
                                             i8tk_stream_t stream) {
    const int rc = check_decode_args(Q, K, V, out_f16, sQ, sK, sV, BH, S, head_dim);
    if (rc != I8TK_OK) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (head_dim == 64)
        return launch_decode<64>(Q, K, V, static_cast<__half*>(out_f16), nullptr, sQ, sK, sV, BH, S,
                                 workspace, workspace_bytes, st);
    return launch_decode<128>(Q, K, V, static_cast<__half*>(out_f16), nullptr, sQ, sK, sV, BH, S,
                              workspace, workspace_bytes, st);
}

extern "C" int i8tk_decode_attention_partial(const int8_t* Q, const int8_t* K, const int8_t* V,
                                             float* part, const float* sQ, const float* sK,
                                             const float* sV, int BH, int S, int head_dim,
                                             void* workspace, size_t workspace_bytes,
                                             i8tk_stream_t stream) {
    const int rc = check_decode_args(Q, K, V, part, sQ, sK, sV, BH, S, head_dim);
    if (rc != I8TK_OK) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (head_dim == 64)
        return launch_decode<64>(Q, K, V, nullptr, part, sQ, sK, sV, BH, S, workspace,
                                 workspace_bytes, st);
    return launch_decode<128>(Q, K, V, nullptr, part, sQ, sK, sV, BH, S, workspace,
                              workspace_bytes, st);
}

extern "C" int i8tk_decode_combine_partials(const float* parts, int nparts, int BH, int head_dim,
                                            void* out_f16, i8tk_stream_t stream) {
    I8TK_REQUIRE(parts && out_f16, I8TK_ERR_INVALID_ARGUMENT, "null pointer argument");
    I8TK_REQUIRE(nparts > 0 && BH > 0, I8TK_ERR_INVALID_ARGUMENT, "nparts and BH must be positive");
    I8TK_REQUIRE(head_dim == 64 || head_dim == 128, I8TK_ERR_UNSUPPORTED, "head_dim must be 64 or 128");
    I8TK_REQUIRE(aligned_to(parts, 16) && aligned_to(out_f16, 16), I8TK_ERR_ALIGNMENT,
                 "parts and out must be 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int grid = (BH + 3) / 4;
    if (head_dim == 64)
        decode_combine_kernel<64><<<grid, 128, 0, st>>>(parts, BH, nparts, 1ll, (long long)BH,
                                                        static_cast<__half*>(out_f16), nullptr);
    else
        decode_combine_kernel<128><<<grid, 128, 0, st>>>(parts, BH, nparts, 1ll, (long long)BH,
                                                         static_cast<__half*>(out_f16), nullptr);
    I8TK_CUDA(cudaGetLastError());
    return I8TK_OK;
}
