// INT8 prefill attention (seq_q == seq_kv, no causal mask) for B200.
//
// Replaces int8_attention_forward of the reference (kernels/int8_attention.cu:926-1028,
// kernel :227-645).  Same arithmetic contract --
//   score[i][j] = (q_i . k_j) * sQ_i * sK_j / sqrt(D)          (int8 x int8 -> int32)
//   out_i       = sum_j softmax(score_i)_j * sV_j * v_j          (P*sV and V in fp16, fp32 accumulate)
// -- on the 5th-generation tensor cores:
//
// * One CTA per (b*h, 128 query rows).  QK^T is tcgen05.mma kind::i8 into a
//   128x128 int32 accumulator in tensor memory (two buffers); PV is tcgen05.mma
//   kind::f16 accumulating the 128xD fp32 output in tensor memory across all KV
//   tiles.
// * A pre-pass dequantises V once per call, V16 = fp16(V * sV), into the workspace: every
//   128-row query tile of a head reads the same V, so converting it inside the attention
//   kernel repeated the work S/128 times and took a fifth of its instructions.  Q and K
//   tiles (int8) and V16 tiles (fp16) arrive by TMA; V16 lands directly in the MN-major
//   128-byte-swizzled layout the PV instruction reads.
// * Eight softmax warps, two per TMEM lane quarter, each thread owning half of the KV
//   positions of a tile (32 of 64) for one query row.  The scores are read from tensor memory once
//   (tcgen05.ld), converted without the conversion unit (|q.k| < 2^22, so the
//   integer is added to the bit pattern of 1.5*2^23 and 1.5*2^23 subtracted as a
//   float), scaled by sK and kept in registers; the row maximum is combined across
//   the two halves through shared memory.  A LAZY running maximum (it only moves
//   when the true maximum exceeds it by 2^8, so p <= 256 stays comfortably inside
//   fp16) makes rescaling the output accumulator in tensor memory (tcgen05.ld /
//   tcgen05.st) rare.  The exponentials of tile j (special-function unit) are
//   interleaved, eight columns at a time, with the conversion of tile j+1's scores
//   (integer and FMA pipes), which take over the registers just released; Q.K^T
//   therefore runs two tiles ahead of P.V (one tile at head_dim 128, which keeps a single
//   score tile in tensor memory).  P goes as fp16 pairs into one of two blocks of tensor
//   memory (tcgen05.st), from where the P.V instruction reads
//   its A operand: no shared-memory round trip, no swizzle arithmetic, no proxy fence.
//   Packed fp32x2 arithmetic throughout.
// * K and V16 tiles move through rings of kRing stages, so a late tile does not hold up the
//   single thread that issues both products in turn.
// * Every mbarrier wait is bounded; on expiry a status word is set and all
//   roles fall through to the common exit, which frees tensor memory.
//
// * KV tiles are 64 positions.  At head_dim 64 and 128 a CTA then needs 96 registers per thread, 256
//   columns of tensor memory and at most 88 KB of shared memory, so TWO CTAs share an SM and their
//   sixteen softmax warps hide one another's waits; at head_dim 256 the 256-column output leaves
//   room for one CTA.
//
// Supported: head_dim 64, 128 and 256, any seq_len (a
// partial last tile is masked: the operand tiles then hold rows of the next head or TMA's zero
// fill, whose scores are set to -inf).
#include "tcgen05.cuh"

#include <cmath>

namespace i8tk {
namespace {

constexpr int kQT = 128;                 // query rows per CTA
constexpr int kSoftmaxWarps = 8;         // two per TMEM lane quarter: each thread owns half of a score row
constexpr int kPrefillThreads = (2 + kSoftmaxWarps) * 32;   // TMA, MMA, 8 softmax warps
constexpr int kRing = 3;                 // stages of the K ring and of the V16 ring
constexpr float kLazyStep = 8.0f;        // log2 units the true max may run ahead of the reference max

// D: head_dim; KT: KV positions per tile (128, or 64 at head_dim 256, where a 128-position tile
// would need 128 + 128 score columns, 128 for P and 256 for the output: more than the 512
// columns of tensor memory, and K + V16 stages of 96 KB each).
template <int D, int KT>
struct PrefillCfg {
    static constexpr int HK = KT / 2;                      // KV positions of a tile per softmax thread
    static constexpr int ROW_BYTES = D < 128 ? D : 128;    // bytes of a Q/K row per swizzled slab
    static constexpr int QK_SLABS = D / ROW_BYTES;         // 128-byte slabs of a Q or K row (2 at head_dim 256)
    static constexpr int Q_SLAB = kQT * ROW_BYTES;
    static constexpr int K_SLAB = KT * ROW_BYTES;
    static constexpr int Q_BYTES = kQT * D;                // int8 query tile
    static constexpr int K_BYTES = KT * D;                 // int8 key tile
    static constexpr int V16_BYTES = KT * D * 2;           // fp16 V tile
    static constexpr int V_SLAB = KT * 128;                // KT rows of 128 bytes (64 fp16 columns)
    static constexpr int OFF_Q = 0;
    static constexpr int OFF_K = OFF_Q + Q_BYTES;
    static constexpr int OFF_V16 = OFF_K + kRing * K_BYTES;
    static constexpr int OFF_SCALES = OFF_V16 + kRing * V16_BYTES; // 8 warps x 2 tiles x sK[HK] fp32
    static constexpr int OFF_XCH = OFF_SCALES + kSoftmaxWarps * 2 * HK * 4;    // [2][2 halves][128 rows] fp32
    static constexpr int OFF_BARS = OFF_XCH + 2 * 2 * kQT * 4;
    static constexpr int NUM_BARS = 24;
    static constexpr int SMEM_BYTES = 1024 + OFF_BARS + NUM_BARS * 8 + 16;
    // S0 | S1 | P0 | P1 | O; half of the tensor memory where that is enough, so that two CTAs fit an SM
    static constexpr int TMEM_COLS = (((D == 256) ? 256 : ((D == 128 && KT == 64) ? 1 : 2) * KT + KT) + D <= 256) ? 256 : 512;
    // head_dim 64 and 128 on 64-position tiles: 96 registers, 44 / 88 KB of shared memory and 256
    // columns per CTA, i.e. two CTAs and sixteen softmax warps per SM to hide the waits of one another
    // (B8 H8 S4096 D64: 582 -> 522 us; B4 H8 S4096 D128, where the 256 columns leave room for one score
    // tile only, so Q.K^T runs one tile ahead instead of two: 311 -> 297 us; 32-position tiles with two
    // score buffers at D=128: 552 us)
    static constexpr int CTAS_PER_SM = ((D == 64 || D == 128) && KT == 64) ? 2 : 1;
    // score tiles of KT int32 columns: two, or one where the other would cost the second CTA per SM
    static constexpr int NSB = (D == 128 && KT == 64) ? 1 : 2;
    static constexpr int TM_S0 = 0;
    static constexpr int TM_P = NSB * KT;                  // two fp16 P tiles of KT / 2 columns (two values per column)
    static constexpr int TM_O = (D == 256) ? 256 : TM_P + KT; // fp32 output, D columns
    static_assert(TM_P + KT <= TM_O && TM_O + D <= TMEM_COLS, "tensor-memory layout");
    static_assert(SMEM_BYTES <= 232448, "shared memory of an SM");
};

enum Bar : int {
    B_QFULL = 0,
    B_KFULL = 1,      // [kRing]
    B_KEMPTY = 4,     // [kRing]
    B_SFULL = 7,      // [2]
    B_SEMPTY = 9,     // [2]
    B_PFULL = 11,     // [2]
    B_V16FULL = 13,   // [kRing]
    B_V16EMPTY = 16,  // [kRing]
    B_PVDONE = 19,    // [2]
};

// Pre-pass: V16[row][d] = fp16(V[row][d] * sV[row]) -- one rounding, from the fp32 product.
// 16 elements per thread; rows of D int8.
__global__ void __launch_bounds__(256)
dequant_v_kernel(const int8_t* __restrict__ V, const float* __restrict__ sV, __half* __restrict__ V16,
                 long long vecs, int vecs_per_row, uint32_t* __restrict__ status) {
    pdl_wait();
    pdl_launch_dependents();
    if (blockIdx.x == 0 && threadIdx.x == 0) clear_call_status(status);
    for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < vecs;
         v += (long long)gridDim.x * blockDim.x) {
        const float sc = sV[v / vecs_per_row];
        const uint4 w = *reinterpret_cast<const uint4*>(V + v * 16);
        const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
        uint32_t o[8];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float f0 = (float)(int)(int8_t)(ww[k] & 0xff) * sc, f1 = (float)(int)(int8_t)((ww[k] >> 8) & 0xff) * sc;
            const float f2 = (float)(int)(int8_t)((ww[k] >> 16) & 0xff) * sc, f3 = (float)(int)(int8_t)(ww[k] >> 24) * sc;
            const __half2 ha = __floats2half2_rn(f0, f1), hb = __floats2half2_rn(f2, f3);
            o[2 * k] = *reinterpret_cast<const uint32_t*>(&ha);
            o[2 * k + 1] = *reinterpret_cast<const uint32_t*>(&hb);
        }
        *reinterpret_cast<uint4*>(V16 + v * 16) = make_uint4(o[0], o[1], o[2], o[3]);
        *reinterpret_cast<uint4*>(V16 + v * 16 + 8) = make_uint4(o[4], o[5], o[6], o[7]);
    }
}

__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}

template <int D, int KT>
__global__ void __launch_bounds__(kPrefillThreads, PrefillCfg<D, KT>::CTAS_PER_SM)
prefill_attention_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                         const __grid_constant__ CUtensorMap tmV, const float* __restrict__ sQ,
                         const float* __restrict__ sK,
                         __half* __restrict__ out, int S, float score_scale_log2,
                         uint32_t* __restrict__ status) {
    using Cfg = PrefillCfg<D, KT>;
    constexpr int kKT = KT;
    constexpr int HK = Cfg::HK;
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw_s = smem_u32(smem_raw);
    const uint32_t base_s = (raw_s + 1023u) & ~1023u;       // swizzle patterns are functions of address bits
    unsigned char* base = smem_raw + (base_s - raw_s);
    const uint32_t bars = base_s + Cfg::OFF_BARS;
    auto bar = [&](int i) -> uint32_t { return bars + 8u * i; };
    const uint32_t tmem_slot = bars + Cfg::NUM_BARS * 8;
    volatile uint32_t* tmem_slot_p = reinterpret_cast<volatile uint32_t*>(base + Cfg::OFF_BARS + Cfg::NUM_BARS * 8);

    pdl_wait();                 // stream order towards the producers of Q, K, V and the scales
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int bh = blockIdx.y;
    const int q0 = blockIdx.x * kQT;
    const int nt = (S + kKT - 1) / kKT;                     // KV tiles; the last one may be partial
    const int tail_valid = S - (nt - 1) * kKT;              // KV positions of the last tile (1..128)
    const long long total_rows = (long long)gridDim.y * S;  // rows of the [BH*S] scale arrays
    const int row_base = bh * S;                            // first row of this (b,h) in the [BH*S, D] views

    if (threadIdx.x == 0) {
        mbar_init(bar(B_QFULL), 1);
        for (int i = 0; i < kRing; ++i) {
            mbar_init(bar(B_KFULL + i), 1);
            mbar_init(bar(B_KEMPTY + i), 1);
            mbar_init(bar(B_V16FULL + i), 1);
            mbar_init(bar(B_V16EMPTY + i), 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar(B_SFULL + i), 1);
            mbar_init(bar(B_SEMPTY + i), kSoftmaxWarps);
            mbar_init(bar(B_PFULL + i), kSoftmaxWarps);
            mbar_init(bar(B_PVDONE + i), 1);
        }
        fence_mbar_init();
    }
    if (warp == 1) tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_p;

    if (warp == 0) {
        // ================= TMA producers =================
        // Two lanes with independent loops: K tiles are freed by Q.K^T (which runs two tiles ahead),
        // V16 tiles by P.V; one loop waiting for both would make Q.K^T of tile j wait for P.V of
        // tile j-2, which is issued after it.
        if (lane == 0) {
            mbar_expect_tx(bar(B_QFULL), Cfg::Q_BYTES);
#pragma unroll
            for (int sl = 0; sl < Cfg::QK_SLABS; ++sl)
                tma_load_2d(base_s + Cfg::OFF_Q + sl * Cfg::Q_SLAB, &tmQ, sl * 128, row_base + q0, bar(B_QFULL));
            for (int j = 0; j < nt; ++j) {
                const int st = j % kRing;
                if (!mbar_wait_spin_bounded(bar(B_KEMPTY + st), ((j / kRing) & 1) ^ 1)) {
                    note_timeout(status);
                    break;
                }
                mbar_expect_tx(bar(B_KFULL + st), Cfg::K_BYTES);
#pragma unroll
                for (int sl = 0; sl < Cfg::QK_SLABS; ++sl)
                    tma_load_2d(base_s + Cfg::OFF_K + st * Cfg::K_BYTES + sl * Cfg::K_SLAB, &tmK, sl * 128,
                                row_base + j * kKT, bar(B_KFULL + st));
            }
        } else if (lane == 1) {
            for (int j = 0; j < nt; ++j) {
                const int st = j % kRing;
                if (!mbar_wait_spin_bounded(bar(B_V16EMPTY + st), ((j / kRing) & 1) ^ 1)) {
                    note_timeout(status);
                    break;
                }
                // fp16 V: one box of KT rows x 64 columns (128 bytes) per slab of the MN-major operand
                mbar_expect_tx(bar(B_V16FULL + st), Cfg::V16_BYTES);
#pragma unroll
                for (int sl = 0; sl < D / 64; ++sl)
                    tma_load_2d(base_s + Cfg::OFF_V16 + st * Cfg::V16_BYTES + sl * Cfg::V_SLAB, &tmV, sl * 128,
                                row_base + j * kKT, bar(B_V16FULL + st));
            }
        }
    } else if (warp == 1) {
        // ================= MMA issuer =================
        if (elect_one()) {
            constexpr uint32_t idesc_qk = idesc_i8(kQT, kKT);
            constexpr uint32_t idesc_pv = idesc_f16(kQT, D, true);
            bool ok = mbar_wait_spin_bounded(bar(B_QFULL), 0);
            auto issue_pv = [&](int t) -> bool {
                // O (+)= P_t . V_t : 8 steps of 16 KV positions
                if (!mbar_wait_spin_bounded(bar(B_PFULL + (t & 1)), (t >> 1) & 1)) return false;
                const int vs = t % kRing;                // stage of the V16 ring
                if (!mbar_wait_spin_bounded(bar(B_V16FULL + vs), (t / kRing) & 1)) return false;
                tc_fence_after();
                const uint32_t v16 = base_s + Cfg::OFF_V16 + vs * Cfg::V16_BYTES;
                const uint64_t db0 = smem_desc_sw128_mn(v16, Cfg::V_SLAB);
#pragma unroll
                for (int i = 0; i < kKT / 16; ++i) {
                    // A: P in tensor memory, 8 columns (16 KV positions as fp16 pairs) per step
                    const uint32_t ta = tmem_base + Cfg::TM_P + (t & 1) * (kKT / 2) + i * 8;
                    // B: MN-major fp16, 16 rows of 128 bytes per step
                    const uint64_t db = db0 + (uint64_t)(128 * i);
                    mma_f16_ta(tmem_base + Cfg::TM_O, ta, db, idesc_pv, (t | i) != 0);
                }
                tc_commit(bar(B_V16EMPTY + vs));
                tc_commit(bar(B_PVDONE + (t & 1)));
                return true;
            };
            // Q.K^T runs two tiles ahead of P.V: the softmax warps convert the scores of tile j+1
            // while they exponentiate tile j, so S(j+1) has to be on its way before P(j-1) is complete.
            for (int j = 0; j < nt + 2 && ok; ++j) {
                if (j < nt) {
                    const int st = j % Cfg::NSB;         // score buffer
                    const int kst = j % kRing;           // stage of the K ring
                    if (!mbar_wait_spin_bounded(bar(B_KFULL + kst), (j / kRing) & 1) ||
                        !mbar_wait_spin_bounded(bar(B_SEMPTY + st), ((j / Cfg::NSB) & 1) ^ 1)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t ks = base_s + Cfg::OFF_K + kst * Cfg::K_BYTES;
                    // 32 bytes of a row per instruction: +2 (16-byte units) inside a swizzled slab,
                    // the next slab after four of them (head_dim 256)
#pragma unroll
                    for (int k = 0; k < D / 32; ++k) {
                        const uint32_t qa = base_s + Cfg::OFF_Q + (k / 4) * Cfg::Q_SLAB;
                        const uint32_t ka = ks + (k / 4) * Cfg::K_SLAB;
                        const uint64_t da = (D >= 128) ? smem_desc_sw128(qa) : smem_desc_sw64(qa);
                        const uint64_t db = (D >= 128) ? smem_desc_sw128(ka) : smem_desc_sw64(ka);
                        mma_i8(tmem_base + Cfg::TM_S0 + st * kKT, da + 2 * (k % 4), db + 2 * (k % 4), idesc_qk,
                               k != 0);
                    }
                    tc_commit(bar(B_KEMPTY + kst));
                    tc_commit(bar(B_SFULL + st));
                }
                if (j >= 2) ok = issue_pv(j - 2);
            }
            if (!ok) note_timeout(status);
        }
    } else {
        // ================= softmax: half a query row (64 KV positions of every tile) per thread =================
        const int sw = warp - 2;                         // 0..7
        const int q = warp & 3;                          // TMEM lane quarter of this warp
        const int half = sw >> 2;                        // columns half*64 .. +63 of every score tile
        const int r = q * 32 + lane;                     // row inside the tile
        float* wsc = reinterpret_cast<float*>(base + Cfg::OFF_SCALES) + sw * (2 * HK);   // [tile & 1][sK[HK]] of these columns
        float* xch = reinterpret_cast<float*>(base + Cfg::OFF_XCH);                 // [2][half][row]
        // query rows past the end of a ragged sequence are computed on clamped operands and never stored
        const float qscale = sQ[min((long long)row_base + q0 + r, total_rows - 1)] * score_scale_log2;     // > 0
        const f32x2 qs2 = pack2(qscale, qscale);
        const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
        // int32 -> fp32 without the conversion unit: |q.k| <= 127*127*128 < 2^22, so adding the
        // score to the bit pattern of 1.5*2^23 and subtracting 1.5*2^23 as a float is exact
        constexpr uint32_t kMagicI = 0x4B400000u;
        const f32x2 nmagic2 = pack2(-12582912.f, -12582912.f);
        float m_ref = -INFINITY;
        f32x2 l2 = pack2(0.f, 0.f);
        bool ok = true;
        // this warp's per-position scales, fetched ahead of the tile that uses them
        float pk0, pk1 = 0.f;
        auto prefetch = [&](int j) {
            // positions past the end of the arrays (ragged last tile of the last head) read the last element
            const long long o0 = (long long)row_base + j * kKT + half * HK + lane;
            const size_t oa = (size_t)min(o0, total_rows - 1), ob = (size_t)min(o0 + 32, total_rows - 1);
            asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(pk0) : "l"(sK + oa));
            if constexpr (HK > 32) asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(pk1) : "l"(sK + ob));
        };
        auto commit_scales = [&](int j) {                // prefetched registers -> this warp's block for tile j
            float* w = wsc + (j & 1) * HK;
            w[lane] = pk0;
            if constexpr (HK > 32) w[32 + lane] = pk1;
            __syncwarp();
        };
        // y = (q.k) * sK for 8 columns of a score block held in registers, and their maximum
        auto convert8 = [&](const uint32_t* sr8, const float* k8, f32x2* y4, float& mx) {
            const float4 ka = *reinterpret_cast<const float4*>(k8);
            const float4 kb = *reinterpret_cast<const float4*>(k8 + 4);
            const f32x2 t01 = add2(pack2(__uint_as_float(sr8[0] + kMagicI), __uint_as_float(sr8[1] + kMagicI)), nmagic2);
            const f32x2 t23 = add2(pack2(__uint_as_float(sr8[2] + kMagicI), __uint_as_float(sr8[3] + kMagicI)), nmagic2);
            const f32x2 t45 = add2(pack2(__uint_as_float(sr8[4] + kMagicI), __uint_as_float(sr8[5] + kMagicI)), nmagic2);
            const f32x2 t67 = add2(pack2(__uint_as_float(sr8[6] + kMagicI), __uint_as_float(sr8[7] + kMagicI)), nmagic2);
            y4[0] = mul2(t01, pack2(ka.x, ka.y));
            y4[1] = mul2(t23, pack2(ka.z, ka.w));
            y4[2] = mul2(t45, pack2(kb.x, kb.y));
            y4[3] = mul2(t67, pack2(kb.z, kb.w));
            const float2 a = unpack2(y4[0]), b = unpack2(y4[1]), c = unpack2(y4[2]), d = unpack2(y4[3]);
            mx = max3(max3(mx, a.x, a.y), max3(b.x, b.y, c.x), fmaxf(c.y, fmaxf(d.x, d.y)));
        };
        // partial last tile: its scores were converted like any other (the operand rows past the
        // end hold the next head's data or TMA's zero fill, so they are finite); this pass, run once
        // per CTA, then removes the columns that do not exist and recomputes the maximum
        auto mask_tail = [&](f32x2* yy, float& mx) {
            mx = -INFINITY;
#pragma unroll
            for (int e = 0; e < HK / 2; ++e) {
                float2 v = unpack2(yy[e]);
                const int col = half * HK + 2 * e;
                if (col >= tail_valid) v.x = -INFINITY;
                if (col + 1 >= tail_valid) v.y = -INFINITY;
                yy[e] = pack2(v.x, v.y);
                mx = fmaxf(mx, fmaxf(v.x, v.y));
            }
        };
        // p = 2^(y*qscale - m_ref) for 8 columns, stored as four fp16 pairs into this row's lane of the
        // P tile in tensor memory (sV is already in V16)
        auto exp8 = [&](const f32x2* y4, f32x2 nm2, uint32_t dst) {
            const float2 a = unpack2(fma2(y4[0], qs2, nm2)), b = unpack2(fma2(y4[1], qs2, nm2));
            const float2 c = unpack2(fma2(y4[2], qs2, nm2)), d = unpack2(fma2(y4[3], qs2, nm2));
            const float p0 = ex2_approx(a.x), p1 = ex2_approx(a.y), p2 = ex2_approx(b.x), p3 = ex2_approx(b.y);
            const float p4 = ex2_approx(c.x), p5 = ex2_approx(c.y), p6 = ex2_approx(d.x), p7 = ex2_approx(d.y);
            l2 = add2(l2, add2(add2(pack2(p0, p1), pack2(p2, p3)), add2(pack2(p4, p5), pack2(p6, p7))));
            tmem_st4(dst, pack_h2(p0, p1), pack_h2(p2, p3), pack_h2(p4, p5), pack_h2(p6, p7));
        };

        // ---- prologue: scores of tile 0 into registers ----
        f32x2 y[HK / 2];
        float mx = -INFINITY;
        prefetch(0);
        commit_scales(0);
        if (nt > 1) prefetch(1);
        {
            const bool got = mbar_wait_spin_bounded(bar(B_SFULL), 0);
            ok = __all_sync(0xffffffffu, got);
            if (ok) {
                tc_fence_after();
                uint32_t sr[2][16];
                const uint32_t s_addr = lane_addr + Cfg::TM_S0 + half * HK;
                tmem_ld16(s_addr, sr[0]);
#pragma unroll
                for (int cc = 0; cc < HK / 16; ++cc) {
                    tmem_ld_wait(sr[cc & 1]);
                    if (cc < HK / 16 - 1) tmem_ld16(s_addr + (cc + 1) * 16, sr[(cc + 1) & 1]);
                    convert8(&sr[cc & 1][0], wsc + cc * 16, &y[cc * 8], mx);
                    convert8(&sr[cc & 1][8], wsc + cc * 16 + 8, &y[cc * 8 + 4], mx);
                }
                if (nt == 1 && tail_valid < kKT) mask_tail(y, mx);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(B_SEMPTY));
            }
        }

        for (int j = 0; j < nt && ok; ++j) {
            const int st = j & 1;
            const bool has_next = j + 1 < nt;
            // ---- row maximum across the two halves (shared memory, one named barrier per lane quarter) ----
            xch[(st * 2 + half) * kQT + r] = mx;
            asm volatile("bar.sync %0, 64;" ::"r"(1 + q) : "memory");
            mx = fmaxf(mx, xch[(st * 2 + (half ^ 1)) * kQT + r]) * qscale;     // log2 units

            // lazy reference maximum: move it only when the true one ran ahead by kLazyStep
            const bool move = mx > m_ref + kLazyStep;
            const float m_new = move ? mx : m_ref;
            const float corr = move ? ex2_approx(m_ref - m_new) : 1.0f;
            if (move) l2 = mul2(l2, pack2(corr, corr));
            const bool warp_moves = __any_sync(0xffffffffu, move);

            // ---- this tile's P buffer is free once PV of tile j-2 retired; the output accumulator
            // is touched only when the maximum moved, and then PV of tile j-1 must have retired too ----
            if (j >= 2) {
                const bool got2 = mbar_wait_spin_bounded(bar(B_PVDONE + st), ((j - 2) >> 1) & 1);
                if (!__all_sync(0xffffffffu, got2)) { ok = false; break; }
            }
            if (j > 0 && warp_moves) {
                const bool got3 = mbar_wait_spin_bounded(bar(B_PVDONE + (st ^ 1)), ((j - 1) >> 1) & 1);
                if (!__all_sync(0xffffffffu, got3)) { ok = false; break; }
                tc_fence_after();
                uint32_t o[32];                          // this thread rescales its half of the output columns
#pragma unroll 1
                for (int cc = 0; cc < D / 64; ++cc) {
                    const uint32_t oa = lane_addr + Cfg::TM_O + half * (D / 2) + cc * 32;
                    tmem_ld32(oa, o);
                    tmem_ld_wait(o);
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
                    tmem_st32(oa, o);
                }
                tmem_st_wait();
            }
            m_ref = m_new;

            // ---- exponentials of this tile (special-function unit) interleaved, 8 columns at a time,
            // with the conversion of the NEXT tile's scores (integer and FMA pipes), which take over
            // the registers the exponentials have just released ----
            const uint32_t prow = lane_addr + Cfg::TM_P + st * (kKT / 2) + half * (HK / 2);   // this thread's HK / 2 columns of P
            const f32x2 nm2 = pack2(-m_ref, -m_ref);
            mx = -INFINITY;
            if (has_next) {
                commit_scales(j + 1);
                if (j + 2 < nt) prefetch(j + 2);
                const int sb1 = (j + 1) % Cfg::NSB;       // score buffer of the next tile
                const bool got = mbar_wait_spin_bounded(bar(B_SFULL + sb1), ((j + 1) / Cfg::NSB) & 1);
                if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
                tc_fence_after();
                const float* ksc = wsc + (st ^ 1) * HK;
                const uint32_t s_addr = lane_addr + Cfg::TM_S0 + sb1 * kKT + half * HK;
                uint32_t sr[2][16];
                tmem_ld16(s_addr, sr[0]);
#pragma unroll
                for (int cc = 0; cc < HK / 16; ++cc) {
                    tmem_ld_wait(sr[cc & 1]);
                    if (cc < HK / 16 - 1) tmem_ld16(s_addr + (cc + 1) * 16, sr[(cc + 1) & 1]);
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int c = cc * 2 + h;        // 16-byte chunk of P / 8 columns
                        exp8(&y[c * 4], nm2, prow + c * 4);
                        convert8(&sr[cc & 1][h * 8], ksc + c * 8, &y[c * 4], mx);
                    }
                }
                if (j + 2 == nt && tail_valid < kKT) mask_tail(y, mx);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(B_SEMPTY + sb1));
            } else {
#pragma unroll
                for (int c = 0; c < HK / 8; ++c) exp8(&y[c * 4], nm2, prow + c * 4);
            }
            tmem_st_wait();                              // P is in tensor memory before the MMA thread is told
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(B_PFULL + st));
        }
        // ---- epilogue: O / l -> fp16, each thread its half of the output columns ----
        if (ok) {
            const bool got = mbar_wait_spin_bounded(bar(B_PVDONE + ((nt - 1) & 1)), ((nt - 1) >> 1) & 1);
            ok = __all_sync(0xffffffffu, got);
        }
        if (ok) {
            tc_fence_after();
            const float2 lp = unpack2(l2);
            float l = lp.x + lp.y;
            xch[half * kQT + r] = l;
            asm volatile("bar.sync %0, 64;" ::"r"(1 + q) : "memory");
            l += xch[(half ^ 1) * kQT + r];
            const float inv = 1.0f / l;
            __half* orow = out + ((size_t)row_base + q0 + r) * D + half * (D / 2);
            uint32_t o[32];
#pragma unroll 1
            for (int cc = 0; cc < D / 64; ++cc) {
                tmem_ld32(lane_addr + Cfg::TM_O + half * (D / 2) + cc * 32, o);
                tmem_ld_wait(o);
                uint32_t hp[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2)
                    hp[i >> 1] = pack_h2(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv);
                if (q0 + r < S) {
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        *reinterpret_cast<uint4*>(orow + cc * 32 + k * 8) =
                            make_uint4(hp[4 * k], hp[4 * k + 1], hp[4 * k + 2], hp[4 * k + 3]);
                }
            }
        } else if (lane == 0) {
            note_timeout(status);
        }
    }

    // common exit: every role ends here, then the allocating warp frees tensor memory
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}

template <int D, int KT>
int launch_prefill(const int8_t* Q, const int8_t* K, const int8_t* V, __half* out, const float* sQ,
                   const float* sK, const float* sV, int BH, int S, uint32_t* status, __half* V16,
                   cudaStream_t st) {
    using Cfg = PrefillCfg<D, KT>;
    static bool attr_done[64] = {false};
    int dev = 0;
    I8TK_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        I8TK_CUDA(cudaFuncSetAttribute(prefill_attention_kernel<D, KT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       Cfg::SMEM_BYTES));
        attr_done[dev] = true;
    }
    const unsigned long long rows = (unsigned long long)BH * S;
    // V once through the dequantiser, then the attention kernel behind it
    const long long vecs = (long long)rows * (D / 16);
    long long blocks = (vecs + 255) / 256;
    if (blocks > 148ll * 16) blocks = 148ll * 16;
    I8TK_CUDA(launch_after(dequant_v_kernel, dim3((unsigned)blocks), dim3(256), 0, st, V, sV, V16, vecs, D / 16, status));

    // Q and K as byte matrices [rows][D]: boxes of one swizzled slab (a whole row up to 128 bytes)
    const CUtensorMapSwizzle sw = (D >= 128) ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
    CUtensorMap tmQ, tmK, tmV;
    int rc = encode_map_2d_u8(&tmQ, Q, rows, D, kQT, Cfg::ROW_BYTES, sw);
    I8TK_REQUIRE(rc == 0, I8TK_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", rc);
    rc = encode_map_2d_u8(&tmK, K, rows, D, KT, Cfg::ROW_BYTES, sw);
    I8TK_REQUIRE(rc == 0, I8TK_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", rc);
    // fp16 V as a byte matrix [rows][2*D]: boxes of KT rows x 128 bytes (64 columns), 128-byte swizzle
    rc = encode_map_2d_u8(&tmV, V16, rows, 2ull * D, KT, 128, CU_TENSOR_MAP_SWIZZLE_128B);
    I8TK_REQUIRE(rc == 0, I8TK_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", rc);
    const float score_scale_log2 = 1.4426950408889634f / sqrtf((float)D);
    dim3 grid((S + kQT - 1) / kQT, BH);
    I8TK_CUDA(launch_after(prefill_attention_kernel<D, KT>, grid, dim3(kPrefillThreads), Cfg::SMEM_BYTES, st, tmQ, tmK,
                           tmV, sQ, sK, out, S, score_scale_log2, status));
    return I8TK_OK;
}

size_t attention_workspace(long long rows, int D) { return 256 + round_up((size_t)rows * D * 2, 256); }

}  // namespace
}  // namespace i8tk

using namespace i8tk;

extern "C" size_t i8tk_attention_workspace_bytes(int batch, int heads, int seq_len, int head_dim) {
    if (batch <= 0 || heads <= 0 || seq_len <= 0 || (head_dim != 64 && head_dim != 128 && head_dim != 256)) return 0;
    return attention_workspace((long long)batch * heads * seq_len, head_dim);
}

extern "C" int i8tk_attention_forward(const int8_t* Q, const int8_t* K, const int8_t* V, void* out_f16,
                                      const float* sQ, const float* sK, const float* sV, int batch,
                                      int heads, int seq_len, int head_dim, void* workspace,
                                      size_t workspace_bytes, i8tk_stream_t stream) {
    I8TK_REQUIRE(Q && K && V && out_f16 && sQ && sK && sV, I8TK_ERR_INVALID_ARGUMENT, "null pointer argument");
    I8TK_REQUIRE(batch > 0 && heads > 0 && seq_len > 0, I8TK_ERR_INVALID_ARGUMENT, "sizes must be positive");
    I8TK_REQUIRE(head_dim == 64 || head_dim == 128 || head_dim == 256, I8TK_ERR_UNSUPPORTED,
                 "prefill attention supports head_dim 64, 128 or 256 (got %d)", head_dim);
    I8TK_REQUIRE((long long)batch * heads <= 65535, I8TK_ERR_UNSUPPORTED, "batch*heads must be <= 65535");
    I8TK_REQUIRE((long long)batch * heads * seq_len < (1ll << 31), I8TK_ERR_UNSUPPORTED, "too many rows");
    I8TK_REQUIRE(aligned_to(Q, 16) && aligned_to(K, 16) && aligned_to(V, 16) && aligned_to(out_f16, 16),
                 I8TK_ERR_ALIGNMENT, "Q, K, V and out must be 16-byte aligned");
    const size_t need = attention_workspace((long long)batch * heads * seq_len, head_dim);
    I8TK_REQUIRE(workspace != nullptr && workspace_bytes >= need, I8TK_ERR_WORKSPACE,
                 "attention workspace too small: need %zu bytes, got %zu", need, workspace_bytes);
    I8TK_REQUIRE(aligned_to(workspace, 256), I8TK_ERR_ALIGNMENT, "workspace must be 256-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    uint32_t* status = static_cast<uint32_t*>(workspace);
    __half* V16 = reinterpret_cast<__half*>(static_cast<unsigned char*>(workspace) + 256);
    const int BH = batch * heads;
    if (head_dim == 64)
        return launch_prefill<64, 64>(Q, K, V, static_cast<__half*>(out_f16), sQ, sK, sV, BH, seq_len, status, V16, st);
    if (head_dim == 128)
        return launch_prefill<128, 64>(Q, K, V, static_cast<__half*>(out_f16), sQ, sK, sV, BH, seq_len, status, V16, st);
    return launch_prefill<256, 64>(Q, K, V, static_cast<__half*>(out_f16), sQ, sK, sV, BH, seq_len, status, V16, st);
}
