// Fused INT8 MLP for B200:  x.W1 -> dequant(+bias) -> GELU -> per-token requant
// -> .W2 -> dequant -> requant.
//
// Replaces int8_mlp_forward_impl and its public wrappers of the reference
// (kernels/int8_mlp.cu:999-1314): same stage arithmetic --
//   GEMM epilogue  v = (float)acc * sa[row] * sb[col] (+ bias[col]); GELU(tanh
//                  form); fp16 store; row absmax taken on the fp32 value
//                  (kernels/int8_mlp.cu:437-449)
//   requantiser    amax = max(absmax,1e-8); q = rne(clamp(fp16(v) * (127/amax)));
//                  scale = amax/127            (kernels/int8_mlp.cu:768-825)
// -- with the two GEMMs on the 5th-generation tensor cores:
//
// * tcgen05.mma kind::i8 (int8 x int8 -> int32), 128 x BN x 32 per instruction,
//   issued by one elected thread; accumulators live in tensor memory (TMEM),
//   two buffers of BN columns so the epilogue of one tile overlaps the MMAs
//   of the next.
// * Operands are K-major in shared memory in the 128-byte-swizzled layout,
//   brought in by TMA (cp.async.bulk.tensor.2d) through a ring of stages that
//   completes on mbarriers; a stage is handed back to the TMA warp by
//   tcgen05.commit when the MMAs that read it have retired.
// * Warp roles in a persistent CTA (one per SM): warp 0 = TMA producer, warp 1 =
//   TMEM allocator + MMA issuer, warps 2..17 = epilogue (four warps per TMEM lane
//   quarter, each taking a quarter of the tile's columns: tcgen05.ld 32 lanes x 16
//   columns at a time, the next load in flight while the current block goes
//   registers -> dequant / bias / GELU / absmax -> fp16, in packed fp32x2 math).
// * Fused requantisation: a tile's fp16 values wait in shared memory (a stash of
//   32 rows x BN/4 columns per warp) while the maxima of its rows are exchanged
//   with the other SMs that work on the same 128 rows -- one word per (row, tile)
//   in global memory that is its own "written" flag, no fence, atomic or counter.
//   With a short K loop (GEMM1) the tile is quantised one tile later, the maxima
//   having been read ahead of time into registers that the drain has freed; with
//   a long one (GEMM2) at once, under the MMAs of the next tile.  int8 rows leave
//   as 16-byte stores that cover whole row segments.
// * Every wait on an mbarrier is bounded; on a timeout the kernel records a
//   status word, all roles fall through to the common exit and TMEM is freed.
//
// Weights are consumed either prepacked as [N][K] (K-major operand) or as the
// reference holds them, [K][N], through MN-major operand descriptors -- no
// transpose pass in either case.
#include "tcgen05.cuh"

#include <cstdlib>
#include <type_traits>

namespace i8tk {
namespace {

constexpr int BM = 128;          // rows per tile (= TMEM lanes)
constexpr int BK = 128;          // K bytes per stage: one 128-byte swizzle row
constexpr int kEpiWarp0 = 2;     // first epilogue warp
constexpr int kEpiWarps = 16;    // four per TMEM lane quarter, each takes a quarter of the columns
constexpr int kSlices = kEpiWarps / 4;
constexpr int kGemmThreads = (kEpiWarp0 + kEpiWarps) * 32;

// STASH kernels (fused requantisation deferred by a tile: GEMM1) keep a whole tile of fp16
// values in shared memory, paid for with one pipeline stage at the wider tiles.  The kernel
// that requantises at once (GEMM2) does it from registers and spends that memory on a deeper
// operand ring: its main loop is bound by how many bytes are in flight, not by the tensor
// pipe (two stages 161 k cycles, three 110 k at M=16384 1024->4096).
// PAIR: two CTAs share a 256-row tile (cta_group::2); each stages its own 128 rows of A and
// half of B's columns, so a stage is a third smaller and the ring a half deeper.
template <int BN, bool FUSED, bool STASH, bool PAIR = false>
struct GemmCfg {
    static_assert(!PAIR || BN == 256, "CTA pairs are built for the 256-wide tile");
    static constexpr int STAGES = PAIR ? (STASH ? 4 : 6)
        : (BN == 256) ? (STASH ? 3 : 4) : (BN == 192 ? ((FUSED && !STASH) ? 5 : 4) : (STASH ? 5 : 6));
    static constexpr int HC = BN / kSlices;                  // columns per epilogue warp
    static constexpr int A_BYTES = BM * BK;
    static constexpr int B_BYTES = (PAIR ? BN / 2 : BN) * BK;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int TMEM_COLS = (2 * BN <= 256) ? 256 : 512;   // two accumulator buffers, power of two
    static constexpr int AUX_BYTES = kEpiWarps * 2 * HC * 4;        // per epilogue warp: [scale|bias][HC] fp32
    static constexpr int CMB_BYTES = 2 * kEpiWarps * 32 * 4;        // [2][quarter][slice][32 rows] row maxima
    // per epilogue warp: 32 rows x HC fp16 (STASH), 32 rows x 16 fp16 of store staging for the
    // fp16 output, nothing when the codes leave from registers
    static constexpr int CSTAGE_WARP_BYTES = STASH ? 32 * HC * 2 : (FUSED ? 0 : 32 * 32);
    static constexpr int CSTAGE_BYTES = kEpiWarps * CSTAGE_WARP_BYTES;
    static constexpr int BAR_BYTES = (2 * STAGES + 4) * 8 + 16;
    static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + AUX_BYTES + CMB_BYTES + BAR_BYTES + CSTAGE_BYTES;
};

struct EpiParams {
    const float* scale_a;     // [M] or [1]
    const float* scale_b;     // [N] or [1]
    const float* bias;        // [N] or nullptr
    __half* C;                // [M, N] fp16
    float* out_absmax;        // [1] or nullptr (atomic max, must start at 0)
    int a_per_row;
    int b_per_col;
    // fused per-row requantisation (FUSED kernels): int8 C and its row scales
    int8_t* C8;               // [M, N] int8
    float* row_scale;         // [M]
    // [M / 128][N / BN][128] row maxima, one word per (row, tile), which every bit set
    // marks as not yet written (the caller fills the array with 0xFF bytes)
    uint32_t* row_parts;
    int a_from_prev;          // A is written by the kernel launched just before this one
    // static-scale mode (non-fused kernels): when set, the epilogue writes int8 codes
    // rne(clamp(v * static_inv[0])) to C8 instead of fp16 to C
    const float* static_inv;
    int clear_status;         // this launch is the first of its call: it clears the call's status word
    float* zero_word;         // ... and zeroes this float (the tensor-wide maximum of the legacy output)
    // row-maxima flags of the OTHER GEMM of the layer, set to all ones for that GEMM's next run
    uint4* preset_ptr;
    unsigned long long preset_words16;
};

// GELU, tanh form: 0.5 x (1 + tanh(y)), y = kC (x + kA x^3)
// (kernels/int8_common.cuh:9-13).  tanh.approx has a relative error of about
// 2^-11, the same size as the fp16 rounding the value goes through next.
// GELU on a packed pair: five packed fp32 instructions and two MUFU.TANH.
__device__ __forceinline__ f32x2 gelu_tanh2(f32x2 x) {
    constexpr float kC = 0.7978845608028654f, kA = 0.044715f;
    const f32x2 u = mul2(x, x);
    const f32x2 y = mul2(x, fma2(u, pack2(kC * kA, kC * kA), pack2(kC, kC)));
    const float2 yy = unpack2(y);
    float t0, t1;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t0) : "f"(yy.x));
    asm("tanh.approx.f32 %0, %1;" : "=f"(t1) : "f"(yy.y));
    const f32x2 hx = mul2(x, pack2(0.5f, 0.5f));
    return fma2(hx, pack2(t0, t1), hx);
}

// The reference's source order, one rounding per operation and the library tanh
// (kernels/int8_mlp.cu:437-440, kernels/int8_common.cuh:9-13): what I8TK_MLP_REFERENCE_ROUNDING
// selects.  About three times the instructions of the packed form above.
__device__ __forceinline__ float epilogue_exact(float acc, float sa, float sb, float bias, bool gelu) {
    float v = __fadd_rn(__fmul_rn(__fmul_rn(acc, sa), sb), bias);
    if (gelu) {
        constexpr float kC = 0.7978845608028654f, kA = 0.044715f;
        const float cube = __fmul_rn(__fmul_rn(__fmul_rn(kA, v), v), v);
        const float t = tanhf(__fmul_rn(kC, __fadd_rn(v, cube)));
        v = __fmul_rn(__fmul_rn(0.5f, v), __fadd_rn(1.f, t));
    }
    return v;
}

// int32 accumulator -> fp32 (cvt.rn.f32.s32).  An integer/FMA-pipe emulation through 2^23
// magic numbers was measured and is slower: the conversion unit is not the bottleneck.
__device__ __forceinline__ float i2f(uint32_t acc) { return (float)(int)acc; }

// Read-only load that is issued where it is written: the compiler may not sink it down to
// its first use, which is the point of loading a tile ahead.
__device__ __forceinline__ float ld_nc_now(const float* p) {
    float v;
    asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}

// Row maxima travel between the SMs that share a row block as plain words in global
// memory: one word per (row, half tile), written once with a relaxed store and read with
// relaxed loads that go to L2.  A maximum is a non-negative float, so its sign bit is
// clear; the array starts as all ones, and a set sign bit therefore means "not written
// yet".  The word is its own flag: no fence, counter or atomic is involved.
__device__ __forceinline__ void publish_row_max(uint32_t* slot, float rmax) {
    asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(slot), "r"(__float_as_uint(rmax) & 0x7FFFFFFFu) : "memory");
}
// Lane = row.  `col` points at this lane's row in part 0; part k of the same row is 128
// words further (the array is [row block][part][128 rows], so a warp reads and writes whole
// 128-byte lines).  Waits (bounded) until all `parts` words are written and returns their
// maximum; false in *ok when the wait ran out.
constexpr int kGatherAhead = 16;   // parts per row that can be looked at ahead of time
__device__ __forceinline__ void gather_issue(const uint32_t* col, int parts, uint32_t (&g)[kGatherAhead]) {
#pragma unroll
    for (int k = 0; k < kGatherAhead; ++k) {
        g[k] = 0u;
        if (k < parts)
            asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(g[k]) : "l"(col + k * 128) : "memory");
    }
}
// True (for the whole warp) when the early look found every word written; *mx is then the row's maximum.
__device__ __forceinline__ bool gather_check(const uint32_t (&g)[kGatherAhead], float* mx) {
    uint32_t any = 0u;
    float m = 0.f;
#pragma unroll
    for (int k = 0; k < kGatherAhead; ++k) {
        any |= g[k];
        m = fmaxf(m, __uint_as_float(g[k]));
    }
    *mx = m;
    return __all_sync(0xffffffffu, (any & 0x80000000u) == 0u);
}
__device__ __forceinline__ float gather_row_max(const uint32_t* col, int parts, bool* ok) {
    float mx = 0.f;
    bool ready = false;
    for (uint32_t spin = 0; spin < (1u << 16); ++spin) {
        uint32_t any = 0u;
        mx = 0.f;
#pragma unroll 8
        for (int k = 0; k < parts; ++k) {
            uint32_t a;
            asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(a) : "l"(col + k * 128) : "memory");
            any |= a;
            mx = fmaxf(mx, __uint_as_float(a));
        }
        ready = (any & 0x80000000u) == 0u;
        if (__all_sync(0xffffffffu, ready)) break;
    }
    *ok = ready;
    return mx;
}

// 16-byte slot of chunk j of row r in a warp's stash (rows of HC fp16, HC / 8 chunks): XOR
// with low row bits spreads a column of chunks over the banks and stays inside the row.
template <int HC>
__device__ __forceinline__ int stash_swz(int r, int j) {
    constexpr int kChunks = HC / 8;
    constexpr int kMask = (kChunks % 8 == 0) ? 7 : ((kChunks % 4 == 0) ? 3 : 1);
    return j ^ (r & kMask);
}

// Eight fp16 values (one 16-byte chunk) * inv -> eight int8, round to nearest even: adding
// 1.5 * 2^23 leaves the integer in the low mantissa bits, whose low byte is the int8 code.
template <bool CLAMP>
__device__ __forceinline__ uint2 quant8_f16(uint4 h, f32x2 inv2) {
    const f32x2 magic2 = pack2(12582912.f, 12582912.f);
    const __half2* hp = reinterpret_cast<const __half2*>(&h);
    uint32_t b[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float2 f = __half22float2(hp[k]);
        f32x2 t = mul2(pack2(f.x, f.y), inv2);
        if (CLAMP) {
            const float2 tt = unpack2(t);
            t = pack2(fmaxf(-128.f, fminf(127.f, tt.x)), fmaxf(-128.f, fminf(127.f, tt.y)));
        }
        const float2 rr = unpack2(add2(t, magic2));
        b[k] = prmt(__float_as_uint(rr.x), __float_as_uint(rr.y), 0x0040u);
    }
    return make_uint2(prmt(b[0], b[1], 0x5410u), prmt(b[2], b[3], 0x5410u));
}

__device__ __forceinline__ void atomic_max_pos(float* addr, float v) {
    atomicMax(reinterpret_cast<int*>(addr), __float_as_int(v));   // non-negative floats order as ints
}

// ---------------------------------------------------------------------------
// C[M,N] fp16 = epilogue( A[M,K] int8 . B[N,K]^T int8 ), persistent over tiles.
// N % BN == 0, K % 128 == 0; any M >= 1: the last row block may be partial (TMA fills the
// missing rows of A with zeros; nothing is stored for rows >= M).
// ---------------------------------------------------------------------------
template <int BN, bool GELU, bool FUSED, bool DEFER, bool EXACT = false, bool PAIR = false>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_i8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               EpiParams ep, int M, int N, int K, int b_mn, uint32_t* __restrict__ status) {
    using Cfg = GemmCfg<BN, FUSED, FUSED && DEFER, PAIR>;
    constexpr int STAGES = Cfg::STAGES;

    extern __shared__ unsigned char smem_raw[];
    // 1024-byte alignment: the swizzle pattern is a function of the address bits
    const uint32_t raw_s = smem_u32(smem_raw);
    const uint32_t base_s = (raw_s + 1023u) & ~1023u;
    unsigned char* base = smem_raw + (base_s - raw_s);
    float* aux = reinterpret_cast<float*>(base + STAGES * Cfg::STAGE_BYTES);
    float* cmb = reinterpret_cast<float*>(base + STAGES * Cfg::STAGE_BYTES + Cfg::AUX_BYTES);
    constexpr int kBarOff = STAGES * Cfg::STAGE_BYTES + Cfg::AUX_BYTES + Cfg::CMB_BYTES;
    const uint32_t bars = base_s + kBarOff;
    const uint32_t full0 = bars;                       // [STAGES]  TMA landed
    const uint32_t empty0 = bars + STAGES * 8;         // [STAGES]  MMAs done with the stage
    const uint32_t tfull0 = bars + 2 * STAGES * 8;     // [2]       accumulator complete
    const uint32_t tempty0 = tfull0 + 16;              // [2]       accumulator drained
    const uint32_t tmem_slot = tempty0 + 16;
    volatile uint32_t* tmem_slot_p = reinterpret_cast<volatile uint32_t*>(base + kBarOff + (2 * STAGES + 4) * 8);
    unsigned char* cstage_base = base + kBarOff + Cfg::BAR_BYTES;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int tiles_n = N / BN;
    const int row_blocks = (M + BM - 1) / BM;
    // a unit of the persistent loop: one tile, or with PAIR the two tiles of a 256-row block
    // that a CTA pair works on together (the odd CTA's tile may lie wholly below row M)
    const int num_tiles = PAIR ? ((row_blocks + 1) / 2) * tiles_n : row_blocks * tiles_n;
    const int kblocks = K / BK;
    const uint32_t cta_rank = PAIR ? cluster_ctarank() : 0u;
    const int u0 = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    const int ustride = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    auto unit_m0 = [&](int u) { return PAIR ? (u / tiles_n) * (2 * BM) + (int)cta_rank * BM : (u / tiles_n) * BM; };

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(tfull0 + 8 * b, 1);
            mbar_init(tempty0 + 8 * b, PAIR ? 2 * kEpiWarps : kEpiWarps);     // one arrival per epilogue warp
        }
        fence_mbar_init();
    }
    if (warp == 1) {
        if constexpr (PAIR) tmem_alloc_pair(tmem_slot, Cfg::TMEM_COLS);
        else tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    }
    tc_fence_before();
    __syncthreads();
    if constexpr (PAIR) cluster_sync_all();    // the partner's barriers exist before anything is sent to them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_p;
    pdl_launch_dependents();                    // the next GEMM may set itself up as SMs become free

    if (warp == 0) {
        // ================= TMA producer =================
        if (elect_one()) {
            int it = 0;
            bool ok = true;
            if (ep.a_from_prev) pdl_wait();              // A comes from the kernel before this one
            for (int tile = u0; tile < num_tiles && ok; tile += ustride) {
                const int m0 = unit_m0(tile);
                const int n0 = (tile % tiles_n) * BN;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int st = it % STAGES;
                    if (!mbar_wait_spin_bounded(empty0 + 8 * st, ((it / STAGES) & 1) ^ 1)) {
                        note_timeout(status);
                        ok = false;
                        break;
                    }
                    const uint32_t sa = base_s + st * Cfg::STAGE_BYTES;
                    if constexpr (PAIR) {
                        // both CTAs' bytes are counted on the even CTA's barrier: its MMA warp
                        // starts when the whole 256-row stage is there
                        const uint32_t fbar = mapa_shared(full0 + 8 * st, 0);
                        if (cta_rank == 0) mbar_expect_tx(full0 + 8 * st, 2 * Cfg::STAGE_BYTES);
                        const int nb = n0 + (int)cta_rank * (BN / 2);
                        tma_load_2d_pair(sa, &tmA, kb * BK, m0, fbar);
                        if (!b_mn) tma_load_2d_pair(sa + Cfg::A_BYTES, &tmB, kb * BK, nb, fbar);
                        else tma_load_2d_pair(sa + Cfg::A_BYTES, &tmB, nb, kb * BK, fbar);
                        continue;
                    }
                    mbar_expect_tx(full0 + 8 * st, Cfg::STAGE_BYTES);
                    tma_load_2d(sa, &tmA, kb * BK, m0, full0 + 8 * st);
                    if (!b_mn) {
                        tma_load_2d(sa + Cfg::A_BYTES, &tmB, kb * BK, n0, full0 + 8 * st);
                    } else {
                        // weight held as [K][N]: one box of 128 k-rows x 128 n-bytes per 128-wide slab
#pragma unroll
                        for (int j = 0; j < BN / 128; ++j)
                            tma_load_2d(sa + Cfg::A_BYTES + j * (128 * BK), &tmB, n0 + j * 128, kb * BK,
                                        full0 + 8 * st);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ================= MMA issuer =================
        if (cta_rank == 0 && elect_one()) {
            const uint32_t idesc = idesc_i8(PAIR ? 2 * BM : BM, BN, b_mn != 0);
            int it = 0, lt = 0;
            bool ok = true;
            for (int tile = u0; tile < num_tiles && ok; tile += ustride, ++lt) {
                const int buf = lt & 1;
                if (!mbar_wait_spin_bounded(tempty0 + 8 * buf, ((lt >> 1) & 1) ^ 1)) {
                    note_timeout(status);
                    break;
                }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + buf * BN;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int st = it % STAGES;
                    if (!mbar_wait_spin_bounded(full0 + 8 * st, (it / STAGES) & 1)) {
                        note_timeout(status);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sa = base_s + st * Cfg::STAGE_BYTES;
                    const uint64_t da = smem_desc_sw128(sa);
                    const uint64_t db = b_mn ? smem_desc_sw128_mn(sa + Cfg::A_BYTES, 128 * BK)
                                             : smem_desc_sw128(sa + Cfg::A_BYTES);
                    // per instruction 32 of K: K-major operands advance 32 bytes (+2 in 16-byte
                    // units); the MN-major one advances 32 rows of 128 bytes (+256)
                    const uint32_t db_step = b_mn ? 256u : 2u;
#pragma unroll
                    for (int k = 0; k < BK / 32; ++k) {
                        if constexpr (PAIR) mma_i8_pair(tmem_d, da + 2 * k, db + (uint64_t)(db_step * k), idesc, (kb | k) != 0);
                        else mma_i8(tmem_d, da + 2 * k, db + (uint64_t)(db_step * k), idesc, (kb | k) != 0);
                    }
                    // stage reusable when these MMAs retire (PAIR: in both CTAs)
                    if constexpr (PAIR) tc_commit_pair(empty0 + 8 * st, 3);
                    else tc_commit(empty0 + 8 * st);
                }
                if (ok) {                                 // accumulator complete
                    if constexpr (PAIR) tc_commit_pair(tfull0 + 8 * buf, 3);
                    else tc_commit(tfull0 + 8 * buf);
                }
            }
        }
    } else {
        // ================= epilogue =================
        const int ew = warp - kEpiWarp0;                  // 0..15
        const int q = warp & 3;                           // TMEM lane quarter this warp may read
        const int slice = ew >> 2;                        // which quarter of the tile's columns
        constexpr int HC = Cfg::HC;                       // columns per warp
        constexpr int NCH = HC / 16;                      // 16-column blocks per warp
        constexpr int NPF = (HC + 31) / 32;
        const int c0 = slice * HC;
        float* sb = aux + ew * (2 * HC);                  // this warp's column scales ...
        float* bb = sb + HC;                              // ... and bias, in shared memory
        unsigned char* cst = cstage_base + ew * Cfg::CSTAGE_WARP_BYTES;

        // Column scales, bias and the row scale are fetched one tile ahead (registers), and
        // dropped into this warp's block of shared memory just before the tile that uses them.
        float pf_s[NPF], pf_b[NPF], pf_sa = 0.f;
        auto prefetch = [&](int tile) {
            const int pm0 = unit_m0(tile), pn0 = (tile % tiles_n) * BN;
#pragma unroll
            for (int j = 0; j < NPF; ++j) {
                const int cj = j * 32 + lane;
                const int col = pn0 + c0 + (cj < HC ? cj : 0);
                pf_s[j] = ld_nc_now(ep.b_per_col ? ep.scale_b + col : ep.scale_b);
                pf_b[j] = ep.bias ? ld_nc_now(ep.bias + col) : 0.f;
            }
            pf_sa = ld_nc_now(ep.a_per_row ? ep.scale_a + min(pm0 + q * 32 + lane, M - 1) : ep.scale_a);
        };
        pdl_wait();     // row scales and the row-maxima flags come from the kernels before this one
        if (ew == 0) {
            if (ep.clear_status && blockIdx.x == 0 && lane == 0) {
                clear_call_status(status);
                if (ep.zero_word) *ep.zero_word = 0.f;
            }
            // Each GEMM of the layer leaves the other one's flag array as it must be found: GEMM2
            // runs when GEMM1 has finished with its flags and the next forward's GEMM1 cannot read
            // them before GEMM2 is complete, and the other way round.  A caller that keeps the
            // workspace to itself can therefore skip the preset kernel from the second call on.
            if (ep.preset_ptr) {
                const uint4 ones = make_uint4(0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu);
                for (unsigned long long i = (unsigned long long)blockIdx.x * 32 + lane; i < ep.preset_words16;
                     i += (unsigned long long)gridDim.x * 32)
                    ep.preset_ptr[i] = ones;
            }
        }
        if (u0 < num_tiles) prefetch(u0);

        // Requantisation of a tile whose fp16 values sit in this warp's stash: wait for the
        // maxima of its row block, then 16 columns (16 bytes of int8) per lane and step, a row
        // segment of HC bytes across consecutive lanes.
        [[maybe_unused]] uint32_t gahead[(FUSED && DEFER) ? kGatherAhead : 1];
        [[maybe_unused]] auto finalize = [&](int fm0, int fn0, bool looked_ahead) {
            if constexpr (FUSED) {
                bool ok = true;
                float amax = 0.f;
                bool have = false;
                if constexpr (DEFER) {
                    if (looked_ahead) have = gather_check(gahead, &amax);
                }
                if (!have) amax = gather_row_max(ep.row_parts + (size_t)fm0 * tiles_n + q * 32 + lane, tiles_n, &ok);
                amax = fmaxf(amax, 1e-8f);
                if (!ok) {
                    // a sibling CTA never published: the row scale becomes NaN, so the failure
                    // also shows in the data, downstream and without a host round trip
                    note_timeout(status);
                    amax = __int_as_float(0x7fc00000);
                }
                const float inv_l = 127.f / amax;
                if (fn0 == 0 && slice == 0 && fm0 + q * 32 + lane < M) ep.row_scale[fm0 + q * 32 + lane] = amax / 127.f;
                constexpr int SEGS = HC / 16;              // 16-column segments per row
                int8_t* c8blk = ep.C8 + (size_t)(fm0 + q * 32) * N + fn0 + c0;
                auto body = [&](auto clamp_tag) {
                    constexpr bool kClamp = decltype(clamp_tag)::value;
#pragma unroll
                    for (int it = 0; it < SEGS; ++it) {
                        const int item = it * 32 + lane;
                        const int r = item / SEGS, seg = item % SEGS;
                        const float inv = __shfl_sync(0xffffffffu, inv_l, r);
                        const f32x2 inv2 = pack2(inv, inv);
                        const unsigned char* rowp = cst + r * (HC * 2);
                        const uint4 h0 = *reinterpret_cast<const uint4*>(rowp + (stash_swz<HC>(r, 2 * seg) << 4));
                        const uint4 h1 = *reinterpret_cast<const uint4*>(rowp + (stash_swz<HC>(r, 2 * seg + 1) << 4));
                        const uint2 w0 = quant8_f16<kClamp>(h0, inv2);
                        const uint2 w1 = quant8_f16<kClamp>(h1, inv2);
                        if (fm0 + q * 32 + r < M)
                            *reinterpret_cast<uint4*>(c8blk + (size_t)r * N + seg * 16) = make_uint4(w0.x, w0.y, w1.x, w1.y);
                    }
                };
                // values above the fp16 range were stored as inf: only then can a product
                // leave [-128, 127], so ordinary rows skip the clamp
                if (__any_sync(0xffffffffu, !(amax <= 65504.f))) body(std::true_type{});
                else body(std::false_type{});
                __syncwarp();                              // stash reads done before it is rewritten
            }
        };

        int p_m0 = -1, p_n0 = 0;                          // DEFER: tile waiting in the stash
        int lt = 0;
        for (int tile = u0; tile < num_tiles; tile += ustride, ++lt) {
            const int buf = lt & 1;
            const int m0 = unit_m0(tile);
            const int n0 = (tile % tiles_n) * BN;

            __syncwarp();
#pragma unroll
            for (int j = 0; j < NPF; ++j) {
                const int cj = j * 32 + lane;
                if (cj < HC) {
                    sb[cj] = pf_s[j];
                    bb[cj] = pf_b[j];
                }
            }
            const float sa = pf_sa;
            const f32x2 sa2 = pack2(sa, sa);
            __syncwarp();
            if (tile + ustride < num_tiles) prefetch(tile + ustride);

            const bool got = mbar_wait_spin_bounded(tfull0 + 8 * buf, (lt >> 1) & 1);
            if (!__all_sync(0xffffffffu, got)) {
                if (lane == 0) note_timeout(status);
                break;
            }
            tc_fence_after();

            float rmax = 0.f;
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN + c0;
            uint32_t hv[FUSED ? HC / 2 : 1];              // FUSED: this row's values as packed fp16
            uint32_t r[2][16];
            tmem_ld16(taddr, r[0]);
#pragma unroll
            for (int cc = 0; cc < NCH; ++cc) {
                tmem_ld_wait(r[cc & 1]);                                   // block cc is in r[cc & 1]
                if (cc + 1 < NCH) tmem_ld16(taddr + (cc + 1) * 16, r[(cc + 1) & 1]);
                if constexpr (FUSED && DEFER) {
                    // the other accumulator block is dead from here on: its registers take an
                    // early look at the previous tile's row maxima while this block is worked on
                    if (cc == NCH - 1 && p_m0 >= 0 && tiles_n <= kGatherAhead)
                        gather_issue(ep.row_parts + (size_t)p_m0 * tiles_n + q * 32 + lane, tiles_n, gahead);
                }
                const uint32_t* rr = r[cc & 1];
                uint32_t packed[8];
                [[maybe_unused]] float vf[FUSED ? 1 : 16];    // non-fused: the fp32 values, for the static-scale store
#pragma unroll
                for (int j = 0; j < 16; j += 4) {
                    const float4 s4 = *reinterpret_cast<const float4*>(sb + cc * 16 + j);
                    const float4 b4 = *reinterpret_cast<const float4*>(bb + cc * 16 + j);
                    f32x2 v01, v23;
                    if constexpr (EXACT) {
                        v01 = pack2(epilogue_exact(i2f(rr[j]), sa, s4.x, b4.x, GELU),
                                    epilogue_exact(i2f(rr[j + 1]), sa, s4.y, b4.y, GELU));
                        v23 = pack2(epilogue_exact(i2f(rr[j + 2]), sa, s4.z, b4.z, GELU),
                                    epilogue_exact(i2f(rr[j + 3]), sa, s4.w, b4.w, GELU));
                    } else {
                        v01 = fma2(mul2(pack2(i2f(rr[j]), i2f(rr[j + 1])), sa2), pack2(s4.x, s4.y), pack2(b4.x, b4.y));
                        v23 = fma2(mul2(pack2(i2f(rr[j + 2]), i2f(rr[j + 3])), sa2), pack2(s4.z, s4.w), pack2(b4.z, b4.w));
                        if (GELU) {
                            v01 = gelu_tanh2(v01);
                            v23 = gelu_tanh2(v23);
                        }
                    }
                    const float2 a = unpack2(v01), b = unpack2(v23);
                    if constexpr (!FUSED) {
                        vf[j] = a.x; vf[j + 1] = a.y; vf[j + 2] = b.x; vf[j + 3] = b.y;
                    }
                    rmax = fmaxf(fmaxf(rmax, fmaxf(fabsf(a.x), fabsf(a.y))), fmaxf(fabsf(b.x), fabsf(b.y)));
                    const __half2 ha = __floats2half2_rn(a.x, a.y);
                    const __half2 hb = __floats2half2_rn(b.x, b.y);
                    packed[j >> 1] = *reinterpret_cast<const uint32_t*>(&ha);
                    packed[(j >> 1) + 1] = *reinterpret_cast<const uint32_t*>(&hb);
                }
                if constexpr (FUSED) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) hv[cc * 8 + j] = packed[j];
                } else if (ep.static_inv != nullptr) {
                    // static-scale mode: the code is rne(clamp(v * inv)) of the fp32 value
                    // (kernels/int8_mlp.cu:905-909, kernels/int8_common.cuh:17-19); this lane's
                    // 16 codes are 16 contiguous bytes of its row
                    const float inv = *ep.static_inv;
                    uint32_t w4[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        uint32_t w = 0;
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float v = vf[4 * j + e];
                            const int c = __float2int_rn(fmaxf(-128.f, fminf(127.f, v * inv)));
                            w |= (uint32_t)(c & 0xff) << (8 * e);
                        }
                        w4[j] = w;
                    }
                    if (m0 + q * 32 + lane < M)
                        *reinterpret_cast<uint4*>(ep.C8 + (size_t)(m0 + q * 32 + lane) * N + n0 + c0 + cc * 16) =
                            make_uint4(w4[0], w4[1], w4[2], w4[3]);
                } else {
                    // 32 rows x 32 bytes through this warp's staging block, so that two lanes
                    // store each row's 32 bytes and a store instruction covers 16 rows
                    __half* cblk = ep.C + (size_t)(m0 + q * 32) * N + n0 + c0;
                    __syncwarp();
#pragma unroll
                    for (int j = 0; j < 2; ++j)
                        *reinterpret_cast<uint4*>(cst + lane * 32 + ((j ^ ((lane >> 2) & 1)) << 4)) =
                            make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
                    __syncwarp();
#pragma unroll
                    for (int it = 0; it < 2; ++it) {
                        const int rr2 = it * 16 + (lane >> 1);
                        const int j = lane & 1;
                        const uint4 v = *reinterpret_cast<const uint4*>(cst + rr2 * 32 + ((j ^ ((rr2 >> 2) & 1)) << 4));
                        if (m0 + q * 32 + rr2 < M) *reinterpret_cast<uint4*>(cblk + (size_t)rr2 * N + cc * 16 + j * 8) = v;
                    }
                }
            }
            // accumulator buffer drained: hand it back to the MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if constexpr (PAIR) mbar_arrive_cluster(mapa_shared(tempty0 + 8 * buf, 0));   // the MMA warp sits in the even CTA
                else mbar_arrive(tempty0 + 8 * buf);
            }

            if (ep.out_absmax) {
                float wmax;
                asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(wmax) : "f"(rmax));
                if (lane == 0) atomic_max_pos(ep.out_absmax, wmax);
            }

            if constexpr (FUSED) {
                // ---- the four warps that share these 32 rows combine their maxima in shared
                // memory (double buffered, one named barrier per lane quarter) and the first
                // of them publishes one word per row for this tile ----
                float* cq = cmb + (buf * 4 + q) * (kSlices * 32);
                cq[slice * 32 + lane] = rmax;
                asm volatile("bar.sync %0, %1;" ::"r"(1 + q), "n"(kSlices * 32) : "memory");
                const bool live = !PAIR || m0 < M;          // the odd CTA's rows may all lie below M
                if (slice == 0 && live) {
                    float m4 = rmax;
#pragma unroll
                    for (int k = 1; k < kSlices; ++k) m4 = fmaxf(m4, cq[k * 32 + lane]);
                    publish_row_max(ep.row_parts + ((size_t)m0 * tiles_n + (tile % tiles_n) * 128) + q * 32 + lane, m4);
                }
                if constexpr (DEFER) {
                    // requantise the PREVIOUS tile: by now every CTA that shares its row block
                    // has published, so its maxima are there at the first look
                    if (p_m0 >= 0) finalize(p_m0, p_n0, tiles_n <= kGatherAhead);
                }
                if constexpr (DEFER) {
#pragma unroll
                    for (int jc = 0; jc < HC / 8; ++jc)
                        *reinterpret_cast<uint4*>(cst + lane * (HC * 2) + (stash_swz<HC>(lane, jc) << 4)) =
                            make_uint4(hv[4 * jc], hv[4 * jc + 1], hv[4 * jc + 2], hv[4 * jc + 3]);
                    __syncwarp();
                    p_m0 = live ? m0 : -1;
                    p_n0 = n0;
                } else if (live) {
                    // at once, straight from the registers that hold this lane's row: with a long K
                    // loop the MMAs of the next tile cover the wait for the other tiles' maxima.
                    // 16 codes = one 16-byte store per 16-column block of the lane's own row.
                    bool ok = true;
                    float amax = gather_row_max(ep.row_parts + (size_t)m0 * tiles_n + q * 32 + lane, tiles_n, &ok);
                    amax = fmaxf(amax, 1e-8f);
                    if (!ok) {
                        note_timeout(status);                 // a sibling CTA never published
                        amax = __int_as_float(0x7fc00000);    // NaN scale: the failure travels with the data
                    }
                    if (n0 == 0 && slice == 0 && m0 + q * 32 + lane < M) ep.row_scale[m0 + q * 32 + lane] = amax / 127.f;
                    const float inv = 127.f / amax;
                    const f32x2 inv2 = pack2(inv, inv);
                    int8_t* c8row = ep.C8 + (size_t)(m0 + q * 32 + lane) * N + n0 + c0;
                    const bool store = m0 + q * 32 + lane < M;
                    auto codes = [&](auto clamp_tag) {
                        constexpr bool kClamp = decltype(clamp_tag)::value;
#pragma unroll
                        for (int cc = 0; cc < NCH; ++cc) {
                            const uint2 w0 = quant8_f16<kClamp>(make_uint4(hv[8 * cc], hv[8 * cc + 1], hv[8 * cc + 2], hv[8 * cc + 3]), inv2);
                            const uint2 w1 = quant8_f16<kClamp>(make_uint4(hv[8 * cc + 4], hv[8 * cc + 5], hv[8 * cc + 6], hv[8 * cc + 7]), inv2);
                            if (store) *reinterpret_cast<uint4*>(c8row + cc * 16) = make_uint4(w0.x, w0.y, w1.x, w1.y);
                        }
                    };
                    // values above the fp16 range were stored as inf: only then can a product leave
                    // [-128, 127], so ordinary rows skip the clamp
                    if (__any_sync(0xffffffffu, !(amax <= 65504.f))) codes(std::true_type{});
                    else codes(std::false_type{});
                }
            }
        }
        if constexpr (FUSED && DEFER) {
            if (p_m0 >= 0) finalize(p_m0, p_n0, false);
        }
    }

    // common exit: every role ends here, then the allocating warp frees TMEM
    tc_fence_before();
    __syncthreads();
    if constexpr (PAIR) cluster_sync_all();    // neither CTA leaves while the other may still signal it
    if (warp == 1) {
        tc_fence_after();
        if constexpr (PAIR) tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
        else tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------
// Per-tensor requantiser of the legacy output surface: fp16 [M,N] + one absmax for
// the whole tensor -> int8 [M,N], the scale goes to *tensor_scale
// (kernels/int8_mlp.cu:799-825).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
requant_tensor_kernel(const __half* __restrict__ H, const float* __restrict__ absmax,
                      int8_t* __restrict__ out, float* __restrict__ tensor_scale, long long M, int N) {
    const long long total_vec = M * N / 16;
    const float amax = fmaxf(absmax[0], 1e-8f);
    const float inv = 127.f / amax;
    if (blockIdx.x == 0 && threadIdx.x == 0) tensor_scale[0] = amax / 127.f;
    for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < total_vec;
         v += (long long)gridDim.x * blockDim.x) {
        const long long e0 = v * 16;
        const uint4 h0 = *reinterpret_cast<const uint4*>(H + e0);
        const uint4 h1 = *reinterpret_cast<const uint4*>(H + e0 + 8);
        const __half2* hp0 = reinterpret_cast<const __half2*>(&h0);
        const __half2* hp1 = reinterpret_cast<const __half2*>(&h1);
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 a = __half22float2(i < 2 ? hp0[2 * i] : hp1[2 * i - 4]);
            const float2 b = __half22float2(i < 2 ? hp0[2 * i + 1] : hp1[2 * i - 3]);
            const int q0 = __float2int_rn(fmaxf(-128.f, fminf(127.f, a.x * inv)));
            const int q1 = __float2int_rn(fmaxf(-128.f, fminf(127.f, a.y * inv)));
            const int q2 = __float2int_rn(fmaxf(-128.f, fminf(127.f, b.x * inv)));
            const int q3 = __float2int_rn(fmaxf(-128.f, fminf(127.f, b.y * inv)));
            w[i] = (uint32_t)(q0 & 0xff) | ((uint32_t)(q1 & 0xff) << 8) | ((uint32_t)(q2 & 0xff) << 16) |
                   ((uint32_t)(q3 & 0xff) << 24);
        }
        *reinterpret_cast<uint4*>(out + e0) = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

// Workspace presets of one forward: `words16` 16-byte words of all ones, one float of zero.
__global__ void __launch_bounds__(256)
preset_kernel(uint4* __restrict__ ones, size_t words16, float* __restrict__ zero, uint32_t* __restrict__ status) {
    pdl_wait();                 // plain stream order towards whatever precedes the call
    pdl_launch_dependents();
    if (blockIdx.x == 0 && threadIdx.x == 0) clear_call_status(status);
    const uint4 v = make_uint4(0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < words16; i += (size_t)gridDim.x * blockDim.x)
        ones[i] = v;
    if (blockIdx.x == 0 && threadIdx.x == 0) *zero = 0.f;
}

// int8 [R][C] -> [C][R]; 64x64 tiles, 4-byte global accesses on both sides.
__global__ void __launch_bounds__(256)
transpose_i8_kernel(const int8_t* __restrict__ in, int8_t* __restrict__ out, int R, int C) {
    __shared__ int8_t tile[64][68];
    const int c0 = blockIdx.x * 64, r0 = blockIdx.y * 64;
    const bool fast_in = (C % 4) == 0, fast_out = (R % 4) == 0;
    for (int i = threadIdx.x; i < 64 * 16; i += 256) {
        const int r = i / 16, c4 = (i % 16) * 4;
        if (r0 + r < R) {
            if (fast_in && c0 + c4 + 3 < C) {
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
            if (fast_out && r0 + r4 + 3 < R) {
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

int transpose_i8(const int8_t* in, int8_t* out, int R, int C, cudaStream_t st) {
    dim3 grid((C + 63) / 64, (R + 63) / 64);
    transpose_i8_kernel<<<grid, 256, 0, st>>>(in, out, R, C);
    I8TK_CUDA(cudaGetLastError());
    return I8TK_OK;
}

// int8 matrix [rows][cols] row-major, box of box_rows x 128 bytes, 128-byte swizzle
int make_map(CUtensorMap* map, const int8_t* ptr, int rows, int cols, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    I8TK_REQUIRE(fn != nullptr, I8TK_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(ptr), dims, strides, box,
                          estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    I8TK_REQUIRE(r == CUDA_SUCCESS, I8TK_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return I8TK_OK;
}

// int8 weight [K][N] row-major (N contiguous): box of 128 k-rows x 128 n-bytes, 128-byte swizzle
int make_map_mn(CUtensorMap* map, const int8_t* ptr, int K, int N) {
    EncodeTiledFn fn = encode_fn();
    I8TK_REQUIRE(fn != nullptr, I8TK_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)K};
    const cuuint64_t strides[1] = {(cuuint64_t)N};
    const cuuint32_t box[2] = {128u, (cuuint32_t)BK};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(ptr), dims, strides, box,
                          estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    I8TK_REQUIRE(r == CUDA_SUCCESS, I8TK_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return I8TK_OK;
}

// Encoded tensor maps of the last few (pointer, shape, box) combinations this thread asked for:
// a descriptor depends on nothing else, and a serving loop calls with the same weights and
// the same activation buffers over and over, so the driver call (about a microsecond each,
// four per forward) is paid once.
struct MapKey {
    const void* ptr;
    int a, b, box, mn;
    bool operator==(const MapKey& o) const { return ptr == o.ptr && a == o.a && b == o.b && box == o.box && mn == o.mn; }
};
int cached_map(CUtensorMap* out, const int8_t* ptr, int a, int b, int box, bool mn) {
    constexpr int kSlots = 16;
    thread_local MapKey keys[kSlots] = {};
    thread_local CUtensorMap maps[kSlots];
    thread_local int next = 0;
    const MapKey k{ptr, a, b, box, mn ? 1 : 0};
    for (int i = 0; i < kSlots; ++i)
        if (keys[i].ptr != nullptr && keys[i] == k) { *out = maps[i]; return I8TK_OK; }
    const int rc = mn ? make_map_mn(out, ptr, a, b) : make_map(out, ptr, a, b, box);
    if (rc != I8TK_OK) return rc;
    keys[next] = k;
    maps[next] = *out;
    next = (next + 1) % kSlots;
    return I8TK_OK;
}

int sm_count_mlp() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] > 0) return cached[dev];
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 148;
    cached[dev] = n;
    return n;
}
// CTAs of a persistent launch.  Fused kernels: the CTAs that share a row block wait for
// one another, so every round of the persistent loop covers whole row blocks.
int gemm_grid(int M, int N, int bn, bool fused, bool pair = false) {
    const int sms = sm_count_mlp();
    const int tiles_n = N / bn;
    const int row_blocks = (M + BM - 1) / BM;
    if (pair) {     // counted in CTA pairs, each on one 256-row unit at a time
        const long long units = (long long)((row_blocks + 1) / 2) * tiles_n;
        int pairs = units < sms / 2 ? (int)units : sms / 2;
        if (fused && pairs > tiles_n) pairs = (pairs / tiles_n) * tiles_n;
        return 2 * (pairs > 0 ? pairs : 1);
    }
    const long long tiles = (long long)row_blocks * tiles_n;
    int grid = tiles < sms ? (int)tiles : sms;
    if (fused && grid > tiles_n) grid = (grid / tiles_n) * tiles_n;
    return grid > 0 ? grid : 1;
}

// Tile width: among the widths that divide N, the one with the least
// (rounds of the persistent loop) x (tile width); ties go to the wider tile.
int pick_bn(int M, int N, bool b_mn, bool fused) {
    const int widths[3] = {256, 192, 128};
    int best = 128;
    long long best_cost = -1;
    for (int i = 0; i < 3; ++i) {
        const int bn = widths[i];
        if (N % bn) continue;
        if (b_mn && bn % 128) continue;          // [K][N] weights come in 128-wide slabs
        const long long tiles = (long long)((M + BM - 1) / BM) * (N / bn);
        const int grid = gemm_grid(M, N, bn, fused);
        const long long cost = ((tiles + grid - 1) / grid) * bn;
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = bn; }
    }
    return best;
}

template <int BN, bool GELU, bool FUSED, bool DEFER, bool EXACT = false, bool PAIR = false>
int launch_gemm(const int8_t* A, const int8_t* B, bool b_mn, const EpiParams& ep, int M, int N, int K,
                uint32_t* status, cudaStream_t st) {
    using Cfg = GemmCfg<BN, FUSED, FUSED && DEFER, PAIR>;
    static_assert(Cfg::SMEM_BYTES <= 232448, "tile configuration exceeds the shared memory of an SM");
    static bool attr_done[64] = {false};
    int dev = 0;
    I8TK_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        I8TK_CUDA(cudaFuncSetAttribute(gemm_i8_kernel<BN, GELU, FUSED, DEFER, EXACT, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       Cfg::SMEM_BYTES));
        attr_done[dev] = true;
    }
    CUtensorMap tmA, tmB;
    int rc = cached_map(&tmA, A, M, K, BM, false);
    if (rc != I8TK_OK) return rc;
    rc = b_mn ? cached_map(&tmB, B, K, N, 0, true) : cached_map(&tmB, B, N, K, PAIR ? BN / 2 : BN, false);
    if (rc != I8TK_OK) return rc;
    const int grid = gemm_grid(M, N, BN, FUSED, PAIR);
    I8TK_REQUIRE(!FUSED || N / BN <= sm_count_mlp() / (PAIR ? 2 : 1), I8TK_ERR_UNSUPPORTED,
                 "row of %d tiles does not fit one round of CTAs", N / BN);
    I8TK_CUDA(launch_after_clustered(gemm_i8_kernel<BN, GELU, FUSED, DEFER, EXACT, PAIR>, dim3(grid), dim3(kGemmThreads),
                                     Cfg::SMEM_BYTES, st, PAIR ? 2 : 1, tmA, tmB, ep, M, N, K, b_mn ? 1 : 0, status));
    return I8TK_OK;
}

// I8TK_MLP_PAIRS (read once): 0 keeps every GEMM on single CTAs, 1 puts the requantise-at-once
// GEMM on CTA pairs wherever it has two row blocks; unset: pairs where they were measured to
// pay, i.e. when the persistent loop runs more than one round (1-4 % of the forward at
// M = 8192 and 16384: a third less operand traffic into each SM, a half deeper ring; with one
// tile per CTA the cluster launch and the paired start cost more than that saves: M=4096
// 44.2 vs 42.9 us).
int pairs_mode() {
    static const int mode = [] {
        const char* e = std::getenv("I8TK_MLP_PAIRS");
        return (e && (e[0] == '0' || e[0] == '1')) ? e[0] - '0' : 2;
    }();
    return mode;
}

template <bool GELU, bool FUSED, bool DEFER, bool EXACT = false>
int launch_gemm_bn(const int8_t* A, const int8_t* B, bool b_mn, const EpiParams& ep, int M, int N, int K,
                   uint32_t* status, cudaStream_t st) {
    const int best = pick_bn(M, N, b_mn, FUSED);
    if constexpr (FUSED && !DEFER && !EXACT) {
        const int mode = pairs_mode();
        const long long tiles = (long long)((M + BM - 1) / BM) * (N / 256);
        if (best == 256 && M > BM && (mode == 1 || (mode == 2 && tiles > sm_count_mlp())))
            return launch_gemm<256, GELU, FUSED, DEFER, EXACT, true>(A, B, b_mn, ep, M, N, K, status, st);
    }
    if (best == 256) return launch_gemm<256, GELU, FUSED, DEFER, EXACT>(A, B, b_mn, ep, M, N, K, status, st);
    if (best == 192) return launch_gemm<192, GELU, FUSED, DEFER, EXACT>(A, B, b_mn, ep, M, N, K, status, st);
    return launch_gemm<128, GELU, FUSED, DEFER, EXACT>(A, B, b_mn, ep, M, N, K, status, st);
}

int requant_grid(long long vecs) {
    long long b = (vecs + 255) / 256;
    if (b > 148ll * 8) b = 148ll * 8;
    if (b < 1) b = 1;
    return (int)b;
}

// workspace carve-up
struct MlpWorkspace {
    uint32_t* status;
    float* tensor_absmax; // [1]   starts at zero (legacy per-tensor output scale only)
    float* static_scales; // [4]   static-scale mode: hidden scale, its inverse, output scale, its inverse
    uint32_t* parts1;     // [T/128][d_ff / BN1][128]     row maxima of GEMM1 per tile; these two
    uint32_t* parts2;     // [T/128][d_model / BN2][128]  are contiguous and start as 0xFF bytes
    float* hid_scale;     // [T]
    int8_t* hid_i8;       // [T, d_ff]
    __half* out_f16;      // [T, d_model]   (legacy per-tensor output scale only)
    size_t bytes;
    size_t ones_bytes;    // parts1 .. parts2
};

// d_model and d_ff are multiples of 128 here (the caller pads other widths first).
MlpWorkspace carve(void* base, int T, int d_model, int d_ff, int flags) {
    MlpWorkspace w{};
    size_t off = 0;
    auto take = [&](size_t n) { size_t o = off; off = round_up(off + n, 256); return o; };
    unsigned char* b = static_cast<unsigned char*>(base);
    const bool b_mn = !(flags & I8TK_MLP_PREPACKED);
    const size_t o_status = take(256);
    const size_t o_tabs = take(128);
    const size_t o_stat = take(128);
    const size_t Tp = (size_t)((T + 127) / 128) * 128;       // rows of the flag arrays: whole row blocks
    const size_t o_p1 = take(Tp * (d_ff / pick_bn(T, d_ff, b_mn, true)) * 4);
    const size_t o_p2 = take(Tp * (d_model / pick_bn(T, d_model, b_mn, true)) * 4);
    const size_t ones_end = off;
    const size_t o_hsc = take((size_t)T * 4);
    const size_t o_hi8 = take((size_t)T * d_ff);
    const size_t o_o16 = take((size_t)T * d_model * 2);
    w.bytes = off;
    w.ones_bytes = ones_end - o_p1;
    if (b) {
        w.status = reinterpret_cast<uint32_t*>(b + o_status);
        w.tensor_absmax = reinterpret_cast<float*>(b + o_tabs);
        w.static_scales = reinterpret_cast<float*>(b + o_stat);
        w.parts1 = reinterpret_cast<uint32_t*>(b + o_p1);
        w.parts2 = reinterpret_cast<uint32_t*>(b + o_p2);
        w.hid_scale = reinterpret_cast<float*>(b + o_hsc);
        w.hid_i8 = reinterpret_cast<int8_t*>(b + o_hi8);
        w.out_f16 = reinterpret_cast<__half*>(b + o_o16);
    }
    return w;
}

// Static-scale mode (kernels/int8_mlp.cu:830-844): hidden scale = sx*sw1*d_model (a bound that
// holds for any input), output scale = that * sw2 * d_ff; both with their reciprocals.  The
// widths are the caller's, not the padded ones.  Also clears the call's status word.
__global__ void static_scales_kernel(const float* __restrict__ sx, const float* __restrict__ sw1,
                                     const float* __restrict__ sw2, float* __restrict__ out4,
                                     float* __restrict__ out_tensor_scale, int d_model, int d_ff,
                                     uint32_t* __restrict__ status) {
    pdl_wait();
    pdl_launch_dependents();
    if (threadIdx.x != 0) return;
    clear_call_status(status);
    const float sh = sx[0] * sw1[0] * (float)d_model;
    const float so = sh * sw2[0] * (float)d_ff;
    out4[0] = sh;
    out4[1] = 1.f / sh;
    out4[2] = so;
    out4[3] = 1.f / so;
    if (out_tensor_scale) *out_tensor_scale = so;
}

// Zero-padded copy of a row-major matrix of `elem`-byte elements: dst [drows][dcols] receives
// src [srows][scols] in its top-left corner and zeros elsewhere (either may be the larger one
// in each dimension: the same kernel crops).  One thread per destination element.
__global__ void __launch_bounds__(256)
pad_copy_kernel(const unsigned char* __restrict__ src, long long srows, long long scols,
                unsigned char* __restrict__ dst, long long drows, long long dcols, int elem) {
    const long long total = drows * dcols;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / dcols, c = i - r * dcols;
        const bool in = r < srows && c < scols;
        for (int e = 0; e < elem; ++e) dst[i * elem + e] = in ? src[(r * scols + c) * elem + e] : (unsigned char)0;
    }
}

int pad_copy(const void* src, long long srows, long long scols, void* dst, long long drows, long long dcols,
             int elem, cudaStream_t st) {
    const long long total = drows * dcols;
    long long blocks = (total + 255) / 256;
    if (blocks > 148ll * 16) blocks = 148ll * 16;
    if (blocks < 1) blocks = 1;
    pad_copy_kernel<<<(unsigned)blocks, 256, 0, st>>>(static_cast<const unsigned char*>(src), srows, scols,
                                                      static_cast<unsigned char*>(dst), drows, dcols, elem);
    I8TK_CUDA(cudaGetLastError());
    return I8TK_OK;
}

inline int pad128(int v) { return (v + 127) / 128 * 128; }

// Buffers of the padded route (widths that are not multiples of 128), behind the core's workspace.
struct PadLayout {
    size_t x, w1, w2, s1, s2, b1, out, total;
};
PadLayout pad_layout(size_t core_bytes, int T, int dmp, int dffp) {
    PadLayout l;
    size_t off = core_bytes;
    auto take = [&](size_t n) { size_t o = off; off = round_up(off + n, 256); return o; };
    l.x = take((size_t)T * dmp);
    l.w1 = take((size_t)dmp * dffp);
    l.w2 = take((size_t)dmp * dffp);
    l.s1 = take((size_t)dffp * 4);
    l.s2 = take((size_t)dmp * 4);
    l.b1 = take((size_t)dffp * 4);
    l.out = take((size_t)T * dmp);
    l.total = off;
    return l;
}

// The forward on widths that are multiples of 128.  `true_dm` / `true_dff` are the caller's
// widths (they differ from d_model / d_ff on the padded route and only enter the static scales).
int mlp_core(const int8_t* x, const int8_t* W1, const int8_t* W2, int8_t* out, const float* scale_x,
             const float* scale_W1, const float* scale_W2, const float* bias1, float* out_row_scales,
             float* out_tensor_scale, int T, int d_model, int d_ff, int true_dm, int true_dff, int flags,
             const MlpWorkspace& w, cudaStream_t st) {
    // Weights as the caller holds them ([K][N], N contiguous) are read in place through
    // MN-major operand descriptors; prepacked ones ([N][K]) through K-major descriptors.
    const bool b_mn = !(flags & I8TK_MLP_PREPACKED);
    const bool exact = (flags & I8TK_MLP_REFERENCE_ROUNDING) != 0;
    int rc;
    const int per_token = (flags & I8TK_MLP_X_PER_TOKEN) ? 1 : 0;
    const int per_channel = (flags & I8TK_MLP_W_PER_CHANNEL) ? 1 : 0;

    if (flags & I8TK_MLP_STATIC_SCALES) {
        // GEMM1 writes int8 hidden codes under the static hidden scale, GEMM2 int8 output codes
        // under the static output scale (kernels/int8_mlp.cu:1194-1225); no row maxima, no fp16.
        I8TK_CUDA(launch_after(static_scales_kernel, dim3(1), dim3(32), 0, st, scale_x, scale_W1, scale_W2,
                               w.static_scales, out_tensor_scale, true_dm, true_dff, w.status));
        EpiParams e1{scale_x, scale_W1, nullptr, nullptr, nullptr, 0, 0, w.hid_i8, nullptr, nullptr, 1,
                     w.static_scales + 1, 0, nullptr, nullptr, 0};
        rc = exact ? launch_gemm<128, true, false, false, true>(x, W1, b_mn, e1, T, d_ff, d_model, w.status, st)
                   : launch_gemm<128, true, false, false, false>(x, W1, b_mn, e1, T, d_ff, d_model, w.status, st);
        if (rc != I8TK_OK) return rc;
        EpiParams e2{w.static_scales, scale_W2, nullptr, nullptr, nullptr, 0, 0, out, nullptr, nullptr, 1,
                     w.static_scales + 3, 0, nullptr, nullptr, 0};
        return launch_gemm<128, false, false, false, false>(w.hid_i8, W2, b_mn, e2, T, d_model, d_ff, w.status, st);
    }

    // presets: row-maxima flags all ones, the tensor-wide maximum zero, the call's status word
    // clear.  A kernel rather than a memset so that GEMM1 can be launched behind it
    // programmatically and set itself up meanwhile.  With I8TK_MLP_WORKSPACE_KEPT the previous
    // forward on this workspace has left the flags preset (each GEMM resets the other's array)
    // and GEMM1 clears the two words itself: no preset launch.
    const bool kept = (flags & I8TK_MLP_WORKSPACE_KEPT) != 0;
    // sizes of the two flag arrays as carve() lays them out
    const size_t p1_words = (size_t)(reinterpret_cast<unsigned char*>(w.parts2) - reinterpret_cast<unsigned char*>(w.parts1)) / 16;
    const size_t p2_words = w.ones_bytes / 16 - p1_words;
    if (!kept) {
        const size_t words = w.ones_bytes / 16;
        int blocks = (int)((words + 255) / 256);
        if (blocks > 296) blocks = 296;
        if (blocks < 1) blocks = 1;
        I8TK_CUDA(launch_after(preset_kernel, dim3(blocks), dim3(256), 0, st, reinterpret_cast<uint4*>(w.parts1),
                               words, w.tensor_absmax, w.status));
    }

    // GEMM1: hidden = GELU((x . W1) * sx * sW1 + b1), requantised per token inside the
    // GEMM's epilogue: the fp16 values of a tile wait in shared memory while the row
    // maxima of its row block (12-16 tiles on as many SMs) are exchanged through global
    // memory, and are quantised one tile later, when that exchange has long finished.
    {
        // a_from_prev: x may come from the kernel launched just before this one (a quantiser that
        // lets its successor start early), so the producer warp waits for it like everyone else
        EpiParams e1{scale_x, scale_W1, bias1, nullptr, nullptr, per_token, per_channel,
                     w.hid_i8, w.hid_scale, w.parts1, 1, nullptr, kept ? 1 : 0, w.tensor_absmax,
                     reinterpret_cast<uint4*>(w.parts2), p2_words};
        if (exact)
            rc = launch_gemm_bn<true, true, true, true>(x, W1, b_mn, e1, T, d_ff, d_model, w.status, st);
        else
            rc = launch_gemm_bn<true, true, true>(x, W1, b_mn, e1, T, d_ff, d_model, w.status, st);
        if (rc != I8TK_OK) return rc;
    }
    if (out_row_scales) {
        // GEMM2: out = (hidden_i8 . W2) * sh * sW2, requantised per token the same way, but
        // at once: with K = d_ff the MMAs of the next tile cover the exchange
        EpiParams e2{w.hid_scale, scale_W2, nullptr, nullptr, nullptr, 1, per_channel,
                     out, out_row_scales, w.parts2, 1, nullptr, 0, nullptr, reinterpret_cast<uint4*>(w.parts1), p1_words};
        return launch_gemm_bn<false, true, false>(w.hid_i8, W2, b_mn, e2, T, d_model, d_ff, w.status, st);
    }
    // legacy per-tensor output scale: fp16 out + global absmax, then one requant pass
    EpiParams e2{w.hid_scale, scale_W2, nullptr, w.out_f16, w.tensor_absmax, 1, per_channel,
                 nullptr, nullptr, nullptr, 1, nullptr, 0, nullptr, reinterpret_cast<uint4*>(w.parts1), p1_words};
    rc = launch_gemm_bn<false, false, false>(w.hid_i8, W2, b_mn, e2, T, d_model, d_ff, w.status, st);
    if (rc != I8TK_OK) return rc;
    requant_tensor_kernel<<<requant_grid((long long)T * d_model / 16), 256, 0, st>>>(
        w.out_f16, w.tensor_absmax, out, out_tensor_scale, T, d_model);
    I8TK_CUDA(cudaGetLastError());
    return I8TK_OK;
}

}  // namespace
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

extern "C" int i8tk_linear_i8_f16(const int8_t* x, const int8_t* W, const float* scale_x, const float* scale_W,
                                  const float* bias, void* out_f16, int T, int K, int N, int flags,
                                  void* workspace, size_t workspace_bytes, i8tk_stream_t stream) {
    I8TK_REQUIRE(x && W && scale_x && scale_W && out_f16, I8TK_ERR_INVALID_ARGUMENT, "null pointer argument");
    I8TK_REQUIRE(T > 0 && K > 0 && N > 0, I8TK_ERR_INVALID_ARGUMENT, "sizes must be positive");
    I8TK_REQUIRE((flags & ~(I8TK_MLP_PREPACKED | I8TK_MLP_X_PER_TOKEN | I8TK_MLP_W_PER_CHANNEL)) == 0,
                 I8TK_ERR_INVALID_ARGUMENT, "unknown flag bits 0x%x", flags);
    I8TK_REQUIRE(K % 128 == 0 && N % 128 == 0, I8TK_ERR_UNSUPPORTED,
                 "K and N must be multiples of 128 (got %d, %d)", K, N);
    I8TK_REQUIRE(aligned_to(x, 16) && aligned_to(W, 16) && aligned_to(out_f16, 16), I8TK_ERR_ALIGNMENT,
                 "x, W and out must be 16-byte aligned");
    I8TK_REQUIRE(workspace != nullptr && workspace_bytes >= 256 && aligned_to(workspace, 256), I8TK_ERR_WORKSPACE,
                 "workspace: 256 bytes, 256-byte aligned (the status block)");
    const bool b_mn = !(flags & I8TK_MLP_PREPACKED);
    EpiParams e{scale_x, scale_W, bias, static_cast<__half*>(out_f16), nullptr, (flags & I8TK_MLP_X_PER_TOKEN) ? 1 : 0,
                (flags & I8TK_MLP_W_PER_CHANNEL) ? 1 : 0, nullptr, nullptr, nullptr, 1, nullptr, 1, nullptr, nullptr, 0};
    return launch_gemm_bn<false, false, false>(x, W, b_mn, e, T, N, K, static_cast<uint32_t*>(workspace),
                                               static_cast<cudaStream_t>(stream));
}

extern "C" size_t i8tk_mlp_workspace_bytes(int T, int d_model, int d_ff, int flags) {
    if (T <= 0 || d_model <= 0 || d_ff <= 0) return 0;
    const int dmp = pad128(d_model), dffp = pad128(d_ff);
    const size_t core = carve(nullptr, T, dmp, dffp, flags).bytes;
    if (dmp == d_model && dffp == d_ff) return core;
    return pad_layout(core, T, dmp, dffp).total;
}

extern "C" int i8tk_mlp_forward(const int8_t* x, const int8_t* W1, const int8_t* W2, int8_t* out,
                                const float* scale_x, const float* scale_W1, const float* scale_W2,
                                const float* bias1, float* out_row_scales, float* out_tensor_scale,
                                int T, int d_model, int d_ff, int flags, void* workspace,
                                size_t workspace_bytes, i8tk_stream_t stream) {
    I8TK_REQUIRE(x && W1 && W2 && out && scale_x && scale_W1 && scale_W2, I8TK_ERR_INVALID_ARGUMENT,
                 "null pointer argument");
    I8TK_REQUIRE(out_row_scales || out_tensor_scale, I8TK_ERR_INVALID_ARGUMENT,
                 "one of out_row_scales / out_tensor_scale must be given");
    I8TK_REQUIRE(T > 0 && d_model > 0 && d_ff > 0, I8TK_ERR_INVALID_ARGUMENT, "sizes must be positive");
    I8TK_REQUIRE((flags & ~63) == 0, I8TK_ERR_INVALID_ARGUMENT, "unknown flag bits 0x%x", flags);
    if (flags & I8TK_MLP_STATIC_SCALES) {
        I8TK_REQUIRE(!(flags & (I8TK_MLP_X_PER_TOKEN | I8TK_MLP_W_PER_CHANNEL)) && bias1 == nullptr &&
                         out_row_scales == nullptr && out_tensor_scale != nullptr,
                     I8TK_ERR_INVALID_ARGUMENT,
                     "static-scale mode takes per-tensor scales, no bias, and reports one output scale");
    }
    const int dmp = pad128(d_model), dffp = pad128(d_ff);
    const bool padded = dmp != d_model || dffp != d_ff;
    const size_t core_bytes = carve(nullptr, T, dmp, dffp, flags).bytes;
    const size_t need = padded ? pad_layout(core_bytes, T, dmp, dffp).total : core_bytes;
    I8TK_REQUIRE(workspace != nullptr && workspace_bytes >= need, I8TK_ERR_WORKSPACE,
                 "mlp workspace too small: need %zu bytes, got %zu", need, workspace_bytes);
    I8TK_REQUIRE(aligned_to(workspace, 256), I8TK_ERR_ALIGNMENT, "workspace must be 256-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const MlpWorkspace w = carve(workspace, T, dmp, dffp, flags);
    if (!padded) {
        I8TK_REQUIRE(aligned_to(x, 16) && aligned_to(W1, 16) && aligned_to(W2, 16) && aligned_to(out, 16),
                     I8TK_ERR_ALIGNMENT, "x, W1, W2 and out must be 16-byte aligned");
        return mlp_core(x, W1, W2, out, scale_x, scale_W1, scale_W2, bias1, out_row_scales, out_tensor_scale, T,
                        d_model, d_ff, d_model, d_ff, flags, w, st);
    }

    // Widths that are not multiples of 128 (the reference sends these to its scalar kernels,
    // kernels/int8_mlp.cu:1023-1026): operands are copied into zero-padded buffers of the next
    // multiple of 128 and the tensor-core forward runs on those.  Zero columns of x and zero
    // rows of W1 add nothing to a dot product; padded hidden channels are GELU(0) = 0, never the
    // row maximum, and meet zero rows of W2; padded output columns are zero and are cropped.
    unsigned char* base = static_cast<unsigned char*>(workspace);
    const PadLayout l = pad_layout(core_bytes, T, dmp, dffp);
    int8_t* xp = reinterpret_cast<int8_t*>(base + l.x);
    int8_t* w1p = reinterpret_cast<int8_t*>(base + l.w1);
    int8_t* w2p = reinterpret_cast<int8_t*>(base + l.w2);
    float* s1p = reinterpret_cast<float*>(base + l.s1);
    float* s2p = reinterpret_cast<float*>(base + l.s2);
    float* b1p = reinterpret_cast<float*>(base + l.b1);
    int8_t* outp = reinterpret_cast<int8_t*>(base + l.out);
    const bool prepacked = (flags & I8TK_MLP_PREPACKED) != 0;
    const bool per_channel = (flags & I8TK_MLP_W_PER_CHANNEL) != 0;
    int rc = pad_copy(x, T, d_model, xp, T, dmp, 1, st);
    if (rc != I8TK_OK) return rc;
    rc = prepacked ? pad_copy(W1, d_ff, d_model, w1p, dffp, dmp, 1, st) : pad_copy(W1, d_model, d_ff, w1p, dmp, dffp, 1, st);
    if (rc != I8TK_OK) return rc;
    rc = prepacked ? pad_copy(W2, d_model, d_ff, w2p, dmp, dffp, 1, st) : pad_copy(W2, d_ff, d_model, w2p, dffp, dmp, 1, st);
    if (rc != I8TK_OK) return rc;
    if (per_channel) {
        rc = pad_copy(scale_W1, 1, d_ff, s1p, 1, dffp, 4, st);
        if (rc != I8TK_OK) return rc;
        rc = pad_copy(scale_W2, 1, d_model, s2p, 1, dmp, 4, st);
        if (rc != I8TK_OK) return rc;
    }
    if (bias1) {
        rc = pad_copy(bias1, 1, d_ff, b1p, 1, dffp, 4, st);
        if (rc != I8TK_OK) return rc;
    }
    rc = mlp_core(xp, w1p, w2p, outp, scale_x, per_channel ? s1p : scale_W1, per_channel ? s2p : scale_W2,
                  bias1 ? b1p : nullptr, out_row_scales, out_tensor_scale, T, dmp, dffp, d_model, d_ff, flags, w, st);
    if (rc != I8TK_OK) return rc;
    return pad_copy(outp, T, dmp, out, T, d_model, 1, st);
}
