// INT8-KV decode attention (seq_q == 1) for B200: split-KV flash decoding.
//
// Replaces int8_decode_attention_forward of the reference
// (kernels/int8_decode_attention.cu:443-547: launcher, :274-386 partial
// kernel, :389-426 combine kernel).  Same arithmetic contract --
//   score_j = (q . k_j) * sQ * sK_j / sqrt(D)        (int8 x int8 -> int32 dot)
//   out     = sum_j softmax(score)_j * sV_j * v_j    (fp32 accumulate, fp16 out)
// -- different machine mapping:
//
// * The KV cache is cut into tiles of 32 positions; the tiles of all (b,h)
//   rows form one flat sequence that is divided EVENLY over a single wave of
//   persistent warps (one resident warp slot each), so every SM streams the
//   same number of bytes and no warp ever restarts its pipeline.  A warp's
//   range may cross (b,h) boundaries; it leaves one unnormalised
//   (m, l, acc[D]) row per (b,h) segment it touched.
// * Each warp owns a private ring of shared-memory stages.  K, V and the two
//   scale vectors of a tile are streamed HBM -> shared memory by 1-D bulk
//   async copies (the TMA engine) that complete on an mbarrier; several tiles
//   per warp are always in flight, so the bytes in flight per SM (~200 KB)
//   cover HBM3e latency x bandwidth.  No block-level barrier exists anywhere.
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
// * A small second kernel merges the rows of a (b,h) by log-sum-exp.  The
//   same row format is the exchange format of the multi-GPU sequence-sharded
//   path.
#include "common.cuh"

#include <cmath>
#include <cstdlib>

namespace i8tk {
namespace {

constexpr int kSub = 32;              // KV positions per warp pass (one per lane)
constexpr int kConsumers = 4;         // consumer warps per CTA; one more warp feeds the ring
constexpr int kTile = kSub * kConsumers;   // KV positions per stage: one sub-tile per consumer warp
constexpr int kThreads = (kConsumers + 1) * 32;
constexpr float kLog2e = 1.4426950408889634f;

template <int D>
struct DecodeTraits {
    static constexpr int LPR = D / 16;                 // lanes per row (16 B each)
    static constexpr int RPP = 32 / LPR;               // rows per warp pass
    static constexpr int STAGES = (D == 64) ? 4 : 3;   // ring depth per CTA
    static constexpr int TILE_BYTES = kTile * D;       // one of K or V: 8 KB / 16 KB contiguous
    static constexpr int SCALE_BYTES = kTile * 4;      // one of sK or sV
    static constexpr int STAGE_BYTES = 2 * TILE_BYTES + 2 * SCALE_BYTES;  // K | V | sK | sV
    static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
    static constexpr int SMEM_BYTES = RING_BYTES + 2 * STAGES * 8;
    static constexpr int CTAS_PER_SM = (D == 64) ? 3 : 2;
    static constexpr int ROW_FLOATS = D + 4;           // m, l, 0, 0, acc[D]
};

// Whole-row runs (short contexts): two sets of kConsumers row slots in shared memory behind the
// ring and its barriers, then the barrier the consumer warps meet on.
template <int D>
constexpr int kWholeSlotBytes = 2 * kConsumers * (D + 4) * 4;
template <int D>
constexpr int kWholeSmemBytes = DecodeTraits<D>::SMEM_BYTES + kWholeSlotBytes<D> + 16;
// cluster form: one merged row per segment parity behind those, then 2 + 2 barriers
template <int D>
constexpr int kClusterRowOff = DecodeTraits<D>::SMEM_BYTES + kWholeSlotBytes<D> + 16;
template <int D>
constexpr int kClusterBarOff = kClusterRowOff<D> + 2 * (D + 4) * 4;
template <int D>
constexpr int kClusterSmemBytes = kClusterBarOff<D> + 32;
constexpr int kWholeRowMaxTiles = 16;        // a row of at most this many tiles is never split across CTAs

// How the flat tile sequence is divided.  CTA c scans flat tiles
// [c*tpc, min(total, (c+1)*tpc)); flat tile f is tile f % tpb of (b,h) f / tpb.
struct DecodePlan {
    int tpb;             // tiles per (b,h) = ceil(S / kTile)
    int tpc;             // tiles per CTA
    int nctas;           // CTAs launched
    int maxseg;          // (b,h) segments a CTA can touch
    long long total;     // BH * tpb
};

// Paged KV cache (PAGED kernels): K, V and their scales live in pools of fixed-size pages,
// laid out [page][head][position in page][D] (scales [page][head][position in page]); request
// b owns pages page_table[b][0 .. ceil(seq_lens[b] / page)) in sequence order.
//
// Requests differ in length, and the lengths are known on the device only, so the division of
// the work is made there: decode_ragged_plan_kernel counts the tiles every request really has
// (ceil(seq_lens[b] / kTile) per head, none for an empty request), lays the tiles of all (b,h)
// rows end to end, cuts that sequence into equal runs, one per CTA, and leaves for CTA c the row
// and tile its run starts at.  A short request therefore costs what it reads, not what the
// longest one does.
struct PagedKV {
    const int* page_table;   // [B][max_pages]
    const int* seq_lens;     // [B] positions in use
    int H;                   // heads per request: b = bh / H, h = bh % H
    int page;                // positions per page: 16, 32, 64 or 128
    int max_pages;           // row length of page_table
    int B;                   // requests
    int max_len;             // host-side bound on seq_lens: longer entries are read as this
    int num_pages;           // pages in the pools, or 0 when the caller gave no bound: ids are then trusted
    const int* hdr;          // plan: [0] tiles per CTA, [1] tiles in all
    const int* prefix;       // plan: [B+1] tiles per head of the requests before b
    const int4* starts;      // plan: [nctas] {first (b,h) row, first tile in it, tiles of the run, 0}
};

__device__ __forceinline__ int tiles_of(int len) { return len > 0 ? (len + kTile - 1) / kTile : 0; }
// A page id as the producer uses it: with a bound given, an id outside [0, num_pages) is
// recorded in the status block and page 0 is read in its place.
__device__ __forceinline__ int checked_page(const PagedKV& pg, const int* id_ptr, uint32_t* status) {
    const int id = __ldg(id_ptr);
    if (pg.num_pages > 0 && (unsigned)id >= (unsigned)pg.num_pages) {
        note_bad_index(status);
        return 0;
    }
    return id;
}
// A request's length as the kernels use it: inside [0, max_len], so that a damaged entry can
// neither walk off its page-table row nor leave the workspace sized from max_len.
__device__ __forceinline__ int request_len(const int* seq_lens, int b, int max_len) {
    const int len = __ldg(seq_lens + b);
    return len < 0 ? 0 : (len > max_len ? max_len : len);
}

// First (b,h) row at or after `bh` that has tiles, and its tile count.  Called only while tiles
// of the CTA's run remain, so such a row exists; the bound keeps a damaged plan inside the arrays.
__device__ __forceinline__ int row_with_tiles(const PagedKV& pg, int bh, int& tpb) {
    const int BH = pg.B * pg.H;
    while (bh < BH) {
        tpb = tiles_of(request_len(pg.seq_lens, bh / pg.H, pg.max_len));
        if (tpb > 0) return bh;
        bh = (bh / pg.H + 1) * pg.H;
    }
    tpb = 1 << 30;
    return BH - 1;
}

// One CTA of 1024 threads: tiles per request, their exclusive prefix sum, how many of the
// launched CTAs take a run (about kTargetTiles tiles each, at least one resident wave, at most
// the grid), the run length, and the starting point of every CTA of the scan.
constexpr int kPlanSmemRequests = 4096;      // prefix sums of up to this many requests are searched in shared memory

__global__ void __launch_bounds__(1024)
decode_ragged_plan_kernel(const int* __restrict__ seq_lens, int B, int H, int max_len, int nctas, int resident,
                          int target_tiles, int* __restrict__ hdr, int* __restrict__ prefix, int4* __restrict__ starts,
                          uint32_t* __restrict__ status) {
    __shared__ int warp_tot[32];
    __shared__ int s_prefix[kPlanSmemRequests + 1];
    pdl_wait();
    pdl_launch_dependents();
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    if (t == 0) clear_call_status(status);
    const bool in_smem = B <= kPlanSmemRequests;
    const int per = (B + 1023) / 1024;
    const int lo = min(B, t * per), hi = min(B, lo + per);
    int sum = 0;
    for (int b = lo; b < hi; ++b) sum += tiles_of(request_len(seq_lens, b, max_len));
    int inc = sum;                                   // inclusive scan over the threads
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += v;
    }
    if (lane == 31) warp_tot[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        int w = warp_tot[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += v;
        }
        warp_tot[lane] = w;
    }
    __syncthreads();
    int base = inc - sum + (warp > 0 ? warp_tot[warp - 1] : 0);
    for (int b = lo; b < hi; ++b) {
        prefix[b] = base;
        if (in_smem) s_prefix[b] = base;
        base += tiles_of(request_len(seq_lens, b, max_len));
    }
    if (t == 1023) {
        prefix[B] = warp_tot[31];
        if (in_smem) s_prefix[B] = warp_tot[31];
    }
    __syncthreads();                                 // the prefix sums are read back below by other threads
    const int* pre = in_smem ? s_prefix : prefix;

    const long long total = (long long)warp_tot[31] * H;
    long long use = total / target_tiles;            // CTAs that take a run
    if (use < resident) use = resident;
    if (use > nctas) use = nctas;
    long long tpc = (total + use - 1) / use;
    if (tpc < 1) tpc = 1;
    if (t == 0) {
        hdr[0] = (int)tpc;
        hdr[1] = (int)total;
    }
    for (int c = t; c < nctas; c += 1024) {
        const long long f0 = (long long)c * tpc;
        int4 st = make_int4(0, 0, 0, 0);
        if (f0 < total) {
            int a = 0, z = B - 1;                    // largest b with prefix[b] * H <= f0
            while (a < z) {
                const int mid = (a + z + 1) >> 1;
                if ((long long)pre[mid] * H <= f0) a = mid; else z = mid - 1;
            }
            const int tb = pre[a + 1] - pre[a];                  // > 0: f0 lies inside request a
            const long long rem = f0 - (long long)pre[a] * H;
            const int h = (int)(rem / tb);
            st = make_int4(a * H + h, (int)(rem - (long long)h * tb), (int)min(tpc, total - f0), 0);
        }
        starts[c] = st;
    }
}

__device__ __forceinline__ int dot16(const int4& q, const int4& k) {
    int d = __dp4a(q.x, k.x, 0);
    d = __dp4a(q.y, k.y, d);
    d = __dp4a(q.z, k.z, d);
    d = __dp4a(q.w, k.w, d);
    return d;
}

// acc[0..1] (four floats) += w * int8x4(word).  The word is XORed with
// 0x80808080 so its bytes are u = v + 128 in [0, 255]; prmt drops byte j into
// the low mantissa of 0x4B000000 (= 2^23), and adding -(2^23 + 128) recovers v
// exactly in fp32.  The add and the FMA are issued as packed fp32x2 pairs.
__device__ __forceinline__ void fma_i8x4(f32x2* acc, uint32_t raw, f32x2 w2, f32x2 neg_magic2) {
    const uint32_t b = raw ^ 0x80808080u;
    f32x2 f01 = pack2(__uint_as_float(prmt(b, 0x4B000000u, 0x7650u)),
                      __uint_as_float(prmt(b, 0x4B000000u, 0x7651u)));
    f32x2 f23 = pack2(__uint_as_float(prmt(b, 0x4B000000u, 0x7652u)),
                      __uint_as_float(prmt(b, 0x4B000000u, 0x7653u)));
    f01 = add2(f01, neg_magic2);
    f23 = add2(f23, neg_magic2);
    acc[0] = fma2(w2, f01, acc[0]);
    acc[1] = fma2(w2, f23, acc[1]);
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
    float r;
    asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
    return r;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Wait on a ring barrier (bounded either way).  The parked form (try_wait with a time hint) wakes
// up about a microsecond late, which a CTA with a handful of tiles pays at every tile: measured
// 19 k cycles for an 8-tile run whose copies and arithmetic need 5 k.
constexpr int kEagerWaitTiles = 24;
__device__ __forceinline__ bool ring_wait(uint32_t bar, uint32_t parity, bool eager) {
    return eager ? mbar_wait_spin_bounded(bar, parity) : mbar_wait_bounded(bar, parity);
}

// Bounded wait on a barrier that CTAs of the cluster arrive on: acquire at cluster scope, so that what
// they wrote to their shared memory before arriving can be read through the cluster's window.
__device__ __forceinline__ bool mbar_wait_cluster_bounded(uint32_t bar, uint32_t parity, uint32_t limit = (1u << 22)) {
    for (uint32_t i = 0; i < limit; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
// The same location of rank `rank`'s shared memory, as an ordinary pointer.
__device__ __forceinline__ const float* cluster_generic(const float* mine, uint32_t rank) {
    unsigned long long out;
    asm volatile("mapa.u64 %0, %1, %2;" : "=l"(out) : "l"(reinterpret_cast<unsigned long long>(mine)), "r"(rank));
    return reinterpret_cast<const float*>(out);
}

// Log-sum-exp merge of `n` unnormalised rows {m, l, 0, 0, acc[D]} by one warp: lane holds D / 32
// consecutive output dims.  Rows with l <= 0 (no positions) are skipped.
template <int D, typename RowPtr>
__device__ __forceinline__ void merge_rows(RowPtr row_ptr, int n, int lane, float& L, float (&a)[D / 32],
                                           float* max_out = nullptr) {
    constexpr int DPL = D / 32;
    float gm = -INFINITY;
    for (int i = lane; i < n; i += 32) {
        const float2 ml = *reinterpret_cast<const float2*>(row_ptr(i));
        if (ml.y > 0.f) gm = fmaxf(gm, ml.x);
    }
    gm = warp_max(gm);
    L = 0.f;
#pragma unroll
    for (int k = 0; k < DPL; ++k) a[k] = 0.f;
#pragma unroll 4
    for (int i = 0; i < n; ++i) {
        const float* r = row_ptr(i);
        const float2 ml = *reinterpret_cast<const float2*>(r);
        if (ml.y <= 0.f) continue;                 // empty part
        const float wgt = ex2_approx(ml.x - gm);
        L = fmaf(ml.y, wgt, L);
        if constexpr (DPL == 4) {
            const float4 v = *reinterpret_cast<const float4*>(r + 4 + lane * 4);
            a[0] = fmaf(v.x, wgt, a[0]); a[1] = fmaf(v.y, wgt, a[1]);
            a[2] = fmaf(v.z, wgt, a[2]); a[3] = fmaf(v.w, wgt, a[3]);
        } else {
            const float2 v = *reinterpret_cast<const float2*>(r + 4 + lane * 2);
            a[0] = fmaf(v.x, wgt, a[0]); a[1] = fmaf(v.y, wgt, a[1]);
        }
    }
    if (max_out) *max_out = gm;
}
// The normalised fp16 output row (o points at its first element); a row without positions gives zeros.
template <int D>
__device__ __forceinline__ void store_out_row(__half* o, int lane, float L, const float (&a)[D / 32]) {
    constexpr int DPL = D / 32;
    const float inv = L > 0.f ? 1.0f / L : 0.f;
    o += lane * DPL;
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
}

// ---------------------------------------------------------------------------
// Pass 1: persistent CTAs over the flat tile sequence.  Warp kConsumers feeds
// the ring (one lane issues the bulk copies); warps 0..kConsumers-1 each scan
// one 32-position sub-tile of every stage and keep their own running
// (m, l, acc).  full[s]: copies of stage s landed; empty[s]: all consumers are
// done with stage s.
// SCALES_BULK: the per-position scales ride the bulk copies (needs S % 4 == 0
// and 16-byte aligned scale arrays); otherwise the owning lane loads them.
// ---------------------------------------------------------------------------
// PAGED: K, V, sK, sV are page pools addressed through `pg` and every request has its own
// length (S is then the longest one: tiles past a request's end carry no bytes).
// WHOLE: every CTA's run is made of whole (b,h) rows (short contexts: a row is a few tiles), so
// nothing has to be merged across CTAs: the four consumer warps fold their rows in shared memory
// and warp 0 writes the fp16 output row -- no second kernel.
// WHOLE 2: the same on a thread-block CLUSTER per row (few rows, e.g. one request): the ranks of
// the cluster split the row's tiles, each folds its warps' rows into one, tells rank 0 by an
// arrival on a barrier in rank 0's shared memory, and rank 0 reads the ranks' rows through
// distributed shared memory, merges and writes the output.  The ranks keep their shared memory
// alive until rank 0 says it has read it (a barrier of their own, arrived on remotely).
template <int D, bool SCALES_BULK, bool PAGED, int WHOLE = 0>
__global__ void __launch_bounds__(kThreads)
decode_partial_kernel(const int8_t* __restrict__ Q, const int8_t* __restrict__ K,
                      const int8_t* __restrict__ V, const float* __restrict__ sQ,
                      const float* __restrict__ sK, const float* __restrict__ sV,
                      float* __restrict__ rows,     // [nctas * maxseg * kConsumers, D+4]
                      int S, DecodePlan plan, float score_scale_log2,
                      uint32_t* __restrict__ status, PagedKV pg, __half* __restrict__ out) {
    static_assert(!PAGED || SCALES_BULK, "paged scales always ride the bulk copies");
    static_assert(WHOLE == 0 || !PAGED, "whole-row runs are planned on the host, for the contiguous cache");
    constexpr bool CLUSTER = WHOLE == 2;
    using T = DecodeTraits<D>;
    constexpr int LPR = T::LPR, RPP = T::RPP, STAGES = T::STAGES;

    extern __shared__ __align__(128) unsigned char smem[];
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    int ntl, bh0, tb0;                          // tiles of this CTA, row and tile it starts at
    const int tpb = plan.tpb;
    [[maybe_unused]] uint32_t crank = 0, csize = 1;
    [[maybe_unused]] int nrows = 0;
    int row_first = 0, row_end = 0;             // the tiles of a row this CTA takes (all of them unless CLUSTER)
    if constexpr (PAGED) {
        pdl_wait();                             // the run's start comes from the plan kernel just before this one
        const int4 st = pg.starts[blockIdx.x];
        bh0 = st.x;
        tb0 = st.y;
        ntl = st.z;
        if (ntl <= 0) return;
    } else if constexpr (CLUSTER) {
        // rank r of a cluster of n takes tiles [r * tpr, (r + 1) * tpr) of each of the cluster's rows
        // (plan.tpc is tpr, plan.maxseg the rows per cluster); a rank may have none
        crank = cluster_ctarank();
        csize = cluster_nctarank();
        const int BH = (int)(plan.total / tpb);
        bh0 = (int)(blockIdx.x / csize) * plan.maxseg;
        nrows = min(plan.maxseg, BH - bh0);
        row_first = min(tpb, (int)crank * plan.tpc);
        row_end = min(tpb, row_first + plan.tpc);
        tb0 = row_first;
        ntl = nrows * (row_end - row_first);
    } else {
        const long long f0 = (long long)blockIdx.x * plan.tpc;
        if (f0 >= plan.total) return;
        ntl = (int)min((long long)plan.tpc, plan.total - f0);
        bh0 = (int)(f0 / tpb);
        tb0 = (int)(f0 - (long long)bh0 * tpb);
    }
    if constexpr (!CLUSTER) row_end = tpb;

    // A CTA with a short run spends its time waiting for its few tiles to arrive: it polls the
    // barriers eagerly.  A long run is bound by bandwidth, its waits are rare and short, and the
    // parked form keeps the waiting warps off the issue slots (and the power budget).
    const bool eager = ntl <= kEagerWaitTiles;
    const uint32_t ring_s = smem_u32(smem);
    const uint32_t full0 = ring_s + T::RING_BYTES;
    const uint32_t empty0 = full0 + STAGES * 8;

    if (threadIdx.x == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, kConsumers);
        }
        if constexpr (WHOLE != 0) mbar_init(ring_s + T::SMEM_BYTES + kWholeSlotBytes<D>, kConsumers);
        if constexpr (CLUSTER) {
            for (int b = 0; b < 2; ++b) {
                mbar_init(ring_s + kClusterBarOff<D> + 8 * b, csize);        // rows of all ranks are there (rank 0's is used)
                mbar_init(ring_s + kClusterBarOff<D> + 16 + 8 * b, 1);       // rank 0 has read this rank's row
            }
        }
        fence_mbar_init();
    }
    __syncthreads();
    if constexpr (CLUSTER) cluster_sync_all();  // every rank's barriers exist before anyone arrives on them
    // Launched programmatically behind whatever precedes it in the stream: the wait keeps plain
    // stream order (no global memory is read or written before that work has completed), only the
    // launch itself and the set-up above may overlap its tail.
    pdl_wait();
    pdl_launch_dependents();                    // the next kernel may be scheduled as SMs drain
    if (blockIdx.x == 0 && threadIdx.x == 0) clear_call_status(status);

    if (warp == kConsumers) {
        // ---- producer: one lane walks the tile list and keeps the ring full ----
        // contiguous cache: one lane issues the four copies of a tile; paged cache: lane q issues
        // the copies of page q of the tile, so a tile of eight 16-position pages costs no more
        // issue time than one page
        if (!PAGED && lane != 0) return;
        const uint64_t stream_once = l2_policy_evict_first();   // K, V and their scales are read once
        int p_bh = bh0, p_tb = tb0;
        int p_tpb = row_end;                        // one past the last tile of row p_bh this CTA takes
        if constexpr (PAGED) p_tpb = tiles_of(request_len(pg.seq_lens, bh0 / pg.H, pg.max_len));
        for (int i = 0; i < ntl; ++i) {
            const int st = i % STAGES;
            if (i >= STAGES) {
                if (!ring_wait(empty0 + 8 * st, ((i / STAGES) - 1) & 1, eager)) {
                    if (lane == 0) note_timeout(status);
                    return;
                }
            }
            const int pos0 = p_tb * kTile;
            const uint32_t bar = full0 + 8 * st;
            const uint32_t dst = ring_s + st * T::STAGE_BYTES;
            if constexpr (PAGED) {
                // the tile is made of 128 / page pages; those past the request's end do not exist
                const int b = p_bh / pg.H, h = p_bh - b * pg.H;
                const int len = request_len(pg.seq_lens, b, pg.max_len);
                const int ppt = kTile / pg.page;
                int npg = (len - pos0 + pg.page - 1) / pg.page;
                npg = npg < 0 ? 0 : (npg > ppt ? ppt : npg);
                const uint32_t kv_bytes = (uint32_t)pg.page * D, sc_bytes = (uint32_t)pg.page * 4;
                const int* ids = pg.page_table + (size_t)b * pg.max_pages + pos0 / pg.page;
                if (pg.page > 32) {
                    // large pages: the scales ride bulk copies of their own (256-512 B each)
                    if (lane == 0) mbar_expect_tx(bar, (uint32_t)npg * 2 * (kv_bytes + sc_bytes));
                    if (lane < npg) {
                        const int q = lane;
                        const size_t first = ((size_t)checked_page(pg, ids + q, status) * pg.H + h) * pg.page;   // first position of the page
                        bulk_g2s_hint(dst + 2 * T::TILE_BYTES + q * sc_bytes, sK + first, sc_bytes, bar, stream_once);
                        bulk_g2s_hint(dst + 2 * T::TILE_BYTES + T::SCALE_BYTES + q * sc_bytes, sV + first, sc_bytes, bar,
                                      stream_once);
                        bulk_g2s_hint(dst + q * kv_bytes, K + first * D, kv_bytes, bar, stream_once);
                        bulk_g2s_hint(dst + T::TILE_BYTES + q * kv_bytes, V + first * D, kv_bytes, bar, stream_once);
                    }
                } else {
                    // small pages (16 or 32 positions): a tile is 4-8 pages and four bulk copies per
                    // page would be bound by copy issue, so only K and V travel as bulk copies; the
                    // 64-128 bytes of scales per page go as 16-byte asynchronous copies of the page's
                    // lane, which the stage's barrier is told to wait for before lane 0 arrives
                    if (lane < npg) {
                        const size_t first = ((size_t)checked_page(pg, ids + lane, status) * pg.H + h) * pg.page;
                        bulk_g2s_hint(dst + lane * kv_bytes, K + first * D, kv_bytes, bar, stream_once);
                        bulk_g2s_hint(dst + T::TILE_BYTES + lane * kv_bytes, V + first * D, kv_bytes, bar, stream_once);
                        const uint32_t dk = dst + 2 * T::TILE_BYTES + lane * sc_bytes;
                        for (uint32_t o = 0; o < sc_bytes; o += 16) {
                            cp_async16(dk + o, reinterpret_cast<const unsigned char*>(sK + first) + o);
                            cp_async16(dk + T::SCALE_BYTES + o, reinterpret_cast<const unsigned char*>(sV + first) + o);
                        }
                        cp_async_mbar_arrive(bar);
                    }
                    __syncwarp();
                    if (lane == 0) mbar_expect_tx(bar, (uint32_t)npg * 2 * kv_bytes);
                }
            } else {
            const int nrow = min(kTile, S - pos0);
            const size_t row = (size_t)p_bh * S + pos0;
            const uint32_t kv_bytes = (uint32_t)nrow * D;
            if constexpr (SCALES_BULK) {
                const uint32_t sc_bytes = (uint32_t)nrow * 4;       // multiple of 16: S % 4 == 0
                mbar_expect_tx(bar, 2 * kv_bytes + 2 * sc_bytes);
                bulk_g2s_hint(dst + 2 * T::TILE_BYTES, sK + row, sc_bytes, bar, stream_once);
                bulk_g2s_hint(dst + 2 * T::TILE_BYTES + T::SCALE_BYTES, sV + row, sc_bytes, bar, stream_once);
            } else {
                mbar_expect_tx(bar, 2 * kv_bytes);
            }
            bulk_g2s_hint(dst, K + row * D, kv_bytes, bar, stream_once);
            bulk_g2s_hint(dst + T::TILE_BYTES, V + row * D, kv_bytes, bar, stream_once);
            }
            if (++p_tb == p_tpb) {
                p_tb = row_first;
                ++p_bh;
                if constexpr (PAGED) {
                    if (i + 1 < ntl) p_bh = row_with_tiles(pg, p_bh, p_tpb);
                }
            }
        }
        return;
    }

    // ---- consumers ------------------------------------------------------------
    const int c = lane % LPR;                       // 16-byte chunk of a row
    const int g = lane / LPR;                       // row within a pass
    const int own = warp * kSub + g + RPP * c;      // position in the tile whose softmax this lane runs
    const f32x2 neg_magic2 = pack2(-8388736.0f, -8388736.0f);   // -(2^23 + 128)

    int c_bh = bh0, c_tb = tb0;
    int c_tpb = row_end;                            // one past the last tile of row c_bh this CTA takes
    if constexpr (PAGED) c_tpb = tiles_of(request_len(pg.seq_lens, bh0 / pg.H, pg.max_len));
    int i = 0;                                      // tiles of this CTA consumed so far
    // (a rank of a cluster goes through all the cluster's rows even when it has no tiles of them)
    for (int seg = 0; CLUSTER ? seg < nrows : i < ntl; ++seg) {
        // ---- one (b,h) segment: tiles [c_tb, c_tb + seg_tiles) of row c_bh ----
        const int seg_tiles = min(ntl - i, c_tpb - c_tb);
        const int4 q4 = *reinterpret_cast<const int4*>(Q + (size_t)c_bh * D + c * 16);
        const float qs = sQ[c_bh] * score_scale_log2;
        const float* sKb = sK + (size_t)c_bh * S;
        const float* sVb = sV + (size_t)c_bh * S;
        const int Sb = PAGED ? request_len(pg.seq_lens, c_bh / pg.H, pg.max_len) : S;    // positions of this (b,h) row
        float m = -INFINITY, l = 0.f;
        f32x2 acc[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] = pack2(0.f, 0.f);

        float sk_next = 0.f, sv_next = 0.f;         // scales when they do not ride the bulk copies
        if constexpr (!SCALES_BULK) {
            const int pos = c_tb * kTile + own;
            if (pos < S) { sk_next = sKb[pos]; sv_next = sVb[pos]; }
        }

        for (int t = 0; t < seg_tiles; ++t, ++i) {
            const int pos0 = (c_tb + t) * kTile;
            const bool valid = (pos0 + own) < Sb;

            float sk0 = 0.f, sv0 = 0.f;
            if constexpr (!SCALES_BULK) {
                sk0 = sk_next;
                sv0 = sv_next;
                const int pos = pos0 + kTile + own;     // next tile of this segment, if any
                sk_next = 0.f;
                sv_next = 0.f;
                if (t + 1 < seg_tiles && pos < S) { sk_next = sKb[pos]; sv_next = sVb[pos]; }
            }

            const int st = i % STAGES;
            const bool got = ring_wait(full0 + 8 * st, (i / STAGES) & 1, eager);
            if (!__all_sync(0xffffffffu, got)) {
                if (lane == 0) note_timeout(status);
                return;
            }

            if (pos0 + warp * kSub < Sb) {          // this warp's sub-tile has rows (warp-uniform)
                const unsigned char* stage = smem + st * T::STAGE_BYTES;
                const int4* Kt = reinterpret_cast<const int4*>(stage + warp * kSub * D);
                const int4* Vt = reinterpret_cast<const int4*>(stage + T::TILE_BYTES + warp * kSub * D);
                if constexpr (SCALES_BULK) {
                    const float* sc = reinterpret_cast<const float*>(stage + 2 * T::TILE_BYTES);
                    sk0 = valid ? sc[own] : 0.f;
                    sv0 = valid ? sc[kTile + own] : 0.f;
                }

                // ---- QK^T partial dots, then one full dot per lane ------------
                int d[LPR];
#pragma unroll
                for (int k = 0; k < LPR; ++k) {
                    const int4 kw = Kt[(g + RPP * k) * LPR + c];
                    d[k] = dot16(q4, kw);
                }
                const int tot = reduce_scatter<LPR>(d, c);

                // ---- online softmax, log2 units, one position per lane ---------
                const float s = valid ? (float)tot * (qs * sk0) : -INFINITY;
                const float m_new = fmaxf(m, warp_max(s));
                if (m_new > m) {                    // warp-uniform, rare after the first tiles
                    const float corr = ex2_approx(m - m_new);
                    const f32x2 corr2 = pack2(corr, corr);
                    l *= corr;
#pragma unroll
                    for (int k = 0; k < 8; ++k) acc[k] = mul2(acc[k], corr2);
                    m = m_new;
                }
                const float p = ex2_approx(s - m);
                l += p;
                const float wgt = p * sv0;

                // ---- PV: acc[16 dims of chunk c] += w_row * v_row ---------------
#pragma unroll
                for (int k = 0; k < LPR; ++k) {
                    const float wk = __shfl_sync(0xffffffffu, wgt, (lane & ~(LPR - 1)) | k);
                    const f32x2 w2 = pack2(wk, wk);
                    const int4 vw = Vt[(g + RPP * k) * LPR + c];
                    fma_i8x4(acc + 0, (uint32_t)vw.x, w2, neg_magic2);
                    fma_i8x4(acc + 2, (uint32_t)vw.y, w2, neg_magic2);
                    fma_i8x4(acc + 4, (uint32_t)vw.z, w2, neg_magic2);
                    fma_i8x4(acc + 6, (uint32_t)vw.w, w2, neg_magic2);
                }
            }

            // every lane of this warp is done reading the stage
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + 8 * st);
        }

        // ---- end of the segment: fold the row groups and emit the row ----------
        float a[16];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float2 v = unpack2(acc[k]);
            a[2 * k] = v.x;
            a[2 * k + 1] = v.y;
        }
#pragma unroll
        for (int o = LPR; o < 32; o <<= 1) {
#pragma unroll
            for (int k = 0; k < 16; ++k) a[k] += __shfl_xor_sync(0xffffffffu, a[k], o);
        }
        const float lsum = warp_sum(l);
        // paged: slot (row + CTA) is unique because the CTAs' runs are ordered by row
        float* row = PAGED ? rows + ((size_t)(c_bh + blockIdx.x) * kConsumers + warp) * T::ROW_FLOATS
                           : rows + (((size_t)blockIdx.x * plan.maxseg + seg) * kConsumers + warp) * T::ROW_FLOATS;
        if constexpr (WHOLE != 0) {
            // this warp's row goes to shared memory instead (two sets of slots, by segment parity:
            // warp 0 reaches the next segment's barrier only after it has merged this one)
            row = reinterpret_cast<float*>(smem + T::SMEM_BYTES) + ((seg & 1) * kConsumers + warp) * T::ROW_FLOATS;
        }
        if (lane == 0) *reinterpret_cast<float4*>(row) = make_float4(m, lsum, 0.f, 0.f);
        if (g == 0) {
            float4* dst = reinterpret_cast<float4*>(row + 4 + c * 16);
#pragma unroll
            for (int k = 0; k < 4; ++k)
                dst[k] = make_float4(a[4 * k], a[4 * k + 1], a[4 * k + 2], a[4 * k + 3]);
        }
        if constexpr (WHOLE != 0) {
            // the consumer warps meet on a barrier of their own, one phase per segment; the wait is
            // bounded like every other, so a warp that gave up earlier cannot hold the rest
            const uint32_t fin_bar = ring_s + T::SMEM_BYTES + kWholeSlotBytes<D>;
            __syncwarp();
            if (lane == 0) mbar_arrive(fin_bar);
            const bool met = ring_wait(fin_bar, seg & 1, true);
            if (!__all_sync(0xffffffffu, met)) {
                if (lane == 0) note_timeout(status);
                return;
            }
            if (warp == 0) {
                const float* slots = reinterpret_cast<const float*>(smem + T::SMEM_BYTES) + (seg & 1) * kConsumers * T::ROW_FLOATS;
                float L;
                float o[D / 32];
                if constexpr (!CLUSTER) {
                    merge_rows<D>([&](int r) { return slots + r * T::ROW_FLOATS; }, kConsumers, lane, L, o);
                    store_out_row<D>(out + (size_t)c_bh * D, lane, L, o);
                } else {
                    constexpr int DPL = D / 32;
                    const uint32_t ph = (uint32_t)(seg >> 1) & 1u;
                    const uint32_t all_bar = ring_s + kClusterBarOff<D> + 8 * (seg & 1);
                    const uint32_t read_bar = ring_s + kClusterBarOff<D> + 16 + 8 * (seg & 1);
                    // this rank's slot of segment seg - 2 is about to be overwritten: rank 0 must have read it
                    bool fine = true;
                    if (seg >= 2) fine = mbar_wait_cluster_bounded(read_bar, ph ^ 1u);
                    float gm;
                    merge_rows<D>([&](int r) { return slots + r * T::ROW_FLOATS; }, kConsumers, lane, L, o, &gm);
                    float* mine = reinterpret_cast<float*>(smem + kClusterRowOff<D>) + (seg & 1) * T::ROW_FLOATS;
                    if (lane == 0) *reinterpret_cast<float4*>(mine) = make_float4(L > 0.f ? gm : -INFINITY, L, 0.f, 0.f);
#pragma unroll
                    for (int k = 0; k < DPL; ++k) mine[4 + lane * DPL + k] = o[k];
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(mapa_shared(all_bar, 0));       // release at cluster scope
                    if (crank == 0) {
                        fine = fine && mbar_wait_cluster_bounded(all_bar, ph);
                        if (__all_sync(0xffffffffu, fine)) {
                            float L2;
                            float o2[DPL];
                            merge_rows<D>([&](int r) { return cluster_generic(mine, (uint32_t)r); }, (int)csize, lane, L2, o2);
                            store_out_row<D>(out + (size_t)c_bh * D, lane, L2, o2);
                            __syncwarp();
                            if (lane < (int)csize) mbar_arrive_cluster(mapa_shared(read_bar, (uint32_t)lane));
                        }
                    }
                    if (!__all_sync(0xffffffffu, fine)) {
                        if (lane == 0) note_timeout(status);
                        return;
                    }
                }
            }
        }
        if constexpr (CLUSTER) {
            ++c_bh;                                 // same tile range of the next row
            continue;
        }
        c_tb += seg_tiles;
        if (c_tb == c_tpb) {
            c_tb = 0;
            ++c_bh;
            if constexpr (PAGED) {
                if (i < ntl) c_bh = row_with_tiles(pg, c_bh, c_tpb);
            }
        }
    }
    if constexpr (CLUSTER) {
        // a rank's shared memory must outlive rank 0's reads of its last two rows
        if (warp == 0) {
            bool fine = true;
            for (int seg = max(0, nrows - 2); seg < nrows; ++seg)
                fine = fine && mbar_wait_cluster_bounded(ring_s + kClusterBarOff<D> + 16 + 8 * (seg & 1), (uint32_t)(seg >> 1) & 1u);
            if (!__all_sync(0xffffffffu, fine) && lane == 0) note_timeout(status);
        }
    }
}

// ---------------------------------------------------------------------------
// Pass 2: log-sum-exp merge of the rows of one (b,h).  One warp per (b,h).
// FLAT: rows were written by the consumer warps of pass 1 (indexed through
// the plan).  Otherwise: row (s, bh) of a gathered [nparts, BH, D+4] array.
// Writes either the normalised fp16 output or one merged row.
// ---------------------------------------------------------------------------
// RAGGED (with FLAT): the rows were written under the device-side plan of a paged cache; a
// request without positions gets a zero output row.
// QUANT: one CTA per request with one warp per head (blockDim = 32 * heads); besides (or
// instead of) the fp16 row, the token's heads*D outputs leave as int8 codes with ONE scale per
// token -- the input format of the INT8 GEMM that follows attention (the output projection):
// scale = max(|fp16 out|, 1e-8) / 127 over the whole token, code = rne(fp16 out / scale), the
// per-token quantiser's arithmetic (tests/test_int8.py:47-63) on the fp16 values.
struct QuantOut {
    int8_t* codes;           // [B][heads * D]
    float* scales;           // [B]
};

template <int D, bool FLAT, bool RAGGED = false, bool QUANT = false>
__global__ void __launch_bounds__(QUANT ? 1024 : 128)
decode_combine_kernel(const float* __restrict__ rows, int BH, int nparts, DecodePlan plan,
                      __half* __restrict__ out, float* __restrict__ row_out, PagedKV pg, QuantOut qo) {
    constexpr int ROW = D + 4;
    constexpr int DPL = D / 32;
    [[maybe_unused]] __shared__ float head_max[32];
    pdl_wait();                                 // rows of the scan launched just before this kernel
    const int wpc = QUANT ? (int)(blockDim.x >> 5) : 4;      // (b,h) rows per CTA
    const int bh = blockIdx.x * wpc + (threadIdx.x >> 5);
    if (!QUANT && bh >= BH) return;
    const int lane = threadIdx.x & 31;

    int c_first = 0, n = nparts;
    if constexpr (RAGGED) {
        const int b = bh / pg.H, h = bh - b * pg.H;
        const int p0 = pg.prefix[b], tb = pg.prefix[b + 1] - p0, tpc = pg.hdr[0];
        const long long fb = (long long)p0 * pg.H + (long long)h * tb;    // first flat tile of the row
        c_first = (int)(fb / tpc);
        n = tb > 0 ? ((int)((fb + tb - 1) / tpc) - c_first + 1) * kConsumers : 0;
    } else if constexpr (FLAT) {
        const long long fb = (long long)bh * plan.tpb;
        c_first = (int)(fb / plan.tpc);
        n = ((int)((fb + plan.tpb - 1) / plan.tpc) - c_first + 1) * kConsumers;
    }
    auto row_ptr = [&](int i) -> const float* {
        if constexpr (RAGGED) {
            const int cta = c_first + i / kConsumers;
            return rows + ((size_t)(bh + cta) * kConsumers + i % kConsumers) * ROW;
        } else if constexpr (FLAT) {
            const int cta = c_first + i / kConsumers;
            const int seg = bh - (int)(((long long)cta * plan.tpc) / plan.tpb);
            return rows + (((size_t)cta * plan.maxseg + seg) * kConsumers + i % kConsumers) * ROW;
        } else {
            return rows + ((size_t)i * BH + bh) * ROW;
        }
    };

    float L, gm;
    float a[DPL];
    merge_rows<D>(row_ptr, n, lane, L, a, &gm);

    if constexpr (QUANT) {
        const float inv = L > 0.f ? 1.0f / L : 0.f;
        float v[DPL];
        float amax = 0.f;
#pragma unroll
        for (int k = 0; k < DPL; ++k) {
            v[k] = __half2float(__float2half_rn(a[k] * inv));        // the fp16 output, widened again
            amax = fmaxf(amax, fabsf(v[k]));
        }
        amax = warp_max(amax);
        if (lane == 0) head_max[threadIdx.x >> 5] = amax;
        __syncthreads();
        float tmax = lane < wpc ? head_max[lane] : 0.f;
        tmax = fmaxf(warp_max(tmax), 1e-8f);
        const float scale = __fdiv_rn(tmax, 127.f);
        uint32_t packed = 0;
#pragma unroll
        for (int k = 0; k < DPL; ++k) {
            const int c = __float2int_rn(fmaxf(-128.f, fminf(127.f, __fdiv_rn(v[k], scale))));
            packed |= (uint32_t)(c & 0xff) << (8 * k);
        }
        int8_t* q = qo.codes + (size_t)bh * D + lane * DPL;
        if constexpr (DPL == 4) *reinterpret_cast<uint32_t*>(q) = packed;
        else *reinterpret_cast<uint16_t*>(q) = (uint16_t)packed;
        if (threadIdx.x == 0) qo.scales[blockIdx.x] = scale;
        if (out != nullptr) {
            __half* o = out + (size_t)bh * D + lane * DPL;
#pragma unroll
            for (int k = 0; k < DPL; ++k) o[k] = __float2half_rn(v[k]);
        }
        return;
    }
    if (out != nullptr) {
        store_out_row<D>(out + (size_t)bh * D, lane, L, a);
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
// Pass 2 for the KV-sequence-sharded path, fused with the exchange between
// GPUs.  Every rank runs this kernel at the same time (one process per GPU).
// CTA c of every rank handles the same four (b,h) rows:
//   1. merge this rank's own partial rows of a (b,h) into one (m, l, acc) row,
//   2. store that row into slot [rank] of EVERY rank's gather buffer -- plain
//      stores through peer-mapped pointers, NVLink/NVSwitch carries them --
//   3. fence, then set flag [rank][c] = epoch on every rank,
//   4. wait (bounded) until flags [r][c] of all ranks r show this epoch in the
//      local flag array, then merge the world-size rows and write fp16.
// No collective library call, no host round trip; the only data crossing the
// links are the rows themselves (B*H*(D+4) floats per rank pair).
// `peer_parts[r]` / `peer_flags[r]` are rank r's buffers as mapped into this
// process ([2][world][BH][D+4] floats and [world][gridDim.x] words, flags zeroed
// once at set-up); `epoch` starts at 1 and increases by one per call on all ranks.
// ---------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(128)
decode_exchange_kernel(const float* __restrict__ rows, int BH, DecodePlan plan, int empty,
                       float* const* __restrict__ peer_parts, uint32_t* const* __restrict__ peer_flags,
                       int rank, int world, uint32_t epoch, uint32_t spin_limit, __half* __restrict__ out,
                       uint32_t* __restrict__ status) {
    constexpr int ROW = D + 4;
    constexpr int DPL = D / 32;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int bh = blockIdx.x * 4 + warp;
    const bool active = bh < BH;
    pdl_wait();                                 // rows of the scan launched just before this kernel
    if (empty && blockIdx.x == 0 && threadIdx.x == 0) clear_call_status(status);   // no scan ran to do it

    // ---- 1. local merge ------------------------------------------------------
    float gm = -INFINITY, L = 0.f;
    float a[DPL];
#pragma unroll
    for (int k = 0; k < DPL; ++k) a[k] = 0.f;
    if (active && !empty) {
        const long long fb = (long long)bh * plan.tpb;
        const int c_first = (int)(fb / plan.tpc);
        const int n = ((int)((fb + plan.tpb - 1) / plan.tpc) - c_first + 1) * kConsumers;
        auto row_ptr = [&](int i) -> const float* {
            const int cta = c_first + i / kConsumers;
            const int seg = bh - (int)(((long long)cta * plan.tpc) / plan.tpb);
            return rows + (((size_t)cta * plan.maxseg + seg) * kConsumers + i % kConsumers) * ROW;
        };
        for (int i = lane; i < n; i += 32) {
            const float2 ml = *reinterpret_cast<const float2*>(row_ptr(i));
            if (ml.y > 0.f) gm = fmaxf(gm, ml.x);
        }
        gm = warp_max(gm);
        for (int i = 0; i < n; ++i) {
            const float* r = row_ptr(i);
            const float2 ml = *reinterpret_cast<const float2*>(r);
            if (ml.y <= 0.f) continue;
            const float wgt = ex2_approx(ml.x - gm);
            L = fmaf(ml.y, wgt, L);
#pragma unroll
            for (int k = 0; k < DPL; ++k) a[k] = fmaf(r[4 + lane * DPL + k], wgt, a[k]);
        }
        if (!(L > 0.f)) gm = -INFINITY;
    }

    // ---- 2. push the row to every rank (own slot included) ---------------------
    if (active) {
        for (int p = 0; p < world; ++p) {
            float* dst = peer_parts[p] + (((size_t)(epoch & 1u) * world + rank) * BH + bh) * ROW;
            if (lane == 0) *reinterpret_cast<float4*>(dst) = make_float4(gm, L, 0.f, 0.f);
            if constexpr (DPL == 4)
                *reinterpret_cast<float4*>(dst + 4 + lane * 4) = make_float4(a[0], a[1], a[2], a[3]);
            else
                *reinterpret_cast<float2*>(dst + 4 + lane * 2) = make_float2(a[0], a[1]);
        }
    }
    // ---- 3. publish -------------------------------------------------------------
    __threadfence_system();
    __syncthreads();
    const int slot = blockIdx.x;
    if (threadIdx.x < world) {
        uint32_t* f = peer_flags[threadIdx.x] + (size_t)rank * gridDim.x + slot;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(epoch) : "memory");
    }
    // ---- 4. wait for every rank's rows of this CTA, then merge -------------------
    if (threadIdx.x < world) {
        const uint32_t* f = peer_flags[rank] + (size_t)threadIdx.x * gridDim.x + slot;
        bool seen = false;
        for (uint32_t spin = 0; spin < spin_limit; ++spin) {
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
            if ((int32_t)(v - epoch) >= 0) { seen = true; break; }
        }
        if (!seen) note_timeout(status);
    }
    __syncthreads();
    if (!active) return;

    // two gather buffers, alternated by epoch parity: a fast rank may already be pushing the
    // next call's rows while a slow one is still reading this call's
    const float* mine = peer_parts[rank] + (size_t)(epoch & 1u) * world * BH * ROW;
    float gm2 = -INFINITY;
    for (int r = lane; r < world; r += 32) {
        const float* rp = mine + ((size_t)r * BH + bh) * ROW;
        const float m_r = __ldcg(rp), l_r = __ldcg(rp + 1);
        if (l_r > 0.f) gm2 = fmaxf(gm2, m_r);
    }
    gm2 = warp_max(gm2);
    float L2 = 0.f;
    float b[DPL];
#pragma unroll
    for (int k = 0; k < DPL; ++k) b[k] = 0.f;
    for (int r = 0; r < world; ++r) {
        const float* rp = mine + ((size_t)r * BH + bh) * ROW;
        const float m_r = __ldcg(rp), l_r = __ldcg(rp + 1);
        if (l_r <= 0.f) continue;
        const float wgt = ex2_approx(m_r - gm2);
        L2 = fmaf(l_r, wgt, L2);
#pragma unroll
        for (int k = 0; k < DPL; ++k) b[k] = fmaf(__ldcg(rp + 4 + lane * DPL + k), wgt, b[k]);
    }
    const float inv = 1.0f / L2;
    __half* o = out + (size_t)bh * D + lane * DPL;
    if constexpr (DPL == 4) {
        __half2 h0 = __floats2half2_rn(b[0] * inv, b[1] * inv);
        __half2 h1 = __floats2half2_rn(b[2] * inv, b[3] * inv);
        uint2 pk;
        pk.x = *reinterpret_cast<uint32_t*>(&h0);
        pk.y = *reinterpret_cast<uint32_t*>(&h1);
        *reinterpret_cast<uint2*>(o) = pk;
    } else {
        *reinterpret_cast<__half2*>(o) = __floats2half2_rn(b[0] * inv, b[1] * inv);
    }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
// Optional timing probe: events recorded on the launch stream immediately
// before and after the streaming (pass 1) kernel of the next calls made by
// this thread.
thread_local cudaEvent_t g_probe_start = nullptr;
thread_local cudaEvent_t g_probe_stop = nullptr;

// Polls the exchange kernel spends on another rank's flag before it gives up (each is a load
// that travels to memory another GPU writes: about a microsecond, so the default is seconds).
constexpr unsigned int kExchangeSpinDefault = 1u << 21;
unsigned int g_exchange_spin_limit = kExchangeSpinDefault;

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

int env_int(const char* name, int dflt) {
    const char* e = getenv(name);
    return e ? atoi(e) : dflt;
}
// Tuning overrides, read from the environment once per process.
int forced_ctas() { static const int v = env_int("I8TK_DECODE_CTAS", 0); return v; }
int scales_by_ldg() { static const int v = env_int("I8TK_DECODE_SCALES_LDG", 0); return v; }
int whole_row_tiles(int dflt) { static const int v = env_int("I8TK_DECODE_WHOLE_TILES", -1); return v >= 0 ? v : dflt; }
int paged_target_tiles(int dflt) { static const int v = env_int("I8TK_DECODE_TARGET_TILES", 0); return v > 0 ? v : dflt; }

// CTAs are persistent over contiguous runs of the flat tile sequence.  The
// count is between one and four resident waves: about 64 tiles per CTA keeps
// the cost of filling a ring negligible while leaving the hardware scheduler
// room to even out SM-to-SM speed differences; tiny problems get at least
// kMinTiles tiles per CTA.  I8TK_DECODE_CTAS overrides the count (tuning only).
constexpr int kTargetTiles = 64;
// Paged cache: longer runs measured faster (fewer ring fills against page-sized copies);
// I8TK_DECODE_TARGET_TILES overrides it (tuning only).
constexpr int kPagedTargetTiles = 128;

DecodePlan make_plan(int BH, int S, int D, int sms) {
    constexpr int kMinTiles = 2;
    const int ctas_per_sm = (D == 64) ? DecodeTraits<64>::CTAS_PER_SM : DecodeTraits<128>::CTAS_PER_SM;
    DecodePlan p;
    p.tpb = (S + kTile - 1) / kTile;
    p.total = (long long)BH * p.tpb;
    const long long slots = (long long)sms * ctas_per_sm;
    long long want = p.total / kTargetTiles;
    if (want < slots) want = slots;
    if (want > 4 * slots) want = 4 * slots;
    const long long cap = (p.total + kMinTiles - 1) / kMinTiles;
    if (want > cap) want = cap;
    const int forced = forced_ctas();
    if (forced > 0) want = forced;
    if (want > p.total) want = p.total;
    if (want < 1) want = 1;
    p.tpc = (int)((p.total + want - 1) / want);
    p.nctas = (int)((p.total + p.tpc - 1) / p.tpc);
    p.maxseg = (p.tpc + p.tpb - 1) / p.tpb + 1;
    return p;
}

// Runs of whole rows for contexts of at most kWholeRowMaxTiles tiles: as many CTAs as rows, up
// to one resident wave; beyond that a CTA takes several rows, one after the other.
DecodePlan make_whole_plan(int BH, int S, int D, int sms) {
    const int ctas_per_sm = (D == 64) ? DecodeTraits<64>::CTAS_PER_SM : DecodeTraits<128>::CTAS_PER_SM;
    DecodePlan p;
    p.tpb = (S + kTile - 1) / kTile;
    p.total = (long long)BH * p.tpb;
    const long long cap = (long long)sms * ctas_per_sm;
    const int rows_per_cta = (int)((BH + cap - 1) / cap);
    p.tpc = rows_per_cta * p.tpb;
    p.nctas = (BH + rows_per_cta - 1) / rows_per_cta;
    p.maxseg = rows_per_cta;
    return p;
}

// One cluster of `cluster` CTAs per row: rank r takes tiles [r * tpc, (r + 1) * tpc) of it.
DecodePlan make_cluster_plan(int BH, int S, int cluster) {
    DecodePlan p;
    p.tpb = (S + kTile - 1) / kTile;
    p.total = (long long)BH * p.tpb;
    p.tpc = (p.tpb + cluster - 1) / cluster;     // tiles per rank
    p.nctas = BH * cluster;
    p.maxseg = 1;                                // rows per cluster
    return p;
}

size_t rows_bytes(const DecodePlan& p, int D) {
    return (size_t)p.nctas * p.maxseg * kConsumers * (D + 4) * sizeof(float);
}

// Workspace of the paged entry point behind the 256-byte status block: one row slot per
// (row + CTA) pair, the plan header, the CTAs' starting points and the tile prefix sums.
struct RaggedLayout {
    size_t rows_off, hdr_off, starts_off, prefix_off, total;
};

RaggedLayout ragged_layout(int BH, int B, int nctas, int D) {
    auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
    RaggedLayout l;
    l.rows_off = 256;
    l.hdr_off = l.rows_off + up((size_t)(BH + nctas) * kConsumers * (D + 4) * sizeof(float));
    l.starts_off = l.hdr_off + 256;
    l.prefix_off = l.starts_off + up((size_t)nctas * sizeof(int4));
    l.total = l.prefix_off + up((size_t)(B + 1) * sizeof(int));
    return l;
}

// Large enough for the contiguous and for the paged entry points (a batch has at most BH requests).
size_t workspace_bytes(int BH, int S, int D) {
    const DecodePlan p = make_plan(BH, S, D, sm_count());
    const size_t flat = 256 + rows_bytes(p, D);
    const size_t ragged = ragged_layout(BH, BH, p.nctas, D).total;
    return flat > ragged ? flat : ragged;
}

// `whole_out`: the plan is one of whole rows (make_whole_plan) and the scan writes the fp16 output itself.
// WHOLE 2: `cluster` CTAs per row (make_cluster_plan).
template <int D, bool SCALES_BULK, bool PAGED = false, int WHOLE = 0>
int launch_partial(const int8_t* Q, const int8_t* K, const int8_t* V, const float* sQ,
                   const float* sK, const float* sV, float* rows, int S, const DecodePlan& p,
                   uint32_t* status, cudaStream_t stream, PagedKV pg = PagedKV{}, __half* whole_out = nullptr,
                   int cluster = 1) {
    using T = DecodeTraits<D>;
    constexpr int kSmem = WHOLE == 2 ? kClusterSmemBytes<D> : (WHOLE == 1 ? kWholeSmemBytes<D> : T::SMEM_BYTES);
    static bool attr_done[64] = {false};   // per template instance
    int dev = 0;
    I8TK_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        I8TK_CUDA(cudaFuncSetAttribute(decode_partial_kernel<D, SCALES_BULK, PAGED, WHOLE>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
        attr_done[dev] = true;
    }
    const float score_scale_log2 = kLog2e / sqrtf((float)D);
    if (g_probe_start) I8TK_CUDA(cudaEventRecord(g_probe_start, stream));
    I8TK_CUDA(launch_after_clustered(decode_partial_kernel<D, SCALES_BULK, PAGED, WHOLE>, dim3(p.nctas), dim3(kThreads),
                                     kSmem, stream, cluster, Q, K, V, sQ, sK, sV, rows, S, p, score_scale_log2, status, pg,
                                     whole_out));
    if (g_probe_stop) I8TK_CUDA(cudaEventRecord(g_probe_stop, stream));
    return I8TK_OK;
}

// Whether the device can co-schedule clusters of `cluster` CTAs of the cluster form of the scan at
// all (a partitioned or otherwise restricted device may not): asked once per size, otherwise the
// other plans are used.
template <int D>
bool clusters_fit(int cluster, bool bulk) {
    static int known[64][9] = {};            // 0 unknown, 1 yes, -1 no
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || cluster < 2 || cluster > 8) return false;
    int& k = known[dev][cluster];
    if (k == 0) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)cluster);
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = kClusterSmemBytes<D>;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = (unsigned)cluster;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int n = 0;
        cudaError_t e = cudaFuncSetAttribute(decode_partial_kernel<D, true, false, 2>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, kClusterSmemBytes<D>);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(decode_partial_kernel<D, false, false, 2>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, kClusterSmemBytes<D>);
        if (e == cudaSuccess) e = cudaOccupancyMaxActiveClusters(&n, decode_partial_kernel<D, true, false, 2>, &cfg);
        if (e != cudaSuccess) (void)cudaGetLastError();
        k = (e == cudaSuccess && n > 0) ? 1 : -1;
    }
    (void)bulk;
    return k > 0;
}

template <int D>
int launch_decode(const int8_t* Q, const int8_t* K, const int8_t* V, __half* out, float* part,
                  const float* sQ, const float* sK, const float* sV, int BH, int S,
                  void* workspace, size_t wbytes, cudaStream_t stream, QuantOut qo = QuantOut{}, int heads = 0) {
    using T = DecodeTraits<D>;
    const DecodePlan p = make_plan(BH, S, D, sm_count());
    const size_t need = 256 + rows_bytes(p, D);
    I8TK_REQUIRE(workspace != nullptr && wbytes >= need, I8TK_ERR_WORKSPACE,
                 "decode workspace too small: need %zu bytes, got %zu", need, wbytes);
    I8TK_REQUIRE(aligned_to(workspace, 256), I8TK_ERR_ALIGNMENT, "workspace must be 256-byte aligned");

    uint32_t* status = reinterpret_cast<uint32_t*>(workspace);
    float* rows = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(workspace) + 256);
    const bool bulk_scales = (S % 4 == 0) && aligned_to(sK, 16) && aligned_to(sV, 16) &&
                             scales_by_ldg() == 0;
    int rc;
    // Short contexts, fp16 output: runs of whole rows, merged inside the scan's CTAs -- one launch.
    // Measured against the split plan + merge kernel: it wins (1.2-1.9 us of 6-20 us per step) while
    // a row is at most 8 tiles, or at most 16 with enough rows to keep the SMs busy on whole rows
    // (a single CTA streams a row at a few tens of GB/s), and while the rows fit two resident
    // waves (beyond that equal runs of tiles balance better than whole rows).
    const int wt = whole_row_tiles(kWholeRowMaxTiles);
    const long long slots = (long long)sm_count() * T::CTAS_PER_SM;
    bool whole = p.tpb <= wt && (p.tpb <= wt / 2 || BH >= 24) && BH <= 2 * slots;
    // Longer rows (up to 4 x that, 8192 positions) when the rows by themselves fill the machine: whole rows
    // on at least three quarters of the resident slots read as fast as equal runs and save the merge kernel
    // (B32 H12 ctx 4096 34.8 vs 36.9 us, ctx 8192 66.3 vs 70.5 us, B16 H32 D128 ctx 8192 163.8 vs 168.4 us;
    // break-even at ctx 16384, 5 % slower at 32768, where fewer CTAs keep fewer bytes in flight).
    if (!whole && p.tpb <= 4 * wt && BH <= 2 * slots) {
        const long long per_cta = (BH + slots - 1) / slots;
        whole = 4 * ((BH + per_cta - 1) / per_cta) >= 3 * slots;
    }
    // Few rows (one request, a handful of heads): a cluster of up to eight CTAs per row, merged through
    // distributed shared memory, while a rank gets at most four tiles and all clusters are resident.
    // (Measured: B1 H12 ctx 1024 / 2048 / 4096 5.0 / 5.4 / 6.6 us per step replayed from a CUDA graph against
    // 6.2 / 8.4 / 9 us; below 8 tiles a row is done sooner by a single CTA.)
    if (out != nullptr && part == nullptr && qo.codes == nullptr && wt > 0 && forced_ctas() == 0 && p.tpb >= 8) {
        int cl = 8;
        while (cl > 2 && (cl > p.tpb || (long long)BH * cl > slots)) cl >>= 1;
        if (cl <= p.tpb && (long long)BH * cl <= slots && (p.tpb + cl - 1) / cl <= 4 &&
            clusters_fit<D>(cl, bulk_scales)) {
            const DecodePlan cp = make_cluster_plan(BH, S, cl);
            return bulk_scales ? launch_partial<D, true, false, 2>(Q, K, V, sQ, sK, sV, rows, S, cp, status, stream,
                                                                   PagedKV{}, out, cl)
                               : launch_partial<D, false, false, 2>(Q, K, V, sQ, sK, sV, rows, S, cp, status, stream,
                                                                    PagedKV{}, out, cl);
        }
    }
    if (out != nullptr && part == nullptr && qo.codes == nullptr && whole && forced_ctas() == 0) {
        const DecodePlan wp = make_whole_plan(BH, S, D, sm_count());
        return bulk_scales
                   ? launch_partial<D, true, false, 1>(Q, K, V, sQ, sK, sV, rows, S, wp, status, stream, PagedKV{}, out)
                   : launch_partial<D, false, false, 1>(Q, K, V, sQ, sK, sV, rows, S, wp, status, stream, PagedKV{}, out);
    }
    if (bulk_scales)
        rc = launch_partial<D, true>(Q, K, V, sQ, sK, sV, rows, S, p, status, stream);
    else
        rc = launch_partial<D, false>(Q, K, V, sQ, sK, sV, rows, S, p, status, stream);
    if (rc != I8TK_OK) return rc;
    // the merge may be scheduled while the scan drains: it waits (pdl_wait) for the scan's rows
    if (qo.codes != nullptr) {
        I8TK_CUDA(launch_after(decode_combine_kernel<D, true, false, true>, dim3(BH / heads), dim3(32 * heads), 0,
                               stream, (const float*)rows, BH, 0, p, out, part, PagedKV{}, qo));
        return I8TK_OK;
    }
    I8TK_CUDA(launch_after(decode_combine_kernel<D, true>, dim3((BH + 3) / 4), dim3(128), 0, stream,
                           (const float*)rows, BH, 0, p, out, part, PagedKV{}, QuantOut{}));
    return I8TK_OK;
}

// ---------------------------------------------------------------------------
// Scratch for the entry point that allocates nothing: a fixed block of device
// memory that is part of the library image.  Every GPU that loads the library
// carries it until the process exits.
// ---------------------------------------------------------------------------
constexpr size_t kStaticScratchBytes = 8u << 20;     // 8 MiB
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code `g_static_scratch` is only a handle for the symbol, not a device
// address.  The address is looked up once per device, with that device current.
int static_scratch_ptr(void** out) {
    static void* resolved[64] = {nullptr};
    int dev = 0;
    I8TK_CUDA(cudaGetDevice(&dev));
    I8TK_REQUIRE(dev >= 0 && dev < 64, I8TK_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
    if (resolved[dev] == nullptr) {
        void* p = nullptr;
        I8TK_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
        I8TK_REQUIRE(p != nullptr, I8TK_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
        resolved[dev] = p;
    }
    *out = resolved[dev];
    return I8TK_OK;
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

extern "C" int i8tk_decode_plan(int BH, int S, int head_dim, int* nctas, int* tiles_per_cta) {
    I8TK_REQUIRE(BH > 0 && S > 0 && nctas && tiles_per_cta, I8TK_ERR_INVALID_ARGUMENT, "bad plan arguments");
    I8TK_REQUIRE(head_dim == 64 || head_dim == 128, I8TK_ERR_UNSUPPORTED, "head_dim must be 64 or 128");
    const DecodePlan p = make_plan(BH, S, head_dim, sm_count());
    *nctas = p.nctas;
    *tiles_per_cta = p.tpc;
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

extern "C" int i8tk_decode_attention_forward_q8(const int8_t* Q, const int8_t* K, const int8_t* V,
                                                int8_t* out_i8, float* out_scales, void* out_f16,
                                                const float* sQ, const float* sK, const float* sV,
                                                int batch, int heads, int S, int head_dim,
                                                void* workspace, size_t workspace_bytes, i8tk_stream_t stream) {
    I8TK_REQUIRE(out_i8 && out_scales, I8TK_ERR_INVALID_ARGUMENT, "null pointer argument");
    I8TK_REQUIRE(batch > 0 && heads > 0 && heads <= 32, I8TK_ERR_UNSUPPORTED,
                 "per-token output quantisation takes 1..32 heads (one warp per head), got %d", heads);
    I8TK_REQUIRE((long long)batch * heads < (1ll << 31), I8TK_ERR_UNSUPPORTED, "batch * heads too large");
    I8TK_REQUIRE(aligned_to(out_i8, 4) && aligned_to(out_scales, 4), I8TK_ERR_ALIGNMENT,
                 "out_i8 and out_scales must be 4-byte aligned");
    const int BH = batch * heads;
    // the fp16 row is optional here: any aligned non-null pointer satisfies the common checks
    const int rc = check_decode_args(Q, K, V, out_f16 ? out_f16 : static_cast<void*>(out_i8), sQ, sK, sV, BH, S, head_dim);
    if (rc != I8TK_OK) return rc;
    I8TK_REQUIRE(out_f16 != nullptr || aligned_to(out_i8, 16), I8TK_ERR_ALIGNMENT, "out_i8 must be 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const QuantOut qo{out_i8, out_scales};
    if (head_dim == 64)
        return launch_decode<64>(Q, K, V, static_cast<__half*>(out_f16), nullptr, sQ, sK, sV, BH, S, workspace,
                                 workspace_bytes, st, qo, heads);
    return launch_decode<128>(Q, K, V, static_cast<__half*>(out_f16), nullptr, sQ, sK, sV, BH, S, workspace,
                              workspace_bytes, st, qo, heads);
}

extern "C" size_t i8tk_decode_static_scratch_bytes(void) { return kStaticScratchBytes; }

extern "C" int i8tk_decode_attention_forward_static(const int8_t* Q, const int8_t* K, const int8_t* V,
                                                    void* out_f16, const float* sQ, const float* sK,
                                                    const float* sV, int BH, int S, int head_dim,
                                                    i8tk_stream_t stream) {
    int rc = check_decode_args(Q, K, V, out_f16, sQ, sK, sV, BH, S, head_dim);
    if (rc != I8TK_OK) return rc;
    // what the contiguous forward really uses: the status block and the partial rows of its plan
    const size_t need = 256 + rows_bytes(make_plan(BH, S, head_dim, sm_count()), head_dim);
    I8TK_REQUIRE(need <= kStaticScratchBytes, I8TK_ERR_WORKSPACE,
                 "this shape needs %zu bytes of scratch; the built-in block holds %zu -- use "
                 "i8tk_decode_attention_forward with a caller-provided workspace",
                 need, (size_t)kStaticScratchBytes);
    void* scratch = nullptr;
    rc = static_scratch_ptr(&scratch);      // first call on a device resolves the symbol address
    if (rc != I8TK_OK) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (head_dim == 64)
        return launch_decode<64>(Q, K, V, static_cast<__half*>(out_f16), nullptr, sQ, sK, sV, BH, S,
                                 scratch, kStaticScratchBytes, st);
    return launch_decode<128>(Q, K, V, static_cast<__half*>(out_f16), nullptr, sQ, sK, sV, BH, S,
                              scratch, kStaticScratchBytes, st);
}

extern "C" int i8tk_decode_static_check_status(i8tk_stream_t stream) {
    void* scratch = nullptr;
    const int rc = static_scratch_ptr(&scratch);
    if (rc != I8TK_OK) return rc;
    uint32_t words[2] = {0u, 0u};
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    I8TK_CUDA(cudaMemcpyAsync(words, scratch, sizeof(words), cudaMemcpyDeviceToHost, st));
    I8TK_CUDA(cudaStreamSynchronize(st));
    if (words[0] == kDeviceTimeoutMagic) {
        I8TK_CUDA(cudaMemsetAsync(scratch, 0, sizeof(words), st));
        set_error("a kernel of i8tk_decode_attention_forward_static gave up a bounded wait");
        return I8TK_ERR_DEVICE_TIMEOUT;
    }
    return I8TK_OK;
}

extern "C" int i8tk_decode_exchange_ctas(int BH) { return BH > 0 ? (BH + 3) / 4 : 0; }

extern "C" int i8tk_decode_set_exchange_spin_limit(unsigned int polls) {
    g_exchange_spin_limit = polls ? polls : kExchangeSpinDefault;
    return I8TK_OK;
}

extern "C" int i8tk_decode_attention_seq_sharded(const int8_t* Q, const int8_t* K, const int8_t* V,
                                                 void* out_f16, const float* sQ, const float* sK,
                                                 const float* sV, int BH, int S_local, int head_dim,
                                                 void* workspace, size_t workspace_bytes,
                                                 const void* peer_parts, const void* peer_flags,
                                                 int rank, int world, unsigned int epoch,
                                                 i8tk_stream_t stream) {
    I8TK_REQUIRE(Q && out_f16 && sQ && workspace && peer_parts && peer_flags, I8TK_ERR_INVALID_ARGUMENT,
                 "null pointer argument");
    I8TK_REQUIRE(BH > 0 && S_local >= 0, I8TK_ERR_INVALID_ARGUMENT, "BH must be positive and S_local >= 0");
    I8TK_REQUIRE(world >= 1 && world <= 32 && rank >= 0 && rank < world, I8TK_ERR_INVALID_ARGUMENT,
                 "need 0 <= rank < world <= 32 (rank=%d world=%d)", rank, world);
    I8TK_REQUIRE(epoch != 0, I8TK_ERR_INVALID_ARGUMENT, "epoch starts at 1");
    I8TK_REQUIRE(head_dim == 64 || head_dim == 128, I8TK_ERR_UNSUPPORTED,
                 "decode attention supports head_dim 64 or 128 (got %d)", head_dim);
    I8TK_REQUIRE(aligned_to(workspace, 256) && workspace_bytes >= 256, I8TK_ERR_WORKSPACE,
                 "workspace must be 256-byte aligned and at least 256 bytes");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    uint32_t* status = reinterpret_cast<uint32_t*>(workspace);
    float* rows = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(workspace) + 256);
    DecodePlan p{};
    if (S_local > 0) {
        const int rc = check_decode_args(Q, K, V, out_f16, sQ, sK, sV, BH, S_local, head_dim);
        if (rc != I8TK_OK) return rc;
        p = make_plan(BH, S_local, head_dim, sm_count());
        const size_t need = 256 + rows_bytes(p, head_dim);
        I8TK_REQUIRE(workspace_bytes >= need, I8TK_ERR_WORKSPACE,
                     "decode workspace too small: need %zu bytes, got %zu", need, workspace_bytes);
        const bool bulk = (S_local % 4 == 0) && aligned_to(sK, 16) && aligned_to(sV, 16);
        int rc2;
        if (head_dim == 64)
            rc2 = bulk ? launch_partial<64, true>(Q, K, V, sQ, sK, sV, rows, S_local, p, status, st)
                       : launch_partial<64, false>(Q, K, V, sQ, sK, sV, rows, S_local, p, status, st);
        else
            rc2 = bulk ? launch_partial<128, true>(Q, K, V, sQ, sK, sV, rows, S_local, p, status, st)
                       : launch_partial<128, false>(Q, K, V, sQ, sK, sV, rows, S_local, p, status, st);
        if (rc2 != I8TK_OK) return rc2;
    }
    const int grid = (BH + 3) / 4;
    float* const* pp = static_cast<float* const*>(peer_parts);
    uint32_t* const* pf = static_cast<uint32_t* const*>(peer_flags);
    const int empty = S_local == 0 ? 1 : 0;
    if (head_dim == 64)
        I8TK_CUDA(launch_after(decode_exchange_kernel<64>, dim3(grid), dim3(128), 0, st, (const float*)rows, BH, p,
                               empty, pp, pf, rank, world, epoch, g_exchange_spin_limit, static_cast<__half*>(out_f16),
                               status));
    else
        I8TK_CUDA(launch_after(decode_exchange_kernel<128>, dim3(grid), dim3(128), 0, st, (const float*)rows, BH, p,
                               empty, pp, pf, rank, world, epoch, g_exchange_spin_limit, static_cast<__half*>(out_f16),
                               status));
    return I8TK_OK;
}

static int paged_forward(const int8_t* Q, const int8_t* K_pool, const int8_t* V_pool,
                         void* out_f16, const float* sQ, const float* sK_pool,
                         const float* sV_pool, const int32_t* page_table,
                         const int32_t* seq_lens, int batch, int heads, int max_seq_len,
                         int page_size, int max_pages_per_seq, int head_dim, int num_pages, void* workspace,
                         size_t workspace_bytes, i8tk_stream_t stream) {
    I8TK_REQUIRE(Q && K_pool && V_pool && out_f16 && sQ && sK_pool && sV_pool && page_table && seq_lens,
                 I8TK_ERR_INVALID_ARGUMENT, "null pointer argument");
    I8TK_REQUIRE(batch > 0 && heads > 0 && max_seq_len > 0 && max_pages_per_seq > 0, I8TK_ERR_INVALID_ARGUMENT,
                 "sizes must be positive");
    I8TK_REQUIRE(head_dim == 64 || head_dim == 128, I8TK_ERR_UNSUPPORTED, "head_dim must be 64 or 128 (got %d)",
                 head_dim);
    I8TK_REQUIRE(page_size == 16 || page_size == 32 || page_size == 64 || page_size == 128, I8TK_ERR_UNSUPPORTED,
                 "page_size must be 16, 32, 64 or 128 (got %d)", page_size);
    I8TK_REQUIRE((long long)max_pages_per_seq * page_size >= max_seq_len, I8TK_ERR_INVALID_ARGUMENT,
                 "max_seq_len %d does not fit %d pages of %d", max_seq_len, max_pages_per_seq, page_size);
    I8TK_REQUIRE(aligned_to(Q, 16) && aligned_to(K_pool, 16) && aligned_to(V_pool, 16) && aligned_to(sK_pool, 16) &&
                     aligned_to(sV_pool, 16),
                 I8TK_ERR_ALIGNMENT, "Q, the pools and their scales must be 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int BH = batch * heads;
    // the longest request only sizes the grid; the runs are cut on the device from the real lengths
    const DecodePlan p = make_plan(BH, max_seq_len, head_dim, sm_count());
    const RaggedLayout lay = ragged_layout(BH, batch, p.nctas, head_dim);
    I8TK_REQUIRE(workspace != nullptr && workspace_bytes >= lay.total, I8TK_ERR_WORKSPACE,
                 "decode workspace too small: need %zu bytes, got %zu", lay.total, workspace_bytes);
    I8TK_REQUIRE(aligned_to(workspace, 256), I8TK_ERR_ALIGNMENT, "workspace must be 256-byte aligned");
    unsigned char* ws = reinterpret_cast<unsigned char*>(workspace);
    uint32_t* status = reinterpret_cast<uint32_t*>(ws);
    float* rows = reinterpret_cast<float*>(ws + lay.rows_off);
    int* hdr = reinterpret_cast<int*>(ws + lay.hdr_off);
    int4* starts = reinterpret_cast<int4*>(ws + lay.starts_off);
    int* prefix = reinterpret_cast<int*>(ws + lay.prefix_off);
    const PagedKV pg{page_table, seq_lens, heads, page_size, max_pages_per_seq, batch, max_seq_len, num_pages, hdr, prefix, starts};
    const int resident = sm_count() * (head_dim == 64 ? DecodeTraits<64>::CTAS_PER_SM : DecodeTraits<128>::CTAS_PER_SM);
    I8TK_CUDA(launch_after(decode_ragged_plan_kernel, dim3(1), dim3(1024), 0, st, seq_lens, batch, heads, max_seq_len,
                           p.nctas, resident < p.nctas ? resident : p.nctas, paged_target_tiles(kPagedTargetTiles), hdr,
                           prefix, starts, status));
    int rc;
    if (head_dim == 64) {
        rc = launch_partial<64, true, true>(Q, K_pool, V_pool, sQ, sK_pool, sV_pool, rows, max_seq_len, p, status, st, pg);
        if (rc != I8TK_OK) return rc;
        I8TK_CUDA(launch_after(decode_combine_kernel<64, true, true>, dim3((BH + 3) / 4), dim3(128), 0, st,
                               (const float*)rows, BH, 0, p, static_cast<__half*>(out_f16), (float*)nullptr, pg, QuantOut{}));
    } else {
        rc = launch_partial<128, true, true>(Q, K_pool, V_pool, sQ, sK_pool, sV_pool, rows, max_seq_len, p, status, st, pg);
        if (rc != I8TK_OK) return rc;
        I8TK_CUDA(launch_after(decode_combine_kernel<128, true, true>, dim3((BH + 3) / 4), dim3(128), 0, st,
                               (const float*)rows, BH, 0, p, static_cast<__half*>(out_f16), (float*)nullptr, pg, QuantOut{}));
    }
    return I8TK_OK;
}

extern "C" int i8tk_decode_attention_paged(const int8_t* Q, const int8_t* K_pool, const int8_t* V_pool,
                                           void* out_f16, const float* sQ, const float* sK_pool,
                                           const float* sV_pool, const int32_t* page_table,
                                           const int32_t* seq_lens, int batch, int heads, int max_seq_len,
                                           int page_size, int max_pages_per_seq, int head_dim, void* workspace,
                                           size_t workspace_bytes, i8tk_stream_t stream) {
    return paged_forward(Q, K_pool, V_pool, out_f16, sQ, sK_pool, sV_pool, page_table, seq_lens, batch, heads,
                         max_seq_len, page_size, max_pages_per_seq, head_dim, 0, workspace, workspace_bytes, stream);
}

extern "C" int i8tk_decode_attention_paged_checked(const int8_t* Q, const int8_t* K_pool, const int8_t* V_pool,
                                                   void* out_f16, const float* sQ, const float* sK_pool,
                                                   const float* sV_pool, const int32_t* page_table,
                                                   const int32_t* seq_lens, int batch, int heads, int max_seq_len,
                                                   int page_size, int max_pages_per_seq, int head_dim, int num_pages,
                                                   void* workspace, size_t workspace_bytes, i8tk_stream_t stream) {
    I8TK_REQUIRE(num_pages > 0, I8TK_ERR_INVALID_ARGUMENT, "num_pages must be positive (got %d)", num_pages);
    return paged_forward(Q, K_pool, V_pool, out_f16, sQ, sK_pool, sV_pool, page_table, seq_lens, batch, heads,
                         max_seq_len, page_size, max_pages_per_seq, head_dim, num_pages, workspace, workspace_bytes,
                         stream);
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
    const DecodePlan none{};
    if (head_dim == 64)
        decode_combine_kernel<64, false><<<grid, 128, 0, st>>>(parts, BH, nparts, none,
                                                               static_cast<__half*>(out_f16), nullptr, PagedKV{}, QuantOut{});
    else
        decode_combine_kernel<128, false><<<grid, 128, 0, st>>>(parts, BH, nparts, none,
                                                                static_cast<__half*>(out_f16), nullptr, PagedKV{}, QuantOut{});
    I8TK_CUDA(cudaGetLastError());
    return I8TK_OK;
}
