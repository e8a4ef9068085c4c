/*
 * i8tk.h -- C ABI of the B200 (sm_100a) INT8 transformer-kernel library.
 *
 * Drop-in boundary for the hot path of Ashuuuri/int8-transformer-kernels:
 * split-KV flash-decoding attention over an INT8 KV cache, the per-token INT8
 * quantiser that feeds it, and the fused INT8 MLP.  Every entry point takes
 * plain device pointers and sizes, an explicit CUDA stream, caller-owned
 * workspace, and returns an int status (0 = success).  Nothing here allocates
 * device memory, synchronises the device, or depends on PyTorch.
 *
 * The reference exposes the same operations as C++-linkage launchers declared
 * in kernels/int8_ext.cu:27-70 (raw pointers + ints, void return, legacy
 * default stream, library-owned static scratch).  Each declaration below cites
 * the reference interface it replaces.
 */
#ifndef I8TK_H_
#define I8TK_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* A cudaStream_t passed through an opaque pointer (NULL = legacy default stream). */
typedef void* i8tk_stream_t;

enum i8tk_status {
    I8TK_OK = 0,
    I8TK_ERR_INVALID_ARGUMENT = 1,  /* null pointer, non-positive size, bad flag      */
    I8TK_ERR_UNSUPPORTED = 2,       /* a head_dim the kernel does not take, a shape too large */
    I8TK_ERR_WORKSPACE = 3,         /* workspace null or smaller than *_workspace_bytes */
    I8TK_ERR_ALIGNMENT = 4,         /* pointer not aligned as documented              */
    I8TK_ERR_CUDA = 5,              /* a CUDA runtime/driver call or launch failed    */
    I8TK_ERR_DEVICE_TIMEOUT = 6     /* a bounded device-side wait gave up             */
};

/* Human-readable name of a status code (static storage). */
const char* i8tk_status_string(int status);
/* Detail of the last failure on the calling thread (static thread-local storage). */
const char* i8tk_last_error(void);
/* Library version, major*10000 + minor*100 + patch. */
int i8tk_version(void);

/* Every device-side wait in this library is bounded.  A kernel that gives up
 * returns normally (the context stays usable) after recording the fact in the
 * status block, the first 8 bytes of the workspace it was given:
 *   word 0  a marker for "a wait of the LAST call on this workspace gave up"; the first
 *           kernel of every call clears it, so it needs no initialisation
 *   word 1  a count of such give-ups that no kernel ever clears: zero it once after
 *           allocating the workspace and it tells, however rarely it is read, whether
 *           any call since then failed
 * The outputs of a call that gave up are not valid (the fused MLP also turns the row
 * scales it could not finish into NaN, so the failure travels with the data).
 * i8tk_check_status_word copies word 0 back (it synchronises `stream`) and returns
 * I8TK_ERR_DEVICE_TIMEOUT if the marker is there.  i8tk_selftest_bounded_wait
 * launches a probe kernel that waits `polls` times (about a microsecond each)
 * on a barrier nothing signals and then records the give-up in the 8-byte block at
 * status_word.  Neither has a counterpart in the reference, which checks no CUDA
 * error at all. */
int i8tk_check_status_word(const void* status_word, i8tk_stream_t stream);
int i8tk_selftest_bounded_wait(void* status_word, int polls, i8tk_stream_t stream);

/* ------------------------------------------------------------------------
 * Per-token symmetric INT8 quantiser.
 * Replaces the torch code tests/test_int8.py:47-63 (quantize_per_token) ==
 * validation/validate_int8.py:63-66 (q_per_token); the reference has no native
 * per-token quantiser (kernels/quant_utils.cu is per-tensor).
 *   x       [rows, cols] fp32 (or fp16 for the _f16 form), row-major
 *   q       [rows, cols] int8
 *   scales  [rows]       fp32:  max(absmax,1e-8)/127, codes = clamp(rne(x/scale),-128,127)
 * Results are bit-identical to the torch code for finite inputs.  A NaN in a row is ignored by
 * the row maximum here (fmaxf drops it) where torch's amax propagates it into the scale; the
 * NaN element itself becomes an unspecified code in both.  cols >= 1.
 * ---------------------------------------------------------------------- */
int i8tk_quantize_per_token_f32(const float* x, int8_t* q, float* scales,
                                int64_t rows, int cols, i8tk_stream_t stream);
int i8tk_quantize_per_token_f16(const void* x_f16, int8_t* q, float* scales,
                                int64_t rows, int cols, i8tk_stream_t stream);

/* Producer-side quantisation: the steps either side of the INT8 path that the reference
 * leaves to eager torch code (several elementwise kernels per tensor,
 * bench/bench_block.py:59-63,93-94,107-151) and names as its largest remaining cost
 * (OPTIMIZATION.md:241-246).  No counterpart among the reference's launchers.
 *
 * i8tk_layernorm_quantize_f16: y = LayerNorm(x) without affine parameters over the last
 * dimension (biased variance, `eps` inside the square root, as torch's F.layer_norm), rounded
 * to fp16 as torch would store it, then quantised per token with the scale
 * i8tk_quantize_per_token_f16 would give that fp16 tensor and the code round(y * (1/scale))
 * (rows up to 2048 wide; wider rows divide).  A code can differ by one step from the
 * divide-then-round result when the quotient lies within 1.6e-5 of k + 0.5; against torch's
 * LayerNorm followed by the quantiser the codes differ by at most one step on < 0.2 % of the
 * elements, because the normalised value itself differs in its last bit that often.
 *   x [rows, d_model] fp16, 16-byte aligned; q [rows, d_model] int8; scales [rows] fp32.
 *   d_model a multiple of 8, at most 4096.
 *
 * i8tk_kv_append_quantize_f16: the new token's K and V rows, k_new / v_new [BH, head_dim]
 * fp16, quantised per token and written into the INT8 cache K / V [BH, S_cap, head_dim] at
 * position pos_per_row[bh] (device int32[BH]) or, when pos_per_row is NULL, at `pos` for every
 * row; their scales go to sK / sV [BH, S_cap].  Rows whose position is outside [0, S_cap) are
 * skipped.  head_dim a multiple of 32, at most 256.
 *
 * i8tk_quantize_qkv_heads_f16: the fused QKV projection qkv [batch*seq_len, 3*heads*head_dim]
 * fp16 (q heads, then k heads, then v heads in each row) quantised per token and per head
 * straight into the head-major layout the attention kernels take: out int8
 * [3][batch][heads][seq_len][head_dim], scales fp32 [3][batch][heads][seq_len] -- the split,
 * view, transpose and contiguous copies of bench/bench_block.py:96-101 disappear into the
 * quantiser.  Codes and scales are bit-identical to i8tk_quantize_per_token_f16 on the
 * transposed tensors.  head_dim 64 or 128.
 *
 * i8tk_dequantize_per_token_f16: out = fp16(q * scales[row] (+ residual)), the step after the
 * INT8 MLP (bench/bench_block.py:113: .float() * scale -> .half(), then the residual add);
 * residual_f16 may be NULL.  cols a multiple of 16. */
int i8tk_quantize_qkv_heads_f16(const void* qkv_f16, int8_t* out, float* scales,
                                int batch, int seq_len, int heads, int head_dim, i8tk_stream_t stream);
int i8tk_dequantize_per_token_f16(const int8_t* q, const float* scales, const void* residual_f16,
                                  void* out_f16, int64_t rows, int cols, i8tk_stream_t stream);
int i8tk_layernorm_quantize_f16(const void* x_f16, int8_t* q, float* scales,
                                int64_t rows, int d_model, float eps, i8tk_stream_t stream);
int i8tk_kv_append_quantize_f16(const void* k_new_f16, const void* v_new_f16,
                                int8_t* K, int8_t* V, float* sK, float* sV,
                                const int32_t* pos_per_row, int pos,
                                int BH, int S_cap, int head_dim, i8tk_stream_t stream);

/* Per-tensor FP16 -> INT8 with a dynamically computed scale, and the inverse.
 * Replaces quantize_fp16_to_int8 / dequantize_int8_to_fp16
 * (kernels/int8_common.cuh:54-59, kernels/quant_utils.cu:57-77).
 * d_scale (device float[1]) receives absmax/127 (it is also the cell the
 * absmax reduction runs in); codes = clamp(rne(x/scale), -128, 127). */
int i8tk_quantize_fp16_to_int8(const void* x_f16, int8_t* q, float* d_scale,
                               int64_t n, i8tk_stream_t stream);
int i8tk_dequantize_int8_to_fp16(const int8_t* q, void* out_f16, float scale,
                                 int64_t n, i8tk_stream_t stream);

/* ------------------------------------------------------------------------
 * INT8-KV decode attention (seq_q == 1), split-KV flash decoding.
 * Replaces int8_decode_attention_forward (kernels/int8_ext.cu:34-38,
 * kernels/int8_decode_attention.cu:443-547).
 *   Q  [BH, D] int8          sQ [BH]    fp32
 *   K  [BH, S, D] int8       sK [BH*S]  fp32      (contiguous, row-major)
 *   V  [BH, S, D] int8       sV [BH*S]  fp32
 *   out [BH, D] fp16
 * score_j = (q.k_j) * sQ * sK_j / sqrt(D); out = softmax(score) . (sV_j * v_j).
 * D in {64,128}.  Q, K, V must be 16-byte aligned, scales 4-byte aligned.
 * workspace: >= i8tk_decode_workspace_bytes(BH,S,D) bytes, 256-byte aligned,
 * private to this call until it completes on `stream`.
 * ---------------------------------------------------------------------- */
size_t i8tk_decode_workspace_bytes(int BH, int S, int head_dim);
int i8tk_decode_attention_forward(const int8_t* Q, const int8_t* K, const int8_t* V,
                                  void* out_f16,
                                  const float* sQ, const float* sK, const float* sV,
                                  int BH, int S, int head_dim,
                                  void* workspace, size_t workspace_bytes,
                                  i8tk_stream_t stream);

/* The same forward with the result leaving as INT8 for the GEMM that follows attention (the
 * output projection): one scale per token over its heads*head_dim outputs,
 *   out_scales[b] = max(|fp16 out[b]|, 1e-8) / 127,   out_i8[b][:] = rne(fp16 out[b][:] / scale)
 * -- exactly what i8tk_quantize_per_token_f16 gives on the fp16 result viewed as
 * [batch, heads*head_dim], without writing and re-reading that tensor (the eager
 * quantise-after-attention step of bench/bench_block.py:107-113; OPTIMIZATION.md:241-246).
 *   out_i8 int8 [batch, heads*head_dim]; out_scales fp32 [batch]; out_f16 fp16 [batch*heads,
 *   head_dim] or NULL.  1 <= heads <= 32.  Workspace as i8tk_decode_attention_forward with
 *   BH = batch*heads.  No counterpart among the reference's launchers. */
int i8tk_decode_attention_forward_q8(const int8_t* Q, const int8_t* K, const int8_t* V,
                                     int8_t* out_i8, float* out_scales, void* out_f16,
                                     const float* sQ, const float* sK, const float* sV,
                                     int batch, int heads, int S, int head_dim,
                                     void* workspace, size_t workspace_bytes, i8tk_stream_t stream);

/* The same operation for callers that must not allocate device memory and have
 * no spare buffer to lend: plugin "enqueue" hooks of serving runtimes, code
 * running after the application has handed the whole device to its own memory
 * pool, or hot loops where an allocation would stall the device.  It has no
 * counterpart in the reference (whose launcher grows a cudaMalloc'ed static
 * buffer on demand, kernels/int8_decode_attention.cu:430-440).
 *
 * The scratch is a fixed 8 MiB block that is part of the library image
 * (i8tk_decode_static_scratch_bytes()); every GPU that loads the library
 * carries it until the process exits.  The call itself allocates nothing and
 * frees nothing.  Shapes whose partial rows (plus the 256-byte status block) do
 * not fit the block are refused with I8TK_ERR_WORKSPACE -- on a 148-SM part the
 * serving shapes need well under 4 MiB; only very many (b,h) rows with a very
 * short context go over.
 *
 * The first call on each device looks up the device address of the block
 * (cudaGetSymbolAddress); make that first call outside any stream capture.
 * All calls on a device share the one block and it keeps whatever the last
 * call left there; the kernels overwrite every row they later read, so nothing
 * has to be cleared.  Two calls that may run on the GPU at the same time
 * (different streams) would race on it: serialise them, or use the
 * workspace form above for one of them.  Two host threads that make their
 * first call on the same device at the same moment both look the address up
 * and store the same value: harmless.
 *
 * The caller cannot reach the block, so its status block is read through
 * i8tk_decode_static_check_status: it synchronises `stream`, returns
 * I8TK_ERR_DEVICE_TIMEOUT if a kernel of the last static call on the current
 * device gave up a bounded wait, and clears the record. */
size_t i8tk_decode_static_scratch_bytes(void);
int i8tk_decode_static_check_status(i8tk_stream_t stream);
int i8tk_decode_attention_forward_static(const int8_t* Q, const int8_t* K, const int8_t* V,
                                         void* out_f16,
                                         const float* sQ, const float* sK, const float* sV,
                                         int BH, int S, int head_dim, i8tk_stream_t stream);

/* Paged INT8 KV cache with a length per request: the layout a serving stack keeps (the
 * reference's own kernel takes contiguous tensors only; its benchmark compares against a
 * paged peer, bench/bench_decode_sota.py:44,65-90).
 *   K_pool, V_pool  int8 [num_pages, heads, page_size, head_dim]
 *   sK_pool, sV_pool fp32 [num_pages, heads, page_size]
 *   page_table      int32 [batch, max_pages_per_seq] (device): request b holds, in sequence
 *                   order, pages page_table[b][0 .. ceil(seq_lens[b] / page_size))
 *   seq_lens        int32 [batch] (device), each in [0, max_seq_len]; a request of length 0
 *                   gets a zero output row
 *   Q int8 [batch*heads, head_dim], sQ fp32 [batch*heads], out fp16 [batch*heads, head_dim]
 * max_seq_len is a host-side upper bound on seq_lens (it sizes the grid and the workspace:
 * i8tk_decode_workspace_bytes(batch*heads, max_seq_len, head_dim)); an entry of seq_lens outside
 * [0, max_seq_len] is read as the nearer end of that range, so a damaged length cannot send the
 * kernels past a page-table row.  Page ids are trusted here (see the _checked form below).  The lengths themselves
 * are read on the device only: a one-CTA kernel counts the 128-position tiles each request
 * really has and cuts their sequence into equal runs for the CTAs of the scan, so a batch of
 * mixed lengths takes the time of the bytes it reads, not of batch x the longest request.
 * page_size 16, 32, 64 or 128; head_dim 64 or 128; pools 16-byte aligned. */
int i8tk_decode_attention_paged(const int8_t* Q, const int8_t* K_pool, const int8_t* V_pool,
                                void* out_f16, const float* sQ,
                                const float* sK_pool, const float* sV_pool,
                                const int32_t* page_table, const int32_t* seq_lens,
                                int batch, int heads, int max_seq_len, int page_size,
                                int max_pages_per_seq, int head_dim,
                                void* workspace, size_t workspace_bytes, i8tk_stream_t stream);
/* The same with the number of pages in the pools given: a page id outside [0, num_pages) met
 * on the device is not followed -- page 0 is read in its place, so nothing outside the pools
 * is touched -- and recorded in the status block: i8tk_check_status_word on the workspace then
 * returns I8TK_ERR_INVALID_ARGUMENT (the output rows of the requests concerned are not valid). */
int i8tk_decode_attention_paged_checked(const int8_t* Q, const int8_t* K_pool, const int8_t* V_pool,
                                        void* out_f16, const float* sQ,
                                        const float* sK_pool, const float* sV_pool,
                                        const int32_t* page_table, const int32_t* seq_lens,
                                        int batch, int heads, int max_seq_len, int page_size,
                                        int max_pages_per_seq, int head_dim, int num_pages,
                                        void* workspace, size_t workspace_bytes, i8tk_stream_t stream);

/* Sequence-sharded form: the same scan over this caller's KV positions, but
 * the result is left as ONE unnormalised online-softmax partial per (b,h):
 *   part[bh] = { m (log2 units), l, 0, 0, acc[0..D) }   -- D+4 floats per row
 * to be merged across shards with i8tk_decode_combine_partials.  Generalises
 * the partial/combine hand-off of kernels/int8_decode_attention.cu:274-426
 * from splits inside one GPU to KV chunks on several GPUs. */
int i8tk_decode_attention_partial(const int8_t* Q, const int8_t* K, const int8_t* V,
                                  float* part,
                                  const float* sQ, const float* sK, const float* sV,
                                  int BH, int S, int head_dim,
                                  void* workspace, size_t workspace_bytes,
                                  i8tk_stream_t stream);
/* parts: [nparts, BH, D+4] fp32 as written above (gathered from all shards);
 * out: [BH, D] fp16.  Partials with l <= 0 (empty shard) are skipped, as
 * kernels/int8_decode_attention.cu:414 does. */
int i8tk_decode_combine_partials(const float* parts, int nparts, int BH, int head_dim,
                                 void* out_f16, i8tk_stream_t stream);

/* KV-sequence-sharded decode with the exchange fused into the merge kernel:
 * every rank (one process per GPU) calls this at the same step with its own
 * chunk of the KV sequence (S_local positions, may be 0).  The kernel merges
 * the local partials, stores the merged (m, l, acc) row of each (b,h) straight
 * into every rank's gather buffer through peer-mapped pointers (NVLink), sets a
 * per-CTA flag there, waits -- bounded -- for the other ranks' flags and writes
 * the final fp16 result on every rank.  No collective library is involved.
 *   peer_parts  device array of `world` pointers: rank r's gather buffer,
 *               2 * world * BH * (D+4) floats, mapped into this process
 *   peer_flags  device array of `world` pointers: rank r's flag array,
 *               world * i8tk_decode_exchange_ctas(BH) 32-bit words, zeroed once
 *   epoch       1 on the first call, +1 on every call, the same on all ranks
 * The buffers must be peer-accessible allocations (e.g. torch symmetric
 * memory).  Extends the partial/combine hand-off of
 * kernels/int8_decode_attention.cu:389-426 across GPUs; no counterpart in the
 * reference, which is single-GPU. */
int i8tk_decode_exchange_ctas(int BH);
/* How many times the exchange kernel polls another rank's flag before it gives up (each poll is
 * a load of memory a peer writes, about a microsecond; default 2^21, i.e. seconds).  0 restores
 * the default.  Process-wide; a supervisor that prefers a fast error to a long wait lowers it. */
int i8tk_decode_set_exchange_spin_limit(unsigned int polls);
int i8tk_decode_attention_seq_sharded(const int8_t* Q, const int8_t* K, const int8_t* V,
                                      void* out_f16,
                                      const float* sQ, const float* sK, const float* sV,
                                      int BH, int S_local, int head_dim,
                                      void* workspace, size_t workspace_bytes,
                                      const void* peer_parts, const void* peer_flags,
                                      int rank, int world, unsigned int epoch,
                                      i8tk_stream_t stream);

/* Floats per (b,h) row of a partial: head_dim + 4. */
int i8tk_decode_partial_stride(int head_dim);

/* Measurement hook (no counterpart in the reference): two cudaEvent_t handles
 * that the decode calls made afterwards BY THIS THREAD record on their stream
 * immediately before and after the streaming (pass 1) kernel, so a benchmark
 * can time that kernel apart from the merge kernel.  Pass NULL, NULL to stop. */
int i8tk_decode_set_probe_events(void* start_event, void* stop_event);

/* Describes how a call would be divided (for tests and tuning): the number of
 * persistent CTAs launched and the 128-position KV tiles each one scans. */
int i8tk_decode_plan(int BH, int S, int head_dim, int* nctas, int* tiles_per_cta);

/* ------------------------------------------------------------------------
 * INT8 prefill attention (seq_q == seq_kv, no causal mask), per-token scales.
 * Replaces int8_attention_forward (kernels/int8_ext.cu:28-32,
 * kernels/int8_attention.cu:926-1028).
 *   Q, K, V  [batch, heads, seq_len, head_dim] int8, contiguous
 *   sQ, sK, sV  fp32 [batch*heads*seq_len]
 *   out      [batch, heads, seq_len, head_dim] fp16
 * score[i][j] = (q_i.k_j) * sQ_i * sK_j / sqrt(D); P*sV and V go through fp16
 * into an fp32 accumulator, as in the reference.  Any seq_len >= 1 (a partial
 * last tile of 128 positions is masked; the reference takes a scalar fallback
 * when seq_len is not a multiple of 64).  head_dim 64 or 128: anything else
 * returns I8TK_ERR_UNSUPPORTED.  workspace: i8tk_attention_workspace_bytes(...) bytes,
 * 256-byte aligned (the status word and an fp16 copy of V * sV, made once per call so
 * that the query tiles of a head do not each convert V again).
 * ---------------------------------------------------------------------- */
size_t i8tk_attention_workspace_bytes(int batch, int heads, int seq_len, int head_dim);
int i8tk_attention_forward(const int8_t* Q, const int8_t* K, const int8_t* V, void* out_f16,
                           const float* sQ, const float* sK, const float* sV,
                           int batch, int heads, int seq_len, int head_dim,
                           void* workspace, size_t workspace_bytes, i8tk_stream_t stream);

/* ------------------------------------------------------------------------
 * Fused INT8 MLP:  out = requant( (requant(GELU((x.W1)*sx*sW1 + b1))) . W2 * sh * sW2 )
 * Replaces int8_mlp_forward, int8_mlp_forward_per_channel,
 * int8_mlp_forward_per_channel_bias and int8_mlp_forward_prepacked
 * (kernels/int8_ext.cu:40-68, kernels/int8_mlp.cu:1231-1314) with one entry
 * point and flags.
 *   x   [T, d_model] int8
 *   W1  [d_model, d_ff] int8, W2 [d_ff, d_model] int8          (default), or
 *   W1T [d_ff, d_model],      W2T [d_model, d_ff] when I8TK_MLP_PREPACKED
 *   scale_x   fp32 [T]       (I8TK_MLP_X_PER_TOKEN)   else [1]
 *   scale_W1  fp32 [d_ff]    (I8TK_MLP_W_PER_CHANNEL) else [1]
 *   scale_W2  fp32 [d_model] (I8TK_MLP_W_PER_CHANNEL) else [1]
 *   bias1     fp32 [d_ff] or NULL       (added before GELU)
 *   out       [T, d_model] int8
 *   out_row_scales  fp32 [T] or NULL.  Non-NULL: the output is requantised per
 *                   token and its scales written here.  NULL: legacy dynamic
 *                   per-tensor output scale, written to *out_tensor_scale.
 *   out_tensor_scale device fp32[1] or NULL (required when out_row_scales is NULL)
 * Any positive T, d_model and d_ff.  Widths that are multiples of 128 run in place (all
 * pointers 16-byte aligned); other widths are first copied into zero-padded buffers of the
 * next multiple of 128 inside the workspace, which changes no result (no alignment needed
 * then).  The reference gates T, d_model and d_ff on 128 and otherwise takes scalar kernels
 * under static scales that leave out_row_scales unwritten
 * (kernels/int8_mlp.cu:1023-1026,1194-1225); that arithmetic is available here, for any
 * shape, as I8TK_MLP_STATIC_SCALES: per-tensor scales only, no bias, hidden codes under the
 * scale sx*sW1*d_model and output codes under that * sW2 * d_ff, which is written to
 * *out_tensor_scale (out_row_scales must be NULL).
 *
 * Workspace reuse.  A forward starts with a small kernel that presets the row-maxima flag
 * arrays in the workspace.  Both GEMMs also leave those arrays preset when they are done with
 * them, so a caller that gives the SAME workspace to consecutive calls of the SAME T, d_model,
 * d_ff and layout flags on one stream, and lets nothing else write to it in between, may pass
 * I8TK_MLP_WORKSPACE_KEPT from the second call on: the preset kernel is then skipped (2-4 us
 * per forward).  The first call on a workspace, or after a change of shape, must not pass it.
 *
 * Rounding of the first epilogue.  By default v = fma(acc*sx, sW1, b1) and GELU uses the
 * hardware tanh approximation (relative error 2^-11, the size of the fp16 rounding that
 * follows): against the reference's source order this moves an int8 code of the hidden
 * activations by one step on about 1 % of the elements, inside the reference's own
 * tolerance for its kernel (max-abs 0.05 against its simulation).  With
 * I8TK_MLP_REFERENCE_ROUNDING the epilogue follows the reference's source operation by
 * operation -- (acc*sx)*sW1 then + b1, each rounded, and tanhf (kernels/int8_mlp.cu:437-440,
 * kernels/int8_common.cuh:9-13) -- at roughly half the GEMM1 speed.
 * ---------------------------------------------------------------------- */
enum i8tk_mlp_flags {
    I8TK_MLP_X_PER_TOKEN = 1,
    I8TK_MLP_W_PER_CHANNEL = 2,
    I8TK_MLP_PREPACKED = 4,
    I8TK_MLP_REFERENCE_ROUNDING = 8,
    I8TK_MLP_STATIC_SCALES = 16,
    I8TK_MLP_WORKSPACE_KEPT = 32
};
size_t i8tk_mlp_workspace_bytes(int T, int d_model, int d_ff, int flags);
int i8tk_mlp_forward(const int8_t* x, const int8_t* W1, const int8_t* W2, int8_t* out,
                     const float* scale_x, const float* scale_W1, const float* scale_W2,
                     const float* bias1, float* out_row_scales, float* out_tensor_scale,
                     int T, int d_model, int d_ff, int flags,
                     void* workspace, size_t workspace_bytes, i8tk_stream_t stream);

/* One INT8 GEMM of the MLP on its own: out fp16 [T, N] = (x . W) * scale_x[row] * scale_W[col]
 * (+ bias[col]), x int8 [T, K], W int8 [K, N] (or [N, K] with I8TK_MLP_PREPACKED), scale_x fp32
 * [T] with I8TK_MLP_X_PER_TOKEN else [1], scale_W fp32 [N] with I8TK_MLP_W_PER_CHANNEL else [1].
 * The tensor-core kernel of i8tk_mlp_forward with its plain epilogue
 * (kernels/int8_mlp.cu:333-485 with apply_gelu = false and no row statistics); used for the
 * attention output projection when attention hands over INT8 (i8tk_decode_attention_forward_q8).
 * K and N multiples of 128; workspace: 256 bytes (the status block). */
int i8tk_linear_i8_f16(const int8_t* x, const int8_t* W, const float* scale_x, const float* scale_W,
                       const float* bias, void* out_f16, int T, int K, int N, int flags,
                       void* workspace, size_t workspace_bytes, i8tk_stream_t stream);

/* W1 [d_model,d_ff] -> W1T [d_ff,d_model]; W2 [d_ff,d_model] -> W2T [d_model,d_ff].
 * Replaces transpose_int8_weights (kernels/int8_ext.cu:58-61,
 * kernels/int8_mlp.cu:1288-1297). */
int i8tk_transpose_int8_weights(const int8_t* W1, const int8_t* W2,
                                int8_t* W1T, int8_t* W2T,
                                int d_model, int d_ff, i8tk_stream_t stream);

#ifdef __cplusplus
}  /* extern "C" */
#endif
#endif  /* I8TK_H_ */
