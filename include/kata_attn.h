/* kata_attn.h - C ABI of the B200 gated-GQA attention path of the kata engine.
 *
 * The reference engine (wolfjpy/kata) has no plugin or FFI interface: its attention kernels are looked up by name in a
 * Metal library and encoded inline by Engine (src/gpu.cpp:17-25). The boundary this library replaces is therefore the
 * set of per-layer attention calls Engine makes and the raw KV-plane access the prefix cache uses. Each entry point
 * below names the reference call site it stands in for (paths relative to the reference project root).
 *
 * Model geometry is fixed (config/kata_m6.h:16-32): 24 query heads, 4 KV heads (6 query heads per KV head), head_dim
 * 256, rotary dims 64 (pairs (i, i+32)), theta 1e7, RMSNorm eps 1e-6, softmax scale 1/16.
 *
 * Conventions
 *  - Every pointer named d_* is DEVICE memory owned by the caller; h_* is HOST memory. The context owns the KV cache,
 *    the scale planes and all scratch; nothing is allocated after kata_attn_create returns, except where noted.
 *  - Calls enqueue work on the caller's CUDA stream (a cudaStream_t passed as void*; NULL = the default stream) and
 *    return without synchronising, except the plane read/write and kata_attn_check calls.
 *  - Every function returns KATA_OK or an error code; nothing aborts the process (the reference prints and exit(1)s,
 *    src/engine.cpp:195). kata_attn_last_error gives a message for the last failing call on that context.
 *  - One context per GPU; a context is not re-entrant.
 *  - Batches: the reference is single-sequence. Here a context holds n_seqs independent sequences; calls take a list
 *    of sequence ids with one position each. Per-sequence semantics are exactly the batch-1 semantics.
 */
#ifndef KATA_ATTN_H
#define KATA_ATTN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KATA_HEADS 24
#define KATA_KV_HEADS 4
#define KATA_HEAD_DIM 256
#define KATA_Q_DIM 6144      /* 24 * 256: one token's query / gate / output row */
#define KATA_KV_DIM 1024     /* 4 * 256: one token's K or V row */
#define KATA_QFULL_DIM 12288 /* per head [query 256 | gate 256] */
#define KATA_MAX_BATCH 64    /* sequences per call */
#define KATA_MAX_CHUNK 1024  /* tokens per prefill call (Engine::kMaxChunk, src/engine.h:38) */
#define KATA_MAX_VERIFY 8    /* tokens per scalar decode call (Engine::kMaxVerify, src/engine.h:97) */
#define KATA_STATIC_MAX_BATCH 8 /* sequences per kata_attn_decode_static call */

enum { KATA_OK = 0, KATA_ERR_ARG = 1, KATA_ERR_RANGE = 2, KATA_ERR_MODE = 3, KATA_ERR_CUDA = 4, KATA_ERR_DEVICE_WAIT = 5, KATA_ERR_NOMEM = 6 };
enum { KATA_KV_FP16 = 0, KATA_KV_INT8 = 1, KATA_KV_INT8V = 2, KATA_KV_INT8G = 3 };   /* KATA_KV=fp16|int8|int8v (src/engine.cpp:54-59); int8v: keys fp16, values int8 (src/engine.h:71-73);
   int8g (no reference mode): int8 keys with one fp16 scale per 64 dims (4 per head row) and int8 values with one per row: the granularity the reference measured as
   closing most of the int8 quality gap (docs/reports/M11-int8-kv.en.md:52-55) but could not fold into its matrix kernels (:94-97). rint rounding only. */
enum { KATA_ROUND_RINT = 0, KATA_ROUND_HALF_AWAY = 1 };  /* rint (ties to even) is what the reference kernel does (shaders/flash.metal:170) */
enum { KATA_ACT_F32 = 0, KATA_ACT_BF16 = 1, KATA_ACT_F16 = 2 };   /* dtype of qfull / kproj / vproj / out (the reference's activations are fp32) */

typedef struct kata_attn_ctx kata_attn_ctx;

typedef struct kata_attn_config {
    int32_t device;         /* CUDA device ordinal */
    int32_t n_layers;       /* attention layers sharing this context (16 for the trunk; the MTP head is a 1-layer context) */
    int32_t n_seqs;         /* independent sequences held (reference: 1) */
    const int32_t* max_ctx; /* [n_seqs] rows reserved per layer for each sequence (Engine::maxCtx) */
    int32_t kv_mode;        /* KATA_KV_* ; fixed for the life of the context (docs/reports/M11-int8-kv.en.md:69-71) */
    int32_t quant_round;    /* KATA_ROUND_* ; int8 mode only */
    int32_t dec_chunk;      /* keys per decode split; 0 = sized from the SM count (reference: 128, KATA_DEC_CHUNK) */
    int32_t flags;          /* bit 0: use the mma.sync prefill kernel for fp16 caches too (cross-check of the tcgen05 kernel) */
} kata_attn_config;

/* Engine::load, cache part (src/engine.cpp:54-60,79): allocates, zero-filled (src/gpu.cpp:26-30), per sequence
 * K and V planes [n_layers][max_ctx][1024] (fp16, or int8 plus fp16 scale planes [n_layers][max_ctx][4]; int8v: K fp16, V int8 plus
 * its scale plane) and all scratch. */
int kata_attn_create(const kata_attn_config* cfg, kata_attn_ctx** out);
int kata_attn_destroy(kata_attn_ctx* ctx);

/* Engine::resetState, cache part (src/engine.cpp:88-95): zero the caches and scale planes. */
int kata_attn_reset(kata_attn_ctx* ctx, void* stream);

/* Engine::numericsTag, KV part (src/engine.cpp:517-521): "fp16", "fp16+kv8", "fp16+kv8v" or "fp16+kv8g"; checkpoints of different tags never mix. */
const char* kata_attn_numerics_tag(const kata_attn_ctx* ctx);
const char* kata_attn_last_error(const kata_attn_ctx* ctx);

/* Synchronises the stream and reports a device-side wait that ran out (KATA_ERR_DEVICE_WAIT) or a CUDA error.
 * Device-side waits in this library are bounded; none can spin forever. */
int kata_attn_check(kata_attn_ctx* ctx, void* stream);

/* k_attn_prep / k_attn_prep_b (shaders/attn.metal:5-37, shaders/prefill.metal:179-206; encoded at src/engine.cpp:168,
 * 274, 360, 404, 473, 608), with k_cvt_q_half (shaders/flash.metal:71) and, in the int8 modes, k_kv_quant_sym
 * (Engine::dKvQuant, src/engine.cpp:524-527) fused in (int8v: for the value rows only; the key rows are stored as fp16).
 * For sequence seq_ids[b] and token t < T at position pos0[b]+t, head slots [h0, h0+nh): slots 0..23 query heads
 * (RMSNorm, partial RoPE, gate split), 24..27 key heads (RMSNorm, RoPE, append to the K plane), 28..31 value heads
 * (append to the V plane). h0=24, nh=8 appends K/V only (src/engine.cpp:402-404).
 *   d_qfull [n][T][12288], d_kproj, d_vproj [n][T][1024]: act_dtype; d_qnorm, d_knorm: fp32 [256].
 *   d_q16   [n][T][6144] fp16, the query after norm and RoPE times 1/16 (what the matrix attention kernels read); may be NULL.
 *   d_q32   [n][T][6144] fp32, unscaled (the reference's qout; read by kata_attn_decode_scalar); may be NULL.
 *   d_gate  [n][T][6144] fp32 gate logits; may be NULL when nh covers no query head. */
int kata_attn_prep(kata_attn_ctx* ctx, int32_t layer, int32_t n, const int32_t* seq_ids, const int32_t* pos0, int32_t T,
                   const void* d_qfull, const void* d_kproj, const void* d_vproj, int32_t act_dtype,
                   const float* d_qnorm, const float* d_knorm, void* d_q16, float* d_q32, float* d_gate,
                   int32_t h0, int32_t nh, void* stream);

/* Engine::dKvQuant + k_kv_quant_sym (src/engine.cpp:524-527, shaders/flash.metal:157-178) as a stand-alone call:
 * quantise T fp16 rows d_ks, d_vs [T][1024] into rows pos0.. of one sequence's int8 planes. Bit-exact with the
 * reference arithmetic: scale = fp16(amax/127) (1.0 for an all-zero row), code = clamp(round(v * (1/float(scale)))).
 * int8v contexts quantise d_vs only (d_ks may be NULL and is ignored: the key plane holds fp16 rows). */
int kata_attn_kv_quant(kata_attn_ctx* ctx, int32_t layer, int32_t seq, const void* d_ks, const void* d_vs, int32_t T, int32_t pos0, void* stream);

/* Engine::dDecAttn (src/engine.cpp:119-127): k_dec_q_pack + k_attn_dec_split[_q8|_k16v8] + k_attn_dec_combine
 * (shaders/flash.metal:77-152). T in 1..KATA_MAX_VERIFY query tokens per sequence at positions pos_base[b]+t (1: step, 2: verify2,
 * up to 8: Engine::verifyWide, src/engine.cpp:602-622, which the reference sends through its scalar kernels); token t sees keys
 * [first_pos, pos_base[b]+t]; first_pos is 0 for the trunk and 1 for the MTP-head cache (src/engine.cpp:362).
 *   d_q16, d_gate as written by kata_attn_prep; d_out [n][T][6144] out_dtype = softmax(q k^T) v * sigmoid(gate). */
int kata_attn_decode(kata_attn_ctx* ctx, int32_t layer, int32_t n, const int32_t* seq_ids, const int32_t* pos_base, int32_t T, int32_t first_pos,
                     const void* d_q16, const float* d_gate, void* d_out, int32_t out_dtype, void* stream);

/* The scalar path: k_attn_split(_b) + k_attn_combine(_b) (shaders/attn.metal:66-117, shaders/prefill.metal:209-261;
 * KATA_SCALAR_DEC, src/engine.cpp:169-175, 365, 478, 617). fp32 query, fp16 cache only, T <= KATA_MAX_VERIFY. */
int kata_attn_decode_scalar(kata_attn_ctx* ctx, int32_t layer, int32_t n, const int32_t* seq_ids, const int32_t* pos_base, int32_t T, int32_t first_pos,
                            const float* d_q32, const float* d_gate, float* d_out, void* stream);

/* k_flash_prefill / k_flash_prefill_q8 / k_flash_prefill_k16v8 (shaders/flash.metal:10-68, 198-250; encoded at src/engine.cpp:279, 614): causal flash
 * attention of M <= KATA_MAX_CHUNK query rows per sequence at positions pos_base[b]+r over keys [0, pos_base[b]+r] of
 * the cache (this chunk's rows must already have been appended by kata_attn_prep). d_q16, d_gate, d_out: [n][M][6144], each on a 16-byte
 * boundary (the kernel moves them in 128-bit pieces). */
int kata_attn_prefill(kata_attn_ctx* ctx, int32_t layer, int32_t n, const int32_t* seq_ids, const int32_t* pos_base, int32_t M,
                      const void* d_q16, const float* d_gate, void* d_out, int32_t out_dtype, void* stream);

/* No reference counterpart (the reference is single-device). Exchange of the split-KV parts between the GPUs of one box without a library
 * collective: each rank pushes its part rows {O[256], m, l} (as kata_attn_decode_partial writes them) into every peer's exchange buffer
 * with plain 8-byte stores over NVLink (each value together with the call's number, which is its flag), waits for the peers' rows in its own buffer and merges + gates, all in one kernel
 * on the caller's stream. Set-up: every rank creates an exchange (one cudaMalloc, exported as a CUDA IPC handle of
 * KATA_PEER_HANDLE_BYTES bytes), the ranks swap handles by any host channel, and each opens the others'; inside one process
 * kata_attn_peer_open_pointers takes the buffers' device addresses instead. All ranks must issue the same sequence of exchange calls.
 * Waits are bounded (about a second, kata_attn_peer_set_wait_polls): when a peer's rows do not arrive the call's output is left
 * unwritten and kata_attn_peer_check returns KATA_ERR_DEVICE_WAIT (then see kata_attn_peer_resync). world <= 8, T in {1, 2}. */
#define KATA_PEER_HANDLE_BYTES 64
typedef struct kata_attn_peer kata_attn_peer;
int kata_attn_peer_create(int32_t device, int32_t rank, int32_t world, kata_attn_peer** out, void* handle_out /* KATA_PEER_HANDLE_BYTES, may be NULL */);
int kata_attn_peer_open(kata_attn_peer* px, const void* handles /* world x KATA_PEER_HANDLE_BYTES, in rank order; the own slot is ignored */);
int kata_attn_peer_open_pointers(kata_attn_peer* px, void* const* buffers /* [world] device addresses from kata_attn_peer_buffer */);
void* kata_attn_peer_buffer(kata_attn_peer* px);
int kata_attn_peer_set_wait_polls(kata_attn_peer* px, uint32_t polls);
/* d_part [T*24][258] fp32 (this rank's part), d_gate [T][6144] fp32, d_out [T][6144]: out = merge over ranks, normalised and gated. */
int kata_attn_peer_exchange_merge(kata_attn_peer* px, const float* d_part, int32_t T, const float* d_gate, void* d_out, int32_t out_dtype, void* stream);
/* kata_attn_decode_partial into the exchange's own part buffer followed by kata_attn_peer_exchange_merge: the whole cross-GPU decode of
 * one layer (this rank's keys [key_lo, key_hi) of sequence seq) as one call. */
int kata_attn_peer_decode(kata_attn_peer* px, kata_attn_ctx* ctx, int32_t layer, int32_t seq, int32_t pos_base, int32_t T, int32_t key_lo, int32_t key_hi,
                          const void* d_q16, const float* d_gate, void* d_out, int32_t out_dtype, void* stream);
/* The layer loop of a split-KV decode step in one call: per layer kata_attn_prep (head slots [0, 32) when `appends`, i.e. on the rank that owns the
 * sequence's tail, else the query heads only) and kata_attn_peer_decode, over [n_layers][T][...] device arrays as in kata_attn_layers_step. */
int kata_attn_peer_layers_step(kata_attn_peer* px, kata_attn_ctx* ctx, int32_t n_layers, int32_t seq, int32_t pos, int32_t T, int32_t key_lo, int32_t key_hi, int32_t appends,
                               const void* d_qfull, const void* d_kproj, const void* d_vproj, int32_t act_dtype, const float* d_qnorm, const float* d_knorm,
                               void* d_q16, float* d_gate, void* d_out, int32_t out_dtype, void* stream);
int kata_attn_peer_check(kata_attn_peer* px, void* stream);   /* synchronises the stream; KATA_ERR_DEVICE_WAIT after a wait that ran out */
/* After KATA_ERR_DEVICE_WAIT the ranks' call counters no longer agree (the stored values are matched against the call number, and the rank whose peer
 * skipped or failed a call has counted one call more), so every later exchange would time out as well. Once the ranks have agreed over their
 * host channel that none of them has an exchange in flight (streams synchronised), each calls this with the same call_number: it
 * synchronises the device, clears the local buffer and the error word and sets the counter. Alternatively destroy and recreate on all ranks. */
int kata_attn_peer_resync(kata_attn_peer* px, uint32_t call_number);
const char* kata_attn_peer_last_error(const kata_attn_peer* px);
int kata_attn_peer_destroy(kata_attn_peer* px);              /* call on every rank only after all ranks have finished their exchanges */

/* No reference counterpart. Declares that row 0 of sequence seq's planes holds absolute position first_position (default
 * 0): afterwards every call takes absolute positions and the context maps position p to row p - first_position. Used
 * when a long sequence is split by keys across GPUs and each rank stores only its slice. */
int kata_attn_set_position_offset(kata_attn_ctx* ctx, int32_t seq, int32_t first_position);

/* No reference counterpart (the reference is single-device). Sharding by KV-head group: this context computes KV heads
 * [kv_head_lo, kv_head_lo + kv_head_n) only (default: all 4). kata_attn_prep then normalises, rotates and appends only those K/V heads and
 * writes q16 / q32 / gate only for their query heads (6 per KV head: heads 6*kv .. 6*kv + 5); kata_attn_decode and kata_attn_prefill read
 * only those heads' cache columns and write only those heads' 256-wide column blocks of d_out, leaving the rest untouched. Attention needs
 * no exchange between the ranks of such a group; a consumer that wants whole rows gathers the column blocks (T * 6144 / ranks values per
 * rank). Row layout and planes are unchanged (a rank's other heads stay zero). kata_attn_decode_scalar, kata_attn_decode_partial and the
 * mma.sync prefill kernel compute all four heads and return KATA_ERR_MODE on a context that owns a subset. */
int kata_attn_set_kv_heads(kata_attn_ctx* ctx, int32_t kv_head_lo, int32_t kv_head_n);

/* Split-KV across GPUs (no reference counterpart: the reference is single-device). Each rank holds keys
 * [key_lo, key_hi) of sequence seq in ITS context at rows [0, key_hi-key_lo) (row = key - key_lo) and computes, per
 * (token, head), the unnormalised partial of k_attn_dec_split merged over its local splits:
 *   d_part [T*24][258] fp32 = { O[256], m, l }. The ranks exchange parts (e.g. an NCCL all-gather) and each calls
 * kata_attn_merge_parts, which applies k_attn_dec_combine's merge (shaders/flash.metal:147-151) over ranks and the gate. */
int kata_attn_decode_partial(kata_attn_ctx* ctx, int32_t layer, int32_t seq, int32_t pos_base, int32_t T, int32_t key_lo, int32_t key_hi,
                             const void* d_q16, float* d_part, void* stream);
int kata_attn_merge_parts(kata_attn_ctx* ctx, const float* d_parts, int32_t n_parts, int32_t T, const float* d_gate, void* d_out, int32_t out_dtype, void* stream);

/* The transform the engine applies to the attention output before the output projection: per 1024-wide block of a row,
 * y = (1/32) * H_1024 (sign (.) x), natural-order Walsh-Hadamard (k_rms_fwht mode 3 + fwht1024: shaders/ops.metal:23-50,
 * shaders/common.h:22-42; Engine::dRmsFwht(..., 6144, 3) at src/engine.cpp:176 and the batched form at :287).
 * d_x, d_out: [rows][width] fp32 (may alias), d_sign: [width] fp32 (+-1; the engine's sg6144), width a multiple of 1024.
 * The butterflies run in the reference's order (bits 0-1, 2-6, 7-9, then the 1/32), so the result is bit-identical to an
 * fp32 evaluation in that order. Needs no context. */
int kata_attn_out_fwht(const float* d_x, const float* d_sign, float* d_out, int64_t rows, int32_t width, void* stream);

/* KV planes for the prefix cache: Engine::kvPlanes / kvPlaneRow / kvPlanePtr (src/engine.h:74-81), used by
 * PrefixCache::restore and ::writeFile (src/ckpt.cpp:98, 134). Plane order and row sizes match the reference:
 * fp16 -> {K, V} rows of 2048 B; int8 -> {K, V, K scales, V scales} rows of 1024, 1024, 8, 8 B;
 * int8v -> {K, V, V scales} rows of 2048, 1024, 8 B; int8g -> {K, V, K scales, V scales} rows of 1024, 1024, 32, 8 B (K scales: [head][64-dim group]).
 * The reference reads and writes shared memory directly; here the copy is explicit and synchronous. */
int32_t kata_attn_kv_planes(const kata_attn_ctx* ctx);
size_t kata_attn_kv_plane_row_bytes(const kata_attn_ctx* ctx, int32_t plane);
int kata_attn_kv_plane_read(kata_attn_ctx* ctx, int32_t layer, int32_t seq, int32_t plane, int32_t row0, int32_t nrows, void* h_dst);
int kata_attn_kv_plane_write(kata_attn_ctx* ctx, int32_t layer, int32_t seq, int32_t plane, int32_t row0, int32_t nrows, const void* h_src);
/* Device address of row 0 of a plane (kvPlanePtr, src/engine.h:79-81; the restore at src/ckpt.cpp:98 writes rows through it).
 * The attention kernels are launched so that they may request cache rows before the kernel enqueued just before them has completed
 * (rows that kernel does not write). The library knows what its own kernels write; it cannot know what a caller's kernel writes through
 * this pointer. So: once a plane pointer has been handed out, no row is requested early any more (a few microseconds per long decode),
 * until the caller starts declaring its writes with kata_attn_mark_rows_written; from then on only declared rows are held back. */
void* kata_attn_kv_plane_ptr(kata_attn_ctx* ctx, int32_t layer, int32_t seq, int32_t plane);
/* No reference counterpart (the reference's restore writes shared memory from the host, between forwards). Declares that device work
 * the caller has enqueued on the stream since the last library call writes rows at positions >= pos_lo of sequence seq (-1: of every
 * sequence) through plane pointers: the next library call on that stream reads none of these rows before that work has completed.
 * Several declarations before the next call add up. A caller that uses plane pointers for writing and calls this even once promises to
 * declare every such write (before the call that follows it on the stream). */
int kata_attn_mark_rows_written(kata_attn_ctx* ctx, int32_t seq, int32_t pos_lo);

/* No counterpart in the reference. kata_attn_decode for callers that cannot allocate device memory and therefore have no
 * context: engines that give all device memory to their own pools at start-up (a library cudaMalloc then fails), and
 * loops that forbid cudaMalloc/cudaFree because they synchronise the device. Allocates nothing: the caller owns the fp16
 * K and V rows (d_k_rows, d_v_rows: [total_rows][1024], 16-byte aligned; sequence i's position p is row seq_row0[i] + p)
 * and the split-KV scratch is a fixed array of about 2.2 MB inside the library image, held by every GPU that loads the
 * library until the process exits. Same semantics and outputs as kata_attn_decode (fp16 cache). Limits: n <=
 * KATA_STATIC_MAX_BATCH (more: KATA_ERR_RANGE), T in {1,2}, at most 148 CTAs. The first call on a device does that
 * device's set-up and must be made outside stream capture. All calls on a device share the scratch: calls that overlap
 * on the GPU race on it and must be serialised by the caller, the first call included (two host threads making a device's first call
 * at the same time also race on the set-up). A bounded device wait that runs out is not reported by this call (it only enqueues work):
 * kata_attn_decode_static_check tells. */
int kata_attn_decode_static(const void* d_k_rows, const void* d_v_rows, int64_t total_rows, int32_t n, const int64_t* seq_row0, const int32_t* pos_base,
                            int32_t T, int32_t first_pos, const void* d_q16, const float* d_gate, void* d_out, int32_t out_dtype, void* stream);

/* No counterpart in the reference. Synchronises the stream and returns KATA_ERR_DEVICE_WAIT if a bounded device-side wait ran out in the
 * last kata_attn_decode_static call on the current device (its output is then invalid), else KATA_OK. Allocates nothing. */
int kata_attn_decode_static_check(void* stream);

/* Number of kernels this library has launched on this context since creation (for accounting in benchmarks). */
uint64_t kata_attn_launch_count(const kata_attn_ctx* ctx);

/* No reference counterpart (the reference cuts a sequence into fixed chunks of 128 keys, src/engine.cpp:120-121). How a decode launch over n sequences
 * with kend[b] - first_row keys each would be shared out: the key tiles (tile_keys = 16 for fp16 keys, 32 for int8 keys) of all (sequence, KV head)
 * segments form one list, sequence after sequence and KV head after KV head, ntiles[b] tiles per segment; CTA c works on tiles [first_tile[c],
 * first_tile[c + 1]). cps > 0: segments of equal length got cps CTAs of their own each. merge_in_kernel: 1 when no segment is cut between more than 8
 * CTAs (the last contributor merges), else the combine grid runs; max_contrib: the CTAs of the most-cut segment. dec_chunk > 0 asks for ranges of that
 * many keys (the reference's split size) instead of one range per SM. Host code only, no GPU needed. Returns the number of CTAs (first_tile takes one
 * entry more), -1 for arguments out of range (first_tile_cap too small included). */
int kata_attn_decode_plan(int32_t n, const int32_t* kend, int32_t first_row, int32_t kvh_n, int32_t tile_keys, int32_t sm_count, int32_t dec_chunk, int32_t max_items,
                          int32_t* ntiles, int32_t* first_tile, int32_t first_tile_cap, int32_t* cps, int32_t* merge_in_kernel, int32_t* max_contrib);

/* No reference counterpart (the reference computes one sequence on one queue). How a tcgen05 prefill launch of n sequences at positions pos[]
 * and M rows each would be shared out over pairs_avail CTA pairs (one per two SMs; at most 74 are used) by a context that computes KV heads
 * [kvh_lo, kvh_lo + kvh_n): host code only, no GPU needed. Work items are (sequence, KV head, query tile of 128 rows, head pair of the KV head) in the
 * order: order[] (the batch's sequences, shortest first), KV head, query tile last to first, head pair. Pair p computes `*rounds` whole items
 * (round k: item n_pairs * k + p, pairs counted backwards in odd rounds) and then the key tiles from (item0[p], tile0[p]) up to, not including,
 * (item0[p + 1], tile0[p + 1]) of the items that follow the rounds (numbered from 0; a key tile is 128 keys). Returns the number of pairs, or -1
 * for arguments out of range. item0, tile0: 75 entries; order: n entries; tiles_scratch: 96 * n * kvh_n / 4 entries at least (one per item). */
int kata_attn_prefill_plan(int32_t M, int32_t n, const int32_t* pos, int32_t kvh_lo, int32_t kvh_n, int32_t pairs_avail, int32_t* tiles_scratch,
                           int32_t* rounds, int32_t* item0, int32_t* tile0, uint8_t* order);

/* No reference counterpart: the reference's buffers are shared between CPU and GPU (MTL::ResourceStorageModeShared, src/gpu.cpp:26-30), so
 * Engine::step / verify2 / verifyWide (src/engine.cpp:161-178, 469-483, 602-622) hand attention the very rows the CPU sees. A caller on a
 * discrete GPU whose projections and output rows live in (pinned) host memory runs a whole step through this routine instead: for each of
 * n_layers layers the projections are copied up, kata_attn_prep (all 32 head slots) and kata_attn_decode (T <= KATA_MAX_VERIFY tokens per
 * sequence, fp32 rows out) run, and the rows are copied down; two copy streams and doubled device rows keep the copies of the neighbouring
 * layers under the layer that computes. Everything is enqueued behind `stream`, which is complete when the last rows are on the host.
 *   h_qfull [n_layers][n][T][12288], h_kproj, h_vproj [n_layers][n][T][1024]: act_dtype of the create call, host memory (pinned for the copies to overlap);
 *   d_qnorm, d_knorm [n_layers][256] fp32, device; h_out [n_layers][n][T][6144] fp32, host.
 * create allocates the device rows for max_n sequences of max_T tokens (on `device`, the context's) and the streams; run allocates nothing. */
/* The layer loop of Engine::step / verify2 / verifyWide (src/engine.cpp:161-178, 469-483, 602-622: prep, then decode, layer after layer) in one call
 * for rows that are on the device already: row l of every [n_layers][...] array belongs to layer l (d_qfull [n_layers][n][T][12288], d_kproj, d_vproj
 * [..][1024] act_dtype; d_qnorm, d_knorm [n_layers][256]; d_q16, d_gate, d_out [n_layers][n][T][6144]). One crossing of the language boundary per token
 * instead of two per layer; the launches are the same. */
int kata_attn_layers_step(kata_attn_ctx* ctx, int32_t n_layers, int32_t n, const int32_t* seq_ids, const int32_t* pos0, int32_t T, int32_t first_pos,
                          const void* d_qfull, const void* d_kproj, const void* d_vproj, int32_t act_dtype, const float* d_qnorm, const float* d_knorm,
                          void* d_q16, float* d_gate, void* d_out, int32_t out_dtype, void* stream);

/* kata_attn_decode for layers 0..n_layers-1 over the same [n_layers][...] arrays, nothing appended: the attention kernels by themselves. */
int kata_attn_layers_decode(kata_attn_ctx* ctx, int32_t n_layers, int32_t n, const int32_t* seq_ids, const int32_t* pos_base, int32_t T, int32_t first_pos,
                            const void* d_q16, const float* d_gate, void* d_out, int32_t out_dtype, void* stream);

typedef struct kata_attn_host_step kata_attn_host_step;
int kata_attn_host_step_create(kata_attn_ctx* ctx, int32_t device, int32_t max_n, int32_t max_T, int32_t act_dtype, kata_attn_host_step** out);
int kata_attn_host_step_destroy(kata_attn_host_step* hs);
int kata_attn_host_step_run(kata_attn_host_step* hs, int32_t n_layers, int32_t n, const int32_t* seq_ids, const int32_t* pos0, int32_t T, int32_t first_pos,
                            const void* h_qfull, const void* h_kproj, const void* h_vproj, const float* d_qnorm, const float* d_knorm, float* h_out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* KATA_ATTN_H */
