/* C ABI of the draft model's attention: non-causal sliding-window attention of a block of tokens over a ring of K/V rows.
 *
 * Replaces, one call for one dispatch, the attention kernels of the reference's block drafter (src/draft.cpp:112-123,
 * 196-209; src/draft.h:8-11, 36):
 *   k_draft_qk      shaders/draft.metal:203-233   per-head RMSNorm(128, eps 1e-6) + RoPE (pairs (i, i+64), theta = pos * 1e7^(-i/64))
 *                                                 of the block's Q and K rows, K and V rows written to the ring as fp16
 *   k_draft_ctx_kv  shaders/draft.metal:264-281   the same K/V treatment for context rows (no query)
 *   k_draft_attn    shaders/draft.metal:235-262   query row t (position pos0 + t) attends the keys at positions
 *                                                 [pos0 + t - window + 1, pos0 + T - 1] (the whole block: not causal), fp32 softmax
 * Geometry is the reference's: 32 query heads, 8 KV heads, head_dim 128, scale 1/sqrt(128); per layer one K ring and one V ring of
 * [ring][8 * 128] fp16, position p at row p mod ring (src/draft.h:36). The block's own rows are written at p mod ring as well: the
 * reference's k_draft_qk indexes the ring with the unwrapped position (shaders/draft.metal:231-232), which only holds while
 * positions stay below the ring size.
 * Everything is allocated in kata_draft_create; the calls enqueue on the caller's stream and allocate nothing. */
#ifndef KATA_DRAFT_H
#define KATA_DRAFT_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KATA_DRAFT_HEADS 32
#define KATA_DRAFT_KV_HEADS 8
#define KATA_DRAFT_HEAD_DIM 128
#define KATA_DRAFT_Q_DIM 4096      /* 32 * 128 */
#define KATA_DRAFT_KV_DIM 1024     /* 8 * 128 */
#define KATA_DRAFT_MAX_BLOCK 16    /* query rows per attention call (Draft::kBlock = 8, src/draft.h:9) */
#define KATA_DRAFT_MAX_ROWS 64     /* rows per kata_draft_qk call (Draft::kNMax, src/draft.h:35) */

typedef struct kata_draft_ctx kata_draft_ctx;

typedef struct kata_draft_config {
    int32_t device;
    int32_t n_layers;   /* Draft::kLayers = 5 */
    int32_t ring;       /* Draft::kRing = 4096: a power of two, >= window + KATA_DRAFT_MAX_BLOCK */
    int32_t window;     /* Draft::kWindow = 2048 */
} kata_draft_config;

/* Status codes are those of kata_attn.h (0 = ok, 1 = bad argument, 2 = out of range, 4 = CUDA error, 6 = out of memory). */
int kata_draft_create(const kata_draft_config* cfg, kata_draft_ctx** out);   /* rings zero-filled (src/gpu.cpp:26-30) */
int kata_draft_destroy(kata_draft_ctx* ctx);
int kata_draft_reset(kata_draft_ctx* ctx, void* stream);                      /* zero the rings */
const char* kata_draft_last_error(const kata_draft_ctx* ctx);

/* k_draft_qk, and with d_qin == NULL k_draft_ctx_kv: rows t < T at positions pos0 + t.
 *   d_qin [T][4096], d_kin, d_vin [T][1024] fp32; d_qnorm, d_knorm fp32 [128]; d_qout [T][4096] fp32 (normed, rotated, unscaled).
 *   K (normed, rotated) and V rows go to the layer's rings as fp16. T in 1..KATA_DRAFT_MAX_ROWS. */
int kata_draft_qk(kata_draft_ctx* ctx, int32_t layer, const float* d_qin, const float* d_kin, const float* d_vin,
                  const float* d_qnorm, const float* d_knorm, float* d_qout, int32_t pos0, int32_t T, void* stream);

/* k_draft_attn: d_q [T][4096] fp32 as kata_draft_qk wrote it, d_out [T][4096] fp32. T in 1..KATA_DRAFT_MAX_BLOCK. Every position in
 * [max(0, pos0 - window + 1), pos0 + T) must have been written to the ring. */
int kata_draft_attn(kata_draft_ctx* ctx, int32_t layer, const float* d_q, float* d_out, int32_t pos0, int32_t T, void* stream);

/* Device address of row 0 of a layer's K (value = 0) or V (value = 1) ring: [ring][1024] fp16. */
void* kata_draft_ring_ptr(kata_draft_ctx* ctx, int32_t layer, int32_t value);
/* Synchronous copies of ring rows [row0, row0 + nrows) (2048 bytes each) to and from host memory. */
int kata_draft_ring_read(kata_draft_ctx* ctx, int32_t layer, int32_t value, int32_t row0, int32_t nrows, void* h_dst);
int kata_draft_ring_write(kata_draft_ctx* ctx, int32_t layer, int32_t value, int32_t row0, int32_t nrows, const void* h_src);
uint64_t kata_draft_launch_count(const kata_draft_ctx* ctx);

#ifdef __cplusplus
}
#endif
#endif
