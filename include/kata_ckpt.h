/* kata_ckpt.h - KV segments of the engine's prefix-cache checkpoint files ("BNSCKPT1", version 2).
 * Counterpart of the KV part of PrefixCache::restore / writeFile in the reference (src/ckpt.cpp:16-34, 84-107, 127-140):
 * same header, same 4 KiB-aligned segment offsets, same per-layer plane order, so the KV segments of a file written by
 * either side are readable by the other. The GDN, conv, hidden-state and logits segments belong to the engine; files
 * written here leave them as holes of the right size. */
#ifndef KATA_CKPT_H
#define KATA_CKPT_H
#include <stdint.h>
#include "kata_attn.h"
#ifdef __cplusplus
extern "C" {
#endif
/* layoutFor (src/ckpt.cpp:30-34): out8 = {tokensOff, gdnOff, convOff, kvOff, mtpOff, hOff, logitsOff, total} */
void kata_ckpt_layout(uint32_t n, uint64_t gdn_bytes, uint64_t conv_bytes, uint32_t n_attn, uint32_t kv_row, int has_mtp, uint64_t* out8);
/* prefixHashes (src/ckpt.cpp:36-39) of tokens[0, n): out2 = {hash0, hash1} */
void kata_ckpt_prefix_hash(const int32_t* tokens, uint32_t n, uint64_t* out2);
/* The acceptance checks of PrefixCache::restore (src/ckpt.cpp:91-96), no cache involved: KATA_OK and *n_out = stored token
 * count, or KATA_ERR_RANGE for a truncated, foreign or mismatching file. */
int kata_ckpt_probe(const char* path, const int32_t* tokens, uint32_t n_tokens, uint64_t model_fp, const char* tag, uint32_t n_attn, uint32_t kv_row,
                    uint64_t gdn_bytes, uint64_t conv_bytes, int want_mtp, uint32_t* n_out);
/* PrefixCache::writeFile, KV part (src/ckpt.cpp:127-140): header + tokens + KV planes of layers [0, n_attn) + MTP K/V (mtp may be NULL).
 * The file is left as "<path>.tmp": its header, hashes and size are already valid, so under its final name the reference's restore
 * (src/ckpt.cpp:91-101) would accept it although the engine's segments are still holes. The engine writes its GDN, conv, hidden-state and
 * logits segments into "<path>.tmp" at the offsets kata_ckpt_layout gives and then calls kata_ckpt_publish(path), which renames the
 * file to <path> (the rename of src/ckpt.cpp:138). */
int kata_ckpt_write_kv(kata_attn_ctx* trunk, kata_attn_ctx* mtp, int32_t seq, const char* path, const int32_t* tokens, uint32_t n, uint64_t model_fp, uint32_t n_attn,
                       uint64_t gdn_bytes, uint64_t conv_bytes, int32_t last_tok);
int kata_ckpt_publish(const char* path);
/* PrefixCache::restore, KV part (src/ckpt.cpp:84-107): checks, then plane-wise restore; on failure the caches are reset. */
int kata_ckpt_read_kv(kata_attn_ctx* trunk, kata_attn_ctx* mtp, int32_t seq, const char* path, const int32_t* tokens, uint32_t n_tokens, uint64_t model_fp, uint32_t n_attn,
                      uint64_t gdn_bytes, uint64_t conv_bytes, uint32_t* n_out);
#ifdef __cplusplus
}
#endif
#endif
