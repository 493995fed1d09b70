/* kata_engine.h - C entry points over kata::AttnEngine (kata_b200/csrc/attn_engine.hpp), the C++ class that carries the attention
 * branches of the reference's Engine under the Engine's own method names. A C++ caller includes the class directly; these
 * functions exist so that the same call sequences can be driven from C and from the test-suite. Each one names the Engine
 * method whose attention branch it is (src/engine.cpp of the reference). All pointers are device pointers; kv: 0 fp16, 1 int8,
 * 2 int8v. Status codes are those of kata_attn.h. */
#ifndef KATA_ENGINE_H
#define KATA_ENGINE_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif
void* kata_engine_create(int device, int nAttn, int maxCtx, int kv);   /* Engine::load, cache part (src/engine.cpp:54-60,79); NULL on failure */
void kata_engine_destroy(void* e);
/* Engine::step (src/engine.cpp:161-178): k_attn_prep (+dKvQuant) -> dDecAttn(T=1) */
int kata_engine_step_attn(void* e, int ai, uint32_t pos, const float* qfull, const float* k, const float* v, const float* qn, const float* kn, void* q16, float* gate, float* out, void* stream);
/* Engine::verify2 (src/engine.cpp:469-483): k_attn_prep_b(32, 2) -> dDecAttn(T=2) */
int kata_engine_verify2_attn(void* e, int ai, uint32_t pos, const float* qfull, const float* k, const float* v, const float* qn, const float* kn, void* q16, float* gate, float* out, void* stream);
/* Engine::verifyWide (src/engine.cpp:602-622): k_attn_prep_b(32, T <= 8) -> decode of T tokens */
int kata_engine_verify_wide_attn(void* e, int ai, uint32_t T, uint32_t pos, const float* qfull, const float* k, const float* v, const float* qn, const float* kn, void* q16, float* gate, float* out, void* stream);
/* Engine::prefill (src/engine.cpp:267-289): k_attn_prep_b(32, M) -> k_cvt_q_half -> k_flash_prefill[_q8] */
int kata_engine_prefill_attn(void* e, int ai, uint32_t M, uint32_t pos0, const float* qfull, const float* k, const float* v, const float* qn, const float* kn, void* q16, float* gate, float* out, void* stream);
/* Engine::mtpRows (src/engine.cpp:358-368): R <= 2 rows on the MTP head's 1-layer fp16 cache, first valid key at position 1 */
int kata_engine_mtp_rows_attn(void* e, uint32_t R, uint32_t pos0, const float* qfull, const float* k, const float* v, const float* qn, const float* kn, void* q16, float* gate, float* out, void* stream);
/* Engine::encMtpKv (src/engine.cpp:402-404): K/V head slots only (h0 = 24, 8 slots) into the MTP cache */
int kata_engine_enc_mtp_kv(void* e, uint32_t R, uint32_t p0, const float* k, const float* v, const float* kn, void* stream);
/* Engine::dKvQuant (src/engine.cpp:524-527): T fp16 scratch rows into layer ai at pos0 */
int kata_engine_kv_quant(void* e, uint32_t T, uint32_t pos0, uint32_t ai, const void* ks, const void* vs, void* stream);
/* Engine::dRmsFwht(..., 6144, 3) (src/engine.cpp:176, 287) */
int kata_engine_attn_out_fwht(void* e, const float* attn_out, const float* sign, float* xp, uint32_t rows, void* stream);
/* Engine::resetState (src/engine.cpp:88-95), numericsTag (:517-521), kvPlanes / kvPlaneRow / kvPlanePtr / mtpKvPtr (src/engine.h:74-81) */
int kata_engine_reset_state(void* e, void* stream);
const char* kata_engine_numerics_tag(void* e);
uint32_t kata_engine_kv_planes(void* e);
size_t kata_engine_kv_plane_row(void* e, uint32_t plane);
void* kata_engine_kv_plane_ptr(void* e, uint32_t layer, uint32_t plane);
void* kata_engine_mtp_kv_ptr(void* e, int value);
int kata_engine_kv_plane_read(void* e, uint32_t layer, uint32_t plane, uint32_t n, void* h_dst);
int kata_engine_kv_plane_write(void* e, uint32_t layer, uint32_t plane, uint32_t n, const void* h_src);
int kata_engine_mtp_plane_read(void* e, int value, uint32_t n, void* h_dst);
int kata_engine_check(void* e, void* stream);
#ifdef __cplusplus
}
#endif
#endif
