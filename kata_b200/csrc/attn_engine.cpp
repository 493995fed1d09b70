// C entry points over kata::AttnEngine (declared in include/kata_engine.h) so that the engine-named call sequences can be driven
// from C and are exercised by the test-suite through the same code an Engine port would call.
#include "attn_engine.hpp"
#include "../../include/kata_engine.h"

#define ENG(e) static_cast<kata::AttnEngine*>(e)

extern "C" {
// kvInt8: 0 fp16, 1 int8, 2 int8v
void* kata_engine_create(int device, int nAttn, int maxCtx, int kvInt8) { try { return new kata::AttnEngine(device, nAttn, maxCtx, kvInt8 == 1, true, kvInt8 == 2); } catch (...) { return nullptr; } }
void kata_engine_destroy(void* e) { delete ENG(e); }
int kata_engine_step_attn(void* e, int ai, uint32_t pos, const float* qfull, const float* k, const float* v, const float* qn, const float* kn, void* q16, float* gate, float* out, void* stream) {
    return !e ? KATA_ERR_ARG : ENG(e)->stepAttn(ai, pos, qfull, k, v, qn, kn, q16, gate, out, stream); }
int kata_engine_verify2_attn(void* e, int ai, uint32_t pos, const float* qfull, const float* k, const float* v, const float* qn, const float* kn, void* q16, float* gate, float* out, void* stream) {
    return !e ? KATA_ERR_ARG : ENG(e)->verify2Attn(ai, pos, qfull, k, v, qn, kn, q16, gate, out, stream); }
int kata_engine_prefill_attn(void* e, int ai, uint32_t M, uint32_t pos0, const float* qfull, const float* k, const float* v, const float* qn, const float* kn, void* q16, float* gate, float* out, void* stream) {
    return !e ? KATA_ERR_ARG : ENG(e)->prefillAttn(ai, M, pos0, qfull, k, v, qn, kn, q16, gate, out, stream); }
int kata_engine_verify_wide_attn(void* e, int ai, uint32_t T, uint32_t pos, const float* qfull, const float* k, const float* v, const float* qn, const float* kn, void* q16, float* gate, float* out, void* stream) {
    return e ? ENG(e)->verifyWideAttn(ai, T, pos, qfull, k, v, qn, kn, q16, gate, out, stream) : KATA_ERR_ARG; }
int kata_engine_mtp_rows_attn(void* e, uint32_t R, uint32_t pos0, const float* qfull, const float* k, const float* v, const float* qn, const float* kn, void* q16, float* gate, float* out, void* stream) {
    return e ? ENG(e)->mtpRowsAttn(R, pos0, qfull, k, v, qn, kn, q16, gate, out, stream) : KATA_ERR_ARG; }
int kata_engine_enc_mtp_kv(void* e, uint32_t R, uint32_t p0, const float* k, const float* v, const float* kn, void* stream) { return e ? ENG(e)->encMtpKv(R, p0, k, v, kn, stream) : KATA_ERR_ARG; }
int kata_engine_kv_quant(void* e, uint32_t T, uint32_t pos0, uint32_t ai, const void* ks, const void* vs, void* stream) { return e ? ENG(e)->dKvQuant(T, pos0, ai, ks, vs, stream) : KATA_ERR_ARG; }
int kata_engine_attn_out_fwht(void* e, const float* attn_out, const float* sign, float* xp, uint32_t rows, void* stream) { return e ? ENG(e)->attnOutFwht(attn_out, sign, xp, rows, stream) : KATA_ERR_ARG; }
int kata_engine_reset_state(void* e, void* stream) { return e ? ENG(e)->resetState(stream) : KATA_ERR_ARG; }
const char* kata_engine_numerics_tag(void* e) { return e ? kata_attn_numerics_tag(ENG(e)->trunk()) : ""; }
uint32_t kata_engine_kv_planes(void* e) { return e ? ENG(e)->kvPlanes() : 0; }
size_t kata_engine_kv_plane_row(void* e, uint32_t plane) { return e ? ENG(e)->kvPlaneRow(plane) : 0; }
void* kata_engine_kv_plane_ptr(void* e, uint32_t layer, uint32_t plane) { return e ? ENG(e)->kvPlanePtr(layer, plane) : nullptr; }
void* kata_engine_mtp_kv_ptr(void* e, int value) { return e ? ENG(e)->mtpKvPtr(value != 0) : nullptr; }
int kata_engine_kv_plane_read(void* e, uint32_t layer, uint32_t plane, uint32_t n, void* h_dst) { return e ? ENG(e)->kvPlaneRead(layer, plane, n, h_dst) : KATA_ERR_ARG; }
int kata_engine_kv_plane_write(void* e, uint32_t layer, uint32_t plane, uint32_t n, const void* h_src) { return e ? ENG(e)->kvPlaneWrite(layer, plane, n, h_src) : KATA_ERR_ARG; }
int kata_engine_mtp_plane_read(void* e, int value, uint32_t n, void* h_dst) { return e && ENG(e)->mtp() ? kata_attn_kv_plane_read(ENG(e)->mtp(), 0, 0, value ? 1 : 0, 0, (int32_t)n, h_dst) : KATA_ERR_ARG; }
int kata_engine_check(void* e, void* stream) {
    if (!e) return KATA_ERR_ARG;
    const int rc = ENG(e)->check(stream);
    return rc || !ENG(e)->mtp() ? rc : kata_attn_check(ENG(e)->mtp(), stream); }
}
