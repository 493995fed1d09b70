// C entry points over kata::AttnEngine so that the engine-named call sequences are exercised by the test-suite
// (one T=1 step and one T=2 verify through the same code an Engine port would call).
#include "attn_engine.hpp"

extern "C" {
// kvInt8: 0 fp16, 1 int8, 2 int8v
void* kata_engine_create(int device, int nAttn, int maxCtx, int kvInt8) { try { return new kata::AttnEngine(device, nAttn, maxCtx, kvInt8 == 1, true, kvInt8 == 2); } catch (...) { return nullptr; } }
void kata_engine_destroy(void* e) { delete static_cast<kata::AttnEngine*>(e); }
int kata_engine_step_attn(void* e, int ai, uint32_t pos, const float* qfull, const float* k, const float* v, const float* qn, const float* kn, void* q16, float* gate, float* out, void* stream) {
    return static_cast<kata::AttnEngine*>(e)->stepAttn(ai, pos, qfull, k, v, qn, kn, q16, gate, out, stream); }
int kata_engine_verify2_attn(void* e, int ai, uint32_t pos, const float* qfull, const float* k, const float* v, const float* qn, const float* kn, void* q16, float* gate, float* out, void* stream) {
    return static_cast<kata::AttnEngine*>(e)->verify2Attn(ai, pos, qfull, k, v, qn, kn, q16, gate, out, stream); }
int kata_engine_prefill_attn(void* e, int ai, uint32_t M, uint32_t pos0, const float* qfull, const float* k, const float* v, const float* qn, const float* kn, void* q16, float* gate, float* out, void* stream) {
    return static_cast<kata::AttnEngine*>(e)->prefillAttn(ai, M, pos0, qfull, k, v, qn, kn, q16, gate, out, stream); }
int kata_engine_check(void* e, void* stream) { return static_cast<kata::AttnEngine*>(e)->check(stream); }
}
