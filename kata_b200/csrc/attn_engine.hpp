// C++ mirror of the attention part of the reference's Engine (src/engine.h, src/engine.cpp), for host code that wants
// the engine's own method names over the C ABI of include/kata_attn.h. Each method is the per-layer attention branch of
// the Engine method it is named after: the Metal dispatches of that branch, replaced by the calls that stand in for them.
// Header-only; all pointers are device pointers unless named h_*.
#pragma once
#include <cstdint>
#include <stdexcept>
#include <string>

#include "../../include/kata_attn.h"

namespace kata {

class AttnEngine {
public:
    // Engine::load, cache part (src/engine.cpp:54-60,79): trunk caches for nAttn layers plus the MTP head's 1-layer fp16 cache.
    // kvInt8K / kvInt8V as the reference derives them from KATA_KV = fp16 | int8 | int8v (src/engine.cpp:54): int8v keeps the keys in fp16.
    AttnEngine(int device, int nAttn, int maxCtx, bool kvInt8K, bool hasMtp = true, bool kvInt8V = false) : maxCtx_(maxCtx), kvInt8_(kvInt8K || kvInt8V) {
        int32_t rows = maxCtx;
        kata_attn_config cfg{device, nAttn, 1, &rows, kvInt8K ? KATA_KV_INT8 : kvInt8V ? KATA_KV_INT8V : KATA_KV_FP16, KATA_ROUND_RINT, 0, 0};
        if (kata_attn_create(&cfg, &attn_) != KATA_OK) throw std::runtime_error("kata_attn_create failed");
        if (hasMtp) { kata_attn_config m = cfg; m.n_layers = 1; m.kv_mode = KATA_KV_FP16; if (kata_attn_create(&m, &mtp_) != KATA_OK) { kata_attn_destroy(attn_); throw std::runtime_error("kata_attn_create (mtp) failed"); } }
    }
    ~AttnEngine() { if (attn_) kata_attn_destroy(attn_); if (mtp_) kata_attn_destroy(mtp_); }
    AttnEngine(const AttnEngine&) = delete; AttnEngine& operator=(const AttnEngine&) = delete;

    // Engine::step, attention branch (src/engine.cpp:161-178): k_attn_prep (+dKvQuant) then dDecAttn(T=1, firstPos=0).
    int stepAttn(int ai, uint32_t pos, const float* bufQfull, const float* bufK, const float* bufV, const float* qNorm, const float* kNorm,
                 void* q16, float* bufGate, float* bufAttnO, void* stream) { return decodeRows(attn_, ai, pos, 1, 0, bufQfull, bufK, bufV, qNorm, kNorm, q16, bufGate, bufAttnO, stream); }
    // Engine::verify2, attention branch (src/engine.cpp:469-483): k_attn_prep_b (32, 2) then dDecAttn(T=2).
    int verify2Attn(int ai, uint32_t pos, const float* pQfull, const float* pK, const float* pV, const float* qNorm, const float* kNorm,
                    void* q16, float* pGate, float* pAttnO, void* stream) { return decodeRows(attn_, ai, pos, 2, 0, pQfull, pK, pV, qNorm, kNorm, q16, pGate, pAttnO, stream); }
    // Engine::verifyWide, attention branch (src/engine.cpp:602-622): k_attn_prep_b (32, T <= kMaxVerify = 8) then the decode of T tokens.
    int verifyWideAttn(int ai, uint32_t T, uint32_t pos, const float* pQfull, const float* pK, const float* pV, const float* qNorm, const float* kNorm,
                       void* q16, float* pGate, float* pAttnO, void* stream) { return decodeRows(attn_, ai, pos, (int)T, 0, pQfull, pK, pV, qNorm, kNorm, q16, pGate, pAttnO, stream); }
    // Engine::dRmsFwht(e, bufAttnO, nullptr, sg6144, 0, bufXp, 6144, 3) (src/engine.cpp:176, 287): the transform between attention and the output projection
    int attnOutFwht(const float* bufAttnO, const float* sg6144, float* bufXp, uint32_t rows, void* stream) { return kata_attn_out_fwht(bufAttnO, sg6144, bufXp, rows, KATA_Q_DIM, stream); }
    // Engine::mtpRows, attention part (src/engine.cpp:358-368): R <= 2 rows on the MTP head's cache, first valid key at position 1.
    int mtpRowsAttn(uint32_t R, uint32_t pos0, const float* mQfull, const float* mKp, const float* mVp, const float* qNorm, const float* kNorm,
                    void* q16, float* mGate, float* mAttnO, void* stream) { return decodeRows(mtp_, 0, pos0, (int)R, 1, mQfull, mKp, mVp, qNorm, kNorm, q16, mGate, mAttnO, stream); }
    // Engine::prefill, attention branch (src/engine.cpp:267-289): k_attn_prep_b (32, M), k_cvt_q_half, k_flash_prefill[_q8].
    int prefillAttn(int ai, uint32_t M, uint32_t pos0, const float* pQfull, const float* pK, const float* pV, const float* qNorm, const float* kNorm,
                    void* pQh, float* pGate, float* pAttnO, void* stream) {
        const int32_t seq = 0, p = (int32_t)pos0;
        int rc = kata_attn_prep(attn_, ai, 1, &seq, &p, (int32_t)M, pQfull, pK, pV, KATA_ACT_F32, qNorm, kNorm, pQh, nullptr, pGate, 0, 32, stream);
        return rc ? rc : kata_attn_prefill(attn_, ai, 1, &seq, &p, (int32_t)M, pQh, pGate, pAttnO, KATA_ACT_F32, stream);
    }
    // Engine::encMtpKv, cache part (src/engine.cpp:402-404): K/V head slots only (h0 = 24, 8 slots) into the MTP cache.
    int encMtpKv(uint32_t R, uint32_t p0, const float* pK, const float* pV, const float* kNorm, void* stream) {
        const int32_t seq = 0, p = (int32_t)p0;
        return kata_attn_prep(mtp_, 0, 1, &seq, &p, (int32_t)R, nullptr, pK, pV, KATA_ACT_F32, nullptr, kNorm, nullptr, nullptr, nullptr, 24, 8, stream);
    }
    // Engine::dKvQuant (src/engine.cpp:524-527): T fp16 scratch rows into layer ai at pos0 (int8 mode).
    int dKvQuant(uint32_t T, uint32_t pos0, uint32_t ai, const void* kvScrK, const void* kvScrV, void* stream) { return kata_attn_kv_quant(attn_, (int32_t)ai, 0, kvScrK, kvScrV, (int32_t)T, (int32_t)pos0, stream); }
    // Engine::resetState, cache part (src/engine.cpp:88-95)
    int resetState(void* stream) { int rc = kata_attn_reset(attn_, stream); return rc || !mtp_ ? rc : kata_attn_reset(mtp_, stream); }
    // Engine::numericsTag, KV part (src/engine.cpp:517-521)
    std::string numericsTag() const { return kata_attn_numerics_tag(attn_); }
    // Engine::kvPlanes / kvPlaneRow / kvPlanePtr (src/engine.h:74-81); the pointer is a DEVICE address here
    uint32_t kvPlanes() const { return (uint32_t)kata_attn_kv_planes(attn_); }
    size_t kvPlaneRow(uint32_t plane) const { return kata_attn_kv_plane_row_bytes(attn_, (int32_t)plane); }
    uint8_t* kvPlanePtr(uint32_t attnLayer, uint32_t plane) const { return (uint8_t*)kata_attn_kv_plane_ptr(attn_, (int32_t)attnLayer, 0, (int32_t)plane); }
    uint8_t* mtpKvPtr(bool value) const { return mtp_ ? (uint8_t*)kata_attn_kv_plane_ptr(mtp_, 0, 0, value ? 1 : 0) : nullptr; }
    // what PrefixCache::restore / writeFile do per (layer, plane) (src/ckpt.cpp:98,134), through a host bounce buffer
    int kvPlaneRead(uint32_t a, uint32_t plane, uint32_t n, void* h_dst) { return kata_attn_kv_plane_read(attn_, (int32_t)a, 0, (int32_t)plane, 0, (int32_t)n, h_dst); }
    int kvPlaneWrite(uint32_t a, uint32_t plane, uint32_t n, const void* h_src) { return kata_attn_kv_plane_write(attn_, (int32_t)a, 0, (int32_t)plane, 0, (int32_t)n, h_src); }
    int check(void* stream) { return kata_attn_check(attn_, stream); }
    const char* lastError() const { return kata_attn_last_error(attn_); }
    kata_attn_ctx* trunk() const { return attn_; }
    kata_attn_ctx* mtp() const { return mtp_; }
    uint32_t maxCtx() const { return (uint32_t)maxCtx_; }
    bool kvInt8() const { return kvInt8_; }

private:
    int decodeRows(kata_attn_ctx* c, int layer, uint32_t pos, int T, int firstPos, const float* qfull, const float* k, const float* v, const float* qNorm, const float* kNorm,
                   void* q16, float* gate, float* out, void* stream) {
        if (!c) return KATA_ERR_ARG;
        const int32_t seq = 0, p = (int32_t)pos;
        int rc = kata_attn_prep(c, layer, 1, &seq, &p, T, qfull, k, v, KATA_ACT_F32, qNorm, kNorm, q16, nullptr, gate, 0, 32, stream);
        return rc ? rc : kata_attn_decode(c, layer, 1, &seq, &p, T, firstPos, q16, gate, out, KATA_ACT_F32, stream);
    }
    kata_attn_ctx* attn_ = nullptr; kata_attn_ctx* mtp_ = nullptr; int maxCtx_; bool kvInt8_;
};

}  // namespace kata
