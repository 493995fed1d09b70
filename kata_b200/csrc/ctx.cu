// Context object and the C ABI of libkata_attn (declared in include/kata_attn.h): cache arenas in the reference's
// plane layout, argument checking, the per-call batch descriptor, and the KV-plane copies the prefix cache uses.
// Mirrors the cache part of Engine::load / resetState / numericsTag and kvPlanes / kvPlaneRow / kvPlanePtr
// (src/engine.cpp:54-60, 79, 88-95, 517-521; src/engine.h:74-81).
#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <new>

#include "kata_internal.cuh"
#include "peer_exchange.cuh"

namespace kata {
size_t scalar_scratch_floats_pm();
size_t scalar_scratch_floats_acc();
int decode_max_slots(int sm_count);
cudaError_t configure_decode(int kv_mode);
cudaError_t configure_decode_scalar();
cudaError_t launch_out_fwht(const float* x, const float* sign, float* out, int64_t rows, int width, cudaStream_t s);
cudaError_t configure_prefill(int kv_mode);
size_t prefill_part_o_bytes(); size_t prefill_part_ml_bytes(); size_t prefill_part_flag_bytes();
cudaError_t launch_decode_mma_ex(Ctx& c, const Batch& b, int T, int first_row, int key_off, const int32_t* kend_override, const __half* q16, const float* gate, void* out, int out_dtype,
                                 float* part_out, cudaStream_t s, int tok_stride = 0, int tok0 = 0, const PeerSink* sink = nullptr, bool* sink_used = nullptr);
int decode_partial_impl(kata_attn_ctx* h, int32_t layer, int32_t seq, int32_t pos_base, int32_t T, int32_t key_lo, int32_t key_hi, const void* d_q16, float* d_part,
                        const PeerSink* sink, const float* d_gate, void* d_out, int32_t out_dtype, bool* sink_used, void* stream);
}  // namespace kata

struct kata_attn_ctx { kata::Ctx c; };

using kata::Ctx;

namespace {

int fail(Ctx& c, int code, const char* fmt, ...) {
    char buf[512]; va_list ap; va_start(ap, fmt); vsnprintf(buf, sizeof buf, fmt, ap); va_end(ap);
    c.err = buf; return code;
}
int cuda_fail(Ctx& c, cudaError_t e, const char* what) { return fail(c, KATA_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e)); }

struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int dev) { cudaGetDevice(&prev); if (prev != dev) cudaSetDevice(dev); else prev = -1; }
    ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
};

// validates (layer, sequence ids, positions) and fills the descriptor; rows [pos, pos+span) must exist for every sequence
int make_batch(Ctx& c, int layer, int n, const int32_t* seq_ids, const int32_t* pos, int span, kata::Batch& b, bool touches_cache = true) {
    if (layer < 0 || layer >= c.cfg.n_layers) return fail(c, KATA_ERR_RANGE, "layer %d outside [0,%d)", layer, c.cfg.n_layers);
    if (n < 1 || n > KATA_MAX_BATCH || !seq_ids || !pos) return fail(c, KATA_ERR_ARG, "batch of %d sequences (1..%d) needs seq_ids and positions", n, KATA_MAX_BATCH);
    b.n = n;
    for (int i = 0; i < n; i++) {
        const int s = seq_ids[i];
        if (s < 0 || s >= c.cfg.n_seqs) return fail(c, KATA_ERR_RANGE, "sequence id %d outside [0,%d)", s, c.cfg.n_seqs);
        const int64_t local = (int64_t)pos[i] - c.pos_off[s];
        if (pos[i] < 0 || (touches_cache && (local < 0 || local + span > c.max_ctx[s]))) return fail(c, KATA_ERR_RANGE, "positions [%d,%d) of sequence %d fall outside its %d rows starting at position %d", pos[i], pos[i] + span, s, c.max_ctx[s], c.pos_off[s]);
        b.seq[i] = s; b.pos[i] = pos[i]; b.row_base[i] = c.row_of(layer, s) - c.pos_off[s];
    }
    return KATA_OK;
}

struct PlaneRef { uint8_t* base; size_t row_bytes; };
bool plane_ref(Ctx& c, int plane, PlaneRef& r) {
    // kvPlanePtr (src/engine.h:79-81): plane 2 is the K scales when the keys are int8, else the V scales
    if (plane == 0) { r = {(uint8_t*)c.k_arena, (size_t)kata::kKVD * c.elt_k}; return true; }
    if (plane == 1) { r = {(uint8_t*)c.v_arena, (size_t)kata::kKVD * c.elt_v}; return true; }
    if (c.k8() && plane == 2) { r = {(uint8_t*)c.ksc, (size_t)2 * c.ksc_per_row()}; return true; }
    if (c.v8() && plane == (c.k8() ? 3 : 2)) { r = {(uint8_t*)c.vsc, 8}; return true; }
    return false;
}

}  // namespace

extern "C" {

int kata_attn_create(const kata_attn_config* cfg, kata_attn_ctx** out) {
    if (!cfg || !out) return KATA_ERR_ARG;
    *out = nullptr;
    if (cfg->n_layers < 1 || cfg->n_seqs < 1 || !cfg->max_ctx || (cfg->kv_mode != KATA_KV_FP16 && cfg->kv_mode != KATA_KV_INT8 && cfg->kv_mode != KATA_KV_INT8V && cfg->kv_mode != KATA_KV_INT8G) ||
        (cfg->kv_mode == KATA_KV_INT8G && (cfg->quant_round != KATA_ROUND_RINT || (cfg->flags & 1))) ||
        (cfg->quant_round != KATA_ROUND_RINT && cfg->quant_round != KATA_ROUND_HALF_AWAY) || cfg->dec_chunk < 0) return KATA_ERR_ARG;
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || cfg->device < 0 || cfg->device >= ndev) return KATA_ERR_CUDA;
    kata_attn_ctx* h = new (std::nothrow) kata_attn_ctx();
    if (!h) return KATA_ERR_NOMEM;
    Ctx& c = h->c; c.cfg = *cfg; c.cfg.max_ctx = nullptr;
    DeviceGuard guard(cfg->device);
    cudaDeviceGetAttribute(&c.sm_count, cudaDevAttrMultiProcessorCount, cfg->device);
    c.elt_k = (cfg->kv_mode == KATA_KV_INT8 || cfg->kv_mode == KATA_KV_INT8G) ? 1 : 2; c.elt_v = cfg->kv_mode == KATA_KV_FP16 ? 2 : 1;
    c.tag = cfg->kv_mode == KATA_KV_INT8 ? "fp16+kv8" : cfg->kv_mode == KATA_KV_INT8V ? "fp16+kv8v" : cfg->kv_mode == KATA_KV_INT8G ? "fp16+kv8g" : "fp16";   // Engine::numericsTag, src/engine.cpp:517-521
    int64_t rows = 0;
    for (int s = 0; s < cfg->n_seqs; s++) {
        if (cfg->max_ctx[s] < 1) { delete h; return KATA_ERR_ARG; }
        c.max_ctx.push_back(cfg->max_ctx[s]); c.pos_off.push_back(0); c.append_lo.push_back(INT32_MAX); c.seq_row0.push_back(rows); rows += (int64_t)cfg->n_layers * cfg->max_ctx[s];
    }
    c.total_rows = rows;
    c.max_items = kata::decode_max_slots(c.sm_count * 8);
    bool ok = cudaMalloc(&c.k_arena, (size_t)rows * kata::kKVD * c.elt_k) == cudaSuccess && cudaMalloc(&c.v_arena, (size_t)rows * kata::kKVD * c.elt_v) == cudaSuccess;
    if (ok && c.k8()) ok = cudaMalloc((void**)&c.ksc, (size_t)rows * 2 * c.ksc_per_row()) == cudaSuccess;
    if (ok && c.v8()) ok = cudaMalloc((void**)&c.vsc, (size_t)rows * 8) == cudaSuccess;
    ok = ok && cudaMalloc((void**)&c.part_o, (size_t)c.max_items * 12 * kata::kD * 4) == cudaSuccess && cudaMalloc((void**)&c.part_ml, (size_t)c.max_items * 32 * 4) == cudaSuccess &&
         cudaMalloc((void**)&c.counters, 4 * KATA_MAX_BATCH * 4) == cudaSuccess && cudaMalloc((void**)&c.d_err, 4) == cudaSuccess;
    if (ok && cfg->kv_mode == KATA_KV_FP16)
        ok = cudaMalloc((void**)&c.sc_pm, kata::scalar_scratch_floats_pm() * 4) == cudaSuccess && cudaMalloc((void**)&c.sc_pl, kata::scalar_scratch_floats_pm() * 4) == cudaSuccess &&
             cudaMalloc((void**)&c.sc_pacc, kata::scalar_scratch_floats_acc() * 4) == cudaSuccess;
    ok = ok && cudaMalloc((void**)&c.pf_part_o, kata::prefill_part_o_bytes()) == cudaSuccess && cudaMalloc((void**)&c.pf_part_ml, kata::prefill_part_ml_bytes()) == cudaSuccess &&
         cudaMalloc((void**)&c.pf_part_flag, kata::prefill_part_flag_bytes()) == cudaSuccess && cudaMemset(c.pf_part_flag, 0, kata::prefill_part_flag_bytes()) == cudaSuccess;
    int64_t stage_rows = 0;
    if (ok && c.v8()) {   // staging arena of the tcgen05 prefill: one layer of every sequence, the int8 planes' codes expanded to fp16
        for (int sq = 0; sq < cfg->n_seqs; sq++) { c.stage_row0.push_back(stage_rows); stage_rows += cfg->max_ctx[sq]; }
        const size_t sb = (size_t)stage_rows * kata::kKVD * 2;
        ok = cudaMalloc((void**)&c.v16_stage, sb) == cudaSuccess && cudaMemset(c.v16_stage, 0, sb) == cudaSuccess;
        if (ok && c.k8()) ok = cudaMalloc((void**)&c.k16_stage, sb) == cudaSuccess && cudaMemset(c.k16_stage, 0, sb) == cudaSuccess;
    }
    if (!ok) { cudaGetLastError(); kata_attn_destroy(h); return KATA_ERR_NOMEM; }
    {   // decode: rank-4 tile views (a 128-byte column block = 64 fp16 or 128 int8 elements); tcgen05 prefill (fp16): the half tiles of a CTA pair
        const int tile_rows = c.k8() ? 32 : 16;   // keys per decode tile: 32 when both planes are int8
        if (!kata::make_tile_tmap(&c.tm_k_tile, c.k_arena, c.elt_k, rows, tile_rows, 256 * c.elt_k / 128) || !kata::make_tile_tmap(&c.tm_v_tile, c.v_arena, c.elt_v, rows, tile_rows, 256 * c.elt_v / 128) ||
            (!c.k8() && !kata::make_tile_tmap(&c.tm_k64h, c.k_arena, 2, rows, 64, 4)) || (!c.v8() && !kata::make_tile_tmap(&c.tm_v128h, c.v_arena, 2, rows, 128, 2)) ||
            (c.k8() && !kata::make_tile_tmap(&c.tm_k64h_stage, c.k16_stage, 2, stage_rows, 64, 4)) || (c.v8() && !kata::make_tile_tmap(&c.tm_v128h_stage, c.v16_stage, 2, stage_rows, 128, 2))) { kata_attn_destroy(h); return KATA_ERR_CUDA; }
    }
    if (kata::configure_decode(cfg->kv_mode) != cudaSuccess || kata::configure_prefill(cfg->kv_mode) != cudaSuccess || (cfg->kv_mode == KATA_KV_FP16 && kata::configure_decode_scalar() != cudaSuccess)) { cudaGetLastError(); kata_attn_destroy(h); return KATA_ERR_CUDA; }
    cudaMemset(c.counters, 0, 4 * KATA_MAX_BATCH * 4); cudaMemset(c.d_err, 0, 4);
    float invf[32]; for (int i = 0; i < 32; i++) invf[i] = powf(10000000.0f, -(float)i / 32.0f);   // shaders/attn.metal:26
    kata::set_inv_freq(invf);
    if (kata_attn_reset(h, nullptr) != KATA_OK || cudaDeviceSynchronize() != cudaSuccess) { kata_attn_destroy(h); return KATA_ERR_CUDA; }
    *out = h;
    return KATA_OK;
}

int kata_attn_destroy(kata_attn_ctx* h) {
    if (!h) return KATA_ERR_ARG;
    Ctx& c = h->c; DeviceGuard guard(c.cfg.device);
    void* ptrs[] = {c.k_arena, c.v_arena, c.ksc, c.vsc, c.part_o, c.part_ml, c.counters, c.d_err, c.sc_pm, c.sc_pl, c.sc_pacc, c.k16_stage, c.v16_stage, c.pf_part_o, c.pf_part_ml, c.pf_part_flag};
    for (void* p : ptrs) if (p) cudaFree(p);
    delete h;
    return KATA_OK;
}

int kata_attn_reset(kata_attn_ctx* h, void* stream) {
    if (!h) return KATA_ERR_ARG;
    Ctx& c = h->c; DeviceGuard guard(c.cfg.device); cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e = cudaMemsetAsync(c.k_arena, 0, (size_t)c.total_rows * kata::kKVD * c.elt_k, s); if (e == cudaSuccess) e = cudaMemsetAsync(c.v_arena, 0, (size_t)c.total_rows * kata::kKVD * c.elt_v, s);
    if (e == cudaSuccess && c.ksc) e = cudaMemsetAsync(c.ksc, 0, (size_t)c.total_rows * 2 * c.ksc_per_row(), s);
    if (e == cudaSuccess && c.vsc) e = cudaMemsetAsync(c.vsc, 0, (size_t)c.total_rows * 8, s);
    return e == cudaSuccess ? KATA_OK : cuda_fail(c, e, "reset");
}

const char* kata_attn_numerics_tag(const kata_attn_ctx* h) { return h ? h->c.tag.c_str() : ""; }
const char* kata_attn_last_error(const kata_attn_ctx* h) { return h ? h->c.err.c_str() : "null context"; }
uint64_t kata_attn_launch_count(const kata_attn_ctx* h) { return h ? h->c.launches : 0; }

int kata_attn_out_fwht(const float* d_x, const float* d_sign, float* d_out, int64_t rows, int32_t width, void* stream) {
    if (!d_x || !d_sign || !d_out) return KATA_ERR_ARG;
    if (rows < 0 || width < 1024 || width % 1024 != 0) return KATA_ERR_RANGE;
    if (rows == 0) return KATA_OK;
    return kata::launch_out_fwht(d_x, d_sign, d_out, rows, width, (cudaStream_t)stream) == cudaSuccess ? KATA_OK : KATA_ERR_CUDA;
}

int kata_attn_check(kata_attn_ctx* h, void* stream) {
    if (!h) return KATA_ERR_ARG;
    Ctx& c = h->c; DeviceGuard guard(c.cfg.device);
    cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream); if (e != cudaSuccess) return cuda_fail(c, e, "synchronize");
    int32_t flag = 0; e = cudaMemcpy(&flag, c.d_err, 4, cudaMemcpyDeviceToHost); if (e != cudaSuccess) return cuda_fail(c, e, "read error word");
    if (flag) { cudaMemset(c.d_err, 0, 4); cudaMemset(c.pf_part_flag, 0, kata::prefill_part_flag_bytes()); return fail(c, KATA_ERR_DEVICE_WAIT, "a bounded device-side wait ran out (code %d); results of that call are invalid", flag); }
    return KATA_OK;
}

int kata_attn_prep(kata_attn_ctx* h, int32_t layer, int32_t n, const int32_t* seq_ids, const int32_t* pos0, int32_t T,
                   const void* d_qfull, const void* d_kproj, const void* d_vproj, int32_t act_dtype,
                   const float* d_qnorm, const float* d_knorm, void* d_q16, float* d_q32, float* d_gate, int32_t h0, int32_t nh, void* stream) {
    if (!h) return KATA_ERR_ARG;
    Ctx& c = h->c;
    if (T < 1 || T > KATA_MAX_CHUNK) return fail(c, KATA_ERR_RANGE, "prep of %d tokens (1..%d)", T, KATA_MAX_CHUNK);
    if (h0 < 0 || nh < 1 || h0 + nh > 32) return fail(c, KATA_ERR_ARG, "head slots [%d,%d) outside [0,32)", h0, h0 + nh);
    if (act_dtype != KATA_ACT_F32 && act_dtype != KATA_ACT_BF16 && act_dtype != KATA_ACT_F16) return fail(c, KATA_ERR_ARG, "unknown activation dtype %d", act_dtype);
    const bool hasQ = h0 < 24, hasK = h0 < 28 && h0 + nh > 24, hasV = h0 + nh > 28;
    if ((hasQ && (!d_qfull || !d_qnorm)) || (hasK && (!d_kproj || !d_knorm)) || (hasV && !d_vproj)) return fail(c, KATA_ERR_ARG, "a projection or norm weight needed by head slots [%d,%d) is null", h0, h0 + nh);
    kata::Batch b{}; if (int rc = make_batch(c, layer, n, seq_ids, pos0, T, b, /*touches_cache=*/h0 + nh > 24)) return rc;
    DeviceGuard guard(c.cfg.device);
    cudaError_t e = kata::launch_prep(c, b, T, d_qfull, d_kproj, d_vproj, act_dtype, d_qnorm, d_knorm, (__half*)d_q16, d_q32, d_gate, h0, nh, (cudaStream_t)stream);
    if (e == cudaSuccess && h0 + nh > 24) { c.wrote_no_rows(); for (int i = 0; i < n; i++) c.wrote_rows_from(b.seq[i], b.pos[i]); }
    else if (e == cudaSuccess) c.wrote_no_rows();
    return e == cudaSuccess ? KATA_OK : cuda_fail(c, e, "prep launch");
}

int kata_attn_kv_quant(kata_attn_ctx* h, int32_t layer, int32_t seq, const void* d_ks, const void* d_vs, int32_t T, int32_t pos0, void* stream) {
    if (!h) return KATA_ERR_ARG;
    Ctx& c = h->c;
    if (!c.v8()) return fail(c, KATA_ERR_MODE, "kv_quant needs an int8 or int8v context (this one is %s)", c.tag.c_str());
    if ((c.k8() && !d_ks) || !d_vs || T < 1 || T > KATA_MAX_CHUNK) return fail(c, KATA_ERR_ARG, "kv_quant of %d rows (1..%d) needs the scratch rows of every int8 plane", T, KATA_MAX_CHUNK);
    kata::Batch b{}; if (int rc = make_batch(c, layer, 1, &seq, &pos0, T, b)) return rc;
    DeviceGuard guard(c.cfg.device);
    cudaError_t e = kata::launch_kv_quant(c, b.row_base[0] + pos0, (const __half*)d_ks, (const __half*)d_vs, T, (cudaStream_t)stream);
    if (e == cudaSuccess) { c.wrote_no_rows(); c.wrote_rows_from(seq, pos0); }
    return e == cudaSuccess ? KATA_OK : cuda_fail(c, e, "kv_quant launch");
}

int kata_attn_decode(kata_attn_ctx* h, int32_t layer, int32_t n, const int32_t* seq_ids, const int32_t* pos_base, int32_t T, int32_t first_pos,
                     const void* d_q16, const float* d_gate, void* d_out, int32_t out_dtype, void* stream) {
    if (!h) return KATA_ERR_ARG;
    Ctx& c = h->c;
    if (T < 1 || T > KATA_MAX_VERIFY) return fail(c, KATA_ERR_RANGE, "decode takes 1..%d query tokens, not %d", KATA_MAX_VERIFY, T);
    if (!d_q16 || !d_gate || !d_out) return fail(c, KATA_ERR_ARG, "decode needs q16, gate and out");
    if (out_dtype != KATA_ACT_F32 && out_dtype != KATA_ACT_BF16 && out_dtype != KATA_ACT_F16) return fail(c, KATA_ERR_ARG, "unknown output dtype %d", out_dtype);
    kata::Batch b{}; if (int rc = make_batch(c, layer, n, seq_ids, pos_base, T, b)) return rc;
    for (int i = 0; i < n; i++) if (first_pos < 0 || first_pos > pos_base[i]) return fail(c, KATA_ERR_RANGE, "first_pos %d outside [0, pos_base=%d]", first_pos, pos_base[i]);
    DeviceGuard guard(c.cfg.device);
    // The kernel takes the 6 heads of a KV head x 2 tokens as its 16-row block. A wide verify (T up to 8, Engine::verifyWide,
    // src/engine.cpp:602-622) runs as launches of two tokens each: the rows of all T tokens are in the cache already and token t
    // sees keys <= pos_base + t, so the passes are independent; the keys are read once per pass (wide verifies are short-context).
    for (int t0 = 0; t0 < T; t0 += 2) {
        kata::Batch bt = b;
        for (int i = 0; i < n; i++) bt.pos[i] = b.pos[i] + t0;
        cudaError_t e = kata::launch_decode_mma_ex(c, bt, std::min(2, T - t0), first_pos, 0, nullptr, (const __half*)d_q16, d_gate, d_out, out_dtype, nullptr, (cudaStream_t)stream, T, t0);
        if (e != cudaSuccess) return cuda_fail(c, e, "decode launch");
    }
    return KATA_OK;
}

int kata_attn_decode_scalar(kata_attn_ctx* h, int32_t layer, int32_t n, const int32_t* seq_ids, const int32_t* pos_base, int32_t T, int32_t first_pos,
                            const float* d_q32, const float* d_gate, float* d_out, void* stream) {
    if (!h) return KATA_ERR_ARG;
    Ctx& c = h->c;
    if (c.kvh_n != KATA_KV_HEADS) return fail(c, KATA_ERR_MODE, "the scalar path computes all four KV heads (this context owns %d)", c.kvh_n);
    if (c.cfg.kv_mode != KATA_KV_FP16) return fail(c, KATA_ERR_MODE, "the scalar path reads an fp16 cache only (the reference disables it for int8, src/engine.cpp:169)");
    if (T < 1 || T > KATA_MAX_VERIFY) return fail(c, KATA_ERR_RANGE, "scalar decode takes 1..%d query tokens, not %d", KATA_MAX_VERIFY, T);
    if (!d_q32 || !d_gate || !d_out) return fail(c, KATA_ERR_ARG, "scalar decode needs q32, gate and out");
    kata::Batch b{}; if (int rc = make_batch(c, layer, n, seq_ids, pos_base, T, b)) return rc;
    for (int i = 0; i < n; i++) if (first_pos < 0 || first_pos > pos_base[i]) return fail(c, KATA_ERR_RANGE, "first_pos %d outside [0, pos_base=%d]", first_pos, pos_base[i]);
    DeviceGuard guard(c.cfg.device);
    cudaError_t e = kata::launch_decode_scalar(c, b, T, first_pos, d_q32, d_gate, d_out, (cudaStream_t)stream);
    c.wrote_no_rows();
    return e == cudaSuccess ? KATA_OK : cuda_fail(c, e, "scalar decode launch");
}

int kata_attn_prefill(kata_attn_ctx* h, int32_t layer, int32_t n, const int32_t* seq_ids, const int32_t* pos_base, int32_t M,
                      const void* d_q16, const float* d_gate, void* d_out, int32_t out_dtype, void* stream) {
    if (!h) return KATA_ERR_ARG;
    Ctx& c = h->c;
    if (M < 1 || M > KATA_MAX_CHUNK) return fail(c, KATA_ERR_RANGE, "prefill chunk of %d rows (1..%d)", M, KATA_MAX_CHUNK);
    if (!d_q16 || !d_gate || !d_out) return fail(c, KATA_ERR_ARG, "prefill needs q16, gate and out");
    if (((uintptr_t)d_q16 | (uintptr_t)d_gate | (uintptr_t)d_out) & 15) return fail(c, KATA_ERR_ARG, "prefill needs q16, gate and out on 16-byte boundaries");
    if (out_dtype != KATA_ACT_F32 && out_dtype != KATA_ACT_BF16 && out_dtype != KATA_ACT_F16) return fail(c, KATA_ERR_ARG, "unknown output dtype %d", out_dtype);
    if (c.kvh_n != KATA_KV_HEADS && (c.cfg.flags & 1)) return fail(c, KATA_ERR_MODE, "the mma.sync prefill kernel computes all four KV heads (this context owns %d)", c.kvh_n);
    kata::Batch b{}; if (int rc = make_batch(c, layer, n, seq_ids, pos_base, M, b)) return rc;
    DeviceGuard guard(c.cfg.device);
    cudaError_t e = kata::launch_prefill(c, b, M, (const __half*)d_q16, d_gate, d_out, out_dtype, (cudaStream_t)stream);
    c.wrote_no_rows();
    return e == cudaSuccess ? KATA_OK : cuda_fail(c, e, "prefill launch");
}

int kata_attn_decode_partial(kata_attn_ctx* h, int32_t layer, int32_t seq, int32_t pos_base, int32_t T, int32_t key_lo, int32_t key_hi,
                             const void* d_q16, float* d_part, void* stream) {
    return kata::decode_partial_impl(h, layer, seq, pos_base, T, key_lo, key_hi, d_q16, d_part, nullptr, nullptr, nullptr, KATA_ACT_F32, nullptr, stream);
}

int kata_attn_merge_parts(kata_attn_ctx* h, const float* d_parts, int32_t n_parts, int32_t T, const float* d_gate, void* d_out, int32_t out_dtype, void* stream) {
    if (!h) return KATA_ERR_ARG;
    Ctx& c = h->c;
    if (!d_parts || !d_gate || !d_out || n_parts < 1 || T < 1 || T > 2 || out_dtype < KATA_ACT_F32 || out_dtype > KATA_ACT_F16) return fail(c, KATA_ERR_ARG, "merge_parts: %d parts, T=%d", n_parts, T);
    DeviceGuard guard(c.cfg.device);
    cudaError_t e = kata::launch_merge_parts(c, d_parts, n_parts, T, d_gate, d_out, out_dtype, (cudaStream_t)stream);
    c.wrote_no_rows();
    return e == cudaSuccess ? KATA_OK : cuda_fail(c, e, "merge_parts launch");
}

int kata_attn_set_kv_heads(kata_attn_ctx* h, int32_t kv_head_lo, int32_t kv_head_n) {
    if (!h) return KATA_ERR_ARG;
    Ctx& c = h->c;
    if (kv_head_lo < 0 || kv_head_n < 1 || kv_head_lo + kv_head_n > KATA_KV_HEADS) return fail(c, KATA_ERR_RANGE, "KV heads [%d,%d) outside [0,%d)", kv_head_lo, kv_head_lo + kv_head_n, KATA_KV_HEADS);
    c.kvh_lo = kv_head_lo; c.kvh_n = kv_head_n; c.pf_plan_M = -1;   // the cached prefill plan was made for another head range
    return KATA_OK;
}

int kata_attn_set_position_offset(kata_attn_ctx* h, int32_t seq, int32_t first_position) {
    if (!h) return KATA_ERR_ARG;
    Ctx& c = h->c;
    if (seq < 0 || seq >= c.cfg.n_seqs || first_position < 0) return fail(c, KATA_ERR_RANGE, "sequence %d / first position %d", seq, first_position);
    c.pos_off[seq] = first_position;
    return KATA_OK;
}

int32_t kata_attn_kv_planes(const kata_attn_ctx* h) { return h ? 2 + (h->c.k8() ? 1 : 0) + (h->c.v8() ? 1 : 0) : 0; }   // Engine::kvPlanes, src/engine.h:74
size_t kata_attn_kv_plane_row_bytes(const kata_attn_ctx* h, int32_t plane) {
    if (!h) return 0;
    PlaneRef r; return plane_ref(const_cast<Ctx&>(h->c), plane, r) ? r.row_bytes : 0;
}
void* kata_attn_kv_plane_ptr(kata_attn_ctx* h, int32_t layer, int32_t seq, int32_t plane) {
    if (!h) return nullptr;
    Ctx& c = h->c; PlaneRef r;
    if (!plane_ref(c, plane, r) || layer < 0 || layer >= c.cfg.n_layers || seq < 0 || seq >= c.cfg.n_seqs) return nullptr;
    c.ext_ptr = true;   // from now on caller kernels may write cache rows: see kata_attn_mark_rows_written
    return r.base + (size_t)c.row_of(layer, seq) * r.row_bytes;
}
int kata_attn_mark_rows_written(kata_attn_ctx* h, int32_t seq, int32_t pos_lo) {
    if (!h) return KATA_ERR_ARG;
    Ctx& c = h->c;
    if (seq < -1 || seq >= c.cfg.n_seqs || pos_lo < 0) return fail(c, KATA_ERR_RANGE, "sequence %d (or -1 for all) / first written position %d", seq, pos_lo);
    c.ext_declared = true;
    if (!c.prev_mark) c.wrote_no_rows();   // several marks before the next call add up
    for (int s = 0; s < c.cfg.n_seqs; s++) if (seq < 0 || s == seq) c.wrote_rows_from(s, pos_lo);
    c.prev_mark = true;
    return KATA_OK;
}
static int plane_copy(kata_attn_ctx* h, int32_t layer, int32_t seq, int32_t plane, int32_t row0, int32_t nrows, void* host, bool to_host) {
    if (!h) return KATA_ERR_ARG;
    Ctx& c = h->c; PlaneRef r;
    if (!plane_ref(c, plane, r)) return fail(c, KATA_ERR_ARG, "plane %d does not exist in mode %s", plane, c.tag.c_str());
    if (layer < 0 || layer >= c.cfg.n_layers || seq < 0 || seq >= c.cfg.n_seqs) return fail(c, KATA_ERR_RANGE, "layer %d / sequence %d out of range", layer, seq);
    if (row0 < 0 || nrows < 0 || (int64_t)row0 + nrows > c.max_ctx[seq] || (!host && nrows)) return fail(c, KATA_ERR_RANGE, "rows [%d,%d) exceed max_ctx %d", row0, row0 + nrows, c.max_ctx[seq]);
    if (!nrows) return KATA_OK;
    DeviceGuard guard(c.cfg.device);
    uint8_t* dev = r.base + ((size_t)c.row_of(layer, seq) + row0) * r.row_bytes; const size_t bytes = (size_t)nrows * r.row_bytes;
    cudaError_t e = cudaDeviceSynchronize();   // rows may still be in flight on any stream (the reference's writer reads live rows after a completed forward)
    if (e == cudaSuccess) e = to_host ? cudaMemcpy(host, dev, bytes, cudaMemcpyDeviceToHost) : cudaMemcpy(dev, host, bytes, cudaMemcpyHostToDevice);
    return e == cudaSuccess ? KATA_OK : cuda_fail(c, e, "plane copy");
}
int kata_attn_kv_plane_read(kata_attn_ctx* h, int32_t layer, int32_t seq, int32_t plane, int32_t row0, int32_t nrows, void* h_dst) { return plane_copy(h, layer, seq, plane, row0, nrows, h_dst, true); }
int kata_attn_kv_plane_write(kata_attn_ctx* h, int32_t layer, int32_t seq, int32_t plane, int32_t row0, int32_t nrows, const void* h_src) { return plane_copy(h, layer, seq, plane, row0, nrows, const_cast<void*>(h_src), false); }

}  // extern "C"

// kata_attn_decode_partial, optionally feeding a cross-GPU exchange: with a sink (and the gate and output rows it needs) the launch may hand this
// rank's rows to the exchange itself (sink_used = true); otherwise they are in d_part as usual.
int kata::decode_partial_impl(kata_attn_ctx* h, int32_t layer, int32_t seq, int32_t pos_base, int32_t T, int32_t key_lo, int32_t key_hi, const void* d_q16, float* d_part,
                              const kata::PeerSink* sink, const float* d_gate, void* d_out, int32_t out_dtype, bool* sink_used, void* stream) {
    if (sink_used) *sink_used = false;
    if (!h) return KATA_ERR_ARG;
    Ctx& c = h->c;
    if (T < 1 || T > 2) return fail(c, KATA_ERR_RANGE, "decode takes 1 or 2 query tokens, not %d", T);
    if (!d_q16 || !d_part) return fail(c, KATA_ERR_ARG, "decode_partial needs q16 and part");
    if (c.kvh_n != KATA_KV_HEADS) return fail(c, KATA_ERR_MODE, "decode_partial computes all four KV heads (this context owns %d)", c.kvh_n);
    if (key_lo < 0 || key_hi < key_lo || pos_base < 0) return fail(c, KATA_ERR_RANGE, "key range [%d,%d) / pos_base %d", key_lo, key_hi, pos_base);
    const int32_t local_rows = std::max(0, std::min(pos_base + T, key_hi) - key_lo);   // rows [0, local_rows) of this context hold keys key_lo..
    if (layer < 0 || layer >= c.cfg.n_layers || seq < 0 || seq >= c.cfg.n_seqs) return fail(c, KATA_ERR_RANGE, "layer %d / sequence %d out of range", layer, seq);
    if (local_rows > c.max_ctx[seq]) return fail(c, KATA_ERR_RANGE, "%d local rows exceed max_ctx %d", local_rows, c.max_ctx[seq]);
    kata::Batch b{}; b.n = 1; b.seq[0] = seq; b.pos[0] = pos_base; b.row_base[0] = c.row_of(layer, seq);
    DeviceGuard guard(c.cfg.device);
    cudaError_t e = kata::launch_decode_mma_ex(c, b, T, 0, key_lo, &local_rows, (const __half*)d_q16, sink ? d_gate : nullptr, sink ? d_out : nullptr, sink ? out_dtype : KATA_ACT_F32, d_part, (cudaStream_t)stream, 0, 0, sink, sink_used);
    return e == cudaSuccess ? KATA_OK : cuda_fail(c, e, "decode_partial launch");
}

