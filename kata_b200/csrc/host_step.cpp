// A decode (or verify) step of all layers for a caller whose activations live in host memory: per layer the projections go up, the rows are
// appended and attended (kata_attn_prep + kata_attn_decode, the two calls of Engine::step / verify2 / verifyWide, src/engine.cpp:161-178,
// 469-483, 602-622), and the output rows come down. The reference has no such routine because it needs none: its buffers are shared between
// the CPU and the GPU (MTL::ResourceStorageModeShared, src/gpu.cpp:26-30), so the matmuls around attention read and write the very rows
// attention works on. On a discrete GPU a caller that keeps those rows on the host pays two copies per layer; this routine hides them
// behind the attention kernels: two copy streams, the device-side input and output rows doubled, so that layer l+1's projections go up and
// layer l-1's rows come down while layer l computes. Everything is enqueued; the caller's stream is complete when the last rows are on the host.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <new>

#include "../../include/kata_attn.h"

struct kata_attn_host_step {
    kata_attn_ctx* ctx = nullptr;
    int device = 0, max_n = 0, max_T = 0, act = KATA_ACT_F32;
    size_t esz = 4;
    void* d_q[2] = {nullptr, nullptr}; void* d_k[2] = {nullptr, nullptr}; void* d_v[2] = {nullptr, nullptr};   // projections of the layer in flight, doubled
    void* d_q16 = nullptr; float* d_gate = nullptr; float* d_out[2] = {nullptr, nullptr};
    cudaStream_t s_in = nullptr, s_out = nullptr;
    cudaEvent_t ev_in[2] = {nullptr, nullptr}, ev_done[2] = {nullptr, nullptr}, ev_down[2] = {nullptr, nullptr}, ev_start = nullptr;
};

namespace {
struct DevGuard { int prev = 0; explicit DevGuard(int d) { cudaGetDevice(&prev); cudaSetDevice(d); } ~DevGuard() { cudaSetDevice(prev); } };
}

extern "C" int kata_attn_host_step_destroy(kata_attn_host_step* h) {
    if (!h) return KATA_ERR_ARG;
    DevGuard g(h->device);
    for (int i = 0; i < 2; i++) {
        cudaFree(h->d_q[i]); cudaFree(h->d_k[i]); cudaFree(h->d_v[i]); cudaFree(h->d_out[i]);
        if (h->ev_in[i]) cudaEventDestroy(h->ev_in[i]);
        if (h->ev_done[i]) cudaEventDestroy(h->ev_done[i]);
        if (h->ev_down[i]) cudaEventDestroy(h->ev_down[i]);
    }
    cudaFree(h->d_q16); cudaFree(h->d_gate);
    if (h->ev_start) cudaEventDestroy(h->ev_start);
    if (h->s_in) cudaStreamDestroy(h->s_in);
    if (h->s_out) cudaStreamDestroy(h->s_out);
    delete h;
    return KATA_OK;
}

extern "C" int kata_attn_host_step_create(kata_attn_ctx* ctx, int32_t device, int32_t max_n, int32_t max_T, int32_t act_dtype, kata_attn_host_step** out) {
    if (!ctx || !out || max_n < 1 || max_n > KATA_MAX_BATCH || max_T < 1 || max_T > KATA_MAX_VERIFY) return KATA_ERR_ARG;
    if (act_dtype != KATA_ACT_F32 && act_dtype != KATA_ACT_BF16 && act_dtype != KATA_ACT_F16) return KATA_ERR_ARG;
    kata_attn_host_step* h = new (std::nothrow) kata_attn_host_step();
    if (!h) return KATA_ERR_NOMEM;
    h->ctx = ctx; h->device = device; h->max_n = max_n; h->max_T = max_T; h->act = act_dtype; h->esz = act_dtype == KATA_ACT_F32 ? 4 : 2;
    DevGuard g(device);
    const size_t rows = (size_t)max_n * max_T;
    bool ok = true;
    for (int i = 0; i < 2 && ok; i++)
        ok = cudaMalloc(&h->d_q[i], rows * 12288 * h->esz) == cudaSuccess && cudaMalloc(&h->d_k[i], rows * 1024 * h->esz) == cudaSuccess && cudaMalloc(&h->d_v[i], rows * 1024 * h->esz) == cudaSuccess &&
             cudaMalloc((void**)&h->d_out[i], rows * 6144 * 4) == cudaSuccess && cudaEventCreateWithFlags(&h->ev_in[i], cudaEventDisableTiming) == cudaSuccess &&
             cudaEventCreateWithFlags(&h->ev_done[i], cudaEventDisableTiming) == cudaSuccess && cudaEventCreateWithFlags(&h->ev_down[i], cudaEventDisableTiming) == cudaSuccess;
    ok = ok && cudaMalloc(&h->d_q16, rows * 6144 * 2) == cudaSuccess && cudaMalloc((void**)&h->d_gate, rows * 6144 * 4) == cudaSuccess &&
         cudaStreamCreateWithFlags(&h->s_in, cudaStreamNonBlocking) == cudaSuccess && cudaStreamCreateWithFlags(&h->s_out, cudaStreamNonBlocking) == cudaSuccess &&
         cudaEventCreateWithFlags(&h->ev_start, cudaEventDisableTiming) == cudaSuccess;
    if (!ok) { cudaGetLastError(); kata_attn_host_step_destroy(h); return KATA_ERR_NOMEM; }
    *out = h;
    return KATA_OK;
}

extern "C" int kata_attn_host_step_run(kata_attn_host_step* h, int32_t n_layers, int32_t n, const int32_t* seq_ids, const int32_t* pos0, int32_t T, int32_t first_pos,
                                       const void* h_qfull, const void* h_kproj, const void* h_vproj, const float* d_qnorm, const float* d_knorm, float* h_out, void* stream) {
    if (!h || !seq_ids || !pos0 || !h_qfull || !h_kproj || !h_vproj || !d_qnorm || !d_knorm || !h_out) return KATA_ERR_ARG;
    if (n < 1 || n > h->max_n || T < 1 || T > h->max_T || n_layers < 1) return KATA_ERR_RANGE;
    DevGuard g(h->device);
    cudaStream_t s = (cudaStream_t)stream;
    const size_t rows = (size_t)n * T, qb = rows * 12288 * h->esz, kb = rows * 1024 * h->esz, ob = rows * 6144 * 4;
    // the copy streams start behind whatever the caller has enqueued so far (its earlier steps read the same device rows)
    if (cudaEventRecord(h->ev_start, s) != cudaSuccess || cudaStreamWaitEvent(h->s_in, h->ev_start, 0) != cudaSuccess || cudaStreamWaitEvent(h->s_out, h->ev_start, 0) != cudaSuccess) return KATA_ERR_CUDA;
    for (int l = 0; l < n_layers; l++) {
        const int b = l & 1;
        if (l >= 2 && cudaStreamWaitEvent(h->s_in, h->ev_done[b], 0) != cudaSuccess) return KATA_ERR_CUDA;   // layer l - 2 has read these input rows
        if (cudaMemcpyAsync(h->d_q[b], (const char*)h_qfull + (size_t)l * qb, qb, cudaMemcpyHostToDevice, h->s_in) != cudaSuccess ||
            cudaMemcpyAsync(h->d_k[b], (const char*)h_kproj + (size_t)l * kb, kb, cudaMemcpyHostToDevice, h->s_in) != cudaSuccess ||
            cudaMemcpyAsync(h->d_v[b], (const char*)h_vproj + (size_t)l * kb, kb, cudaMemcpyHostToDevice, h->s_in) != cudaSuccess ||
            cudaEventRecord(h->ev_in[b], h->s_in) != cudaSuccess || cudaStreamWaitEvent(s, h->ev_in[b], 0) != cudaSuccess) return KATA_ERR_CUDA;
        if (l >= 2 && cudaStreamWaitEvent(s, h->ev_down[b], 0) != cudaSuccess) return KATA_ERR_CUDA;       // layer l - 2's output rows have left these device rows
        int rc = kata_attn_prep(h->ctx, l, n, seq_ids, pos0, T, h->d_q[b], h->d_k[b], h->d_v[b], h->act, d_qnorm + (size_t)l * 256, d_knorm + (size_t)l * 256, h->d_q16, nullptr, h->d_gate, 0, 32, s);
        if (rc == KATA_OK) rc = kata_attn_decode(h->ctx, l, n, seq_ids, pos0, T, first_pos, h->d_q16, h->d_gate, h->d_out[b], KATA_ACT_F32, s);
        if (rc != KATA_OK) return rc;
        if (cudaEventRecord(h->ev_done[b], s) != cudaSuccess || cudaStreamWaitEvent(h->s_out, h->ev_done[b], 0) != cudaSuccess ||
            cudaMemcpyAsync((char*)h_out + (size_t)l * ob, h->d_out[b], ob, cudaMemcpyDeviceToHost, h->s_out) != cudaSuccess || cudaEventRecord(h->ev_down[b], h->s_out) != cudaSuccess) return KATA_ERR_CUDA;
    }
    // the caller's stream is complete when every row is on the host
    for (int b = 0; b < std::min(2, (int)n_layers); b++) if (cudaStreamWaitEvent(s, h->ev_down[b], 0) != cudaSuccess) return KATA_ERR_CUDA;
    return KATA_OK;
}

// The same step for a caller whose rows are on the device already: the layer loop of Engine::step / verify2 / verifyWide (prep, then decode, layer after
// layer) in one call, so that a host in another language pays one crossing per token instead of two per layer. Row l of every [n_layers][...] array
// belongs to layer l; nothing is copied.
extern "C" int kata_attn_layers_step(kata_attn_ctx* ctx, int32_t n_layers, int32_t n, const int32_t* seq_ids, const int32_t* pos0, int32_t T, int32_t first_pos,
                                     const void* d_qfull, const void* d_kproj, const void* d_vproj, int32_t act_dtype, const float* d_qnorm, const float* d_knorm,
                                     void* d_q16, float* d_gate, void* d_out, int32_t out_dtype, void* stream) {
    if (!ctx || n_layers < 1 || n < 1 || T < 1) return KATA_ERR_ARG;
    if (act_dtype != KATA_ACT_F32 && act_dtype != KATA_ACT_BF16 && act_dtype != KATA_ACT_F16) return KATA_ERR_ARG;
    if (out_dtype != KATA_ACT_F32 && out_dtype != KATA_ACT_BF16 && out_dtype != KATA_ACT_F16) return KATA_ERR_ARG;
    const size_t rows = (size_t)n * T, esz = act_dtype == KATA_ACT_F32 ? 4 : 2, osz = out_dtype == KATA_ACT_F32 ? 4 : 2;
    for (int l = 0; l < n_layers; l++) {
        void* q16 = (char*)d_q16 + (size_t)l * rows * 6144 * 2; float* gate = d_gate + (size_t)l * rows * 6144;
        int rc = kata_attn_prep(ctx, l, n, seq_ids, pos0, T, (const char*)d_qfull + (size_t)l * rows * 12288 * esz, (const char*)d_kproj + (size_t)l * rows * 1024 * esz,
                                (const char*)d_vproj + (size_t)l * rows * 1024 * esz, act_dtype, d_qnorm + (size_t)l * 256, d_knorm + (size_t)l * 256, q16, nullptr, gate, 0, 32, stream);
        if (rc == KATA_OK) rc = kata_attn_decode(ctx, l, n, seq_ids, pos0, T, first_pos, q16, gate, (char*)d_out + (size_t)l * rows * 6144 * osz, out_dtype, stream);
        if (rc != KATA_OK) return rc;
    }
    return KATA_OK;
}

// The decode calls alone, layer after layer (the rows prep left in d_q16 and d_gate; nothing is appended): for a caller that times or replays the
// attention kernels by themselves.
extern "C" int kata_attn_layers_decode(kata_attn_ctx* ctx, int32_t n_layers, int32_t n, const int32_t* seq_ids, const int32_t* pos_base, int32_t T, int32_t first_pos,
                                       const void* d_q16, const float* d_gate, void* d_out, int32_t out_dtype, void* stream) {
    if (!ctx || n_layers < 1 || n < 1 || T < 1 || !d_q16 || !d_gate || !d_out) return KATA_ERR_ARG;
    if (out_dtype != KATA_ACT_F32 && out_dtype != KATA_ACT_BF16 && out_dtype != KATA_ACT_F16) return KATA_ERR_ARG;
    const size_t rows = (size_t)n * T, osz = out_dtype == KATA_ACT_F32 ? 4 : 2;
    for (int l = 0; l < n_layers; l++) {
        const int rc = kata_attn_decode(ctx, l, n, seq_ids, pos_base, T, first_pos, (const char*)d_q16 + (size_t)l * rows * 6144 * 2, d_gate + (size_t)l * rows * 6144,
                                        (char*)d_out + (size_t)l * rows * 6144 * osz, out_dtype, stream);
        if (rc != KATA_OK) return rc;
    }
    return KATA_OK;
}

// The layer loop of a decode step whose one sequence is split by keys over the GPUs of a box: per layer this rank's prep (every rank forms the
// query; the rank that owns the tail of the sequence also appends the new K/V rows: head slots [0, 32), the others [0, 24)) and kata_attn_peer_decode
// (this rank's keys [key_lo, key_hi), its part pushed to the peers and the ranks' parts merged). All ranks must make the same call.
extern "C" int kata_attn_peer_layers_step(kata_attn_peer* px, kata_attn_ctx* ctx, int32_t n_layers, int32_t seq, int32_t pos, int32_t T, int32_t key_lo, int32_t key_hi, int32_t appends,
                                          const void* d_qfull, const void* d_kproj, const void* d_vproj, int32_t act_dtype, const float* d_qnorm, const float* d_knorm,
                                          void* d_q16, float* d_gate, void* d_out, int32_t out_dtype, void* stream) {
    if (!px || !ctx || n_layers < 1 || T < 1) return KATA_ERR_ARG;
    if (act_dtype != KATA_ACT_F32 && act_dtype != KATA_ACT_BF16 && act_dtype != KATA_ACT_F16) return KATA_ERR_ARG;
    if (out_dtype != KATA_ACT_F32 && out_dtype != KATA_ACT_BF16 && out_dtype != KATA_ACT_F16) return KATA_ERR_ARG;
    const size_t rows = (size_t)T, esz = act_dtype == KATA_ACT_F32 ? 4 : 2, osz = out_dtype == KATA_ACT_F32 ? 4 : 2;
    for (int l = 0; l < n_layers; l++) {
        void* q16 = (char*)d_q16 + (size_t)l * rows * 6144 * 2; float* gate = d_gate + (size_t)l * rows * 6144;
        int rc = kata_attn_prep(ctx, l, 1, &seq, &pos, T, (const char*)d_qfull + (size_t)l * rows * 12288 * esz, (const char*)d_kproj + (size_t)l * rows * 1024 * esz,
                                (const char*)d_vproj + (size_t)l * rows * 1024 * esz, act_dtype, d_qnorm + (size_t)l * 256, d_knorm + (size_t)l * 256, q16, nullptr, gate, 0, appends ? 32 : 24, stream);
        if (rc == KATA_OK) rc = kata_attn_peer_decode(px, ctx, l, seq, pos, T, key_lo, key_hi, q16, gate, (char*)d_out + (size_t)l * rows * 6144 * osz, out_dtype, stream);
        if (rc != KATA_OK) return rc;
    }
    return KATA_OK;
}
