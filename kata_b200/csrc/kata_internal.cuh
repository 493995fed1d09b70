// Internal declarations shared by the translation units of libkata_attn: the context object, the per-call batch
// descriptor handed to kernels by value, and the launcher prototypes.
#pragma once
#include <algorithm>
#include <climits>
#include <utility>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <string>
#include <vector>

#include "../../include/kata_attn.h"

namespace kata {

constexpr int kH = KATA_HEADS, kKvh = KATA_KV_HEADS, kD = KATA_HEAD_DIM, kG = 6, kQD = KATA_Q_DIM, kKVD = KATA_KV_DIM, kQFull = KATA_QFULL_DIM;
constexpr float kEps = 1e-6f;
constexpr float kLog2e = 1.4426950408889634f;
constexpr int kPartStride = 258;   // one (token, head) partial: O[256], m, l

// What a kernel needs to find the cache rows of the sequences of one call. Passed by value (kernel parameter space),
// so a call needs no host->device copy and no allocation. Row index of (sequence, layer, position) in the K/V arenas
// is row_base[b] + position, with row_base already including the layer offset layer * max_ctx.
struct Batch {
    int32_t n;
    int32_t seq[KATA_MAX_BATCH];        // sequence ids
    int32_t pos[KATA_MAX_BATCH];        // pos0 / pos_base per sequence
    int64_t row_base[KATA_MAX_BATCH];   // arena row of position 0 of (sequence, layer)
    int32_t item_start[KATA_MAX_BATCH + 1];   // decode: first work item of sequence b (prefix sum of 4 * n_splits[b])
    int32_t n_splits[KATA_MAX_BATCH];
};

struct Ctx {
    kata_attn_config cfg{};
    std::vector<int32_t> max_ctx;
    std::vector<int32_t> pos_off;      // absolute position held by row 0 of each sequence (0 unless the sequence is a key slice)
    std::vector<int64_t> seq_row0;     // arena row of (sequence, layer 0, position 0)
    int64_t total_rows = 0;
    int elt_k = 2, elt_v = 2;           // bytes per cached K / V element (int8: 1, 1; int8v: 2, 1)
    bool k8() const { return elt_k == 1; } bool v8() const { return elt_v == 1; } bool kg() const { return cfg.kv_mode == KATA_KV_INT8G; }   // kg: four K scales per head row (one per 64 dims)
    int ksc_per_row() const { return kg() ? 16 : 4; }
    void* k_arena = nullptr; void* v_arena = nullptr;      // [total_rows][1024] fp16 or int8
    __half* ksc = nullptr; __half* vsc = nullptr;          // [total_rows][4] fp16 scales of the int8 planes
    // decode scratch: per work item (sequence, kv head, split) the unnormalised partial rows and their (m, l)
    float* part_o = nullptr; float* part_ml = nullptr; int32_t* counters = nullptr; int32_t max_items = 0;
    // What the kernel launched last through this context wrote into the cache: nothing (prev_append false), or rows from position append_lo[s]
    // on in sequence s. The decode kernel may load rows that kernel cannot be writing before it waits for it (dependent launch).
    bool prev_append = false; std::vector<int32_t> append_lo;
    // Caller kernels may write cache rows through kata_attn_kv_plane_ptr. Once such a pointer has been handed out (ext_ptr) and until the caller
    // has started to declare its writes with kata_attn_mark_rows_written (ext_declared), no row is loaded before the wait. A mark stands for
    // "the kernel enqueued just before the next library call writes rows from this position on" (prev_mark: the record comes from marks).
    bool ext_ptr = false, ext_declared = false, prev_mark = false;
    void wrote_no_rows() { if (prev_append) std::fill(append_lo.begin(), append_lo.end(), INT32_MAX); prev_append = false; prev_mark = false; }
    void wrote_rows_from(int seq, int pos) { append_lo[seq] = std::min(append_lo[seq], pos); prev_append = true; }
    // scalar-path scratch (k_attn_split partials)
    float* sc_pm = nullptr; float* sc_pl = nullptr; float* sc_pacc = nullptr;
    // TMA descriptors over the K and V arenas viewed as [row][kv head][256]: 16-row x 128-byte boxes, 128-byte swizzle
    CUtensorMap tm_k_tile{}, tm_v_tile{};   // rank-4 views for decode: one TMA instruction per 16-key tile of one KV head
    __half* k16_stage = nullptr; __half* v16_stage = nullptr; std::vector<int64_t> stage_row0;   // int8 mode: one layer of fp16-expanded codes for the tcgen05 prefill, [sum of max_ctx][1024] each; first row per sequence
    CUtensorMap tm_k64h_stage{}, tm_v128h_stage{};
    CUtensorMap tm_k64h{}, tm_v128h{};   // rank-4 views for the tcgen05 prefill (fp16 mode): 64 keys x 256 dims of K, 128 keys x 128 dims of V (the halves a CTA of a pair loads)
    float* pf_part_o = nullptr; float* pf_part_ml = nullptr; int32_t* pf_part_flag = nullptr;   // tcgen05 prefill: partial rows and (m, l) of items cut between CTA pairs; one flag per part (up while the part waits to be folded into its item's head)
    // host-side work plan of the last tcgen05 prefill launch, reused while (chunk length, positions) stay the same (the layers of a chunk)
    alignas(8) unsigned char pf_plan_cache[2048] = {}; int pf_plan_M = -1, pf_plan_n = -1; int32_t pf_plan_pos[KATA_MAX_BATCH] = {}; int32_t pf_plan_tiles[(KATA_MAX_CHUNK / 128) * (KATA_HEADS / 2) * KATA_MAX_BATCH] = {};
    int32_t* d_err = nullptr;           // device error word: nonzero after a bounded wait ran out
    int kvh_lo = 0, kvh_n = KATA_KV_HEADS;   // KV heads this context computes (kata_attn_set_kv_heads): a rank of a head-sharded group owns a subset
    int sm_count = 148;
    uint64_t launches = 0;
    std::string err;
    std::string tag;
    int64_t row_of(int layer, int seq) const { return seq_row0[seq] + (int64_t)layer * max_ctx[seq]; }
};

// launchers (defined next to their kernels); each returns a cudaError_t from the launch
cudaError_t launch_prep(Ctx& c, const Batch& b, int T, const void* qfull, const void* kproj, const void* vproj, int act_dtype,
                        const float* qnorm, const float* knorm, __half* q16, float* q32, float* gate, int h0, int nh, cudaStream_t s);
cudaError_t launch_kv_quant(Ctx& c, int64_t row0, const __half* ks, const __half* vs, int T, cudaStream_t s);
cudaError_t launch_decode_mma(Ctx& c, const Batch& b, int T, int first_pos, int n_items, const __half* q16, const float* gate, void* out, int out_dtype,
                              float* part_out /* non-null: write merged partials instead of the gated output */, cudaStream_t s);
cudaError_t launch_merge_parts(Ctx& c, const float* parts, int n_parts, int T, const float* gate, void* out, int out_dtype, cudaStream_t s);
cudaError_t launch_decode_scalar(Ctx& c, const Batch& b, int T, int first_pos, const float* q32, const float* gate, float* out, cudaStream_t s);
cudaError_t launch_prefill(Ctx& c, const Batch& b, int M, const __half* q16, const float* gate, void* out, int out_dtype, cudaStream_t s);
void set_inv_freq(const float* host32);   // uploads the 32 inverse RoPE frequencies to constant memory of the current device
// rank-3 map over an arena [rows][4][256 elements of elt bytes]; box = {box_inner elements, 1, box_rows}; returns false on failure
// Launch with programmatic stream serialisation: the grid is set up (and its CTAs may start) while the previous kernel of the stream drains.
// Such a kernel must execute griddepcontrol.wait (pdl_wait below) before it touches anything an earlier kernel wrote.
#ifdef __CUDACC__
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args&&... args) {
    cudaLaunchConfig_t cfg{}; cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = s;
    cudaLaunchAttribute at[1]; at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(std::forward<Args>(args))...);
}
// Output rows in the activation dtype the caller asked for (kind = KATA_ACT_*): fp32, bf16 or fp16, rounded to nearest even.
__device__ __forceinline__ void store_act(void* out, int64_t i, float y, int kind) {
    if (kind == KATA_ACT_BF16) reinterpret_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(y);
    else if (kind == KATA_ACT_F16) reinterpret_cast<__half*>(out)[i] = __float2half_rn(y);
    else reinterpret_cast<float*>(out)[i] = y;
}
__device__ __forceinline__ void store_act2(void* out, int64_t i, float y0, float y1, int kind) {   // elements i, i+1; i even
    if (kind == KATA_ACT_BF16) reinterpret_cast<__nv_bfloat162*>(out)[i >> 1] = __floats2bfloat162_rn(y0, y1);
    else if (kind == KATA_ACT_F16) reinterpret_cast<__half2*>(out)[i >> 1] = __floats2half2_rn(y0, y1);
    else *reinterpret_cast<float2*>(reinterpret_cast<float*>(out) + i) = make_float2(y0, y1);
}
__device__ __forceinline__ void store_act4(void* out, int64_t i, float4 y, int kind) {   // elements i .. i+3; i a multiple of 4
    if (kind == KATA_ACT_BF16) { const __nv_bfloat162 a = __floats2bfloat162_rn(y.x, y.y), b = __floats2bfloat162_rn(y.z, y.w); *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(out) + i) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b)); }
    else if (kind == KATA_ACT_F16) { const __half2 a = __floats2half2_rn(y.x, y.y), b = __floats2half2_rn(y.z, y.w); *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(out) + i) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b)); }
    else *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + i) = y;
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }                  // every earlier kernel of the stream is complete and visible
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }   // the next kernel may be set up from now on
#endif

bool make_matrix_tmap(CUtensorMap* out, const void* base, int64_t rows, int64_t cols, int box_cols, int box_rows);
bool make_tile_tmap(CUtensorMap* out, void* base, int elt, int64_t rows, int box_rows, int box_blocks);

}  // namespace kata
