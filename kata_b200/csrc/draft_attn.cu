// Attention of the block drafter: non-causal sliding-window attention of a block of T query rows over a ring of K/V rows, and the
// norm + RoPE + ring-append kernel that feeds it. C ABI in include/kata_draft.h.
// Replaces k_draft_qk, k_draft_ctx_kv and k_draft_attn of the reference (shaders/draft.metal:203-281; encoded at src/draft.cpp:112-123,
// 196-209): 32 query heads, 8 KV heads, head_dim 128, scale 1/sqrt(128), fp16 rings of [ring][8 * 128] per layer, query row t at
// position pos0 + t sees the keys at positions [pos0 + t - window + 1, pos0 + T - 1].
//
// The reference scans the keys one by one per (head, row) with fp32 query x fp16 key products and fp32 probabilities. Here the 4 heads
// of a KV head x T rows form one row block (row = t * 4 + j) so that each key is read once per KV head, and the two contractions run on
// mma.sync m16n8k16 with the fp32 operands split into two fp16 terms (x = hi + lo, both products accumulated in fp32): Q.K^T and P.V then
// carry about 22 significant bits of q and p, against 24 in the reference's scalar loop, and the fp16 K/V values are exact either way.
//
// HBM-bound and small (window 2048: 8.4 MB of K+V per layer), so the design goes for memory-level parallelism: the window is cut into
// chunks of at most 128 keys, one CTA per (chunk, KV head) (about one CTA per SM), each CTA requests its whole chunk at once with 16-byte
// cp.async copies in two groups (ring rows are gathered by position mod ring), splits the query block while the copies fly, and its eight
// warps take (row tile, 16-key sub-tile) pairs with private online-softmax state, starting on the first group while the second lands. Warp partials are merged through shared memory, chunk partials
// (O, m, l) through a small combine grid launched with programmatic stream serialisation.
#include <algorithm>
#include <climits>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <new>
#include <string>

#include "kata_internal.cuh"
#include "ptx.cuh"
#include "../../include/kata_draft.h"

struct kata_draft_ctx {
    kata_draft_config cfg{};
    __half* kring = nullptr; __half* vring = nullptr;     // [n_layers][ring][1024] fp16
    float* part_o = nullptr; float* part_ml = nullptr;     // chunk partials: [8 KV heads][max splits][64 rows][128], and their (m, l)
    int sm_count = 148;
    uint64_t launches = 0;
    std::string err;
};

namespace kata {
namespace {

using namespace ptx;

constexpr int kDH = KATA_DRAFT_HEADS, kDKV = KATA_DRAFT_KV_HEADS, kDD = KATA_DRAFT_HEAD_DIM, kDQD = KATA_DRAFT_Q_DIM, kDKVD = KATA_DRAFT_KV_DIM;
constexpr int kDRowStride = 272;                 // bytes per staged row: 128 fp16 + 16 pad (the eight rows of an ldmatrix fall in distinct banks)
constexpr int kDChunk = 128, kDMaxSplits = 48;   // most keys per CTA; most chunks per call
constexpr int kDRows = 4 * KATA_DRAFT_MAX_BLOCK; // 64 rows of the query block
constexpr int kOffQhi = 0, kOffQlo = kDRows * kDRowStride, kOffK = 2 * kDRows * kDRowStride, kOffV = kOffK + kDChunk * kDRowStride, kDraftSmem = kOffV + kDChunk * kDRowStride;
constexpr int kMoStride = 132;                   // floats per row of a warp's partial O in the merge buffer (which reuses the shared window from its start)
constexpr int kDWarps = 8, kDThreads = kDWarps * 32;
constexpr int kMergeBytes = kDWarps * 16 * kMoStride * 4;
static_assert(kMergeBytes <= kDraftSmem, "merge buffer must fit the shared window");

__constant__ float c_draft_inv_freq[64];   // 1e7^(-i/64), shaders/draft.metal:226

struct DraftPlan { int32_t pos0, T, win, ring_mask, klo, khi, chunk, n_splits; };   // keys [klo, khi) of the call, cut into n_splits chunks

__device__ __forceinline__ void split2(float a, float b, uint32_t& hi, uint32_t& lo) {   // two fp32 values -> packed fp16 heads and fp16 remainders
    const __half2 h = __floats2half2_rn(a, b); const float2 hf = __half22float2(h);
    const __half2 l = __floats2half2_rn(a - hf.x, b - hf.y);
    hi = *reinterpret_cast<const uint32_t*>(&h); lo = *reinterpret_cast<const uint32_t*>(&l);
}

// grid (n_splits, 8 KV heads) x 256 threads
__global__ void __launch_bounds__(kDThreads) draft_attn_kernel(const DraftPlan p, const float* __restrict__ q, const __half* __restrict__ kring, const __half* __restrict__ vring,
                                                         float* __restrict__ part_o, float* __restrict__ part_ml) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ float s_ml[kDWarps][16][2];
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5, g = lane >> 2, t4 = lane & 3, split = blockIdx.x, kvh = blockIdx.y;
    const uint32_t sm = smem_u32(smem);
    const int k0 = p.klo + split * p.chunk, k1 = min(k0 + p.chunk, p.khi), nk = k1 - k0, rows_pad = (nk + 15) & ~15;
    const uint32_t off_v = kOffK + p.chunk * kDRowStride;   // the K area holds p.chunk rows
    pdl_wait(); pdl_launch_dependents();   // the ring rows of this block and q come from the kernel launched just before

    // ---- the chunk's K and V rows, all requested at once in two groups of sub-tiles (position p lives at ring row p mod ring); rows past
    // the chunk arrive as zeros
    const int n_sub = rows_pad >> 4, sub_a = (n_sub + 1) >> 1;   // sub-tiles [0, sub_a) form the first group
    auto request = [&](int row_from, int row_to) {
        for (int idx = row_from * 16 + tid; idx < row_to * 16; idx += kDThreads) {
            const int r = idx >> 4, c = idx & 15; const bool ok = r < nk;
            const int64_t src = (int64_t)((k0 + (ok ? r : 0)) & p.ring_mask) * kDKVD + kvh * kDD + c * 8;
            cp_async16(sm + kOffK + r * kDRowStride + c * 16, kring + src, ok ? 16u : 0u);
            cp_async16(sm + off_v + r * kDRowStride + c * 16, vring + src, ok ? 16u : 0u);
        }
        cp_async_commit();
    };
    request(0, sub_a * 16); request(sub_a * 16, rows_pad);
    // ---- the query block (rows t*4 + j, zero up to the next multiple of 16), split into fp16 head and remainder, while the copies fly:
    // the loads of a thread's (up to 8) chunks are issued together, then converted
    const int rows = 4 * p.T, n_mt = (rows + 15) >> 4;
    {
        float4 v[8];
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const int idx = tid + u * kDThreads, r = idx >> 5, c4 = idx & 31; v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (r < rows) v[u] = __ldg(reinterpret_cast<const float4*>(q + (int64_t)(r >> 2) * kDQD + (kvh * 4 + (r & 3)) * kDD + c4 * 4));
        }
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const int idx = tid + u * kDThreads, r = idx >> 5, c4 = idx & 31;
            if (r < n_mt * 16) {
                uint2 hi, lo; split2(v[u].x, v[u].y, hi.x, lo.x); split2(v[u].z, v[u].w, hi.y, lo.y);
                *reinterpret_cast<uint2*>(smem + kOffQhi + r * kDRowStride + c4 * 8) = hi; *reinterpret_cast<uint2*>(smem + kOffQlo + r * kDRowStride + c4 * 8) = lo;
            }
        }
    }
    static_assert(8 * kDThreads == kDRows * 32, "a thread stages 8 chunks of the query block");
    cp_async_wait<1>();
    __syncthreads();

    // ---- warp w: row tile w % n_mt, 16-key sub-tiles w / n_mt, + n_kw, ...
    const int n_kw = kDWarps / n_mt, mt = w % n_mt, kw = w / n_mt; const bool active = kw < n_kw;
    float o[16][4]; float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;
#pragma unroll
    for (int j = 0; j < 16; j++) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f; }
    {
        const int r0 = mt * 16 + g, r1 = r0 + 8;
        const int lo0 = r0 < rows ? p.pos0 + (r0 >> 2) + 1 - p.win : INT_MAX, lo1 = r1 < rows ? p.pos0 + (r1 >> 2) + 1 - p.win : INT_MAX;   // first visible key of rows g and g + 8
        const uint32_t qa_hi = sm + kOffQhi + (mt * 16 + (lane & 15)) * kDRowStride + (lane >> 4) * 16, qa_lo = qa_hi + (kOffQlo - kOffQhi);
        const float sc = 0.08838834764831845f * kLog2e;   // 1/sqrt(128), scores kept in log2 units
        auto run = [&](int st_from, int st_to) {
        for (int st = st_from; st < st_to; st += n_kw) {
            const uint32_t ka = sm + kOffK + (st * 16 + (lane & 7) + ((lane >> 4) << 3)) * kDRowStride + ((lane >> 3) & 1) * 16;
            float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}}, s2[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};   // heads and remainders on separate chains
#pragma unroll
            for (int kk = 0; kk < 8; kk++) {
                uint32_t a0, a1, a2, a3, c0, c1, c2, c3, b0, b1, b2, b3;
                ldsm_x4(qa_hi + kk * 32, a0, a1, a2, a3); ldsm_x4(qa_lo + kk * 32, c0, c1, c2, c3); ldsm_x4(ka + kk * 32, b0, b1, b2, b3);
                mma16816(s[0], a0, a1, a2, a3, b0, b1); mma16816(s[1], a0, a1, a2, a3, b2, b3);
                mma16816(s2[0], c0, c1, c2, c3, b0, b1); mma16816(s2[1], c0, c1, c2, c3, b2, b3);
            }
#pragma unroll
            for (int nt = 0; nt < 2; nt++)
#pragma unroll
                for (int e = 0; e < 4; e++) s[nt][e] += s2[nt][e];
            const int key0 = k0 + st * 16;
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < 2; nt++)
#pragma unroll
                for (int e = 0; e < 2; e++) {   // mask by select: window start per row, end of the chunk
                    const int key = key0 + nt * 8 + 2 * t4 + e;
                    s[nt][e] = (key >= lo0 && key < k1) ? s[nt][e] * sc : -INFINITY; s[nt][2 + e] = (key >= lo1 && key < k1) ? s[nt][2 + e] * sc : -INFINITY;
                    mx0 = fmaxf(mx0, s[nt][e]); mx1 = fmaxf(mx1, s[nt][2 + e]);
                }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
            const float al0 = (mn0 == -INFINITY) ? 1.0f : ex2(m0 - mn0), al1 = (mn1 == -INFINITY) ? 1.0f : ex2(m1 - mn1);
            const float sub0 = (mn0 == -INFINITY) ? 0.0f : mn0, sub1 = (mn1 == -INFINITY) ? 0.0f : mn1;
            m0 = mn0; m1 = mn1;
            float pr[2][4];
#pragma unroll
            for (int nt = 0; nt < 2; nt++) { pr[nt][0] = ex2(s[nt][0] - sub0); pr[nt][1] = ex2(s[nt][1] - sub0); pr[nt][2] = ex2(s[nt][2] - sub1); pr[nt][3] = ex2(s[nt][3] - sub1); }
            l0 = l0 * al0 + ((pr[0][0] + pr[0][1]) + (pr[1][0] + pr[1][1])); l1 = l1 * al1 + ((pr[0][2] + pr[0][3]) + (pr[1][2] + pr[1][3]));
            if (__any_sync(0xffffffffu, al0 != 1.0f || al1 != 1.0f)) {
#pragma unroll
                for (int j = 0; j < 16; j++) { o[j][0] *= al0; o[j][1] *= al0; o[j][2] *= al1; o[j][3] *= al1; }
            }
            uint32_t ph[4], pl[4];   // the probabilities as the A operand of P.V: heads and remainders
            split2(pr[0][0], pr[0][1], ph[0], pl[0]); split2(pr[0][2], pr[0][3], ph[1], pl[1]); split2(pr[1][0], pr[1][1], ph[2], pl[2]); split2(pr[1][2], pr[1][3], ph[3], pl[3]);
            const uint32_t va = sm + off_v + (st * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * kDRowStride + (lane >> 4) * 16;
#pragma unroll
            for (int j2 = 0; j2 < 8; j2++) {
                uint32_t b0, b1, b2, b3; ldsm_x4_t(va + j2 * 32, b0, b1, b2, b3);
                mma16816(o[2 * j2], ph[0], ph[1], ph[2], ph[3], b0, b1); mma16816(o[2 * j2 + 1], ph[0], ph[1], ph[2], ph[3], b2, b3);
                mma16816(o[2 * j2], pl[0], pl[1], pl[2], pl[3], b0, b1); mma16816(o[2 * j2 + 1], pl[0], pl[1], pl[2], pl[3], b2, b3);
            }
        }
        };
        // this warp's sub-tiles kw, kw + n_kw, ...: those of the first group now, the rest when the second group has landed
        const int first_b = kw + ((max(sub_a - kw, 0) + n_kw - 1) / n_kw) * n_kw;   // its first sub-tile >= sub_a
        if (active) run(kw, sub_a);
        cp_async_wait<0>();
        __syncthreads();   // (every warp, whether it has sub-tiles or not)
        if (active) run(first_b, n_sub);
        l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    }
    // ---- merge the warps that shared a row tile, write the chunk's partial rows: the warps exchange their row maxima, each scales its own
    // partial O by 2^(m - M) in registers, and the scaled partials are summed from shared memory (the merge buffer reuses the K/V area)
    if (active && t4 == 0) { s_ml[w][g][0] = m0; s_ml[w][g][1] = l0; s_ml[w][g + 8][0] = m1; s_ml[w][g + 8][1] = l1; }
    __syncthreads();   // the maxima are visible; nobody reads K/V any more
    float* mo_all = reinterpret_cast<float*>(smem);   // the query block and the K/V rows are no longer needed
    const int64_t slot0 = (int64_t)(kvh * p.n_splits + split) * kDRows;
    if (active) {
        float M0 = -INFINITY, M1 = -INFINITY;
        for (int k = 0; k < n_kw; k++) { M0 = fmaxf(M0, s_ml[k * n_mt + mt][g][0]); M1 = fmaxf(M1, s_ml[k * n_mt + mt][g + 8][0]); }
        const float w0 = (m0 == -INFINITY) ? 0.0f : ex2(m0 - M0), w1 = (m1 == -INFINITY) ? 0.0f : ex2(m1 - M1);
        float* mo = mo_all + w * 16 * kMoStride;
#pragma unroll
        for (int j = 0; j < 16; j++) {
            *reinterpret_cast<float2*>(mo + g * kMoStride + 8 * j + 2 * t4) = make_float2(o[j][0] * w0, o[j][1] * w0);
            *reinterpret_cast<float2*>(mo + (g + 8) * kMoStride + 8 * j + 2 * t4) = make_float2(o[j][2] * w1, o[j][3] * w1);
        }
        if (kw == 0 && t4 == 0) {   // (M, l) of rows g and g + 8 of this row tile
            float L0 = 0.0f, L1 = 0.0f;
            for (int k = 0; k < n_kw; k++) {
                const int ww = k * n_mt + mt; const float a = s_ml[ww][g][0], b = s_ml[ww][g + 8][0];
                L0 += s_ml[ww][g][1] * ((a == -INFINITY) ? 0.0f : ex2(a - M0)); L1 += s_ml[ww][g + 8][1] * ((b == -INFINITY) ? 0.0f : ex2(b - M1));
            }
            const int r0 = mt * 16 + g;
            if (r0 < rows) { part_ml[(slot0 + r0) * 2] = M0; part_ml[(slot0 + r0) * 2 + 1] = L0; }
            if (r0 + 8 < rows) { part_ml[(slot0 + r0 + 8) * 2] = M1; part_ml[(slot0 + r0 + 8) * 2 + 1] = L1; }
        }
    }
    __syncthreads();
    for (int idx = tid; idx < rows * 32; idx += kDThreads) {   // four dims of one row per thread
        const int r = idx >> 5, c4 = idx & 31, rmt = r >> 4, rr = r & 15;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int k = 0; k < n_kw; k++) { const float4 v = *reinterpret_cast<const float4*>(mo_all + ((k * n_mt + rmt) * 16 + rr) * kMoStride + c4 * 4); a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w; }
        *reinterpret_cast<float4*>(part_o + (slot0 + r) * kDD + c4 * 4) = a;
    }
}

// grid (32 heads, T) x 128 threads: merge of the chunk partials of one output row, weights 2^(m - M), then O / l
__global__ void __launch_bounds__(128) draft_combine_kernel(const DraftPlan p, const float* __restrict__ part_o, const float* __restrict__ part_ml, float* __restrict__ out) {
    const int h = blockIdx.x, t = blockIdx.y, d = threadIdx.x, kvh = h >> 2, r = t * 4 + (h & 3);
    pdl_wait(); pdl_launch_dependents();
    float M = -INFINITY;
    for (int s = 0; s < p.n_splits; s++) M = fmaxf(M, part_ml[((int64_t)(kvh * p.n_splits + s) * kDRows + r) * 2]);
    float L = 0.0f, A = 0.0f;
    for (int s = 0; s < p.n_splits; s++) {
        const int64_t slot = (int64_t)(kvh * p.n_splits + s) * kDRows + r; const float mm = part_ml[slot * 2], wt = (mm == -INFINITY) ? 0.0f : ex2(mm - M);
        L += part_ml[slot * 2 + 1] * wt; A += part_o[slot * kDD + d] * wt;
    }
    out[(int64_t)t * kDQD + h * kDD + d] = A / L;
}

// k_draft_qk / k_draft_ctx_kv: one warp per (head slot, row); slots 0..31 query heads, 32..39 key heads, 40..47 value heads. Lane j holds dims
// j, 32+j, 64+j, 96+j: the sum of squares is formed as the reference's threadgroup does (a butterfly inside each 32 consecutive dims, the four
// group sums added in order) and the RoPE pairs (i, i+64) sit in one lane. Explicit round-to-nearest intrinsics keep the compiler from contracting.
__global__ void __launch_bounds__(256) draft_qk_kernel(const float* __restrict__ qin, const float* __restrict__ kin, const float* __restrict__ vin, const float* __restrict__ qnorm, const float* __restrict__ knorm,
                                                       float* __restrict__ qout, __half* __restrict__ kring, __half* __restrict__ vring, const int pos0, const int ring_mask, const int h0, const int nh) {
    pdl_wait(); pdl_launch_dependents();
    const int lane = threadIdx.x & 31, slot = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (slot >= nh) return;
    const int h = h0 + slot, t = blockIdx.y, pos = pos0 + t; const int64_t ring_row = (int64_t)(pos & ring_mask) * kDKVD;
    if (h >= kDH + kDKV) {
        const int vh = h - kDH - kDKV;
#pragma unroll
        for (int s = 0; s < 4; s++) vring[ring_row + vh * kDD + 32 * s + lane] = __float2half_rn(__ldg(vin + (int64_t)t * kDKVD + vh * kDD + 32 * s + lane));
        return;
    }
    const bool isK = h >= kDH; const int hh = isK ? h - kDH : h;
    const float* src = isK ? kin + (int64_t)t * kDKVD + hh * kDD : qin + (int64_t)t * kDQD + hh * kDD; const float* wgt = isK ? knorm : qnorm;
    float v[4], tot = 0.0f;
#pragma unroll
    for (int s = 0; s < 4; s++) {
        v[s] = __ldg(src + 32 * s + lane);
        float x = __fmul_rn(v[s], v[s]);
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) x = __fadd_rn(x, __shfl_xor_sync(0xffffffffu, x, off));
        tot = __fadd_rn(tot, x);
    }
    const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, 128.0f), 1e-6f)));
    float x[4];
#pragma unroll
    for (int s = 0; s < 4; s++) x[s] = __fmul_rn(__fmul_rn(v[s], r), __ldg(wgt + 32 * s + lane));
#pragma unroll
    for (int s = 0; s < 2; s++) {   // pair (i, i + 64), i = 32*s + lane
        const float theta = __fmul_rn((float)pos, c_draft_inv_freq[32 * s + lane]);
        float sn, cs; sincosf(theta, &sn, &cs);
        const float a = x[s], b = x[s + 2];
        x[s] = __fsub_rn(__fmul_rn(a, cs), __fmul_rn(b, sn)); x[s + 2] = __fadd_rn(__fmul_rn(a, sn), __fmul_rn(b, cs));
    }
#pragma unroll
    for (int s = 0; s < 4; s++) {
        if (isK) kring[ring_row + hh * kDD + 32 * s + lane] = __float2half_rn(x[s]);
        else qout[(int64_t)t * kDQD + hh * kDD + 32 * s + lane] = x[s];
    }
}

int dfail(kata_draft_ctx* c, int code, const char* fmt, ...) {
    char buf[384]; va_list ap; va_start(ap, fmt); vsnprintf(buf, sizeof buf, fmt, ap); va_end(ap);
    c->err = buf; return code;
}
struct DevGuard {
    int prev = -1;
    explicit DevGuard(int dev) { cudaGetDevice(&prev); if (prev != dev) cudaSetDevice(dev); else prev = -1; }
    ~DevGuard() { if (prev >= 0) cudaSetDevice(prev); }
};

}  // namespace
}  // namespace kata

using namespace kata;

extern "C" {

int kata_draft_create(const kata_draft_config* cfg, kata_draft_ctx** out) {
    if (!cfg || !out) return KATA_ERR_ARG;
    *out = nullptr;
    if (cfg->n_layers < 1 || cfg->window < 1 || cfg->ring < 16 || (cfg->ring & (cfg->ring - 1)) != 0 || cfg->ring < cfg->window + KATA_DRAFT_MAX_BLOCK ||
        cfg->window + KATA_DRAFT_MAX_BLOCK > kDChunk * kDMaxSplits) return KATA_ERR_ARG;
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || cfg->device < 0 || cfg->device >= ndev) return KATA_ERR_CUDA;
    kata_draft_ctx* c = new (std::nothrow) kata_draft_ctx();
    if (!c) return KATA_ERR_NOMEM;
    c->cfg = *cfg;
    DevGuard guard(cfg->device);
    cudaDeviceGetAttribute(&c->sm_count, cudaDevAttrMultiProcessorCount, cfg->device);
    const size_t ring_bytes = (size_t)cfg->n_layers * cfg->ring * kDKVD * 2;
    bool ok = cudaMalloc((void**)&c->kring, ring_bytes) == cudaSuccess && cudaMalloc((void**)&c->vring, ring_bytes) == cudaSuccess &&
              cudaMalloc((void**)&c->part_o, (size_t)kDKV * kDMaxSplits * kDRows * kDD * 4) == cudaSuccess && cudaMalloc((void**)&c->part_ml, (size_t)kDKV * kDMaxSplits * kDRows * 2 * 4) == cudaSuccess;
    if (!ok) { cudaGetLastError(); kata_draft_destroy(c); return KATA_ERR_NOMEM; }
    float invf[64]; for (int i = 0; i < 64; i++) invf[i] = powf(10000000.0f, -(float)i / 64.0f);
    if (cudaMemcpyToSymbol(c_draft_inv_freq, invf, sizeof invf) != cudaSuccess ||
        cudaFuncSetAttribute(draft_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDraftSmem) != cudaSuccess ||
        kata_draft_reset(c, nullptr) != KATA_OK || cudaDeviceSynchronize() != cudaSuccess) { cudaGetLastError(); kata_draft_destroy(c); return KATA_ERR_CUDA; }
    *out = c;
    return KATA_OK;
}

int kata_draft_destroy(kata_draft_ctx* c) {
    if (!c) return KATA_ERR_ARG;
    DevGuard guard(c->cfg.device);
    void* ptrs[] = {c->kring, c->vring, c->part_o, c->part_ml};
    for (void* p : ptrs) if (p) cudaFree(p);
    delete c;
    return KATA_OK;
}

int kata_draft_reset(kata_draft_ctx* c, void* stream) {
    if (!c) return KATA_ERR_ARG;
    DevGuard guard(c->cfg.device);
    const size_t ring_bytes = (size_t)c->cfg.n_layers * c->cfg.ring * kDKVD * 2;
    cudaError_t e = cudaMemsetAsync(c->kring, 0, ring_bytes, (cudaStream_t)stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(c->vring, 0, ring_bytes, (cudaStream_t)stream);
    return e == cudaSuccess ? KATA_OK : dfail(c, KATA_ERR_CUDA, "reset: %s", cudaGetErrorString(e));
}

const char* kata_draft_last_error(const kata_draft_ctx* c) { return c ? c->err.c_str() : "null context"; }
uint64_t kata_draft_launch_count(const kata_draft_ctx* c) { return c ? c->launches : 0; }

void* kata_draft_ring_ptr(kata_draft_ctx* c, int32_t layer, int32_t value) {
    if (!c || layer < 0 || layer >= c->cfg.n_layers) return nullptr;
    return (value ? c->vring : c->kring) + (size_t)layer * c->cfg.ring * kDKVD;
}

static int ring_copy(kata_draft_ctx* c, int32_t layer, int32_t value, int32_t row0, int32_t nrows, void* host, bool to_host) {
    if (!c) return KATA_ERR_ARG;
    if (layer < 0 || layer >= c->cfg.n_layers || row0 < 0 || nrows < 0 || (int64_t)row0 + nrows > c->cfg.ring || (!host && nrows)) return dfail(c, KATA_ERR_RANGE, "layer %d, ring rows [%d,%d) of %d", layer, row0, row0 + nrows, c->cfg.ring);
    if (!nrows) return KATA_OK;
    DevGuard guard(c->cfg.device);
    uint8_t* dev = (uint8_t*)kata_draft_ring_ptr(c, layer, value) + (size_t)row0 * kDKVD * 2; const size_t bytes = (size_t)nrows * kDKVD * 2;
    cudaError_t e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = to_host ? cudaMemcpy(host, dev, bytes, cudaMemcpyDeviceToHost) : cudaMemcpy(dev, host, bytes, cudaMemcpyHostToDevice);
    return e == cudaSuccess ? KATA_OK : dfail(c, KATA_ERR_CUDA, "ring copy: %s", cudaGetErrorString(e));
}
int kata_draft_ring_read(kata_draft_ctx* c, int32_t layer, int32_t value, int32_t row0, int32_t nrows, void* h_dst) { return ring_copy(c, layer, value, row0, nrows, h_dst, true); }
int kata_draft_ring_write(kata_draft_ctx* c, int32_t layer, int32_t value, int32_t row0, int32_t nrows, const void* h_src) { return ring_copy(c, layer, value, row0, nrows, const_cast<void*>(h_src), false); }

int kata_draft_qk(kata_draft_ctx* c, int32_t layer, const float* d_qin, const float* d_kin, const float* d_vin, const float* d_qnorm, const float* d_knorm,
                  float* d_qout, int32_t pos0, int32_t T, void* stream) {
    if (!c) return KATA_ERR_ARG;
    if (layer < 0 || layer >= c->cfg.n_layers) return dfail(c, KATA_ERR_RANGE, "layer %d outside [0,%d)", layer, c->cfg.n_layers);
    if (T < 1 || T > KATA_DRAFT_MAX_ROWS || pos0 < 0 || (int64_t)pos0 + T > INT32_MAX) return dfail(c, KATA_ERR_RANGE, "%d rows (1..%d) at position %d", T, KATA_DRAFT_MAX_ROWS, pos0);
    if (!d_kin || !d_vin || !d_knorm || (d_qin && (!d_qnorm || !d_qout))) return dfail(c, KATA_ERR_ARG, "qk needs kin, vin, knorm, and qnorm + qout when qin is given");
    DevGuard guard(c->cfg.device);
    const int h0 = d_qin ? 0 : kDH, nh = kDH + 2 * kDKV - h0;
    const cudaError_t e = launch_pdl(draft_qk_kernel, dim3((nh + 7) / 8, T), dim3(256), 0, (cudaStream_t)stream, d_qin, d_kin, d_vin, d_qnorm, d_knorm, d_qout,
                                     (__half*)kata_draft_ring_ptr(c, layer, 0), (__half*)kata_draft_ring_ptr(c, layer, 1), (int)pos0, c->cfg.ring - 1, h0, nh);
    if (e != cudaSuccess) return dfail(c, KATA_ERR_CUDA, "qk launch: %s", cudaGetErrorString(e));
    c->launches++;
    return KATA_OK;
}

int kata_draft_attn(kata_draft_ctx* c, int32_t layer, const float* d_q, float* d_out, int32_t pos0, int32_t T, void* stream) {
    if (!c) return KATA_ERR_ARG;
    if (layer < 0 || layer >= c->cfg.n_layers) return dfail(c, KATA_ERR_RANGE, "layer %d outside [0,%d)", layer, c->cfg.n_layers);
    if (T < 1 || T > KATA_DRAFT_MAX_BLOCK || pos0 < 0 || (int64_t)pos0 + T > INT32_MAX) return dfail(c, KATA_ERR_RANGE, "block of %d rows (1..%d) at position %d", T, KATA_DRAFT_MAX_BLOCK, pos0);
    if (!d_q || !d_out) return dfail(c, KATA_ERR_ARG, "attn needs q and out");
    DevGuard guard(c->cfg.device);
    DraftPlan p{}; p.pos0 = pos0; p.T = T; p.win = c->cfg.window; p.ring_mask = c->cfg.ring - 1;
    p.klo = std::max(0, pos0 + 1 - c->cfg.window); p.khi = pos0 + T;   // row 0 has the earliest window start; every row sees up to the end of the block
    const int nkeys = p.khi - p.klo, want = std::max(1, std::min(kDMaxSplits, c->sm_count / kDKV));   // one CTA per SM (two per SM with 64-key chunks measured slower: 10.9 against 10.0 us, and twice the partials for the combine grid)
    p.chunk = std::min(kDChunk, ((nkeys + want - 1) / want + 15) & ~15);
    p.n_splits = (nkeys + p.chunk - 1) / p.chunk;   // <= kDMaxSplits: create() bounded window + block by kDChunk * kDMaxSplits
    if (p.n_splits > kDMaxSplits) { p.chunk = kDChunk; p.n_splits = (nkeys + kDChunk - 1) / kDChunk; }
    const __half* kr = (const __half*)kata_draft_ring_ptr(c, layer, 0); const __half* vr = (const __half*)kata_draft_ring_ptr(c, layer, 1);
    cudaError_t e = launch_pdl(draft_attn_kernel, dim3(p.n_splits, kDKV), dim3(kDThreads), (size_t)std::max(kMergeBytes, kOffK + 2 * p.chunk * kDRowStride), (cudaStream_t)stream, p, d_q, kr, vr, c->part_o, c->part_ml);
    if (e == cudaSuccess) e = launch_pdl(draft_combine_kernel, dim3(kDH, T), dim3(128), 0, (cudaStream_t)stream, p, (const float*)c->part_o, (const float*)c->part_ml, d_out);
    if (e != cudaSuccess) return dfail(c, KATA_ERR_CUDA, "attn launch: %s", cudaGetErrorString(e));
    c->launches += 2;
    return KATA_OK;
}

}  // extern "C"
