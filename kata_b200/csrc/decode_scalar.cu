// The fp32 (CUDA-core) decode path: attention of T <= 8 query tokens per sequence over the fp16 cache with the fp32 query (not rounded to
// fp16) and fp32 arithmetic throughout. It stands in for the reference's scalar route (k_attn_split(_b) + k_attn_combine(_b),
// shaders/attn.metal:66-117, shaders/prefill.metal:209-261; chosen by KATA_SCALAR_DEC and by Engine::verifyWide, src/engine.cpp:169-175,
// 365, 478, 617) and is the cross-check of the tensor-core kernels. Same math: scores q.k/16, key j visible to token t when
// first_pos <= j <= pos + t, softmax, weighted V sum, times sigmoid(gate); splits merged with weights exp(m - M).
//
// Organisation (written for the GPU, not after the shader, which walks the keys one by one per query token and re-reads K/V per token):
//  - a CTA of 4 warps takes one chunk of keys of one KV head for a group of up to 4 query tokens (24 rows = 6 heads x 4 tokens), so a K/V
//    row is read once for all rows that share it;
//  - keys are processed in tiles of 32, brought into shared memory with 16-byte cp.async (K rows padded to 528 bytes);
//  - scores: a LANE IS A KEY. Each warp owns 6 of the 24 rows; a lane forms the 256-long dot product of its key with the row (K as 128-bit
//    shared-memory loads, the query row broadcast), so the softmax needs one warp reduction per row and tile instead of one per key;
//  - values: a THREAD IS TWO HEAD DIMS. The tile's probabilities go through shared memory; each thread accumulates its two dims of all
//    24 rows over the 32 keys (probabilities broadcast, V read as consecutive half2).
//  - the chunk's unnormalised rows and (m, l) go to scratch and a second kernel merges the chunks and applies the gate.
#include <algorithm>

#include "kata_internal.cuh"
#include "ptx.cuh"

namespace kata {
namespace {

using namespace ptx;

constexpr int kFTile = 32, kFWarps = 4, kFThreads = 32 * kFWarps, kFTok = 4, kFRows = 6 * kFTok, kFRowsPerWarp = kFRows / kFWarps;
constexpr int kFKStride = 2 * kD + 16;           // bytes per K row in shared memory: 8 consecutive keys' 16-byte pieces fall into 8 different bank groups
constexpr int kMaxChunks = 32;                   // chunks per (token, head): bounds the scratch
constexpr int kGroupTokens = 16;                 // (sequence, token) pairs per launch: bounds the scratch
constexpr int kOffQ = 0, kOffK = kOffQ + kFRows * kD * 4, kOffV = kOffK + kFTile * kFKStride, kOffP = kOffV + kFTile * kD * 2, kOffA = kOffP + kFRows * kFTile * 4, kFSmem = kOffA + kFRows * 4;

// grid (chunks, KV heads, sequences of the launch x token groups)
__global__ void __launch_bounds__(kFThreads) decode_fp32_kernel(const Batch b, const int T, const int first_pos, const int b0, const int chunk_keys, const float* __restrict__ q,
                                                                const __half* __restrict__ K, const __half* __restrict__ V, float* __restrict__ pm, float* __restrict__ pl, float* __restrict__ pacc) {
    extern __shared__ __align__(16) uint8_t sm[];
    float* s_q = reinterpret_cast<float*>(sm + kOffQ); float* s_p = reinterpret_cast<float*>(sm + kOffP); float* s_alpha = reinterpret_cast<float*>(sm + kOffA);
    const int n_tg = (T + kFTok - 1) / kFTok, chunk = blockIdx.x, kvh = blockIdx.y, bi = b0 + blockIdx.z / n_tg, t0 = (blockIdx.z % n_tg) * kFTok, nt = min(kFTok, T - t0), R = 6 * nt;
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const int pos = b.pos[bi], lo = first_pos + chunk * chunk_keys, hi = min(lo + chunk_keys, pos + t0 + nt);   // keys [lo, hi) of this chunk that any row of the group may see
    if (chunk >= b.n_splits[bi]) return;
    // the group's query rows, scaled by 1/16 (exact), row = (t - t0) * 6 + head of the KV head
    for (int i = tid; i < R * (kD / 4); i += kFThreads) {
        const int row = i / (kD / 4), c4 = i % (kD / 4), t = t0 + row / 6, j = row % 6;
        float4 v = *reinterpret_cast<const float4*>(q + ((int64_t)bi * T + t) * kQD + (kvh * 6 + j) * kD + c4 * 4);
        v.x *= 0.0625f; v.y *= 0.0625f; v.z *= 0.0625f; v.w *= 0.0625f;
        *reinterpret_cast<float4*>(s_q + row * kD + c4 * 4) = v;
    }
    float m[kFRowsPerWarp], l[kFRowsPerWarp], acc[kFRows][2];
#pragma unroll
    for (int i = 0; i < kFRowsPerWarp; i++) { m[i] = -INFINITY; l[i] = 0.0f; }
#pragma unroll
    for (int r = 0; r < kFRows; r++) { acc[r][0] = 0.0f; acc[r][1] = 0.0f; }
    const __half* Kb = K + b.row_base[bi] * kKVD + kvh * kD; const __half* Vb = V + b.row_base[bi] * kKVD + kvh * kD;
    const uint32_t sm_k = smem_u32(sm + kOffK), sm_v = smem_u32(sm + kOffV);

    for (int k0 = lo; k0 < hi; k0 += kFTile) {
        // ---- the tile's K and V rows into shared memory (rows past the chunk are zero-filled)
        for (int i = tid; i < kFTile * 32; i += kFThreads) {
            const int key = i >> 5, piece = i & 31, kj = k0 + key; const uint32_t n = kj < hi ? 16u : 0u; const int64_t src = (int64_t)min(kj, hi - 1) * kKVD + piece * 8;
            cp_async16(sm_k + key * kFKStride + piece * 16, Kb + src, n); cp_async16(sm_v + key * (2 * kD) + piece * 16, Vb + src, n);
        }
        cp_async_commit(); cp_async_wait<0>();
        __syncthreads();
        // ---- scores of this warp's rows: lane = key
#pragma unroll
        for (int i = 0; i < kFRowsPerWarp; i++) {
            const int row = w + kFWarps * i;
            if (row < R) {   // warp-uniform
                const float* qr = s_q + row * kD; const uint8_t* kr = sm + kOffK + lane * kFKStride;
                float s = 0.0f;
#pragma unroll 8
                for (int c = 0; c < kD / 8; c++) {
                    const uint4 kk = *reinterpret_cast<const uint4*>(kr + c * 16); const __half2* kh = reinterpret_cast<const __half2*>(&kk);
                    const float4 qa = *reinterpret_cast<const float4*>(qr + c * 8), qb = *reinterpret_cast<const float4*>(qr + c * 8 + 4);
                    const float2 f0 = __half22float2(kh[0]), f1 = __half22float2(kh[1]), f2 = __half22float2(kh[2]), f3 = __half22float2(kh[3]);
                    s = fmaf(qa.x, f0.x, s); s = fmaf(qa.y, f0.y, s); s = fmaf(qa.z, f1.x, s); s = fmaf(qa.w, f1.y, s);
                    s = fmaf(qb.x, f2.x, s); s = fmaf(qb.y, f2.y, s); s = fmaf(qb.z, f3.x, s); s = fmaf(qb.w, f3.y, s);
                }
                const int kj = k0 + lane;
                if (kj >= hi || kj > pos + t0 + row / 6) s = -INFINITY;   // beyond the chunk, or after this row's token
                float mx = s;
#pragma unroll
                for (int off = 16; off >= 1; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
                const float mn = fmaxf(m[i], mx);
                const float alpha = (m[i] == -INFINITY) ? 0.0f : expf(m[i] - mn), p = (s == -INFINITY) ? 0.0f : expf(s - mn);
                float ps = p;
#pragma unroll
                for (int off = 16; off >= 1; off >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, off);
                l[i] = l[i] * alpha + ps; m[i] = mn;
                s_p[row * kFTile + lane] = p;
                if (lane == 0) s_alpha[row] = alpha;
            }
        }
        __syncthreads();
        // ---- values: thread = dims 2*tid, 2*tid + 1 of every row
#pragma unroll
        for (int r = 0; r < kFRows; r++) if (r < R) { const float a = s_alpha[r]; acc[r][0] *= a; acc[r][1] *= a; }
#pragma unroll 4
        for (int key = 0; key < kFTile; key++) {
            const float2 v = __half22float2(*reinterpret_cast<const __half2*>(sm + kOffV + key * (2 * kD) + tid * 4));
#pragma unroll
            for (int r = 0; r < kFRows; r++) if (r < R) { const float p = s_p[r * kFTile + key]; acc[r][0] = fmaf(p, v.x, acc[r][0]); acc[r][1] = fmaf(p, v.y, acc[r][1]); }
        }
        __syncthreads();   // the tile buffers and the probabilities are rewritten by the next tile
    }
    // ---- the chunk's partial rows: [launch-local token][head][chunk]
    const int64_t tok0 = (int64_t)(bi - b0) * T + t0;
#pragma unroll
    for (int r = 0; r < kFRows; r++) if (r < R) {
        const int64_t ti = (tok0 + r / 6) * kH + kvh * 6 + r % 6;
        *reinterpret_cast<float2*>(pacc + (ti * kMaxChunks + chunk) * kD + 2 * tid) = make_float2(acc[r][0], acc[r][1]);
    }
    if (lane == 0) {
#pragma unroll
        for (int i = 0; i < kFRowsPerWarp; i++) { const int row = w + kFWarps * i; if (row < R) { const int64_t ti = (tok0 + row / 6) * kH + kvh * 6 + row % 6; pm[ti * kMaxChunks + chunk] = m[i]; pl[ti * kMaxChunks + chunk] = l[i]; } }
    }
}

// Merge of the chunks of one (token, head) and the output gate: grid (24 heads, tokens of the launch), a thread per two head dims.
__global__ void __launch_bounds__(kD / 2) merge_fp32_kernel(const Batch b, const int T, const int b0, const float* __restrict__ pm, const float* __restrict__ pl, const float* __restrict__ pacc,
                                                            const float* __restrict__ gate, float* __restrict__ out) {
    const int h = blockIdx.x, z = blockIdx.y, bi = b0 + z / T, t = z % T, tid = threadIdx.x, n = b.n_splits[bi];
    const int64_t ti = (int64_t)z * kH + h;
    float M = -INFINITY;
    for (int c = 0; c < n; c++) M = fmaxf(M, pm[ti * kMaxChunks + c]);
    float L = 0.0f, A0 = 0.0f, A1 = 0.0f;
    for (int c = 0; c < n; c++) {
        const float mm = pm[ti * kMaxChunks + c];
        if (mm == -INFINITY) continue;   // a chunk none of whose keys this token sees: nothing was accumulated, nothing is read
        const float wt = expf(mm - M); const float2 a = *reinterpret_cast<const float2*>(pacc + (ti * kMaxChunks + c) * kD + 2 * tid);
        L += pl[ti * kMaxChunks + c] * wt; A0 += a.x * wt; A1 += a.y * wt;
    }
    const int64_t o = ((int64_t)bi * T + t) * kQD + h * kD + 2 * tid; const float2 g = *reinterpret_cast<const float2*>(gate + o);
    *reinterpret_cast<float2*>(out + o) = make_float2((A0 / L) * (1.0f / (1.0f + expf(-g.x))), (A1 / L) * (1.0f / (1.0f + expf(-g.y))));
}

}  // namespace

size_t scalar_scratch_floats_pm() { return (size_t)kGroupTokens * kH * kMaxChunks; }
size_t scalar_scratch_floats_acc() { return (size_t)kGroupTokens * kH * kMaxChunks * kD; }
cudaError_t configure_decode_scalar() { return cudaFuncSetAttribute(decode_fp32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kFSmem); }

cudaError_t launch_decode_scalar(Ctx& c, const Batch& b_in, int T, int first_pos, const float* q32, const float* gate, float* out, cudaStream_t s) {
    Batch b = b_in;
    // one chunk size for the launch: whole tiles, at least 128 keys, at most kMaxChunks chunks for the longest sequence
    int span = 1; for (int i = 0; i < b.n; i++) span = std::max(span, b.pos[i] + T - first_pos);
    const int chunk_keys = std::max(128, ((span + kMaxChunks - 1) / kMaxChunks + kFTile - 1) / kFTile * kFTile);
    int max_chunks = 1;
    for (int i = 0; i < b.n; i++) { b.n_splits[i] = std::max(1, (b.pos[i] + T - first_pos + chunk_keys - 1) / chunk_keys); max_chunks = std::max(max_chunks, b.n_splits[i]); }
    const int per_launch = std::max(1, kGroupTokens / T), n_tg = (T + kFTok - 1) / kFTok;
    for (int b0 = 0; b0 < b.n; b0 += per_launch) {
        const int nb = std::min(per_launch, b.n - b0);
        decode_fp32_kernel<<<dim3(max_chunks, kKvh, nb * n_tg), kFThreads, kFSmem, s>>>(b, T, first_pos, b0, chunk_keys, q32, (const __half*)c.k_arena, (const __half*)c.v_arena, c.sc_pm, c.sc_pl, c.sc_pacc);
        merge_fp32_kernel<<<dim3(kH, nb * T), kD / 2, 0, s>>>(b, T, b0, c.sc_pm, c.sc_pl, c.sc_pacc, gate, out);
        c.launches += 2;
    }
    return cudaGetLastError();
}

}  // namespace kata
