// The scalar (CUDA-core) split-KV decode path: flash-decoding on fp32 ALUs with the six query heads of a KV head
// sharing each K/V row, then a merge of the splits with the sigmoid output gate.
// Follows k_attn_split / k_attn_split_b and k_attn_combine / k_attn_combine_b of the reference
// (shaders/attn.metal:66-117, shaders/prefill.metal:209-261) and the engine's choice of split count
// (src/engine.cpp:171). It is the cross-check of the tensor-core path and serves T up to 8 query tokens; it is not
// the fast path (it re-reads K/V once per query token and runs on fp32 ALUs).
#include "kata_internal.cuh"

namespace kata {
namespace {

constexpr int kMaxS = 32;         // splits per (token, kv head), as the reference caps it
constexpr int kGroupTokens = 16;  // (sequence, token) pairs per launch: bounds the scratch

__global__ void __launch_bounds__(256) split_scalar_kernel(const Batch b, const int T, const int first_pos, const int b0, const float* __restrict__ q,
                                                           const __half* __restrict__ K, const __half* __restrict__ V, float* pm, float* pl, float* pacc) {
    __shared__ float tm[8][6], tl[8][6]; __shared__ float tacc[8][3][256];
    const int split = blockIdx.x, kvh = blockIdx.y, z = blockIdx.z, bi = b0 + z / T, t = z % T;
    const int S = b.n_splits[bi]; if (split >= S) return;
    const int tid = threadIdx.x, lane = tid & 31, sg = tid >> 5;
    const int npos = b.pos[bi] + t + 1, span = npos - first_pos, per = (span + S - 1) / S, lo = first_pos + min(split * per, span), hi = min(lo + per, npos);
    const int sper = (hi - lo + 7) / 8, slo = min(lo + sg * sper, hi), shi = min(slo + sper, hi);
    const float* qt = q + ((int64_t)bi * T + t) * kQD;
    const __half* Kb = K + b.row_base[bi] * kKVD + kvh * kD + lane * 8; const __half* Vb = V + b.row_base[bi] * kKVD + kvh * kD + lane * 8;
    float qv[6][8];
#pragma unroll
    for (int h = 0; h < 6; h++)
#pragma unroll
        for (int d = 0; d < 8; d++) qv[h][d] = qt[(kvh * 6 + h) * kD + lane * 8 + d] * 0.0625f;
    float m[6], l[6], acc[6][8];
#pragma unroll
    for (int h = 0; h < 6; h++) { m[h] = -INFINITY; l[h] = 0.0f;
#pragma unroll
        for (int d = 0; d < 8; d++) acc[h][d] = 0.0f; }
    for (int j = slo; j < shi; j++) {
        const uint4 kr = *reinterpret_cast<const uint4*>(Kb + (int64_t)j * kKVD), vr = *reinterpret_cast<const uint4*>(Vb + (int64_t)j * kKVD);
        float kf[8], vf[8];
        { const __half2* kh = reinterpret_cast<const __half2*>(&kr); const __half2* vh = reinterpret_cast<const __half2*>(&vr);
#pragma unroll
          for (int i = 0; i < 4; i++) { const float2 a = __half22float2(kh[i]), c = __half22float2(vh[i]); kf[2 * i] = a.x; kf[2 * i + 1] = a.y; vf[2 * i] = c.x; vf[2 * i + 1] = c.y; } }
#pragma unroll
        for (int h = 0; h < 6; h++) {
            float p = 0.0f;
#pragma unroll
            for (int d = 0; d < 8; d++) p += qv[h][d] * kf[d];
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) p += __shfl_xor_sync(0xffffffffu, p, off);
            const float mn = fmaxf(m[h], p), a = expf(m[h] - mn), e = expf(p - mn);
            l[h] = l[h] * a + e;
#pragma unroll
            for (int d = 0; d < 8; d++) acc[h][d] = acc[h][d] * a + e * vf[d];
            m[h] = mn;
        }
    }
    if (lane == 0) {
#pragma unroll
        for (int h = 0; h < 6; h++) { tm[sg][h] = m[h]; tl[sg][h] = l[h]; }
    }
    // merge the 8 warps in two rounds of 3 heads; thread tid then owns dimension tid
#pragma unroll
    for (int hg = 0; hg < 2; hg++) {
#pragma unroll
        for (int hh = 0; hh < 3; hh++)
#pragma unroll
            for (int d = 0; d < 8; d++) tacc[sg][hh][lane * 8 + d] = acc[hg * 3 + hh][d];
        __syncthreads();
#pragma unroll
        for (int hh = 0; hh < 3; hh++) {
            const int h = hg * 3 + hh;
            float M = -INFINITY;
#pragma unroll
            for (int s = 0; s < 8; s++) M = fmaxf(M, tm[s][h]);
            float L = 0.0f, A = 0.0f;
#pragma unroll
            for (int s = 0; s < 8; s++) { const float w = (tm[s][h] == -INFINITY) ? 0.0f : expf(tm[s][h] - M); L += tl[s][h] * w; A += tacc[s][hh][tid] * w; }
            const int64_t ti = (int64_t)z * 24 + kvh * 6 + h;
            pacc[(ti * kMaxS + split) * kD + tid] = A;
            if (tid == 0) { pm[ti * kMaxS + split] = M; pl[ti * kMaxS + split] = L; }
        }
        __syncthreads();
    }
}

// grid (24, tokens of the group)
__global__ void __launch_bounds__(256) combine_scalar_kernel(const Batch b, const int T, const int b0, const float* __restrict__ pm, const float* __restrict__ pl, const float* __restrict__ pacc,
                                                             const float* __restrict__ gate, float* __restrict__ out) {
    const int h = blockIdx.x, z = blockIdx.y, bi = b0 + z / T, t = z % T, tid = threadIdx.x, S = b.n_splits[bi];
    const int64_t ti = (int64_t)z * 24 + h;
    float M = -INFINITY; for (int s = 0; s < S; s++) M = fmaxf(M, pm[ti * kMaxS + s]);
    float L = 0.0f, A = 0.0f;
    for (int s = 0; s < S; s++) { const float mm = pm[ti * kMaxS + s]; const float w = (mm == -INFINITY) ? 0.0f : expf(mm - M); L += pl[ti * kMaxS + s] * w; A += pacc[(ti * kMaxS + s) * kD + tid] * w; }
    const int64_t o = ((int64_t)bi * T + t) * kQD + h * kD + tid;
    out[o] = (A / L) * (1.0f / (1.0f + expf(-gate[o])));
}

}  // namespace

size_t scalar_scratch_floats_pm() { return (size_t)kGroupTokens * 24 * kMaxS; }
size_t scalar_scratch_floats_acc() { return (size_t)kGroupTokens * 24 * kMaxS * kD; }

cudaError_t launch_decode_scalar(Ctx& c, const Batch& b_in, int T, int first_pos, const float* q32, const float* gate, float* out, cudaStream_t s) {
    Batch b = b_in;
    int maxS = 1;
    for (int i = 0; i < b.n; i++) { const int npos = b.pos[i] + T; b.n_splits[i] = std::min(kMaxS, std::max(1, npos / 64)); maxS = std::max(maxS, b.n_splits[i]); }
    const int per_launch = std::max(1, kGroupTokens / T);
    for (int b0 = 0; b0 < b.n; b0 += per_launch) {
        const int nb = std::min(per_launch, b.n - b0);
        split_scalar_kernel<<<dim3(maxS, kKvh, nb * T), 256, 0, s>>>(b, T, first_pos, b0, q32, (const __half*)c.k_arena, (const __half*)c.v_arena, c.sc_pm, c.sc_pl, c.sc_pacc);
        combine_scalar_kernel<<<dim3(kH, nb * T), 256, 0, s>>>(b, T, b0, c.sc_pm, c.sc_pl, c.sc_pacc, gate, out);
        c.launches += 2;
    }
    return cudaGetLastError();
}

}  // namespace kata
