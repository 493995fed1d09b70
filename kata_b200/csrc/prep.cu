// Attention prep for the gated-GQA layers: per-head Q/K RMSNorm, partial RoPE on dims 0..63, gate split, append of the
// K and V rows to the cache, with the fp16 prescaled query and (int8 mode) quantise-on-append fused in.
// Follows k_attn_prep / k_attn_prep_b (shaders/attn.metal:5-37, shaders/prefill.metal:179-206), k_cvt_q_half
// (shaders/flash.metal:71) and k_kv_quant_sym (shaders/flash.metal:157-178) of the reference.
//
// Memory-bound elementwise work: one CTA of 256 threads per (head slot, token, sequence), thread = head dimension,
// coalesced 1 KB row reads and writes. Arithmetic is written with explicit round-to-nearest intrinsics so that no
// multiply-add is contracted: the sums, the normalisation and the quantiser then round exactly as the scalar
// restatement does, and the int8 codes and scales are bit-exact.
#include "kata_internal.cuh"

namespace kata {

__constant__ float c_inv_freq[32];
void set_inv_freq(const float* host32) { cudaMemcpyToSymbol(c_inv_freq, host32, 32 * sizeof(float)); }

namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return __ldg(p); }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }

// sum over the 256 threads: xor butterfly inside each warp, then the 8 warp partials added in order
__device__ __forceinline__ float block_sum256(float v, float* part, int lane, int wid) {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, off));
    if (lane == 0) part[wid] = v;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int s = 0; s < 8; s++) tot = __fadd_rn(tot, part[s]);
    __syncthreads();
    return tot;
}
__device__ __forceinline__ float block_max256(float v, float* part, int lane, int wid) {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
    if (lane == 0) part[wid] = v;
    __syncthreads();
    float m = 0.0f;
#pragma unroll
    for (int s = 0; s < 8; s++) m = fmaxf(m, part[s]);
    __syncthreads();
    return m;
}

// symmetric int8 quantisation of one 256-wide head row held one value per thread (already rounded to fp16)
__device__ __forceinline__ void quant_store(__half hv, int8_t* dst_row, __half* sc_slot, int tid, int lane, int wid, float* part, int round_mode) {
    const float v = __half2float(hv);
    const float amax = block_max256(fabsf(v), part, lane, wid);
    const __half sc = amax > 0.0f ? __float2half_rn(__fdiv_rn(amax, 127.0f)) : __float2half_rn(1.0f);
    const float inv = __fdiv_rn(1.0f, __half2float(sc));
    const float x = __fmul_rn(v, inv);
    float r = round_mode == KATA_ROUND_HALF_AWAY ? roundf(x) : rintf(x);
    r = fminf(fmaxf(r, -127.0f), 127.0f);
    dst_row[tid] = (int8_t)(int)r;
    if (tid == 0) *sc_slot = sc;
}

template <typename TIn, bool INT8>
__global__ void __launch_bounds__(256) prep_kernel(const Batch b, const int T, const TIn* __restrict__ qfull, const TIn* __restrict__ kproj, const TIn* __restrict__ vproj,
                                                   const float* __restrict__ qnorm, const float* __restrict__ knorm, __half* __restrict__ q16, float* __restrict__ q32, float* __restrict__ gate,
                                                   void* k_arena, void* v_arena, __half* ksc, __half* vsc, const int h0, const int round_mode) {
    __shared__ float xs[256]; __shared__ float part[8];
    const int h = blockIdx.x + h0, t = blockIdx.y, bi = blockIdx.z, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int pos = b.pos[bi] + t; const int64_t row = b.row_base[bi] + pos; const int64_t tok = (int64_t)bi * T + t;
    if (h >= 28) {   // value head: fp16 copy (or quantise) into the cache row
        const int vh = h - 28; const __half hv = __float2half_rn(ldf(vproj + tok * kKVD + vh * kD + tid));
        if (!INT8) reinterpret_cast<__half*>(v_arena)[row * kKVD + vh * kD + tid] = hv;
        else quant_store(hv, reinterpret_cast<int8_t*>(v_arena) + row * kKVD + vh * kD, vsc + row * 4 + vh, tid, lane, wid, part, round_mode);
        return;
    }
    float v; const float* w;
    if (h < 24) { v = ldf(qfull + tok * kQFull + h * 512 + tid); if (gate) gate[tok * kQD + h * kD + tid] = ldf(qfull + tok * kQFull + h * 512 + 256 + tid); w = qnorm; }
    else { v = ldf(kproj + tok * kKVD + (h - 24) * kD + tid); w = knorm; }
    const float tot = block_sum256(__fmul_rn(v, v), part, lane, wid);
    const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, 256.0f), kEps)));
    const float x = __fmul_rn(__fmul_rn(v, r), __ldg(w + tid));
    xs[tid] = x;
    __syncthreads();
    float outv = x;
    if (tid < 64) {   // partial RoPE: pair (i, i+32); the angle is formed in fp32 from the shared inverse-frequency table
        const int i = tid & 31; const float theta = __fmul_rn((float)pos, c_inv_freq[i]);
        float s, c; sincosf(theta, &s, &c);
        const float a = xs[i], bb = xs[i + 32];
        outv = tid < 32 ? __fsub_rn(__fmul_rn(a, c), __fmul_rn(bb, s)) : __fadd_rn(__fmul_rn(a, s), __fmul_rn(bb, c));
    }
    if (h < 24) {
        if (q32) q32[tok * kQD + h * kD + tid] = outv;
        if (q16) q16[tok * kQD + h * kD + tid] = __float2half_rn(outv * 0.0625f);   // 1/sqrt(256), exact in fp16
    } else {
        const int kh = h - 24; const __half hv = __float2half_rn(outv);
        if (!INT8) reinterpret_cast<__half*>(k_arena)[row * kKVD + kh * kD + tid] = hv;
        else quant_store(hv, reinterpret_cast<int8_t*>(k_arena) + row * kKVD + kh * kD, ksc + row * 4 + kh, tid, lane, wid, part, round_mode);
    }
}

// grid (8, T): x < 4 key head x, else value head x-4 (the reference's k_kv_quant_sym launch shape)
__global__ void __launch_bounds__(256) kv_quant_kernel(const __half* __restrict__ ks, const __half* __restrict__ vs, int8_t* kq, int8_t* vq, __half* ksc, __half* vsc, const int64_t row0, const int round_mode) {
    __shared__ float part[8];
    const bool isV = blockIdx.x >= 4; const int head = blockIdx.x & 3, t = blockIdx.y, tid = threadIdx.x;
    const __half hv = (isV ? vs : ks)[(int64_t)t * kKVD + head * kD + tid]; const int64_t row = row0 + t;
    quant_store(hv, (isV ? vq : kq) + row * kKVD + head * kD, (isV ? vsc : ksc) + row * 4 + head, tid, tid & 31, tid >> 5, part, round_mode);
}

}  // namespace

cudaError_t launch_prep(Ctx& c, const Batch& b, int T, const void* qfull, const void* kproj, const void* vproj, int act_dtype,
                        const float* qnorm, const float* knorm, __half* q16, float* q32, float* gate, int h0, int nh, cudaStream_t s) {
    const dim3 grid(nh, T, b.n), block(256);
    const bool i8 = c.cfg.kv_mode == KATA_KV_INT8;
#define KATA_PREP(TIN, I8) prep_kernel<TIN, I8><<<grid, block, 0, s>>>(b, T, (const TIN*)qfull, (const TIN*)kproj, (const TIN*)vproj, qnorm, knorm, q16, q32, gate, c.k_arena, c.v_arena, c.ksc, c.vsc, h0, c.cfg.quant_round)
    if (act_dtype == KATA_ACT_F32) { if (i8) KATA_PREP(float, true); else KATA_PREP(float, false); }
    else { if (i8) KATA_PREP(__nv_bfloat16, true); else KATA_PREP(__nv_bfloat16, false); }
#undef KATA_PREP
    c.launches++;
    return cudaGetLastError();
}

cudaError_t launch_kv_quant(Ctx& c, int64_t row0, const __half* ks, const __half* vs, int T, cudaStream_t s) {
    kv_quant_kernel<<<dim3(8, T), 256, 0, s>>>(ks, vs, (int8_t*)c.k_arena, (int8_t*)c.v_arena, c.ksc, c.vsc, row0, c.cfg.quant_round);
    c.launches++;
    return cudaGetLastError();
}

}  // namespace kata
