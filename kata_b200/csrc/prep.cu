// Attention prep for the gated-GQA layers: per-head Q/K RMSNorm, partial RoPE on dims 0..63, gate split, append of the
// K and V rows to the cache, with the fp16 prescaled query and quantise-on-append (int8 planes: both in int8 mode, V only in int8v mode) fused in.
// Follows k_attn_prep / k_attn_prep_b (shaders/attn.metal:5-37, shaders/prefill.metal:179-206), k_cvt_q_half
// (shaders/flash.metal:71) and k_kv_quant_sym (shaders/flash.metal:157-178) of the reference.
//
// Memory-bound elementwise work: one warp per (head slot, token) row, eight rows per CTA, lane-strided (coalesced)
// accesses, shuffles only (no shared memory, no block barrier). Arithmetic is written with explicit round-to-nearest intrinsics so that no
// multiply-add is contracted: the sums, the normalisation and the quantiser then round exactly as the scalar
// restatement does, and the int8 codes and scales are bit-exact.
#include <algorithm>

#include "kata_internal.cuh"

namespace kata {

__constant__ float c_inv_freq[32];
void set_inv_freq(const float* host32) { cudaMemcpyToSymbol(c_inv_freq, host32, 32 * sizeof(float)); }

namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return __ldg(p); }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <> __device__ __forceinline__ float ldf<__half>(const __half* p) { return __half2float(*p); }

// One warp per (head slot, token) row. Lane j holds dims j, 32+j, ..., 224+j, so the sum of squares is formed exactly as
// the reference's threadgroup does it (an xor butterfly inside each group of 32 consecutive dims, then the 8 group sums
// added in order) and the RoPE pair (i, i+32) sits in one lane.
__device__ __forceinline__ float row_sum256(const float (&v)[8]) {
    float tot = 0.0f;
#pragma unroll
    for (int s = 0; s < 8; s++) {
        float x = v[s];
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) x = __fadd_rn(x, __shfl_xor_sync(0xffffffffu, x, off));
        tot = __fadd_rn(tot, x);
    }
    return tot;
}
__device__ __forceinline__ float row_max256(const float (&v)[8]) {
    float m = 0.0f;
#pragma unroll
    for (int s = 0; s < 8; s++) m = fmaxf(m, v[s]);
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
    return m;
}

// symmetric int8 quantisation of one 256-wide head row (values already rounded to fp16), lane j holding dims 32*s + j
__device__ __forceinline__ void quant_store_row(const __half (&hv)[8], int8_t* dst_row, __half* sc_slot, int lane, int round_mode) {
    float v[8], a[8];
#pragma unroll
    for (int s = 0; s < 8; s++) { v[s] = __half2float(hv[s]); a[s] = fabsf(v[s]); }
    const float amax = row_max256(a);
    const __half sc = amax > 0.0f ? __float2half_rn(__fdiv_rn(amax, 127.0f)) : __float2half_rn(1.0f);
    const float inv = __fdiv_rn(1.0f, __half2float(sc));
#pragma unroll
    for (int s = 0; s < 8; s++) {
        const float x = __fmul_rn(v[s], inv);
        float r = round_mode == KATA_ROUND_HALF_AWAY ? roundf(x) : rintf(x);
        r = fminf(fmaxf(r, -127.0f), 127.0f);
        dst_row[32 * s + lane] = (int8_t)(int)r;
    }
    if (lane == 0) *sc_slot = sc;
}

// The same per 64-dim group of the row (groups = register pairs (2g, 2g + 1) of every lane): four scales, sc4[g]. rint only.
__device__ __forceinline__ void quant_store_row_g4(const __half (&hv)[8], int8_t* dst_row, __half* sc4, int lane) {
#pragma unroll
    for (int g = 0; g < 4; g++) {
        const float v0 = __half2float(hv[2 * g]), v1 = __half2float(hv[2 * g + 1]);
        float amax = fmaxf(fabsf(v0), fabsf(v1));
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        const __half sc = amax > 0.0f ? __float2half_rn(__fdiv_rn(amax, 127.0f)) : __float2half_rn(1.0f);
        const float inv = __fdiv_rn(1.0f, __half2float(sc));
        dst_row[32 * (2 * g) + lane] = (int8_t)(int)fminf(fmaxf(rintf(__fmul_rn(v0, inv)), -127.0f), 127.0f);
        dst_row[32 * (2 * g + 1) + lane] = (int8_t)(int)fminf(fmaxf(rintf(__fmul_rn(v1, inv)), -127.0f), 127.0f);
        if (lane == 0) sc4[g] = sc;
    }
}

// grid (ceil(nh / 8), T, n) x 256 threads: warp w of a CTA handles head slot h0 + 8*blockIdx.x + w of one token
template <typename TIn, bool K8, bool V8, bool KG>
__global__ void __launch_bounds__(256) prep_kernel(const Batch b, const int T, const TIn* __restrict__ qfull, const TIn* __restrict__ kproj, const TIn* __restrict__ vproj,
                                                   const float* __restrict__ qnorm, const float* __restrict__ knorm, __half* __restrict__ q16, float* __restrict__ q32, float* __restrict__ gate,
                                                   void* k_arena, void* v_arena, __half* ksc, __half* vsc, const int h0, const int nh, const int round_mode, const int kvh_mask) {
    pdl_wait(); pdl_launch_dependents();   // launched with programmatic stream serialisation
    const int lane = threadIdx.x & 31, slot = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (slot >= nh) return;
    const int h = h0 + slot, t = blockIdx.y, bi = blockIdx.z;
    if (!((kvh_mask >> (h < 24 ? h / 6 : (h - 24) & 3)) & 1)) return;   // a head slot of a KV head this context does not own
    const int pos = b.pos[bi] + t; const int64_t row = b.row_base[bi] + pos; const int64_t tok = (int64_t)bi * T + t;
    if (h >= 28) {   // value head: fp16 copy (or quantise) into the cache row
        const int vh = h - 28; __half hv[8];
#pragma unroll
        for (int s = 0; s < 8; s++) hv[s] = __float2half_rn(ldf(vproj + tok * kKVD + vh * kD + 32 * s + lane));
        if (!V8) {
#pragma unroll
            for (int s = 0; s < 8; s++) reinterpret_cast<__half*>(v_arena)[row * kKVD + vh * kD + 32 * s + lane] = hv[s];
        } else quant_store_row(hv, reinterpret_cast<int8_t*>(v_arena) + row * kKVD + vh * kD, vsc + row * 4 + vh, lane, round_mode);
        return;
    }
    float v[8]; const float* w;
    if (h < 24) {
        const TIn* src = qfull + tok * kQFull + h * 512;
#pragma unroll
        for (int s = 0; s < 8; s++) v[s] = ldf(src + 32 * s + lane);
        if (gate) {
#pragma unroll
            for (int s = 0; s < 8; s++) gate[tok * kQD + h * kD + 32 * s + lane] = ldf(src + 256 + 32 * s + lane);
        }
        w = qnorm;
    } else {
        const TIn* src = kproj + tok * kKVD + (h - 24) * kD;
#pragma unroll
        for (int s = 0; s < 8; s++) v[s] = ldf(src + 32 * s + lane);
        w = knorm;
    }
    float sq[8];
#pragma unroll
    for (int s = 0; s < 8; s++) sq[s] = __fmul_rn(v[s], v[s]);
    const float tot = row_sum256(sq);
    const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, 256.0f), kEps)));
    float x[8];
#pragma unroll
    for (int s = 0; s < 8; s++) x[s] = __fmul_rn(__fmul_rn(v[s], r), __ldg(w + 32 * s + lane));
    {   // partial RoPE: pair (lane, lane + 32) = elements 0 and 1 of this lane; the angle is formed in fp32 from the shared table
        const float theta = __fmul_rn((float)pos, c_inv_freq[lane]);
        float sn, cs; sincosf(theta, &sn, &cs);
        const float a = x[0], bb = x[1];
        x[0] = __fsub_rn(__fmul_rn(a, cs), __fmul_rn(bb, sn)); x[1] = __fadd_rn(__fmul_rn(a, sn), __fmul_rn(bb, cs));
    }
    if (h < 24) {
#pragma unroll
        for (int s = 0; s < 8; s++) {
            if (q32) q32[tok * kQD + h * kD + 32 * s + lane] = x[s];
            if (q16) q16[tok * kQD + h * kD + 32 * s + lane] = __float2half_rn(x[s] * 0.0625f);   // 1/sqrt(256), exact in fp16
        }
    } else {
        const int kh = h - 24; __half hv[8];
#pragma unroll
        for (int s = 0; s < 8; s++) hv[s] = __float2half_rn(x[s]);
        if (!K8) {
#pragma unroll
            for (int s = 0; s < 8; s++) reinterpret_cast<__half*>(k_arena)[row * kKVD + kh * kD + 32 * s + lane] = hv[s];
        } else if (KG) quant_store_row_g4(hv, reinterpret_cast<int8_t*>(k_arena) + row * kKVD + kh * kD, ksc + row * 16 + kh * 4, lane);
        else quant_store_row(hv, reinterpret_cast<int8_t*>(k_arena) + row * kKVD + kh * kD, ksc + row * 4 + kh, lane, round_mode);
    }
}

// grid (T) x 256 threads: warp w < 4 key head w, else value head w-4 (the reference's k_kv_quant_sym covers the same 8 rows per token)
__global__ void __launch_bounds__(256) kv_quant_kernel(const __half* __restrict__ ks, const __half* __restrict__ vs, int8_t* kq, int8_t* vq, __half* ksc, __half* vsc, const int64_t row0, const int round_mode, const int kg) {
    const int lane = threadIdx.x & 31, wq = threadIdx.x >> 5, t = blockIdx.x; const bool isV = wq >= 4; const int head = wq & 3; const int64_t row = row0 + t;
    if (!isV && !kq) return;   // int8v: the key plane holds fp16 rows
    __half hv[8];
#pragma unroll
    for (int s = 0; s < 8; s++) hv[s] = (isV ? vs : ks)[(int64_t)t * kKVD + head * kD + 32 * s + lane];
    if (!isV && kg) quant_store_row_g4(hv, kq + row * kKVD + head * kD, ksc + row * 16 + head * 4, lane);   // four scales per key row
    else quant_store_row(hv, (isV ? vq : kq) + row * kKVD + head * kD, (isV ? vsc : ksc) + row * 4 + head, lane, round_mode);
}

// grid (width / 1024, rows) x 256 threads: element i = tid*4 + r of the block; bits 0-1 of i live in the thread's float4, bits 2-6 in the lane,
// bits 7-9 in the warp index, and the butterflies are taken in that order as fwht1024 does (shaders/common.h:22-42).
// A CTA walks rows of its column block kFwhtRows at a time and loads the next kFwhtRows while it works (16 bytes per thread and row in flight;
// with one row at a time and one ahead the kernel sat at 0.79 of the copy rate, with two at 0.85, with four at 0.88, with eight at 0.86); the third stage takes the rows in turn, 128 threads each.
constexpr int kFwhtRows = 4;
__global__ void __launch_bounds__(256) out_fwht_kernel(const float* __restrict__ x, const float* __restrict__ sign, float* __restrict__ out, const int width, const int64_t rows) {
    __shared__ float xs[kFwhtRows][1024];
    const int tid = threadIdx.x, lane = tid & 31;
    const float4 sg = *reinterpret_cast<const float4*>(sign + blockIdx.x * 1024 + tid * 4);
    const int64_t col = blockIdx.x * 1024 + tid * 4, step = gridDim.y;
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    auto load = [&](int64_t row) { return row < rows ? __ldcs(reinterpret_cast<const float4*>(x + row * width + col)) : zero; };   // read once: streaming load
    float4 nxt[kFwhtRows];
#pragma unroll
    for (int u = 0; u < kFwhtRows; u++) nxt[u] = load(blockIdx.y + u * step);
    for (int64_t row = blockIdx.y; row < rows; row += kFwhtRows * step) {
        float4 in[kFwhtRows];
#pragma unroll
        for (int u = 0; u < kFwhtRows; u++) { in[u] = nxt[u]; nxt[u] = load(row + (kFwhtRows + u) * step); }
#pragma unroll
        for (int u = 0; u < kFwhtRows; u++) {
            float v0 = __fmul_rn(in[u].x, sg.x), v1 = __fmul_rn(in[u].y, sg.y), v2 = __fmul_rn(in[u].z, sg.z), v3 = __fmul_rn(in[u].w, sg.w);
            { const float a = __fadd_rn(v0, v1), b = __fsub_rn(v0, v1), c = __fadd_rn(v2, v3), d = __fsub_rn(v2, v3); v0 = a; v1 = b; v2 = c; v3 = d; }
            { const float a = __fadd_rn(v0, v2), b = __fadd_rn(v1, v3), c = __fsub_rn(v0, v2), d = __fsub_rn(v1, v3); v0 = a; v1 = b; v2 = c; v3 = d; }
#pragma unroll
            for (int m = 1; m < 32; m <<= 1) {
                const float p0 = __shfl_xor_sync(0xffffffffu, v0, m), p1 = __shfl_xor_sync(0xffffffffu, v1, m), p2 = __shfl_xor_sync(0xffffffffu, v2, m), p3 = __shfl_xor_sync(0xffffffffu, v3, m);
                const bool up = lane & m;
                v0 = up ? __fsub_rn(p0, v0) : __fadd_rn(v0, p0); v1 = up ? __fsub_rn(p1, v1) : __fadd_rn(v1, p1);
                v2 = up ? __fsub_rn(p2, v2) : __fadd_rn(v2, p2); v3 = up ? __fsub_rn(p3, v3) : __fadd_rn(v3, p3);
            }
            *reinterpret_cast<float4*>(xs[u] + tid * 4) = make_float4(v0, v1, v2, v3);
        }
        __syncthreads();
#pragma unroll
        for (int u2 = 0; u2 < kFwhtRows / 2; u2++) {   // bits 7-9: threads 0-127 take row 2 * u2, threads 128-255 row 2 * u2 + 1
            float* xr = xs[2 * u2 + (tid >> 7)]; const int t7 = tid & 127;
            float e[8];
#pragma unroll
            for (int j = 0; j < 8; j++) e[j] = xr[t7 + 128 * j];
#pragma unroll
            for (int s = 0; s < 3; s++) {
                const int h = 1 << s;
#pragma unroll
                for (int j = 0; j < 8; j++) if (!(j & h)) { const float a = e[j], b = e[j | h]; e[j] = __fadd_rn(a, b); e[j | h] = __fsub_rn(a, b); }
            }
#pragma unroll
            for (int j = 0; j < 8; j++) xr[t7 + 128 * j] = e[j];
        }
        __syncthreads();
#pragma unroll
        for (int u = 0; u < kFwhtRows; u++) {
            const int64_t r_ = row + u * step;
            if (r_ < rows) {
                const float4 r = *reinterpret_cast<const float4*>(xs[u] + tid * 4);
                __stcs(reinterpret_cast<float4*>(out + r_ * width + col), make_float4(r.x * 0.03125f, r.y * 0.03125f, r.z * 0.03125f, r.w * 0.03125f));
            }
        }
        __syncthreads();   // xs is reused by the next rows
    }
}

}  // namespace

cudaError_t launch_out_fwht(const float* x, const float* sign, float* out, int64_t rows, int width, cudaStream_t s) {
    const int nb = width / 1024; const int per_sm = std::min(8, (227 * 1024) / (kFwhtRows * 4096 + 1024));   // CTAs of 256 threads an SM holds with kFwhtRows rows of shared memory each
    const unsigned gy = (unsigned)std::min<int64_t>(rows, std::max(1, 148 * per_sm / nb));
    out_fwht_kernel<<<dim3(nb, gy), 256, 0, s>>>(x, sign, out, width, rows);
    return cudaGetLastError();
}

cudaError_t launch_prep(Ctx& c, const Batch& b, int T, const void* qfull, const void* kproj, const void* vproj, int act_dtype,
                        const float* qnorm, const float* knorm, __half* q16, float* q32, float* gate, int h0, int nh, cudaStream_t s) {
    const dim3 grid((nh + 7) / 8, T, b.n), block(256);
    const int mode = c.cfg.kv_mode;
    cudaError_t le = cudaSuccess;
#define KATA_PREP(TIN, K8, V8) le = mode == KATA_KV_INT8G ? launch_pdl(prep_kernel<TIN, true, true, true>, grid, block, 0, s, b, T, (const TIN*)qfull, (const TIN*)kproj, (const TIN*)vproj, qnorm, knorm, q16, q32, gate, c.k_arena, c.v_arena, c.ksc, c.vsc, h0, nh, (int)c.cfg.quant_round, ((1 << c.kvh_n) - 1) << c.kvh_lo) : launch_pdl(prep_kernel<TIN, K8, V8, false>, grid, block, 0, s, b, T, (const TIN*)qfull, (const TIN*)kproj, (const TIN*)vproj, qnorm, knorm, q16, q32, gate, c.k_arena, c.v_arena, c.ksc, c.vsc, h0, nh, (int)c.cfg.quant_round, ((1 << c.kvh_n) - 1) << c.kvh_lo)
    if (act_dtype == KATA_ACT_F32) { if (mode == KATA_KV_INT8) KATA_PREP(float, true, true); else if (mode == KATA_KV_INT8V) KATA_PREP(float, false, true); else KATA_PREP(float, false, false); }
    else if (act_dtype == KATA_ACT_BF16) { if (mode == KATA_KV_INT8) KATA_PREP(__nv_bfloat16, true, true); else if (mode == KATA_KV_INT8V) KATA_PREP(__nv_bfloat16, false, true); else KATA_PREP(__nv_bfloat16, false, false); }
    else { if (mode == KATA_KV_INT8) KATA_PREP(__half, true, true); else if (mode == KATA_KV_INT8V) KATA_PREP(__half, false, true); else KATA_PREP(__half, false, false); }
#undef KATA_PREP
    if (le != cudaSuccess) return le;
    c.launches++;
    return cudaGetLastError();
}

cudaError_t launch_kv_quant(Ctx& c, int64_t row0, const __half* ks, const __half* vs, int T, cudaStream_t s) {
    kv_quant_kernel<<<dim3(T), 256, 0, s>>>(ks, vs, c.k8() ? (int8_t*)c.k_arena : nullptr, (int8_t*)c.v_arena, c.ksc, c.vsc, row0, c.cfg.quant_round, c.kg() ? 1 : 0);
    c.launches++;
    return cudaGetLastError();
}

}  // namespace kata
