// Causal flash prefill on mma.sync tiles: the first, simple prefill path (64 query rows of one head per CTA, 32-key
// K/V tiles double-buffered with cp.async, the per-warp 16x16 tile routine shared with the decode kernel).
// Replaces k_flash_prefill / k_flash_prefill_q8 / k_flash_prefill_k16v8 of the reference (shaders/flash.metal:10-68, 198-250; encoded at
// src/engine.cpp:279, 614): query row r of the chunk sits at position pos_base + r and attends keys [0, pos_base + r]
// of the cache prefix; output = O / l * sigmoid(gate). Chunked prefill over a restored or earlier-computed prefix is
// the same call with pos_base > 0.
#include <algorithm>

#include "attn_tile.cuh"

namespace kata {
namespace {

using namespace ptx;

constexpr int kPfWarps = 4, kPfThreads = kPfWarps * 32, kBM = 16 * kPfWarps, kBN = 32;

template <bool K8, bool V8> struct PfGeo {   // K8 / V8: the K / V plane holds int8 codes
    static constexpr int kKStride = TileGeo<K8>::kRowStride, kVStride = TileGeo<V8>::kRowStride;
    static constexpr int kKChunks = TileGeo<K8>::kRowBytes / 16, kVChunks = TileGeo<V8>::kRowBytes / 16;   // 16-byte chunks per K / V row
    static constexpr int kKTileBytes = kBN * kKStride, kVTileBytes = kBN * kVStride;                     // K and V part of a stage
    static constexpr int kStageBytes = kKTileBytes + kVTileBytes;
    static constexpr int kOffStages = kBM * kQStride;
    static constexpr int kSmem = kOffStages + 2 * kStageBytes;
};

template <bool K8, bool V8>
__global__ void __launch_bounds__(kPfThreads, 2) prefill_mma_kernel(const Batch b, const int M, const __half* __restrict__ q16, const float* __restrict__ gate, void* __restrict__ out, const int out_kind,
                                                                    const uint8_t* __restrict__ k_arena, const uint8_t* __restrict__ v_arena, const __half* __restrict__ ksc, const __half* __restrict__ vsc) {
    using G = PfGeo<K8, V8>;
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5, g = lane >> 2, t4 = lane & 3;
    const int qt = gridDim.x - 1 - blockIdx.x, h = blockIdx.y, bi = blockIdx.z, kvh = h / kG;   // the longest (latest) query tiles start first
    const int q0 = qt * kBM, rows_valid = min(kBM, M - q0), pos_base = b.pos[bi], kend = pos_base + q0 + rows_valid, n_tiles = (kend + kBN - 1) / kBN;
    const uint32_t sm_base = smem_u32(smem);
    constexpr int kEltK = K8 ? 1 : 2, kEltV = V8 ? 1 : 2;
    const uint8_t* Kg = k_arena + (b.row_base[bi] * kKVD + kvh * kD) * kEltK; const uint8_t* Vg = v_arena + (b.row_base[bi] * kKVD + kvh * kD) * kEltV;

    for (int ch = tid; ch < kBM * 32; ch += kPfThreads) {
        const int r = ch >> 5, c16 = ch & 31; uint4 v = make_uint4(0, 0, 0, 0);
        if (r < rows_valid) v = *reinterpret_cast<const uint4*>(q16 + ((int64_t)bi * M + q0 + r) * kQD + h * kD + c16 * 8);
        stage_q_chunk<K8>(smem + r * kQStride, c16, v);
    }
    auto load_tile = [&](int kt, int buf) {
        const uint32_t dst0 = sm_base + G::kOffStages + buf * G::kStageBytes;
        for (int idx = tid; idx < kBN * G::kKChunks; idx += kPfThreads) {
            const int r = idx / G::kKChunks, c = idx - r * G::kKChunks, key = kt * kBN + r; const bool ok = key < kend;
            cp_async16(dst0 + r * G::kKStride + c * 16, Kg + (int64_t)(ok ? key : 0) * (kKVD * kEltK) + c * 16, ok ? 16u : 0u);   // rows past the range arrive as zeros
        }
        for (int idx = tid; idx < kBN * G::kVChunks; idx += kPfThreads) {
            const int r = idx / G::kVChunks, c = idx - r * G::kVChunks, key = kt * kBN + r; const bool ok = key < kend;
            cp_async16(dst0 + G::kKTileBytes + r * G::kVStride + c * 16, Vg + (int64_t)(ok ? key : 0) * (kKVD * kEltV) + c * 16, ok ? 16u : 0u);
        }
    };
    const int row0 = q0 + 16 * w + g, row1 = row0 + 8;
    const int lim0 = row0 < M ? pos_base + row0 + 1 : 0, lim1 = row1 < M ? pos_base + row1 + 1 : 0;
    const int warp_lim = pos_base + min(q0 + 16 * w + 16, M);   // no row of this warp sees keys >= warp_lim
    RowState st; st.clear();
    const uint32_t q_sm = sm_base + (16 * w) * kQStride;

    load_tile(0, 0); cp_async_commit();
    for (int kt = 0; kt < n_tiles; kt++) {
        if (kt + 1 < n_tiles) load_tile(kt + 1, (kt + 1) & 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const uint32_t kbuf = sm_base + G::kOffStages + (kt & 1) * G::kStageBytes, vbuf = kbuf + G::kKTileBytes;
#pragma unroll 1
        for (int sub = 0; sub < kBN / 16; sub++) {
            const int key0 = kt * kBN + sub * 16;
            if (key0 >= warp_lim) break;
            float ks_[2][2] = {{1.f, 1.f}, {1.f, 1.f}}, vs_[2][2] = {{1.f, 1.f}, {1.f, 1.f}};
            if (V8) {
#pragma unroll
                for (int nt = 0; nt < 2; nt++)
#pragma unroll
                    for (int e = 0; e < 2; e++) { const int key = min(key0 + nt * 8 + 2 * t4 + e, kend - 1); if (K8) ks_[nt][e] = __half2float(ksc[(b.row_base[bi] + key) * 4 + kvh]); vs_[nt][e] = __half2float(vsc[(b.row_base[bi] + key) * 4 + kvh]); }
            }
            tile_qk_softmax_pv<K8, V8>(q_sm, kbuf + sub * 16 * G::kKStride, vbuf + sub * 16 * G::kVStride, key0, lim0, lim1, ks_, vs_, st, lane);
        }
        __syncthreads();
    }
    st.finish_l();
    const float inv0 = 1.0f / st.l0, inv1 = 1.0f / st.l1;
#pragma unroll
    for (int j = 0; j < 32; j++) {
#pragma unroll
        for (int half = 0; half < 2; half++) {
            const int row = half ? row1 : row0; if (row >= M) continue;
            const float inv = half ? inv1 : inv0; const int64_t base = ((int64_t)bi * M + row) * kQD + h * kD;
            if (!V8) {
                const int d = dim_of<false>(j, 0, t4); const float2 gt = *reinterpret_cast<const float2*>(gate + base + d);
                const float y0 = st.o[j][2 * half] * inv * sigmoid_fast(gt.x), y1 = st.o[j][2 * half + 1] * inv * sigmoid_fast(gt.y);
                store_act2(out, base + d, y0, y1, out_kind);
            } else {
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    const int d = dim_of<true>(j, c, t4); const float y = st.o[j][2 * half + c] * inv * sigmoid_fast(gate[base + d]);
                    store_act(out, base + d, y, out_kind);
                }
            }
        }
    }
}

}  // namespace

cudaError_t configure_prefill_mma(int kv_mode) {   // per device, once per context
    return kv_mode == KATA_KV_INT8  ? cudaFuncSetAttribute(prefill_mma_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, PfGeo<true, true>::kSmem)
         : kv_mode == KATA_KV_INT8V ? cudaFuncSetAttribute(prefill_mma_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, PfGeo<false, true>::kSmem)
                                    : cudaFuncSetAttribute(prefill_mma_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, PfGeo<false, false>::kSmem);
}

cudaError_t launch_prefill_mma(Ctx& c, const Batch& b, int M, const __half* q16, const float* gate, void* out, int out_dtype, cudaStream_t s) {
    const dim3 grid((M + kBM - 1) / kBM, kH, b.n);
#define KATA_PFM(K8, V8) prefill_mma_kernel<K8, V8><<<grid, kPfThreads, PfGeo<K8, V8>::kSmem, s>>>(b, M, q16, gate, out, out_dtype, (const uint8_t*)c.k_arena, (const uint8_t*)c.v_arena, c.ksc, c.vsc)
    if (c.cfg.kv_mode == KATA_KV_INT8) KATA_PFM(true, true); else if (c.cfg.kv_mode == KATA_KV_INT8V) KATA_PFM(false, true); else KATA_PFM(false, false);
#undef KATA_PFM
    c.launches++;
    return cudaGetLastError();
}

}  // namespace kata
