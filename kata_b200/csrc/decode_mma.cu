// Split-KV decode / T<=2 speculative-verify attention over the fp16 or int8 KV cache, with the merge of the splits and
// the sigmoid output gate fused into the same kernel.
// Replaces k_dec_q_pack + k_attn_dec_split[_q8] + k_attn_dec_combine of the reference (shaders/flash.metal:77-152,
// host side Engine::dDecAttn, src/engine.cpp:119-127). Same math and rounding points: fp16 query prescaled by 1/16,
// rows of the 16-row block = 6 heads of one KV head x T tokens (row = t*6 + j), fp32 scores, P rounded to fp16 before
// P.V (after the V scale in int8 mode), l summed from the unrounded p, masked rows/keys at -inf, merge weights exp(m-M).
//
// Design (HBM-bound: 1 KiB of K+V per key and KV head at fp16, read exactly once):
//  - The work is the list of 16-key tiles of every (sequence, KV head) segment. It is cut into one contiguous,
//    equal-sized range per CTA (one CTA per SM), so ragged batches balance to within one tile and each key is read once.
//  - Inside a CTA each of the 4 warps owns every 4th tile of the range and streams it through its own 3-stage shared
//    memory ring: one 512-byte (fp16) or 256-byte (int8) bulk async copy per K or V row, issued one row per lane and
//    tracked by an mbarrier per stage. Rows are padded by 16 bytes so ldmatrix reads are bank-conflict free.
//  - Q.K^T and P.V run on mma.sync m16n8k16 (fp16 in, fp32 accumulate) straight from ldmatrix fragments; the softmax
//    state lives in registers and uses quad shuffles only. int8 rows are dequantised in registers (byte permute onto
//    the fp16 magic number 1024+x, then subtract), with the per-key scales applied to S and to P as the reference does.
//  - A CTA whose range ends inside a segment writes an unnormalised partial (O, m, l); the last CTA to finish a segment
//    (atomic ticket) merges the partials, normalises, applies the gate and writes the output row. No second kernel.
// Every mbarrier wait is bounded; on a timeout the kernel records an error word and skips the arithmetic.
#include <algorithm>

#include "attn_tile.cuh"

namespace kata {
namespace {

using namespace ptx;

constexpr int kWarps = 4, kThreads = kWarps * 32, kStages = 3, kTile = 16;
constexpr int kOffBars = 16 * kQStride;             // 8448
constexpr int kOffMl = kOffBars + 128;              // per-warp (m, l) exchange: [4][16][2] floats = 512 B
constexpr int kOffStages = kOffMl + 512;            // 9088, 16-byte aligned
constexpr int kMergeStride = 264;                   // floats per row of the cross-warp merge buffer

template <bool I8> struct Geo {
    static constexpr int kRowBytes = TileGeo<I8>::kRowBytes;
    static constexpr int kRowStride = TileGeo<I8>::kRowStride;
    static constexpr int kTileBytes = kTile * kRowStride;
    static constexpr int kStageBytes = 2 * kTileBytes;
    static constexpr int kWarpBytes = (kStages * kStageBytes > 16 * kMergeStride * 4) ? kStages * kStageBytes : 16 * kMergeStride * 4;
    static constexpr int kSmem = kOffStages + kWarps * kWarpBytes;
};

struct DecPlan {
    int32_t n, T, first_row, key_off, n_ctas, q_tiles, r_tiles;   // CTA c owns tiles [c*q + min(c,r), (c+1)*q + min(c+1,r))
    int32_t pos[KATA_MAX_BATCH];         // absolute position of token 0
    int32_t kend[KATA_MAX_BATCH];        // local rows [first_row, kend) hold this call's keys; absolute key = key_off + row
    int64_t row_base[KATA_MAX_BATCH];
    int32_t tile_start[KATA_MAX_BATCH + 1];
    int32_t ntiles[KATA_MAX_BATCH];      // tiles per KV head of sequence b (>= 1)
};

__device__ __forceinline__ int cta_first_tile(const DecPlan& p, int c) { return c * p.q_tiles + min(c, p.r_tiles); }
__device__ __forceinline__ int cta_of_tile(const DecPlan& p, int tile) {
    const int big = p.r_tiles * (p.q_tiles + 1);
    return tile < big ? tile / (p.q_tiles + 1) : p.r_tiles + (tile - big) / p.q_tiles;
}

template <bool I8>
__global__ void __launch_bounds__(kThreads, 1) decode_mma_kernel(const DecPlan p, const __half* __restrict__ q16, const float* __restrict__ gate, void* __restrict__ out, const int out_bf16,
                                                                 float* __restrict__ part_out, const uint8_t* __restrict__ k_arena, const uint8_t* __restrict__ v_arena,
                                                                 const __half* __restrict__ ksc, const __half* __restrict__ vsc,
                                                                 float* scratch_o, float* scratch_ml, int32_t* counters, int32_t* err) {
    using G = Geo<I8>;
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5, g = lane >> 2, t4 = lane & 3;
    const uint32_t sm_base = smem_u32(smem);
    const uint32_t q_base = sm_base, bars = sm_base + kOffBars + w * kStages * 8, my_stage0 = sm_base + kOffStages + w * G::kWarpBytes;
    float* sm_ml = reinterpret_cast<float*>(smem + kOffMl);
    __shared__ int s_flag;

    if (lane == 0) { for (int s = 0; s < kStages; s++) mbar_init(bars + s * 8, 1); }
    fence_mbar_init();
    __syncthreads();

    const int cta = blockIdx.x;
    int tile = cta_first_tile(p, cta); const int tile_end = cta_first_tile(p, cta + 1);
    int b = 0; uint32_t it = 0; bool dead = false;   // it: tiles this warp has issued so far (ring position and phase)

    while (tile < tile_end) {
        while (p.tile_start[b + 1] <= tile) b++;
        const int nt = p.ntiles[b], kvh = (tile - p.tile_start[b]) / nt, lt0 = (tile - p.tile_start[b]) - kvh * nt;
        const int seg_first = p.tile_start[b] + kvh * nt, seg_end = seg_first + nt, my_end = min(tile_end, seg_end), n_here = my_end - tile;
        const int T = p.T, kend = p.kend[b], pos_rel = p.pos[b] - p.key_off;   // token t sees local rows < min(kend, pos_rel + t + 1)
        const uint8_t* Kg = k_arena + (p.row_base[b] * kKVD + kvh * kD) * (I8 ? 1 : 2);
        const uint8_t* Vg = v_arena + (p.row_base[b] * kKVD + kvh * kD) * (I8 ? 1 : 2);

        // ---- stage the 16-row Q block (rows t*6+j; rows >= 6T zero). int8: columns permuted inside each 16-dim block to
        // match the contraction order of the dequantised K fragments (logical c<8 -> dim 4*(c/2)+c%2, else 4*((c-8)/2)+2+c%2).
        for (int ch = tid; ch < 16 * 32; ch += kThreads) {
            const int r = ch >> 5, c16 = ch & 31; uint4 v = make_uint4(0, 0, 0, 0);
            if (r < 6 * T) { const int t = r / 6, j = r - 6 * t; v = *reinterpret_cast<const uint4*>(q16 + ((int64_t)b * T + t) * kQD + (kvh * 6 + j) * kD + c16 * 8); }
            stage_q_chunk<I8>(smem + r * kQStride, c16, v);
        }
        __syncthreads();

        // ---- this warp's tiles of the segment: local tiles lt0 + w, lt0 + w + 4, ...
        const int n_mine = n_here > w ? (n_here - w + kWarps - 1) / kWarps : 0;
        RowState st; st.clear();
        const int lim_row0 = (g < 6 * T) ? min(kend, pos_rel + (g >= 6 ? 1 : 0) + 1) : 0;          // rows g and g+8: exclusive local key limit
        const int lim_row1 = (g + 8 < 6 * T) ? min(kend, pos_rel + ((g + 8) >= 6 ? 1 : 0) + 1) : 0;

        int n_issued = 0, n_waited = 0;
        auto issue = [&](int i) {   // bring in this warp's i-th tile of the segment
            if (dead) return;
            n_issued = i + 1;
            const int key0 = p.first_row + (lt0 + w + i * kWarps) * kTile, nk = max(0, min(kTile, kend - key0));
            const uint32_t sx = (it + (uint32_t)i) % kStages, dst = my_stage0 + sx * G::kStageBytes, bar = bars + sx * 8;
            fence_proxy_async();
            if (lane == 0) mbar_arrive_expect_tx(bar, (uint32_t)(nk * 2 * G::kRowBytes));
            __syncwarp();
            const int r = lane & 15; const bool isv = lane >= 16;
            if (r < nk) bulk_g2s(dst + (isv ? G::kTileBytes : 0) + r * G::kRowStride, (isv ? Vg : Kg) + (int64_t)(key0 + r) * (kKVD * (I8 ? 1 : 2)), G::kRowBytes, bar);
            else if (isv) { uint4* z = reinterpret_cast<uint4*>(smem + (dst - sm_base) + G::kTileBytes + r * G::kRowStride); for (int c = 0; c < G::kRowBytes / 16; c++) z[c] = make_uint4(0, 0, 0, 0); }
        };

        const uint32_t it_seg = it;
        for (int i = 0; i < min(kStages - 1, n_mine); i++) issue(i);
        for (int i = 0; i < n_mine; i++) {
            __syncwarp();
            if (i + kStages - 1 < n_mine) issue(i + kStages - 1);
            const uint32_t cur = it_seg + (uint32_t)i, stg = cur % kStages, par = (cur / kStages) & 1u;
            const uint32_t kt = my_stage0 + stg * G::kStageBytes, vt = kt + G::kTileBytes;
            const int key0 = p.first_row + (lt0 + w + i * kWarps) * kTile;
            float ks_[2][2] = {{1.f, 1.f}, {1.f, 1.f}}, vs_[2][2] = {{1.f, 1.f}, {1.f, 1.f}};
            if (I8) {   // per-key scales of this thread's four score columns (keys key0 + nt*8 + 2*t4 + e)
#pragma unroll
                for (int ntl = 0; ntl < 2; ntl++)
#pragma unroll
                    for (int e = 0; e < 2; e++) { const int key = min(key0 + ntl * 8 + 2 * t4 + e, max(kend - 1, 0)); ks_[ntl][e] = __half2float(ksc[(p.row_base[b] + key) * 4 + kvh]); vs_[ntl][e] = __half2float(vsc[(p.row_base[b] + key) * 4 + kvh]); }
            }
            if (dead) continue;
            if (!mbar_wait_bounded(bars + stg * 8, par)) { dead = true; atomicExch(err, 1); continue; }
            n_waited = i + 1;
            tile_qk_softmax_pv<I8>(q_base, kt, vt, key0, lim_row0, lim_row1, ks_, vs_, st, lane);
        }
        if (dead) {   // give copies already in flight a bounded chance to land before this CTA's shared memory is reused or released
            for (int x = n_waited + 1; x < n_issued; x++) { const uint32_t cur = it_seg + (uint32_t)x; mbar_wait_bounded(bars + (cur % kStages) * 8, (cur / kStages) & 1u, 1u << 16); }
        }
        it = it_seg + (uint32_t)n_mine;

        // ---- merge the 4 warps of the CTA (all copies of this segment have landed: every issued tile was waited for)
        st.finish_l();
        __syncwarp();
        float* mo = reinterpret_cast<float*>(smem + kOffStages + w * G::kWarpBytes);
#pragma unroll
        for (int j = 0; j < 32; j++)
#pragma unroll
            for (int c = 0; c < 2; c++) { const int d = dim_of<I8>(j, c, t4); mo[g * kMergeStride + d] = st.o[j][c]; mo[(g + 8) * kMergeStride + d] = st.o[j][2 + c]; }
        if (t4 == 0) { sm_ml[(w * 16 + g) * 2] = st.m0; sm_ml[(w * 16 + g) * 2 + 1] = st.l0; sm_ml[(w * 16 + g + 8) * 2] = st.m1; sm_ml[(w * 16 + g + 8) * 2 + 1] = st.l1; }
        __syncthreads();

        const int seg = b * 4 + kvh, c_first = cta_of_tile(p, seg_first), c_last = cta_of_tile(p, seg_end - 1), n_contrib = c_last - c_first + 1;
        const int d0 = 2 * tid;   // this thread merges dims d0, d0+1 of every live row
        const bool whole = (n_contrib == 1);
        float* slot_o = scratch_o + (int64_t)(cta + seg) * (12 * kD); float* slot_ml = scratch_ml + (int64_t)(cta + seg) * 32;
        for (int r = 0; r < 6 * T; r++) {
            float M = -INFINITY;
#pragma unroll
            for (int ww = 0; ww < kWarps; ww++) M = fmaxf(M, sm_ml[(ww * 16 + r) * 2]);
            float L = 0.0f, A0 = 0.0f, A1 = 0.0f;
#pragma unroll
            for (int ww = 0; ww < kWarps; ww++) {
                const float mm = sm_ml[(ww * 16 + r) * 2]; const float wt = (mm == -INFINITY) ? 0.0f : ex2(mm - M);
                const float* src = reinterpret_cast<const float*>(smem + kOffStages + ww * G::kWarpBytes) + r * kMergeStride + d0;
                L += sm_ml[(ww * 16 + r) * 2 + 1] * wt; A0 += src[0] * wt; A1 += src[1] * wt;
            }
            if (whole) {
                const int t = r / 6, j = r - 6 * t, head = kvh * 6 + j;
                if (part_out) { float* po = part_out + ((int64_t)(b * T + t) * kH + head) * kPartStride; po[d0] = A0; po[d0 + 1] = A1; if (tid == 0) { po[256] = M * 0.6931471805599453f; po[257] = L; } }
                else {
                    const int64_t oi = ((int64_t)b * T + t) * kQD + head * kD + d0; const float2 gt = *reinterpret_cast<const float2*>(gate + oi);
                    const float y0 = (A0 / L) * (1.0f / (1.0f + __expf(-gt.x))), y1 = (A1 / L) * (1.0f / (1.0f + __expf(-gt.y)));
                    if (out_bf16) reinterpret_cast<__nv_bfloat162*>(out)[oi >> 1] = __floats2bfloat162_rn(y0, y1); else *reinterpret_cast<float2*>(reinterpret_cast<float*>(out) + oi) = make_float2(y0, y1);
                }
            } else {
                *reinterpret_cast<float2*>(slot_o + r * kD + d0) = make_float2(A0, A1);
                if (tid == 0) { slot_ml[r * 2] = M; slot_ml[r * 2 + 1] = L; }
            }
        }
        if (!whole) {   // ticket: the last contributor of the segment merges everybody's partials
            __threadfence();
            __syncthreads();
            if (tid == 0) { const int old = atomicAdd(&counters[seg], 1); s_flag = (old == n_contrib - 1); }
            __syncthreads();
            if (s_flag) {
                __threadfence();
                for (int r = 0; r < 6 * T; r++) {
                    float M = -INFINITY;
                    for (int c = c_first; c <= c_last; c++) M = fmaxf(M, __ldcg(scratch_ml + (int64_t)(c + seg) * 32 + r * 2));
                    float L = 0.0f, A0 = 0.0f, A1 = 0.0f;
                    for (int c = c_first; c <= c_last; c++) {
                        const float mm = __ldcg(scratch_ml + (int64_t)(c + seg) * 32 + r * 2); const float wt = (mm == -INFINITY) ? 0.0f : ex2(mm - M);
                        const float2 a = __ldcg(reinterpret_cast<const float2*>(scratch_o + (int64_t)(c + seg) * (12 * kD) + r * kD + d0));
                        L += __ldcg(scratch_ml + (int64_t)(c + seg) * 32 + r * 2 + 1) * wt; A0 += a.x * wt; A1 += a.y * wt;
                    }
                    const int t = r / 6, j = r - 6 * t, head = kvh * 6 + j;
                    if (part_out) { float* po = part_out + ((int64_t)(b * T + t) * kH + head) * kPartStride; po[d0] = A0; po[d0 + 1] = A1; if (tid == 0) { po[256] = M * 0.6931471805599453f; po[257] = L; } }
                    else {
                        const int64_t oi = ((int64_t)b * T + t) * kQD + head * kD + d0; const float2 gt = *reinterpret_cast<const float2*>(gate + oi);
                        const float y0 = (A0 / L) * (1.0f / (1.0f + __expf(-gt.x))), y1 = (A1 / L) * (1.0f / (1.0f + __expf(-gt.y)));
                        if (out_bf16) reinterpret_cast<__nv_bfloat162*>(out)[oi >> 1] = __floats2bfloat162_rn(y0, y1); else *reinterpret_cast<float2*>(reinterpret_cast<float*>(out) + oi) = make_float2(y0, y1);
                    }
                }
                if (tid == 0) counters[seg] = 0;   // ready for the next call on this stream
            }
        }
        __syncthreads();   // merge buffers and the Q block are reused by the next segment
        tile = my_end;
    }
}

// Merge of per-rank partials {O[256], m, l} (m in natural-log units) and the output gate: k_attn_dec_combine with "split" = rank.
__global__ void __launch_bounds__(256) merge_parts_kernel(const float* __restrict__ parts, const int n_parts, const int T, const float* __restrict__ gate, void* __restrict__ out, const int out_bf16) {
    const int h = blockIdx.x, t = blockIdx.y, tid = threadIdx.x; const int64_t row = (int64_t)t * kH + h, stride = (int64_t)T * kH * kPartStride;
    float M = -INFINITY; for (int r = 0; r < n_parts; r++) M = fmaxf(M, parts[r * stride + row * kPartStride + 256]);
    float L = 0.0f, A = 0.0f;
    for (int r = 0; r < n_parts; r++) { const float* pp = parts + r * stride + row * kPartStride; const float mm = pp[256]; const float wt = (mm == -INFINITY) ? 0.0f : expf(mm - M); L += pp[257] * wt; A += pp[tid] * wt; }
    const int64_t oi = (int64_t)t * kQD + h * kD + tid; const float y = (A / L) * (1.0f / (1.0f + expf(-gate[oi])));
    if (out_bf16) reinterpret_cast<__nv_bfloat16*>(out)[oi] = __float2bfloat16_rn(y); else reinterpret_cast<float*>(out)[oi] = y;
}

}  // namespace

int decode_max_slots(int sm_count) { return sm_count + 4 * KATA_MAX_BATCH; }

// key_off / kend_override serve the split-KV-across-GPUs call: local row = absolute key - key_off, rows [first_row, kend).
cudaError_t launch_decode_mma_ex(Ctx& c, const Batch& b, int T, int first_row, int key_off, const int32_t* kend_override, const __half* q16, const float* gate, void* out, int out_dtype,
                                 float* part_out, cudaStream_t s) {
    static bool attr_set[2] = {false, false};
    DecPlan p{}; p.n = b.n; p.T = T; p.first_row = first_row; p.key_off = key_off;
    int total = 0;
    for (int i = 0; i < b.n; i++) {
        p.pos[i] = b.pos[i]; p.row_base[i] = b.row_base[i]; p.kend[i] = kend_override ? kend_override[i] : b.pos[i] + T;
        const int nkeys = std::max(0, p.kend[i] - first_row); p.ntiles[i] = std::max(1, (nkeys + kTile - 1) / kTile);
        p.tile_start[i] = total; total += 4 * p.ntiles[i];
    }
    for (int i = b.n; i <= KATA_MAX_BATCH; i++) p.tile_start[i] = total;
    const int chunk_tiles = c.cfg.dec_chunk > 0 ? std::max(1, c.cfg.dec_chunk / kTile) : 0;
    int n_ctas = chunk_tiles ? (total + chunk_tiles - 1) / chunk_tiles : c.sm_count;
    n_ctas = std::max(1, std::min(std::min(n_ctas, total), c.sm_count * 8));
    if (n_ctas + 4 * b.n > c.max_items) n_ctas = c.max_items - 4 * b.n;
    p.n_ctas = n_ctas; p.q_tiles = total / n_ctas; p.r_tiles = total % n_ctas;
    const bool i8 = c.cfg.kv_mode == KATA_KV_INT8;
    if (!attr_set[i8]) {
        cudaError_t e = i8 ? cudaFuncSetAttribute(decode_mma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, Geo<true>::kSmem)
                           : cudaFuncSetAttribute(decode_mma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, Geo<false>::kSmem);
        if (e != cudaSuccess) return e;
        attr_set[i8] = true;
    }
    if (i8) decode_mma_kernel<true><<<n_ctas, kThreads, Geo<true>::kSmem, s>>>(p, q16, gate, out, out_dtype == KATA_ACT_BF16, part_out, (const uint8_t*)c.k_arena, (const uint8_t*)c.v_arena, c.ksc, c.vsc, c.part_o, c.part_ml, c.counters, c.d_err);
    else decode_mma_kernel<false><<<n_ctas, kThreads, Geo<false>::kSmem, s>>>(p, q16, gate, out, out_dtype == KATA_ACT_BF16, part_out, (const uint8_t*)c.k_arena, (const uint8_t*)c.v_arena, c.ksc, c.vsc, c.part_o, c.part_ml, c.counters, c.d_err);
    c.launches++;
    return cudaGetLastError();
}

cudaError_t launch_decode_mma(Ctx& c, const Batch& b, int T, int first_pos, int, const __half* q16, const float* gate, void* out, int out_dtype, float* part_out, cudaStream_t s) {
    return launch_decode_mma_ex(c, b, T, first_pos, 0, nullptr, q16, gate, out, out_dtype, part_out, s);
}

cudaError_t launch_merge_parts(Ctx& c, const float* parts, int n_parts, int T, const float* gate, void* out, int out_dtype, cudaStream_t s) {
    merge_parts_kernel<<<dim3(kH, T), 256, 0, s>>>(parts, n_parts, T, gate, out, out_dtype == KATA_ACT_BF16);
    c.launches++;
    return cudaGetLastError();
}

}  // namespace kata
