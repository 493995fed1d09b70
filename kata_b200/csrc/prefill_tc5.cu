// Causal flash prefill on the 5th-generation tensor cores (tcgen05) for the fp16 KV cache.
// Replaces k_cvt_q_half + k_flash_prefill of the reference (shaders/flash.metal:10-71; encoded at src/engine.cpp:279,
// 614) with the same math: fp16 Q (prescaled by 1/16) x fp16 K -> fp32 scores, causal mask key > position -> -inf,
// online softmax, P rounded to fp16 before P.V, l summed from the unrounded p, output O / l * sigmoid(gate).
//
// One CTA = 128 query rows of one head (row r of the chunk sits at position pos_base + r and sees keys [0, pos_base + r]).
//   warps 0-7  softmax: two threads per query row (tensor-memory lane = row): warp w < 4 takes the first 64 keys of a tile, warp w + 4
//              the last 64; the pair exchanges its row maxima through shared memory (64-thread named barrier) once per tile, each
//              writes its half of P, keeps its own partial l, and owns 128 of the 256 O columns for rescales and the epilogue
//   warp 8     TMA producer for Q (once) and the K tiles;  warp 9  TMA producer for the V tiles
//   warp 10    issues the MMAs (one elected thread)
// Shared memory: Q, one K tile and one V tile of 128 keys, each 4 column blocks of [128 rows][128 bytes] with the
// 128-byte swizzle, exactly as TMA writes them and as the MMA descriptors read them (Q, K: K-major; V: MN-major, so the
// [key][dim] rows of the cache are used as they lie). Tensor memory (512 columns): O 128x256 fp32 in columns [0,256),
// two score buffers S0, S1 of 128x128 fp32 in [256,384) and [384,512); P (fp16, two per column) overwrites the first 64
// columns of its S buffer and is the tensor-memory A operand of P.V.
// Pipeline: the MMA thread issues S(j+1) = Q.K(j+1)^T before P(j).V(j), so the tensor pipe computes the next scores while
// the softmax warps work on the current ones; K(j+1) is loaded as soon as S(j) has completed, V(j+1) as soon as P(j).V(j)
// has. The running maximum is only raised when a row's new maximum exceeds it by more than 8 (in log2 units); then the
// whole warp rescales its O rows in tensor memory after waiting for the previous P.V. P stays below 2^8, well inside fp16.
// Every wait is bounded and shares the context's abort word; tensor memory is always released before the CTA exits.
#include <algorithm>

#include "kata_internal.cuh"
#include "ptx.cuh"
#include "tc5.cuh"

namespace kata {
namespace {

using namespace ptx;

constexpr int kTcThreads = 352, kBMq = 128, kBNk = 128;
constexpr int kBlk = 128 * 128;                  // one column block: 128 rows x 128 bytes
constexpr int kTileB = 4 * kBlk;                 // 64 KB: a 128 x 256 fp16 tile
constexpr int kSmemTc = 3 * kTileB + 1024 + 256; // Q, K, V + alignment slack + barriers
constexpr uint32_t kIdescS = tc5::idesc_f16(128, 128, false), kIdescPV = tc5::idesc_f16(128, 256, true);

// barrier slots (8 bytes each) after the tiles
enum { B_QFULL = 0, B_KFULL, B_KEMPTY, B_VFULL, B_VEMPTY, B_SFULL0, B_SFULL1, B_PREADY0, B_PREADY1, B_ODONE, B_COUNT };

__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, const int32_t* abort_flag) {   // same outcome for every lane of the warp
    const bool ok = mbar_wait_bounded(bar, parity, abort_flag);
    return __all_sync(0xffffffffu, ok);
}

__global__ void __launch_bounds__(kTcThreads, 1) prefill_tc5_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                                                                   const Batch b, const int M, const float* __restrict__ gate, void* __restrict__ out, const int out_bf16, int32_t* err) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const int qt = gridDim.x - 1 - blockIdx.x, h = blockIdx.y, bi = blockIdx.z, kvh = h / kG;   // longest query tiles first
    const int q0 = qt * kBMq, rows_valid = min(kBMq, M - q0), pos_base = b.pos[bi], kend = pos_base + q0 + rows_valid, n_tiles = (kend + kBNk - 1) / kBNk;
    const int row0 = (int)b.row_base[bi];
    const uint32_t sm0 = smem_u32(smem_raw), base = (sm0 + 1023u) & ~1023u;
    const uint32_t q_sm = base, k_sm = base + kTileB, v_sm = base + 2 * kTileB, bars = base + 3 * kTileB;
    uint8_t* v_gen = smem_raw + (v_sm - sm0);
    __shared__ uint32_t s_tmem; __shared__ float s_xmax[2][2][128];   // [tile parity][key half][row]: row maxima (and at the end the partial l) exchanged by the two threads of a row
    auto bar = [&](int i) { return bars + 8u * (uint32_t)i; };

    if (tid == 0) {
        for (int i = 0; i < B_COUNT; i++) mbar_init(bar(i), (i == B_PREADY0 || i == B_PREADY1) ? 256u : 1u);
        fence_mbar_init();
    }
    if (w == 0) tc5::tmem_alloc(smem_u32(&s_tmem), 512);
    tc5::fence_before_sync();
    __syncthreads();
    tc5::fence_after_sync();
    const uint32_t tmem = s_tmem, t_o = tmem, t_s0 = tmem + 256;

    if (w == 8) {
        // ---- Q once, then K tiles: K(j) may overwrite the buffer when S(j-1) has completed
        if (lane == 0) {
            mbar_arrive_expect_tx(bar(B_QFULL), kTileB);
            for (int kb = 0; kb < 4; kb++) tma_load_2d(q_sm + kb * kBlk, &tm_q, h * kD + kb * 64, bi * M + q0, bar(B_QFULL));
            for (int j = 0; j < n_tiles; j++) {
                if (j >= 1 && !mbar_wait_bounded(bar(B_KEMPTY), (uint32_t)(j - 1) & 1u, err)) { atomicExch(err, 11); break; }
                mbar_arrive_expect_tx(bar(B_KFULL), kTileB);
                for (int kb = 0; kb < 4; kb++) tma_load_3d(k_sm + kb * kBlk, &tm_k, kb * 64, kvh, row0 + j * kBNk, bar(B_KFULL));
            }
        }
    } else if (w == 9) {
        if (lane == 0) {
            for (int j = 0; j < n_tiles; j++) {
                if (j >= 1 && !mbar_wait_bounded(bar(B_VEMPTY), (uint32_t)(j - 1) & 1u, err)) { atomicExch(err, 12); break; }
                mbar_arrive_expect_tx(bar(B_VFULL), kTileB);
                for (int kb = 0; kb < 4; kb++) tma_load_3d(v_sm + kb * kBlk, &tm_v, kb * 64, kvh, row0 + j * kBNk, bar(B_VFULL));
            }
        }
    } else if (w == 10) {
        if (lane == 0) {
            auto issue_s = [&](int j) {   // S(j) = Q K(j)^T: 4 column blocks x 4 k-steps of 16 dims
                const uint32_t d = t_s0 + (uint32_t)(j & 1) * 128u;
#pragma unroll
                for (int kb = 0; kb < 4; kb++)
#pragma unroll
                    for (int ks = 0; ks < 4; ks++)
                        tc5::mma_ss(d, tc5::smem_desc_sw128(q_sm + kb * kBlk + ks * 32, 16, 1024), tc5::smem_desc_sw128(k_sm + kb * kBlk + ks * 32, 16, 1024), kIdescS, (kb | ks) != 0);
                tc5::commit(bar(B_SFULL0 + (j & 1)));
                tc5::commit(bar(B_KEMPTY));
            };
            bool ok = mbar_wait_bounded(bar(B_QFULL), 0, err) && mbar_wait_bounded(bar(B_KFULL), 0, err);
            if (!ok) atomicExch(err, 13);
            if (ok) { tc5::fence_after_sync(); issue_s(0); }
            for (int j = 0; ok && j < n_tiles; j++) {
                if (j + 1 < n_tiles) {
                    if (!mbar_wait_bounded(bar(B_KFULL), (uint32_t)(j + 1) & 1u, err)) { atomicExch(err, 14); break; }
                    tc5::fence_after_sync(); issue_s(j + 1);
                }
                if (!mbar_wait_bounded(bar(B_PREADY0 + (j & 1)), (uint32_t)(j >> 1) & 1u, err) || !mbar_wait_bounded(bar(B_VFULL), (uint32_t)j & 1u, err)) { atomicExch(err, 15); break; }
                tc5::fence_after_sync();
                const uint32_t a = t_s0 + (uint32_t)(j & 1) * 128u;   // P(j): fp16 pairs in the first 64 columns of its S buffer
#pragma unroll
                for (int ks = 0; ks < 8; ks++)   // 16 keys per step; V is MN-major: 64-dim blocks 16 KB apart, 8-key groups 1 KB apart
                    tc5::mma_ts(t_o, a + ks * 8, tc5::smem_desc_sw128(v_sm + ks * 2048, kBlk, 1024), kIdescPV, (j | ks) != 0);
                tc5::commit(bar(B_ODONE));
                tc5::commit(bar(B_VEMPTY));
            }
        }
    } else {
        // ---- softmax warps: two threads per query row, split by key half
        const int g = w >> 2, r = tid & 127, qpos = pos_base + q0 + r;               // this row sees keys <= qpos (and < kend)
        const int lim = min(kend, qpos + 1);
        const uint32_t lane_sel = (uint32_t)((w & 3) * 32) << 16;
        const int pair_bar = 1 + (w & 3);   // named barrier of warps w and w + 4 (64 threads)
        float m = -INFINITY, l = 0.0f; bool alive = true;
        // Every thread runs every iteration and meets its partner at the pair barrier whatever happens: a wait that ran out only switches the work off.
        for (int j = 0; j < n_tiles; j++) {
            const uint32_t t_s = t_s0 + (uint32_t)(j & 1) * 128u + lane_sel;
            if (alive && !warp_wait(bar(B_SFULL0 + (j & 1)), (uint32_t)(j >> 1) & 1u, err)) { atomicExch(err, 16); alive = false; }
            tc5::fence_after_sync();
            uint32_t v[2][32];
#pragma unroll
            for (int c = 0; c < 2; c++) tc5::ld32(t_s + g * 64 + c * 32, v[c]);
            tc5::wait_ld();
            const int key0 = j * kBNk + g * 64;
            if (j * kBNk + kBNk > min(kend, pos_base + q0 + 1)) {   // the tile reaches past what the first row may see: mask by select
#pragma unroll
                for (int c = 0; c < 2; c++)
#pragma unroll
                    for (int i = 0; i < 32; i++) if (key0 + c * 32 + i >= lim) v[c][i] = 0xff800000u;   // -inf
            }
            float mx = -INFINITY;
#pragma unroll
            for (int c = 0; c < 2; c++)
#pragma unroll
                for (int i = 0; i < 32; i++) mx = fmaxf(mx, __uint_as_float(v[c][i]));
            s_xmax[j & 1][g][r] = mx;
            asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");   // both halves of the row's scores are in registers and both maxima are visible
            do {
            if (!alive) break;
            const float mt = fmaxf(mx, s_xmax[j & 1][g ^ 1][r]) * kLog2e;
            const bool need = (j == 0) ? false : (mt > m + 8.0f);
            if (j == 0) m = mt;
            if (__any_sync(0xffffffffu, need)) {   // raise the reference maximum: rescale this thread's half of the O row after the previous P.V has landed
                if (!warp_wait(bar(B_ODONE), (uint32_t)(j - 1) & 1u, err)) { atomicExch(err, 17); alive = false; break; }
                tc5::fence_after_sync();
                const float alpha = need ? ex2(m - mt) : 1.0f;
                if (need) { m = mt; l *= alpha; }
#pragma unroll 1
                for (int c = 0; c < 4; c++) {
                    uint32_t o[32]; tc5::ld32(t_o + lane_sel + g * 128 + c * 32, o); tc5::wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    tc5::st32(t_o + lane_sel + g * 128 + c * 32, o);
                }
                tc5::wait_st();
            }
            const float msub = (m == -INFINITY) ? 0.0f : m;
            float sum = 0.0f; uint32_t pk[32];
#pragma unroll
            for (int c = 0; c < 2; c++)
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    const float p0 = ex2(fmaf(__uint_as_float(v[c][i]), kLog2e, -msub)), p1 = ex2(fmaf(__uint_as_float(v[c][i + 1]), kLog2e, -msub));
                    sum += p0 + p1; pk[c * 16 + (i >> 1)] = pack_h2(p0, p1);
                }
            l += sum;
            tc5::st32(t_s + g * 32, pk);   // P: keys 0-63 in columns [0,32), keys 64-127 in [32,64) of the S buffer (the partner's scores there are in its registers since the pair barrier)
            tc5::wait_st();
            if (j * kBNk + kBNk > kend) {   // tail tile: rows of V past the range were loaded as they lie in memory; zero them (0 x garbage must stay 0)
                // P(j-1).V(j-1) done first, so that the V barrier cannot still be in the phase of tile j-1 when its parity is tested
                if ((j >= 1 && !warp_wait(bar(B_ODONE), (uint32_t)(j - 1) & 1u, err)) || !warp_wait(bar(B_VFULL), (uint32_t)j & 1u, err)) { atomicExch(err, 18); alive = false; break; }
                if (g == 0 && j * kBNk + r >= kend) {
#pragma unroll
                    for (int kb = 0; kb < 4; kb++)
#pragma unroll
                        for (int c = 0; c < 8; c++) *reinterpret_cast<uint4*>(v_gen + kb * kBlk + r * 128 + c * 16) = make_uint4(0, 0, 0, 0);
                }
                fence_proxy_async();
            }
            tc5::fence_before_sync();
            mbar_arrive(bar(B_PREADY0 + (j & 1)));
            } while (0);
        }
        // ---- epilogue: O / l * sigmoid(gate); the two threads of a row add their partial l and write 128 columns each
        s_xmax[n_tiles & 1][g][r] = l;
        asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
        l += s_xmax[n_tiles & 1][g ^ 1][r];
        if (alive && warp_wait(bar(B_ODONE), (uint32_t)(n_tiles - 1) & 1u, err)) {
            tc5::fence_after_sync();
            const float inv = 1.0f / l; const bool store = r < rows_valid;
            const int64_t obase = ((int64_t)bi * M + q0 + r) * kQD + h * kD + g * 128;
#pragma unroll 1
            for (int c = 0; c < 4; c++) {
                uint32_t o[32]; tc5::ld32(t_o + lane_sel + g * 128 + c * 32, o); tc5::wait_ld();
                if (store) {
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        const float4 g4 = *reinterpret_cast<const float4*>(gate + obase + c * 32 + i);
                        const float y0 = __uint_as_float(o[i]) * inv * (1.0f / (1.0f + __expf(-g4.x))), y1 = __uint_as_float(o[i + 1]) * inv * (1.0f / (1.0f + __expf(-g4.y)));
                        const float y2 = __uint_as_float(o[i + 2]) * inv * (1.0f / (1.0f + __expf(-g4.z))), y3 = __uint_as_float(o[i + 3]) * inv * (1.0f / (1.0f + __expf(-g4.w)));
                        if (out_bf16) { __nv_bfloat162* d2 = reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<__nv_bfloat16*>(out) + obase + c * 32 + i); d2[0] = __floats2bfloat162_rn(y0, y1); d2[1] = __floats2bfloat162_rn(y2, y3); }
                        else *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + obase + c * 32 + i) = make_float4(y0, y1, y2, y3);
                    }
                }
            }
        } else if (alive) atomicExch(err, 19);
    }
    tc5::fence_before_sync();
    __syncthreads();
    if (w == 0) tc5::tmem_dealloc(tmem, 512);
}

}  // namespace

cudaError_t launch_prefill_mma(Ctx& c, const Batch& b, int M, const __half* q16, const float* gate, void* out, int out_dtype, cudaStream_t s);

// fp16 cache: tcgen05 kernel (unless the context was created with the legacy-path flag); int8 cache: mma.sync kernel.
cudaError_t launch_prefill(Ctx& c, const Batch& b, int M, const __half* q16, const float* gate, void* out, int out_dtype, cudaStream_t s) {
    if (c.cfg.kv_mode == KATA_KV_INT8 || (c.cfg.flags & 1)) return launch_prefill_mma(c, b, M, q16, gate, out, out_dtype, s);
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(prefill_tc5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTc);
        if (e != cudaSuccess) return e;
        attr_set = true;
    }
    CUtensorMap tm_q;
    if (!make_matrix_tmap(&tm_q, q16, (int64_t)b.n * M, kQD, 64, 128)) return cudaErrorInvalidValue;
    const dim3 grid((M + kBMq - 1) / kBMq, kH, b.n);
    prefill_tc5_kernel<<<grid, kTcThreads, kSmemTc, s>>>(tm_q, c.tm_k128, c.tm_v128, b, M, gate, out, out_dtype == KATA_ACT_BF16, c.d_err);
    c.launches++;
    return cudaGetLastError();
}

}  // namespace kata
