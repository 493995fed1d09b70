// One warp, one 16-row query block, one 16-key tile: S = Q K^T, masked online softmax, O += P V.
// Shared by the decode kernel (rows = 6 heads x T tokens of a KV head) and the mma.sync prefill kernel (rows = 16
// consecutive query positions of one head). Tile order and rounding points follow the reference's matrix kernels
// (shaders/flash.metal:39-60, 112-132): fp16 Q (prescaled by 1/16) x fp16 or int8 K with fp32 accumulation; int8
// scores multiplied by the key's fp16 scale; P = exp(S - m) rounded to fp16 (after the V scale in int8 mode);
// l accumulated from the unrounded p; fully masked rows keep m = -inf and contribute nothing.
//
// Fragment layouts (mma.sync.m16n8k16, g = lane/4, t4 = lane%4): accumulator element 0,1 = row g, columns 2*t4, 2*t4+1;
// elements 2,3 = row g+8. K/V rows sit in shared memory with a 16-byte pad per row so the eight row addresses of an
// ldmatrix fall in distinct banks. int8 rows are dequantised in registers: ldmatrix moves raw bytes (as b16 pairs),
// a byte permute drops them onto the fp16 pattern 0x64xx (= 1024 + x), and one half2 subtract removes the bias.
#pragma once
#include "kata_internal.cuh"
#include "ptx.cuh"

namespace kata {

template <bool I8> struct TileGeo {
    static constexpr int kRowBytes = I8 ? 256 : 512;      // one head's K or V row in the cache
    static constexpr int kRowStride = kRowBytes + 16;     // in shared memory
};
constexpr int kQStride = 528;                              // bytes per staged Q row (256 fp16 + 16 pad)

// dimension held by O accumulator element (n-tile j, column c in {0,1}) of a thread with quad index t4
template <bool I8> __device__ __forceinline__ int dim_of(int j, int c, int t4) {
    if (!I8) return 8 * j + 2 * t4 + c;
    return (j >> 1) * 16 + 4 * t4 + 2 * c + (j & 1);
}

// int8 mode wants the Q block's columns permuted inside each 16-dim block to the contraction order of the dequantised
// K fragments: dim d = 4*tq + rem  ->  column (rem>>1)*8 + 2*tq + (rem&1).
__device__ __forceinline__ int q8_col_of_dim(int d16) { const int tq = d16 >> 2, rem = d16 & 3; return (rem >> 1) * 8 + 2 * tq + (rem & 1); }

__device__ __forceinline__ uint32_t deq2(uint32_t x, uint32_t sel) {   // two biased bytes of x -> half2 of the signed values
    const uint32_t h = ptx::prmt(x, 0x64646464u, sel);
    const __half2 r = __hsub2(*reinterpret_cast<const __half2*>(&h), __floats2half2_rn(1152.0f, 1152.0f));
    return *reinterpret_cast<const uint32_t*>(&r);
}

struct RowState {   // softmax state of rows g and g+8 (m in log2 units, l partial over this thread's columns) and the O block
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;
    float o[32][4];
    __device__ __forceinline__ void clear() {
        m0 = m1 = -INFINITY; l0 = l1 = 0.0f;
#pragma unroll
        for (int j = 0; j < 32; j++) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f; }
    }
    __device__ __forceinline__ void finish_l() {   // sum l over the quad that shares a row
        l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    }
};

// q_sm: shared address of the warp's 16-row Q block (row stride kQStride). k_sm / v_sm: shared addresses of the tile's 16
// K and V rows (row stride TileGeo::kRowStride). key0: index of the tile's first key; row g sees keys < lim0, row g+8
// keys < lim1 (0 for a dead row). ks/vs: int8 mode, the fp16 scales of this thread's four score columns
// (keys key0 + nt*8 + 2*t4 + e -> [nt][e]).
template <bool I8, bool V8 = I8>   // I8: int8 keys, V8: int8 values
__device__ __forceinline__ void tile_qk_softmax_pv(const uint32_t q_sm, const uint32_t k_sm, const uint32_t v_sm, const int key0, const int lim0, const int lim1,
                                                   const float (&ks)[2][2], const float (&vs)[2][2], RowState& st, const int lane) {
    using G = TileGeo<I8>; using GV = TileGeo<V8>;
    using namespace ptx;
    const int t4 = lane & 3;
    float s[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
    const uint32_t qa = q_sm + (lane & 15) * kQStride + (lane >> 4) * 16;
    const uint32_t ka = k_sm + ((lane & 7) + ((lane >> 4) << 3)) * G::kRowStride + ((lane >> 3) & 1) * 16;
    if (!I8) {
        float s2[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};   // second pair of accumulator chains: halves the dependent-MMA latency
#pragma unroll
        for (int kk = 0; kk < 16; kk += 2) {
            uint32_t a0, a1, a2, a3, b0, b1, b2, b3, c0, c1, c2, c3, d0, d1, d2, d3;
            ldsm_x4(qa + kk * 32, a0, a1, a2, a3); ldsm_x4(ka + kk * 32, b0, b1, b2, b3);
            ldsm_x4(qa + kk * 32 + 32, c0, c1, c2, c3); ldsm_x4(ka + kk * 32 + 32, d0, d1, d2, d3);
            mma16816(s[0], a0, a1, a2, a3, b0, b1); mma16816(s[1], a0, a1, a2, a3, b2, b3);
            mma16816(s2[0], c0, c1, c2, c3, d0, d1); mma16816(s2[1], c0, c1, c2, c3, d2, d3);
        }
#pragma unroll
        for (int nt = 0; nt < 2; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) s[nt][e] += s2[nt][e];
    } else {
        // an 8x8 b16 matrix covers 8 keys x 16 int8 dims; a thread's register = dims 4*t4..4*t4+3 of key g
#pragma unroll
        for (int k2 = 0; k2 < 8; k2++) {
            uint32_t r0, r1, r2, r3; ldsm_x4(ka + k2 * 32, r0, r1, r2, r3);   // r0: keys 0-7 block 2*k2, r1: keys 0-7 block 2*k2+1, r2, r3: keys 8-15
            r0 ^= 0x80808080u; r1 ^= 0x80808080u; r2 ^= 0x80808080u; r3 ^= 0x80808080u;
            uint32_t a0, a1, a2, a3;
            ldsm_x4(qa + (2 * k2) * 32, a0, a1, a2, a3);
            mma16816(s[0], a0, a1, a2, a3, deq2(r0, 0x4140u), deq2(r0, 0x4342u)); mma16816(s[1], a0, a1, a2, a3, deq2(r2, 0x4140u), deq2(r2, 0x4342u));
            ldsm_x4(qa + (2 * k2 + 1) * 32, a0, a1, a2, a3);
            mma16816(s[0], a0, a1, a2, a3, deq2(r1, 0x4140u), deq2(r1, 0x4342u)); mma16816(s[1], a0, a1, a2, a3, deq2(r3, 0x4140u), deq2(r3, 0x4342u));
        }
#pragma unroll
        for (int nt = 0; nt < 2; nt++) { s[nt][0] *= ks[nt][0]; s[nt][1] *= ks[nt][1]; s[nt][2] *= ks[nt][0]; s[nt][3] *= ks[nt][1]; }
    }
    // mask by select (never by arithmetic: rows past the valid range may hold anything)
#pragma unroll
    for (int nt = 0; nt < 2; nt++)
#pragma unroll
        for (int e = 0; e < 2; e++) { const int key = key0 + nt * 8 + 2 * t4 + e; if (key >= lim0) s[nt][e] = -INFINITY; if (key >= lim1) s[nt][2 + e] = -INFINITY; }
    // online softmax in the log2 domain
    float mx0 = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1])) * kLog2e, mx1 = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3])) * kLog2e;
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(st.m0, mx0), mn1 = fmaxf(st.m1, mx1);
    const float al0 = (mn0 == -INFINITY) ? 1.0f : ex2(st.m0 - mn0), al1 = (mn1 == -INFINITY) ? 1.0f : ex2(st.m1 - mn1);
    const float sub0 = (mn0 == -INFINITY) ? 0.0f : mn0, sub1 = (mn1 == -INFINITY) ? 0.0f : mn1;
    st.m0 = mn0; st.m1 = mn1;
    float pr[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; nt++) { pr[nt][0] = ex2(fmaf(s[nt][0], kLog2e, -sub0)); pr[nt][1] = ex2(fmaf(s[nt][1], kLog2e, -sub0)); pr[nt][2] = ex2(fmaf(s[nt][2], kLog2e, -sub1)); pr[nt][3] = ex2(fmaf(s[nt][3], kLog2e, -sub1)); }
    st.l0 = st.l0 * al0 + ((pr[0][0] + pr[0][1]) + (pr[1][0] + pr[1][1]));
    st.l1 = st.l1 * al1 + ((pr[0][2] + pr[0][3]) + (pr[1][2] + pr[1][3]));
    if (__any_sync(0xffffffffu, al0 != 1.0f || al1 != 1.0f)) {
#pragma unroll
        for (int j = 0; j < 32; j++) { st.o[j][0] *= al0; st.o[j][1] *= al0; st.o[j][2] *= al1; st.o[j][3] *= al1; }
    }
    if (V8) {
#pragma unroll
        for (int nt = 0; nt < 2; nt++) { pr[nt][0] *= vs[nt][0]; pr[nt][1] *= vs[nt][1]; pr[nt][2] *= vs[nt][0]; pr[nt][3] *= vs[nt][1]; }
    }
    const uint32_t pa0 = pack_h2(pr[0][0], pr[0][1]), pa1 = pack_h2(pr[0][2], pr[0][3]), pa2 = pack_h2(pr[1][0], pr[1][1]), pa3 = pack_h2(pr[1][2], pr[1][3]);
    const uint32_t va = v_sm + ((lane & 7) + ((lane >> 3) & 1) * 8) * GV::kRowStride + (lane >> 4) * 16;
    if (!V8) {
#pragma unroll
        for (int j2 = 0; j2 < 16; j2++) {
            uint32_t b0, b1, b2, b3; ldsm_x4_t(va + j2 * 32, b0, b1, b2, b3);
            mma16816(st.o[2 * j2], pa0, pa1, pa2, pa3, b0, b1); mma16816(st.o[2 * j2 + 1], pa0, pa1, pa2, pa3, b2, b3);
        }
    } else {
        // transposed b16 load of int8 rows: register = { V[2*t4][2g], V[2*t4][2g+1], V[2*t4+1][2g], V[2*t4+1][2g+1] } within the matrix
#pragma unroll
        for (int j2 = 0; j2 < 8; j2++) {
            uint32_t r0, r1, r2, r3; ldsm_x4_t(va + j2 * 32, r0, r1, r2, r3);   // r0: keys 0-7 block 2*j2, r1: keys 8-15 block 2*j2, r2, r3: block 2*j2+1
            r0 ^= 0x80808080u; r1 ^= 0x80808080u; r2 ^= 0x80808080u; r3 ^= 0x80808080u;
            mma16816(st.o[4 * j2 + 0], pa0, pa1, pa2, pa3, deq2(r0, 0x4240u), deq2(r1, 0x4240u));
            mma16816(st.o[4 * j2 + 1], pa0, pa1, pa2, pa3, deq2(r0, 0x4341u), deq2(r1, 0x4341u));
            mma16816(st.o[4 * j2 + 2], pa0, pa1, pa2, pa3, deq2(r2, 0x4240u), deq2(r3, 0x4240u));
            mma16816(st.o[4 * j2 + 3], pa0, pa1, pa2, pa3, deq2(r2, 0x4341u), deq2(r3, 0x4341u));
        }
    }
}

// Stage one 16-byte chunk (8 fp16 values, dims c16*8..c16*8+7) of a Q row into shared memory, permuting for int8 mode.
template <bool I8> __device__ __forceinline__ void stage_q_chunk(uint8_t* q_row_sm, int c16, uint4 v) {
    if (!I8) { *reinterpret_cast<uint4*>(q_row_sm + c16 * 16) = v; return; }
    const __half* hv = reinterpret_cast<const __half*>(&v); __half* dst = reinterpret_cast<__half*>(q_row_sm) + (c16 >> 1) * 16;
#pragma unroll
    for (int e = 0; e < 8; e++) dst[q8_col_of_dim((c16 & 1) * 8 + e)] = hv[e];
}

__device__ __forceinline__ float sigmoid_fast(float x) { return ptx::sigmoid_approx(x); }

}  // namespace kata

// ---------------------------------------------------------------------------------------------------------------------
// Warp-specialised tile routines of the decode kernel. A ring of the kernel has one "score" warp and two "value" warps that
// overlap across tiles: the score warp computes S = Q K^T for the tile's keys, the online-softmax state (m, l) and the fp16 P
// block, and hands P plus the rescale factors of its two row groups to the value warps through a two-slot shared-memory
// buffer; each value warp owns a 16 x 128 half of the O block, applies the rescale and accumulates O += P V. While the value
// warps work on tile i the score warp is already on tile i+1. Arithmetic and rounding points are those of tile_qk_softmax_pv.
//
// A tile holds NK sub-blocks of 16 keys (NK = 1: fp16 cache, NK = 2: int8 cache, where the per-tile costs - barriers, shuffles,
// the Q fragments - weigh more against half the bytes). K and V tiles are read as TMA wrote them: column blocks of
// [16*NK keys][128 bytes], block b holding bytes [128b, 128b+128) of every row, 16-byte chunk c of row r stored at chunk c ^ (r & 7).
namespace kata {

// In the int8 path the codes are not fully dequantised: the byte permute leaves code + 1152 in fp16 (exact:
// 0x64xx = 1024 + (code ^ 0x80)), the MMAs run on these biased values, and the bias terms 1152 * sum_d q_d (scores) and
// 1152 * sum_k P_k (output) are subtracted afterwards in fp32. This removes the half2 subtract per pair of codes.
constexpr float kI8Bias = 1152.0f;
__device__ __forceinline__ uint32_t deq2_biased(uint32_t x, uint32_t sel) { return ptx::prmt(x, 0x64646464u, sel); }

// dimension of O element (n-tile j of 16, column c) held by the value warp of half h
template <bool I8> __device__ __forceinline__ int pair_dim_of(int h, int j, int c, int t4) { return h * 128 + dim_of<I8>(j, c, t4); }

template <int NK> struct PSlot {
    static constexpr int kStride = 32 * NK + 16;          // bytes per row of the fp16 P block (16 pad: conflict-free ldmatrix)
    static constexpr int kBytes = 16 * kStride + 64;      // P block + 16 rescale factors
};

struct ScoreState { float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f; };
template <int NJ> struct ValueStateT {   // NJ n-tiles of 8 dims: 16 = one half of the head
    float ps0 = 0.0f, ps1 = 0.0f;   // int8 mode: running sums of the fp16-rounded P (bias term of the biased V fragments)
    float o[NJ][4];
    __device__ __forceinline__ void clear() {
        ps0 = ps1 = 0.0f;
#pragma unroll
        for (int j = 0; j < NJ; j++) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f; }
    }
    __device__ __forceinline__ void finish_bias(float bias) {
        ps0 += __shfl_xor_sync(0xffffffffu, ps0, 1); ps0 += __shfl_xor_sync(0xffffffffu, ps0, 2);
        ps1 += __shfl_xor_sync(0xffffffffu, ps1, 1); ps1 += __shfl_xor_sync(0xffffffffu, ps1, 2);
#pragma unroll
        for (int j = 0; j < NJ; j++) { o[j][0] -= bias * ps0; o[j][1] -= bias * ps0; o[j][2] -= bias * ps1; o[j][3] -= bias * ps1; }
    }
};

// Score warp, one tile. Returns the unrounded-then-scaled P values pr[n-tile][4] (n-tile nt = 8 keys: keys key0 + 8*nt + 2*t4 + e are
// elements e and 2 + e for rows g and g + 8) and the rescale factors of rows g and g + 8. ks/vs: int8 scales of this thread's score
// columns ([nt][e]); qs: int8 mode, sums over the 256 dims of Q rows g and g+8.
// KG (int8 keys with one scale per 64 dims): ksg[nt][e] holds the four fp16 group scales of the key of score column (nt, e) as two packed
// words, qsg[row half][group] the sums of the staged Q rows g and g + 8 over each 64-dim group; the contraction is then cut into the four
// groups and each group's partial score takes its own scale: S = sum_g ks_g * (Q_g . Kq_g), the finer key quantisation the reference measured
// but could not fold into its matrix path (docs/reports/M11-int8-kv.en.md:52-55, 94-97).
template <bool I8, bool V8, int NK, bool KG = false>   // I8: int8 keys; V8: int8 values (P takes the value scale before it is rounded to fp16)
__device__ __forceinline__ void score_tile(const uint32_t q_sm, const uint32_t k_sm, const int key0, const int lim0, const int lim1,
                                           const float (&ks)[2 * NK][2], const float (&vs)[2 * NK][2], const float (&qs)[2], ScoreState& st, const int lane,
                                           float (&pr)[2 * NK][4], float& al0, float& al1, const uint2 (*ksg)[2] = nullptr, const float (*qsg)[4] = nullptr) {
    using namespace ptx;
    constexpr uint32_t kBlk = 16 * NK * 128;   // bytes of one 128-byte column block of the tile
    constexpr int NT = 2 * NK;
    const int t4 = lane & 3;
    const uint32_t rx = lane & 7, q1 = (lane >> 3) & 1;
    const uint32_t qa = q_sm + (lane & 15) * kQStride + (lane >> 4) * 16;
    const uint32_t ka = k_sm + (rx + ((lane >> 4) << 3)) * 128;   // lanes 0-15: keys 0-7, lanes 16-31: keys 8-15 of a sub-block; two 16-byte chunks per step
    const uint32_t ko[4] = {((0 + q1) ^ rx) << 4, ((2 + q1) ^ rx) << 4, ((4 + q1) ^ rx) << 4, ((6 + q1) ^ rx) << 4};
    float s[NT][4], s2[NT][4];   // two accumulator chains per n-tile: halves the dependent-MMA latency
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int e = 0; e < 4; e++) { s[nt][e] = 0.0f; s2[nt][e] = 0.0f; }
    if (!I8) {
#pragma unroll
        for (int kk = 0; kk < 16; kk += 2) {   // chunk 2*kk + q1 of the 512-byte row: block kk/4, chunk 2*(kk%4) + q1 inside it
            uint32_t a0, a1, a2, a3, c0, c1, c2, c3;
            ldsm_x4(qa + kk * 32, a0, a1, a2, a3); ldsm_x4(qa + kk * 32 + 32, c0, c1, c2, c3);
#pragma unroll
            for (int sb = 0; sb < NK; sb++) {
                uint32_t b0, b1, b2, b3, d0, d1, d2, d3;
                ldsm_x4(ka + sb * 2048 + (kk >> 2) * kBlk + ko[kk & 3], b0, b1, b2, b3); ldsm_x4(ka + sb * 2048 + (kk >> 2) * kBlk + ko[(kk & 3) + 1], d0, d1, d2, d3);
                mma16816(s[2 * sb], a0, a1, a2, a3, b0, b1); mma16816(s[2 * sb + 1], a0, a1, a2, a3, b2, b3);
                mma16816(s2[2 * sb], c0, c1, c2, c3, d0, d1); mma16816(s2[2 * sb + 1], c0, c1, c2, c3, d2, d3);
            }
        }
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) s[nt][e] += s2[nt][e];
    } else if (KG) {
        float tot[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; nt++) { tot[nt][0] = tot[nt][1] = tot[nt][2] = tot[nt][3] = 0.0f; }
#pragma unroll
        for (int g4 = 0; g4 < 4; g4++) {
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int e = 0; e < 4; e++) { s[nt][e] = 0.0f; s2[nt][e] = 0.0f; }
#pragma unroll
            for (int k2 = 2 * g4; k2 < 2 * g4 + 2; k2++) {
                uint32_t a0, a1, a2, a3, c0, c1, c2, c3;
                ldsm_x4(qa + (2 * k2) * 32, a0, a1, a2, a3); ldsm_x4(qa + (2 * k2 + 1) * 32, c0, c1, c2, c3);
#pragma unroll
                for (int sb = 0; sb < NK; sb++) {
                    uint32_t r0, r1, r2, r3;
                    ldsm_x4(ka + sb * 2048 + (k2 >> 2) * kBlk + ko[k2 & 3], r0, r1, r2, r3);
                    r0 ^= 0x80808080u; r1 ^= 0x80808080u; r2 ^= 0x80808080u; r3 ^= 0x80808080u;
                    mma16816(s[2 * sb], a0, a1, a2, a3, deq2_biased(r0, 0x4140u), deq2_biased(r0, 0x4342u)); mma16816(s[2 * sb + 1], a0, a1, a2, a3, deq2_biased(r2, 0x4140u), deq2_biased(r2, 0x4342u));
                    mma16816(s2[2 * sb], c0, c1, c2, c3, deq2_biased(r1, 0x4140u), deq2_biased(r1, 0x4342u)); mma16816(s2[2 * sb + 1], c0, c1, c2, c3, deq2_biased(r3, 0x4140u), deq2_biased(r3, 0x4342u));
                }
            }
            const float b0 = kI8Bias * qsg[0][g4], b1 = kI8Bias * qsg[1][g4];   // this group's scores were formed against code + 1152
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const uint32_t w0 = (g4 < 2) ? ksg[nt][0].x : ksg[nt][0].y, w1 = (g4 < 2) ? ksg[nt][1].x : ksg[nt][1].y;   // packed fp16 scales of groups (0,1) or (2,3)
                const float k0 = __half2float(__ushort_as_half((unsigned short)((g4 & 1) ? (w0 >> 16) : (w0 & 0xffffu)))), k1 = __half2float(__ushort_as_half((unsigned short)((g4 & 1) ? (w1 >> 16) : (w1 & 0xffffu))));
                tot[nt][0] = fmaf(s[nt][0] + s2[nt][0] - b0, k0, tot[nt][0]); tot[nt][1] = fmaf(s[nt][1] + s2[nt][1] - b0, k1, tot[nt][1]);
                tot[nt][2] = fmaf(s[nt][2] + s2[nt][2] - b1, k0, tot[nt][2]); tot[nt][3] = fmaf(s[nt][3] + s2[nt][3] - b1, k1, tot[nt][3]);
            }
        }
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) s[nt][e] = tot[nt][e];
    } else {
#pragma unroll
        for (int k2 = 0; k2 < 8; k2++) {   // int8: 16-byte chunk = 16-dim block; r0: keys 0-7 block 2*k2, r1: keys 0-7 block 2*k2+1, r2, r3: keys 8-15
            uint32_t a0, a1, a2, a3, c0, c1, c2, c3;
            ldsm_x4(qa + (2 * k2) * 32, a0, a1, a2, a3); ldsm_x4(qa + (2 * k2 + 1) * 32, c0, c1, c2, c3);
#pragma unroll
            for (int sb = 0; sb < NK; sb++) {
                uint32_t r0, r1, r2, r3;
                ldsm_x4(ka + sb * 2048 + (k2 >> 2) * kBlk + ko[k2 & 3], r0, r1, r2, r3);
                r0 ^= 0x80808080u; r1 ^= 0x80808080u; r2 ^= 0x80808080u; r3 ^= 0x80808080u;
                mma16816(s[2 * sb], a0, a1, a2, a3, deq2_biased(r0, 0x4140u), deq2_biased(r0, 0x4342u)); mma16816(s[2 * sb + 1], a0, a1, a2, a3, deq2_biased(r2, 0x4140u), deq2_biased(r2, 0x4342u));
                mma16816(s2[2 * sb], c0, c1, c2, c3, deq2_biased(r1, 0x4140u), deq2_biased(r1, 0x4342u)); mma16816(s2[2 * sb + 1], c0, c1, c2, c3, deq2_biased(r3, 0x4140u), deq2_biased(r3, 0x4342u));
            }
        }
        const float b0 = kI8Bias * qs[0], b1 = kI8Bias * qs[1];   // the scores were formed against code + 1152
#pragma unroll
        for (int nt = 0; nt < NT; nt++) { s[nt][0] = (s[nt][0] + s2[nt][0] - b0) * ks[nt][0]; s[nt][1] = (s[nt][1] + s2[nt][1] - b0) * ks[nt][1]; s[nt][2] = (s[nt][2] + s2[nt][2] - b1) * ks[nt][0]; s[nt][3] = (s[nt][3] + s2[nt][3] - b1) * ks[nt][1]; }
    }
    // mask by select (never by arithmetic: rows past the valid range may hold anything)
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int e = 0; e < 2; e++) { const int key = key0 + nt * 8 + 2 * t4 + e; if (key >= lim0) s[nt][e] = -INFINITY; if (key >= lim1) s[nt][2 + e] = -INFINITY; }
    // online softmax in the log2 domain
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < NT; nt++) { mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1])); mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3])); }
    mx0 *= kLog2e; mx1 *= kLog2e;
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(st.m0, mx0), mn1 = fmaxf(st.m1, mx1);
    al0 = (mn0 == -INFINITY) ? 1.0f : ex2(st.m0 - mn0); al1 = (mn1 == -INFINITY) ? 1.0f : ex2(st.m1 - mn1);
    const float sub0 = (mn0 == -INFINITY) ? 0.0f : mn0, sub1 = (mn1 == -INFINITY) ? 0.0f : mn1;
    st.m0 = mn0; st.m1 = mn1;
    float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
    for (int nt = 0; nt < NT; nt += 2) {   // the row sum is formed per 16-key sub-block as (p0 + p1) + (p2 + p3), sub-blocks added in order
        float q0 = 0.0f, q1s = 0.0f;
#pragma unroll
        for (int u = 0; u < 2; u++) {
            pr[nt + u][0] = ex2(fmaf(s[nt + u][0], kLog2e, -sub0)); pr[nt + u][1] = ex2(fmaf(s[nt + u][1], kLog2e, -sub0));
            pr[nt + u][2] = ex2(fmaf(s[nt + u][2], kLog2e, -sub1)); pr[nt + u][3] = ex2(fmaf(s[nt + u][3], kLog2e, -sub1));
        }
        q0 = (pr[nt][0] + pr[nt][1]) + (pr[nt + 1][0] + pr[nt + 1][1]); q1s = (pr[nt][2] + pr[nt][3]) + (pr[nt + 1][2] + pr[nt + 1][3]);
        sum0 += q0; sum1 += q1s;
    }
    st.l0 = st.l0 * al0 + sum0; st.l1 = st.l1 * al1 + sum1;
    if (V8) {
#pragma unroll
        for (int nt = 0; nt < NT; nt++) { pr[nt][0] *= vs[nt][0]; pr[nt][1] *= vs[nt][1]; pr[nt][2] *= vs[nt][0]; pr[nt][3] *= vs[nt][1]; }
    }
}

// the score warp publishes P (fp16) and the two rescale factors of its rows into a slot
template <int NK>
__device__ __forceinline__ void score_publish(const uint32_t p_sm, float* alpha_gen, const float (&pr)[2 * NK][4], const float al0, const float al1, const int lane) {
    const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
    for (int nt = 0; nt < 2 * NK; nt++) {
        const uint32_t off = (uint32_t)((8 * nt + 2 * t4) * 2);
        asm volatile("st.shared.b32 [%0], %1;" ::"r"(p_sm + g * PSlot<NK>::kStride + off), "r"(ptx::pack_h2(pr[nt][0], pr[nt][1])) : "memory");
        asm volatile("st.shared.b32 [%0], %1;" ::"r"(p_sm + (g + 8) * PSlot<NK>::kStride + off), "r"(ptx::pack_h2(pr[nt][2], pr[nt][3])) : "memory");
    }
    if (t4 == 0) { alpha_gen[g] = al0; alpha_gen[g + 8] = al1; }
}

// Value warp, one tile: O = O * alpha + P V over the tile's keys and the dims [vh * 8 * NJ, (vh + 1) * 8 * NJ) of the head.
template <bool I8, int NJ, int NK>
__device__ __forceinline__ void value_tile(const uint32_t v_sm, const uint32_t p_sm, const float* alpha_gen, ValueStateT<NJ>& st, const int lane, const int vh) {
    using namespace ptx;
    constexpr uint32_t kBlk = 16 * NK * 128;
    const int g = lane >> 2;
    const float al0 = alpha_gen[g], al1 = alpha_gen[g + 8];
    uint32_t pa[NK][4];
#pragma unroll
    for (int sb = 0; sb < NK; sb++) ldsm_x4(p_sm + (lane & 15) * PSlot<NK>::kStride + sb * 32 + (lane >> 4) * 16, pa[sb][0], pa[sb][1], pa[sb][2], pa[sb][3]);
    if (__any_sync(0xffffffffu, al0 != 1.0f || al1 != 1.0f)) {
#pragma unroll
        for (int j = 0; j < NJ; j++) { st.o[j][0] *= al0; st.o[j][1] *= al0; st.o[j][2] *= al1; st.o[j][3] *= al1; }
    }
    if (I8) {
        float a0 = 0.0f, a1 = 0.0f;
#pragma unroll
        for (int sb = 0; sb < NK; sb++) {
            const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&pa[sb][0])), f1 = __half22float2(*reinterpret_cast<const __half2*>(&pa[sb][1]));
            const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&pa[sb][2])), f3 = __half22float2(*reinterpret_cast<const __half2*>(&pa[sb][3]));
            a0 += (f0.x + f0.y) + (f2.x + f2.y); a1 += (f1.x + f1.y) + (f3.x + f3.y);
        }
        st.ps0 = st.ps0 * al0 + a0; st.ps1 = st.ps1 * al1 + a1;
    }
    const uint32_t rx = lane & 7, ud = lane >> 4;
    // fp16: 16-byte chunk 2*j + ud of the 512-byte row, j = vh * NJ/2 + j2; int8: chunk 2*j + ud of the 256-byte row, j = vh * NJ/4 + j2
    const uint32_t va = v_sm + (rx + ((lane >> 3) & 1) * 8) * 128 + (uint32_t)vh * (NJ == 32 ? 0u : kBlk * (I8 ? 1u : 2u));
    const uint32_t vo[4] = {((0 + ud) ^ rx) << 4, ((2 + ud) ^ rx) << 4, ((4 + ud) ^ rx) << 4, ((6 + ud) ^ rx) << 4};
    if (!I8) {
#pragma unroll
        for (int j2 = 0; j2 < NJ / 2; j2++)
#pragma unroll
            for (int sb = 0; sb < NK; sb++) {
                uint32_t b0, b1, b2, b3; ldsm_x4_t(va + sb * 2048 + (j2 >> 2) * kBlk + vo[j2 & 3], b0, b1, b2, b3);
                mma16816(st.o[2 * j2], pa[sb][0], pa[sb][1], pa[sb][2], pa[sb][3], b0, b1); mma16816(st.o[2 * j2 + 1], pa[sb][0], pa[sb][1], pa[sb][2], pa[sb][3], b2, b3);
            }
    } else {
#pragma unroll
        for (int j2 = 0; j2 < NJ / 4; j2++)
#pragma unroll
            for (int sb = 0; sb < NK; sb++) {   // r0: keys 0-7 block 2*j, r1: keys 8-15 block 2*j, r2, r3: block 2*j+1
                uint32_t r0, r1, r2, r3; ldsm_x4_t(va + sb * 2048 + (j2 >> 2) * kBlk + vo[j2 & 3], r0, r1, r2, r3);
                r0 ^= 0x80808080u; r1 ^= 0x80808080u; r2 ^= 0x80808080u; r3 ^= 0x80808080u;
                mma16816(st.o[4 * j2 + 0], pa[sb][0], pa[sb][1], pa[sb][2], pa[sb][3], deq2_biased(r0, 0x4240u), deq2_biased(r1, 0x4240u));
                mma16816(st.o[4 * j2 + 1], pa[sb][0], pa[sb][1], pa[sb][2], pa[sb][3], deq2_biased(r0, 0x4341u), deq2_biased(r1, 0x4341u));
                mma16816(st.o[4 * j2 + 2], pa[sb][0], pa[sb][1], pa[sb][2], pa[sb][3], deq2_biased(r2, 0x4240u), deq2_biased(r3, 0x4240u));
                mma16816(st.o[4 * j2 + 3], pa[sb][0], pa[sb][1], pa[sb][2], pa[sb][3], deq2_biased(r2, 0x4341u), deq2_biased(r3, 0x4341u));
            }
    }
}

}  // namespace kata
