// Split-KV decode / T<=2 speculative-verify attention over the fp16 or int8 KV cache, with the merge of the splits and
// the sigmoid output gate fused into the same kernel.
// Replaces k_dec_q_pack + k_attn_dec_split[_q8 | _k16v8] + k_attn_dec_combine of the reference (shaders/flash.metal:77-152,
// 252-306; host side Engine::dDecAttn, src/engine.cpp:119-127). Same math and rounding points: fp16 query prescaled by 1/16,
// rows of the 16-row block = 6 heads of one KV head x T tokens (row = t*6 + j), fp32 scores, P rounded to fp16 before
// P.V (after the V scale where the values are int8), l summed from the unrounded p, masked rows/keys at -inf, merge weights exp(m-M).
//
// Design (HBM-bound: 1 KiB of K+V per key and KV head at fp16, read exactly once):
//  - The work is the list of tiles (16 keys at fp16, 32 at int8: 16 KiB of K+V; 16 keys = 12 KiB with fp16 keys and int8 values) of every (sequence, KV head) segment. It is cut into
//    one contiguous, equal-sized range per CTA (one CTA per SM), so ragged batches balance to within one tile and each key is read once.
//  - Inside a CTA the tiles of the range go round-robin to 4 rings. A ring is a 3-stage shared-memory ring with three warps on one
//    scheduler: a score warp (S = Q K^T, online softmax, P) and two value warps (O += P V on one half of the head dims each) that overlap
//    across tiles through a two-slot P hand-over ('P full' / 'P empty' mbarriers). A 13th warp is the producer: its lane r refills ring
//    r's stage as soon as the ring's three warps have released it ('full' / 'empty' mbarriers), with one TMA instruction per K tile and
//    one per V tile (rank-4 tensor-map view of the arena, 128-byte swizzle, so ldmatrix reads are bank-conflict free without padding).
//    Measured on B200: per-row bulk copies (one 512-byte copy per lane) capped the kernel near 4.9 TB/s because of the TMA unit's
//    operation rate; 8 boxes per stage reached 5.8 TB/s but cost the issuing math warp ~600 clocks per tile; tile views issued by a
//    warp of their own reach 6.1 TB/s at batch 8 and 6.8 TB/s at batch 64. Prefetching further ahead into L2 made it slower.
//  - Q.K^T and P.V run on mma.sync m16n8k16 (fp16 in, fp32 accumulate) straight from ldmatrix fragments. The softmax state lives in
//    registers and uses quad shuffles. int8 rows are dequantised in registers (byte permute onto the fp16 magic number 1024+x; the bias
//    is taken out of the accumulators afterwards), with the per-key scales applied to S and to P as the reference does.
//  - A CTA whose range ends inside a segment writes an unnormalised partial (O, m, l); with at most 8 contributors per segment the last
//    CTA to finish it (atomic ticket) merges the partials straight from L2, normalises, applies the gate and writes the output row;
//    segments split further (batch 1 at long context) are merged by decode_combine_kernel.
//  - The kernels are launched with programmatic stream serialisation: barrier set-up overlaps the previous kernel's tail.
// Every mbarrier wait is bounded; on a timeout the kernel records an error word and skips the arithmetic.
#include <algorithm>

#include "attn_tile.cuh"
#include "peer_exchange.cuh"

namespace kata {
namespace {

using namespace ptx;

// Development aid, compiled only with -DKATA_PF_TRACE (never in the shipped library): every CTA records %globaltimer stamps of its phases.
#ifdef KATA_PF_TRACE
__device__ unsigned long long g_dec_trace[8 * 1536];
__device__ __forceinline__ void dec_stamp(int slot) { if (blockIdx.x < 1536) { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); g_dec_trace[blockIdx.x * 8 + slot] = t; } }
#else
__device__ __forceinline__ void dec_stamp(int) {}
#endif

constexpr int kRings = 4, kWarps = 3 * kRings + 1, kThreads = kWarps * 32, kMaxStages = 8;
constexpr int kOffBars = 16 * kQStride;             // 8448: the barrier block: per ring and stage a 'full' and an 'empty' barrier,
constexpr int kOffEBars = kRings * kMaxStages * 8, kOffPBars = 2 * kOffEBars;   // inside the barrier block: then per ring two 'P full' and two 'P empty' barriers
constexpr int kOffQsum = kOffBars + 704;            // int8 modes: sum over the 256 dims of each staged Q row (16 floats), then its sums over each 64-dim group ([16][4])
constexpr int kOffMl = kOffQsum + 320;              // (row sums: 16 floats, then [16][4] sums per 64-dim group) per-ring (m, l) exchange: [4][16][2] floats = 512 B
constexpr int kOffPair = kOffMl + 512;              // per-ring hand-over from the score warp to the value warp: two slots of (P block 16 x 48 B, 16 rescale factors)
constexpr int kPairBytes = 2 * PSlot<2>::kBytes;    // 2688 (sized for the 32-key tiles of the int8 mode)
constexpr int kOffStages = kOffPair + kRings * kPairBytes;   // the stage area itself starts at the next 1024-byte boundary of the shared window (found at run time)
constexpr int kMergeStride = 264;                   // floats per row of the cross-ring merge buffer

// MODE = the context's cache mode: 0 fp16, 1 int8 (K and V), 2 int8v (K fp16, V int8: k_attn_dec_split_k16v8, shaders/flash.metal:252-306),
// 3 int8g (as 1 with four key scales per head row, one per 64 dims)
template <int MODE> struct Geo {
    static constexpr bool K8 = MODE == KATA_KV_INT8 || MODE == KATA_KV_INT8G, V8 = MODE != KATA_KV_FP16, KG = MODE == KATA_KV_INT8G;
    static constexpr int kKRowBytes = TileGeo<K8>::kRowBytes, kVRowBytes = TileGeo<V8>::kRowBytes;
    static constexpr int kVBoxes = kVRowBytes / 128;              // 128-byte column boxes per V tile
    static constexpr int kNK = K8 ? 2 : 1, kTile = 16 * kNK;      // keys per tile: 16 (fp16 keys) or 32 (int8 keys): 16 KiB of K+V (12 KiB in int8v mode)
    static constexpr int kKTileBytes = kTile * kKRowBytes, kVTileBytes = kTile * kVRowBytes;   // column blocks of [kTile rows][128 bytes], 128-byte swizzle, no padding
    static constexpr int kStageBytes = kKTileBytes + kVTileBytes;
    static constexpr int kStages = MODE == KATA_KV_INT8V ? 4 : 3;   // tiles in flight per ring: 48 KB
    static constexpr int kRingBytes = (kStages * kStageBytes > 16 * kMergeStride * 4) ? kStages * kStageBytes : 16 * kMergeStride * 4;
    static constexpr int kSmem = kOffStages + 1024 + kRings * kRingBytes;   // 1024 bytes of slack for the run-time alignment
};

struct DecPlan {
    int32_t n, T, first_row, key_off, n_ctas, q_tiles, r_tiles;   // CTA c owns tiles [c*q + min(c,r), (c+1)*q + min(c+1,r))
    int32_t cps;                         // > 0: every (sequence, KV head) segment has the same number of tiles and is cut between exactly cps CTAs of its own (no CTA works on two segments)
    int32_t kvh_lo, kvh_n;               // KV heads of this launch: a sequence's tiles are those of heads kvh_lo .. kvh_lo + kvh_n - 1, head after head
    int32_t tok_stride, tok0;            // rows of q16 / gate / out per sequence, and the row of this launch's token 0 (a wide verify runs as launches of 2 tokens)
    int32_t merge_in_kernel;             // 1: the last contributor of a segment merges its partials; 0: decode_combine_kernel does
    int32_t pos[KATA_MAX_BATCH];         // absolute position of token 0
    int32_t kend[KATA_MAX_BATCH];        // local rows [first_row, kend) hold this call's keys; absolute key = key_off + row
    int32_t safe_row[KATA_MAX_BATCH];    // local rows below this are not being written by the kernel launched just before: they may be loaded before the dependent-launch wait
    int64_t row_base[KATA_MAX_BATCH];
    int32_t tile_start[KATA_MAX_BATCH + 1];
    int32_t ntiles[KATA_MAX_BATCH];      // tiles per KV head of sequence b (>= 1)
};

__host__ __device__ __forceinline__ int cta_first_tile(const DecPlan& p, int c) {
    if (p.cps) { const int seg = c / p.cps, j = c - seg * p.cps, nt = p.ntiles[0]; return seg * nt + (int)((int64_t)nt * j / p.cps); }
    return c * p.q_tiles + (c < p.r_tiles ? c : p.r_tiles);
}
__host__ __device__ __forceinline__ int cta_of_tile(const DecPlan& p, int tile) {
    if (p.cps) { const int nt = p.ntiles[0], seg = tile / nt, lt = tile - seg * nt; return seg * p.cps + (int)(((int64_t)(lt + 1) * p.cps + nt - 1) / nt) - 1; }   // the last share whose first tile is <= lt
    const int big = p.r_tiles * (p.q_tiles + 1);
    return tile < big ? tile / (p.q_tiles + 1) : p.r_tiles + (tile - big) / p.q_tiles;
}

template <int MODE>
__global__ void __launch_bounds__(kThreads, 1) decode_mma_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                                                                 const DecPlan p, const __half* __restrict__ q16, const float* __restrict__ gate, void* __restrict__ out, const int out_kind,
                                                                 float* __restrict__ part_out, const __half* __restrict__ ksc, const __half* __restrict__ vsc,
                                                                 float* scratch_o, float* scratch_ml, int32_t* counters, int32_t* err) {
    using G = Geo<MODE>; constexpr bool K8 = G::K8, V8 = G::V8, KG = G::KG; constexpr int kStages = G::kStages, kTile = G::kTile, NK = G::kNK; using PS = PSlot<NK>;
    if (threadIdx.x == 0) { prefetch_tmap(&tm_k); prefetch_tmap(&tm_v); dec_stamp(0); }
    if (!p.merge_in_kernel) pdl_launch_dependents();   // the next kernel is the combine grid, which starts no loads of its own before it has waited for this one: it may be set up at once
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5, ring = w & 3, h = w >> 2, g = lane >> 2, t4 = lane & 3;   // warps ring, ring+4 and ring+8 sit on the same scheduler: h = 0 score warp, h = 1, 2 value warps
    const uint32_t sm_base = smem_u32(smem);
    const uint32_t q_base = sm_base, bars = sm_base + kOffBars + ring * kMaxStages * 8, ebars = sm_base + kOffBars + kOffEBars + ring * kMaxStages * 8, stage_off = ((sm_base + kOffStages + 1023u) & ~1023u) - sm_base, ring_stage0 = sm_base + stage_off + ring * G::kRingBytes;   // swizzled TMA boxes want 1024-byte alignment
    float* sm_ml = reinterpret_cast<float*>(smem + kOffMl);
    const uint32_t p_sm = sm_base + kOffPair + ring * kPairBytes;
    const uint32_t pfull = sm_base + kOffBars + kOffPBars + ring * 16, pempty = pfull + kRings * 16;
    __shared__ int s_flag;

    if (h == 0 && lane == 0) { for (int s = 0; s < kStages; s++) { mbar_init(bars + s * 8, 1); mbar_init(ebars + s * 8, 3); } for (int s = 0; s < 2; s++) { mbar_init(pfull + s * 8, 1); mbar_init(pempty + s * 8, 2); } }
    fence_mbar_init();
    __syncthreads();
    // Launched with programmatic stream serialisation: everything above overlapped the previous kernel's tail. Each warp waits for that kernel
    // (griddepcontrol.wait) before it reads what it may have written (Q, gate, the newest cache rows, scratch); the producer warp first starts
    // the loads of tiles that kernel cannot touch. Dependents are released only after the wait, so whatever ran before the previous kernel is complete.
    bool waited = false;

    const int cta = blockIdx.x;
    int tile = cta_first_tile(p, cta); const int tile_end = cta_first_tile(p, cta + 1);
    int b = 0; uint32_t it = 0; bool dead = false;   // it: tiles this ring has consumed so far (ring position and phase)

    while (tile < tile_end) {
        while (p.tile_start[b + 1] <= tile) b++;
        const int nt = p.ntiles[b], kvl = (tile - p.tile_start[b]) / nt, kvh = p.kvh_lo + kvl, lt0 = (tile - p.tile_start[b]) - kvl * nt;
        const int seg_first = p.tile_start[b] + kvl * nt, seg_end = seg_first + nt, my_end = min(tile_end, seg_end), n_here = my_end - tile;
        const int T = p.T, kend = p.kend[b], pos_rel = p.pos[b] - p.key_off;   // token t sees local rows < min(kend, pos_rel + t + 1)

        // ---- this ring's tiles of the segment: local tiles lt0 + ring, lt0 + ring + 4, ...
        const int n_mine = n_here > ring ? (n_here - ring + kRings - 1) / kRings : 0;
        ScoreState ss;                 // softmax state, kept by the ring's score warp (h == 0)
        ValueStateT<16> vst; vst.clear();   // 16 x 128 half of the O block, kept by the ring's value warps (h == 1: dims 0..127, h == 2: dims 128..255)
        const int lim_row0 = (g < 6 * T) ? min(kend, pos_rel + (g >= 6 ? 1 : 0) + 1) : 0;          // rows g and g+8: exclusive local key limit
        const int lim_row1 = (g + 8 < 6 * T) ? min(kend, pos_rel + 2) : 0;                          // rows 8..11 belong to token 1

        const uint32_t it_seg = it;
        const int row0 = (int)p.row_base[b];   // arena row of position 0 (row coordinates of the tensor maps are 32-bit)
        // ---- producer warp (lane r serves ring r): brings in the ring's tiles of this segment, one TMA instruction for a K tile and one for a V
        // tile, refilling a stage as soon as the ring's three warps have released it. The first kStages tiles per ring fly while Q is staged.
        auto produce = [&](int i_from, int i_to) {
            const int r = lane, nm = n_here > r ? (n_here - r + kRings - 1) / kRings : 0;
            for (int i = i_from; i < min(i_to, nm); i++) {
                const uint32_t cur = it + (uint32_t)i, sx = cur % kStages;
                const uint32_t bar = sm_base + kOffBars + r * kMaxStages * 8 + sx * 8, ebar = bar + kOffEBars, dst = sm_base + stage_off + r * G::kRingBytes + sx * G::kStageBytes;
                if (i >= kStages && !dead && !mbar_wait_bounded(ebar, ((cur / kStages) - 1u) & 1u, err)) { dead = true; atomicExch(err, 3); }
                const int key0 = p.first_row + (lt0 + r + i * kRings) * kTile;
                mbar_arrive_expect_tx(bar, (uint32_t)G::kStageBytes);   // TMA counts whole boxes, out-of-range rows included
                tma_load_4d(dst, &tm_k, 0, row0 + key0, 0, kvh, bar); tma_load_4d(dst + G::kKTileBytes, &tm_v, 0, row0 + key0, 0, kvh, bar);
            }
            return nm;
        };
        if (h == 3) {   // every stage is free here
            int n_early = 0;
            if (!waited && lane < kRings) {   // leading tiles of this ring that lie wholly below the rows the previous kernel may be writing
                while (n_early < kStages && p.first_row + (lt0 + lane + n_early * kRings + 1) * kTile <= p.safe_row[b]) n_early++;
                produce(0, n_early);
            }
            if (!waited) { pdl_wait(); pdl_launch_dependents(); waited = true; }
            if (lane < kRings) produce(n_early, kStages);
        } else if (!waited) { pdl_wait(); pdl_launch_dependents(); waited = true; if (tid == 0) dec_stamp(1); }
        auto load_scale = [&](int i, const __half* plane) -> uint32_t {
            const int k0 = p.first_row + (lt0 + ring + i * kRings) * kTile;
            return __ldg(reinterpret_cast<const unsigned short*>(plane) + (p.row_base[b] + min(k0 + (lane & (kTile - 1)), max(kend - 1, 0))) * 4 + kvh);
        };
        auto load_kscale = [&](int i, uint32_t& lo, uint32_t& hi) {   // the key scale(s) of this lane's key of the ring's i-th tile: one fp16, or (int8g) four as two words
            if (!KG) { lo = load_scale(i, ksc); return; }
            const int k0 = p.first_row + (lt0 + ring + i * kRings) * kTile;
            const uint2 u = __ldg(reinterpret_cast<const uint2*>(ksc + (p.row_base[b] + min(k0 + (lane & (kTile - 1)), max(kend - 1, 0))) * 16 + kvh * 4));
            lo = u.x; hi = u.y;
        };
        uint32_t kA = 0, kB = 0, kC = 0, vA = 0, vB = 0, vC = 0, kA2 = 0, kB2 = 0, kC2 = 0;
        if (V8 && h == 0) {   // score warp: the loads fly while the Q block is staged
            if (n_mine > 0) { if (K8) load_kscale(0, kA, kA2); vA = load_scale(0, vsc); }
            if (n_mine > 1) { if (K8) load_kscale(1, kB, kB2); vB = load_scale(1, vsc); }
            if (n_mine > 2) { if (K8) load_kscale(2, kC, kC2); vC = load_scale(2, vsc); }
        }
        // ---- stage the 16-row Q block (rows t*6+j; rows >= 6T zero); int8 mode permutes columns inside each 16-dim block
        for (int ch = tid; ch < 16 * 32; ch += kThreads) {
            const int r = ch >> 5, c16 = ch & 31; uint4 v = make_uint4(0, 0, 0, 0);
            if (r < 6 * T) { const int t = r / 6, j = r - 6 * t; v = *reinterpret_cast<const uint4*>(q16 + ((int64_t)b * p.tok_stride + p.tok0 + t) * kQD + (kvh * 6 + j) * kD + c16 * 8); }
            stage_q_chunk<K8>(smem + r * kQStride, c16, v);
        }
        __syncthreads();
        if (K8) {   // row sums of the staged Q block (any column order): warp w sums rows 2w and 2w+1
#pragma unroll
            for (int rr = 0; rr < 2; rr++) {
                const int r = 2 * (w & 7) + rr; const uint4 v = *reinterpret_cast<const uint4*>(smem + r * kQStride + lane * 16); const __half2* hp = reinterpret_cast<const __half2*>(&v);
                float a = 0.0f;
#pragma unroll
                for (int e = 0; e < 4; e++) { const float2 f = __half22float2(hp[e]); a += f.x + f.y; }
                // a lane's 16 bytes are 8 dims of one 16-dim block (permuted inside it): lanes 8q .. 8q+7 hold the 64-dim group q
#pragma unroll
                for (int off = 4; off >= 1; off >>= 1) a += __shfl_xor_sync(0xffffffffu, a, off);
                if (KG && (lane & 7) == 0) reinterpret_cast<float*>(smem + kOffQsum)[16 + r * 4 + (lane >> 3)] = a;
                a += __shfl_xor_sync(0xffffffffu, a, 8); a += __shfl_xor_sync(0xffffffffu, a, 16);
                if (lane == 0) reinterpret_cast<float*>(smem + kOffQsum)[r] = a;
            }
            __syncthreads();
        }
        const float qs_[2] = {K8 ? reinterpret_cast<const float*>(smem + kOffQsum)[g] : 0.0f, K8 ? reinterpret_cast<const float*>(smem + kOffQsum)[g + 8] : 0.0f};
        float qsg_[2][4];
#pragma unroll
        for (int g4 = 0; g4 < 4; g4++) { qsg_[0][g4] = KG ? reinterpret_cast<const float*>(smem + kOffQsum)[16 + g * 4 + g4] : 0.0f; qsg_[1][g4] = KG ? reinterpret_cast<const float*>(smem + kOffQsum)[16 + (g + 8) * 4 + g4] : 0.0f; }

        if (h == 3) {
            if (lane < kRings) it += (uint32_t)produce(kStages, 1 << 30);   // 'it' of producer lane r counts ring r's tiles
            __syncwarp();
        } else if (h == 0) {
            // ---- score warp: S = Q K^T, online softmax, P and the rescale factors handed to the value warp; runs up to two tiles ahead
            // int8: lane j fetches the K and V scale of the tile's key j (mod the tile length), three tiles ahead; they are kept as raw fp16 bits so
            // that nothing depends on a load until its tile comes up (the scale planes are first touched here: DRAM latency)
            // (the first three tiles' scales were requested before the Q block was staged)
            for (int i = 0; i < n_mine; i++) {
                const uint32_t cur = it_seg + (uint32_t)i, stg = cur % kStages, par = (cur / kStages) & 1u, slot = cur & 1u;
                const uint32_t kt = ring_stage0 + stg * G::kStageBytes;
                const int key0 = p.first_row + (lt0 + ring + i * kRings) * kTile;
                const uint32_t k_cur = kA, k_cur2 = kA2, v_cur = vA; kA = kB; kB = kC; kA2 = kB2; kB2 = kC2; vA = vB; vB = vC;
                if (V8 && i + 3 < n_mine) { if (K8) load_kscale(i + 3, kC, kC2); vC = load_scale(i + 3, vsc); }
                // A wait that runs out is recorded once; afterwards waits are skipped but the control flow (and every arrival) stays intact.
                if (!dead && !mbar_wait_bounded(bars + stg * 8, par, err)) { dead = true; atomicExch(err, 1); }
                float ks_[2 * NK][2], vs_[2 * NK][2]; uint2 ksg_[2 * NK][2];
#pragma unroll
                for (int q = 0; q < 4 * NK; q++) {
                    const int src = 8 * (q >> 1) + 2 * t4 + (q & 1);
                    if (KG) { ksg_[q >> 1][q & 1] = make_uint2(__shfl_sync(0xffffffffu, k_cur, src), __shfl_sync(0xffffffffu, k_cur2, src)); ks_[q >> 1][q & 1] = 1.0f; }
                    else ks_[q >> 1][q & 1] = K8 ? __half2float(__ushort_as_half((unsigned short)__shfl_sync(0xffffffffu, k_cur, src))) : 1.0f;
                    vs_[q >> 1][q & 1] = V8 ? __half2float(__ushort_as_half((unsigned short)__shfl_sync(0xffffffffu, v_cur, src))) : 1.0f;
                }
                if (i == 0 && tid == 0 && it_seg == 0) dec_stamp(2);
                float pr[2 * NK][4], al0, al1;
                score_tile<K8, V8, NK, KG>(q_base, kt, key0, lim_row0, lim_row1, ks_, vs_, qs_, ss, lane, pr, al0, al1, ksg_, qsg_);
                __syncwarp();
                if (lane == 0) mbar_arrive(ebars + stg * 8);   // K of this stage is no longer needed
                if (cur >= 2 && !dead && !mbar_wait_bounded(pempty + slot * 8, ((cur >> 1) - 1u) & 1u, err)) { dead = true; atomicExch(err, 4); }
                score_publish<NK>(p_sm + slot * PS::kBytes, reinterpret_cast<float*>(smem + kOffPair + ring * kPairBytes + slot * PS::kBytes + 16 * PS::kStride), pr, al0, al1, lane);
                __syncwarp();
                if (lane == 0) mbar_arrive(pfull + slot * 8);
            }
            ss.l0 += __shfl_xor_sync(0xffffffffu, ss.l0, 1); ss.l0 += __shfl_xor_sync(0xffffffffu, ss.l0, 2);
            ss.l1 += __shfl_xor_sync(0xffffffffu, ss.l1, 1); ss.l1 += __shfl_xor_sync(0xffffffffu, ss.l1, 2);
            if (t4 == 0) { sm_ml[(ring * 16 + g) * 2] = ss.m0; sm_ml[(ring * 16 + g) * 2 + 1] = ss.l0; sm_ml[(ring * 16 + g + 8) * 2] = ss.m1; sm_ml[(ring * 16 + g + 8) * 2 + 1] = ss.l1; }
        } else {
            // ---- value warps: O = O * alpha + P V on their half of the head dims
            const int vh = h - 1;
            for (int i = 0; i < n_mine; i++) {
                const uint32_t cur = it_seg + (uint32_t)i, stg = cur % kStages, par = (cur / kStages) & 1u, slot = cur & 1u;
                const uint32_t vt = ring_stage0 + stg * G::kStageBytes + G::kKTileBytes;
                const int key0 = p.first_row + (lt0 + ring + i * kRings) * kTile;
                if (!dead && !mbar_wait_bounded(bars + stg * 8, par, err)) { dead = true; atomicExch(err, 1); }
                if (key0 + kTile > kend) {   // tail tile: rows past the range were loaded as they lie in memory; zero those V rows (0 x garbage must stay 0)
                    const int nk = max(0, kend - key0);
                    constexpr int kHB = G::kVBoxes / 2;   // boxes of this warp's half
                    for (int idx = lane; idx < (kTile - nk) * kHB * 8; idx += 32) {
                        const int r = nk + idx / (kHB * 8), rem = idx % (kHB * 8);
                        *reinterpret_cast<uint4*>(smem + (vt - sm_base) + (vh * kHB + (rem >> 3)) * (kTile * 128) + r * 128 + (rem & 7) * 16) = make_uint4(0, 0, 0, 0);
                    }
                    fence_proxy_async();   // generic-proxy writes to a stage that a TMA write refills later
                    __syncwarp();
                }
                if (!dead && !mbar_wait_bounded(pfull + slot * 8, (cur >> 1) & 1u, err)) { dead = true; atomicExch(err, 5); }
                value_tile<V8, 16, NK>(vt, p_sm + slot * PS::kBytes, reinterpret_cast<const float*>(smem + kOffPair + ring * kPairBytes + slot * PS::kBytes + 16 * PS::kStride), vst, lane, vh);
                __syncwarp();
                if (lane == 0) { mbar_arrive(pempty + slot * 8); mbar_arrive(ebars + stg * 8); }
            }
            if (V8) vst.finish_bias(kI8Bias);
        }
        if (h != 3) it = it_seg + (uint32_t)n_mine;

        // ---- merge the 4 rings of the CTA (every issued tile was waited for, so no copy is in flight)
        __syncthreads();
        if (tid == 0) dec_stamp(3);
        float* mo = reinterpret_cast<float*>(smem + stage_off + ring * G::kRingBytes);
        if (h == 1 || h == 2) {
#pragma unroll
            for (int j = 0; j < 16; j++)
#pragma unroll
                for (int c = 0; c < 2; c++) { const int d = pair_dim_of<V8>(h - 1, j, c, t4); mo[g * kMergeStride + d] = vst.o[j][c]; mo[(g + 8) * kMergeStride + d] = vst.o[j][2 + c]; }
        }
        __syncthreads();

        const int seg = b * 4 + kvh, c_first = cta_of_tile(p, seg_first), c_last = cta_of_tile(p, seg_end - 1), n_contrib = c_last - c_first + 1;
        const int d0 = 2 * (tid & 127), rsel = tid >> 7; const bool merger = h < 3;   // a thread of the 12 ring warps merges dims d0, d0+1 of rows rsel, rsel+3, ...
        const bool whole = (n_contrib == 1);
        const int rows = 6 * T;
        float* slot_o = scratch_o + (int64_t)(cta + seg) * (12 * kD); float* slot_ml = scratch_ml + (int64_t)(cta + seg) * 32;
        auto emit = [&](int r, float M, float L, float A0, float A1) {   // final value of row r, dims d0, d0+1
            const int t = r / 6, j = r - 6 * t, head = kvh * 6 + j;
            if (part_out) { float* po = part_out + ((int64_t)(b * p.tok_stride + p.tok0 + t) * kH + head) * kPartStride; po[d0] = A0; po[d0 + 1] = A1; if ((tid & 127) == 0) { po[256] = M * 0.6931471805599453f; po[257] = L; } }
            else {
                const int64_t oi = ((int64_t)b * p.tok_stride + p.tok0 + t) * kQD + head * kD + d0; const float2 gt = *reinterpret_cast<const float2*>(gate + oi);
                const float y0 = (A0 / L) * sigmoid_fast(gt.x), y1 = (A1 / L) * sigmoid_fast(gt.y);
                store_act2(out, oi, y0, y1, out_kind);
            }
        };
        for (int r = merger ? rsel : rows; r < rows; r += kThreads / 128) {
            float M = -INFINITY;
#pragma unroll
            for (int ww = 0; ww < kRings; ww++) M = fmaxf(M, sm_ml[(ww * 16 + r) * 2]);
            float L = 0.0f, A0 = 0.0f, A1 = 0.0f;
#pragma unroll
            for (int ww = 0; ww < kRings; ww++) {
                const float mm = sm_ml[(ww * 16 + r) * 2]; const float wt = (mm == -INFINITY) ? 0.0f : ex2(mm - M);
                const float* src = reinterpret_cast<const float*>(smem + stage_off + ww * G::kRingBytes) + r * kMergeStride + d0;
                L += sm_ml[(ww * 16 + r) * 2 + 1] * wt; A0 += src[0] * wt; A1 += src[1] * wt;
            }
            if (whole) emit(r, M, L, A0, A1);
            else { *reinterpret_cast<float2*>(slot_o + r * kD + d0) = make_float2(A0, A1); if ((tid & 127) == 0) { slot_ml[r * 2] = M; slot_ml[r * 2 + 1] = L; } }
        }
        if (!whole && p.merge_in_kernel) {   // ticket: the last contributor of the segment merges everybody's partials
            __threadfence();
            __syncthreads();
            if (tid == 0) { const int old = atomicAdd(&counters[seg], 1); s_flag = (old == n_contrib - 1); }
            __syncthreads();
            if (s_flag) {
                // Every contributor's partial is visible (ticket + fences). At most 8 contributors: every thread pulls its two dims of its rows straight
                // from L2 (independent loads), forms the row maximum and the weights exp(m - M), and emits the final rows.
                __threadfence();
                for (int r = merger ? rsel : rows; r < rows; r += kThreads / 128) {
                    float M = -INFINITY;
                    for (int c = 0; c < n_contrib; c++) M = fmaxf(M, __ldcg(scratch_ml + (int64_t)(c_first + c + seg) * 32 + r * 2));
                    float L = 0.0f, A0 = 0.0f, A1 = 0.0f;
#pragma unroll 4
                    for (int c = 0; c < n_contrib; c++) {
                        const int64_t sl = c_first + c + seg; const float mm = __ldcg(scratch_ml + sl * 32 + r * 2); const float wt = (mm == -INFINITY) ? 0.0f : ex2(mm - M);
                        const float2 oo = __ldcg(reinterpret_cast<const float2*>(scratch_o + sl * (12 * kD) + r * kD + d0));
                        L += __ldcg(scratch_ml + sl * 32 + r * 2 + 1) * wt; A0 += oo.x * wt; A1 += oo.y * wt;
                    }
                    emit(r, M, L, A0, A1);
                }
                if (tid == 0) counters[seg] = 0;   // ready for the next call on this stream
            }
        }
        __syncthreads();   // merge buffers and the Q block are reused by the next segment
        tile = my_end;
    }
    if (tid == 0) dec_stamp(4);
}

// Merge of the per-CTA partials of every split segment, one CTA per (row, segment). Used instead of the in-kernel ticket merge when a segment
// has many contributors (batch 1 at long context: 37 per KV head; 256 per KV head with the reference's 128-key splits at 32K): a single
// last-arriver CTA would pull all of them through one SM, while this grid does it in parallel: 1024 threads = 4 groups of 256 head dims,
// group q folding contributors q, q+4, ... with a running maximum of its own (nothing is sized by the contributor count). Launched with programmatic stream serialisation: the grid is set up while the decode kernel drains and waits for it here.
constexpr int kCombineThreads = 1024;
__global__ void __launch_bounds__(kCombineThreads) decode_combine_kernel(const DecPlan p, const float* __restrict__ gate, void* __restrict__ out, const int out_kind, float* __restrict__ part_out,
                                                                         const float* __restrict__ scratch_o, const float* __restrict__ scratch_ml, const PeerSink px) {
    __shared__ float s_acc[4][256]; __shared__ float s_Mq[4], s_Lq[4]; __shared__ int s_ok;
    const int r = blockIdx.x, b = blockIdx.y / p.kvh_n, kvl = blockIdx.y % p.kvh_n, kvh = p.kvh_lo + kvl, seg = b * 4 + kvh, tid = threadIdx.x, d = tid & 255, q = tid >> 8;
    const int nt = p.ntiles[b], seg_first = p.tile_start[b] + kvl * nt, c_first = cta_of_tile(p, seg_first), c_last = cta_of_tile(p, seg_first + nt - 1), n_c = c_last - c_first + 1;
    pdl_wait();              // the decode kernel's partials are complete and visible from here on
    pdl_launch_dependents();
#ifdef KATA_PF_TRACE
    if (tid == 0) { unsigned long long tt; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(tt)); g_dec_trace[(1400 + blockIdx.y * 12 + blockIdx.x) * 8 + 5] = tt; }
#endif
    const int t = r / 6, j = r - 6 * t, head = kvh * 6 + j;
    float A, M, L;
    if (n_c == 1) {   // a single contributor wrote the final row itself; only a cross-GPU exchange still has work to do with it
        if (px.world == 0 || q) return;
        const float* po = part_out + ((int64_t)(b * p.tok_stride + p.tok0 + t) * kH + head) * kPartStride;
        A = po[d]; M = po[256] * 1.4426950408889634f; L = po[257];
    } else {
        // Group q of 256 threads takes contributors q, q + 4, ...: every thread requests (m, l, O[d]) of up to twelve of them at once (one round
        // trip to L2 for the 37 contributors of a 32K sequence; m and l are the same addresses across a group: broadcasts) and folds them
        // into its own running (M, L, A); the four groups are then folded through shared memory.
        const float* ml = scratch_ml + (int64_t)(c_first + seg) * 32 + r * 2;   // contributor c: ml[c * 32] = m, ml[c * 32 + 1] = l
        const float* po = scratch_o + (int64_t)(c_first + seg) * (12 * kD) + r * kD + d;
        float Mq = -INFINITY, Lq = 0.0f, Aq = 0.0f;
        for (int c0 = q; c0 < n_c; c0 += 48) {
            float mm[12], ll[12], oo[12];
#pragma unroll
            for (int u = 0; u < 12; u++) {
                const int c = c0 + 4 * u; const bool ok = c < n_c;
                mm[u] = ok ? __ldcg(ml + c * 32) : -INFINITY; ll[u] = ok ? __ldcg(ml + c * 32 + 1) : 0.0f; oo[u] = ok ? __ldcg(po + (int64_t)c * (12 * kD)) : 0.0f;
            }
            float Mn = Mq;
#pragma unroll
            for (int u = 0; u < 12; u++) Mn = fmaxf(Mn, mm[u]);
            const float keep = (Mq == -INFINITY) ? 0.0f : ex2(Mq - Mn);
            Aq *= keep; Lq *= keep; Mq = Mn;
#pragma unroll
            for (int u = 0; u < 12; u++) { const float wt = (mm[u] == -INFINITY) ? 0.0f : ex2(mm[u] - Mn); Aq = fmaf(oo[u], wt, Aq); Lq = fmaf(ll[u], wt, Lq); }
        }
        s_acc[q][d] = Aq;
        if (d == 0) { s_Mq[q] = Mq; s_Lq[q] = Lq; }
        __syncthreads();
        if (q) return;
        M = fmaxf(fmaxf(s_Mq[0], s_Mq[1]), fmaxf(s_Mq[2], s_Mq[3]));
        A = 0.0f; L = 0.0f;
#pragma unroll
        for (int g4 = 0; g4 < 4; g4++) { const float wt = (s_Mq[g4] == -INFINITY) ? 0.0f : ex2(s_Mq[g4] - M); A = fmaf(s_acc[g4][d], wt, A); L = fmaf(s_Lq[g4], wt, L); }
    }
    // 256 threads from here on (thread d = head dim d)
    if (px.world > 0) {   // split-KV across GPUs: this rank's row goes straight into the exchange (push to the peers, wait for theirs, merge, gate)
        peer_row_exchange(px, t, head, d, A, M * 0.6931471805599453f, L, gate, out, out_kind, &s_ok, 1);
    } else if (part_out) { float* po2 = part_out + ((int64_t)(b * p.tok_stride + p.tok0 + t) * kH + head) * kPartStride; po2[d] = A; if (d == 0) { po2[256] = M * 0.6931471805599453f; po2[257] = L; } }
    else {
        const int64_t oi = ((int64_t)b * p.tok_stride + p.tok0 + t) * kQD + head * kD + d; const float y = (A / L) * sigmoid_fast(gate[oi]);
        store_act(out, oi, y, out_kind);
    }
#ifdef KATA_PF_TRACE
    if (tid == 0) { unsigned long long tt; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(tt)); g_dec_trace[(1400 + blockIdx.y * 12 + blockIdx.x) * 8 + 6] = tt; }
#endif
}

// Merge of per-rank partials {O[256], m, l} (m in natural-log units) and the output gate: k_attn_dec_combine with "split" = rank.
__global__ void __launch_bounds__(256) merge_parts_kernel(const float* __restrict__ parts, const int n_parts, const int T, const float* __restrict__ gate, void* __restrict__ out, const int out_kind) {
    const int h = blockIdx.x, t = blockIdx.y, tid = threadIdx.x; const int64_t row = (int64_t)t * kH + h, stride = (int64_t)T * kH * kPartStride;
    float M = -INFINITY; for (int r = 0; r < n_parts; r++) M = fmaxf(M, parts[r * stride + row * kPartStride + 256]);
    float L = 0.0f, A = 0.0f;
    for (int r = 0; r < n_parts; r++) { const float* pp = parts + r * stride + row * kPartStride; const float mm = pp[256]; const float wt = (mm == -INFINITY) ? 0.0f : expf(mm - M); L = fmaf(pp[257], wt, L); A = fmaf(pp[tid], wt, A); }   // one fused multiply-add per part, as the peer exchange forms the same sums
    const int64_t oi = (int64_t)t * kQD + h * kD + tid; const float y = (A / L) * (1.0f / (1.0f + expf(-gate[oi])));
    store_act(out, oi, y, out_kind);
}

}  // namespace

#ifdef KATA_PF_TRACE
extern "C" int kata_debug_dec_trace(unsigned long long* h) { return (int)cudaMemcpyFromSymbol(h, g_dec_trace, sizeof(g_dec_trace)); }
#endif

int decode_max_slots(int sm_count) { return sm_count + 4 * KATA_MAX_BATCH; }

// Shared-memory opt-in of the decode kernel on the current device (function attributes are per device: done once per context).
cudaError_t configure_decode(int kv_mode) {
    return kv_mode == KATA_KV_INT8G ? cudaFuncSetAttribute(decode_mma_kernel<KATA_KV_INT8G>, cudaFuncAttributeMaxDynamicSharedMemorySize, Geo<KATA_KV_INT8G>::kSmem)
         : kv_mode == KATA_KV_INT8  ? cudaFuncSetAttribute(decode_mma_kernel<KATA_KV_INT8>, cudaFuncAttributeMaxDynamicSharedMemorySize, Geo<KATA_KV_INT8>::kSmem)
         : kv_mode == KATA_KV_INT8V ? cudaFuncSetAttribute(decode_mma_kernel<KATA_KV_INT8V>, cudaFuncAttributeMaxDynamicSharedMemorySize, Geo<KATA_KV_INT8V>::kSmem)
                                    : cudaFuncSetAttribute(decode_mma_kernel<KATA_KV_FP16>, cudaFuncAttributeMaxDynamicSharedMemorySize, Geo<KATA_KV_FP16>::kSmem);
}

static int max_contributors(const DecPlan& p) {
    auto cta_of = [&](int tile) { return cta_of_tile(p, tile); };
    int m = 1;
    for (int i = 0; i < p.n; i++) for (int kv = 0; kv < p.kvh_n; kv++) { const int f = p.tile_start[i] + kv * p.ntiles[i]; m = std::max(m, cta_of(f + p.ntiles[i] - 1) - cta_of(f) + 1); }
    return m;
}

// The work split of a decode launch (host code only): p.n, p.kend[], p.first_row and p.kvh_n are set; fills the tile counts, the CTA ranges and
// the choice of where the segments' partials are merged. tile_keys: 16 (fp16 keys) or 32 (int8 keys).
static void split_decode_tiles(DecPlan& p, const int tile_keys, const int sm_count, const int dec_chunk, const int max_items) {
    int total = 0;
    for (int i = 0; i < p.n; i++) {
        const int nkeys = std::max(0, p.kend[i] - p.first_row); p.ntiles[i] = std::max(1, (nkeys + tile_keys - 1) / tile_keys);
        p.tile_start[i] = total; total += p.kvh_n * p.ntiles[i];
    }
    for (int i = p.n; i <= KATA_MAX_BATCH; i++) p.tile_start[i] = total;
    const int chunk_tiles = dec_chunk > 0 ? std::max(1, dec_chunk / tile_keys) : 0;
    int n_ctas = chunk_tiles ? (total + chunk_tiles - 1) / chunk_tiles : sm_count;
    n_ctas = std::max(1, std::min(std::min(n_ctas, total), sm_count * 8));
    if (n_ctas + 4 * p.n > max_items) n_ctas = max_items - 4 * p.n;
    p.cps = 0; p.n_ctas = n_ctas; p.q_tiles = total / n_ctas; p.r_tiles = total % n_ctas;
    // A CTA whose range crosses from one segment into the next pays for it (ring merge, partial write, the Q block of the next segment, the
    // pipeline filled again: 4 to 5 us measured, which made the few such CTAs the last to finish). When all segments are equally long (one
    // sequence, or a batch of equal lengths) and their number divides nearly all SMs, every segment gets the same number of CTAs of its own.
    if (!chunk_tiles) {
        bool same = true; for (int i = 1; i < p.n; i++) same = same && p.ntiles[i] == p.ntiles[0];
        const int n_seg = p.n * p.kvh_n, cps = n_seg <= sm_count ? sm_count / n_seg : 0;
        if (same && cps >= 1 && cps * n_seg * 100 >= sm_count * 97 && p.ntiles[0] >= cps && cps * n_seg + 4 * p.n <= max_items) { p.cps = cps; p.n_ctas = cps * n_seg; p.q_tiles = p.ntiles[0] / cps; p.r_tiles = p.ntiles[0] % cps; }
    }
    p.merge_in_kernel = max_contributors(p) <= 8;   // contributors of the most-split segment decide where the merge runs
}

// The same as plain arrays, for tests of the host logic that have no GPU: kend[b] keys (from first_row on) per sequence. first_tile takes n_ctas + 1
// entries (CTA c works on tiles [first_tile[c], first_tile[c + 1]) of the list: sequence after sequence, KV head after KV head, ntiles[b] tiles each).
// Returns the number of CTAs, or -1 for arguments out of range.
extern "C" int kata_attn_decode_plan(int32_t n, const int32_t* kend, int32_t first_row, int32_t kvh_n, int32_t tile_keys, int32_t sm_count, int32_t dec_chunk, int32_t max_items,
                                     int32_t* ntiles, int32_t* first_tile, int32_t first_tile_cap, int32_t* cps, int32_t* merge_in_kernel, int32_t* max_contrib) {
    if (n < 1 || n > KATA_MAX_BATCH || !kend || kvh_n < 1 || kvh_n > KATA_KV_HEADS || (tile_keys != 16 && tile_keys != 32) || sm_count < 1 || max_items <= 4 * n || !ntiles || !first_tile || !cps || !merge_in_kernel || !max_contrib) return -1;
    DecPlan p{}; p.n = n; p.T = 1; p.first_row = first_row; p.kvh_lo = 0; p.kvh_n = kvh_n;
    for (int i = 0; i < n; i++) p.kend[i] = kend[i];
    split_decode_tiles(p, tile_keys, sm_count, dec_chunk, max_items);
    if (p.n_ctas + 1 > first_tile_cap) return -1;
    for (int i = 0; i < n; i++) ntiles[i] = p.ntiles[i];
    for (int cta = 0; cta <= p.n_ctas; cta++) first_tile[cta] = cta < p.n_ctas ? cta_first_tile(p, cta) : p.tile_start[KATA_MAX_BATCH];
    for (int cta = 0; cta < p.n_ctas; cta++) for (int tile = first_tile[cta]; tile < (cta + 1 < p.n_ctas ? cta_first_tile(p, cta + 1) : p.tile_start[KATA_MAX_BATCH]); tile++) if (cta_of_tile(p, tile) != cta) return -2;   // the two maps disagree
    *cps = p.cps; *merge_in_kernel = p.merge_in_kernel; *max_contrib = max_contributors(p);
    return p.n_ctas;
}

// key_off / kend_override serve the split-KV-across-GPUs call: local row = absolute key - key_off, rows [first_row, kend).
cudaError_t launch_decode_mma_ex(Ctx& c, const Batch& b, int T, int first_row, int key_off, const int32_t* kend_override, const __half* q16, const float* gate, void* out, int out_dtype,
                                 float* part_out, cudaStream_t s, int tok_stride, int tok0, const PeerSink* sink, bool* sink_used) {
    if (sink_used) *sink_used = false;
    const int mode = c.cfg.kv_mode, kTile = c.k8() ? 32 : 16;
    DecPlan p{}; p.n = b.n; p.T = T; p.first_row = first_row; p.key_off = key_off; p.kvh_lo = c.kvh_lo; p.kvh_n = c.kvh_n; p.tok_stride = tok_stride > 0 ? tok_stride : T; p.tok0 = tok0;
    for (int i = 0; i < b.n; i++) {
        p.pos[i] = b.pos[i]; p.row_base[i] = b.row_base[i]; p.kend[i] = kend_override ? kend_override[i] : b.pos[i] + T;
        p.safe_row[i] = c.prev_append ? std::min<int64_t>(p.kend[i], (int64_t)c.append_lo[b.seq[i]] - key_off) : p.kend[i];
    }
    split_decode_tiles(p, kTile, c.sm_count, c.cfg.dec_chunk, c.max_items);
    const int n_ctas = p.n_ctas;
    // Early loads pay when a CTA streams for long (batch 8 at 16-32K: -2 us of 140); with short ranges (batch 1: 55 tiles per CTA) they take
    // bandwidth from the previous kernel's last CTAs, which everybody then waits for (+2 us of 31): switched off there.
    // Nor are rows loaded early while caller kernels may be writing any of them through a plane pointer without having said which.
    if (p.q_tiles < 128 || (c.ext_ptr && !c.ext_declared)) for (int i = 0; i < b.n; i++) p.safe_row[i] = 0;
    const CUtensorMap& mk = c.tm_k_tile; const CUtensorMap& mv = c.tm_v_tile;
#define KATA_DEC(M) launch_pdl(decode_mma_kernel<M>, dim3(n_ctas), dim3(kThreads), Geo<M>::kSmem, s, mk, mv, p, q16, gate, out, out_dtype, part_out, c.ksc, c.vsc, c.part_o, c.part_ml, c.counters, c.d_err)
    static_assert(Geo<KATA_KV_INT8>::kTile == 32 && Geo<KATA_KV_INT8G>::kTile == 32 && Geo<KATA_KV_INT8V>::kTile == 16 && Geo<KATA_KV_FP16>::kTile == 16, "the tile views of the context are built for these tile heights");
    const cudaError_t le = mode == KATA_KV_INT8G ? KATA_DEC(KATA_KV_INT8G) : mode == KATA_KV_INT8 ? KATA_DEC(KATA_KV_INT8) : mode == KATA_KV_INT8V ? KATA_DEC(KATA_KV_INT8V) : KATA_DEC(KATA_KV_FP16);
#undef KATA_DEC
    c.wrote_no_rows();   // this kernel writes no cache rows
    if (le != cudaSuccess) return le;
    c.launches++;
    if (!p.merge_in_kernel) {
        // with a cross-GPU exchange to feed (one sequence, rows in [T][6144] order) the combine grid does the exchange as well
        const bool fuse = sink && sink->world > 0 && b.n == 1 && tok0 == 0 && p.tok_stride == T;
        const cudaError_t e = launch_pdl(decode_combine_kernel, dim3(6 * T, c.kvh_n * b.n), dim3(kCombineThreads), 0, s, p, gate, out, (int)out_dtype, part_out, (const float*)c.part_o, (const float*)c.part_ml, fuse ? *sink : PeerSink{});
        if (fuse && sink_used && e == cudaSuccess) *sink_used = true;
        if (e != cudaSuccess) return e;
        c.launches++;
    }
    return cudaGetLastError();
}

cudaError_t launch_decode_mma(Ctx& c, const Batch& b, int T, int first_pos, int, const __half* q16, const float* gate, void* out, int out_dtype, float* part_out, cudaStream_t s) {
    return launch_decode_mma_ex(c, b, T, first_pos, 0, nullptr, q16, gate, out, out_dtype, part_out, s, T, 0, nullptr, nullptr);
}

cudaError_t launch_merge_parts(Ctx& c, const float* parts, int n_parts, int T, const float* gate, void* out, int out_dtype, cudaStream_t s) {
    merge_parts_kernel<<<dim3(kH, T), 256, 0, s>>>(parts, n_parts, T, gate, out, out_dtype);
    c.launches++;
    return cudaGetLastError();
}

}  // namespace kata

// =====================================================================================================================
// kata_attn_decode_static: the decode/verify kernel above for callers that cannot allocate device memory.
//
// Who that is: a host engine that hands the whole GPU to its own memory pools at start-up (a later cudaMalloc from a
// library simply fails there), and serving loops where cudaMalloc/cudaFree are banned because they synchronise the
// device. Such a caller owns the K/V rows itself and has no kata_attn_ctx (creating one allocates the caches and scratch).
//
// The split-KV partials, their (m, l) pairs, the per-segment tickets and the error word live in the file-scope array
// below instead of context memory. It has a fixed size (about 2.2 MB), is part of the library image, and every GPU that
// loads the library keeps it until the process exits. Consequences the caller must know:
//  - Limits: at most KATA_STATIC_MAX_BATCH sequences per call and at most 148 CTAs (more SMs are simply not used);
//    a larger batch is rejected with KATA_ERR_RANGE. fp16 rows only.
//  - The first call on a device performs the set-up for that device (symbol address lookup, shared-memory opt-in);
//    make that first call outside any stream capture.
//  - All calls on a device share the array and it keeps the previous call's contents. The ticket counters and the
//    error word are cleared on the stream before every launch; partial slots are always written before they are read.
//    Two calls that overlap on the GPU (different streams, or the same call issued from two threads) race on the array:
//    serialise them.
namespace kata {
namespace {

constexpr int kStaticMaxBatch = KATA_STATIC_MAX_BATCH, kStaticMaxCtas = 148, kStaticSlots = kStaticMaxCtas + 4 * kStaticMaxBatch;
struct StaticScratch {
    float part_o[kStaticSlots * 12 * kD];      // unnormalised partial O rows per (CTA, segment) slot
    float part_ml[kStaticSlots * 32];          // their (m, l)
    int32_t counters[4 * KATA_MAX_BATCH];      // segment tickets: must be zero at launch
    int32_t err;                               // set when a bounded device wait runs out
};
static __device__ __align__(256) unsigned char g_static_scratch[sizeof(StaticScratch)];

struct StaticDev { bool ready = false; StaticScratch* scratch = nullptr; int sm_count = 0; };
StaticDev g_static_dev[64];

}  // namespace
}  // namespace kata

// Reports what the static scratch's error word says after the calls enqueued so far on `stream` have completed: KATA_ERR_DEVICE_WAIT when a
// bounded device wait ran out in one of them (their output is then invalid), else KATA_OK. Synchronises the stream; allocates nothing (a
// 4-byte copy from the array inside the library image). The word is cleared before every launch, so it speaks for the last call.
extern "C" int kata_attn_decode_static_check(void* stream) {
    using namespace kata;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return KATA_ERR_CUDA;
    if (cudaStreamSynchronize((cudaStream_t)stream) != cudaSuccess) return KATA_ERR_CUDA;
    if (!g_static_dev[dev].ready) return KATA_OK;   // nothing was ever launched on this device
    int32_t flag = 0;
    if (cudaMemcpy(&flag, &g_static_dev[dev].scratch->err, 4, cudaMemcpyDeviceToHost) != cudaSuccess) return KATA_ERR_CUDA;
    return flag ? KATA_ERR_DEVICE_WAIT : KATA_OK;
}

extern "C" int kata_attn_decode_static(const void* d_k_rows, const void* d_v_rows, int64_t total_rows, int32_t n, const int64_t* seq_row0, const int32_t* pos_base,
                                       int32_t T, int32_t first_pos, const void* d_q16, const float* d_gate, void* d_out, int32_t out_dtype, void* stream) {
    using namespace kata;
    if (!d_k_rows || !d_v_rows || !seq_row0 || !pos_base || !d_q16 || !d_gate || !d_out) return KATA_ERR_ARG;
    if (out_dtype != KATA_ACT_F32 && out_dtype != KATA_ACT_BF16 && out_dtype != KATA_ACT_F16) return KATA_ERR_ARG;
    if (n < 1 || n > kStaticMaxBatch || T < 1 || T > 2 || total_rows < 1 || total_rows > 0x7fffffffLL) return KATA_ERR_RANGE;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return KATA_ERR_CUDA;
    StaticDev& sd = g_static_dev[dev];
    if (!sd.ready) {   // once per device, with that device current: the array's name is only a host-side handle, the kernel needs its device address
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || !ptr) return KATA_ERR_CUDA;
        if (cudaFuncSetAttribute(decode_mma_kernel<KATA_KV_FP16>, cudaFuncAttributeMaxDynamicSharedMemorySize, Geo<KATA_KV_FP16>::kSmem) != cudaSuccess) return KATA_ERR_CUDA;
        if (cudaDeviceGetAttribute(&sd.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return KATA_ERR_CUDA;
        sd.scratch = static_cast<StaticScratch*>(ptr); sd.ready = true;
    }
    DecPlan p{}; p.n = n; p.T = T; p.first_row = first_pos; p.key_off = 0; p.tok_stride = T; p.tok0 = 0; p.kvh_lo = 0; p.kvh_n = kKvh;
    int total = 0;
    for (int i = 0; i < n; i++) {
        if (pos_base[i] < 0 || first_pos < 0 || first_pos > pos_base[i] || seq_row0[i] < 0 || seq_row0[i] + pos_base[i] + T > total_rows) return KATA_ERR_RANGE;
        p.pos[i] = pos_base[i]; p.row_base[i] = seq_row0[i]; p.kend[i] = pos_base[i] + T;
        p.ntiles[i] = std::max(1, (p.kend[i] - first_pos + Geo<KATA_KV_FP16>::kTile - 1) / Geo<KATA_KV_FP16>::kTile);
        p.tile_start[i] = total; total += 4 * p.ntiles[i];
    }
    for (int i = n; i <= KATA_MAX_BATCH; i++) p.tile_start[i] = total;
    const int n_ctas = std::max(1, std::min(std::min(sd.sm_count, kStaticMaxCtas), total));
    p.n_ctas = n_ctas; p.q_tiles = total / n_ctas; p.r_tiles = total % n_ctas; p.merge_in_kernel = max_contributors(p) <= 8;
    CUtensorMap tm_k, tm_v;   // encoded on the host; no device memory involved
    if (!make_tile_tmap(&tm_k, const_cast<void*>(d_k_rows), 2, total_rows, 16, 4) || !make_tile_tmap(&tm_v, const_cast<void*>(d_v_rows), 2, total_rows, 16, 4)) return KATA_ERR_CUDA;
    cudaStream_t s = (cudaStream_t)stream;
    if (cudaMemsetAsync(sd.scratch->counters, 0, sizeof(StaticScratch::counters) + sizeof(int32_t), s) != cudaSuccess) return KATA_ERR_CUDA;   // tickets and the error word start at zero
    decode_mma_kernel<KATA_KV_FP16><<<n_ctas, kThreads, Geo<KATA_KV_FP16>::kSmem, s>>>(tm_k, tm_v, p, (const __half*)d_q16, d_gate, d_out, out_dtype, nullptr, nullptr, nullptr,
                                                                         sd.scratch->part_o, sd.scratch->part_ml, sd.scratch->counters, &sd.scratch->err);
    if (!p.merge_in_kernel) decode_combine_kernel<<<dim3(6 * T, 4 * n), kCombineThreads, 0, s>>>(p, d_gate, d_out, (int)out_dtype, nullptr, sd.scratch->part_o, sd.scratch->part_ml, PeerSink{});
    return cudaGetLastError() == cudaSuccess ? KATA_OK : KATA_ERR_CUDA;
}
