// Causal flash prefill on the 5th-generation tensor cores (tcgen05) for the fp16 KV cache (int8 planes go through an fp16 staging arena).
// Replaces k_cvt_q_half + k_flash_prefill[_q8 | _k16v8] of the reference (shaders/flash.metal:10-71, 198-250; encoded at src/engine.cpp:279,
// 614) with the same math: fp16 Q (prescaled by 1/16) x fp16 K -> fp32 scores, causal mask key > position -> -inf,
// online softmax, P rounded to fp16 before P.V, l summed from the unrounded p, output O / l * sigmoid(gate).
//
// A work item = 128 query rows of two heads of the same KV-head group (row r of the chunk sits at position pos_base + r and sees keys
// [0, pos_base + r]), done by two CTAs (a cluster, cta_group::2). The kernel is persistent: one CTA pair per two SMs, with its barriers,
// tensor memory and pipelines kept across items; the next item's Q, K and V loads and first score MMAs run under the current item's epilogue.
// Work split (PfPlan, made on the host): the items of one (sequence, KV head) are neighbours in the list; a pair first computes whole items dealt in
// rounds, so that a dozen pairs read the same K and V tiles at the same time, then one contiguous range of the key tiles of the remaining items,
// sized so that all pairs carry the same load; with fewer items than pairs (one sequence: 48 items for 74 pairs) the ranges are all there is and
// every SM is still used. The parts of a cut item lie on consecutive pairs: its head (the tiles from 0) is the last part of its pair's range,
// every other part the first of its pair's. A pair computes such a part, writes the unnormalised O rows with their (m, l) to scratch and
// raises the part's flag; the pair that holds the head finishes the item: once its own tiles are done (its Q, K and V tiles are then free)
// its softmax warps copy the other parts into that shared memory as their flags come up and fold them into O in tensor memory with the
// split-KV rule of the decode path (weights exp(m - M)) before the usual epilogue. (A merge kernel behind this one was used before: its CTAs
// could not start until the pairs had left the SMs, and it re-read 30 MB of parts through L2: 15 us after a 50 us launch at batch 1.
// Merging by plain loads in the CTA that finished an item's last part was tried before that: 20 us per item.)
// The host cuts items only when its estimate says the shorter critical path pays for the fold. The pair works on M = 256 tiles: each CTA holds its own head's Q block and O/S
// accumulators and half of every K tile (64 of the 128 keys) and V tile (128 of the 256 dims); the tensor cores of the two SMs exchange
// the halves, so each SM writes and reads half the K/V bytes through its shared memory, which is what bounds an M = 128 tile with
// 256-wide heads (Q, K, V tiles plus their TMA writes ask for more than the 128 bytes per clock an SM's shared memory delivers).
//   warps 0-7  softmax: two threads per query row (tensor-memory lane = row): warp w < 4 takes the first 64 keys of a tile, warp w + 4
//              the last 64; the pair exchanges its row maxima through shared memory (64-thread named barrier) once per tile, each
//              writes its half of P, keeps its own partial l, and owns 128 of the 256 O columns for rescales and the epilogue
//   warp 8     TMA producer for Q (once) and the K half-tiles;  warp 9  TMA producer for the V half-tiles
//   warp 10    (even CTA only) issues the MMAs and commits for both CTAs (one elected thread)
// Shared memory per CTA: Q (4 column blocks of [128 rows][128 bytes]), two stages of a K half-tile (4 blocks of [64 keys][128 bytes]) and
// two stages of a V half-tile (2 blocks of [128 keys][128 bytes]), all with the 128-byte swizzle, exactly as TMA writes them and as the MMA
// descriptors read them (Q, K: K-major; V: MN-major, so the [key][dim] rows of the cache are used as they lie). TMA loads of both CTAs count
// their bytes on the even CTA's 'full' barriers; 'empty', 'scores ready' and 'O done' are committed to both CTAs at once.
// Tensor memory (512 columns per CTA): O 128x256 fp32 in columns [0,256), two score buffers S0, S1 of 128x128 fp32 in [256,384) and
// [384,512); P (fp16, two per column) overwrites the first 64 columns of its S buffer and is the tensor-memory A operand of P.V.
// Pipeline: the MMA thread issues S(j+1) = Q.K(j+1)^T before P(j).V(j), so the tensor pipe computes the next scores while
// the softmax warps work on the current ones; K and V tiles are loaded one tile ahead. The running maximum is only raised when a row's
// new maximum exceeds it by more than 8 (in log2 units); then the warp rescales its O rows in tensor memory after waiting for the
// previous P.V. P stays below 2^8, well inside fp16.
// Phases: a parity wait cannot tell phase k of an mbarrier from phase k - 2, and the softmax warps wait for 'O done' only now and then (a
// rescale, the epilogue), so it has one barrier per tile parity: tile k waits on barrier k & 1 for phase k >> 1, and the phase before it on
// that barrier (tile k - 2) is complete whenever a warp holds the scores of tile k, because the commit that announced them covers every MMA
// issued before. (With a single 'O done' barrier a warp that ran ahead of its peers through a two-tile part read O before the part's P.V
// had completed.) 'V landed' is announced for tail tiles only (the one remote arrival it costs the MMA thread is then off the other tiles'
// issue path); both sides count the tail tiles of the pair and use the count as the other barriers use the tile number.
// Every wait is bounded and shares the context's abort word; tensor memory is always released before the CTAs exit.
#include <algorithm>

#include "kata_internal.cuh"
#include "ptx.cuh"
#include "tc5.cuh"

namespace kata {
namespace {

using namespace ptx;

// Development aid, compiled only with -DKATA_PF_TRACE (never in the shipped library): CTA 0 records %globaltimer stamps of its phases.
#ifdef KATA_PF_TRACE
__device__ unsigned long long g_pf_trace[1280];   // [0,128): phases of the launch; 128 * kind + tile for the per-tile stamps (kinds 1-9)
__device__ unsigned long long g_pf_cta[148 * 4];   // per CTA: start, wait returned, last P.V of the last part complete, exit
#define pf_cta_stamp(k) do { if (blockIdx.x < 148) { unsigned long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); g_pf_cta[blockIdx.x * 4 + (k)] = t_; } } while (0)
__device__ int g_pf_trace_cta = 0, g_pf_trace_level = 1, g_pf_ablate = 0;   // ablate (timing experiments, wrong results): 1 no exp, 2 no score load   // level 0: only the P.V-issued stamp of every tile
#define PF_TRACE_INIT const int pf_ab = g_pf_ablate; const int pf_tr = ((int)blockIdx.x == g_pf_trace_cta) ? 1 + g_pf_trace_level : 0;   /* read once: a stamp must not cost a global load */
#define pf_stamp(slot) do { if (pf_tr && (slot) < 1280) { unsigned long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); g_pf_trace[(slot)] = t_; } } while (0)
#define pf_stamp_clock(slot) do { if (pf_tr) g_pf_trace[(slot)] = (unsigned long long)clock64(); } while (0)
#define pf_stamp_tile(kind, tile) do { if ((tile) < 128u && ((kind) == 3 || pf_tr > 1)) pf_stamp(128 * (kind) + (int)(tile)); } while (0)
#else
#define PF_TRACE_INIT
#define pf_stamp(slot) do { } while (0)
#define pf_stamp_tile(kind, tile) do { } while (0)
#define pf_stamp_clock(slot) do { } while (0)
#define pf_cta_stamp(k) do { } while (0)
#endif

constexpr int kTcThreads = 352, kBMq = 128, kBNk = 128;
constexpr int kBlk = 128 * 128;                  // one column block of 128 rows x 128 bytes (Q, V)
constexpr int kBlkKh = 64 * 128;                 // one column block of a K half-tile: 64 keys x 128 bytes
constexpr int kTileB = 4 * kBlk;                 // 64 KB: the 128 x 256 fp16 Q block
constexpr int kHalfB = 32 * 1024;                // a K or V half-tile
constexpr int kSmemTc = kTileB + 4 * kHalfB + 1024 + 256; // Q, 2 x K half, 2 x V half + alignment slack + barriers
constexpr uint32_t kIdescS = tc5::idesc_f16(256, 128, false), kIdescPV = tc5::idesc_f16(256, 256, true);

// barrier slots (8 bytes each) after the tiles
enum { B_QFULL = 0, B_KFULL0, B_KFULL1, B_KEMPTY0, B_KEMPTY1, B_VFULL0, B_VFULL1, B_VEMPTY0, B_VEMPTY1, B_VLANDED0, B_VLANDED1, B_SFULL0, B_SFULL1, B_PREADY0, B_PREADY1, B_ODONE0, B_ODONE1, B_QEMPTY, B_OFREE, B_COUNT };

__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, const int32_t* abort_flag) {   // same outcome for every lane of the warp
    const bool ok = mbar_wait_bounded(bar, parity, abort_flag);
    return __all_sync(0xffffffffu, ok);
}

// One work item = (query tile, head pair, sequence); PfPlan says which pair computes which.
struct PfStage { int64_t kv_row0[KATA_MAX_BATCH]; };   // SCALED: first row of sequence b in the fp16 staging arena (position 0)
struct PfItem { int q0, rows_valid, pos_base, kend, n_tiles, row0, row0v, h, kvh, bi; int64_t sc_row0; int idx, j0, j1, slot; bool whole; };   // row0 / row0v: row of position 0 in the arena the K / V tiles come from; [j0, j1): this part's key tiles
constexpr int kMaxPairs = 74;      // CTA pairs of a launch (one per two SMs of a B200)
constexpr double kCutCostUs = 5.0, kFoldCostUs = 2.7;   // host-side estimate of what cutting items costs a launch: the wait for a part that ends with the launch and the fold of the first part, then of each further part (measured: 2.7 us per part, L2 -> shared memory bound)
constexpr int kPartE = 2;          // host-side allowance, in key tiles, for what a part costs besides its tiles (Q load, epilogue or partial write)
// Items in list order: sequences shortest first (order[]), per sequence its KV heads, per KV head the query tiles last to first, per query tile the
// three head pairs of the KV head: the 3 * n_q items of one (sequence, KV head) are neighbours and read the same K and V tiles.
// A pair first computes `rounds` whole items, dealt in snake order (round k: item n_pairs * k + pair, pairs reversed in odd rounds), so that in
// every round a dozen pairs work on the same (sequence, KV head) at the same pace and its tiles come from L2 (with contiguous ranges instead, 74
// pairs on 64 different (sequence, KV head)s pull every item's K and V from HBM: 4 TB/s at batch 16). The items after the rounds are
// cut into one contiguous range per pair: pair p works on them from (item0[p], tile0[p]) up to, not including, (item0[p+1], tile0[p+1]),
// item numbers counted from the first item after the rounds; the ranges are sized so that a pair's rounds and range add up to the same load.
struct PfPlan { int32_t n_pairs, rounds; int32_t item0[kMaxPairs + 1]; int32_t tile0[kMaxPairs + 1]; int32_t hp_lo, hp_n; uint8_t order[KATA_MAX_BATCH]; };   // hp_lo, hp_n: the head pairs (3 per KV head) this launch computes
constexpr int kZoneMl = 128 * 1024;   // landing zone over the Q, K and V tiles: a part's 128 KB of rows as they lie in scratch, then the rows' (m, l)
// A part's rows in scratch: 16-byte chunk c (columns 4c .. 4c+3) of row r at chunk index c * 128 + r, so that the 32 rows of a warp (a thread holds one row
// of tensor memory) write and read 512 contiguous bytes per chunk.
constexpr size_t kPartOFloats = (size_t)kBMq * kD, kPartSlots = 2 * 2 * kMaxPairs;   // a slot = one CTA's 128 x 256 partial O, numbered (2 * pair + part) * 2 + CTA; only a pair's first part is ever written (the head of a cut item is merged where it is computed)

// MODE = the context's cache mode. An int8 plane's tiles are its codes expanded to fp16 (exact integers) in a staging arena whose rows are
// kv_row0[b] + position; the per-key scales are applied as k_flash_prefill_q8 does (shaders/flash.metal:10-68 with Q8): S = (Q.Kq) * ksc[key],
// P~ = half(p * vsc[key]), l from p. int8v (k_flash_prefill_k16v8, shaders/flash.metal:198-250): K tiles straight from the fp16 plane, V staged and scaled.
template <int MODE>
__global__ void __launch_bounds__(kTcThreads, 1) prefill_tc5_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                                                                   const Batch b, const int M, const float* __restrict__ gate, void* __restrict__ out, const int out_kind, int32_t* err,
                                                                   const PfStage stg, const __half* __restrict__ ksc, const __half* __restrict__ vsc,
                                                                   const __grid_constant__ PfPlan plan, float* part_o, float* part_ml, int32_t* part_flag) {
    constexpr bool KS = MODE == KATA_KV_INT8, KST = MODE == KATA_KV_INT8 || MODE == KATA_KV_INT8G, SCALED = MODE != KATA_KV_FP16;   // KS: scores take the key scale; KST: K tiles come from the staging arena (int8g: already scaled there); SCALED: P takes the value scale
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const uint32_t rank = tc5::cluster_rank();
    const int n_q = (M + kBMq - 1) / kBMq, grp_items = 3 * n_q, kvh_cnt = plan.hp_n / 3, pair = blockIdx.x / 2;
    const int rounds = plan.rounds, rem0 = rounds * plan.n_pairs;   // rem0: list index of the first item after the rounds
    const int item_lo = plan.item0[pair], tile_lo = plan.tile0[pair], item_hi = plan.item0[pair + 1], tile_hi = plan.tile0[pair + 1];
    const int my_parts = (item_lo == item_hi && tile_lo >= tile_hi) ? 0 : item_hi - item_lo + (tile_hi > 0 ? 1 : 0);   // parts of this pair's range
    const int my_items = rounds + my_parts;
    auto item_of = [&](int it) {   // it-th item or part of this CTA pair
        const int k = it - rounds;   // < 0: a whole item of round `it`
        const int idx = k < 0 ? plan.n_pairs * it + ((it & 1) ? plan.n_pairs - 1 - pair : pair) : rem0 + item_lo + k;
        const int grp = idx / grp_items, mem = idx % grp_items, qt = n_q - 1 - mem / 3;
        PfItem t; t.idx = idx; t.bi = plan.order[grp / kvh_cnt]; t.h = 2 * (plan.hp_lo + (grp % kvh_cnt) * 3 + mem % 3) + (int)rank; t.kvh = t.h / kG;   // heads 2i and 2i+1 form a pair (same KV head)
        t.q0 = qt * kBMq; t.rows_valid = min(kBMq, M - t.q0); t.pos_base = b.pos[t.bi]; t.kend = t.pos_base + t.q0 + t.rows_valid; t.n_tiles = (t.kend + kBNk - 1) / kBNk; t.row0 = KST ? (int)stg.kv_row0[t.bi] : (int)b.row_base[t.bi]; t.row0v = SCALED ? (int)stg.kv_row0[t.bi] : (int)b.row_base[t.bi]; t.sc_row0 = b.row_base[t.bi];
        t.j0 = k == 0 ? tile_lo : 0; t.j1 = (k >= 0 && item_lo + k == item_hi) ? tile_hi : t.n_tiles; t.whole = t.j0 == 0 && t.j1 == t.n_tiles; t.slot = (2 * pair + (k == 0 ? 0 : 1)) * 2 + (int)rank;
        return t;
    };
    // The parts of a cut item lie on consecutive pairs, its head (tiles from 0) last in its pair's range, every other part first in its pair's.
    auto pair_empty = [&](int p) { return plan.item0[p] == plan.item0[p + 1] && plan.tile0[p] >= plan.tile0[p + 1]; };
    auto next_part_pair = [&](int idx, int p) {   // the next pair after p whose range starts inside item idx (a list index), or -1
        for (int q = p + 1; q < plan.n_pairs && plan.item0[q] == idx - rem0; q++) if (!pair_empty(q)) return q;
        return -1;
    };
    auto other_slot = [&](int p2) { return (2 * p2) * 2 + (int)rank; };   // the part at the start of pair p2's range, this CTA's head
    bool merge_here = false; int merge_idx = -1;   // this pair's last part is the head of a cut item: its epilogue folds the other parts in
    if (my_items > 0) { const PfItem tl = item_of(my_items - 1); merge_here = tl.j0 == 0 && tl.j1 < tl.n_tiles; merge_idx = tl.idx; }
    const uint32_t sm0 = smem_u32(smem_raw), base = (sm0 + 1023u) & ~1023u;
    const uint32_t q_sm = base, k_sm = base + kTileB, v_sm = base + kTileB + 2 * kHalfB, bars = base + kTileB + 4 * kHalfB;   // K stage s at k_sm + s * kHalfB, V stage s at v_sm + s * kHalfB
    __shared__ uint32_t s_tmem; __shared__ int s_pick; __shared__ float s_xmax[2][2][128], s_lsum[2][128]; __shared__ __align__(16) float s_stage[8][16 * 36]; __shared__ __align__(16) __half s_sc[2][2][128];   // SCALED: [tile parity][K, V][key] scales of the tile   // [tile parity][key half][row]: row maxima exchanged by the two threads of a row; their partial l
    auto bar = [&](int i) { return bars + 8u * (uint32_t)i; };

    PF_TRACE_INIT
    if (tid == 0) { pf_stamp(0); pf_stamp_clock(126); pf_cta_stamp(0); }
    if (tid == 0) {
        for (int i = 0; i < B_COUNT; i++) mbar_init(bar(i), (i == B_PREADY0 || i == B_PREADY1 || i == B_OFREE) ? 16u : 1u);   // 'P ready', 'O free': one arrival per softmax warp of both CTAs
        fence_mbar_init();
    }
    __syncthreads();
    tc5::cluster_sync_all();   // both CTAs' barriers exist before anything arrives on them from the other side
    if (w == 0) tc5::tmem_alloc2(smem_u32(&s_tmem), 512);
    tc5::fence_before_sync();
    __syncthreads();
    tc5::fence_after_sync();
    const uint32_t tmem = s_tmem, t_o = tmem, t_s0 = tmem + 256;
    if (tid == 0) pf_stamp(1);
    pdl_wait(); pdl_launch_dependents();
    if (tid == 0) pf_cta_stamp(1);
    if (tid == 0) pf_stamp(2);   // launched with programmatic stream serialisation: the set-up above overlapped the previous kernel (the chunk's prep); its rows and Q are read from here on
    // Running counters shared by construction: gt = key tiles so far over all items of this pair (stage, score buffer and phase of the
    // per-tile barriers), it = items so far (phase of the per-item barriers).

    if (w == 8) {
        // ---- per item Q (when the previous item's last S MMA has read the old one), then this CTA's half (64 keys) of every K tile, one tile
        // ahead: stage gt & 1 is free when S(gt-2) has completed
        if (lane == 0) {
            uint32_t gt = 0; bool ok = true;
            for (int it = 0; ok && it < my_items; it++) {
                const PfItem t = item_of(it);
                if (it >= 1 && !mbar_wait_bounded(bar(B_QEMPTY), (uint32_t)(it - 1) & 1u, err)) { atomicExch(err, 10); break; }
                if (rank == 0) mbar_arrive_expect_tx(bar(B_QFULL), 2 * kTileB);
                for (int kb = 0; kb < 4; kb++) tc5::tma_load_2d_pair(q_sm + kb * kBlk, &tm_q, t.h * kD + kb * 64, t.bi * M + t.q0, bar(B_QFULL));
                for (int j = t.j0; j < t.j1; j++, gt++) {
                    const uint32_t st = gt & 1u;
                    if (gt >= 2 && !mbar_wait_bounded(bar(B_KEMPTY0 + st), ((gt >> 1) - 1u) & 1u, err)) { atomicExch(err, 11); ok = false; break; }
                    if (gt >= 2) pf_stamp_tile(8, gt - 2);   // S(gt - 2) has completed
                    if (rank == 0) mbar_arrive_expect_tx(bar(B_KFULL0 + st), 2 * kHalfB);
                    tc5::tma_load_4d_pair(k_sm + st * kHalfB, &tm_k, 0, t.row0 + j * kBNk + 64 * (int)rank, 0, t.kvh, bar(B_KFULL0 + st));
                }
            }
        }
    } else if (w == 9) {
        // ---- this CTA's half (128 dims) of every V tile (lane 0). When the item's last tile has been requested the whole warp asks L2 for the
        // item's gate tile (this CTA's head: rows_valid rows of 1 KB, 24 KB apart), which the epilogue reads one or two tiles of work later:
        // its first touch of those rows would otherwise be a DRAM round trip per epilogue step.
        uint32_t gt = 0; bool ok = true;
        for (int it = 0; ok && it < my_items; it++) {
            const PfItem t = item_of(it);
            for (int j = t.j0; j < t.j1; j++, gt++) {
                if (lane == 0) {
                    const uint32_t st = gt & 1u;
                    if (gt >= 2 && !mbar_wait_bounded(bar(B_VEMPTY0 + st), ((gt >> 1) - 1u) & 1u, err)) { atomicExch(err, 12); ok = false; }
                    if (gt >= 2) pf_stamp_tile(9, gt - 2);   // P.V(gt - 2) has completed
                    if (ok) {
                        if (rank == 0) mbar_arrive_expect_tx(bar(B_VFULL0 + st), 2 * kHalfB);
                        tc5::tma_load_4d_pair(v_sm + st * kHalfB, &tm_v, 0, t.row0v + j * kBNk, 2 * (int)rank, t.kvh, bar(B_VFULL0 + st));
                    }
                }
                ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
                if (!ok) break;
                if (j == t.j1 - 1 && t.j0 == 0) {
                    const float* gt0 = gate + ((int64_t)t.bi * M + t.q0) * kQD + t.h * kD;
                    for (int row = lane; row < t.rows_valid; row += 32) prefetch_l2_bulk(gt0 + (int64_t)row * kQD, kD * 4);
                }
            }
        }
    } else if (w == 10) {
        if (lane == 0 && rank == 0) {
            uint32_t gt = 0, nt = 0; bool ok = true;   // nt: tail tiles so far (barrier and phase of 'V landed')
            auto issue_s = [&](uint32_t g, const int i0, const int i1) {   // S of tile g = Q K^T for both CTAs: 4 column blocks x 4 k-steps of 16 dims = 16 MMAs, of which [i0, i1)
                const uint32_t d = t_s0 + (g & 1u) * 128u, kst = k_sm + (g & 1u) * kHalfB;
#pragma unroll
                for (int i = i0; i < i1; i++) {
                    const int kb = i >> 2, ks = i & 3;
                    tc5::mma_ss2(d, tc5::smem_desc_sw128(q_sm + kb * kBlk + ks * 32, 16, 1024), tc5::smem_desc_sw128(kst + kb * kBlkKh + ks * 32, 16, 1024), kIdescS, i != 0);
                }
                if (i1 == 16) { tc5::commit2(bar(B_SFULL0 + (g & 1u))); tc5::commit2(bar(B_KEMPTY0 + (g & 1u))); }
            };
            for (int it = 0; ok && it < my_items; it++) {
                const PfItem t = item_of(it);
                ok = mbar_wait_bounded(bar(B_QFULL), (uint32_t)it & 1u, err) && mbar_wait_bounded(bar(B_KFULL0 + (gt & 1u)), (gt >> 1) & 1u, err);
                if (!ok) { atomicExch(err, 13); break; }
                pf_stamp(3);
                tc5::fence_after_sync(); issue_s(gt, 0, 16);
                if (t.j1 - t.j0 == 1) tc5::commit2(bar(B_QEMPTY));
                for (int j = t.j0; j < t.j1; j++, gt++) {
                    // The tensor pipe holds only a few queued MMAs, so what this thread does between the last MMA of S(gt+1) and the first of
                    // P.V(gt) is time the pipe may run dry: the barriers P.V(gt) needs are tried while S(gt+1) is being issued ('V full' before
                    // its first MMA, 'P ready' before its last four; P(gt) is normally there by then) and waited for afterwards only if the
                    // try failed. Measured on 29-tile parts: 2 % off the launch.
                    bool v_ok = false, p_ok = false;
                    if (j + 1 < t.j1) {
                        if (!mbar_wait_bounded(bar(B_KFULL0 + ((gt + 1) & 1u)), ((gt + 1) >> 1) & 1u, err)) { atomicExch(err, 14); ok = false; break; }
                        pf_stamp_tile(6, gt + 1);
                        v_ok = mbar_try_wait(bar(B_VFULL0 + (gt & 1u)), (gt >> 1) & 1u) != 0;
                        tc5::fence_after_sync(); issue_s(gt + 1, 0, 12);
                        p_ok = mbar_try_wait(bar(B_PREADY0 + (gt & 1u)), (gt >> 1) & 1u) != 0;
                        issue_s(gt + 1, 12, 16);
                        pf_stamp_tile(1, gt + 1);
                        if (j + 2 == t.j1) tc5::commit2(bar(B_QEMPTY));   // the part's last S MMA: Q may be replaced
                    }
                    // V of the tile has landed in both CTAs, then wait for P
                    if (!v_ok && !mbar_wait_bounded(bar(B_VFULL0 + (gt & 1u)), (gt >> 1) & 1u, err)) { atomicExch(err, 15); ok = false; break; }
                    pf_stamp_tile(7, gt);
                    if (j * kBNk + kBNk > t.kend) { mbar_arrive(bar(B_VLANDED0 + (nt & 1u))); tc5::mbar_arrive_peer(bar(B_VLANDED0 + (nt & 1u))); nt++; }   // a tail tile: the softmax warps of both CTAs zero the rows of V past the range once it has landed
                    if (!p_ok && !mbar_wait_bounded(bar(B_PREADY0 + (gt & 1u)), (gt >> 1) & 1u, err)) { atomicExch(err, 15); ok = false; break; }
                    if (j == t.j0 && it >= 1 && !mbar_wait_bounded(bar(B_OFREE), (uint32_t)(it - 1) & 1u, err)) { atomicExch(err, 15); ok = false; break; }   // the previous item's O has been read out
                    pf_stamp_tile(2, gt);
                    tc5::fence_after_sync();
                    const uint32_t a = t_s0 + (gt & 1u) * 128u, vst = v_sm + (gt & 1u) * kHalfB;   // P: fp16 pairs in the first 64 columns of its S buffer
#pragma unroll
                    for (int ks = 0; ks < 8; ks++)   // 16 keys per step; V half is MN-major: 64-dim blocks 16 KB apart, 8-key groups 1 KB apart
                        tc5::mma_ts2(t_o, a + ks * 8, tc5::smem_desc_sw128(vst + ks * 2048, kBlk, 1024), kIdescPV, (j != t.j0) || ks != 0);
                    tc5::commit2(bar(B_ODONE0 + (gt & 1u)));
                    tc5::commit2(bar(B_VEMPTY0 + (gt & 1u)));
                    pf_stamp_tile(3, gt);
                }
            }
        }
    } else {
        // ---- softmax warps: two threads per query row, split by key half
        const int g = w >> 2, r = tid & 127;
        const uint32_t lane_sel = (uint32_t)((w & 3) * 32) << 16;
        const int pair_bar = 1 + (w & 3);   // named barrier of warps w and w + 4 (64 threads)
        uint32_t gt = 0, nt = 0; bool alive = true;   // nt: tail tiles so far, counted as the MMA thread counts them
        // Every thread runs every iteration and meets its partner at the pair barrier whatever happens: a wait that ran out only switches the work off.
        for (int it = 0; it < my_items; it++) {
        const PfItem t = item_of(it);
        const int q0 = t.q0, rows_valid = t.rows_valid, pos_base = t.pos_base, kend = t.kend, h = t.h, bi = t.bi, j0 = t.j0, j1 = t.j1;
        const int qpos = pos_base + q0 + r, lim = min(kend, qpos + 1);               // this row sees keys <= qpos (and < kend)
        float m = -INFINITY, l = 0.0f;
        for (int j = j0; j < j1; nt += (j * kBNk + kBNk > kend) ? 1u : 0u, j++, gt++) {
            const uint32_t t_s = t_s0 + (gt & 1u) * 128u + lane_sel;
            if (alive && !warp_wait(bar(B_SFULL0 + (gt & 1u)), (gt >> 1) & 1u, err)) { atomicExch(err, 16); alive = false; }
            if (tid == 0) pf_stamp_tile(4, gt);
            tc5::fence_after_sync();
            if (SCALED) {   // the tile's 128 K scales and 128 V scales: one value per softmax thread into shared memory, then everybody reads its 64 + 64
                const int key = min(j * kBNk + (tid & 127), max(kend - 1, 0));
                if (KS || tid >= 128) s_sc[gt & 1u][tid >> 7][tid & 127] = (tid < 128 ? ksc : vsc)[(t.sc_row0 + key) * 4 + t.kvh];
                asm volatile("bar.sync 9, 256;" ::: "memory");   // all eight softmax warps, every tile, whatever happened before
            }
            uint32_t v[2][32];
#ifdef KATA_PF_TRACE
            if (pf_ab & 2) {
#pragma unroll
                for (int c = 0; c < 2; c++)
#pragma unroll
                    for (int i = 0; i < 32; i++) v[c][i] = __float_as_uint((float)(i + (int)gt) * 0.01f);
            } else
#endif
            {
#pragma unroll
            for (int c = 0; c < 2; c++) tc5::ld32(t_s + g * 64 + c * 32, v[c]);
            tc5::wait_ld();
            }
            if (KS) {
                const uint4* kq = reinterpret_cast<const uint4*>(&s_sc[gt & 1u][0][g * 64]);
#pragma unroll
                for (int q8 = 0; q8 < 8; q8++) {
                    const uint4 u = kq[q8]; const __half2* hp = reinterpret_cast<const __half2*>(&u);
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const float2 f = __half22float2(hp[e]); const int i = q8 * 8 + 2 * e;
                        v[i >> 5][i & 31] = __float_as_uint(__uint_as_float(v[i >> 5][i & 31]) * f.x); v[(i + 1) >> 5][(i + 1) & 31] = __float_as_uint(__uint_as_float(v[(i + 1) >> 5][(i + 1) & 31]) * f.y);
                    }
                }
            }
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
            s_xmax[gt & 1u][g][r] = mx;
            asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");   // both halves of the row's scores are in registers and both maxima are visible
            do {
            if (!alive) break;
            const float mt = fmaxf(mx, s_xmax[gt & 1u][g ^ 1][r]) * kLog2e;
            const bool need = (j == j0) ? false : (mt > m + 8.0f);
            if (j == j0) m = mt;
            if (__any_sync(0xffffffffu, need)) {   // raise the reference maximum: rescale this thread's half of the O row after the previous P.V has landed
                if (!warp_wait(bar(B_ODONE0 + ((gt - 1u) & 1u)), ((gt - 1u) >> 1) & 1u, err)) { atomicExch(err, 17); alive = false; break; }
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
#ifdef KATA_PF_TRACE
                    const float p0 = (pf_ab & 1) ? fmaf(__uint_as_float(v[c][i]), kLog2e, -msub) : ex2(fmaf(__uint_as_float(v[c][i]), kLog2e, -msub)), p1 = (pf_ab & 1) ? fmaf(__uint_as_float(v[c][i + 1]), kLog2e, -msub) : ex2(fmaf(__uint_as_float(v[c][i + 1]), kLog2e, -msub));
#else
                    const float p0 = ex2(fmaf(__uint_as_float(v[c][i]), kLog2e, -msub)), p1 = ex2(fmaf(__uint_as_float(v[c][i + 1]), kLog2e, -msub));
#endif
                    sum += p0 + p1;
                    if (SCALED) { const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&s_sc[gt & 1u][1][g * 64 + c * 32 + i])); pk[c * 16 + (i >> 1)] = pack_h2(p0 * f.x, p1 * f.y); }
                    else pk[c * 16 + (i >> 1)] = pack_h2(p0, p1);
                }
            l += sum;
            tc5::st32(t_s + g * 32, pk);   // P: keys 0-63 in columns [0,32), keys 64-127 in [32,64) of the S buffer (the partner's scores there are in its registers since the pair barrier)
            tc5::wait_st();
            if (j * kBNk + kBNk > kend) {   // tail tile: rows of V past the range were loaded as they lie in memory; zero them (0 x garbage must stay 0)
                // (the MMA thread announces the V of a tail tile once it has landed in both CTAs)
                if (!warp_wait(bar(B_VLANDED0 + (nt & 1u)), (nt >> 1) & 1u, err)) { atomicExch(err, 18); alive = false; break; }
                if (g == 0 && j * kBNk + r >= kend) {
                    uint8_t* v_gen = smem_raw + (v_sm + (gt & 1u) * kHalfB - sm0);
#pragma unroll
                    for (int kb = 0; kb < 2; kb++)
#pragma unroll
                        for (int c = 0; c < 8; c++) *reinterpret_cast<uint4*>(v_gen + kb * kBlk + r * 128 + c * 16) = make_uint4(0, 0, 0, 0);
                }
                fence_proxy_async();
            }
            tc5::fence_before_sync();
            __syncwarp();
            if (lane == 0) tc5::mbar_arrive_leader(bar(B_PREADY0 + (gt & 1u)));
            if (tid == 0) pf_stamp_tile(5, gt);
            } while (0);
        }
        // ---- epilogue: the two threads of a row add their partial l and handle 128 columns each
        s_lsum[g][r] = l;
        asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
        l += s_lsum[g ^ 1][r];
        // Tensor memory hands a thread one row (32 columns at a time); global memory wants consecutive lanes on consecutive bytes of one row.
        // Per 32-column block each warp stages its 32 rows in two passes of 16 rows x 32 columns through shared memory (row stride 36 floats:
        // the 128-bit stores of 8 rows and the 128-bit loads of one row both spread over all 32 banks) and writes them back with 8 lanes
        // per row: every 128-bit gate load and output store of a quarter warp is one whole 128-byte line. The gate values of a block are
        // requested (from L2, where the V producer warp has asked for them) one block ahead.
        float* tile = s_stage[w];                     // [16 rows][36]
        const int rq = lane >> 3, cq = (lane & 7) * 4, rbase = 32 * (w & 3);
        const int64_t obase = ((int64_t)bi * M + q0 + rbase) * kQD + h * kD + g * 128 + cq;
        if (j0 == 0) {
        // whole item, or the head of a cut item: O / l * sigmoid(gate) straight to the output rows
        float4 gv[8];   // gate logits of the block in flight: [pass][k] -> warp row 16 * pass + 4 * k + rq, columns cq .. cq + 3 of the block
        auto load_gate = [&](int c, float4 (&dst)[8]) {
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const int row = 16 * (i >> 2) + 4 * (i & 3) + rq; dst[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if (rbase + row < rows_valid) asm volatile("ld.global.nc.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(dst[i].x), "=f"(dst[i].y), "=f"(dst[i].z), "=f"(dst[i].w) : "l"(gate + obase + (int64_t)row * kQD + c * 32));
            }
        };
        load_gate(0, gv);   // in flight while the item's last P.V completes
        if (tid == 0) pf_stamp(56);
        if (alive && !warp_wait(bar(B_ODONE0 + ((gt - 1u) & 1u)), ((gt - 1u) >> 1) & 1u, err)) { atomicExch(err, 19); alive = false; }
        {
            if (tid == 0) { pf_stamp(57); if (it == my_items - 1) pf_cta_stamp(2); }
            tc5::fence_after_sync();
            if (j1 < t.n_tiles) {
                // Head of a cut item (always the pair's last part): every MMA of the pair is complete, so the Q, K and V tiles are free and serve as
                // the landing zone of the other parts' unnormalised rows, one part at a time: when a part's flag is up (raised by the CTA that
                // wrote it; the wait is bounded like every other) the eight warps copy its 128 KB and its (m, l) with cp.async, 32 chunks of 16
                // bytes per thread in flight at once, and each thread folds its row of the part into its row of O in tensor memory with the
                // split-KV rule (k_attn_dec_combine, shaders/flash.metal:143-152, one "split" at a time: new maximum, both sides rescaled).
                // m is finite here: key 0 is in the head.
                const uint8_t* zone = smem_raw + (base - sm0);
                // The parts are folded in the order of their pairs, whatever the order their flags come up in: the sums then round the same way in every launch.
                for (int nx = next_part_pair(t.idx, pair); nx >= 0; nx = next_part_pair(t.idx, nx)) {
                    if (tid == 0) {   // one thread waits for the part's flag and tells the others
                        int got = 0;
                        for (uint32_t i = 0; i < (1u << 21) && !got; i++) {
                            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(got) : "l"(part_flag + other_slot(nx)) : "memory");
                            if (!got && (i & 255u) == 255u && *reinterpret_cast<const volatile int32_t*>(err) != 0) break;
                        }
                        s_pick = got ? nx : -1;
                    }
                    asm volatile("bar.sync 10, 256;" ::: "memory");
                    const int p2 = s_pick;
                    if (p2 < 0) { if (alive) { atomicExch(err, 20); alive = false; } break; }   // the same for all eight warps
                    const int sl = other_slot(p2);
                    if (alive) {   // four groups of copies, one per 32-column block of the two halves, so that a block is folded while the next ones land
                        const float* src = part_o + (size_t)sl * kPartOFloats;
                        if (tid < 64) cp_async16(base + (uint32_t)(kZoneMl + tid * 16), part_ml + (size_t)sl * (2 * kBMq) + tid * 4, 16);
#pragma unroll
                        for (int c = 0; c < 4; c++) {
#pragma unroll
                            for (int u = 0; u < 8; u++) { const int n = 16 * (u >> 2) + 4 * c + (u & 3); cp_async16(base + (uint32_t)(tid + 256 * n) * 16u, src + (size_t)(tid + 256 * n) * 4, 16); }
                            cp_async_commit();
                        }
                    }
                    float2 mlq = make_float2(-INFINITY, 0.0f); float mn = m, a = 1.0f, bq = 0.0f;
                    const float4* zr = reinterpret_cast<const float4*>(zone) + r;
                    auto fold_block = [&](int c) {   // every lane, whatever its row: the tensor-memory loads and stores are warp-wide instructions (rows past the chunk fold garbage that is never stored)
                        uint32_t o[32]; tc5::ld32(t_o + lane_sel + g * 128 + c * 32, o); tc5::wait_ld();
#pragma unroll
                        for (int i = 0; i < 8; i++) {
                            const float4 z = zr[(g * 32 + c * 8 + i) * 128];
                            o[4 * i] = __float_as_uint(fmaf(__uint_as_float(o[4 * i]), a, bq * z.x)); o[4 * i + 1] = __float_as_uint(fmaf(__uint_as_float(o[4 * i + 1]), a, bq * z.y));
                            o[4 * i + 2] = __float_as_uint(fmaf(__uint_as_float(o[4 * i + 2]), a, bq * z.z)); o[4 * i + 3] = __float_as_uint(fmaf(__uint_as_float(o[4 * i + 3]), a, bq * z.w));
                        }
                        tc5::st32(t_o + lane_sel + g * 128 + c * 32, o);
                    };
                    cp_async_wait<3>(); asm volatile("bar.sync 10, 256;" ::: "memory");   // the (m, l) pairs and block 0 have landed (all eight warps, whatever happened)
                    if (alive) {
                        mlq = *reinterpret_cast<const float2*>(zone + kZoneMl + r * 8);
                        mn = fmaxf(m, mlq.x); a = ex2(m - mn); bq = (mlq.x == -INFINITY) ? 0.0f : ex2(mlq.x - mn);
                        fold_block(0);
                    }
                    cp_async_wait<2>(); asm volatile("bar.sync 10, 256;" ::: "memory");
                    if (alive) fold_block(1);
                    cp_async_wait<1>(); asm volatile("bar.sync 10, 256;" ::: "memory");
                    if (alive) fold_block(2);
                    cp_async_wait<0>(); asm volatile("bar.sync 10, 256;" ::: "memory");
                    if (alive) { fold_block(3); tc5::wait_st(); l = fmaf(l, a, bq * mlq.y); m = mn; }
                    asm volatile("bar.sync 10, 256;" ::: "memory");   // everybody has read the part: the zone may take the next one
                }
            }
        }
        if (alive) {
            const float inv = 1.0f / l;
#pragma unroll 1
            for (int c = 0; c < 4; c++) {
                uint32_t o[32]; tc5::ld32(t_o + lane_sel + g * 128 + c * 32, o); tc5::wait_ld();
                if (tid == 0) pf_stamp(58 + 2 * c);
                float4 gc[8];
#pragma unroll
                for (int i = 0; i < 8; i++) gc[i] = gv[i];
                if (tid == 0) pf_stamp(59 + 2 * c);
                if (c + 1 < 4) load_gate(c + 1, gv);
#pragma unroll
                for (int pass = 0; pass < 2; pass++) {
                    if ((lane >> 4) == pass) {
#pragma unroll
                        for (int i = 0; i < 8; i++)
                            *reinterpret_cast<float4*>(tile + (lane & 15) * 36 + 4 * i) = make_float4(__uint_as_float(o[4 * i]) * inv, __uint_as_float(o[4 * i + 1]) * inv, __uint_as_float(o[4 * i + 2]) * inv, __uint_as_float(o[4 * i + 3]) * inv);
                    }
                    __syncwarp();
                    float4 tv[4];
#pragma unroll
                    for (int k = 0; k < 4; k++) tv[k] = *reinterpret_cast<const float4*>(tile + (4 * k + rq) * 36 + cq);
                    __syncwarp();
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        const float4 gg = gc[pass * 4 + k];
                        tv[k].x *= sigmoid_approx(gg.x); tv[k].y *= sigmoid_approx(gg.y); tv[k].z *= sigmoid_approx(gg.z); tv[k].w *= sigmoid_approx(gg.w);
                    }
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        const int row = 16 * pass + 4 * k + rq;
                        if (rbase + row < rows_valid) store_act4(out, obase + (int64_t)row * kQD + c * 32, tv[k], out_kind);
                    }
                }
            }
            if (tid == 0) pf_stamp(66);
            // this warp is done with the item's O: the first P.V of the next item may overwrite it
            tc5::fence_before_sync();
            __syncwarp();
            if (lane == 0) tc5::mbar_arrive_leader(bar(B_OFREE));
        }
        } else {
        // another part of a cut item (always the pair's first part): the unnormalised O rows (fp32) and their (m, l) go to this part's scratch slot,
        // from where the pair that holds the item's head takes them
        float4* po = reinterpret_cast<float4*>(part_o + (size_t)t.slot * kPartOFloats) + r;   // chunk c of this thread's row at po[c * 128]: a warp's 32 rows are 512 contiguous bytes
        if (alive && warp_wait(bar(B_ODONE0 + ((gt - 1u) & 1u)), ((gt - 1u) >> 1) & 1u, err)) {
            tc5::fence_after_sync();
            if (g == 0) *reinterpret_cast<float2*>(part_ml + (size_t)t.slot * (2 * kBMq) + 2 * r) = make_float2(m, l);   // m in log2 units; -inf when the row saw no key of this part
#pragma unroll 1
            for (int c = 0; c < 4; c++) {
                uint32_t o[32]; tc5::ld32(t_o + lane_sel + g * 128 + c * 32, o); tc5::wait_ld();
#pragma unroll
                for (int i = 0; i < 8; i++) __stcg(po + (g * 32 + c * 8 + i) * 128, make_float4(__uint_as_float(o[4 * i]), __uint_as_float(o[4 * i + 1]), __uint_as_float(o[4 * i + 2]), __uint_as_float(o[4 * i + 3])));
            }
            tc5::fence_before_sync();
            __syncwarp();
            if (lane == 0) tc5::mbar_arrive_leader(bar(B_OFREE));
            __threadfence();   // the rows and their (m, l) before the flag
        } else if (alive) { atomicExch(err, 19); alive = false; }
        // the part is in scratch: raise its flag for the pair that holds the item's head (all eight warps meet here whatever happened; the flag only goes up when all is well)
        asm volatile("bar.sync 10, 256;" ::: "memory");
        if (tid == 0 && alive) asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(part_flag + t.slot), "r"(1) : "memory");
        if (tid == 0) pf_stamp(80);
        }
        }
    }
    if (tid == 0) { pf_stamp(67); pf_stamp_clock(127); }
    tc5::fence_before_sync();
    __syncthreads();
    if (tid == 0 && merge_here)   // the flags this CTA consumed go down again for the next launch (its writers start after this kernel has completed)
        for (int p2 = next_part_pair(merge_idx, pair); p2 >= 0; p2 = next_part_pair(merge_idx, p2)) part_flag[other_slot(p2)] = 0;
    tc5::cluster_sync_all();   // neither CTA leaves (or frees tensor memory) while the other may still read its shared memory or arrive on its barriers
    if (w == 0) tc5::tmem_dealloc2(tmem, 512);
    if (tid == 0) { pf_stamp(68); pf_cta_stamp(3); }
}

// int8 planes: expands the codes of rows [0, kend_b) of every sequence of the batch (one layer) to fp16 in the staging arena. The values are
// the integers themselves (exact in fp16); the scales stay with the softmax. 64 threads per 1024-code row, 16 codes per thread.
// grid.z = planes to expand: 2 (K then V), or 1 with first_plane = 1 (V only: the keys are fp16 already).
// ksc_g (int8g contexts only): the key plane has one scale per 64 dims, which a per-key factor in the softmax cannot carry: the K codes are expanded to
// code * scale (rounded to fp16) here, and the kernel then treats the K tiles as plain fp16 keys.
__global__ void __launch_bounds__(256) expand_codes_kernel(const Batch b, const int M, const PfStage stg, const uint8_t* __restrict__ kq, const uint8_t* __restrict__ vq, __half* __restrict__ k16, __half* __restrict__ v16, const int first_plane,
                                                           const __half* __restrict__ ksc_g) {
    const int bi = blockIdx.y, rows = b.pos[bi] + M; const bool isV = (blockIdx.z + first_plane) != 0;
    const uint8_t* src = isV ? vq : kq; __half* dst = isV ? v16 : k16;
    for (int r = blockIdx.x * 4 + (threadIdx.x >> 6); r < rows; r += gridDim.x * 4) {
        const int c16 = threadIdx.x & 63;
        const uint4 u = __ldg(reinterpret_cast<const uint4*>(src + (b.row_base[bi] + r) * kKVD) + c16);
        const uint32_t wd[4] = {u.x ^ 0x80808080u, u.y ^ 0x80808080u, u.z ^ 0x80808080u, u.w ^ 0x80808080u};
        uint32_t o[8];
#pragma unroll
        for (int e = 0; e < 4; e++) {   // byte x -> fp16 0x64xx = 1024 + (code + 128); minus 1152 gives the code exactly
            const uint32_t lo = prmt(wd[e], 0x64646464u, 0x4140u), hi = prmt(wd[e], 0x64646464u, 0x4342u);
            const __half2 bias = __floats2half2_rn(1152.0f, 1152.0f);
            __half2 a = __hsub2(*reinterpret_cast<const __half2*>(&lo), bias), c2 = __hsub2(*reinterpret_cast<const __half2*>(&hi), bias);
            if (ksc_g && !isV) {   // this thread's 16 codes lie in one 64-dim group: head c16 / 16, group (c16 % 16) / 4
                const __half2 sc = __half2half2(ksc_g[(b.row_base[bi] + r) * 16 + (c16 >> 4) * 4 + ((c16 & 15) >> 2)]);
                a = __hmul2(a, sc); c2 = __hmul2(c2, sc);
            }
            o[2 * e] = *reinterpret_cast<const uint32_t*>(&a); o[2 * e + 1] = *reinterpret_cast<const uint32_t*>(&c2);
        }
        uint4* d4 = reinterpret_cast<uint4*>(dst + (stg.kv_row0[bi] + r) * kKVD) + 2 * c16;
        d4[0] = make_uint4(o[0], o[1], o[2], o[3]); d4[1] = make_uint4(o[4], o[5], o[6], o[7]);
    }
}

}  // namespace

#ifdef KATA_PF_TRACE
extern "C" int kata_debug_pf_trace(unsigned long long* h1024) { return (int)cudaMemcpyFromSymbol(h1024, g_pf_trace, sizeof(g_pf_trace)); }
extern "C" int kata_debug_pf_ctas(unsigned long long* h) { return (int)cudaMemcpyFromSymbol(h, g_pf_cta, sizeof(g_pf_cta)); }
extern "C" int kata_debug_pf_trace_cta(int cta, int level, int ablate) { cudaMemcpyToSymbol(g_pf_trace_level, &level, sizeof(int)); cudaMemcpyToSymbol(g_pf_ablate, &ablate, sizeof(int)); return (int)cudaMemcpyToSymbol(g_pf_trace_cta, &cta, sizeof(int)); }
#endif

// scratch of the cut items: partial O rows and their (m, l)
size_t prefill_part_o_bytes() { return kPartSlots * kPartOFloats * sizeof(float); }
size_t prefill_part_ml_bytes() { return kPartSlots * 2 * kBMq * sizeof(float); }
size_t prefill_part_flag_bytes() { return kPartSlots * sizeof(int32_t); }

cudaError_t launch_prefill_mma(Ctx& c, const Batch& b, int M, const __half* q16, const float* gate, void* out, int out_dtype, cudaStream_t s);
cudaError_t configure_prefill_mma(int kv_mode);

// Shared-memory opt-in of the prefill kernels on the current device (function attributes are per device: done once per context).
cudaError_t configure_prefill(int kv_mode) {
    cudaError_t e = configure_prefill_mma(kv_mode);
    if (e == cudaSuccess) e = kv_mode == KATA_KV_INT8G ? cudaFuncSetAttribute(prefill_tc5_kernel<KATA_KV_INT8G>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTc)
                            : kv_mode == KATA_KV_INT8  ? cudaFuncSetAttribute(prefill_tc5_kernel<KATA_KV_INT8>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTc)
                            : kv_mode == KATA_KV_INT8V ? cudaFuncSetAttribute(prefill_tc5_kernel<KATA_KV_INT8V>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTc)
                                                       : cudaFuncSetAttribute(prefill_tc5_kernel<KATA_KV_FP16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTc);
    return e;
}

// The work split of one launch (see PfPlan): depends only on the chunk length, the sequences' positions, the KV heads of the context and the number of
// CTA pairs. tiles_scratch: room for the key-tile count of every item (n_q * 3 * kvh_n * n entries). Pure host code.
static void make_prefill_plan(const int M, const int n, const int32_t* pos, const int kvh_lo, const int kvh_n, const int pairs_avail, int32_t* tiles_scratch, PfPlan& plan_out) {
    const int hp_n = 3 * kvh_n, hp_lo = 3 * kvh_lo;   // head pairs of the KV heads this context computes
    const int n_q = (M + kBMq - 1) / kBMq, grp_items = 3 * n_q, n_items = grp_items * kvh_n * n, max_pairs = std::max(1, std::min(kMaxPairs, pairs_avail));
    uint8_t order[KATA_MAX_BATCH];   // sequences of the batch, shortest first (ties in batch order): the rounds then deal items of like length, and the long
    for (int i = 0; i < n; i++) order[i] = (uint8_t)i;   // items, which only cutting can spread, come last, where the ranges are cut
    std::stable_sort(order, order + n, [&](uint8_t x, uint8_t y) { return pos[x] < pos[y]; });
    int32_t* nt_tab = tiles_scratch;   // key tiles per item in list order (room for the largest launch: 8 query tiles x 12 head pairs x 64 sequences)
    for (int idx = 0; idx < n_items; idx++) { const int grp = idx / grp_items, qt = n_q - 1 - (idx % grp_items) / 3, bi = order[grp / kvh_n], q0 = qt * kBMq; nt_tab[idx] = (pos[bi] + q0 + std::min(kBMq, M - q0) + kBNk - 1) / kBNk; }
    auto tiles_of = [&](int idx) { return (int)nt_tab[idx]; };
    constexpr int kMinPart = 2;   // a part is at least two key tiles
    auto round_item = [&](const PfPlan& pl, int p, int k) { return pl.n_pairs * k + ((k & 1) ? pl.n_pairs - 1 - p : p); };
    auto max_load = [&](const PfPlan& pl) {   // the heaviest pair: its rounds' items and its range, each item or part with the allowance
        const int rem0 = pl.rounds * pl.n_pairs; int worst = 0;
        for (int p = 0; p < pl.n_pairs; p++) {
            int w = 0;
            for (int k = 0; k < pl.rounds; k++) w += tiles_of(round_item(pl, p, k)) + kPartE;
            for (int i = pl.item0[p]; i <= pl.item0[p + 1] && rem0 + i < n_items; i++) {
                const int j0 = i == pl.item0[p] ? pl.tile0[p] : 0, j1 = i == pl.item0[p + 1] ? pl.tile0[p + 1] : tiles_of(rem0 + i);
                if (j1 > j0) w += j1 - j0 + kPartE;
            }
            worst = std::max(worst, w);
        }
        return worst;
    };
    // The items from list index rem0 on, cut into one contiguous range per pair; cap[p] = the weight (tiles + allowance per item) pair p should get.
    // Cuts keep parts of at least two tiles (a cut too close to an item's end moves to the item boundary) and never run backwards.
    auto cut_ranges = [&](PfPlan& pl, const double* cap) {
        const int rem0 = pl.rounds * pl.n_pairs, n_rem = n_items - rem0;
        int idx = 0; int64_t acc = 0; double target = 0.0;   // acc: weight of the items before idx
        pl.item0[0] = 0; pl.tile0[0] = 0;
        for (int p = 1; p < pl.n_pairs; p++) {
            target += cap[p - 1];
            while (idx < n_rem && (double)(acc + tiles_of(rem0 + idx) + kPartE) <= target) { acc += tiles_of(rem0 + idx) + kPartE; idx++; }
            int ci = idx, ct = 0;
            if (idx < n_rem) {
                const int nt = tiles_of(rem0 + idx), jt = (int)(target - (double)acc + 0.5);
                if (jt >= kMinPart && nt - jt >= kMinPart) ct = jt; else if (jt >= kMinPart) ci = idx + 1;
            }
            if (ci < pl.item0[p - 1] || (ci == pl.item0[p - 1] && ct < pl.tile0[p - 1])) { ci = pl.item0[p - 1]; ct = pl.tile0[p - 1]; }
            pl.item0[p] = ci; pl.tile0[p] = ct;
        }
        pl.item0[pl.n_pairs] = n_rem; pl.tile0[pl.n_pairs] = 0;
    };
    int64_t W = 0; for (int i = 0; i < n_items; i++) W += tiles_of(i) + kPartE;
    // Plan A: no rounds, equal ranges of the whole list. With fewer items than pairs the items are cut, but not into ranges shorter than two tiles plus the allowance.
    PfPlan plan{};
    {
        plan.n_pairs = n_items >= max_pairs ? max_pairs : std::max(std::min(n_items, max_pairs), (int)std::min<int64_t>(max_pairs, W / (kPartE + 2)));
        double cap[kMaxPairs]; for (int p = 0; p < plan.n_pairs; p++) cap[p] = (double)W / plan.n_pairs;
        cut_ranges(plan, cap);
    }
    // Plan R (at least as many items as pairs): whole items in rounds, then the last half to one and a half rounds' worth of items cut into ranges
    // that level the pairs (capacities by water-filling over the rounds' loads). Its pairs share K and V tiles through L2, so it is taken
    // with as many rounds as leave it no more than 3 % less balanced than plan A (in a ragged batch the long items, which only cutting can spread,
    // have to fall into the ranges).
    if (n_items >= max_pairs) {
        int rounds = n_items / max_pairs;
        if (n_items - rounds * max_pairs < max_pairs / 2 && rounds >= 1) rounds--;
        const double flat_load = (double)max_load(plan);
        for (int attempt = 0; attempt < 4 && rounds >= 1; attempt++, rounds--) {   // fewer rounds leave more (and longer) items to the ranges
            PfPlan alt{}; alt.n_pairs = max_pairs; alt.rounds = rounds;
            double load[kMaxPairs], cap[kMaxPairs]; double w_rem = 0.0, hi = 0.0, lo = 0.0;
            for (int p = 0; p < max_pairs; p++) { load[p] = 0.0; for (int k = 0; k < alt.rounds; k++) load[p] += tiles_of(round_item(alt, p, k)) + kPartE; hi = std::max(hi, load[p]); }
            for (int i = alt.rounds * max_pairs; i < n_items; i++) w_rem += tiles_of(i) + kPartE;
            hi += w_rem;
            for (int it = 0; it < 50; it++) { const double mid = 0.5 * (lo + hi); double sum = 0.0; for (int p = 0; p < max_pairs; p++) sum += std::max(0.0, mid - load[p]); if (sum < w_rem) lo = mid; else hi = mid; }
            for (int p = 0; p < max_pairs; p++) cap[p] = std::max(0.0, hi - load[p]);
            cut_ranges(alt, cap);
            if ((double)max_load(alt) <= 1.03 * flat_load) { plan = alt; break; }
        }
    }
    // Plan B (only with fewer items than pairs): one part per pair; the spare pairs go, one at a time, to the item whose parts are longest.
    // Better than A when the items are short (a 512-token prompt: items of 1 to 4 tiles).
    if (n_items < max_pairs) {
        int parts[kMaxPairs]; int total = n_items;
        for (int i = 0; i < n_items; i++) parts[i] = 1;
        for (; total < max_pairs; total++) {
            int best = -1, best_len = 0;
            for (int i = 0; i < n_items; i++) { const int len = (tiles_of(i) + parts[i] - 1) / parts[i]; if (tiles_of(i) / (parts[i] + 1) >= kMinPart && len > best_len) { best = i; best_len = len; } }
            if (best < 0) break;
            parts[best]++;
        }
        PfPlan alt{}; alt.n_pairs = total; int p = 0;
        for (int i = 0; i < n_items; i++) for (int m = 0; m < parts[i]; m++, p++) { alt.item0[p] = i; alt.tile0[p] = (int)((int64_t)tiles_of(i) * m / parts[i]); }
        alt.item0[total] = n_items; alt.tile0[total] = 0;
        if (max_load(alt) < max_load(plan)) plan = alt;
    }
    // Plan U: no item is cut (every cut moved to the next item boundary). A cut plan has the shorter critical path but its heads wait for
    // the other parts to be written and fold them in (a few microseconds at the end of the launch). Estimate both in microseconds (a key tile of a
    // CTA pair takes about 2.3 us at the rate the kernel sustains, power-capped) and keep the cheaper.
    {
        const int n_rem = n_items - plan.rounds * plan.n_pairs;
        PfPlan whole = plan; int max_parts = 1, run = 1;   // run: parts so far of the item the current cut lies in
        for (int p = 1; p < whole.n_pairs; p++) {
            if (plan.tile0[p] == 0) { run = 1; continue; }
            const bool same_item = plan.item0[p - 1] == plan.item0[p] && plan.tile0[p - 1] > 0, repeat = same_item && plan.tile0[p - 1] == plan.tile0[p];   // repeat: pair p - 1 is empty, the same cut again
            run = same_item ? run + (repeat ? 0 : 1) : 2; max_parts = std::max(max_parts, run);
            whole.tile0[p] = 0; whole.item0[p] = std::min(whole.item0[p] + 1, n_rem);
        }
        const double t_tile = 2.3, t_cut = max_load(plan) * t_tile + (max_parts > 1 ? kCutCostUs + kFoldCostUs * (max_parts - 2) : 0.0), t_whole = max_load(whole) * t_tile;
        if (t_whole <= t_cut) plan = whole;
    }
    for (int i = 0; i < n; i++) plan.order[i] = order[i];
    plan.hp_lo = hp_lo; plan.hp_n = hp_n;
    plan_out = plan;
}

// The plan as plain arrays, for tests of the host logic that have no GPU (and for a caller that wants to see how a launch would be shared out):
// returns the number of pairs; item0/tile0 take n_pairs + 1 entries each, order takes n. tiles_scratch as in make_prefill_plan.
extern "C" int kata_attn_prefill_plan(int32_t M, int32_t n, const int32_t* pos, int32_t kvh_lo, int32_t kvh_n, int32_t pairs_avail, int32_t* tiles_scratch,
                                      int32_t* rounds, int32_t* item0, int32_t* tile0, uint8_t* order) {
    if (M < 1 || M > KATA_MAX_CHUNK || n < 1 || n > KATA_MAX_BATCH || !pos || kvh_lo < 0 || kvh_n < 1 || kvh_lo + kvh_n > KATA_KV_HEADS || !tiles_scratch || !rounds || !item0 || !tile0 || !order) return -1;
    PfPlan plan{}; make_prefill_plan(M, n, pos, kvh_lo, kvh_n, pairs_avail, tiles_scratch, plan);
    *rounds = plan.rounds;
    for (int p = 0; p <= plan.n_pairs; p++) { item0[p] = plan.item0[p]; tile0[p] = plan.tile0[p]; }
    for (int i = 0; i < n; i++) order[i] = plan.order[i];
    return plan.n_pairs;
}

// tcgen05 kernel (unless the context was created with the legacy-path flag). An int8 cache goes through it as well: the layer's codes are first
// expanded to fp16 in the context's staging arena (one pass over the prefix, a few per cent of the attention time), the scales are applied in
// the softmax. The mma.sync kernel remains the cross-check and serves windowed caches (a position offset), which the staging arena does not cover.
cudaError_t launch_prefill(Ctx& c, const Batch& b, int M, const __half* q16, const float* gate, void* out, int out_dtype, cudaStream_t s) {
    const int mode = c.cfg.kv_mode; const bool i8 = c.v8();
    bool windowed = false; for (int i = 0; i < b.n; i++) windowed |= c.pos_off[b.seq[i]] != 0;
    if (c.kg() && windowed) return cudaErrorNotSupported;   // the mma.sync kernel, which serves windowed int8 caches, has no grouped key scales
    if ((c.cfg.flags & 1) || (i8 && (!c.v16_stage || windowed))) return launch_prefill_mma(c, b, M, q16, gate, out, out_dtype, s);
    CUtensorMap tm_q;
    if (!make_matrix_tmap(&tm_q, q16, (int64_t)b.n * M, kQD, 64, 128)) return cudaErrorInvalidValue;
    PfStage stg{};
    if (i8) {
        int max_rows = 0; for (int i = 0; i < b.n; i++) { stg.kv_row0[i] = c.stage_row0[b.seq[i]]; max_rows = std::max(max_rows, b.pos[i] + M); }
        expand_codes_kernel<<<dim3(std::min((max_rows + 3) / 4, 1024), b.n, c.k8() ? 2 : 1), 256, 0, s>>>(b, M, stg, (const uint8_t*)c.k_arena, (const uint8_t*)c.v_arena, c.k16_stage, c.v16_stage, c.k8() ? 0 : 1, c.kg() ? (const __half*)c.ksc : nullptr);
        c.launches++;
    }
    // persistent CTA pairs, at most one per two SMs; see PfPlan for the way the items are shared out.
    // The plan depends only on (M, positions): the 16 layers of a chunk reuse the one computed for the first (kept in the context, no allocation).
    struct Cached { PfPlan plan; };
    static_assert(sizeof(Cached) <= sizeof(c.pf_plan_cache), "plan cache too small");
    Cached& cached = *reinterpret_cast<Cached*>(c.pf_plan_cache);
    bool hit = c.pf_plan_M == M && c.pf_plan_n == b.n;
    for (int i = 0; hit && i < b.n; i++) hit = c.pf_plan_pos[i] == b.pos[i];
    if (!hit) {
    make_prefill_plan(M, b.n, b.pos, c.kvh_lo, c.kvh_n, c.sm_count / 2, c.pf_plan_tiles, cached.plan);
    c.pf_plan_M = M; c.pf_plan_n = b.n; for (int i = 0; i < b.n; i++) c.pf_plan_pos[i] = b.pos[i];
    }
    const PfPlan& plan = cached.plan;
    const int n_pairs = plan.n_pairs;
    cudaLaunchConfig_t cfg{}; cfg.gridDim = dim3(2 * n_pairs, 1, 1); cfg.blockDim = dim3(kTcThreads); cfg.dynamicSmemBytes = kSmemTc; cfg.stream = s;
    cudaLaunchAttribute at[2]; at[0].id = cudaLaunchAttributeClusterDimension; at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;   // a CTA pair is two neighbours along x
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization; at[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = 2;
#define KATA_PF(MD, TK, TV) cudaLaunchKernelEx(&cfg, prefill_tc5_kernel<MD>, tm_q, TK, TV, b, M, gate, out, (int)out_dtype, c.d_err, stg, (const __half*)c.ksc, (const __half*)c.vsc, plan, c.pf_part_o, c.pf_part_ml, c.pf_part_flag)
    const cudaError_t le = mode == KATA_KV_INT8G ? KATA_PF(KATA_KV_INT8G, c.tm_k64h_stage, c.tm_v128h_stage) : mode == KATA_KV_INT8 ? KATA_PF(KATA_KV_INT8, c.tm_k64h_stage, c.tm_v128h_stage) : mode == KATA_KV_INT8V ? KATA_PF(KATA_KV_INT8V, c.tm_k64h, c.tm_v128h_stage) : KATA_PF(KATA_KV_FP16, c.tm_k64h, c.tm_v128h);
#undef KATA_PF
    if (le != cudaSuccess) return le;
    c.wrote_no_rows();
    c.launches++;
    return cudaGetLastError();
}

}  // namespace kata
