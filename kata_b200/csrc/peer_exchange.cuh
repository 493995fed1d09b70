// Device side of the split-KV exchange between the GPUs of one box (see peer_merge.cu for the protocol): one CTA-wide routine that takes
// this rank's partial of one (token, head) row, stores it into every peer's exchange buffer, waits (bounded) for the peers' rows in the local
// buffer, merges and gates. Used by the stand-alone exchange kernel and by the tail of decode_combine_kernel, where the rank's partial is
// formed, so that a cross-GPU decode layer needs no launch of its own for the exchange.
// Every value travels as one 8-byte store {value, call number}: an aligned 8-byte store arrives whole, so the number is the value's own flag
// and the receiver needs no fence and no separate flag: one crossing of NVLink per layer instead of stores, a system-wide fence (a round trip)
// and a flag store (measured on two GPUs: 11.5 us per layer for the exchange with the fence-and-flag form).
// Remote memory is only ever stored to; every load is from local memory; no TMA, no multicast.
#pragma once
#include "kata_internal.cuh"

namespace kata {

constexpr int kPeerMaxWorld = 8, kPeerRows = 2 * kH;   // T <= 2 tokens x 24 heads

// What a kernel needs to reach the exchange: every rank's buffer (own included), this call's number and the wait budget. world == 0: none.
struct PeerSink { float* base[kPeerMaxWorld]; int32_t rank, world; uint32_t seq, max_polls; int32_t* err; };

// A rank's buffer: [call parity][source rank][row][258] slots of 8 bytes {value bits, call number}: O[256], m, l of the source's part of the row.
__host__ __device__ inline size_t peer_slot_off(int world, int parity, int src_rank, int row) { return (((size_t)parity * world + src_rank) * kPeerRows + row) * kPartStride; }   // in 8-byte slots
inline size_t peer_bytes(int world) { return (size_t)2 * world * kPeerRows * kPartStride * 8; }

#ifdef __CUDACC__
__device__ __forceinline__ void st_slot_sys(uint2* p, float v, uint32_t seq) { asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(seq) : "memory"); }
__device__ __forceinline__ uint2 ld_slot_sys(const uint2* p) { uint2 v; asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory"); return v; }

// Called by 256 threads (tid = head dim) that synchronise on named barrier `bar_id`; v = this rank's unnormalised O[tid] of the row, (m, l) its
// maximum (natural-log units) and sum. s_ok: one int of shared memory. Writes out[t][h][tid] = merge over ranks / l * sigmoid(gate), or nothing
// when a peer's row does not arrive within the budget (the error word then names the rank).
__device__ __forceinline__ void peer_row_exchange(const PeerSink& px, const int t, const int h, const int tid, const float v, const float m, const float l,
                                                  const float* __restrict__ gate, void* __restrict__ out, const int out_kind, int* s_ok, const int bar_id) {
    __shared__ float s_pml[kPeerMaxWorld][2];   // the peers' (m, l) of this row
    const int row = t * kH + h, parity = (int)(px.seq & 1u), world = px.world, rank = px.rank;
    for (int r = 0; r < world; r++) {   // my row into every peer's buffer
        if (r == rank) continue;
        uint2* dst = reinterpret_cast<uint2*>(px.base[r]) + peer_slot_off(world, parity, rank, row);
        st_slot_sys(dst + tid, v, px.seq);
        if (tid < 2) st_slot_sys(dst + 256 + tid, tid == 0 ? m : l, px.seq);
    }
    if (tid == 0) *s_ok = 1;
    asm volatile("bar.sync %0, 256;" ::"r"(bar_id) : "memory");
    // every thread waits for its own element of every peer's row (and threads 0, 1 for the row's m and l): the call number beside the value says it is this call's
    float pv[kPeerMaxWorld];
    const uint2* loc = reinterpret_cast<const uint2*>(px.base[rank]);
#pragma unroll
    for (int r = 0; r < kPeerMaxWorld; r++) {
        pv[r] = 0.0f;
        if (r >= world || r == rank) continue;
        const uint2* src = loc + peer_slot_off(world, parity, r, row);
        bool ok = false;
        for (uint32_t i = 0; i < px.max_polls; i++) {
            const uint2 e = ld_slot_sys(src + tid);
            if (e.y == px.seq) { pv[r] = __uint_as_float(e.x); ok = true; break; }
            if ((i & 63u) == 63u && *reinterpret_cast<const volatile int32_t*>(px.err) != 0) break;   // another row already gave up
            __nanosleep(100);
        }
        if (ok && tid < 2) {
            ok = false;
            for (uint32_t i = 0; i < px.max_polls; i++) {
                const uint2 e = ld_slot_sys(src + 256 + tid);
                if (e.y == px.seq) { s_pml[r][tid] = __uint_as_float(e.x); ok = true; break; }
                if ((i & 63u) == 63u && *reinterpret_cast<const volatile int32_t*>(px.err) != 0) break;
                __nanosleep(100);
            }
        }
        if (!ok) { *s_ok = 0; atomicExch(px.err, 30 + r); }
    }
    asm volatile("bar.sync %0, 256;" ::"r"(bar_id) : "memory");
    if (!*s_ok) return;
    float M = m;
    for (int r = 0; r < world; r++) if (r != rank) M = fmaxf(M, s_pml[r][0]);
    // the ranks' terms are added in rank order, each with one fused multiply-add, whichever rank adds them (merge_parts_kernel does the same): every
    // rank, and the all-gather route, form the same sums bit for bit
    float Ls = 0.0f, As = 0.0f;
#pragma unroll
    for (int r = 0; r < kPeerMaxWorld; r++) {
        if (r >= world) continue;
        const float mm = r == rank ? m : s_pml[r][0], wt = (mm == -INFINITY) ? 0.0f : expf(mm - M);
        Ls = fmaf(r == rank ? l : s_pml[r][1], wt, Ls); As = fmaf(r == rank ? v : pv[r], wt, As);
    }
    const int64_t oi = (int64_t)t * kQD + h * kD + tid; const float y = (As / Ls) * (1.0f / (1.0f + expf(-gate[oi])));
    store_act(out, oi, y, out_kind);
}
#endif

}  // namespace kata
