// Device side of the split-KV exchange between the GPUs of one box (see peer_merge.cu for the protocol): one CTA-wide routine that takes
// this rank's partial of one (token, head) row, stores it into every rank's exchange buffer, raises the row's flag there, waits (bounded)
// for the peers' rows in the local buffer, merges and gates. Used by the stand-alone exchange kernel and by the tail of decode_combine_kernel,
// where the rank's partial is formed, so that a cross-GPU decode layer needs no launch of its own for the exchange.
// Remote memory is only ever stored to; every load is from local memory; no TMA, no multicast.
#pragma once
#include "kata_internal.cuh"

namespace kata {

constexpr int kPeerMaxWorld = 8, kPeerRows = 2 * kH;   // T <= 2 tokens x 24 heads

// What a kernel needs to reach the exchange: every rank's buffer (own included), this call's number and the wait budget. world == 0: none.
struct PeerSink { float* base[kPeerMaxWorld]; int32_t rank, world; uint32_t seq, max_polls; int32_t* err; };

__host__ __device__ inline size_t peer_part_off(int world, int parity, int src_rank, int row) { return (((size_t)parity * world + src_rank) * kPeerRows + row) * kPartStride; }   // in floats
__host__ __device__ inline size_t peer_flag_off(int world, int parity, int src_rank, int row) { return (size_t)2 * world * kPeerRows * kPartStride + ((size_t)parity * world + src_rank) * kPeerRows + row; }   // in 4-byte words
inline size_t peer_bytes(int world) { return ((size_t)2 * world * kPeerRows * kPartStride + (size_t)2 * world * kPeerRows) * 4; }

#ifdef __CUDACC__
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) { asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) { uint32_t v; asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v; }

// Called by 256 threads (tid = head dim) that synchronise on named barrier `bar_id`; v = this rank's unnormalised O[tid] of the row, (m, l) its
// maximum (natural-log units) and sum. s_ok: one int of shared memory. Writes out[t][h][tid] = merge over ranks / l * sigmoid(gate), or nothing
// when a peer's row does not arrive within the budget (the error word then names the rank).
__device__ __forceinline__ void peer_row_exchange(const PeerSink& px, const int t, const int h, const int tid, const float v, const float m, const float l,
                                                  const float* __restrict__ gate, void* __restrict__ out, const int out_kind, int* s_ok, const int bar_id) {
    const int row = t * kH + h, parity = (int)(px.seq & 1u), world = px.world, rank = px.rank;
    for (int r = 0; r < world; r++) {   // my row into everybody's buffer (my own included: the merge then reads one place)
        float* dst = px.base[r] + peer_part_off(world, parity, rank, row);
        dst[tid] = v; if (tid == 0) { dst[256] = m; dst[257] = l; }
    }
    __threadfence_system();
    if (tid == 0) *s_ok = 1;
    asm volatile("bar.sync %0, 256;" ::"r"(bar_id) : "memory");
    if (tid < world) st_release_sys(reinterpret_cast<uint32_t*>(px.base[tid]) + peer_flag_off(world, parity, rank, row), px.seq);
    if (tid < world) {   // thread b waits for rank b's row
        const uint32_t* flag = reinterpret_cast<const uint32_t*>(px.base[rank]) + peer_flag_off(world, parity, tid, row);
        bool ok = false;
        for (uint32_t i = 0; i < px.max_polls; i++) {
            if (ld_acquire_sys(flag) == px.seq) { ok = true; break; }
            if ((i & 63u) == 63u && *reinterpret_cast<const volatile int32_t*>(px.err) != 0) break;   // another row already gave up
            __nanosleep(500);
        }
        if (!ok) { *s_ok = 0; atomicExch(px.err, 30 + tid); }
    }
    asm volatile("bar.sync %0, 256;" ::"r"(bar_id) : "memory");
    if (!*s_ok) return;
    const float* loc = px.base[rank];
    float M = -INFINITY;
    for (int r = 0; r < world; r++) M = fmaxf(M, __ldcg(loc + peer_part_off(world, parity, r, row) + 256));
    float L = 0.0f, A = 0.0f;
    for (int r = 0; r < world; r++) {
        const float* pp = loc + peer_part_off(world, parity, r, row); const float mm = __ldcg(pp + 256), wt = (mm == -INFINITY) ? 0.0f : expf(mm - M);
        L += __ldcg(pp + 257) * wt; A += __ldcg(pp + tid) * wt;
    }
    const int64_t oi = (int64_t)t * kQD + h * kD + tid; const float y = (A / L) * (1.0f / (1.0f + expf(-gate[oi])));
    store_act(out, oi, y, out_kind);
}
#endif

}  // namespace kata
