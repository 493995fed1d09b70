// Split-KV across GPUs without a library collective: every rank pushes its partial rows {O[256], m, l} straight into its
// peers' exchange buffers with ordinary stores over NVLink, raises a per-row flag there, waits (bounded) for the peers' rows
// in its own buffer and applies the reference's split merge (k_attn_dec_combine, shaders/flash.metal:143-152, with "split" =
// rank) plus the output gate: one kernel, no host synchronisation, no NCCL launch on the per-layer path. The reference is
// single-device and has no counterpart.
//
// Memory: one cudaMalloc per rank holding [2 parities][world][48 rows][258] floats and [2][world][48] flags; peers map it
// through CUDA IPC handles (or, inside one process, by plain device pointers). Loads only ever touch local memory; remote
// memory is written, never read, and nothing here uses TMA or multicast.
// Protocol of call number s (1, 2, ...; all ranks issue the same sequence of calls): CTA (head, token) of rank a copies its row
// into slot [s & 1][a][row] of every rank, fences system-wide, stores s into flag [s & 1][a][row] of every rank, then polls its own
// flags [s & 1][b][row] for every b until they read s, and merges. Two parities suffice: a rank cannot finish call s + 1 (and so
// start overwriting parity s & 1 in call s + 2) before every peer has raised its flags of call s + 1, which a peer does only after
// its merge of call s has read parity s & 1.
// Every wait is bounded (about a second); a wait that runs out sets the exchange's error word, the row's output is left unwritten,
// and kata_attn_peer_check reports KATA_ERR_DEVICE_WAIT; the GPU and the attention context stay usable. The exchange itself is then out
// of step (the ranks' call numbers differ): kata_attn_peer_resync on every rank, or a fresh exchange, puts it right.
#include <cstdio>
#include <cstring>
#include <new>
#include <string>

#include "kata_internal.cuh"

namespace kata {
namespace {

constexpr int kPeerMaxWorld = 8, kPeerRows = 2 * kH;   // T <= 2 tokens x 24 heads

struct PeerBases { float* base[kPeerMaxWorld]; };

__host__ __device__ inline size_t peer_part_off(int world, int parity, int src_rank, int row) { return (((size_t)parity * world + src_rank) * kPeerRows + row) * kPartStride; }   // in floats
__host__ __device__ inline size_t peer_flag_off(int world, int parity, int src_rank, int row) { return (size_t)2 * world * kPeerRows * kPartStride + ((size_t)parity * world + src_rank) * kPeerRows + row; }   // in 4-byte words
inline size_t peer_bytes(int world) { return ((size_t)2 * world * kPeerRows * kPartStride + (size_t)2 * world * kPeerRows) * 4; }

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) { asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) { uint32_t v; asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v; }

// grid (24 heads, T) x 256 threads
__global__ void __launch_bounds__(256) peer_push_merge_kernel(const PeerBases pb, const int rank, const int world, const uint32_t seq, const uint32_t max_polls,
                                                              const float* __restrict__ part, const int T, const float* __restrict__ gate, void* __restrict__ out, const int out_kind, int32_t* err) {
    __shared__ int s_ok;
    const int h = blockIdx.x, t = blockIdx.y, tid = threadIdx.x, row = t * kH + h, parity = (int)(seq & 1u);
    pdl_wait(); pdl_launch_dependents();   // the local part comes from the decode kernel launched just before
    const float* mine = part + (int64_t)row * kPartStride;
    const float v = mine[tid], ml = tid < 2 ? mine[256 + tid] : 0.0f;
    for (int r = 0; r < world; r++) {   // my row into everybody's buffer (my own included: the merge then reads one place)
        float* dst = pb.base[r] + peer_part_off(world, parity, rank, row);
        dst[tid] = v; if (tid < 2) dst[256 + tid] = ml;
    }
    __threadfence_system();
    if (tid == 0) s_ok = 1;
    __syncthreads();
    if (tid < world) st_release_sys(reinterpret_cast<uint32_t*>(pb.base[tid]) + peer_flag_off(world, parity, rank, row), seq);
    if (tid < world) {   // thread b waits for rank b's row
        const uint32_t* flag = reinterpret_cast<const uint32_t*>(pb.base[rank]) + peer_flag_off(world, parity, tid, row);
        bool ok = false;
        for (uint32_t i = 0; i < max_polls; i++) {
            if (ld_acquire_sys(flag) == seq) { ok = true; break; }
            if ((i & 63u) == 63u && *reinterpret_cast<const volatile int32_t*>(err) != 0) break;   // another row already gave up
            __nanosleep(500);
        }
        if (!ok) { s_ok = 0; atomicExch(err, 30 + tid); }
    }
    __syncthreads();
    if (!s_ok) return;
    const float* loc = pb.base[rank];
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

}  // namespace
}  // namespace kata

struct kata_attn_peer {
    int device = 0, rank = 0, world = 1;
    float* local = nullptr; int32_t* d_err = nullptr; float* d_part = nullptr;   // d_part: this rank's part rows for kata_attn_peer_decode
    kata::PeerBases bases{}; bool opened = false, ipc[kata::kPeerMaxWorld] = {};
    uint32_t seq = 0, max_polls = 1u << 20;   // about a second of polling at 0.5-1 us per poll
    uint64_t launches = 0;
    std::string err;
};

using namespace kata;

namespace {
struct PeerGuard {
    int prev = -1;
    explicit PeerGuard(int dev) { cudaGetDevice(&prev); if (prev != dev) cudaSetDevice(dev); else prev = -1; }
    ~PeerGuard() { if (prev >= 0) cudaSetDevice(prev); }
};
int pfail(kata_attn_peer* p, int code, const char* msg, cudaError_t e = cudaSuccess) {
    p->err = msg; if (e != cudaSuccess) { p->err += ": "; p->err += cudaGetErrorString(e); }
    return code;
}
}  // namespace

extern "C" {

int kata_attn_peer_create(int32_t device, int32_t rank, int32_t world, kata_attn_peer** out, void* handle_out) {
    if (!out) return KATA_ERR_ARG;
    *out = nullptr;
    if (world < 1 || world > kPeerMaxWorld || rank < 0 || rank >= world) return KATA_ERR_RANGE;
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || device < 0 || device >= ndev) return KATA_ERR_CUDA;
    kata_attn_peer* p = new (std::nothrow) kata_attn_peer();
    if (!p) return KATA_ERR_NOMEM;
    p->device = device; p->rank = rank; p->world = world;
    PeerGuard guard(device);
    if (cudaMalloc((void**)&p->local, peer_bytes(world)) != cudaSuccess || cudaMalloc((void**)&p->d_err, 4) != cudaSuccess || cudaMalloc((void**)&p->d_part, (size_t)kPeerRows * kPartStride * 4) != cudaSuccess) { cudaGetLastError(); kata_attn_peer_destroy(p); return KATA_ERR_NOMEM; }
    cudaMemset(p->local, 0, peer_bytes(world)); cudaMemset(p->d_err, 0, 4);
    p->bases.base[rank] = p->local;
    if (handle_out) {
        static_assert(sizeof(cudaIpcMemHandle_t) == KATA_PEER_HANDLE_BYTES, "handle size");
        cudaIpcMemHandle_t hd;
        if (cudaIpcGetMemHandle(&hd, p->local) != cudaSuccess) { cudaGetLastError(); kata_attn_peer_destroy(p); return KATA_ERR_CUDA; }
        memcpy(handle_out, &hd, sizeof hd);
    }
    if (cudaDeviceSynchronize() != cudaSuccess) { kata_attn_peer_destroy(p); return KATA_ERR_CUDA; }
    p->opened = world == 1;
    *out = p;
    return KATA_OK;
}

int kata_attn_peer_open(kata_attn_peer* p, const void* handles) {
    if (!p || !handles) return KATA_ERR_ARG;
    PeerGuard guard(p->device);
    for (int r = 0; r < p->world; r++) {
        if (r == p->rank) continue;
        cudaIpcMemHandle_t hd; memcpy(&hd, (const uint8_t*)handles + (size_t)r * KATA_PEER_HANDLE_BYTES, sizeof hd);
        void* ptr = nullptr;
        const cudaError_t e = cudaIpcOpenMemHandle(&ptr, hd, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) return pfail(p, KATA_ERR_CUDA, "cudaIpcOpenMemHandle", e);
        p->bases.base[r] = (float*)ptr; p->ipc[r] = true;
    }
    p->opened = true;
    return KATA_OK;
}

int kata_attn_peer_open_pointers(kata_attn_peer* p, void* const* bases) {
    if (!p || !bases) return KATA_ERR_ARG;
    for (int r = 0; r < p->world; r++) if (r != p->rank) { if (!bases[r]) return pfail(p, KATA_ERR_ARG, "null peer buffer"); p->bases.base[r] = (float*)bases[r]; }
    p->opened = true;
    return KATA_OK;
}

void* kata_attn_peer_buffer(kata_attn_peer* p) { return p ? p->local : nullptr; }
const char* kata_attn_peer_last_error(const kata_attn_peer* p) { return p ? p->err.c_str() : "null exchange"; }

int kata_attn_peer_set_wait_polls(kata_attn_peer* p, uint32_t polls) { if (!p || !polls) return KATA_ERR_ARG; p->max_polls = polls; return KATA_OK; }

int kata_attn_peer_exchange_merge(kata_attn_peer* p, const float* d_part, int32_t T, const float* d_gate, void* d_out, int32_t out_dtype, void* stream) {
    if (!p) return KATA_ERR_ARG;
    if (!p->opened) return pfail(p, KATA_ERR_MODE, "the peers' buffers have not been opened");
    if (!d_part || !d_gate || !d_out || T < 1 || T > 2 || (out_dtype != KATA_ACT_F32 && out_dtype != KATA_ACT_BF16 && out_dtype != KATA_ACT_F16)) return pfail(p, KATA_ERR_ARG, "exchange_merge: part, gate, out, T in {1, 2}");
    PeerGuard guard(p->device);
    const uint32_t seq = ++p->seq;
    const cudaError_t e = launch_pdl(peer_push_merge_kernel, dim3(kH, T), dim3(256), 0, (cudaStream_t)stream, p->bases, p->rank, p->world, seq, p->max_polls, d_part, (int)T, d_gate, d_out,
                                     (int)out_dtype, p->d_err);
    if (e != cudaSuccess) return pfail(p, KATA_ERR_CUDA, "exchange launch", e);
    p->launches++;
    return KATA_OK;
}

int kata_attn_peer_decode(kata_attn_peer* p, kata_attn_ctx* ctx, int32_t layer, int32_t seq, int32_t pos_base, int32_t T, int32_t key_lo, int32_t key_hi,
                          const void* d_q16, const float* d_gate, void* d_out, int32_t out_dtype, void* stream) {
    if (!p || !ctx) return KATA_ERR_ARG;
    if (const int rc = kata_attn_decode_partial(ctx, layer, seq, pos_base, T, key_lo, key_hi, d_q16, p->d_part, stream)) return pfail(p, rc, kata_attn_last_error(ctx));
    return kata_attn_peer_exchange_merge(p, p->d_part, T, d_gate, d_out, out_dtype, stream);
}

int kata_attn_peer_check(kata_attn_peer* p, void* stream) {
    if (!p) return KATA_ERR_ARG;
    PeerGuard guard(p->device);
    cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream); if (e != cudaSuccess) return pfail(p, KATA_ERR_CUDA, "synchronize", e);
    int32_t flag = 0; e = cudaMemcpy(&flag, p->d_err, 4, cudaMemcpyDeviceToHost); if (e != cudaSuccess) return pfail(p, KATA_ERR_CUDA, "read error word", e);
    if (flag) { cudaMemset(p->d_err, 0, 4); char b[128]; snprintf(b, sizeof b, "the wait for rank %d's rows ran out; that call's output is invalid", flag - 30); return pfail(p, KATA_ERR_DEVICE_WAIT, b); }
    return KATA_OK;
}

int kata_attn_peer_resync(kata_attn_peer* p, uint32_t call_number) {
    if (!p) return KATA_ERR_ARG;
    PeerGuard guard(p->device);
    cudaError_t e = cudaDeviceSynchronize(); if (e != cudaSuccess) return pfail(p, KATA_ERR_CUDA, "synchronize", e);
    const size_t flag_bytes = (size_t)2 * p->world * kPeerRows * 4;
    e = cudaMemset(reinterpret_cast<uint8_t*>(p->local) + peer_flag_off(p->world, 0, 0, 0) * 4, 0, flag_bytes);
    if (e == cudaSuccess) e = cudaMemset(p->d_err, 0, 4);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return pfail(p, KATA_ERR_CUDA, "resync", e);
    p->seq = call_number;
    return KATA_OK;
}

int kata_attn_peer_destroy(kata_attn_peer* p) {
    if (!p) return KATA_ERR_ARG;
    PeerGuard guard(p->device);
    cudaDeviceSynchronize();
    for (int r = 0; r < p->world; r++) if (p->ipc[r] && p->bases.base[r]) cudaIpcCloseMemHandle(p->bases.base[r]);
    if (p->local) cudaFree(p->local);
    if (p->d_err) cudaFree(p->d_err);
    if (p->d_part) cudaFree(p->d_part);
    cudaGetLastError();
    delete p;
    return KATA_OK;
}

}  // extern "C"
