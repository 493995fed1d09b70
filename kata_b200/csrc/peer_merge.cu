// Split-KV across GPUs without a library collective: every rank pushes its partial rows {O[256], m, l} straight into its
// peers' exchange buffers with ordinary stores over NVLink, waits (bounded) for the peers' rows
// in its own buffer and applies the reference's split merge (k_attn_dec_combine, shaders/flash.metal:143-152, with "split" =
// rank) plus the output gate: one kernel, no host synchronisation, no NCCL launch on the per-layer path. The reference is
// single-device and has no counterpart.
//
// Memory: one cudaMalloc per rank holding [2 parities][world][48 rows][258] slots of 8 bytes {value, call number}; peers map it
// through CUDA IPC handles (or, inside one process, by plain device pointers). Loads only ever touch local memory; remote
// memory is written, never read, and nothing here uses TMA or multicast.
// Protocol of call number s (1, 2, ...; all ranks issue the same sequence of calls): CTA (head, token) of rank a stores every value of its row
// together with s, 8 bytes at a time, into slot [s & 1][a][row] of every peer, then polls its own slots [s & 1][b][row] for every peer b until
// each reads s beside its value, and merges. An aligned 8-byte store arrives whole, so a value is there as soon as its number is: no fence and no
// separate flag (the first version stored the row, fenced system-wide and then raised a flag: a round trip and a crossing of NVLink more, 11.5 us
// per layer on two GPUs). Two parities suffice: a rank cannot finish call s + 1 (and so start overwriting parity s & 1 in call s + 2) before every
// peer has stored its rows of call s + 1, which a peer does only after its merge of call s has read parity s & 1.
// Every wait is bounded (about a second); a wait that runs out sets the exchange's error word, the row's output is left unwritten,
// and kata_attn_peer_check reports KATA_ERR_DEVICE_WAIT; the GPU and the attention context stay usable. The exchange itself is then out
// of step (the ranks' call numbers differ): kata_attn_peer_resync on every rank, or a fresh exchange, puts it right.
#include <cstdio>
#include <cstring>
#include <new>
#include <string>

#include "kata_internal.cuh"
#include "peer_exchange.cuh"

namespace kata {
int decode_partial_impl(kata_attn_ctx* h, int32_t layer, int32_t seq, int32_t pos_base, int32_t T, int32_t key_lo, int32_t key_hi, const void* d_q16, float* d_part,
                        const PeerSink* sink, const float* d_gate, void* d_out, int32_t out_dtype, bool* sink_used, void* stream);
namespace {

// grid (24 heads, T) x 256 threads: the exchange of rows a decode launch left in d_part
__global__ void __launch_bounds__(256) peer_push_merge_kernel(const PeerSink px, const float* __restrict__ part, const float* __restrict__ gate, void* __restrict__ out, const int out_kind) {
    __shared__ int s_ok;
    const int h = blockIdx.x, t = blockIdx.y, tid = threadIdx.x;
    pdl_wait(); pdl_launch_dependents();   // the local part comes from the decode kernel launched just before
    const float* mine = part + (int64_t)(t * kH + h) * kPartStride;
    peer_row_exchange(px, t, h, tid, mine[tid], mine[256], mine[257], gate, out, out_kind, &s_ok, 1);
}

}  // namespace
}  // namespace kata

struct kata_attn_peer {
    int device = 0, rank = 0, world = 1;
    float* local = nullptr; int32_t* d_err = nullptr; float* d_part = nullptr;   // d_part: this rank's part rows for kata_attn_peer_decode
    float* bases[kata::kPeerMaxWorld] = {}; bool opened = false, ipc[kata::kPeerMaxWorld] = {};
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
    p->bases[rank] = p->local;
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
        p->bases[r] = (float*)ptr; p->ipc[r] = true;
    }
    p->opened = true;
    return KATA_OK;
}

int kata_attn_peer_open_pointers(kata_attn_peer* p, void* const* bases) {
    if (!p || !bases) return KATA_ERR_ARG;
    for (int r = 0; r < p->world; r++) if (r != p->rank) { if (!bases[r]) return pfail(p, KATA_ERR_ARG, "null peer buffer"); p->bases[r] = (float*)bases[r]; }
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
    PeerSink px{}; for (int r = 0; r < p->world; r++) px.base[r] = p->bases[r];
    px.rank = p->rank; px.world = p->world; px.seq = ++p->seq; px.max_polls = p->max_polls; px.err = p->d_err;
    const cudaError_t e = launch_pdl(peer_push_merge_kernel, dim3(kH, T), dim3(256), 0, (cudaStream_t)stream, px, d_part, d_gate, d_out, (int)out_dtype);
    if (e != cudaSuccess) return pfail(p, KATA_ERR_CUDA, "exchange launch", e);
    p->launches++;
    return KATA_OK;
}

int kata_attn_peer_decode(kata_attn_peer* p, kata_attn_ctx* ctx, int32_t layer, int32_t seq, int32_t pos_base, int32_t T, int32_t key_lo, int32_t key_hi,
                          const void* d_q16, const float* d_gate, void* d_out, int32_t out_dtype, void* stream) {
    if (!p || !ctx) return KATA_ERR_ARG;
    if (!p->opened) return pfail(p, KATA_ERR_MODE, "the peers' buffers have not been opened");
    if (!d_gate || !d_out || (out_dtype != KATA_ACT_F32 && out_dtype != KATA_ACT_BF16 && out_dtype != KATA_ACT_F16)) return pfail(p, KATA_ERR_ARG, "peer_decode: gate, out and a known output dtype");
    // The exchange of this call, should the decode launch be able to do it itself (it can when its rows leave through the combine grid:
    // long local slices); the call number is only consumed if it did.
    PeerSink px{}; for (int r = 0; r < p->world; r++) px.base[r] = p->bases[r];
    px.rank = p->rank; px.world = p->world; px.seq = p->seq + 1; px.max_polls = p->max_polls; px.err = p->d_err;
    bool used = false;
    if (const int rc = decode_partial_impl(ctx, layer, seq, pos_base, T, key_lo, key_hi, d_q16, p->d_part, &px, d_gate, d_out, out_dtype, &used, stream)) return pfail(p, rc, kata_attn_last_error(ctx));
    if (used) { p->seq++; p->launches++; return KATA_OK; }
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
    e = cudaMemset(p->local, 0, peer_bytes(p->world));   // no slot carries a call number any more
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
    for (int r = 0; r < p->world; r++) if (p->ipc[r] && p->bases[r]) cudaIpcCloseMemHandle(p->bases[r]);
    if (p->local) cudaFree(p->local);
    if (p->d_err) cudaFree(p->d_err);
    if (p->d_part) cudaFree(p->d_part);
    cudaGetLastError();
    delete p;
    return KATA_OK;
}

}  // extern "C"
