// CPU oracle for the gated-GQA attention path of wolfjpy/kata.
//
// THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE. Only the test-suite, the smoke check and the CPU-baseline /
// reference arm of the benchmark may load it. The CUDA library never links or calls anything in this file.
//
// What it is: a plain C++ restatement, written from the reference's shader sources, of every kernel on the
// attention hot path, in the reference's operation order and with the reference's rounding points (fp32 data path;
// K/V rows rounded to fp16 when cached; Q * 1/16 rounded to fp16 on the matrix paths; P rounded to fp16 before P.V).
// Each function cites the reference lines it follows (paths relative to the reference project root).
//
// Pinning status. The reference stores NO golden vectors for this path and its kernels are Metal shaders that cannot be
// compiled or run outside macOS. The only CPU arithmetic the reference holds for this path is its own check,
// tools/probe_flash.cpp:29-34 (fp64 softmax(q.k) v sigmoid(g)) with its input recipe (:16-19, mt19937(5), N(0,1)) and NaN
// poison (:26). Those lines ARE compiled here, lifted by line range into oracle/_ref/probe_ref.cpp by `make ref`
// (probe_ref_shim.h supplies host buffers in place of MTL::Buffer), and tests/test_probe_ref_cpu.py requires:
//   (1) kor_formula_f64 below == the reference's fp64 values bit for bit on the reference's own inputs;
//   (2) the restated matrix kernel (kor_flash_prefill) and the fp32 formula within 2e-4 / 2e-5 of them as judged by the
//       reference's own loop (the reference reports 6.6e-5 for its Metal kernel on this procedure).
// So the FORMULA level of this oracle is pinned to reference code compiled here. What stays UNPINNED ("parity unpinned"
// for these): the accumulation order inside the MSL kernels (restated from source, never executed here), and the prep /
// quantiser kernels, for which the reference has no CPU code; the quantiser is cross-checked bit for bit against an
// independent numpy restatement, and the reference's cross-path equalities (scalar split == matrix split == flash
// prefill, T=2 verify == two T=1 decodes) hold between the restated kernels.
//
// Third-party arithmetic not in the reference tree: Apple MetalPerformancePrimitives matmul2d (Apple SDK
// "MacOSX27.0", closed source) performs Q.K^T and P.V at shaders/flash.metal:44,58,116,130. Its accumulation order
// is unknown; this oracle accumulates in fp32 in index order, which is why floating-point parity is tolerance-level.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <memory>
#include <thread>
#include <vector>

#if defined(__has_include)
#if __has_include("kata_m6.h")
#include "kata_m6.h"   // the reference's own constants, when the build recipe puts its config directory on the include path
#define KOR_HAVE_REF_CONFIG 1
#endif
#endif

namespace {

constexpr uint32_t kH = 24, kKvh = 4, kD = 256, kG = 6, kQD = 6144, kKVD = 1024, kQFull = 12288, kRot = 64;
constexpr float kEps = 1e-6f, kTheta = 10000000.0f;

#ifdef KOR_HAVE_REF_CONFIG
static_assert(kata::kHeads == kH && kata::kKvHeads == kKvh && kata::kHeadDim == kD && kata::kRotDim == kRot, "geometry differs from config/kata_m6.h");
static_assert(kata::kQProjOut == kQFull && kata::kKvDim == kKVD && kata::kAttnOutIn == kQD, "row widths differ from config/kata_m6.h");
static_assert(kata::kRmsEps == kEps && kata::kRopeTheta == kTheta, "eps/theta differ from config/kata_m6.h");
#endif

using f16 = _Float16;
inline float h2f(uint16_t b) { f16 h; std::memcpy(&h, &b, 2); return (float)h; }
inline uint16_t f2h(float f) { f16 h = (f16)f; uint16_t b; std::memcpy(&b, &h, 2); return b; }   // round to nearest even
inline float bf2f(uint16_t b) { uint32_t u = (uint32_t)b << 16; float f; std::memcpy(&f, &u, 4); return f; }
constexpr float kNegInf = -std::numeric_limits<float>::infinity();

// shaders/common.h:45
inline float sigmoidf_(float x) { return 1.0f / (1.0f + std::exp(-x)); }

// Sum over the 32 lanes of a SIMD group as an xor butterfly (16, 8, 4, 2, 1); every lane ends with the same value.
// MSL's simd_sum order is unspecified; the CUDA kernels use this exact order so the two agree bit for bit.
inline float simd_sum32(const float* v) {
    float t[32]; for (int i = 0; i < 32; i++) t[i] = v[i];
    for (int off = 16; off >= 1; off >>= 1) { float n[32]; for (int i = 0; i < 32; i++) n[i] = t[i] + t[i ^ off]; std::memcpy(t, n, sizeof t); }
    return t[0];
}
// threadgroup reduction used by the 256-thread kernels: simd_sum per 32 lanes, then the 8 partials added in order
// (shaders/attn.metal:18-21, :50-54).
inline float tg_sum256(const float* v) { float tot = 0.0f; for (int s = 0; s < 8; s++) tot += simd_sum32(v + 32 * s); return tot; }

// One layer's cache planes. mode 0: K and V fp16; mode 1: both int8 with per-(position, head) fp16 scales (k_flash_prefill_q8 /
// k_attn_dec_split_q8); mode 2: K fp16, V int8 with its scales (k_flash_prefill_k16v8 / k_attn_dec_split_k16v8, shaders/flash.metal:194-306:
// the same tile body with the key scale and mean stripped out).
struct KvView {
    // mode 0 fp16; 1 int8 K and V, one scale per (position, KV head); 2 fp16 K, int8 V; 3 int8 K with one scale per 64 dims (ksc is [pos][4 heads][4 groups]),
    // int8 V per row: the finer K granularity the reference measured (docs/reports/M11-int8-kv.en.md:52-55) but could not fold into its matrix path (:94-97)
    const void* k; const void* v; const uint16_t* ksc; const uint16_t* vsc; const uint16_t* kmn; bool q8, v8, kg;
    KvView(const void* k_, const void* v_, const uint16_t* ksc_, const uint16_t* vsc_, const uint16_t* kmn_, int mode) : k(k_), v(v_), ksc(ksc_), vsc(vsc_), kmn(kmn_), q8(mode == 1), v8(mode == 1 || mode == 2 || mode == 3), kg(mode == 3) {}
    float kSg(uint64_t pos, uint32_t kvh, uint32_t d) const { return h2f(ksc[pos * 16 + kvh * 4 + (d >> 6)]); }   // mode 3: the scale of dim d's group
    float kraw(uint64_t pos, uint32_t kvh, uint32_t d) const { const uint64_t i = pos * kKVD + kvh * kD + d; return (q8 || kg) ? (float)((const int8_t*)k)[i] : h2f(((const uint16_t*)k)[i]); }
    float vraw(uint64_t pos, uint32_t kvh, uint32_t d) const { const uint64_t i = pos * kKVD + kvh * kD + d; return v8 ? (float)((const int8_t*)v)[i] : h2f(((const uint16_t*)v)[i]); }
    float kS(uint64_t pos, uint32_t kvh) const { return q8 ? h2f(ksc[pos * 4 + kvh]) : 1.0f; }
    float vS(uint64_t pos, uint32_t kvh) const { return v8 ? h2f(vsc[pos * 4 + kvh]) : 1.0f; }
    float kM(uint64_t pos, uint32_t kvh) const { return (q8 && kmn) ? h2f(kmn[pos * 4 + kvh]) : 0.0f; }
};

template <class F> void parallel_for(uint32_t n, uint32_t threads, F&& fn) {
    if (threads <= 1 || n <= 1) { for (uint32_t i = 0; i < n; i++) fn(i); return; }
    std::atomic<uint32_t> next{0}; std::vector<std::thread> pool;
    for (uint32_t t = 0; t < std::min(threads, n); t++) pool.emplace_back([&] { for (;;) { const uint32_t i = next.fetch_add(1); if (i >= n) return; fn(i); } });
    for (auto& th : pool) th.join();
}

// ---- shared tile body of k_flash_prefill and k_attn_dec_split (shaders/flash.metal:39-60 and :112-132) ----
// One 16-row block against keys [k0, k0+nk): S = Q.K^T (fp16 x fp16/int8 -> fp32), optional int8 scale/mean fold,
// mask, online softmax (row max, alpha, P = exp(S - m)), P rounded to fp16 (after the V scale in int8 mode),
// l += sum of the UNROUNDED p, O = O*alpha + P.V.
struct RowState { float m[16], l[16]; float o[16][kD]; };
template <class Mask>
void tile_step(const uint16_t* q16 /*[16][stride]*/, size_t qStride, const float* qSum, const KvView& kv, uint32_t kvh, uint32_t k0, int nk, RowState& st, Mask&& masked) {
    float S[16][64]; float P[16][64];
    for (int r = 0; r < 16; r++) for (int c = 0; c < 64; c++) {
        if (c >= nk) { S[r][c] = kNegInf; continue; }   // outside the tensor extent: never read (shaders/flash.metal:41-42)
        float a = 0.0f; for (uint32_t d = 0; d < kD; d++) a += h2f(q16[r * qStride + d]) * kv.kraw(k0 + c, kvh, d);
        if (kv.q8) a = a * kv.kS(k0 + c, kvh) + kv.kM(k0 + c, kvh) * qSum[r];
        if (masked(r, k0 + (uint32_t)c)) a = kNegInf;
        S[r][c] = a;
    }
    for (int r = 0; r < 16; r++) {
        float tmax = kNegInf; for (int c = 0; c < 64; c++) tmax = std::max(tmax, S[r][c]);
        const float mo = st.m[r], mn = std::max(mo, tmax);
        const float alpha = (mn == kNegInf) ? 1.0f : std::exp(mo - mn); st.m[r] = mn;
        const float sub = (mn == kNegInf) ? 0.0f : mn;
        float sum = 0.0f;
        for (int c = 0; c < 64; c++) { const float p = std::exp(S[r][c] - sub); sum += p; const float pv = (kv.v8 && c < nk) ? p * kv.vS(k0 + c, kvh) : p; P[r][c] = h2f(f2h(pv)); }
        st.l[r] = st.l[r] * alpha + sum;
        for (uint32_t d = 0; d < kD; d++) st.o[r][d] *= alpha;
        for (int c = 0; c < nk; c++) { const float p = P[r][c]; if (p == 0.0f) continue; for (uint32_t d = 0; d < kD; d++) st.o[r][d] += p * kv.vraw(k0 + c, kvh, d); }
    }
}
// note on `if (p == 0.0f) continue`: a masked key contributes exactly 0 * V; the matrix unit would produce NaN only
// if V held NaN or Inf there, which the reference avoids for keys beyond the extent by never reading them; keys inside
// the extent always hold finite cache rows.

void init_state(RowState& st) { for (int r = 0; r < 16; r++) { st.m[r] = kNegInf; st.l[r] = 0.0f; std::memset(st.o[r], 0, sizeof st.o[r]); } }

}  // namespace

extern "C" {

// Inverse RoPE frequencies pow(theta, -i/32), i in [0,32), in fp32 (shaders/attn.metal:26). Computed once on the
// host and handed to both the oracle and the CUDA kernels so the two use identical constants.
void kor_inv_freq(float* out32) { for (int i = 0; i < 32; i++) out32[i] = std::pow(kTheta, -(float)i / 32.0f); }

// k_attn_prep / k_attn_prep_b (shaders/attn.metal:5-37, shaders/prefill.metal:179-206).
// For token t in [0,M) at position pos0+t and head slot h in [h0, h0+nh): h<24 query head (RMSNorm, partial RoPE,
// gate split), 24..27 key head (RMSNorm, RoPE, fp16 store at row pos-cacheOff), 28..31 value head (fp16 copy at row
// pos-cacheOffV). Row strides 12288 / 1024 / 1024 in, 6144 out.
void kor_prep(const float* qfull, const float* kproj, const float* vproj, const float* qnorm, const float* knorm, const float* inv_freq,
              float* qout, float* gate_out, uint16_t* kcache, uint16_t* vcache,
              uint32_t pos0, uint32_t M, uint32_t h0, uint32_t nh, uint32_t cacheOff, uint32_t cacheOffV) {
    for (uint32_t t = 0; t < M; t++) for (uint32_t h = h0; h < h0 + nh; h++) {
        const uint32_t pos = pos0 + t;
        if (h >= 28) { const uint32_t vh = h - 28; for (uint32_t d = 0; d < kD; d++) vcache[(uint64_t)(pos - cacheOffV) * kKVD + vh * kD + d] = f2h(vproj[(uint64_t)t * kKVD + vh * kD + d]); continue; }
        float v[kD]; const float* w;
        if (h < 24) { for (uint32_t d = 0; d < kD; d++) { v[d] = qfull[(uint64_t)t * kQFull + h * 512 + d]; gate_out[(uint64_t)t * kQD + h * kD + d] = qfull[(uint64_t)t * kQFull + h * 512 + 256 + d]; } w = qnorm; }
        else { for (uint32_t d = 0; d < kD; d++) v[d] = kproj[(uint64_t)t * kKVD + (h - 24) * kD + d]; w = knorm; }
        float sq[kD]; for (uint32_t d = 0; d < kD; d++) sq[d] = v[d] * v[d];
        const float tot = tg_sum256(sq);
        const float r = 1.0f / std::sqrt(tot / 256.0f + kEps);   // MSL rsqrt, precise variant
        float xs[kD]; for (uint32_t d = 0; d < kD; d++) xs[d] = v[d] * r * w[d];
        float o[kD]; for (uint32_t d = 0; d < kD; d++) o[d] = xs[d];
        for (uint32_t i = 0; i < 32; i++) {   // partial RoPE: pair (i, i+32), angle formed in fp32
            const float theta = (float)pos * inv_freq[i]; const float c = std::cos(theta), s = std::sin(theta);
            const float a = xs[i], b = xs[i + 32]; o[i] = a * c - b * s; o[i + 32] = a * s + b * c;
        }
        if (h < 24) for (uint32_t d = 0; d < kD; d++) qout[(uint64_t)t * kQD + h * kD + d] = o[d];
        else for (uint32_t d = 0; d < kD; d++) kcache[(uint64_t)(pos - cacheOff) * kKVD + (h - 24) * kD + d] = f2h(o[d]);
    }
}

// k_kv_quant_sym / k_kv_quant (shaders/flash.metal:157-192). mode 0: symmetric, rint (ties to even) - the reference
// default; mode 1: symmetric, round half away from zero (not the reference; offered because the benchmark statement
// names it); mode 2: the reference's asymmetric-K variant (values stay symmetric), rint.
void kor_kv_quant(const uint16_t* ks, const uint16_t* vs, int8_t* kq, int8_t* vq, uint16_t* ksc, uint16_t* vsc, uint16_t* kmn, uint32_t pos0, uint32_t T, int mode) {
    auto rnd = [&](float x) { return mode == 1 ? std::round(x) : std::rint(x); };   // mode 3 (grouped K scales) rounds to even like mode 0
    for (uint32_t t = 0; t < T; t++) for (uint32_t g = kq ? 0 : 4; g < 8; g++) {   // kq == nullptr: values only (keys stay fp16)
        const bool isV = g >= 4; const uint32_t head = g & 3; const uint16_t* src = (isV ? vs : ks) + (uint64_t)t * kKVD + head * kD; const uint64_t pos = (uint64_t)pos0 + t;
        int8_t* dst = (isV ? vq : kq) + pos * kKVD + head * kD;
        if (!isV && mode == 3) {   // one scale per 64 dims of the key row: same arithmetic as k_kv_quant_sym on each group; ksc is [pos][4 heads][4 groups]
            for (uint32_t g4 = 0; g4 < 4; g4++) {
                float amax = 0.0f; for (uint32_t d = 64 * g4; d < 64 * g4 + 64; d++) amax = std::max(amax, std::fabs(h2f(src[d])));
                const uint16_t sc = amax > 0.0f ? f2h(amax / 127.0f) : f2h(1.0f); const float inv = 1.0f / h2f(sc);
                for (uint32_t d = 64 * g4; d < 64 * g4 + 64; d++) dst[d] = (int8_t)std::clamp(std::rint(h2f(src[d]) * inv), -127.0f, 127.0f);
                ksc[pos * 16 + head * 4 + g4] = sc;
            }
        } else if (isV || mode != 2) {
            float amax = 0.0f; for (uint32_t d = 0; d < kD; d++) amax = std::max(amax, std::fabs(h2f(src[d])));
            const uint16_t sc = amax > 0.0f ? f2h(amax / 127.0f) : f2h(1.0f); const float inv = 1.0f / h2f(sc);
            for (uint32_t d = 0; d < kD; d++) dst[d] = (int8_t)std::clamp(rnd(h2f(src[d]) * inv), -127.0f, 127.0f);
            if (isV) vsc[pos * 4 + head] = sc; else { ksc[pos * 4 + head] = sc; if (kmn) kmn[pos * 4 + head] = 0; }
        } else {
            float MX = kNegInf, MN = -kNegInf; for (uint32_t d = 0; d < kD; d++) { const float x = h2f(src[d]); MX = std::max(MX, x); MN = std::min(MN, x); }
            const float mean = 0.5f * (MX + MN); float sc = (MX - MN) / 254.0f; if (!(sc > 0.0f)) sc = 1.0f; const float inv = 1.0f / sc;
            for (uint32_t d = 0; d < kD; d++) dst[d] = (int8_t)std::clamp(rnd((h2f(src[d]) - mean) * inv), -127.0f, 127.0f);
            ksc[pos * 4 + head] = f2h(sc); if (kmn) kmn[pos * 4 + head] = f2h(mean);
        }
    }
}

// k_attn_decode (shaders/attn.metal:40-62): one query head, streaming softmax over keys [0, pos], fp32 Q.
void kor_attn_decode(const float* q, const float* gate, const uint16_t* kc, const uint16_t* vc, float* out, uint32_t pos, uint32_t threads) {
    parallel_for(kH, threads, [&](uint32_t h) {
        const uint32_t kvh = h / kG; float m = kNegInf, l = 0.0f; float acc[kD] = {};
        for (uint32_t j = 0; j <= pos; j++) {
            float pr[kD]; for (uint32_t d = 0; d < kD; d++) pr[d] = q[h * kD + d] * h2f(kc[(uint64_t)j * kKVD + kvh * kD + d]);
            const float s = tg_sum256(pr) * 0.0625f;
            const float mn = std::max(m, s), a = std::exp(m - mn), e = std::exp(s - mn);
            l = l * a + e; for (uint32_t d = 0; d < kD; d++) acc[d] = acc[d] * a + e * h2f(vc[(uint64_t)j * kKVD + kvh * kD + d]);
            m = mn;
        }
        for (uint32_t d = 0; d < kD; d++) out[h * kD + d] = (acc[d] / l) * sigmoidf_(gate[h * kD + d]);
    });
}

// k_attn_split / k_attn_split_b (shaders/attn.metal:66-108, shaders/prefill.metal:209-252): ALU flash-decoding.
// Grid (S, 4, T); 8 SIMD groups walk sub-slices; lane owns 8 dims; the 6 heads of a KV head share each row; the
// threadgroup merges its 8 partials. q is fp32 [T][6144]; token t sees keys [firstPos, posBase+t].
void kor_attn_split(const float* q, const uint16_t* kc, const uint16_t* vc, float* pm, float* pl, float* pacc, uint32_t posBase, uint32_t firstPos, uint32_t S, uint32_t T) {
    for (uint32_t t = 0; t < T; t++) for (uint32_t kvh = 0; kvh < kKvh; kvh++) for (uint32_t split = 0; split < S; split++) {
        const uint32_t npos = posBase + t + 1, span = npos - firstPos, per = (span + S - 1) / S, lo = firstPos + std::min(split * per, span), hi = std::min(lo + per, npos);
        float tm[8][6], tl[8][6]; static thread_local float tacc[8][6][kD];
        for (uint32_t sg = 0; sg < 8; sg++) {
            const uint32_t sper = (hi - lo + 7) / 8, slo = std::min(lo + sg * sper, hi), shi = std::min(slo + sper, hi);
            float m[6], l[6]; for (int h = 0; h < 6; h++) { m[h] = kNegInf; l[h] = 0.0f; std::memset(tacc[sg][h], 0, sizeof tacc[sg][h]); }
            for (uint32_t j = slo; j < shi; j++) for (uint32_t h = 0; h < 6; h++) {
                float lane_p[32];
                for (uint32_t lane = 0; lane < 32; lane++) { float p = 0.0f; for (uint32_t d = 0; d < 8; d++) p += (q[(uint64_t)t * kQD + (kvh * 6 + h) * kD + lane * 8 + d] * 0.0625f) * h2f(kc[(uint64_t)j * kKVD + kvh * kD + lane * 8 + d]); lane_p[lane] = p; }
                const float s = simd_sum32(lane_p);
                const float mn = std::max(m[h], s), a = std::exp(m[h] - mn), e = std::exp(s - mn);
                l[h] = l[h] * a + e; for (uint32_t d = 0; d < kD; d++) tacc[sg][h][d] = tacc[sg][h][d] * a + e * h2f(vc[(uint64_t)j * kKVD + kvh * kD + d]);
                m[h] = mn;
            }
            for (int h = 0; h < 6; h++) { tm[sg][h] = m[h]; tl[sg][h] = l[h]; }
        }
        for (uint32_t h = 0; h < 6; h++) {
            float Mx = kNegInf; for (int s = 0; s < 8; s++) Mx = std::max(Mx, tm[s][h]);
            const uint64_t ti = (uint64_t)t * 24 + kvh * 6 + h;
            for (uint32_t d = 0; d < kD; d++) { float A = 0.0f; for (int s = 0; s < 8; s++) { const float w = (tm[s][h] == kNegInf) ? 0.0f : std::exp(tm[s][h] - Mx); A += tacc[s][h][d] * w; } pacc[(ti * S + split) * kD + d] = A; }
            float L = 0.0f; for (int s = 0; s < 8; s++) { const float w = (tm[s][h] == kNegInf) ? 0.0f : std::exp(tm[s][h] - Mx); L += tl[s][h] * w; }
            pm[ti * S + split] = Mx; pl[ti * S + split] = L;
        }
    }
}
// k_attn_combine / k_attn_combine_b (shaders/attn.metal:111-117, shaders/prefill.metal:254-261).
void kor_attn_combine(const float* pm, const float* pl, const float* pacc, const float* gate, float* out, uint32_t S, uint32_t T) {
    for (uint32_t t = 0; t < T; t++) for (uint32_t h = 0; h < kH; h++) {
        const uint64_t ti = (uint64_t)t * 24 + h; float Mx = kNegInf; for (uint32_t s = 0; s < S; s++) Mx = std::max(Mx, pm[ti * S + s]);
        for (uint32_t d = 0; d < kD; d++) { float L = 0.0f, A = 0.0f; for (uint32_t s = 0; s < S; s++) { const float mm = pm[ti * S + s]; const float w = (mm == kNegInf) ? 0.0f : std::exp(mm - Mx); L += pl[ti * S + s] * w; A += pacc[(ti * S + s) * kD + d] * w; }
            out[(uint64_t)t * kQD + h * kD + d] = (A / L) * sigmoidf_(gate[(uint64_t)t * kQD + h * kD + d]); }
    }
}

// k_cvt_q_half (shaders/flash.metal:71): fp32 -> fp16 after the exact power-of-two scale.
void kor_cvt_q_half(const float* src, uint16_t* dst, uint64_t n) { for (uint64_t i = 0; i < n; i++) dst[i] = f2h(src[i] * 0.0625f); }

// k_dec_q_pack (shaders/flash.metal:77-82): qp[kvh][r][d], r = t*6 + j, zero rows >= 6T.
void kor_dec_q_pack(const float* q, uint16_t* qp, uint32_t T) {
    for (uint32_t i = 0; i < 4u * 16u * 256u; i++) { const uint32_t d = i & 255u, r = (i >> 8) & 15u, kvh = i >> 12, t = r / 6u, j = r % 6u;
        qp[i] = (r < 6u * T) ? f2h(q[(uint64_t)t * kQD + (kvh * 6u + j) * kD + d] * 0.0625f) : (uint16_t)0; }
}

// k_flash_prefill / k_flash_prefill_q8 (shaders/flash.metal:10-65): causal flash attention of M rows at positions
// posBase+r against keys [0, posBase+r], 16-row blocks, 64-key tiles, gated output. q16 is fp16 [M][6144] prescaled.
void kor_flash_prefill(const uint16_t* q16, const void* kc, const void* vc, const float* gate, float* out, uint32_t posBase, uint32_t M,
                       const uint16_t* ksc, const uint16_t* vsc, const uint16_t* kmn, int q8, uint32_t threads) {
    const KvView kv(kc, vc, ksc, vsc, kmn, q8); const uint32_t nQt = (M + 15) / 16;
    parallel_for(nQt * kH, threads, [&](uint32_t item) {
        const uint32_t qt = item / kH, h = item % kH, kvh = h / kG, q0 = qt * 16, rowsValid = std::min(16u, M - q0), posEnd = posBase + q0 + rowsValid, nTiles = (posEnd + 63) / 64;
        std::vector<uint16_t> qblk(16 * kD, 0); float qSum[16] = {};
        for (uint32_t r = 0; r < rowsValid; r++) { std::memcpy(&qblk[r * kD], q16 + (uint64_t)(q0 + r) * kQD + h * kD, kD * 2); if (q8) { float lane_s[32] = {}; for (uint32_t d = 0; d < kD; d++) lane_s[d & 31] += h2f(qblk[r * kD + d]); qSum[r] = simd_sum32(lane_s); } }
        auto st = std::make_unique<RowState>(); init_state(*st);
        for (uint32_t kt = 0; kt < nTiles; kt++) { const uint32_t k0 = kt * 64; const int nk = (int)std::min(64u, posEnd - k0);
            tile_step(qblk.data(), kD, qSum, kv, kvh, k0, nk, *st, [&](int r, uint32_t key) { return key > posBase + q0 + (uint32_t)r; }); }
        for (uint32_t r = 0; r < rowsValid; r++) for (uint32_t d = 0; d < kD; d++) { const uint64_t o = (uint64_t)(q0 + r) * kQD + h * kD + d; out[o] = st->o[r][d] / st->l[r] * sigmoidf_(gate[o]); }
    });
}

// k_attn_dec_split / _q8 (shaders/flash.metal:84-137): rows = 6 heads x T<=2 tokens of one KV head; split `split`
// covers keys [firstPos + split*chunk, min(+chunk, posBase+T)) in 64-key tiles; writes unnormalised O and (m, l).
void kor_attn_dec_split(const uint16_t* qp, const void* kc, const void* vc, float* pacc, float* pm, float* pl, uint32_t posBase, uint32_t T, uint32_t firstPos, uint32_t chunk,
                        const uint16_t* ksc, const uint16_t* vsc, const uint16_t* kmn, int q8, uint32_t threads) {
    const KvView kv(kc, vc, ksc, vsc, kmn, q8); const uint32_t posEnd = posBase + T, nSplits = (posEnd - firstPos + chunk - 1) / chunk;
    parallel_for(nSplits * kKvh, threads, [&](uint32_t item) {
        const uint32_t split = item / kKvh, kvh = item % kKvh, lo = firstPos + split * chunk, hi = std::min(lo + chunk, posEnd);
        const uint16_t* qb = qp + (uint64_t)kvh * 16 * kD; float qSum[16] = {};
        if (q8) for (int r = 0; r < 16; r++) { float lane_s[32] = {}; for (uint32_t d = 0; d < kD; d++) lane_s[d & 31] += h2f(qb[r * kD + d]); qSum[r] = simd_sum32(lane_s); }
        auto st = std::make_unique<RowState>(); init_state(*st);
        for (uint32_t k0 = lo; k0 < hi; k0 += 64) { const int nk = (int)std::min(64u, hi - k0);
            tile_step(qb, kD, qSum, kv, kvh, k0, nk, *st, [&](int r, uint32_t key) { return (uint32_t)r >= 6u * T || key > posBase + (uint32_t)r / 6u || key >= hi; }); }
        const uint64_t rowBase = ((uint64_t)kvh * nSplits + split) * 16;
        for (int r = 0; r < 16; r++) { std::memcpy(pacc + (rowBase + r) * kD, st->o[r], kD * 4); pm[rowBase + r] = st->m[r]; pl[rowBase + r] = st->l[r]; }
    });
}
// k_attn_dec_combine (shaders/flash.metal:143-152).
void kor_attn_dec_combine(const float* pacc, const float* pm, const float* pl, const float* gate, float* out, uint32_t posBase, uint32_t T, uint32_t firstPos, uint32_t chunk) {
    const uint32_t nSplits = (posBase + T - firstPos + chunk - 1) / chunk;
    for (uint32_t t = 0; t < T; t++) for (uint32_t h = 0; h < kH; h++) {
        const uint32_t kvh = h / 6, row = t * 6 + h % 6; float Mx = kNegInf; for (uint32_t s = 0; s < nSplits; s++) Mx = std::max(Mx, pm[((uint64_t)kvh * nSplits + s) * 16 + row]);
        for (uint32_t d = 0; d < kD; d++) { float L = 0.0f, A = 0.0f; for (uint32_t s = 0; s < nSplits; s++) { const uint64_t r = ((uint64_t)kvh * nSplits + s) * 16 + row; const float mm = pm[r]; const float w = (mm == kNegInf) ? 0.0f : std::exp(mm - Mx); L += pl[r] * w; A += pacc[r * kD + d] * w; }
            const uint64_t o = (uint64_t)t * kQD + h * kD + d; out[o] = (A / L) * sigmoidf_(gate[o]); }
    }
}

// The reference's own CPU check, lifted out of its Metal host program (tools/probe_flash.cpp:29-34): per (token, head),
// fp64 dot products of the fp16 prescaled Q row with keys [firstPos, posBase+t] of KV head h/6, max-subtracted softmax,
// weighted V sum, times sigmoid(gate). Rows are t in [0,M) stepping tStep, heads stepping hStep (the probe uses 3, 5).
// Works on fp16 or int8 (dequantised codes*scale + mean) caches. out is double [M][6144]; untouched entries stay as given.
void kor_formula_f64(const uint16_t* q16, const void* kc, const void* vc, const float* gate, double* out, uint32_t posBase, uint32_t M, uint32_t firstPos, uint32_t tStep, uint32_t hStep,
                     const uint16_t* ksc, const uint16_t* vsc, const uint16_t* kmn, int q8, uint32_t threads) {
    const KvView kv(kc, vc, ksc, vsc, kmn, q8); const uint32_t nT = (M + tStep - 1) / tStep, nHh = (kH + hStep - 1) / hStep;
    parallel_for(nT * nHh, threads, [&](uint32_t item) {
        const uint32_t t = (item / nHh) * tStep, h = (item % nHh) * hStep, kvh = h / 6, pos = posBase + t; std::vector<double> s(pos + 1 - firstPos); double m = -1e30;
        for (uint32_t j = firstPos; j <= pos; j++) { double a = 0; const double ks = kv.kS(j, kvh), km = kv.kM(j, kvh); for (uint32_t d = 0; d < kD; d++) a += (double)h2f(q16[(uint64_t)t * kQD + h * kD + d]) * ((double)kv.kraw(j, kvh, d) * (kv.kg ? (double)kv.kSg(j, kvh, d) : ks) + km); s[j - firstPos] = a; m = std::max(m, a); }
        double z = 0; for (auto& v : s) { v = std::exp(v - m); z += v; }
        for (uint32_t d = 0; d < kD; d++) { double a = 0; for (uint32_t j = firstPos; j <= pos; j++) a += s[j - firstPos] * ((double)kv.vraw(j, kvh, d) * (double)kv.vS(j, kvh)); a /= z; a *= 1.0 / (1.0 + std::exp(-(double)gate[(uint64_t)t * kQD + h * kD + d])); out[(uint64_t)t * kQD + h * kD + d] = a; }
    });
}

// fp32 evaluation of the same formula (the tolerance reference): q is the fp32 post-prep query [M][6144] (NOT rounded
// to fp16), scale 1/16, softmax and the V sum in fp32, all rows and heads.
void kor_formula_f32(const float* q, const void* kc, const void* vc, const float* gate, float* out, uint32_t posBase, uint32_t M, uint32_t firstPos,
                     const uint16_t* ksc, const uint16_t* vsc, const uint16_t* kmn, int q8, uint32_t threads) {
    const KvView kv(kc, vc, ksc, vsc, kmn, q8);
    parallel_for(M * kH, threads, [&](uint32_t item) {
        const uint32_t t = item / kH, h = item % kH, kvh = h / 6, pos = posBase + t; std::vector<float> s(pos + 1 - firstPos); float m = kNegInf;
        for (uint32_t j = firstPos; j <= pos; j++) { float a = 0; const float ks = kv.kS(j, kvh), km = kv.kM(j, kvh); for (uint32_t d = 0; d < kD; d++) a += (q[(uint64_t)t * kQD + h * kD + d] * 0.0625f) * (kv.kraw(j, kvh, d) * (kv.kg ? kv.kSg(j, kvh, d) : ks) + km); s[j - firstPos] = a; m = std::max(m, a); }
        float z = 0; for (auto& v : s) { v = std::exp(v - m); z += v; }
        float acc[kD] = {}; for (uint32_t j = firstPos; j <= pos; j++) { const float p = s[j - firstPos], vsj = kv.vS(j, kvh); for (uint32_t d = 0; d < kD; d++) acc[d] += p * (kv.vraw(j, kvh, d) * vsj); }
        for (uint32_t d = 0; d < kD; d++) out[(uint64_t)t * kQD + h * kD + d] = (acc[d] / z) * sigmoidf_(gate[(uint64_t)t * kQD + h * kD + d]);
    });
}

// CPU baseline for the decode benchmark: one decode step of one layer for a batch of independent sequences, the
// reference's streaming-softmax decode (k_attn_decode) per (sequence, head), spread over `threads` host threads.
// kc/vc[b] point at the layer plane of sequence b; pos[b] is the query position. q/gate/out are [B][6144].
void kor_decode_batch(const float* q, const float* gate, const uint16_t* const* kc, const uint16_t* const* vc, float* out, const uint32_t* pos, uint32_t B, uint32_t threads) {
    parallel_for(B * kH, threads, [&](uint32_t item) {
        const uint32_t b = item / kH, h = item % kH, kvh = h / kG; const uint16_t* K = kc[b]; const uint16_t* V = vc[b]; const float* qh = q + (uint64_t)b * kQD + h * kD;
        float m = kNegInf, l = 0.0f; float acc[kD] = {};
        for (uint32_t j = 0; j <= pos[b]; j++) {
            float pr[kD]; for (uint32_t d = 0; d < kD; d++) pr[d] = qh[d] * h2f(K[(uint64_t)j * kKVD + kvh * kD + d]);
            const float s = tg_sum256(pr) * 0.0625f; const float mn = std::max(m, s), a = std::exp(m - mn), e = std::exp(s - mn);
            l = l * a + e; for (uint32_t d = 0; d < kD; d++) acc[d] = acc[d] * a + e * h2f(V[(uint64_t)j * kKVD + kvh * kD + d]); m = mn;
        }
        for (uint32_t d = 0; d < kD; d++) out[(uint64_t)b * kQD + h * kD + d] = (acc[d] / l) * sigmoidf_(gate[(uint64_t)b * kQD + h * kD + d]);
    });
}

uint32_t kor_hw_threads() { const uint32_t n = std::thread::hardware_concurrency(); return n ? n : 1; }

// k_rms_fwht mode 3 + fwht1024 (shaders/ops.metal:23-50, shaders/common.h:22-42): per 1024-block y = H (sign (.) x) / 32 in natural order.
// A butterfly stage gives the lower index a + b and the upper a - b whoever computes it, so taking the stages bit 0 .. bit 9 in order
// reproduces the shader's fp32 result bit for bit (registers: bits 0-1, simd shuffles: 2-6, threadgroup transpose: 7-9).
void kor_out_fwht(const float* x, const float* sign, float* out, uint32_t rows, uint32_t width) {
    std::vector<float> v(1024);
    for (uint32_t r = 0; r < rows; r++)
        for (uint32_t blk = 0; blk < width / 1024; blk++) {
            const float* src = x + (size_t)r * width + blk * 1024; const float* sg = sign + blk * 1024;
            for (int i = 0; i < 1024; i++) v[i] = src[i] * sg[i];
            for (int bit = 0; bit < 10; bit++) {
                const int h = 1 << bit;
                for (int i = 0; i < 1024; i++) if (!(i & h)) { const float a = v[i], b = v[i | h]; v[i] = a + b; v[i | h] = a - b; }
            }
            float* dst = out + (size_t)r * width + blk * 1024;
            for (int i = 0; i < 1024; i++) dst[i] = v[i] * 0.03125f;
        }
}

// ---- the block drafter's attention (shaders/draft.metal:203-281; geometry src/draft.h:8-11): 32 query heads, 8 KV heads, head_dim 128 ----
void kor_draft_inv_freq(float* out64) { for (int i = 0; i < 64; i++) out64[i] = std::pow(kTheta, -(float)i / 64.0f); }   // shaders/draft.metal:226

// k_draft_qk (shaders/draft.metal:203-233) and, with qin == nullptr, k_draft_ctx_kv (:264-281): per-head RMSNorm(128) * weight, RoPE on the
// pairs (i, i+64) with theta = pos * inv_freq[i], Q rows to qout (fp32), K rows (fp16) and V rows (fp16 copy) to ring row pos % ring.
void kor_draft_qk(const float* qin, const float* kin, const float* vin, const float* qnorm, const float* knorm, const float* inv_freq,
                  float* qout, uint16_t* kring, uint16_t* vring, uint32_t pos0, uint32_t T, uint32_t ring) {
    const uint32_t H = 32, HKV = 8, D = 128;
    for (uint32_t t = 0; t < T; t++) for (uint32_t h = qin ? 0 : H; h < H + 2 * HKV; h++) {
        const uint32_t pos = pos0 + t; const uint64_t row = (uint64_t)(pos % ring) * (HKV * D);
        if (h >= H + HKV) { const uint32_t vh = h - H - HKV; for (uint32_t d = 0; d < D; d++) vring[row + vh * D + d] = f2h(vin[(uint64_t)t * (HKV * D) + vh * D + d]); continue; }
        const bool isK = h >= H; const uint32_t hh = isK ? h - H : h;
        const float* src = isK ? kin + (uint64_t)t * (HKV * D) + hh * D : qin + (uint64_t)t * (H * D) + hh * D; const float* w = isK ? knorm : qnorm;
        float tot = 0.0f; for (uint32_t sg = 0; sg < 4; sg++) { float sq[32]; for (int i = 0; i < 32; i++) sq[i] = src[32 * sg + i] * src[32 * sg + i]; tot += simd_sum32(sq); }   // part[0] + part[1] + part[2] + part[3]
        const float r = 1.0f / std::sqrt(tot / 128.0f + 1e-6f);
        float xs[128], o[128]; for (uint32_t d = 0; d < D; d++) o[d] = xs[d] = src[d] * r * w[d];
        for (uint32_t i = 0; i < 64; i++) { const float theta = (float)pos * inv_freq[i], c = std::cos(theta), s = std::sin(theta), a = xs[i], b = xs[i + 64]; o[i] = a * c - b * s; o[i + 64] = a * s + b * c; }
        if (isK) for (uint32_t d = 0; d < D; d++) kring[row + hh * D + d] = f2h(o[d]);
        else for (uint32_t d = 0; d < D; d++) qout[(uint64_t)t * (H * D) + hh * D + d] = o[d];
    }
}

// k_draft_attn (shaders/draft.metal:235-262): row t at position pos0 + t scans the keys [max(0, pos + 1 - win), pos0 + T - 1] in position order
// with an online softmax in fp32; the score is the sum over the four 32-lane partial dot products, times 1/sqrt(128).
void kor_draft_attn(const float* q, const uint16_t* kring, const uint16_t* vring, float* out, uint32_t pos0, uint32_t T, uint32_t win, uint32_t ring, uint32_t threads) {
    const uint32_t H = 32, HKV = 8, D = 128; const float scale = 1.0f / std::sqrt(128.0f);
    parallel_for(H * T, threads, [&](uint32_t item) {
        const uint32_t h = item % H, t = item / H, kvh = h / (H / HKV), pos = pos0 + t, lo = pos + 1 > win ? pos + 1 - win : 0, hi = pos0 + T - 1;
        const float* qv = q + (uint64_t)t * (H * D) + h * D;
        float m = kNegInf, l = 0.0f, acc[128] = {};
        for (uint32_t kp = lo; kp <= hi; kp++) {
            const uint16_t* krow = kring + (uint64_t)(kp % ring) * (HKV * D) + kvh * D; const uint16_t* vrow = vring + (uint64_t)(kp % ring) * (HKV * D) + kvh * D;
            float tot = 0.0f; for (uint32_t sg = 0; sg < 4; sg++) { float pr[32]; for (int i = 0; i < 32; i++) pr[i] = qv[32 * sg + i] * h2f(krow[32 * sg + i]); tot += simd_sum32(pr); }
            const float sc = tot * scale, mn = std::max(m, sc), a = std::exp(m - mn), e = std::exp(sc - mn);
            l = l * a + e; for (uint32_t d = 0; d < D; d++) acc[d] = acc[d] * a + e * h2f(vrow[d]);
            m = mn;
        }
        for (uint32_t d = 0; d < D; d++) out[(uint64_t)t * (H * D) + h * D + d] = acc[d] / l;
    });
}

}  // extern "C"
