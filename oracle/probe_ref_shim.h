// Host shim around the lines of the reference's own CPU check (tools/probe_flash.cpp) that oracle/Makefile extracts BY
// LINE RANGE from the reference tree into oracle/_ref/probe_ref.cpp (generated, never committed; no reference source is
// copied into this repository). TEST INFRASTRUCTURE ONLY.
//
// The reference program is a Metal host program; the extracted lines are plain C++ once three things exist:
//   - the five buffers kc, vc, q, gate, out with a contents() method (MTL::Buffer there, host memory here),
//   - a callable run(posBase, M, reps) that makes "the kernel under test" fill `out` (a Metal dispatch there; here a
//     callback, so that the reference's own comparison loop judges whatever implementation the test passes in),
//   - argc / argv (line 13 picks the kernel name from them).
// The extracted lines are: 13 (maxCtx, kernel name), 16-19 (the input recipe: mt19937(5), N(0,1) K/V, then Q x 1/16 and
// the gate, in the reference's draw order), 26-34 (NaN poison beyond the valid keys, the run, and the fp64 check of every
// 3rd token x every 5th head). Nothing in them is edited.
//
// To read the fp64 reference values themselves (the loop only keeps the worst difference) std::fabs is routed through a
// recorder while those lines compile: each checked element calls it three times, the first with (g - a), the value of the
// kernel under test minus the fp64 reference.
#pragma once
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <vector>

namespace probe_shim {
struct HostBuf {
    std::vector<unsigned char> mem;
    void* contents() { return mem.data(); }
};
inline HostBuf g_bufs[5];                     // kc, vc, q, gate, out
inline std::vector<double> g_fabs_args;       // every argument std::fabs saw inside the reference lines, in call order
typedef void (*kernel_fn)(const void* q, const void* kc, const void* vc, const float* gate, float* out, uint32_t pos_base, uint32_t M, void* user);
}  // namespace probe_shim

namespace std {
inline double probe_tap_fabs(double x) { probe_shim::g_fabs_args.push_back(x); return x < 0 ? -x : x; }
}  // namespace std

// Everything the extracted lines name that is not plain C++.
#define PROBE_SHIM_BEGIN                                                                                                   \
    using probe_shim::HostBuf;                                                                                             \
    int argc = 1; char** argv = nullptr; (void)argv;                                                                       \
    HostBuf *kc = &probe_shim::g_bufs[0], *vc = &probe_shim::g_bufs[1], *q = &probe_shim::g_bufs[2], *gate = &probe_shim::g_bufs[3], *out = &probe_shim::g_bufs[4];

// After line 13 has defined maxCtx: the allocations of lines 14-15 (gpu.alloc there), same sizes, zero-filled.
#define PROBE_SHIM_ALLOC                                                                                                   \
    kc->mem.assign((size_t)maxCtx * 1024 * 2, 0); vc->mem.assign((size_t)maxCtx * 1024 * 2, 0);                            \
    q->mem.assign((size_t)1024 * 6144 * 2, 0); gate->mem.assign((size_t)1024 * 6144 * 4, 0); out->mem.assign((size_t)1024 * 6144 * 4, 0); (void)kname;

// The dispatch of lines 20-24, replaced by the callback.
#define PROBE_SHIM_RUN                                                                                                     \
    auto run = [&](uint32_t posBase, uint32_t M, int) {                                                                    \
        if (kernel_under_test) kernel_under_test(q->contents(), kc->contents(), vc->contents(), (const float*)gate->contents(), (float*)out->contents(), posBase, M, user); \
        return 0.0; };
