"""B200-native gated-GQA attention path of the kata engine: CUDA kernels behind a C ABI (``include/kata_attn.h``),
a C++ mirror of the engine's per-layer attention calls, and this thin ctypes loader used by tests and the benchmark."""
