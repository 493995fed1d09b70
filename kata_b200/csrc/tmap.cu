// Host-side construction of the TMA tensor maps over the KV arenas. The driver entry point is looked up at run time so
// the library does not link against libcuda.
#include <cudaTypedefs.h>

#include "kata_internal.cuh"

namespace kata {

static PFN_cuTensorMapEncodeTiled get_encode() {
    static PFN_cuTensorMapEncodeTiled encode = nullptr;
    if (!encode) {
        void* fn = nullptr; cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn) return nullptr;
        encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled>(fn);
    }
    return encode;
}

// rank-2 map over a row-major fp16 matrix [rows][cols]; box = {box_cols, box_rows}, 128-byte swizzle
bool make_matrix_tmap(CUtensorMap* out, const void* base, int64_t rows, int64_t cols, int box_cols, int box_rows) {
    PFN_cuTensorMapEncodeTiled encode = get_encode(); if (!encode) return false;
    const cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows}; const cuuint64_t gstride[1] = {(cuuint64_t)cols * 2};
    const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows}; const cuuint32_t estr[2] = {1u, 1u};
    return encode(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Rank-4 view of an arena for the decode and prefill kernels: a head row of 256 elements is cut into 128-byte column blocks and the block index is made
// a dimension of its own, placed after the row dimension: {x: one 128-byte block, r: rows, c: blocks of the head row, h: KV heads}.
// One box {block, box_rows rows, box_blocks blocks, 1 head} then brings a tile of box_rows keys of one head with a single TMA instruction
// and lands in shared memory as [block][row][128 bytes], each block swizzled as a [rows][128-byte] box of a rank-3 map would be.
bool make_tile_tmap(CUtensorMap* out, void* base, int elt, int64_t rows, int box_rows, int box_blocks) {
    PFN_cuTensorMapEncodeTiled encode = get_encode(); if (!encode) return false;
    const cuuint32_t inner = 128u / (cuuint32_t)elt, blocks = (cuuint32_t)kD / inner;
    const cuuint64_t gdim[4] = {inner, (cuuint64_t)rows, blocks, (cuuint64_t)kKvh};
    const cuuint64_t gstride[3] = {(cuuint64_t)kKVD * elt, 128u, (cuuint64_t)kD * elt};   // bytes between rows, between column blocks, between heads
    const cuuint32_t box[4] = {inner, (cuuint32_t)box_rows, (cuuint32_t)box_blocks, 1u};
    const cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
    return encode(out, elt == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, base, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace kata
