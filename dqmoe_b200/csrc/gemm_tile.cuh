// Pieces shared by the grouped-GEMM kernels (gemm_sm100.cu, gemm_mx_sm100.cu): the row-coalescing staged
// store of the epilogues and the host-side TMA tensor-map construction.
#pragma once

#include "common.cuh"

namespace dq {
namespace gemm {

// Store 32 rows x 32 bf16 columns held one row per lane (packed[16]) so that each store
// instruction writes 64 contiguous bytes of each of 8 rows instead of 16 bytes of each of 32 rows: the rows go
// through a 2 KiB per-warp shared-memory buffer (16-byte pieces XOR-swizzled against bank
// conflicts). row_ptr is this lane's destination (already at the chunk's first column) or null;
// pieces_ok = number of 8-column pieces of the chunk that lie inside the matrix. Used for rows
// that live in another GPU's memory, where 16-byte scattered stores waste NVLink packets.
__device__ __forceinline__ void store_rows_staged(uint4* stage, const uint32_t (&packed)[16], uint8_t* row_ptr,
                                                  int pieces_ok, int lane) {
    __syncwarp();  // the previous use of the buffer has been read out
#pragma unroll
    for (int pc = 0; pc < 4; ++pc)
        stage[lane * 4 + (pc ^ ((lane >> 1) & 3))] =
            make_uint4(packed[pc * 4], packed[pc * 4 + 1], packed[pc * 4 + 2], packed[pc * 4 + 3]);
    __syncwarp();
    const unsigned long long my_ptr = reinterpret_cast<unsigned long long>(row_ptr);
    const int piece = lane & 3;
#pragma unroll
    for (int it = 0; it < 4; ++it) {  // 4 lanes per 64-byte row: 8 rows per instruction
        const int r = it * 8 + (lane >> 2);
        const unsigned long long dst = __shfl_sync(0xffffffffu, my_ptr, r);
        const uint4 v = stage[r * 4 + (piece ^ ((r >> 1) & 3))];
        if (dst != 0 && piece < pieces_ok) {
            Vec16 vv{v.x, v.y, v.z, v.w};
            st16(reinterpret_cast<uint8_t*>(dst) + piece * 16, vv);
        }
    }
}

// ---------------------------------------------------------------- host side: TMA tensor maps

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// 2-D row-major matrix [rows, cols] of 1-, 2- or 4-byte elements, box = 128 bytes x box_rows rows, 128B swizzle.
static inline int make_map(CUtensorMap* map, const void* base, int esz, uint64_t rows, uint64_t cols, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return fail(DQMOE_ERR_CUDA, __FILE__, __LINE__, "cuTensorMapEncodeTiled", "driver entry point not found");
    cuuint64_t gdim[2] = {cols, rows};
    cuuint64_t gstride[1] = {cols * uint64_t(esz)};
    cuuint32_t box[2] = {static_cast<cuuint32_t>(128 / esz), static_cast<cuuint32_t>(box_rows)};
    cuuint32_t estr[2] = {1, 1};
    const CUtensorMapDataType dt = esz == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                   : esz == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    CUresult r = fn(map, dt, 2, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(DQMOE_ERR_CUDA, __FILE__, __LINE__, "cuTensorMapEncodeTiled", "CUresult %d (rows %llu cols %llu)",
                    int(r), (unsigned long long) rows, (unsigned long long) cols);
    return DQMOE_OK;
}

}  // namespace gemm
}  // namespace dq
