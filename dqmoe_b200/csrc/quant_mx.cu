// MXFP8 quantisers: e4m3 values with one UE8M0 (power-of-two) scale per 32 consecutive elements of a row, the
// operand format of the block-scaled tensor-core instruction (gemm_mx_sm100.cu).
//   scale  s = 2^ceil(log2(max(amax, 1e-4) / 448))   (smallest power of two that brings the group inside +-448)
//   bytes  q = e4m3_rne(x / s), stored scale byte = log2(s) + 127
// The division amax / 448 is IEEE fp32; x / s is exact (power of two). Same clamp of amax as the reference's
// torch quantisers (test/util.py:21); the format itself has no counterpart in the reference, which reserves
// mode bits for block-scaled formats without implementing them (csrc/quantization.h:30-38).
//
// Scale bytes exist in two layouts. Row-major [rows, cols/32] is what a caller sees. The grouped GEMM reads the
// "tiled" layout: one 512-byte block per 128 rows and 128 columns, row r of the block at byte
// (r % 32) * 16 + (r / 32) * 4, its four bytes in column order, blocks indexed [row block][column block].
// Weight rows form row blocks by their row index (rows / 128). Expert-sorted activation rows form them by tile:
// block = mtile_prefix[e] + (r - offsets[e]) / 128 and row within the block (r - offsets[e]) % 128, so every tile
// of a ragged expert owns whole blocks.
#include "common.cuh"

namespace dq {
namespace quant_mx {

constexpr int kThreads = 256;
constexpr int kMaxExperts = 1024;

__device__ __forceinline__ uint32_t mx_scale_byte(float amax, float* inv) {
    const float s = __fdiv_rn(fmaxf(amax, 1e-4f), 448.0f);
    const uint32_t bits = __float_as_uint(s);
    const uint32_t e = (bits >> 23) + ((bits & 0x7fffffu) != 0u ? 1u : 0u);
    *inv = __uint_as_float((254u - e) << 23);  // 2^(127 - e) = 1 / s
    return e;
}

// Where the scales of (expert-sorted) row r go in the tiled layout: byte offset of the row's first K block,
// without the K-block term. s_off / s_mt: offsets[E+1] and mtile_prefix[E+1] in shared memory, or null for rows
// that form blocks by their index.
__device__ __forceinline__ size_t tiled_row_base(int64_t r, const int* s_off, const int* s_mt, int E, int kblocks) {
    int64_t block = r >> 7;
    int rit = int(r & 127);
    if (s_off != nullptr) {
        int lo = 0, hi = E;  // expert of sorted row r: last e with s_off[e] <= r
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (s_off[mid] <= r) lo = mid; else hi = mid;
        }
        const int local = int(r) - s_off[lo];
        block = s_mt[lo] + (local >> 7);
        rit = local & 127;
    }
    return size_t(block) * kblocks * 512 + (rit & 31) * 16 + (rit >> 5) * 4;
}

// One warp per row (grid-stride over rows), each lane 8 consecutive bf16 (one 16-byte load) per step: the four
// lanes that share a 32-element group exchange their maxima by shuffles. kGather: output row r is input row
// dest_to_src[r] / k of the expert sort and its scales go to the tiled layout; otherwise rows map to themselves
// and the scales are row-major.
template <bool kGather>
__global__ void __launch_bounds__(kThreads) quant_rows_kernel(const uint8_t* __restrict__ x, int64_t rows, int cols,
                                                              const int* __restrict__ dest_to_src, int k,
                                                              const int* __restrict__ offsets,
                                                              const int* __restrict__ mtile_prefix, int E,
                                                              uint8_t* __restrict__ q, uint8_t* __restrict__ sf) {
    extern __shared__ int s_tab[];  // kGather: offsets[E+1] then mtile_prefix[E+1]
    if constexpr (kGather) {
        for (int i = threadIdx.x; i <= E; i += kThreads) {
            s_tab[i] = offsets[i];
            s_tab[E + 1 + i] = mtile_prefix[i];
        }
        __syncthreads();
    }
    const int lane = threadIdx.x & 31;
    const int64_t warps = int64_t(gridDim.x) * (kThreads / 32);
    const int vecs = cols / 8;     // 16-byte vectors per row
    const int groups = cols / 32;  // scale groups per row
    const int kblocks = cols / 128;
    for (int64_t r = int64_t(blockIdx.x) * (kThreads / 32) + (threadIdx.x >> 5); r < rows; r += warps) {
        int64_t src = r;
        size_t sf_base = size_t(r) * groups;
        if constexpr (kGather) {
            const int slot = dest_to_src[r];
            if (slot < 0) continue;  // a dropped row (they sit behind all experts' rows)
            src = slot / k;
            sf_base = tiled_row_base(r, s_tab, s_tab + E + 1, E, kblocks);
        }
        const uint8_t* xr = x + size_t(src) * cols * 2;
        for (int v0 = 0; v0 < vecs; v0 += 32) {
            const int v = v0 + lane;
            float f[8];
            float amax = 0.0f;
            if (v < vecs) {
                const Vec16 raw = ld_nc16(xr + size_t(v) * 16);
                const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    f[2 * j] = bf16_lo(w[j]);
                    f[2 * j + 1] = bf16_hi(w[j]);
                    amax = fmaxf(amax, fmaxf(fabsf(f[2 * j]), fabsf(f[2 * j + 1])));
                }
            }
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
            if (v < vecs) {
                float inv;
                const uint32_t e = mx_scale_byte(amax, &inv);
                uint2 o;
                o.x = f2e4m3x4(f[0] * inv, f[1] * inv, f[2] * inv, f[3] * inv);
                o.y = f2e4m3x4(f[4] * inv, f[5] * inv, f[6] * inv, f[7] * inv);
                *reinterpret_cast<uint2*>(q + size_t(r) * cols + size_t(v) * 8) = o;
                if ((lane & 3) == 0) {
                    const int g = v >> 2;  // group index within the row
                    if constexpr (kGather)
                        sf[sf_base + size_t(g >> 2) * 512 + (g & 3)] = uint8_t(e);
                    else
                        sf[sf_base + g] = uint8_t(e);
                }
            }
        }
    }
}

// Row-major scales [*, kblocks * 4] -> tiled. One thread per (output row, K block): a 4-byte word each way.
// dest_to_src != null: output row r takes the scales of input row dest_to_src[r] / k (negative: skipped).
__global__ void __launch_bounds__(kThreads) tile_scales_kernel(const uint32_t* __restrict__ sf_rows, int64_t rows, int kblocks,
                                                               const int* __restrict__ dest_to_src, int k,
                                                               const int* __restrict__ offsets,
                                                               const int* __restrict__ mtile_prefix, int E,
                                                               uint8_t* __restrict__ tiled) {
    extern __shared__ int s_tab[];
    const bool sorted = offsets != nullptr;
    if (sorted) {
        for (int i = threadIdx.x; i <= E; i += kThreads) {
            s_tab[i] = offsets[i];
            s_tab[E + 1 + i] = mtile_prefix[i];
        }
        __syncthreads();
    }
    const int64_t total = rows * kblocks;
    for (int64_t i = int64_t(blockIdx.x) * kThreads + threadIdx.x; i < total; i += int64_t(gridDim.x) * kThreads) {
        const int64_t r = i / kblocks;
        const int kb = int(i - r * kblocks);
        if (sorted && r >= s_tab[E]) continue;  // beyond the experts' rows (dropped rows, or an over-long row count)
        int64_t src = r;
        if (dest_to_src != nullptr) {
            const int slot = dest_to_src[r];
            if (slot < 0) continue;
            src = slot / k;
        }
        const size_t base = tiled_row_base(r, sorted ? s_tab : nullptr, sorted ? s_tab + E + 1 : nullptr, E, kblocks);
        *reinterpret_cast<uint32_t*>(tiled + base + size_t(kb) * 512) = sf_rows[size_t(src) * kblocks + kb];
    }
}

static int grid_for(int64_t work_items, int per_block) {
    const int64_t want = (work_items + per_block - 1) / per_block;
    const int64_t cap = int64_t(sm_count()) * 8;
    return int(want < 1 ? 1 : (want < cap ? want : cap));
}


// NVFP4: e2m1 values (two per byte, element 2i in the low nibble), one UE4M3 scale byte per 16 consecutive elements
// of a row, and one fp32 global scale g per group of rows_per_g rows (a whole tensor for activations, one expert's
// rows for weights): x ~ e2m1 * e4m3 * g. One thread per 16-element group:
//   scale byte  = e4m3_rne((amax / 6) / g), saturating at 448
//   nibbles     = e2m1_rne(x * (1 / (e4m3 * g))), saturating at 6; an all-zero group stores zeros
// All divisions IEEE fp32. Scale bytes row-major [rows, cols / 16].
__global__ void __launch_bounds__(kThreads) quant_nvfp4_kernel(const uint8_t* __restrict__ x, int64_t rows, int cols,
                                                               const float* __restrict__ g, int64_t rows_per_g,
                                                               uint8_t* __restrict__ q, uint8_t* __restrict__ sf) {
    const int groups = cols / 16;
    const int64_t total = rows * groups;
    for (int64_t i = blockIdx.x * int64_t(kThreads) + threadIdx.x; i < total; i += int64_t(gridDim.x) * kThreads) {
        const int64_t r = i / groups;
        const Vec16 v0 = ld_nc16(x + i * 32), v1 = ld_nc16(x + i * 32 + 16);
        const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
        float f[16];
        float amax = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            f[2 * j] = bf16_lo(w[j]);
            f[2 * j + 1] = bf16_hi(w[j]);
            amax = fmaxf(amax, fmaxf(fabsf(f[2 * j]), fabsf(f[2 * j + 1])));
        }
        float inv;
        sf[i] = uint8_t(nvfp4_scale_byte(amax, g[r / rows_per_g], &inv));
        float lo[8], hi[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            lo[j] = f[j] * inv;
            hi[j] = f[8 + j] * inv;
        }
        *reinterpret_cast<uint2*>(q + i * 8) = make_uint2(f2e2m1x8(lo), f2e2m1x8(hi));
    }
}

}  // namespace quant_mx
}  // namespace dq

using namespace dq;

extern "C" {

size_t dqmoe_mx_tiled_scale_bytes(int64_t rows, int E_sorted, int cols) {
    if (rows < 0 || cols <= 0 || cols % 128 != 0 || E_sorted < 0) return 0;
    // expert-sorted rows: every expert may add one partly filled 128-row tile
    const int64_t extra = E_sorted < rows ? E_sorted : rows;
    const int64_t blocks = (rows + 127) / 128 + (E_sorted > 0 ? extra : 0);
    return size_t(blocks) * (cols / 128) * 512;
}

int dqmoe_quant_mxfp8(const void* x_bf16, int64_t rows, int cols, void* q, uint8_t* scale, dqmoe_stream_t stream) {
    DQ_CHECK(rows >= 0 && cols > 0);
    if (rows == 0) return DQMOE_OK;
    DQ_CHECK(x_bf16 != nullptr && q != nullptr && scale != nullptr);
    DQ_CHECK_FMT(cols % 32 == 0, "cols=%d: MXFP8 rows are made of 32-element groups", cols);
    DQ_CHECK(is_aligned(x_bf16, 16) && is_aligned(q, 8));
    quant_mx::quant_rows_kernel<false><<<quant_mx::grid_for(rows, quant_mx::kThreads / 32), quant_mx::kThreads, 0,
                                        static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(x_bf16), rows, cols, nullptr, 1, nullptr, nullptr, 0, static_cast<uint8_t*>(q), scale);
    DQ_LAUNCH_CHECK();
    return DQMOE_OK;
}

int dqmoe_permute_quant_mxfp8(const void* x_bf16, int H, int k, const int32_t* dest_to_src, int n, const int32_t* offsets,
                              const int32_t* mtile_prefix, int E, void* q, uint8_t* scale_tiled, dqmoe_stream_t stream) {
    DQ_CHECK(k > 0 && n >= 0 && H > 0 && E > 0 && E <= quant_mx::kMaxExperts);
    if (n == 0) return DQMOE_OK;
    DQ_CHECK(x_bf16 != nullptr && dest_to_src != nullptr && offsets != nullptr && mtile_prefix != nullptr && q != nullptr &&
             scale_tiled != nullptr);
    DQ_CHECK_FMT(H % 128 == 0, "H=%d: the tiled scale layout needs rows of whole 128-column blocks", H);
    DQ_CHECK(is_aligned(x_bf16, 16) && is_aligned(q, 8) && is_aligned(scale_tiled, 16));
    quant_mx::quant_rows_kernel<true><<<quant_mx::grid_for(n, quant_mx::kThreads / 32), quant_mx::kThreads,
                                       size_t(2 * (E + 1)) * sizeof(int), static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(x_bf16), n, H, dest_to_src, k, offsets, mtile_prefix, E, static_cast<uint8_t*>(q),
        scale_tiled);
    DQ_LAUNCH_CHECK();
    return DQMOE_OK;
}

int dqmoe_mx_tile_scales(const uint8_t* scale_rows, int64_t rows, int cols, const int32_t* dest_to_src, int k,
                         const int32_t* offsets, const int32_t* mtile_prefix, int E, uint8_t* scale_tiled,
                         dqmoe_stream_t stream) {
    DQ_CHECK(rows >= 0 && cols > 0);
    if (rows == 0) return DQMOE_OK;
    DQ_CHECK(scale_rows != nullptr && scale_tiled != nullptr);
    DQ_CHECK_FMT(cols % 128 == 0, "cols=%d: the tiled scale layout needs rows of whole 128-column blocks", cols);
    DQ_CHECK(is_aligned(scale_rows, 4) && is_aligned(scale_tiled, 16));
    DQ_CHECK((offsets == nullptr) == (mtile_prefix == nullptr));
    DQ_CHECK(dest_to_src == nullptr || k > 0);
    if (offsets != nullptr)
        DQ_CHECK(E > 0 && E <= quant_mx::kMaxExperts);
    else
        DQ_CHECK_FMT(rows % 128 == 0, "rows=%lld: rows that form blocks by their index must fill whole 128-row blocks",
                     (long long) rows);
    const int kblocks = cols / 128;
    quant_mx::tile_scales_kernel<<<quant_mx::grid_for(rows * kblocks, quant_mx::kThreads), quant_mx::kThreads,
                                   offsets != nullptr ? size_t(2 * (E + 1)) * sizeof(int) : 0,
                                   static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const uint32_t*>(scale_rows), rows, kblocks, dest_to_src, k, offsets, mtile_prefix, E, scale_tiled);
    DQ_LAUNCH_CHECK();
    return DQMOE_OK;
}

int dqmoe_quant_nvfp4(const void* x_bf16, int64_t rows, int cols, const float* gscale, int64_t rows_per_gscale, void* q,
                      uint8_t* scale, dqmoe_stream_t stream) {
    DQ_CHECK(rows >= 0 && cols > 0 && rows_per_gscale > 0);
    if (rows == 0) return DQMOE_OK;
    DQ_CHECK(x_bf16 != nullptr && gscale != nullptr && q != nullptr && scale != nullptr);
    DQ_CHECK_FMT(cols % 16 == 0, "cols=%d: NVFP4 rows are made of 16-element groups", cols);
    DQ_CHECK(is_aligned(x_bf16, 16) && is_aligned(q, 8));
    quant_mx::quant_nvfp4_kernel<<<quant_mx::grid_for(rows * (cols / 16), quant_mx::kThreads), quant_mx::kThreads, 0,
                                   static_cast<cudaStream_t>(stream)>>>(static_cast<const uint8_t*>(x_bf16), rows, cols, gscale,
                                                                        rows_per_gscale, static_cast<uint8_t*>(q), scale);
    DQ_LAUNCH_CHECK();
    return DQMOE_OK;
}

}  // extern "C"
