// Streaming row kernels around the grouped GEMM: expert-order gather of
// activations and their scales, the scatter back to slot order, the weighted
// combine over the k slots of a token, and the gather fused with 1x128 FP8
// quantisation. All are HBM-bound: one warp per row, 16-byte accesses, a grid
// that is a multiple of the SM count.
//
// Replaces expandInputRowsGatherKernel, expandInputScale{,Block}GatherKernel and
// finalizeScatterKernel of the reference (csrc/moe_kernels.h:487-620).
#include "common.cuh"

namespace dq {
namespace permute {

constexpr int kThreads = 256;
constexpr int kWarpsPerBlock = kThreads / 32;

static int grid_for_rows(int64_t rows) {
    const int64_t want = (rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
    const int64_t cap = int64_t(sm_count()) * 8;
    return int(want < cap ? (want > 0 ? want : 1) : cap);
}

__device__ __forceinline__ void copy_row16(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int vecs,
                                           int lane) {
    int i = lane;
    for (; i + 96 < vecs; i += 128) {
        const Vec16 a = ld_nc16(src + size_t(i) * 16);
        const Vec16 b = ld_nc16(src + size_t(i + 32) * 16);
        const Vec16 c = ld_nc16(src + size_t(i + 64) * 16);
        const Vec16 d = ld_nc16(src + size_t(i + 96) * 16);
        st16(dst + size_t(i) * 16, a);
        st16(dst + size_t(i + 32) * 16, b);
        st16(dst + size_t(i + 64) * 16, c);
        st16(dst + size_t(i + 96) * 16, d);
    }
    for (; i < vecs; i += 32) st16(dst + size_t(i) * 16, ld_nc16(src + size_t(i) * 16));
}

// dst[r] = src[map[r] / k]  (kGather)   or   dst[map[r]] = src[r]  (!kGather)
template <bool kGather>
__global__ void __launch_bounds__(kThreads) row_move_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                                            const int* __restrict__ map, int n, int k, int row_vecs,
                                                            const float* __restrict__ src_scale,
                                                            float* __restrict__ dst_scale, int scale_cols) {
    const int lane = threadIdx.x & 31;
    const int warps = gridDim.x * kWarpsPerBlock;
    for (int r = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5); r < n; r += warps) {
        const int m = map[r];
        if (m < 0) continue;
        const size_t s_row = kGather ? size_t(m / k) : size_t(r);
        const size_t d_row = kGather ? size_t(r) : size_t(m);
        copy_row16(src + s_row * row_vecs * 16, dst + d_row * row_vecs * 16, row_vecs, lane);
        if (scale_cols > 0) {
            for (int c = lane; c < scale_cols; c += 32) dst_scale[d_row * scale_cols + c] = src_scale[s_row * scale_cols + c];
        }
    }
}

// out[t, :] = sum_j w[t, j] * d[t, j, :]; one warp per (token, 256-column strip)
__global__ void __launch_bounds__(kThreads) finalize_weighted_kernel(const uint8_t* __restrict__ d,
                                                                     const float* __restrict__ w,
                                                                     uint8_t* __restrict__ out, int T, int k,
                                                                     int row_vecs) {
    const int lane = threadIdx.x & 31;
    const int strips = (row_vecs + 31) / 32;
    const int64_t items = int64_t(T) * strips;
    const int64_t warps = int64_t(gridDim.x) * kWarpsPerBlock;
    for (int64_t it = int64_t(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5); it < items; it += warps) {
        const int t = int(it / strips);
        const int v = int(it % strips) * 32 + lane;
        if (v >= row_vecs) continue;
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int j = 0; j < k; ++j) {
            const float wj = w[size_t(t) * k + j];
            if (wj == 0.0f) continue;
            const Vec16 x = ld_nc16(d + ((size_t(t) * k + j) * row_vecs + v) * 16);
            acc[0] = fmaf(wj, bf16_lo(x.x), acc[0]);
            acc[1] = fmaf(wj, bf16_hi(x.x), acc[1]);
            acc[2] = fmaf(wj, bf16_lo(x.y), acc[2]);
            acc[3] = fmaf(wj, bf16_hi(x.y), acc[3]);
            acc[4] = fmaf(wj, bf16_lo(x.z), acc[4]);
            acc[5] = fmaf(wj, bf16_hi(x.z), acc[5]);
            acc[6] = fmaf(wj, bf16_lo(x.w), acc[6]);
            acc[7] = fmaf(wj, bf16_hi(x.w), acc[7]);
        }
        Vec16 o{pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]),
                pack_bf16x2(acc[6], acc[7])};
        st16(out + (size_t(t) * row_vecs + v) * 16, o);
    }
}

// q[r, :], scale[r, :] = 1x128 FP8 quantisation of bf16 row map[r] / k (map == nullptr: row r).
// One warp per row; a lane owns 8 consecutive columns, so a 128-column group is 16 lanes.
__global__ void __launch_bounds__(kThreads) quant_1x128_kernel(const uint8_t* __restrict__ x, int64_t rows, int cols,
                                                               int k, const int* __restrict__ map,
                                                               uint8_t* __restrict__ q, float* __restrict__ scale) {
    const int lane = threadIdx.x & 31;
    const int groups = (cols + 127) / 128;
    const int64_t warps = int64_t(gridDim.x) * kWarpsPerBlock;
    for (int64_t r = int64_t(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5); r < rows; r += warps) {
        int64_t s_row = r;
        if (map != nullptr) {
            const int m = map[r];
            if (m < 0) continue;
            s_row = m / k;
        }
        const uint8_t* xr = x + size_t(s_row) * cols * 2;
        uint8_t* qr = q + size_t(r) * cols;
        for (int c0 = 0; c0 < cols; c0 += 256) {
            const int c = c0 + lane * 8;
            float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            if (c < cols) {
                const Vec16 raw = ld_nc16(xr + size_t(c) * 2);
                v[0] = bf16_lo(raw.x); v[1] = bf16_hi(raw.x); v[2] = bf16_lo(raw.y); v[3] = bf16_hi(raw.y);
                v[4] = bf16_lo(raw.z); v[5] = bf16_hi(raw.z); v[6] = bf16_lo(raw.w); v[7] = bf16_hi(raw.w);
            }
            float amax = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
            // reduce over the 16 lanes of this 128-column group
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            const float sf = scale_from_amax(amax);
            const float inv = inv_scale(sf);
            if (c < cols) {
                uint2 o;
                o.x = f2e4m3x4(v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv);
                o.y = f2e4m3x4(v[4] * inv, v[5] * inv, v[6] * inv, v[7] * inv);
                *reinterpret_cast<uint2*>(qr + c) = o;
                if ((lane & 15) == 0) scale[size_t(r) * groups + (c >> 7)] = sf;
            }
        }
    }
}

}  // namespace permute
}  // namespace dq

using namespace dq;

extern "C" {

int dqmoe_permute_rows(const void* src, size_t row_bytes, int k, const int32_t* dest_to_src, int n, void* dst,
                       const float* src_scale, int scale_cols, float* dst_scale, dqmoe_stream_t stream) {
    DQ_CHECK(n >= 0 && k > 0 && scale_cols >= 0);
    if (n == 0) return DQMOE_OK;
    DQ_CHECK(src != nullptr && dst != nullptr && dest_to_src != nullptr);
    DQ_CHECK_FMT(row_bytes % 16 == 0 && row_bytes > 0, "row_bytes=%zu must be a multiple of 16", row_bytes);
    DQ_CHECK(is_aligned(src, 16) && is_aligned(dst, 16));
    if (scale_cols > 0) DQ_CHECK(src_scale != nullptr && dst_scale != nullptr);
    permute::row_move_kernel<true><<<permute::grid_for_rows(n), permute::kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), dest_to_src, n, k, int(row_bytes / 16), src_scale,
        dst_scale, scale_cols);
    DQ_LAUNCH_CHECK();
    return DQMOE_OK;
}

int dqmoe_finalize_scatter(const void* rows, size_t row_bytes, const int32_t* dest_to_src, int n, void* d,
                           dqmoe_stream_t stream) {
    DQ_CHECK(n >= 0);
    if (n == 0) return DQMOE_OK;
    DQ_CHECK(rows != nullptr && d != nullptr && dest_to_src != nullptr);
    DQ_CHECK_FMT(row_bytes % 16 == 0 && row_bytes > 0, "row_bytes=%zu must be a multiple of 16", row_bytes);
    DQ_CHECK(is_aligned(rows, 16) && is_aligned(d, 16));
    permute::row_move_kernel<false><<<permute::grid_for_rows(n), permute::kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(rows), static_cast<uint8_t*>(d), dest_to_src, n, 1, int(row_bytes / 16), nullptr,
        nullptr, 0);
    DQ_LAUNCH_CHECK();
    return DQMOE_OK;
}

int dqmoe_finalize_weighted(const void* d_bf16, const float* weights, void* out_bf16, int T, int k, int H,
                            dqmoe_stream_t stream) {
    DQ_CHECK(T >= 0 && k > 0 && H > 0);
    if (T == 0) return DQMOE_OK;
    DQ_CHECK(d_bf16 != nullptr && weights != nullptr && out_bf16 != nullptr);
    DQ_CHECK_FMT(H % 8 == 0, "H=%d must be a multiple of 8", H);
    DQ_CHECK(is_aligned(d_bf16, 16) && is_aligned(out_bf16, 16));
    const int row_vecs = H / 8;
    const int64_t items = int64_t(T) * ((row_vecs + 31) / 32);
    permute::finalize_weighted_kernel<<<permute::grid_for_rows(items), permute::kThreads, 0,
                                        static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(d_bf16), weights, static_cast<uint8_t*>(out_bf16), T, k, row_vecs);
    DQ_LAUNCH_CHECK();
    return DQMOE_OK;
}

int dqmoe_quant_fp8_block_1x128(const void* x_bf16, int64_t rows, int cols, void* q, float* scale,
                                dqmoe_stream_t stream) {
    DQ_CHECK(rows >= 0 && cols > 0);
    if (rows == 0) return DQMOE_OK;
    DQ_CHECK(x_bf16 != nullptr && q != nullptr && scale != nullptr);
    DQ_CHECK_FMT(cols % 8 == 0, "cols=%d must be a multiple of 8", cols);
    DQ_CHECK(is_aligned(x_bf16, 16) && is_aligned(q, 8));
    permute::quant_1x128_kernel<<<permute::grid_for_rows(rows), permute::kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(x_bf16), rows, cols, 1, nullptr, static_cast<uint8_t*>(q), scale);
    DQ_LAUNCH_CHECK();
    return DQMOE_OK;
}

int dqmoe_permute_quant_block_1x128(const void* x_bf16, int H, int k, const int32_t* dest_to_src, int n, void* q,
                                    float* scale, dqmoe_stream_t stream) {
    DQ_CHECK(n >= 0 && k > 0 && H > 0);
    if (n == 0) return DQMOE_OK;
    DQ_CHECK(x_bf16 != nullptr && q != nullptr && scale != nullptr && dest_to_src != nullptr);
    DQ_CHECK_FMT(H % 8 == 0, "H=%d must be a multiple of 8", H);
    DQ_CHECK(is_aligned(x_bf16, 16) && is_aligned(q, 8));
    permute::quant_1x128_kernel<<<permute::grid_for_rows(n), permute::kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(x_bf16), n, H, k, dest_to_src, static_cast<uint8_t*>(q), scale);
    DQ_LAUNCH_CHECK();
    return DQMOE_OK;
}

}  // extern "C"
