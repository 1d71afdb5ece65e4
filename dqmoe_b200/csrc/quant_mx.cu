// MXFP8 quantisers: e4m3 values with one UE8M0 (power-of-two) scale per 32 consecutive elements of a row, the
// operand format of the block-scaled tensor-core instruction (gemm_mx_sm100.cu).
//   scale  s = 2^ceil(log2(max(amax, 1e-4) / 448))   (smallest power of two that brings the group inside +-448)
//   bytes  q = e4m3_rne(x / s), stored scale byte = log2(s) + 127
// The division amax / 448 is IEEE fp32; x / s is exact (power of two). Same clamp of amax as the reference's
// torch quantisers (test/util.py:21); the format itself has no counterpart in the reference, which reserves
// mode bits for block-scaled formats without implementing them (csrc/quantization.h:30-38).
#include "common.cuh"

namespace dq {
namespace quant_mx {

constexpr int kThreads = 256;

__device__ __forceinline__ uint32_t mx_scale_byte(float amax, float* inv) {
    const float s = __fdiv_rn(fmaxf(amax, 1e-4f), 448.0f);
    const uint32_t bits = __float_as_uint(s);
    const uint32_t e = (bits >> 23) + ((bits & 0x7fffffu) != 0u ? 1u : 0u);
    *inv = __uint_as_float((254u - e) << 23);  // 2^(127 - e) = 1 / s
    return e;
}

// One warp per row (grid-stride over rows), each lane 8 consecutive bf16 (one 16-byte load) per step: the four
// lanes that share a 32-element group exchange their maxima by shuffles. src_row(r) maps an output row to its
// input row (identity, or the expert-sort gather).
template <bool kGather>
__global__ void __launch_bounds__(kThreads) quant_rows_kernel(const uint8_t* __restrict__ x, int64_t rows, int cols,
                                                              const int* __restrict__ dest_to_src, int k,
                                                              uint8_t* __restrict__ q, uint8_t* __restrict__ sf) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = int64_t(gridDim.x) * (kThreads / 32);
    const int vecs = cols / 8;     // 16-byte vectors per row
    const int groups = cols / 32;  // scale groups per row
    for (int64_t r = int64_t(blockIdx.x) * (kThreads / 32) + (threadIdx.x >> 5); r < rows; r += warps) {
        int64_t src = r;
        if constexpr (kGather) {
            const int slot = dest_to_src[r];
            if (slot < 0) continue;  // a dropped row
            src = slot / k;
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
                if ((lane & 3) == 0) sf[size_t(r) * groups + (v >> 2)] = uint8_t(e);
            }
        }
    }
}

static int launch_rows(const void* x, int64_t rows, int cols, const int* dest_to_src, int k, void* q, uint8_t* sf,
                       cudaStream_t stream) {
    DQ_CHECK(rows >= 0 && cols > 0);
    if (rows == 0) return DQMOE_OK;
    DQ_CHECK(x != nullptr && q != nullptr && sf != nullptr);
    DQ_CHECK_FMT(cols % 32 == 0, "cols=%d: MXFP8 rows are made of 32-element groups", cols);
    DQ_CHECK(is_aligned(x, 16) && is_aligned(q, 8));
    const int64_t want = (rows + kThreads / 32 - 1) / (kThreads / 32);
    const int64_t cap = int64_t(sm_count()) * 8;
    const int grid = int(want < cap ? want : cap);
    if (dest_to_src != nullptr)
        quant_rows_kernel<true><<<grid, kThreads, 0, stream>>>(static_cast<const uint8_t*>(x), rows, cols, dest_to_src, k,
                                                                static_cast<uint8_t*>(q), sf);
    else
        quant_rows_kernel<false><<<grid, kThreads, 0, stream>>>(static_cast<const uint8_t*>(x), rows, cols, nullptr, 1,
                                                                 static_cast<uint8_t*>(q), sf);
    DQ_LAUNCH_CHECK();
    return DQMOE_OK;
}

}  // namespace quant_mx
}  // namespace dq

extern "C" {

int dqmoe_quant_mxfp8(const void* x_bf16, int64_t rows, int cols, void* q, uint8_t* scale, dqmoe_stream_t stream) {
    return dq::quant_mx::launch_rows(x_bf16, rows, cols, nullptr, 1, q, scale, static_cast<cudaStream_t>(stream));
}

int dqmoe_permute_quant_mxfp8(const void* x_bf16, int H, int k, const int32_t* dest_to_src, int n, void* q,
                              uint8_t* scale, dqmoe_stream_t stream) {
    DQ_CHECK(k > 0 && n >= 0);
    if (n == 0) return DQMOE_OK;
    DQ_CHECK(dest_to_src != nullptr);
    return dq::quant_mx::launch_rows(x_bf16, n, H, dest_to_src, k, q, scale, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
