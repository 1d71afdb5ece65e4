// Dynamic FP8 E4M3 quantisers over bf16 data, bit-exact to the reference's torch
// expressions (test/util.py:18-68): sf = max(amax, 1e-4) / 448 and
// q = e4m3_rne(x * (1 / sf)), both divisions IEEE round-to-nearest. (This file
// must not be compiled with fast-math; the reference's own CUDA quantisers are,
// csrc/moe_kernels.h:136-398 with setup.py:37, and so differ from torch.)
//   rowwise       one scale per row           per_token_cast_to_fp8 / per_channel_cast_to_fp8
//   128x128       one scale per weight block  per_block_cast_to_fp8
//   tensor        one scale per tensor/expert (the reference has it for the intermediate only)
//   requant       second pass for the intermediate when stage 1 collected the amax
#include <mutex>

#include "common.cuh"

namespace dq {
namespace quant {

constexpr int kThreads = 256;

__device__ __forceinline__ void unpack8(const Vec16& raw, float (&v)[8]) {
    v[0] = bf16_lo(raw.x); v[1] = bf16_hi(raw.x); v[2] = bf16_lo(raw.y); v[3] = bf16_hi(raw.y);
    v[4] = bf16_lo(raw.z); v[5] = bf16_hi(raw.z); v[6] = bf16_lo(raw.w); v[7] = bf16_hi(raw.w);
}
__device__ __forceinline__ float amax8(const float (&v)[8], float m) {
#pragma unroll
    for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(v[i]));
    return m;
}
__device__ __forceinline__ uint2 quant8(const float (&v)[8], float inv) {
    uint2 o;
    o.x = f2e4m3x4(v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv);
    o.y = f2e4m3x4(v[4] * inv, v[5] * inv, v[6] * inv, v[7] * inv);
    return o;
}

__device__ __forceinline__ float block_max(float v, float* s_red) {
    v = warp_max(v);
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = v;
    __syncthreads();
    float m = 0.0f;
#pragma unroll
    for (int w = 0; w < kThreads / 32; ++w) m = fmaxf(m, s_red[w]);
    __syncthreads();
    return m;
}

// One block per row (grid-stride): amax pass, then quantise pass (second read hits L1/L2).
__global__ void __launch_bounds__(kThreads) rowwise_kernel(const uint8_t* __restrict__ x, int64_t rows, int cols,
                                                           uint8_t* __restrict__ q, float* __restrict__ scale) {
    __shared__ float s_red[kThreads / 32];
    const int vecs = cols / 8;
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const uint8_t* xr = x + size_t(r) * cols * 2;
        float m = 0.0f;
        for (int i = threadIdx.x; i < vecs; i += kThreads) {
            float v[8];
            unpack8(ld_nc16(xr + size_t(i) * 16), v);
            m = amax8(v, m);
        }
        const float amax = block_max(m, s_red);
        const float sf = scale_from_amax(amax);
        const float inv = inv_scale(sf);
        if (threadIdx.x == 0) scale[r] = sf;
        uint8_t* qr = q + size_t(r) * cols;
        for (int i = threadIdx.x; i < vecs; i += kThreads) {
            float v[8];
            unpack8(ld_nc16(xr + size_t(i) * 16), v);
            *reinterpret_cast<uint2*>(qr + size_t(i) * 8) = quant8(v, inv);
        }
    }
}

// Second pass over the bf16 intermediate when stage 1 already produced the amax: one warp per row
// (grid-stride), four 16-byte vectors per lane in flight, the scale arithmetic once per row.
__global__ void __launch_bounds__(kThreads) requant_rows_kernel(const uint8_t* __restrict__ x, int64_t rows, int cols,
                                                                uint8_t* __restrict__ q, float* __restrict__ scale,
                                                                const float* __restrict__ amax_in, int amax_per_row,
                                                                const int* __restrict__ rows_dev) {
    if (rows_dev != nullptr) rows = rows < *rows_dev ? rows : *rows_dev;  // row count known only on the device
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t(blockIdx.x) * kThreads + threadIdx.x) >> 5;
    const int64_t nwarps = int64_t(gridDim.x) * (kThreads / 32);
    const int vecs = cols / 8;
    for (int64_t r = warp; r < rows; r += nwarps) {
        const float sf = scale_from_amax(amax_in[amax_per_row ? r : 0]);
        const float inv = inv_scale(sf);
        if (lane == 0 && (amax_per_row || r == 0)) scale[amax_per_row ? r : 0] = sf;
        const uint8_t* xr = x + size_t(r) * cols * 2;
        uint8_t* qr = q + size_t(r) * cols;
        for (int i0 = lane; i0 < vecs; i0 += 128) {
            Vec16 raw[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (i0 + 32 * j < vecs) raw[j] = ld_nc16(xr + size_t(i0 + 32 * j) * 16);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (i0 + 32 * j < vecs) {
                    float v[8];
                    unpack8(raw[j], v);
                    *reinterpret_cast<uint2*>(qr + size_t(i0 + 32 * j) * 8) = quant8(v, inv);
                }
            }
        }
    }
}

// One block per 128x128 weight block: 256 threads = 16 column-vectors x 16 row lanes.
__global__ void __launch_bounds__(kThreads) block128_kernel(const uint8_t* __restrict__ w, int e, int rows, int cols,
                                                            uint8_t* __restrict__ q, float* __restrict__ scale) {
    __shared__ float s_red[kThreads / 32];
    const int bc = (cols + 127) / 128, br = (rows + 127) / 128;
    const int64_t blocks = int64_t(e) * br * bc;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    for (int64_t b = blockIdx.x; b < blocks; b += gridDim.x) {
        const int ei = int(b / (int64_t(br) * bc));
        const int rb = int((b / bc) % br), cb = int(b % bc);
        const int c = cb * 128 + tx * 8;
        const uint8_t* base = w + size_t(ei) * rows * cols * 2;
        float m = 0.0f;
        if (c < cols) {
            for (int rr = ty; rr < 128; rr += 16) {
                const int r = rb * 128 + rr;
                if (r < rows) {
                    float v[8];
                    unpack8(ld_nc16(base + (size_t(r) * cols + c) * 2), v);
                    m = amax8(v, m);
                }
            }
        }
        const float amax = block_max(m, s_red);
        const float sf = scale_from_amax(amax);
        const float inv = inv_scale(sf);
        if (threadIdx.x == 0) scale[b] = sf;
        if (c < cols) {
            uint8_t* qbase = q + size_t(ei) * rows * cols;
            for (int rr = ty; rr < 128; rr += 16) {
                const int r = rb * 128 + rr;
                if (r < rows) {
                    float v[8];
                    unpack8(ld_nc16(base + (size_t(r) * cols + c) * 2), v);
                    *reinterpret_cast<uint2*>(qbase + size_t(r) * cols + c) = quant8(v, inv);
                }
            }
        }
    }
}

// per-tensor pass 1: amax of each of e slices into amax[e] (zeroed before)
__global__ void __launch_bounds__(kThreads) tensor_amax_kernel(const uint8_t* __restrict__ x, int64_t vecs_per,
                                                               float* __restrict__ amax) {
    __shared__ float s_red[kThreads / 32];
    const int ei = blockIdx.y;
    const uint8_t* xe = x + size_t(ei) * vecs_per * 16;
    float m = 0.0f;
    for (int64_t i = int64_t(blockIdx.x) * kThreads + threadIdx.x; i < vecs_per; i += int64_t(gridDim.x) * kThreads) {
        float v[8];
        unpack8(ld_nc16(xe + size_t(i) * 16), v);
        m = amax8(v, m);
    }
    m = block_max(m, s_red);
    if (threadIdx.x == 0) atomic_max_nonneg(amax + ei, m);
}
// per-tensor pass 2
__global__ void __launch_bounds__(kThreads) tensor_quant_kernel(const uint8_t* __restrict__ x, int64_t vecs_per,
                                                                const float* __restrict__ amax,
                                                                uint8_t* __restrict__ q, float* __restrict__ scale) {
    const int ei = blockIdx.y;
    const float sf = scale_from_amax(amax[ei]);
    const float inv = inv_scale(sf);
    if (blockIdx.x == 0 && threadIdx.x == 0) scale[ei] = sf;
    const uint8_t* xe = x + size_t(ei) * vecs_per * 16;
    uint8_t* qe = q + size_t(ei) * vecs_per * 8;
    for (int64_t i = int64_t(blockIdx.x) * kThreads + threadIdx.x; i < vecs_per; i += int64_t(gridDim.x) * kThreads) {
        float v[8];
        unpack8(ld_nc16(xe + size_t(i) * 16), v);
        *reinterpret_cast<uint2*>(qe + size_t(i) * 8) = quant8(v, inv);
    }
}

// Scratch of dqmoe_quant_fp8_tensor_static: lives in the library image of every GPU that
// loads it (4 KiB per device) so that the call needs no caller- or library-made allocation.
constexpr int kStaticMaxSlices = 1024;
static __device__ __align__(256) float g_static_amax[kStaticMaxSlices];

// Device address of g_static_amax on the current device. In host code the array's name is
// only a handle for the runtime, not an address a kernel may use, so the address is looked
// up once per device (with that device current) and cached.
static int static_amax_address(float** out) {
    constexpr int kMaxDevices = 64;
    static float* cached[kMaxDevices] = {nullptr};
    static std::mutex mu;  // two host threads may make their first call on a device at once
    int dev = 0;
    DQ_CUDA(cudaGetDevice(&dev));
    DQ_CHECK(dev >= 0 && dev < kMaxDevices);
    std::lock_guard<std::mutex> lk(mu);
    if (cached[dev] == nullptr) {
        float* p = nullptr;
        DQ_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_static_amax));
        DQ_CHECK(p != nullptr);
        cached[dev] = p;
    }
    *out = cached[dev];
    return DQMOE_OK;
}

static int grid_cap(int64_t want, int per_sm) {
    const int64_t cap = int64_t(sm_count()) * per_sm;
    return int(want < cap ? (want > 0 ? want : 1) : cap);
}

}  // namespace quant
}  // namespace dq

using namespace dq;

extern "C" {

int dqmoe_quant_fp8_rowwise(const void* x_bf16, int64_t rows, int cols, void* q, float* scale,
                            dqmoe_stream_t stream) {
    DQ_CHECK(rows >= 0 && cols > 0);
    if (rows == 0) return DQMOE_OK;
    DQ_CHECK(x_bf16 != nullptr && q != nullptr && scale != nullptr);
    DQ_CHECK_FMT(cols % 8 == 0, "cols=%d must be a multiple of 8", cols);
    DQ_CHECK(is_aligned(x_bf16, 16) && is_aligned(q, 8));
    quant::rowwise_kernel<<<quant::grid_cap(rows, 16), quant::kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(x_bf16), rows, cols, static_cast<uint8_t*>(q), scale);
    DQ_LAUNCH_CHECK();
    return DQMOE_OK;
}

int dqmoe_requant_from_amax_dev(const void* act_bf16, int64_t n_max, int I, const float* amax, int per_row, void* q,
                                float* scale, const int32_t* n_rows_device, dqmoe_stream_t stream) {
    DQ_CHECK(n_max >= 0 && I > 0);
    if (n_max == 0) return DQMOE_OK;
    DQ_CHECK(act_bf16 != nullptr && q != nullptr && scale != nullptr && amax != nullptr);
    DQ_CHECK_FMT(I % 8 == 0, "I=%d must be a multiple of 8", I);
    DQ_CHECK(is_aligned(act_bf16, 16) && is_aligned(q, 8));
    quant::requant_rows_kernel<<<quant::grid_cap((n_max + 7) / 8, 8), quant::kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(act_bf16), n_max, I, static_cast<uint8_t*>(q), scale, amax, per_row ? 1 : 0,
        n_rows_device);
    DQ_LAUNCH_CHECK();
    return DQMOE_OK;
}

int dqmoe_requant_from_amax(const void* act_bf16, int64_t n, int I, const float* amax, int per_row, void* q,
                            float* scale, dqmoe_stream_t stream) {
    return dqmoe_requant_from_amax_dev(act_bf16, n, I, amax, per_row, q, scale, nullptr, stream);
}

int dqmoe_quant_fp8_block_128x128(const void* w_bf16, int e, int rows, int cols, void* q, float* scale,
                                  dqmoe_stream_t stream) {
    DQ_CHECK(e >= 0 && rows > 0 && cols > 0);
    if (e == 0) return DQMOE_OK;
    DQ_CHECK(w_bf16 != nullptr && q != nullptr && scale != nullptr);
    DQ_CHECK_FMT(cols % 8 == 0, "cols=%d must be a multiple of 8", cols);
    DQ_CHECK(is_aligned(w_bf16, 16) && is_aligned(q, 8));
    const int64_t blocks = int64_t(e) * ((rows + 127) / 128) * ((cols + 127) / 128);
    quant::block128_kernel<<<quant::grid_cap(blocks, 16), quant::kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(w_bf16), e, rows, cols, static_cast<uint8_t*>(q), scale);
    DQ_LAUNCH_CHECK();
    return DQMOE_OK;
}

int dqmoe_quant_fp8_tensor(const void* x_bf16, int e, int64_t numel_per, void* q, float* scale, float* amax_scratch,
                           dqmoe_stream_t stream) {
    DQ_CHECK(e >= 0 && numel_per >= 0 && e <= 65535);
    if (e == 0 || numel_per == 0) return DQMOE_OK;
    DQ_CHECK(x_bf16 != nullptr && q != nullptr && scale != nullptr && amax_scratch != nullptr);
    DQ_CHECK_FMT(numel_per % 8 == 0, "numel_per=%lld must be a multiple of 8", (long long) numel_per);
    DQ_CHECK(is_aligned(x_bf16, 16) && is_aligned(q, 8));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    DQ_CUDA(cudaMemsetAsync(amax_scratch, 0, size_t(e) * sizeof(float), s));
    const int64_t vecs = numel_per / 8;
    const int gx = quant::grid_cap((vecs + quant::kThreads - 1) / quant::kThreads, e >= 8 ? 2 : 8);
    dim3 grid(gx, e);
    quant::tensor_amax_kernel<<<grid, quant::kThreads, 0, s>>>(static_cast<const uint8_t*>(x_bf16), vecs, amax_scratch);
    DQ_LAUNCH_CHECK();
    quant::tensor_quant_kernel<<<grid, quant::kThreads, 0, s>>>(static_cast<const uint8_t*>(x_bf16), vecs, amax_scratch,
                                                               static_cast<uint8_t*>(q), scale);
    DQ_LAUNCH_CHECK();
    return DQMOE_OK;
}

// Per-tensor / per-expert FP8 quantiser for callers that cannot allocate device memory and
// have no spare buffer to lend: the amax scratch is the library's own static device array.
// Same kernels and results as dqmoe_quant_fp8_tensor. Limits and rules:
//   * at most 1024 slices (e <= 1024); larger e is rejected with an error;
//   * the first call on each device looks up the array's device address (a host-side runtime
//     query, no allocation) - make that first call outside any stream capture;
//   * all calls on one device share the array: it is cleared at the start of every call, and
//     two calls whose kernels overlap on the GPU (different streams) race on it.
int dqmoe_quant_fp8_tensor_static(const void* x_bf16, int e, int64_t numel_per, void* q, float* scale,
                                  dqmoe_stream_t stream) {
    DQ_CHECK(e >= 0 && numel_per >= 0);
    DQ_CHECK_FMT(e <= quant::kStaticMaxSlices, "e=%d exceeds the %d slices the static scratch holds", e,
                 quant::kStaticMaxSlices);
    if (e == 0 || numel_per == 0) return DQMOE_OK;
    DQ_CHECK(x_bf16 != nullptr && q != nullptr && scale != nullptr);
    DQ_CHECK_FMT(numel_per % 8 == 0, "numel_per=%lld must be a multiple of 8", (long long) numel_per);
    DQ_CHECK(is_aligned(x_bf16, 16) && is_aligned(q, 8));
    float* amax = nullptr;
    const int rc = quant::static_amax_address(&amax);
    if (rc != DQMOE_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // the array keeps the previous call's maxima: the reduction must start from zero
    DQ_CUDA(cudaMemsetAsync(amax, 0, size_t(e) * sizeof(float), s));
    const int64_t vecs = numel_per / 8;
    const int gx = quant::grid_cap((vecs + quant::kThreads - 1) / quant::kThreads, e >= 8 ? 2 : 8);
    dim3 grid(gx, e);
    quant::tensor_amax_kernel<<<grid, quant::kThreads, 0, s>>>(static_cast<const uint8_t*>(x_bf16), vecs, amax);
    DQ_LAUNCH_CHECK();
    quant::tensor_quant_kernel<<<grid, quant::kThreads, 0, s>>>(static_cast<const uint8_t*>(x_bf16), vecs, amax,
                                                               static_cast<uint8_t*>(q), scale);
    DQ_LAUNCH_CHECK();
    return DQMOE_OK;
}

}  // extern "C"
