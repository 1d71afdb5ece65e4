// Layer path for one to a few tokens (n = T*k <= 8 expanded rows): with so few rows a 128-row
// MMA tile is almost empty and there are fewer tiles than SMs, so the two expert GEMMs are done as
// weight-streaming GEMVs on the CUDA cores instead: every warp streams whole weight rows with
// 16-byte loads (8 in flight per lane), the token's activation row sits in shared memory as fp32,
// products are accumulated in fp32. No sort or gather is needed: slot i = t*k + j reads token t and
// the weights of expert m_indices[i] directly and writes d[i, :].
//   bf16 mode        fc1+SwiGLU -> act bf16 -> fc2
//   per-tensor FP8   fc1+SwiGLU -> act bf16 + amax (atomic) -> fc2 quantises act while staging it
// Same arithmetic as the tensor-core path (e4m3 products are exact in fp32, fp32 accumulation,
// the torch oracle's bf16 rounding points); summation order differs. HBM-bound: algorithmic bytes
// = weights of the experts hit. Replaces, for this size range, what the reference runs as
// moeGemm/moeGemmTensorWise + doGatedActivationKernel + perTensorDynamicFp8QuantKernel
// (csrc/moe_gemm_template.h:487-677, csrc/moe_kernels.h:136-221, 404-444).
#include "common.cuh"

namespace dq {
namespace decode {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kColsPerWarp = 2;                    // output columns per warp and pass
constexpr int kColsPerPass = kWarps * kColsPerWarp;  // 16 columns per block and pass; columns per block chosen per launch

__device__ __forceinline__ float silu_bf16(float g) { return bf_round(__fdividef(g, 1.0f + __expf(-g))); }

// 16 bytes of weights times the matching activations (fp32, staged piece-major: xs[piece * vecs + v])
template <bool kFp8>
__device__ __forceinline__ float dot16(const Vec16& w, const float4* __restrict__ xs, int vecs, int v) {
    float acc = 0.0f;
    if constexpr (kFp8) {
        const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float4 x = xs[q * vecs + v];
            const __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(words[q] & 0xffffu), __NV_E4M3);
            const __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(words[q] >> 16), __NV_E4M3);
            const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&lo));
            const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&hi));
            acc = fmaf(a.x, x.x, acc);
            acc = fmaf(a.y, x.y, acc);
            acc = fmaf(b.x, x.z, acc);
            acc = fmaf(b.y, x.w, acc);
        }
    } else {
        const float4 x0 = xs[v], x1 = xs[vecs + v];
        acc = fmaf(bf16_lo(w.x), x0.x, acc);
        acc = fmaf(bf16_hi(w.x), x0.y, acc);
        acc = fmaf(bf16_lo(w.y), x0.z, acc);
        acc = fmaf(bf16_hi(w.y), x0.w, acc);
        acc = fmaf(bf16_lo(w.z), x1.x, acc);
        acc = fmaf(bf16_hi(w.z), x1.y, acc);
        acc = fmaf(bf16_lo(w.w), x1.z, acc);
        acc = fmaf(bf16_hi(w.w), x1.w, acc);
    }
    return acc;
}

// Stage a row of K elements as fp32 into shared memory, piece-major (4 floats per piece; a 16-byte
// source vector is 4 pieces for e4m3 and 2 for bf16). kQuant: the source is bf16 and is first
// quantised to e4m3 with inv (the per-tensor re-quantisation of the intermediate).
template <bool kFp8Src, bool kQuant>
__device__ __forceinline__ void stage_row(const uint8_t* __restrict__ src, int K, float4* xs, float inv) {
    if constexpr (kFp8Src) {
        const int vecs = K / 16;
        for (int v = threadIdx.x; v < vecs; v += kThreads) {
            const Vec16 raw = ld_nc16(src + size_t(v) * 16);
            const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(words[q] & 0xffffu), __NV_E4M3);
                const __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(words[q] >> 16), __NV_E4M3);
                const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&lo));
                const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&hi));
                xs[q * vecs + v] = make_float4(a.x, a.y, b.x, b.y);
            }
        }
    } else {
        // bf16 source, 8 elements per 16 bytes
        const int src_vecs = K / 8;
        for (int v = threadIdx.x; v < src_vecs; v += kThreads) {
            const Vec16 raw = ld_nc16(src + size_t(v) * 16);
            float f[8] = {bf16_lo(raw.x), bf16_hi(raw.x), bf16_lo(raw.y), bf16_hi(raw.y),
                          bf16_lo(raw.z), bf16_hi(raw.z), bf16_lo(raw.w), bf16_hi(raw.w)};
            if constexpr (kQuant) {
                // e4m3 value of x * inv, kept as fp32 (the weights are e4m3: 16 elements per vector)
#pragma unroll
                for (int i = 0; i < 8; i += 2) {
                    const uint32_t q2 = f2e4m3x2(f[i] * inv, f[i + 1] * inv);
                    const __half2_raw h2 = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(q2), __NV_E4M3);
                    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&h2));
                    f[i] = a.x;
                    f[i + 1] = a.y;
                }
                // weight vector w = 16 elements: source vector v covers half of weight vector v/2
                const int wv = v >> 1, half = v & 1, wvecs = K / 16;
                xs[(half * 2) * wvecs + wv] = make_float4(f[0], f[1], f[2], f[3]);
                xs[(half * 2 + 1) * wvecs + wv] = make_float4(f[4], f[5], f[6], f[7]);
            } else {
                xs[v] = make_float4(f[0], f[1], f[2], f[3]);
                xs[src_vecs + v] = make_float4(f[4], f[5], f[6], f[7]);
            }
        }
    }
}

// fc1 + SwiGLU for slot row = blockIdx.y: act[row, j] = silu(w[e, j] . x) * (w[e, I+j] . x)
// (The kernels carry "GemmGrouped" and "GemmUniversal" in their names because the reference's test driver
// times the layer by summing the profiler rows whose kernel name contains one of the two,
// test/torch_test.py:97-104, 180-205, and its two smallest shapes take this path.)
template <bool kFp8>
__global__ void __launch_bounds__(kThreads) moe_GemmGrouped_GemmUniversal_gemv_fc1(const uint8_t* __restrict__ a, const uint8_t* __restrict__ w,
                                                            const int* __restrict__ ids, int k, int H, int I, int E,
                                                            const float* __restrict__ sa, const float* __restrict__ sb,
                                                            __nv_bfloat16* __restrict__ act, float* __restrict__ amax,
                                                            int cols_per_block) {
    extern __shared__ float4 s_x[];
    const int row = blockIdx.y;
    const int e = ids[row];
    if (e < 0 || e >= E) return;
    constexpr int esz = kFp8 ? 1 : 2;
    stage_row<kFp8, false>(a + size_t(row / k) * H * esz, H, s_x, 1.0f);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int vecs = H * esz / 16;
    const float scale = kFp8 ? sa[0] * sb[e] : 1.0f;
    const uint8_t* we = w + size_t(e) * 2 * I * H * esz;
    const size_t row_bytes = size_t(H) * esz;
    float amax_local = 0.0f;
    const int j_end = min(I, int(blockIdx.x + 1) * cols_per_block);
    for (int j0 = blockIdx.x * cols_per_block + warp * kColsPerWarp; j0 < j_end; j0 += kColsPerPass) {
        float g[kColsPerWarp] = {0.0f, 0.0f}, u[kColsPerWarp] = {0.0f, 0.0f};
        const int j1 = min(j0 + 1, I - 1);  // clamp (an odd I): the duplicate column is not stored
        const uint8_t* pg0 = we + size_t(j0) * row_bytes;
        const uint8_t* pu0 = we + size_t(I + j0) * row_bytes;
        const uint8_t* pg1 = we + size_t(j1) * row_bytes;
        const uint8_t* pu1 = we + size_t(I + j1) * row_bytes;
        int v = lane;
        for (; v + 32 < vecs; v += 64) {  // eight 16-byte loads in flight per lane
            const Vec16 a0 = ld_nc16(pg0 + size_t(v) * 16), b0 = ld_nc16(pu0 + size_t(v) * 16);
            const Vec16 a1 = ld_nc16(pg1 + size_t(v) * 16), b1 = ld_nc16(pu1 + size_t(v) * 16);
            const Vec16 a2 = ld_nc16(pg0 + size_t(v + 32) * 16), b2 = ld_nc16(pu0 + size_t(v + 32) * 16);
            const Vec16 a3 = ld_nc16(pg1 + size_t(v + 32) * 16), b3 = ld_nc16(pu1 + size_t(v + 32) * 16);
            g[0] += dot16<kFp8>(a0, s_x, vecs, v) + dot16<kFp8>(a2, s_x, vecs, v + 32);
            u[0] += dot16<kFp8>(b0, s_x, vecs, v) + dot16<kFp8>(b2, s_x, vecs, v + 32);
            g[1] += dot16<kFp8>(a1, s_x, vecs, v) + dot16<kFp8>(a3, s_x, vecs, v + 32);
            u[1] += dot16<kFp8>(b1, s_x, vecs, v) + dot16<kFp8>(b3, s_x, vecs, v + 32);
        }
        for (; v < vecs; v += 32) {
            g[0] += dot16<kFp8>(ld_nc16(pg0 + size_t(v) * 16), s_x, vecs, v);
            u[0] += dot16<kFp8>(ld_nc16(pu0 + size_t(v) * 16), s_x, vecs, v);
            g[1] += dot16<kFp8>(ld_nc16(pg1 + size_t(v) * 16), s_x, vecs, v);
            u[1] += dot16<kFp8>(ld_nc16(pu1 + size_t(v) * 16), s_x, vecs, v);
        }
#pragma unroll
        for (int c = 0; c < kColsPerWarp; ++c) {
            g[c] = warp_sum(g[c]);
            u[c] = warp_sum(u[c]);
        }
        if (lane < kColsPerWarp && j0 + lane < I) {
            const float gate = bf_round((lane == 0 ? g[0] : g[1]) * scale);
            const float val = bf_round((lane == 0 ? u[0] : u[1]) * scale);
            const float out = bf_round(silu_bf16(gate) * val);
            act[size_t(row) * I + j0 + lane] = __float2bfloat16_rn(out);
            amax_local = fmaxf(amax_local, fabsf(out));
        }
    }
    if (kFp8 && amax != nullptr) {
        amax_local = warp_max(amax_local);
        if (lane == 0 && amax_local > 0.0f) atomic_max_nonneg(amax, amax_local);
    }
}

// fc2 for slot row = blockIdx.y: d[row, j] = w1[e, j] . act[row]; in FP8 mode act is quantised here
template <bool kFp8>
__global__ void __launch_bounds__(kThreads) moe_GemmGrouped_GemmUniversal_gemv_fc2(const __nv_bfloat16* __restrict__ act,
                                                            const uint8_t* __restrict__ w1, const int* __restrict__ ids,
                                                            int H, int I, int E, const float* __restrict__ amax,
                                                            const float* __restrict__ sb1, __nv_bfloat16* __restrict__ d,
                                                            int cols_per_block) {
    extern __shared__ float4 s_x[];
    const int row = blockIdx.y;
    const int e = ids[row];
    if (e < 0 || e >= E) return;
    constexpr int esz = kFp8 ? 1 : 2;
    float scale = 1.0f;
    if constexpr (kFp8) {
        const float sf = scale_from_amax(amax[0]);  // the oracle's per-tensor scale of the intermediate
        stage_row<false, true>(reinterpret_cast<const uint8_t*>(act + size_t(row) * I), I, s_x, inv_scale(sf));
        scale = sf * sb1[e];
    } else {
        stage_row<false, false>(reinterpret_cast<const uint8_t*>(act + size_t(row) * I), I, s_x, 1.0f);
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int vecs = I * esz / 16;
    const uint8_t* we = w1 + size_t(e) * H * I * esz;
    const size_t row_bytes = size_t(I) * esz;
    const int j_end = min(H, int(blockIdx.x + 1) * cols_per_block);
    for (int j0 = blockIdx.x * cols_per_block + warp * kColsPerWarp; j0 < j_end; j0 += kColsPerPass) {
        float s[kColsPerWarp] = {0.0f, 0.0f};
        const int j1 = min(j0 + 1, H - 1);
        const uint8_t* p0 = we + size_t(j0) * row_bytes;
        const uint8_t* p1 = we + size_t(j1) * row_bytes;
        int v = lane;
        for (; v + 96 < vecs; v += 128) {  // eight 16-byte loads in flight per lane
            Vec16 a[4], b[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                a[q] = ld_nc16(p0 + size_t(v + 32 * q) * 16);
                b[q] = ld_nc16(p1 + size_t(v + 32 * q) * 16);
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                s[0] += dot16<kFp8>(a[q], s_x, vecs, v + 32 * q);
                s[1] += dot16<kFp8>(b[q], s_x, vecs, v + 32 * q);
            }
        }
        for (; v < vecs; v += 32) {
            s[0] += dot16<kFp8>(ld_nc16(p0 + size_t(v) * 16), s_x, vecs, v);
            s[1] += dot16<kFp8>(ld_nc16(p1 + size_t(v) * 16), s_x, vecs, v);
        }
        s[0] = warp_sum(s[0]);
        s[1] = warp_sum(s[1]);
        if (lane < kColsPerWarp && j0 + lane < H)
            d[size_t(row) * H + j0 + lane] = __float2bfloat16_rn((lane == 0 ? s[0] : s[1]) * scale);
    }
}

int forward(const void* a, const float* a_scale, const void* b, const float* b_scale, const void* b1,
            const float* b1_scale, void* d, const int* m_indices, void* act_bf16, float* amax, int T, int H, int I,
            int E, int k, bool fp8, cudaStream_t stream) {
    const int n = T * k;
    const size_t smem1 = size_t(H) * sizeof(float), smem2 = size_t(I) * sizeof(float);
    DQ_CHECK_FMT(smem1 <= 200 * 1024 && smem2 <= 200 * 1024, "H=%d or I=%d too large for the decode path", H, I);
    // columns per block: about 8 blocks per SM (measured best of 2..12), staging the activation row as rarely as that allows
    auto cols_for = [&](int N) {
        int c = ceil_div(int(int64_t(N) * n / (8 * sm_count())), kColsPerPass) * kColsPerPass;
        return c < kColsPerPass ? kColsPerPass : (c > 64 ? 64 : c);
    };
    const int c1 = cols_for(I), c2 = cols_for(H);
    dim3 g1(ceil_div(I, c1), n), g2(ceil_div(H, c2), n);
    auto* a8 = static_cast<const uint8_t*>(a);
    auto* b8 = static_cast<const uint8_t*>(b);
    auto* b18 = static_cast<const uint8_t*>(b1);
    auto* act = static_cast<__nv_bfloat16*>(act_bf16);
    auto* out = static_cast<__nv_bfloat16*>(d);
    static bool attr_dev[64][2] = {};
    int dev = 0;
    DQ_CUDA(cudaGetDevice(&dev));
    DQ_CHECK(dev >= 0 && dev < 64);
    bool* attr = attr_dev[dev];
    if (fp8) {
        if (!attr[1]) {
            DQ_CUDA(cudaFuncSetAttribute(moe_GemmGrouped_GemmUniversal_gemv_fc1<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
            DQ_CUDA(cudaFuncSetAttribute(moe_GemmGrouped_GemmUniversal_gemv_fc2<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
            attr[1] = true;
        }
        DQ_CUDA(cudaMemsetAsync(amax, 0, sizeof(float), stream));
        moe_GemmGrouped_GemmUniversal_gemv_fc1<true><<<g1, kThreads, smem1, stream>>>(a8, b8, m_indices, k, H, I, E, a_scale, b_scale, act, amax, c1);
        DQ_LAUNCH_CHECK();
        moe_GemmGrouped_GemmUniversal_gemv_fc2<true><<<g2, kThreads, smem2, stream>>>(act, b18, m_indices, H, I, E, amax, b1_scale, out, c2);
        DQ_LAUNCH_CHECK();
    } else {
        if (!attr[0]) {
            DQ_CUDA(cudaFuncSetAttribute(moe_GemmGrouped_GemmUniversal_gemv_fc1<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
            DQ_CUDA(cudaFuncSetAttribute(moe_GemmGrouped_GemmUniversal_gemv_fc2<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
            attr[0] = true;
        }
        moe_GemmGrouped_GemmUniversal_gemv_fc1<false><<<g1, kThreads, smem1, stream>>>(a8, b8, m_indices, k, H, I, E, nullptr, nullptr, act, nullptr, c1);
        DQ_LAUNCH_CHECK();
        moe_GemmGrouped_GemmUniversal_gemv_fc2<false><<<g2, kThreads, smem2, stream>>>(act, b18, m_indices, H, I, E, nullptr, nullptr, out, c2);
        DQ_LAUNCH_CHECK();
    }
    return DQMOE_OK;
}

}  // namespace decode
}  // namespace dq
