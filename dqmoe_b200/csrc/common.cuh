// Shared host/device helpers of the dqmoe_b200 library: error reporting for the
// C ABI, the host-mapped device status word, and small device utilities.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>
#include <string>

#include "../../include/dqmoe.h"

namespace dq {

// ---------------------------------------------------------------- host errors

// Message of the last failure on this thread (returned by dqmoe_last_error()).
std::string& last_error();

int fail(int code, const char* file, int line, const char* cond, const char* fmt = nullptr, ...);

// Argument check in the reference's CPU_CHECK form (csrc/util.h:173-195): the
// C ABI returns DQMOE_ERR_INVALID and the Python layer raises RuntimeError with
// the "[ASSERT FAILED] ..." text.
#define DQ_CHECK(cond)                                                              \
    do {                                                                            \
        if (!(cond)) return ::dq::fail(DQMOE_ERR_INVALID, __FILE__, __LINE__, #cond); \
    } while (0)
#define DQ_CHECK_FMT(cond, ...)                                                                  \
    do {                                                                                         \
        if (!(cond)) return ::dq::fail(DQMOE_ERR_INVALID, __FILE__, __LINE__, #cond, __VA_ARGS__); \
    } while (0)
// CUDA failures become error returns; the reference's CUDA_CHECK calls exit()
// (csrc/util.h:61-80).
#define DQ_CUDA(expr)                                                                   \
    do {                                                                                \
        cudaError_t e_ = (expr);                                                        \
        if (e_ != cudaSuccess)                                                          \
            return ::dq::fail(DQMOE_ERR_CUDA, __FILE__, __LINE__, #expr, "%s",          \
                              cudaGetErrorString(e_));                                  \
    } while (0)
#define DQ_LAUNCH_CHECK() DQ_CUDA(cudaGetLastError())

// Host-mapped status word of the current device (allocated once per device in
// pinned host memory; kernels write a non-zero code when a bounded wait gives up).
// Returns the device-side pointer, or nullptr with last_error() set.
int* device_status_word();
// Host view of the same word for the current device.
volatile int* host_status_word();

int sm_count();

namespace decode {
constexpr int kAmaxParts = 4096;  // floats the layer workspace holds for the per-block amax values of the decode path's fc1
}

static inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
static inline bool is_aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// ---------------------------------------------------------------- device utils

// 16-byte vector used by all streaming kernels (coalesced 128-bit accesses).
struct __align__(16) Vec16 {
    uint32_t x, y, z, w;
};

__device__ __forceinline__ Vec16 ld_nc16(const void* p) {
    Vec16 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ void st16(void* p, const Vec16& v) {
    asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// round-to-nearest-even fp32 -> bf16 bits (matches torch's .to(bfloat16))
__device__ __forceinline__ uint32_t f2bf_bits(float f) {
    return static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(f)));
}
// fp32 rounded to the nearest bf16 value (ties to even), returned as fp32. Done as a 16-bit Veltkamp
// split on the fp32 pipe (c = 65537 x; x_hi = c - (c - x), every step rounded) instead of a
// cvt.rn.bf16.f32 round trip: conversions run on the quarter-rate pipe, and the SwiGLU epilogues
// round four times per element. Equal to the cvt result for all normal inputs with |x| < 2^111
// (checked exhaustively on random and tie patterns); subnormal results may differ in the last bit.
__device__ __forceinline__ float bf_round(float f) {
    const float c = __fmul_rn(f, 65537.0f);
    return __fsub_rn(c, __fsub_rn(c, f));
}
// the same through the conversion instruction: one instruction on the quarter-rate pipe instead of three on
// the fp32 pipe, the better trade where the epilogue runs beside the tensor pipe rather than in its place
__device__ __forceinline__ float bf_round_cvt(float f) { return __bfloat162float(__float2bfloat16_rn(f)); }
// two fp32 -> packed bf16x2 with one conversion instruction
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}
// the same for values that are already bf16-representable (their low 16 bits are zero): a byte permute
__device__ __forceinline__ uint32_t pack_bf16x2_exact(float lo, float hi) {
    return __byte_perm(__float_as_uint(lo), __float_as_uint(hi), 0x7632);
}

// two fp32 -> two e4m3 bytes (round-to-nearest-even, saturating to +-448), lo in bits 0..7
__device__ __forceinline__ uint32_t f2e4m3x2(float lo, float hi) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ uint32_t f2e4m3x4(float a, float b, float c, float d) {
    return f2e4m3x2(a, b) | (f2e4m3x2(c, d) << 16);
}

// The reference's torch quantisers: sf = clamp(amax, 1e-4) / 448 ; inv = 1 / sf
// (test/util.py:21-23). Both divisions are IEEE round-to-nearest.
__device__ __forceinline__ float scale_from_amax(float amax) { return __fdiv_rn(fmaxf(amax, 1e-4f), 448.0f); }
__device__ __forceinline__ float inv_scale(float sf) { return __fdiv_rn(1.0f, sf); }

// one e4m3 byte -> fp32 (exact)
__device__ __forceinline__ float e4m3_to_float(uint32_t byte) {
    const __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(byte & 0xffu), __NV_E4M3);
    return __half2float(*reinterpret_cast<const __half*>(&h));
}
// eight floats -> eight e2m1 nibbles (round to nearest even, saturating at 6), element i in nibble i
__device__ __forceinline__ uint32_t f2e2m1x8(const float (&x)[8]) {
    uint32_t out;
    asm("{\n\t"
        ".reg .b8 b0, b1, b2, b3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
        "mov.b32 %0, {b0, b1, b2, b3};\n\t"
        "}"
        : "=r"(out)
        : "f"(x[0]), "f"(x[1]), "f"(x[2]), "f"(x[3]), "f"(x[4]), "f"(x[5]), "f"(x[6]), "f"(x[7]));
    return out;
}
// NVFP4 scale of a 16-value block: the e4m3 byte nearest to (amax / 6) / g (saturating at 448), g = the tensor's
// global scale; *inv = 1 / (value of that byte * g), or 0 for an all-zero block. A value x of the block is stored
// as e2m1(x * inv).
__device__ __forceinline__ uint32_t nvfp4_scale_byte(float amax, float g, float* inv) {
    const uint32_t byte = f2e4m3x2(__fdiv_rn(__fdiv_rn(amax, 6.0f), g), 0.0f) & 0xffu;
    const float d = e4m3_to_float(byte) * g;
    *inv = d > 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    return byte;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// non-negative floats order like their bit patterns
__device__ __forceinline__ void atomic_max_nonneg(float* addr, float v) {
    atomicMax(reinterpret_cast<int*>(addr), __float_as_int(v));
}

}  // namespace dq
