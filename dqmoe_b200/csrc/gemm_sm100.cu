// Grouped GEMM for expert-sorted rows on sm_100a: a persistent, warp-specialised
// kernel with TMA-fed shared-memory stages, tcgen05 MMA (128 x 256 tiles, fp32
// accumulators in TMEM) and fused epilogues:
//   stage 1 (gated): SwiGLU, plus 1x128 dynamic FP8 re-quantisation in block mode
//                    or amax collection in tensor/channel mode;
//   stage 2        : dequantisation and row scatter into the [T, k, H] output.
// In block mode (1x128 activation scales, 128x128 weight scales) the partial sum
// of every 128-wide K block is drained from TMEM, multiplied by its scale pair
// and accumulated in registers while the next K block runs on the tensor cores
// into the other TMEM buffer.
//
// Replaces the six CUTLASS grouped-GEMM variants of the reference and their
// per-expert "configure" kernels (csrc/moe_gemm_template.h:72-1039) together
// with doGatedActivationKernel, scale_1x128_kernel and finalizeScatterKernel
// (csrc/moe_kernels.h:301-444, 581-620).
#include <cuda_fp16.h>

#include <mutex>
#include <type_traits>

#include "common.cuh"
#include "gemm_tile.cuh"
#include "ptx_sm100.cuh"

namespace dq {
namespace gemm {

constexpr int kBM = 128;                          // rows per tile = UMMA M
constexpr int kBoxRows = 128;                     // weight rows per TMA box, two boxes per stage
constexpr int kUmmaN = 2 * kBoxRows;              // 256 accumulator columns per tile
constexpr int kBKBytes = 128;                     // K bytes per stage: one 128-byte swizzle row
constexpr int kUmmaKBytes = 32;                   // K bytes per tcgen05.mma
constexpr int kStages = 4;                          // single-CTA tiles: 4 stages of A 16 KiB + B 32 KiB
constexpr int kStagesPair = 6;                      // CTA pairs: 6 stages of A 16 KiB + B-half 16 KiB
constexpr int kMaxStages = 6;
constexpr int kABytes = kBM * kBKBytes;           // 16 KiB
constexpr int kBBytes = kUmmaN * kBKBytes;        // 32 KiB
constexpr int kStageBytes = kABytes + kBBytes;    // 48 KiB
constexpr int kStageBytesPair = kABytes + kBBytes / 2;  // 32 KiB per CTA of a pair
static_assert(kStages * kStageBytes == kStagesPair * kStageBytesPair, "both layouts fill the same stage area");
constexpr int kThreads = 384;                     // warp 0 TMA, warp 1 MMA, warp 2 scale loader (block mode), warp 3 idle, warps 4..11 epilogue
constexpr int kRegsControl = 56;                  // registers per thread of the TMA/MMA warpgroup
constexpr int kRegsEpilogue = 224;                // registers per thread of the two epilogue warpgroups
constexpr int kEpiWarps = 8;
constexpr int kMaxExperts = 1024;
constexpr int kMaxDevices = 64;
constexpr int kScaleSlots = 8;                     // ring of per-K-block scale sets (block mode)
constexpr int kTmemCols = 512;                    // two accumulator buffers of 256 columns
constexpr long long kWaitLimit = 1000000000LL;    // clock cycles before a wait gives up (~0.5 s)

enum Mode : int { kNone = 0, kTensor = 1, kChannel = 2, kBlock = 3 };

struct Params {
    int n_rows;          // rows of A (expanded rows n)
    int N;               // output columns (stage 1: I, stage 2: H)
    int K;               // reduction length in elements
    int E;
    int n_tiles;         // column tiles per row tile
    int w_rows;          // weight rows per expert (stage 1: 2I, stage 2: H)
    int tile_w_rows;     // weight rows advanced per column tile (stage 1: 128, stage 2: 256)
    int box2_off;        // row offset of the second weight box (stage 1: I, stage 2: 128)
    int kb_count;        // ceil(K bytes / 128)
    const int* offsets;       // [E+1] first row of each expert
    const int* mtile_prefix;  // [E+1] cumulative 128-row tiles
    const float* sa;          // activation scales
    const float* sb;          // weight scales
    void* out;
    float* out_scale;         // stage 1 block mode: [n, ceil(I/128)]
    float* amax;              // stage 1 channel: [n]; tensor: [1]
    const float* bias;        // [E, w_rows] fp32 added to the dequantised product, or nullptr
    const int* dest_to_src;   // stage 2 scatter map or nullptr
    const unsigned long long* row_dst;  // stage 2: address of each row's output row (may be peer memory), or nullptr
    int* status;              // host-mapped status word
};

struct SharedTail {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint64_t epi_sync[4];    // per TMEM lane quarter: the two warps that share a row's 1x128 group
    uint64_t sc_full[kScaleSlots];
    uint64_t sc_empty[kScaleSlots];
    uint32_t tmem_base;
    int abort_flag;
    alignas(16) float amax[2][2][kBM];
    float sc_a[kScaleSlots][kBM];   // activation scale of each tile row for one K block
    float sc_b[kScaleSlots][4];     // weight scales: first group, second group (low / high block row)
    uint4 stage[kEpiWarps][32 * 4]; // per epilogue warp: 32 rows x 64 bytes, for row-coalesced stores
    int mprefix[kMaxExperts + 1];
    int offsets[kMaxExperts + 1];
};

constexpr size_t kSmemBytes = 1024 + size_t(kStages) * kStageBytes + sizeof(SharedTail);

struct Tile {
    int e, row0, row_end, nt;
};

// Tiles are numbered expert-major; inside an expert the row tile runs fastest so
// that concurrently running CTAs share one weight tile and the expert's rows
// stay in L2.
// With CTA pairs a tile is 256 rows: mprefix then counts pairs of 128-row tiles and CTA `sub`
// of the pair takes row tile 2j + sub (the second one is empty when the expert's tile count is odd).
template <bool kPair>
__device__ __forceinline__ Tile decode_tile(int t, int& e_cursor, const SharedTail& st, int n_tiles, int sub) {
    while (t >= st.mprefix[e_cursor + 1] * n_tiles) ++e_cursor;
    const int local = t - st.mprefix[e_cursor] * n_tiles;
    const int mtiles = st.mprefix[e_cursor + 1] - st.mprefix[e_cursor];
    Tile tl;
    tl.e = e_cursor;
    tl.nt = local / mtiles;
    tl.row0 = st.offsets[e_cursor] + ((local % mtiles) * (kPair ? 2 : 1) + sub) * kBM;
    tl.row_end = st.offsets[e_cursor + 1];
    return tl;
}

// Rows of the weight-scale grid a block-mode tile reads: the first 128-column group uses one
// block row; the second group uses `lo` for columns below `c_switch` and `hi` from there on
// (the gate/value boundary of stage 1 need not fall on a 128-row block boundary).
struct ScaleRows {
    int nb0, nb1_lo, nb1_hi, c_switch;
};
__device__ __forceinline__ ScaleRows scale_rows(bool gated, int nt, int N, int NB) {
    ScaleRows r;
    if (gated) {
        r.nb0 = nt;
        const int v0 = N + nt * kBoxRows;  // first value row of this tile
        r.nb1_lo = v0 >> 7;
        r.c_switch = 128 - (v0 & 127);
        r.nb1_hi = r.nb1_lo + 1;
    } else {
        r.nb0 = nt * 2;
        r.nb1_lo = r.nb0 + 1;
        r.nb1_hi = r.nb1_lo;
        r.c_switch = 128;
    }
    r.nb0 = min(r.nb0, NB - 1);
    r.nb1_lo = min(r.nb1_lo, NB - 1);
    r.nb1_hi = min(r.nb1_hi, NB - 1);
    return r;
}

__device__ __forceinline__ float silu_bf16(float g) {
    // the torch oracle evaluates silu on bf16 and rounds the result to bf16 (test/util.py:141-142)
    return bf_round_cvt(__fdividef(g, 1.0f + __expf(-g)));
}

// One 32-column chunk of a tile row per lane: 32 values of 16 bits (packed[16]) or of 32 bits (packed[32], two
// 64-byte halves). cols_left = columns of the matrix from the chunk's first column on.
template <bool kWide, int kWords>
__device__ __forceinline__ void store_chunk(uint4* stage, const uint32_t (&packed)[kWords], uint8_t* row_ptr,
                                            int cols_left, int lane) {
    if constexpr (!kWide) {
        static_assert(kWords == 16, "32 values of 16 bits");
        store_rows_staged(stage, packed, row_ptr, min(4, max(0, (cols_left + 7) / 8)), lane);
    } else {
        static_assert(kWords == 32, "32 values of 32 bits");
        uint32_t half[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) half[i] = packed[i];
        store_rows_staged(stage, half, row_ptr, min(4, max(0, (cols_left + 3) / 4)), lane);
#pragma unroll
        for (int i = 0; i < 16; ++i) half[i] = packed[16 + i];
        store_rows_staged(stage, half, row_ptr != nullptr ? row_ptr + 64 : nullptr,
                          min(4, max(0, (cols_left - 16 + 3) / 4)), lane);
    }
}

// Element type of the unquantised path: bf16, IEEE half or fp32 - the T = bf16 / half / float instantiations
// of the reference's template (csrc/pybind11_register.h:104-151, csrc/moe_gemm_template.h:487-569). fp32
// operands go through the tensor cores as TF32 (kind::tf32), as the reference's float instantiation does
// on its mma.sync path; intermediates and outputs then stay fp32.
enum Elem : int { kElemBf16 = 0, kElemHalf = 1, kElemF32 = 2 };

// Rounding to the storage type of the intermediate and the output.
template <int kElem>
__device__ __forceinline__ float round16(float x) {
    if constexpr (kElem == kElemHalf)
        return __half2float(__float2half_rn(x));
    else if constexpr (kElem == kElemF32)
        return x;
    else
        return bf_round_cvt(x);
}
template <int kElem>
__device__ __forceinline__ uint32_t pack16x2(float lo, float hi) {
    static_assert(kElem != kElemF32, "fp32 outputs are not packed");
    if constexpr (kElem == kElemHalf) {
        const __half2 h = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<const uint32_t*>(&h);
    } else {
        return pack_bf16x2(lo, hi);
    }
}

// two fp32 FMAs in one instruction (packed fp32 of sm_100): a += x * s
__device__ __forceinline__ void ffma2(float& a0, float& a1, uint32_t x0, uint32_t x1, float s0, float s1) {
    const float2 r = __ffma2_rn(make_float2(__uint_as_float(x0), __uint_as_float(x1)), make_float2(s0, s1),
                                make_float2(a0, a1));
    a0 = r.x;
    a1 = r.y;
}

// kBox = weight rows per TMA box (two boxes per stage, 2*kBox accumulator columns): 128 for
// throughput, 64 when a launch would otherwise have fewer tiles than SMs (decode shapes).
template <bool kFp8, int kMode, bool kGated, bool kPair, int kBox, int kElem = kElemBf16>
__global__ void __launch_bounds__(kThreads, 1)
moe_GemmGrouped_GemmUniversal_tcgen05(const __grid_constant__ CUtensorMap tma_a,
                                      const __grid_constant__ CUtensorMap tma_b, const Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    SharedTail& st = *reinterpret_cast<SharedTail*>(smem + size_t(kStages) * kStageBytes);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    constexpr int kBKElems = kFp8 ? kBKBytes : (kElem == kElemF32 ? kBKBytes / 4 : kBKBytes / 2);
    constexpr int kKind = kFp8 ? 0 : (kElem == kElemF32 ? 2 : 1);  // kind::f8f6f4, kind::f16, kind::tf32
    static_assert(kBox == 128 || (kBox == 64 && !kPair && kMode != kBlock), "narrow tiles: single CTA, non-block modes");
    static_assert(kElem == kElemBf16 || (!kFp8 && kMode == kNone), "fp16 / fp32 operands: the unquantised path only");
    static_assert(kElem != kElemF32 || (!kPair && kBox == 128), "fp32 operands: single-CTA 256-column tiles only");
    constexpr int kN = 2 * kBox;                      // accumulator columns of a tile
    constexpr int kStageSz = kPair ? kStageBytesPair : kABytes + kN * kBKBytes;
    constexpr int kNumStages = (kStages * kStageBytes) / kStageSz;   // 4 (wide), 6 (pairs, narrow)
    constexpr int kHalf = kBox / 2;                   // columns of each group owned by one epilogue warpgroup
    constexpr int kChunks = kBox / 64;                // 32-column chunks per thread and group
    // In a pair, CTA 0 (the leader) issues the MMAs for both and owns the barriers they wait on.
    const uint32_t cta_rank = kPair ? ptx::cluster_ctarank() : 0u;
    const bool leader = cta_rank == 0u;
    const int tile_first = kPair ? int(blockIdx.x >> 1) : int(blockIdx.x);
    const int tile_step = kPair ? int(gridDim.x >> 1) : int(gridDim.x);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kNumStages; ++s) {
            ptx::mbar_init(&st.full[s], 1);
            ptx::mbar_init(&st.empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(&st.tmem_full[b], 1);
            ptx::mbar_init(&st.tmem_empty[b], kPair ? 2 * kEpiWarps : kEpiWarps);  // both CTAs' epilogue warps
        }
        for (int i = 0; i < 4; ++i) ptx::mbar_init(&st.epi_sync[i], 2);
        for (int i = 0; i < kScaleSlots; ++i) {
            ptx::mbar_init(&st.sc_full[i], 32);         // every lane of the scale-loader warp
            ptx::mbar_init(&st.sc_empty[i], kEpiWarps);
        }
        st.abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async();
    }
    if constexpr (kPair) ptx::cluster_sync();  // the peer's barriers exist before anything signals them
    if (warp == 1) {
        if constexpr (kPair) {
            ptx::tmem_alloc_pair(&st.tmem_base, kTmemCols);
            ptx::tmem_relinquish_pair();
        } else {
            ptx::tmem_alloc(&st.tmem_base, kTmemCols);
            ptx::tmem_relinquish();
        }
    }
    for (int i = threadIdx.x; i <= p.E; i += kThreads) {
        st.mprefix[i] = p.mtile_prefix[i];
        st.offsets[i] = p.offsets[i];
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    if constexpr (kPair) {
        if (threadIdx.x == 0) {  // tiles of 128 rows -> pairs of tiles, in place
            int prev = st.mprefix[0], run = 0;
            st.mprefix[0] = 0;
            for (int e = 0; e < p.E; ++e) {
                const int next = st.mprefix[e + 1];
                run += (next - prev + 1) >> 1;
                prev = next;
                st.mprefix[e + 1] = run;
            }
        }
        __syncthreads();
        ptx::cluster_sync();  // both CTAs hold their TMEM before the first pair MMA
    }

    const uint32_t tmem_base = st.tmem_base;
    const int total_tiles = st.mprefix[p.E] * p.n_tiles;
    volatile int* abort_flag = &st.abort_flag;
    const int kb_count = p.kb_count;

    // The launch gives every thread 168 registers; the control warpgroup hands most of its
    // share to the epilogue warpgroups, whose block-scaled accumulators live in registers.
    if (warp < 4) {
      ptx::setmaxnreg_dec<kRegsControl>();
      if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            ptx::prefetch_tensormap(&tma_a);
            ptx::prefetch_tensormap(&tma_b);
            uint32_t it = 0;
            int e_cursor = 0;
            bool ok = true;
            for (int t = tile_first; ok && t < total_tiles; t += tile_step) {
                const Tile tl = decode_tile<kPair>(t, e_cursor, st, p.n_tiles, cta_rank);
                const int wrow0 = tl.e * p.w_rows + tl.nt * p.tile_w_rows;
                const int wrow1 = wrow0 + p.box2_off;
                for (int kb = 0; kb < kb_count; ++kb, ++it) {
                    const int s = it % kNumStages;
                    const uint32_t ph = (it / kNumStages) & 1u;
                    if (!ptx::mbar_wait(&st.empty[s], ph ^ 1u, abort_flag, kWaitLimit)) {
                        ok = false;
                        break;
                    }
                    uint8_t* sa = smem + size_t(s) * kStageSz;
                    uint8_t* sb = sa + kABytes;
                    const int k0 = kb * kBKElems;
                    if constexpr (kPair) {
                        // Each CTA loads its own 128 rows of A and its half of the weight tile (CTA 0 the
                        // first 128 rows, CTA 1 the second); all bytes are credited to the leader's barrier.
                        const uint32_t full_leader = ptx::map_to_cta(&st.full[s], 0);
                        if (leader) ptx::mbar_arrive_expect_tx(&st.full[s], 2 * kStageBytesPair);
                        ptx::tma_load_2d_pair(sa, &tma_a, k0, tl.row0, full_leader);
                        ptx::tma_load_2d_pair(sb, &tma_b, k0, leader ? wrow0 : wrow1, full_leader);
                    } else {
                        ptx::mbar_arrive_expect_tx(&st.full[s], kStageSz);
                        ptx::tma_load_2d(sa, &tma_a, k0, tl.row0, &st.full[s]);
                        ptx::tma_load_2d(sb, &tma_b, k0, wrow0, &st.full[s]);
                        ptx::tma_load_2d(sb + kBox * kBKBytes, &tma_b, k0, wrow1, &st.full[s]);
                    }
                }
            }
        }
        __syncwarp();
      } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0 && leader) {
            // operand format code: e4m3 = 0 (kind::f8f6f4); f16 = 0, bf16 = 1 (kind::f16); tf32 = 2 (kind::tf32)
            constexpr uint32_t idesc =
                ptx::make_idesc(kFp8 || kElem == kElemHalf ? 0u : (kElem == kElemF32 ? 2u : 1u), kPair ? 2 * kBM : kBM, kN);
            // issue one K step; in a pair the same call drives both CTAs' tensor cores
            auto mma_step = [&](uint32_t d_tmem, uint32_t a_addr, uint32_t b_addr, uint32_t accumulate) {
                if constexpr (kPair)
                    ptx::umma_pair<kKind>(d_tmem, ptx::smem_desc_sw128(a_addr), ptx::smem_desc_sw128(b_addr), idesc, accumulate);
                else
                    ptx::umma<kKind>(d_tmem, ptx::smem_desc_sw128(a_addr), ptx::smem_desc_sw128(b_addr), idesc, accumulate);
            };
            // completion of everything issued so far -> one barrier (of both CTAs in a pair)
            auto commit = [&](uint64_t* bar) {
                if constexpr (kPair) {
                    ptx::umma_commit_pair(ptx::map_to_cta(bar, 0));
                    ptx::umma_commit_pair(ptx::map_to_cta(bar, 1));
                } else {
                    ptx::umma_commit(bar);
                }
            };
            uint32_t it = 0;
            uint32_t acc_it = 0;
            bool ok = true;
            for (int t = tile_first; ok && t < total_tiles; t += tile_step) {
                if constexpr (kMode != kBlock) {
                    const uint32_t buf = acc_it & 1u;
                    if (!ptx::mbar_wait(&st.tmem_empty[buf], ((acc_it >> 1) & 1u) ^ 1u, abort_flag, kWaitLimit)) {
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
                    for (int kb = 0; kb < kb_count; ++kb, ++it) {
                        const int s = it % kNumStages;
                        if (!ptx::mbar_wait(&st.full[s], (it / kNumStages) & 1u, abort_flag, kWaitLimit)) {
                            ok = false;
                            break;
                        }
                        ptx::tc_fence_after();
                        const uint32_t a_addr = ptx::smem_u32(smem + size_t(s) * kStageSz);
                        const uint32_t b_addr = a_addr + kABytes;
#pragma unroll
                        for (int k = 0; k < kBKBytes / kUmmaKBytes; ++k)
                            mma_step(tmem_base + buf * kUmmaN, a_addr + k * kUmmaKBytes, b_addr + k * kUmmaKBytes,
                                     (kb | k) != 0 ? 1u : 0u);
                        commit(&st.empty[s]);
                    }
                    if (!ok) break;
                    commit(&st.tmem_full[buf]);
                    ++acc_it;
                } else {
                    // Block mode: every K block gets its own TMEM buffer (two alternate).
                    for (int kb = 0; kb < kb_count; ++kb, ++it, ++acc_it) {
                        const uint32_t buf = acc_it & 1u;
                        const int s = it % kNumStages;
                        if (!ptx::mbar_wait(&st.tmem_empty[buf], ((acc_it >> 1) & 1u) ^ 1u, abort_flag, kWaitLimit)) {
                            ok = false;
                            break;
                        }
                        if (!ptx::mbar_wait(&st.full[s], (it / kNumStages) & 1u, abort_flag, kWaitLimit)) {
                            ok = false;
                            break;
                        }
                        ptx::tc_fence_after();
                        const uint32_t a_addr = ptx::smem_u32(smem + size_t(s) * kStageSz);
                        const uint32_t b_addr = a_addr + kABytes;
#pragma unroll
                        for (int k = 0; k < kBKBytes / kUmmaKBytes; ++k)
                            mma_step(tmem_base + buf * kUmmaN, a_addr + k * kUmmaKBytes, b_addr + k * kUmmaKBytes,
                                     k != 0 ? 1u : 0u);
                        commit(&st.tmem_full[buf]);
                        commit(&st.empty[s]);
                    }
                }
            }
        }
        __syncwarp();
      } else if (warp == 2) {
        // ------------------------------------------------------------ scale loader (block mode)
        // Stages the scales of every K block in shared memory ahead of the epilogue warps with
        // 4-byte asynchronous copies, so no global-load latency sits in the accumulation loop.
        if constexpr (kMode == kBlock) {
            const int KB = kb_count;
            const int NB = (p.w_rows + 127) / 128;
            uint32_t it = 0;
            int e_cursor = 0;
            bool ok = true;
            for (int t = tile_first; ok && t < total_tiles; t += tile_step) {
                const Tile tl = decode_tile<kPair>(t, e_cursor, st, p.n_tiles, cta_rank);
                const ScaleRows sr = scale_rows(kGated, tl.nt, p.N, NB);
                const float* src_a[4];
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    src_a[j] = p.sa + size_t(min(tl.row0 + lane + 32 * j, p.n_rows - 1)) * KB;
                const int nb = lane == 0 ? sr.nb0 : (lane == 1 ? sr.nb1_lo : sr.nb1_hi);
                const float* src_b = p.sb + (size_t(tl.e) * NB + nb) * KB;
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    const int slot = it % kScaleSlots;
                    if (!ptx::mbar_wait(&st.sc_empty[slot], ((it / kScaleSlots) & 1u) ^ 1u, abort_flag, kWaitLimit)) {
                        ok = false;
                        break;
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j) ptx::cp_async4(&st.sc_a[slot][lane + 32 * j], src_a[j] + kb);
                    if (lane < 3) ptx::cp_async4(&st.sc_b[slot][lane], src_b + kb);
                    ptx::cp_async_arrive(&st.sc_full[slot]);
                }
            }
            ptx::cp_async_wait_all();
        }
      }
    } else {
        ptx::setmaxnreg_inc<kRegsEpilogue>();
        // ------------------------------------------------------------ epilogue warps
        const int q = warp & 3;            // TMEM lane quarter this warp may read
        const int h = (warp - 4) >> 2;     // which 64-column half of each 128-column group
        const int r_in_tile = q * 32 + lane;
        const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
        uint32_t acc_it = 0;
        uint32_t sc_it = 0;
        uint32_t tile_it = 0;
        uint32_t epi_phase = 0;
        int e_cursor = 0;
        bool ok = true;
        const int I_or_H = p.N;
        // hand a drained accumulator buffer back to the MMA thread (which lives in the leader CTA)
        auto release_tmem = [&](uint32_t b) {
            if constexpr (kPair)
                ptx::mbar_arrive_cluster(ptx::map_to_cta(&st.tmem_empty[b], 0));
            else
                ptx::mbar_arrive(&st.tmem_empty[b]);
        };

        for (int t = tile_first; ok && t < total_tiles; t += tile_step, ++tile_it) {
            const Tile tl = decode_tile<kPair>(t, e_cursor, st, p.n_tiles, cta_rank);
            const int grow = tl.row0 + r_in_tile;
            const bool row_ok = grow < tl.row_end;
            const int grow_ld = min(grow, p.n_rows - 1);

            if constexpr (kMode != kBlock) {
                const uint32_t buf = acc_it & 1u;
                if (!ptx::mbar_wait(&st.tmem_full[buf], (acc_it >> 1) & 1u, abort_flag, kWaitLimit)) {
                    ok = false;
                    break;
                }
                ++acc_it;
                ptx::tc_fence_after();
                const uint32_t t_buf = t_lane + buf * kUmmaN;

                // Per-chunk column constants (channel-mode weight scales, bias) are staged once per warp in its
                // store buffer and read back as broadcast 16-byte loads: floats [0,32) gate / plain scales,
                // [32,64) value scales, [64,96) gate / plain bias, [96,128) value bias. The buffer is free
                // until the staged store of the same chunk.
                float* csw = reinterpret_cast<float*>(st.stage[warp - 4]);
                [[maybe_unused]] const float4* cs4 = reinterpret_cast<const float4*>(st.stage[warp - 4]);
                const bool has_bias = p.bias != nullptr;
                const float* bias_e = has_bias ? p.bias + size_t(tl.e) * p.w_rows : nullptr;
                float row_scale = 1.0f;
                if constexpr (kMode == kTensor) row_scale = p.sa[0] * p.sb[tl.e];
                if constexpr (kMode == kChannel) row_scale = p.sa[grow_ld];
                constexpr int kOutBytes = kElem == kElemF32 ? 4 : 2;

                if constexpr (kGated) {
                    // columns [h*kHalf, (h+1)*kHalf) of the gate group and of the value group
                    float amax_local = 0.0f;
#pragma unroll 1
                    for (int j = 0; j < kChunks; ++j) {
                        uint32_t g[32], v[32];
                        const int c0 = h * kHalf + j * 32;  // column inside the kBox-wide act tile
                        ptx::tmem_ld32(t_buf + c0, g);
                        ptx::tmem_ld32(t_buf + kBox + c0, v);
                        const int col0 = tl.nt * kBox + c0;
                        if (kMode == kChannel || has_bias) {
                            __syncwarp();
                            const int c = min(col0 + lane, I_or_H - 1);
                            if constexpr (kMode == kChannel) {
                                csw[lane] = p.sb[size_t(tl.e) * p.w_rows + c];
                                csw[32 + lane] = p.sb[size_t(tl.e) * p.w_rows + I_or_H + c];
                            }
                            if (has_bias) {
                                csw[64 + lane] = bias_e[c];
                                csw[96 + lane] = bias_e[I_or_H + c];
                            }
                            __syncwarp();
                        }
                        ptx::tmem_wait_ld(g);
                        ptx::tmem_wait_ld(v);
                        uint32_t packed[kElem == kElemF32 ? 32 : 16];
                        // This epilogue runs beside the next tile's MMAs; its roundings use the conversion
                        // instruction (one issue slot each), which measured faster here than bf_round.
#pragma unroll
                        for (int i = 0; i < 32; i += 4) {
                            float sg[4] = {row_scale, row_scale, row_scale, row_scale};
                            float sv[4] = {row_scale, row_scale, row_scale, row_scale};
                            if constexpr (kMode == kChannel) {
                                const float4 a = cs4[i >> 2], b = cs4[8 + (i >> 2)];
                                sg[0] *= a.x, sg[1] *= a.y, sg[2] *= a.z, sg[3] *= a.w;
                                sv[0] *= b.x, sv[1] *= b.y, sv[2] *= b.z, sv[3] *= b.w;
                            }
                            float bg[4] = {0.0f, 0.0f, 0.0f, 0.0f}, bv[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                            if (has_bias) {
                                const float4 a = cs4[16 + (i >> 2)], b = cs4[24 + (i >> 2)];
                                bg[0] = a.x, bg[1] = a.y, bg[2] = a.z, bg[3] = a.w;
                                bv[0] = b.x, bv[1] = b.y, bv[2] = b.z, bv[3] = b.w;
                            }
                            float a4[4];
#pragma unroll
                            for (int u = 0; u < 4; ++u) {
                                const float gate = round16<kElem>(__uint_as_float(g[i + u]) * sg[u] + bg[u]);
                                const float val = round16<kElem>(__uint_as_float(v[i + u]) * sv[u] + bv[u]);
                                const float act = round16<kElem>(round16<kElem>(__fdividef(gate, 1.0f + __expf(-gate))) * val);
                                a4[u] = act;
                                if (col0 + i + u < I_or_H) amax_local = fmaxf(amax_local, fabsf(act));
                            }
                            if constexpr (kElem == kElemF32) {
#pragma unroll
                                for (int u = 0; u < 4; ++u) packed[i + u] = __float_as_uint(a4[u]);
                            } else if constexpr (kElem == kElemHalf) {
                                packed[i >> 1] = pack16x2<kElemHalf>(a4[0], a4[1]);
                                packed[(i >> 1) + 1] = pack16x2<kElemHalf>(a4[2], a4[3]);
                            } else {
                                packed[i >> 1] = pack_bf16x2_exact(a4[0], a4[1]);  // act is already rounded to bf16
                                packed[(i >> 1) + 1] = pack_bf16x2_exact(a4[2], a4[3]);
                            }
                        }
                        uint8_t* optr = row_ok ? static_cast<uint8_t*>(p.out) + (size_t(grow) * I_or_H + col0) * kOutBytes
                                               : nullptr;
                        store_chunk<kElem == kElemF32>(st.stage[warp - 4], packed, optr, I_or_H - col0, lane);
                    }
                    if constexpr (kMode == kChannel) {
                        if (row_ok) atomic_max_nonneg(p.amax + grow, amax_local);
                    }
                    if constexpr (kMode == kTensor) {
                        float m = row_ok ? amax_local : 0.0f;
                        m = warp_max(m);
                        if (lane == 0) atomic_max_nonneg(p.amax, m);
                    }
                } else {
                    // stage 2: this warpgroup's half of each of the two kBox-column groups
                    int orow_idx = grow;
                    if (row_ok && p.dest_to_src != nullptr) orow_idx = p.dest_to_src[grow];
                    uint8_t* orow = static_cast<uint8_t*>(p.out) + size_t(orow_idx) * I_or_H * kOutBytes;
                    if (p.row_dst != nullptr) {  // rows go to explicit addresses (expert parallel: the home rank's output)
                        orow = row_ok ? reinterpret_cast<uint8_t*>(p.row_dst[grow]) : nullptr;
                        orow_idx = orow != nullptr ? 0 : -1;
                    }
#pragma unroll 1
                    for (int c = 0; c < 2 * kChunks; ++c) {
                        uint32_t r[32];
                        const int tc = (c / kChunks) * kBox + h * kHalf + (c % kChunks) * 32;
                        ptx::tmem_ld32(t_buf + tc, r);
                        const int col0 = tl.nt * kN + tc;
                        if (kMode == kChannel || has_bias) {  // column constants of the chunk, as in stage 1
                            __syncwarp();
                            const int cc = min(col0 + lane, I_or_H - 1);
                            if constexpr (kMode == kChannel) csw[lane] = p.sb[size_t(tl.e) * p.w_rows + cc];
                            if (has_bias) csw[64 + lane] = bias_e[cc];
                            __syncwarp();
                        }
                        ptx::tmem_wait_ld(r);
                        uint32_t packed[kElem == kElemF32 ? 32 : 16];
#pragma unroll
                        for (int i = 0; i < 32; i += 4) {
                            float sc[4] = {row_scale, row_scale, row_scale, row_scale};
                            if constexpr (kMode == kChannel) {
                                const float4 a = cs4[i >> 2];
                                sc[0] *= a.x, sc[1] *= a.y, sc[2] *= a.z, sc[3] *= a.w;
                            }
                            float bb[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                            if (has_bias) {
                                const float4 a = cs4[16 + (i >> 2)];
                                bb[0] = a.x, bb[1] = a.y, bb[2] = a.z, bb[3] = a.w;
                            }
                            float o4[4];
#pragma unroll
                            for (int u = 0; u < 4; ++u) o4[u] = __uint_as_float(r[i + u]) * sc[u] + bb[u];
                            if constexpr (kElem == kElemF32) {
#pragma unroll
                                for (int u = 0; u < 4; ++u) packed[i + u] = __float_as_uint(o4[u]);
                            } else {
                                packed[i >> 1] = pack16x2<kElem>(o4[0], o4[1]);
                                packed[(i >> 1) + 1] = pack16x2<kElem>(o4[2], o4[3]);
                            }
                        }
                        store_chunk<kElem == kElemF32>(st.stage[warp - 4], packed,
                                                   row_ok && orow_idx >= 0 ? orow + size_t(col0) * kOutBytes : nullptr,
                                                   I_or_H - col0, lane);
                    }
                }
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) release_tmem(buf);
            } else {
                // ---------------------------------------------------- block-scaled accumulation
                // acc[c*32 + i]: chunk c of this thread's four 32-column chunks.
                float acc[128];
#pragma unroll
                for (int i = 0; i < 128; ++i) acc[i] = 0.0f;

                const int KB = kb_count;                      // scale blocks along K
                const int NB = (p.w_rows + 127) / 128;        // weight scale block rows per expert
                const int c_switch = scale_rows(kGated, tl.nt, I_or_H, NB).c_switch;
                const bool uniform = (c_switch & 31) == 0;

                // Software pipeline over the four 32-column chunks of a K block: while 32 FMAs run
                // on one register set the TMEM load of the next chunk lands in the other.
                // The TMEM buffer must go back to the MMA warp as early as possible (the round trip
                // MMA -> drain -> MMA of one buffer bounds the K-block rate), so per K block: fetch the
                // scales, wait for the buffer, pull the four 32-column chunks through two register
                // sets, release the buffer, and only then add the last two chunks.
                // The loop exists twice: kOneScale when the second column group lies inside one 128-row
                // weight-scale block (always in stage 2; in stage 1 unless I % 128 != 0), where no
                // per-column choice of scale is left in the inner loop, and the general form.
                auto tcol = [&](int c) { return (c >> 1) * kBoxRows + h * 64 + (c & 1) * 32; };
                auto k_loop = [&](auto one_scale_tag) {
                    constexpr bool kOneScale = decltype(one_scale_tag)::value;
                    auto fma_chunk = [&](int c, const uint32_t (&r)[32], float s0, float s1l, float s1h) {
                        const int cin = h * 64 + (c & 1) * 32;  // column inside the 128-column group
                        if (c < 2) {
#pragma unroll
                            for (int i = 0; i < 32; i += 2) ffma2(acc[c * 32 + i], acc[c * 32 + i + 1], r[i], r[i + 1], s0, s0);
                        } else if (kOneScale || uniform) {
                            const float s1 = kOneScale || cin < c_switch ? s1l : s1h;
#pragma unroll
                            for (int i = 0; i < 32; i += 2) ffma2(acc[c * 32 + i], acc[c * 32 + i + 1], r[i], r[i + 1], s1, s1);
                        } else {
#pragma unroll
                            for (int i = 0; i < 32; i += 2)
                                ffma2(acc[c * 32 + i], acc[c * 32 + i + 1], r[i], r[i + 1], (cin + i) < c_switch ? s1l : s1h,
                                      (cin + i + 1) < c_switch ? s1l : s1h);
                        }
                    };
                    uint32_t r0[32], r1[32];
                    for (int kb = 0; kb < KB; ++kb, ++acc_it, ++sc_it) {
                        const int slot = sc_it % kScaleSlots;
                        if (!ptx::mbar_wait(&st.sc_full[slot], (sc_it / kScaleSlots) & 1u, abort_flag, kWaitLimit)) return false;
                        const float a_s = st.sc_a[slot][r_in_tile];
                        const float s0 = a_s * st.sc_b[slot][0], s1l = a_s * st.sc_b[slot][1];
                        const float s1h = kOneScale ? 0.0f : a_s * st.sc_b[slot][2];
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive(&st.sc_empty[slot]);

                        const uint32_t buf = acc_it & 1u;
                        if (!ptx::mbar_wait(&st.tmem_full[buf], (acc_it >> 1) & 1u, abort_flag, kWaitLimit)) return false;
                        ptx::tc_fence_after();
                        const uint32_t t_buf = t_lane + buf * kUmmaN;
                        ptx::tmem_ld32(t_buf + tcol(0), r0);
                        ptx::tmem_ld32(t_buf + tcol(1), r1);
                        ptx::tmem_wait_ld2(r0, r1);
                        fma_chunk(0, r0, s0, s1l, s1h);
                        ptx::tmem_ld32(t_buf + tcol(2), r0);
                        fma_chunk(1, r1, s0, s1l, s1h);
                        ptx::tmem_ld32(t_buf + tcol(3), r1);
                        ptx::tmem_wait_ld2(r0, r1);
                        ptx::tc_fence_before();
                        __syncwarp();
                        if (lane == 0) release_tmem(buf);
                        fma_chunk(2, r0, s0, s1l, s1h);
                        fma_chunk(3, r1, s0, s1l, s1h);
                    }
                    return true;
                };
                if (!kGated || c_switch == 128)
                    ok = k_loop(std::true_type{});
                else
                    ok = k_loop(std::false_type{});
                if (!ok) break;
                if (p.bias != nullptr) {  // the same address in every lane: broadcast loads
                    const float* bias_e = p.bias + size_t(tl.e) * p.w_rows;
#pragma unroll
                    for (int i = 0; i < 128; ++i) {
                        const int cg = kGated ? (i >> 6) * I_or_H + tl.nt * kBoxRows + h * 64 + (i & 63)
                                              : tl.nt * kUmmaN + tcol(i >> 5) + (i & 31);
                        acc[i] += __ldg(bias_e + min(cg, p.w_rows - 1));
                    }
                }

                if constexpr (kGated) {
                    // act columns nt*128 + h*64 + [0, 64): gate = acc[0..63], value = acc[64..127]
                    const int col0 = tl.nt * kBoxRows + h * 64;
                    float amax_local = 0.0f;
                    // The tensor pipe idles during this part (the same warps drain its buffers), so it is
                    // written for throughput: bf16 roundings on the fp32 pipe (bf_round), eight elements
                    // per step and stage by stage so that the exp / reciprocal latencies overlap.
                    auto swiglu = [&](auto full_tag) {
                        constexpr bool kFullTile = decltype(full_tag)::value;  // all 64 columns inside the matrix
#pragma unroll
                        for (int i0 = 0; i0 < 64; i0 += 8) {
                            float g8[8], e8[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                g8[j] = bf_round(acc[i0 + j]);
                                e8[j] = __expf(-g8[j]);
                            }
#pragma unroll
                            for (int j = 0; j < 8; ++j) e8[j] = bf_round(__fdividef(g8[j], 1.0f + e8[j]));
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                float act = bf_round(e8[j] * bf_round(acc[64 + i0 + j]));
                                if (!kFullTile && col0 + i0 + j >= I_or_H) act = 0.0f;
                                acc[i0 + j] = act;
                                amax_local = fmaxf(amax_local, fabsf(act));
                            }
                        }
                    };
                    if (col0 + 64 <= I_or_H)
                        swiglu(std::true_type{});
                    else
                        swiglu(std::false_type{});
                    // the 1x128 group spans both halves: exchange the partial amax through shared memory
                    st.amax[tile_it & 1u][h][r_in_tile] = amax_local;
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(&st.epi_sync[q]);
                    if (!ptx::mbar_wait(&st.epi_sync[q], epi_phase, abort_flag, kWaitLimit)) {
                        ok = false;
                        break;
                    }
                    epi_phase ^= 1u;
                    const float amax = fmaxf(amax_local, st.amax[tile_it & 1u][h ^ 1][r_in_tile]);
                    const float sf = scale_from_amax(amax);
                    const float inv = inv_scale(sf);
                    {
                        uint32_t packed[16];  // 64 e4m3 bytes of this row
#pragma unroll
                        for (int g4 = 0; g4 < 16; ++g4) {
                            const float* a = acc + g4 * 4;
                            packed[g4] = f2e4m3x4(a[0] * inv, a[1] * inv, a[2] * inv, a[3] * inv);
                        }
                        store_rows_staged(st.stage[warp - 4], packed,
                                          row_ok ? reinterpret_cast<uint8_t*>(p.out) + size_t(grow) * I_or_H + col0 : nullptr,
                                          min(4, max(0, (I_or_H - col0 + 15) / 16)), lane);
                        if (row_ok && h == 0) p.out_scale[size_t(grow) * ((I_or_H + 127) / 128) + tl.nt] = sf;
                    }
                } else {
                    int orow_idx = grow;
                    if (row_ok && p.dest_to_src != nullptr) orow_idx = p.dest_to_src[grow];
                    __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.out) + size_t(orow_idx) * I_or_H;
                    if (p.row_dst != nullptr) {
                        orow = row_ok ? reinterpret_cast<__nv_bfloat16*>(p.row_dst[grow]) : nullptr;
                        orow_idx = orow != nullptr ? 0 : -1;
                    }
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int col0 = tl.nt * kUmmaN + (c >> 1) * kBoxRows + h * 64 + (c & 1) * 32;
                        uint32_t packed[16];
#pragma unroll
                        for (int i = 0; i < 32; i += 2) packed[i >> 1] = pack_bf16x2(acc[c * 32 + i], acc[c * 32 + i + 1]);
                        store_rows_staged(st.stage[warp - 4], packed,
                                          row_ok && orow_idx >= 0 ? reinterpret_cast<uint8_t*>(orow + col0) : nullptr,
                                          min(4, max(0, (I_or_H - col0 + 7) / 8)), lane);
                    }
                }
            }
        }
    }

    // ---------------------------------------------------------------- teardown
    if (*abort_flag != 0) {
        // a wait gave up: report instead of trapping, let copies in flight land, then free TMEM
        if (threadIdx.x == 0 && p.status != nullptr) {
            *reinterpret_cast<volatile int*>(p.status) = 100 + (kGated ? 0 : 10) + kMode;
            __threadfence_system();
        }
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
    ptx::tc_fence_before();
    __syncthreads();
    if constexpr (kPair) ptx::cluster_sync();  // the peer has stopped using this CTA's barriers and TMEM
    if (warp == 1) {
        ptx::tc_fence_after();
        if constexpr (kPair)
            ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
        else
            ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---------------------------------------------------------------- host side

template <bool kFp8, int kMode, bool kGated, bool kPair, int kBox, int kElem = kElemBf16>
static int launch(const CUtensorMap& ma, const CUtensorMap& mb, const Params& p, cudaStream_t stream) {
    auto kern = moe_GemmGrouped_GemmUniversal_tcgen05<kFp8, kMode, kGated, kPair, kBox, kElem>;
    // the shared-memory opt-in is per function and per device
    static std::mutex mu;
    static bool configured[kMaxDevices] = {};
    int dev = 0;
    DQ_CUDA(cudaGetDevice(&dev));
    DQ_CHECK(dev >= 0 && dev < kMaxDevices);
    {
        std::lock_guard<std::mutex> lk(mu);
        if (!configured[dev]) {
            DQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kSmemBytes)));
            configured[dev] = true;
        }
    }
    if constexpr (kPair) {
        // clusters of two CTAs on neighbouring SMs; an even grid
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(unsigned(sm_count() & ~1), 1, 1);
        cfg.blockDim = dim3(kThreads, 1, 1);
        cfg.dynamicSmemBytes = kSmemBytes;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        DQ_CUDA(cudaLaunchKernelEx(&cfg, kern, ma, mb, p));
    } else {
        kern<<<sm_count(), kThreads, kSmemBytes, stream>>>(ma, mb, p);
    }
    DQ_LAUNCH_CHECK();
    return DQMOE_OK;
}

// CTA pairs halve the weight bytes each SM stages per flop; they pay off once experts have
// several row tiles.
static bool use_pairs(int n, int E, int quant_mode) {
    // Block mode hands a TMEM buffer back every K block and is bound by that round trip, not by the
    // shared-memory traffic a pair saves (measured: +1 % with pairs, while ragged experts waste more
    // rows in 256-row tiles), so it stays on single CTAs.
    return quant_mode != DQMOE_QUANT_FP8_BLOCK && n / E >= 512;
}

// elem: element type of the unquantised path (kElemBf16 / kElemHalf / kElemF32); bias: [E, gated ? 2N : N] fp32 or nullptr.
int grouped_gemm(const void* a, const float* a_scale, const void* w, const float* w_scale, const int* offsets,
                 const int* mtile_prefix, int n, int N, int K, int E, int quant_mode, int gated, void* out,
                 float* out_scale, float* amax, const int* dest_to_src, const void* row_dst, cudaStream_t stream,
                 int elem, const float* bias) {
    DQ_CHECK(elem == kElemBf16 || ((elem == kElemHalf || elem == kElemF32) && quant_mode == DQMOE_QUANT_NONE));
    DQ_CHECK(quant_mode == DQMOE_QUANT_NONE || quant_mode == DQMOE_QUANT_FP8_TENSOR ||
             quant_mode == DQMOE_QUANT_FP8_CHANNEL || quant_mode == DQMOE_QUANT_FP8_BLOCK);
    DQ_CHECK(n >= 0 && N > 0 && K > 0 && E > 0 && E <= kMaxExperts);
    if (n == 0) return DQMOE_OK;
    const bool fp8 = quant_mode != DQMOE_QUANT_NONE;
    const int esz = fp8 ? 1 : (elem == kElemF32 ? 4 : 2);
    DQ_CHECK_FMT((size_t(K) * esz) % 16 == 0, "K=%d: rows must be a multiple of 16 bytes", K);
    DQ_CHECK_FMT(N % (gated && quant_mode == DQMOE_QUANT_FP8_BLOCK ? 16 : (elem == kElemF32 ? 4 : 8)) == 0,
                 "N=%d: output rows must be 16-byte vectors", N);
    DQ_CHECK(is_aligned(a, 16) && is_aligned(w, 16) && is_aligned(out, 16) && is_aligned(row_dst, 8));
    DQ_CHECK(a != nullptr && w != nullptr && (out != nullptr || row_dst != nullptr) && offsets != nullptr && mtile_prefix != nullptr);
    DQ_CHECK(row_dst == nullptr || !gated);
    if (fp8) DQ_CHECK(a_scale != nullptr && w_scale != nullptr);
    if (gated && quant_mode == DQMOE_QUANT_FP8_BLOCK) DQ_CHECK(out_scale != nullptr);
    if (gated && (quant_mode == DQMOE_QUANT_FP8_TENSOR || quant_mode == DQMOE_QUANT_FP8_CHANNEL)) DQ_CHECK(amax != nullptr);

    // Tile width: 256 accumulator columns, or 128 when the launch would leave many SMs without a tile.
    // The row-tile count is known only on the device; ceil(n/128) + min(E, n) - 1 bounds it.
    const bool pair = elem != kElemF32 && use_pairs(n, E, quant_mode);
    const int mtiles_max = ceil_div(n, kBM) + (E < n ? E : n) - 1;
    const int wide_tiles = mtiles_max * (gated ? ceil_div(N, kBoxRows) : ceil_div(N, kUmmaN));
    // measured on decode shapes: 128-column tiles win when 256-column tiles would fill at most half of
    // the SMs, or when there are at most two row tiles (one or two tokens); otherwise 256 columns win
    const bool narrow = quant_mode != DQMOE_QUANT_FP8_BLOCK && !pair && elem != kElemF32 &&
                        (2 * wide_tiles <= sm_count() || (mtiles_max <= 2 && wide_tiles < 2 * sm_count()));
    const int box = narrow ? 64 : kBoxRows;

    Params p;
    p.n_rows = n;
    p.N = N;
    p.K = K;
    p.E = E;
    p.w_rows = gated ? 2 * N : N;
    p.n_tiles = gated ? ceil_div(N, box) : ceil_div(N, 2 * box);
    p.tile_w_rows = gated ? box : 2 * box;
    p.box2_off = gated ? N : box;
    p.kb_count = ceil_div(K * esz, kBKBytes);
    p.offsets = offsets;
    p.mtile_prefix = mtile_prefix;
    p.sa = a_scale;
    p.sb = w_scale;
    p.out = out;
    p.out_scale = out_scale;
    p.amax = amax;
    p.bias = bias;
    p.dest_to_src = dest_to_src;
    p.row_dst = static_cast<const unsigned long long*>(row_dst);
    p.status = device_status_word();
    if (p.status == nullptr) return DQMOE_ERR_CUDA;

    CUtensorMap ma, mb;
    int rc = make_map(&ma, a, esz, uint64_t(n), uint64_t(K), kBM);
    if (rc != DQMOE_OK) return rc;
    rc = make_map(&mb, w, esz, uint64_t(E) * p.w_rows, uint64_t(K), box);
    if (rc != DQMOE_OK) return rc;

#define DQ_GEMM_LAUNCH(FP8, MODE, PAIR, BOX)                                                 \
    (gated ? launch<FP8, MODE, true, PAIR, BOX>(ma, mb, p, stream) : launch<FP8, MODE, false, PAIR, BOX>(ma, mb, p, stream))
#define DQ_GEMM_CASE(FP8, MODE)                                                              \
    return pair ? DQ_GEMM_LAUNCH(FP8, MODE, true, 128)                                        \
                : (narrow ? DQ_GEMM_LAUNCH(FP8, MODE, false, 64) : DQ_GEMM_LAUNCH(FP8, MODE, false, 128))
#define DQ_GEMM_LAUNCH_F16(PAIR, BOX)                                                          \
    (gated ? launch<false, kNone, true, PAIR, BOX, kElemHalf>(ma, mb, p, stream)                   \
           : launch<false, kNone, false, PAIR, BOX, kElemHalf>(ma, mb, p, stream))
    if (elem == kElemHalf)
        return pair ? DQ_GEMM_LAUNCH_F16(true, 128) : (narrow ? DQ_GEMM_LAUNCH_F16(false, 64) : DQ_GEMM_LAUNCH_F16(false, 128));
#undef DQ_GEMM_LAUNCH_F16
    if (elem == kElemF32)
        return gated ? launch<false, kNone, true, false, 128, kElemF32>(ma, mb, p, stream)
                     : launch<false, kNone, false, false, 128, kElemF32>(ma, mb, p, stream);
    switch (quant_mode) {
        case DQMOE_QUANT_NONE: DQ_GEMM_CASE(false, kNone);
        case DQMOE_QUANT_FP8_TENSOR: DQ_GEMM_CASE(true, kTensor);
        case DQMOE_QUANT_FP8_CHANNEL: DQ_GEMM_CASE(true, kChannel);
        default: return pair ? DQ_GEMM_LAUNCH(true, kBlock, true, 128) : DQ_GEMM_LAUNCH(true, kBlock, false, 128);
    }
#undef DQ_GEMM_CASE
#undef DQ_GEMM_LAUNCH
}

}  // namespace gemm
}  // namespace dq

extern "C" int dqmoe_grouped_gemm(const void* a, const float* a_scale, const void* w, const float* w_scale,
                                  const int32_t* offsets, const int32_t* mtile_prefix, int n, int N, int K, int E,
                                  int quant_mode, int gated, void* out, float* out_scale, float* amax,
                                  const int32_t* dest_to_src, dqmoe_stream_t stream) {
    return dq::gemm::grouped_gemm(a, a_scale, w, w_scale, offsets, mtile_prefix, n, N, K, E, quant_mode, gated, out,
                                  out_scale, amax, dest_to_src, nullptr, static_cast<cudaStream_t>(stream),
                                  dq::gemm::kElemBf16, nullptr);
}

extern "C" int dqmoe_grouped_gemm_rows(const void* a, const float* a_scale, const void* w, const float* w_scale,
                                       const int32_t* offsets, const int32_t* mtile_prefix, int n, int N, int K, int E,
                                       int quant_mode, const void* row_dst, dqmoe_stream_t stream) {
    return dq::gemm::grouped_gemm(a, a_scale, w, w_scale, offsets, mtile_prefix, n, N, K, E, quant_mode, 0, nullptr,
                                  nullptr, nullptr, nullptr, row_dst, static_cast<cudaStream_t>(stream), dq::gemm::kElemBf16,
                                  nullptr);
}
