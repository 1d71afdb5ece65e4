// Grouped GEMM for expert-sorted rows in the MXFP8 mode: e4m3 operands with one UE8M0 (power-of-two) scale per
// row and 32 K elements, for activations and weights alike. The scales ride inside the tensor-core instruction
// (tcgen05.mma.kind::mxf8f6f4.block_scale reads them from TMEM columns), so the fp32 accumulator stays in TMEM
// for the whole K loop: no per-128-K promotion through registers as the fp32-scaled block mode of
// gemm_sm100.cu needs. Same persistent, warp-specialised structure otherwise:
//   warp 0     TMA producer: activation rows + two weight boxes per 128-byte K stage, and the stage's three
//              512-byte scale blocks by untiled bulk copies (no cluster broadcast anywhere)
//   warp 1     MMA issuer: per stage three tcgen05.cp (scale bytes -> TMEM) and four block-scaled MMAs
//   warps 4-11 epilogue: stage 1 SwiGLU + MXFP8 re-quantisation (each thread owns whole 32-column scale groups
//              of its row), stage 2 bf16 rows scattered to d[T, k, H] or to explicit row addresses
// Scale layout in global memory ("tiled"): one 512-byte block per 128 rows and 128 K elements, holding the
// block's 128 x 4 scale bytes in the order tcgen05.cp.32x128b.warpx4 wants them in shared memory - row r of the
// block at byte (r % 32) * 16 + (r / 32) * 4, its four bytes in K order. Blocks are indexed [row block][K block].
// Weight rows form blocks by their row index; activation rows by their tile (cumulative 128-row tile of the
// expert sort + row within the expert), so that tiles of ragged experts still find their scales in whole blocks.
// (4-byte copies that built this layout in shared memory from row-major scales were measured first: they cost
// 45 % of the kernel's throughput.)
// TMEM budget: two 256-column accumulators and the scale columns do not fit 512 columns side by side, so the
// two accumulators overlap by 24 columns; the epilogue of a tile drains the chunk holding those columns first
// and signals it, and only that signal (not the whole epilogue) gates the next tile's first MMA.
// The same kernel serves the NVFP4 mode (kFp4): e2m1 operands, two per byte, with one UE4M3 scale per row and 16 K
// elements plus an fp32 global scale per tensor (per expert for the weights), on
// tcgen05.mma.kind::mxf4nvf4.block_scale.scale_vec::4X. A 128-byte K stage then holds 256 elements, an instruction
// covers K = 64 and reads four scale bytes per row, so a stage carries four 512-byte scale blocks per 128 rows (one
// per 64 K elements, same byte order) and 48 TMEM scale columns; the accumulators overlap by 96 columns, the
// epilogue multiplies by the product of the global scales and, in stage 1, re-quantises to NVFP4 with the
// caller's global scale of the intermediate. Its four stages leave no room for the per-warp store staging
// buffers, so rows are stored with 16-byte stores straight from registers.
// The reference reserves mode bits for block-scaled formats it does not implement (csrc/quantization.h:30-38)
// and names DeepGEMM as its road map (README.md:11); this mode has no counterpart kernel there.
#include "common.cuh"
#include "gemm_tile.cuh"
#include "ptx_sm100.cuh"

#include <mutex>

namespace dq {
namespace gemm_mx {

using gemm::store_rows_staged;

constexpr int kBM = 128;                 // rows per tile = UMMA M
constexpr int kBox = 128;                // weight rows per TMA box, two boxes per stage
constexpr int kN = 2 * kBox;             // 256 accumulator columns per tile
constexpr int kBK = 128;                 // K elements (= bytes) per stage: one 128-byte swizzle row, four scale groups
constexpr int kUmmaK = 32;               // K elements per tcgen05.mma = one scale group
constexpr int kStages = 4;
constexpr int kABytes = kBM * kBK;       // 16 KiB
constexpr int kBBytes = kN * kBK;        // 32 KiB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kSfBlock = 512;            // scale bytes of 128 rows x 4 groups, in tcgen05.cp order
constexpr int kThreads = 384;
constexpr int kRegsControl = 56;
constexpr int kRegsEpilogue = 224;
constexpr int kEpiWarps = 8;
constexpr int kMaxExperts = 1024;
constexpr int kMaxDevices = 64;
constexpr int kTmemCols = 512;

// What differs between the two formats
template <bool kFp4>
struct Fmt {
    static constexpr int kSfAtoms = kFp4 ? 4 : 1;                 // 512-byte scale blocks per 128 rows and stage
    static constexpr int kSfStage = 3 * kSfAtoms * kSfBlock;      // activation rows, first weight box, second weight box
    static constexpr int kSfCols = 12 * kSfAtoms;                 // TMEM columns of a stage's scales: (4 (A) + 8 (B)) per block
    static constexpr int kSfCol = kTmemCols - 2 * kSfCols;        // two alternating sets at the top: 488 / 416
    static constexpr int kAccCol1 = kSfCol - kN;                  // second accumulator [232, 488) / [160, 416); the first is [0, 256)
    static constexpr int kStageElems = kFp4 ? 2 * kBK : kBK;      // K elements per 128-byte stage
    static constexpr bool kStaged = !kFp4;                        // rows leave through the per-warp staging buffers
    static constexpr int kOverlapWarps = kFp4 ? kEpiWarps : 4;    // epilogue warps that own columns the accumulators share
};
constexpr long long kWaitLimit = 1000000000LL;  // clock cycles before a wait gives up (~0.5 s)

struct Params {
    int n_rows, N, K, E;
    int n_tiles;         // column tiles per row tile
    int w_rows;          // weight rows per expert (stage 1: 2I, stage 2: H)
    int tile_w_rows;     // weight rows advanced per column tile (stage 1: 128, stage 2: 256)
    int box2_off;        // row offset of the second weight box (stage 1: I, stage 2: 128)
    int kb_count;        // K stages: K / 128 (MXFP8), K / 256 (NVFP4)
    const int* offsets;
    const int* mtile_prefix;
    int w_blocks;        // E * w_rows / 128: 128-row blocks of the weight scales
    const uint8_t* sfa;  // tiled UE8M0 scales of the activations: [row tiles][K/128][512]
    const uint8_t* sfb;  // tiled UE8M0 scales of the weights: [E * w_rows / 128][K/128][512]
    void* out;
    uint8_t* out_sf;     // stage 1: tiled scales of the output, [row tiles][N/128][512]
    const float* bias;   // [E, w_rows] fp32 or nullptr
    const float* ga;     // NVFP4: global scale of the activations (1 float)
    const float* gw;     // NVFP4: global scale of every expert's weights [E]
    const float* gout;   // NVFP4 stage 1: global scale of the re-quantised intermediate (1 float)
    const int* dest_to_src;
    const unsigned long long* row_dst;
    int* status;
};

template <bool kFp4>
struct Shared {
    uint64_t full[kStages];     // operands and scale blocks of a stage have landed
    uint64_t empty[kStages];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint64_t overlap_free[2];   // the columns a buffer shares with the other one have been drained
    uint32_t tmem_base;
    int abort_flag;
    alignas(128) uint8_t sf[kStages][Fmt<kFp4>::kSfStage];
    uint4 stage[Fmt<kFp4>::kStaged ? kEpiWarps : 1][Fmt<kFp4>::kStaged ? 32 * 4 : 1];  // per-warp store staging (MXFP8)
    int mprefix[kMaxExperts + 1];
    int offsets[kMaxExperts + 1];
};

template <bool kFp4>
constexpr size_t smem_bytes() { return 1024 + size_t(kStages) * kStageBytes + sizeof(Shared<kFp4>); }
static_assert(smem_bytes<false>() <= 227 * 1024 && smem_bytes<true>() <= 227 * 1024, "shared memory of a block");

struct Tile {
    int e, row0, row_end, nt;
    int mtile;  // index of the row tile among all row tiles of the expert sort
};
template <class SharedT>
__device__ __forceinline__ Tile decode_tile(int t, int& e_cursor, const SharedT& st, int n_tiles) {
    while (t >= st.mprefix[e_cursor + 1] * n_tiles) ++e_cursor;
    const int local = t - st.mprefix[e_cursor] * n_tiles;
    const int mtiles = st.mprefix[e_cursor + 1] - st.mprefix[e_cursor];
    Tile tl;
    tl.e = e_cursor;
    tl.nt = local / mtiles;
    tl.mtile = st.mprefix[e_cursor] + local % mtiles;
    tl.row0 = st.offsets[e_cursor] + (local % mtiles) * kBM;
    tl.row_end = st.offsets[e_cursor + 1];
    return tl;
}

// UE8M0 scale of a 32-value group from its amax: the smallest power of two s with amax / s <= 448
// (s = 2^ceil(log2(max(amax, 1e-4) / 448))), returned as the biased exponent byte; *inv = 1 / s exactly.
__device__ __forceinline__ uint32_t mx_scale_byte(float amax, float* inv) {
    const float s = __fdiv_rn(fmaxf(amax, 1e-4f), 448.0f);
    const uint32_t bits = __float_as_uint(s);
    const uint32_t e = (bits >> 23) + ((bits & 0x7fffffu) != 0u ? 1u : 0u);  // s > 0: no sign bit
    *inv = __uint_as_float((254u - e) << 23);                               // 2^(127 - e)
    return e;
}

template <bool kGated, bool kFp4>
__global__ void __launch_bounds__(kThreads, 1)
moe_GemmGrouped_GemmUniversal_tcgen05_mx(const __grid_constant__ CUtensorMap tma_a,
                                         const __grid_constant__ CUtensorMap tma_b, const Params p) {
    using F = Fmt<kFp4>;
    constexpr int kSfAtoms = F::kSfAtoms, kSfStage = F::kSfStage, kSfCols = F::kSfCols, kSfCol = F::kSfCol,
                  kAccCol1 = F::kAccCol1;
    constexpr int kSfPart = kSfAtoms * kSfBlock;  // scale bytes of 128 rows and one stage
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    Shared<kFp4>& st = *reinterpret_cast<Shared<kFp4>*>(smem + size_t(kStages) * kStageBytes);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            ptx::mbar_init(&st.full[s], 1);
            ptx::mbar_init(&st.empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(&st.tmem_full[b], 1);
            ptx::mbar_init(&st.tmem_empty[b], kEpiWarps);
            ptx::mbar_init(&st.overlap_free[b], F::kOverlapWarps);  // the warps that own the shared columns
        }
        st.abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async();
    }
    if (warp == 1) {
        ptx::tmem_alloc(&st.tmem_base, kTmemCols);
        ptx::tmem_relinquish();
    }
    for (int i = threadIdx.x; i <= p.E; i += kThreads) {
        st.mprefix[i] = p.mtile_prefix[i];
        st.offsets[i] = p.offsets[i];
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();

    const uint32_t tmem_base = st.tmem_base;
    const int total_tiles = st.mprefix[p.E] * p.n_tiles;
    volatile int* abort_flag = &st.abort_flag;
    const int kb_count = p.kb_count;
    const int tile_first = int(blockIdx.x), tile_step = int(gridDim.x);

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
                const Tile tl = decode_tile(t, e_cursor, st, p.n_tiles);
                const int wrow0 = tl.e * p.w_rows + tl.nt * p.tile_w_rows;
                const int wrow1 = wrow0 + p.box2_off;
                const uint8_t* sf_a = p.sfa + size_t(tl.mtile) * kb_count * kSfPart;
                const uint8_t* sf_b0 = p.sfb + size_t(min(wrow0 >> 7, p.w_blocks - 1)) * kb_count * kSfPart;
                const uint8_t* sf_b1 = p.sfb + size_t(min(wrow1 >> 7, p.w_blocks - 1)) * kb_count * kSfPart;
                for (int kb = 0; kb < kb_count; ++kb, ++it) {
                    const int s = it % kStages;
                    if (!ptx::mbar_wait(&st.empty[s], ((it / kStages) & 1u) ^ 1u, abort_flag, kWaitLimit)) {
                        ok = false;
                        break;
                    }
                    uint8_t* sa = smem + size_t(s) * kStageBytes;
                    uint8_t* sb = sa + kABytes;
                    ptx::mbar_arrive_expect_tx(&st.full[s], kStageBytes + kSfStage);
                    ptx::tma_load_2d(sa, &tma_a, kb * kBK, tl.row0, &st.full[s]);
                    ptx::tma_load_2d(sb, &tma_b, kb * kBK, wrow0, &st.full[s]);
                    ptx::tma_load_2d(sb + kBox * kBK, &tma_b, kb * kBK, wrow1, &st.full[s]);
                    ptx::bulk_load(&st.sf[s][0], sf_a + size_t(kb) * kSfPart, kSfPart, &st.full[s]);
                    ptx::bulk_load(&st.sf[s][kSfPart], sf_b0 + size_t(kb) * kSfPart, kSfPart, &st.full[s]);
                    ptx::bulk_load(&st.sf[s][2 * kSfPart], sf_b1 + size_t(kb) * kSfPart, kSfPart, &st.full[s]);
                }
            }
        }
        __syncwarp();
      } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = kFp4 ? ptx::make_idesc_nvf4(kBM, kN) : ptx::make_idesc_mx(kBM, kN);
            uint32_t it = 0;
            uint32_t acc_it = 0;
            bool ok = true;
            for (int t = tile_first; ok && t < total_tiles; t += tile_step, ++acc_it) {
                const uint32_t buf = acc_it & 1u;
                // this buffer's previous tile is drained, and the other buffer's tile (the one just before this)
                // has given up the columns the two share
                if (!ptx::mbar_wait(&st.tmem_empty[buf], ((acc_it >> 1) & 1u) ^ 1u, abort_flag, kWaitLimit)) break;
                if (acc_it > 0 &&
                    !ptx::mbar_wait(&st.overlap_free[buf ^ 1u], ((acc_it - 1) >> 1) & 1u, abort_flag, kWaitLimit))
                    break;
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + (buf ? kAccCol1 : 0);
                for (int kb = 0; kb < kb_count; ++kb, ++it) {
                    const int s = it % kStages;
                    if (!ptx::mbar_wait(&st.full[s], (it / kStages) & 1u, abort_flag, kWaitLimit)) {
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
                    const uint32_t a_addr = ptx::smem_u32(smem + size_t(s) * kStageBytes);
                    const uint32_t b_addr = a_addr + kABytes;
                    const uint32_t sf_addr = ptx::smem_u32(&st.sf[s][0]);
                    const uint32_t sf_col = tmem_base + kSfCol + (it & 1u) * kSfCols;
                    // scale bytes of this stage -> TMEM (executed in order with the MMAs around them). MXFP8: one block
                    // per 128 rows serves the stage's four instructions (byte k of a column each); NVFP4: block k
                    // serves instruction k, the weights' two 128-row blocks side by side in 8 columns.
#pragma unroll
                    for (int k = 0; k < kSfAtoms; ++k) {
                        const uint32_t col_b = sf_col + (kFp4 ? 16 + 8 * k : 4);
                        ptx::tmem_cp_sf(sf_col + 4 * k, ptx::smem_desc_sf(sf_addr + k * kSfBlock));
                        ptx::tmem_cp_sf(col_b, ptx::smem_desc_sf(sf_addr + kSfPart + k * kSfBlock));
                        ptx::tmem_cp_sf(col_b + 4, ptx::smem_desc_sf(sf_addr + 2 * kSfPart + k * kSfBlock));
                    }
#pragma unroll
                    for (int k = 0; k < kBK / kUmmaK; ++k) {
                        const uint64_t da = ptx::smem_desc_sw128(a_addr + k * kUmmaK), db = ptx::smem_desc_sw128(b_addr + k * kUmmaK);
                        if constexpr (kFp4)
                            ptx::umma_nvf4(d_tmem, da, db, idesc, sf_col + 4 * k, sf_col + 16 + 8 * k, (kb | k) != 0 ? 1u : 0u);
                        else
                            ptx::umma_mx(d_tmem, da, db, ptx::idesc_mx_with_sf_id(idesc, k), sf_col, sf_col + 4,
                                         (kb | k) != 0 ? 1u : 0u);
                    }
                    ptx::umma_commit(&st.empty[s]);
                }
                if (!ok) break;
                ptx::umma_commit(&st.tmem_full[buf]);
            }
        }
        __syncwarp();
      }
    } else {
        ptx::setmaxnreg_inc<kRegsEpilogue>();
        // ------------------------------------------------------------ epilogue warps
        const int q = warp & 3;            // TMEM lane quarter this warp may read
        const int h = (warp - 4) >> 2;     // which 64-column half of each 128-column group
        const int r_in_tile = q * 32 + lane;
        const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
        uint32_t acc_it = 0;
        int e_cursor = 0;
        bool ok = true;
        const int N = p.N;
        uint4* stage_buf = st.stage[F::kStaged ? warp - 4 : 0];  // MXFP8 only
        float* csw = reinterpret_cast<float*>(stage_buf);
        const float4* cs4 = reinterpret_cast<const float4*>(stage_buf);

        for (int t = tile_first; ok && t < total_tiles; t += tile_step, ++acc_it) {
            const Tile tl = decode_tile(t, e_cursor, st, p.n_tiles);
            const int grow = tl.row0 + r_in_tile;
            const bool row_ok = grow < tl.row_end;
            const uint32_t buf = acc_it & 1u;
            if (!ptx::mbar_wait(&st.tmem_full[buf], (acc_it >> 1) & 1u, abort_flag, kWaitLimit)) {
                ok = false;
                break;
            }
            ptx::tc_fence_after();
            const uint32_t t_buf = t_lane + (buf ? kAccCol1 : 0);
            // The columns shared with the other buffer are the last ones of buffer 0 and the first ones of buffer 1.
            // MXFP8 (24 columns): the chunk order starts there, and the warps that own the chunk holding them (h = 1
            // for buffer 0, h = 0 for buffer 1) report once it is drained. NVFP4 (96 columns, every warp owns some):
            // see below.
            const bool owns_overlap = h == (buf == 0u ? 1 : 0);
            const bool has_bias = p.bias != nullptr;
            const float* bias_e = has_bias ? p.bias + size_t(tl.e) * p.w_rows : nullptr;
            auto overlap_drained = [&](int chunks_done) {
                if (owns_overlap && chunks_done == 1) {
                    ptx::tc_fence_before();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(&st.overlap_free[buf]);
                }
            };

            if constexpr (kFp4) {
                // Both NVFP4 epilogues read this warp's 128 accumulator columns into registers first and hand the
                // buffer back at once - the shared columns to the other buffer's next tile, the whole buffer to the
                // tile after - so that all arithmetic and all stores overlap the tensor core's next tiles.
                uint32_t r[4][32];
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    ptx::tmem_ld32(t_buf + (c >> 1) * kBox + h * 64 + (c & 1) * 32, r[c]);
#pragma unroll
                for (int c = 0; c < 4; ++c) ptx::tmem_wait_ld(r[c]);
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    ptx::mbar_arrive(&st.overlap_free[buf]);
                    ptx::mbar_arrive(&st.tmem_empty[buf]);
                }
                const float alpha = p.ga[0] * p.gw[tl.e];
                if constexpr (kGated) {
                    // r[j] = gate, r[2 + j] = value of act columns nt*128 + h*64 + j*32 + [0, 32): four scale groups
                    // of 16 per thread and row, packed two values per byte
                    const float gout = p.gout[0];
                    uint32_t sf_bytes = 0;
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const int col0 = tl.nt * kBox + h * 64 + j * 32;
                        float act[32];
                        float amax[2] = {0.0f, 0.0f};
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const float bg = has_bias ? __ldg(bias_e + col0 + i) : 0.0f;
                            const float bv = has_bias ? __ldg(bias_e + N + col0 + i) : 0.0f;
                            const float gate = bf_round_cvt(__uint_as_float(r[j][i]) * alpha + bg);
                            const float val = bf_round_cvt(__uint_as_float(r[2 + j][i]) * alpha + bv);
                            act[i] = bf_round_cvt(bf_round_cvt(__fdividef(gate, 1.0f + __expf(-gate))) * val);
                            amax[i >> 4] = fmaxf(amax[i >> 4], fabsf(act[i]));
                        }
                        uint32_t w4[4];
#pragma unroll
                        for (int b = 0; b < 2; ++b) {
                            float inv;
                            sf_bytes |= nvfp4_scale_byte(amax[b], gout, &inv) << (16 * j + 8 * b);
#pragma unroll
                            for (int hf = 0; hf < 2; ++hf) {
                                float x8[8];
#pragma unroll
                                for (int i = 0; i < 8; ++i) x8[i] = act[16 * b + 8 * hf + i] * inv;
                                w4[2 * b + hf] = f2e2m1x8(x8);
                            }
                        }
                        if (row_ok)
                            st16(static_cast<uint8_t*>(p.out) + (size_t(grow) * N + col0) / 2, Vec16{w4[0], w4[1], w4[2], w4[3]});
                    }
                    // scale bytes of this row's four groups into the tile's block of the next GEMM's 64-wide K block
                    *reinterpret_cast<uint32_t*>(p.out_sf + (size_t(tl.mtile) * (N / 64) + tl.nt * 2 + h) * kSfBlock +
                                                 (r_in_tile & 31) * 16 + (r_in_tile >> 5) * 4) = sf_bytes;
                } else {
                    int orow_idx = grow;
                    if (row_ok && p.dest_to_src != nullptr) orow_idx = p.dest_to_src[grow];
                    uint8_t* orow = static_cast<uint8_t*>(p.out) + size_t(orow_idx) * N * 2;
                    if (p.row_dst != nullptr) {
                        orow = row_ok ? reinterpret_cast<uint8_t*>(p.row_dst[grow]) : nullptr;
                        orow_idx = orow != nullptr ? 0 : -1;
                    }
                    if (row_ok && orow_idx >= 0) {
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            const int col0 = tl.nt * kN + (c >> 1) * kBox + h * 64 + (c & 1) * 32;
#pragma unroll
                            for (int i = 0; i < 32; i += 8) {
                                if (col0 + i < N) {
                                    float y[8];
#pragma unroll
                                    for (int u = 0; u < 8; ++u)
                                        y[u] = __uint_as_float(r[c][i + u]) * alpha +
                                               (has_bias ? __ldg(bias_e + min(col0 + i + u, N - 1)) : 0.0f);
                                    st16(orow + size_t(col0 + i) * 2, Vec16{pack_bf16x2(y[0], y[1]), pack_bf16x2(y[2], y[3]),
                                                                          pack_bf16x2(y[4], y[5]), pack_bf16x2(y[6], y[7])});
                                }
                            }
                        }
                    }
                }
                continue;  // the buffer has been handed back above
            } else if constexpr (kGated) {
                // act columns nt*128 + h*64 + [0, 64): two scale groups of 32
                uint32_t pk[2][8];   // e4m3 bytes of the two groups in the order they were drained
                uint32_t sf_bytes = 0;
#pragma unroll
                for (int jj = 0; jj < 2; ++jj) {
                    const int j = buf == 0u ? 1 - jj : jj;
                    uint32_t g[32], v[32];
                    const int c0 = h * 64 + j * 32;
                    ptx::tmem_ld32(t_buf + c0, g);
                    ptx::tmem_ld32(t_buf + kBox + c0, v);
                    const int col0 = tl.nt * kBox + c0;
                    if (has_bias) {
                        __syncwarp();
                        const int c = min(col0 + lane, N - 1);
                        csw[lane] = bias_e[c];
                        csw[32 + lane] = bias_e[N + c];
                        __syncwarp();
                    }
                    ptx::tmem_wait_ld(g);
                    ptx::tmem_wait_ld(v);
                    overlap_drained(jj + 1);
                    float act[32];
                    float amax = 0.0f;
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        float bg[4] = {0.0f, 0.0f, 0.0f, 0.0f}, bv[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                        if (has_bias) {
                            const float4 a = cs4[i >> 2], b = cs4[8 + (i >> 2)];
                            bg[0] = a.x, bg[1] = a.y, bg[2] = a.z, bg[3] = a.w;
                            bv[0] = b.x, bv[1] = b.y, bv[2] = b.z, bv[3] = b.w;
                        }
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            // roundings as in the fp32-scaled block mode: product, silu and their product to bf16
                            const float gate = bf_round_cvt(__uint_as_float(g[i + u]) + bg[u]);
                            const float val = bf_round_cvt(__uint_as_float(v[i + u]) + bv[u]);
                            float a = bf_round_cvt(bf_round_cvt(__fdividef(gate, 1.0f + __expf(-gate))) * val);
                            if (col0 + i + u >= N) a = 0.0f;
                            act[i + u] = a;
                            amax = fmaxf(amax, fabsf(a));
                        }
                    }
                    float inv;
                    const uint32_t e8 = mx_scale_byte(amax, &inv);
                    sf_bytes |= e8 << (8 * j);
#pragma unroll
                    for (int i = 0; i < 32; i += 4)
                        pk[jj][i >> 2] = f2e4m3x4(act[i] * inv, act[i + 1] * inv, act[i + 2] * inv, act[i + 3] * inv);
                }
                uint32_t packed[16];  // back into column order (buffer 0 drains its second group first)
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    packed[i] = buf == 0u ? pk[1][i] : pk[0][i];
                    packed[8 + i] = buf == 0u ? pk[0][i] : pk[1][i];
                }
                const int colh = tl.nt * kBox + h * 64;
                store_rows_staged(stage_buf, packed,
                                  row_ok ? static_cast<uint8_t*>(p.out) + size_t(grow) * N + colh : nullptr,
                                  min(4, max(0, (N - colh + 15) / 16)), lane);
                // scale bytes of this row's two groups into the tile's block of the next GEMM's K block nt (written for
                // all 128 rows of the tile: the block belongs to this tile alone)
                *reinterpret_cast<uint16_t*>(p.out_sf + (size_t(tl.mtile) * (N / 128) + tl.nt) * kSfBlock + (r_in_tile & 31) * 16 +
                                             (r_in_tile >> 5) * 4 + h * 2) = uint16_t(sf_bytes);
            } else {
                int orow_idx = grow;
                if (row_ok && p.dest_to_src != nullptr) orow_idx = p.dest_to_src[grow];
                uint8_t* orow = static_cast<uint8_t*>(p.out) + size_t(orow_idx) * N * 2;
                if (p.row_dst != nullptr) {  // rows go to explicit addresses (expert parallel: the home rank's output)
                    orow = row_ok ? reinterpret_cast<uint8_t*>(p.row_dst[grow]) : nullptr;
                    orow_idx = orow != nullptr ? 0 : -1;
                }
#pragma unroll 1
                for (int cc = 0; cc < 4; ++cc) {
                    const int c = buf == 0u ? 3 - cc : cc;
                    uint32_t r[32];
                    const int tc = (c >> 1) * kBox + h * 64 + (c & 1) * 32;
                    ptx::tmem_ld32(t_buf + tc, r);
                    const int col0 = tl.nt * kN + tc;
                    if (has_bias) {
                        __syncwarp();
                        csw[lane] = bias_e[min(col0 + lane, N - 1)];
                        __syncwarp();
                    }
                    ptx::tmem_wait_ld(r);
                    overlap_drained(cc + 1);
                    uint32_t packed[16];
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        float bb[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                        if (has_bias) {
                            const float4 a = cs4[i >> 2];
                            bb[0] = a.x, bb[1] = a.y, bb[2] = a.z, bb[3] = a.w;
                        }
                        packed[i >> 1] = pack_bf16x2(__uint_as_float(r[i]) + bb[0], __uint_as_float(r[i + 1]) + bb[1]);
                        packed[(i >> 1) + 1] = pack_bf16x2(__uint_as_float(r[i + 2]) + bb[2], __uint_as_float(r[i + 3]) + bb[3]);
                    }
                    store_rows_staged(stage_buf, packed,
                                      row_ok && orow_idx >= 0 ? orow + size_t(col0) * 2 : nullptr,
                                      min(4, max(0, (N - col0 + 7) / 8)), lane);
                }
            }
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&st.tmem_empty[buf]);
        }
    }

    // ---------------------------------------------------------------- teardown
    if (*abort_flag != 0) {
        // a wait gave up: report instead of trapping, let copies in flight land, then free TMEM
        if (threadIdx.x == 0 && p.status != nullptr) {
            *reinterpret_cast<volatile int*>(p.status) = 120 + (kGated ? 0 : 10) + 4;
            __threadfence_system();
        }
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
}

template <bool kGated, bool kFp4>
static int launch(const CUtensorMap& ma, const CUtensorMap& mb, const Params& p, cudaStream_t stream) {
    auto kern = moe_GemmGrouped_GemmUniversal_tcgen05_mx<kGated, kFp4>;
    static std::mutex mu;
    static bool configured[kMaxDevices] = {};
    int dev = 0;
    DQ_CUDA(cudaGetDevice(&dev));
    DQ_CHECK(dev >= 0 && dev < kMaxDevices);
    {
        std::lock_guard<std::mutex> lk(mu);
        if (!configured[dev]) {
            DQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem_bytes<kFp4>())));
            configured[dev] = true;
        }
    }
    kern<<<sm_count(), kThreads, smem_bytes<kFp4>(), stream>>>(ma, mb, p);
    DQ_LAUNCH_CHECK();
    return DQMOE_OK;
}

// fp4 = false: MXFP8 (a, w e4m3; scales UE8M0 per 32). fp4 = true: NVFP4 (a, w e2m1 pairs; scales UE4M3 per 16;
// ga / gw / gout the global scales). K and N count elements.
int grouped_gemm_mx(const void* a, const uint8_t* a_sf, const void* w, const uint8_t* w_sf, const int* offsets,
                    const int* mtile_prefix, int n, int N, int K, int E, int gated, void* out, uint8_t* out_sf,
                    const int* dest_to_src, const void* row_dst, const float* bias, bool fp4, const float* ga,
                    const float* gw, const float* gout, cudaStream_t stream) {
    DQ_CHECK(n >= 0 && N > 0 && K > 0 && E > 0 && E <= kMaxExperts);
    if (n == 0) return DQMOE_OK;
    const char* mode = fp4 ? "NVFP4" : "MXFP8";
    const int stage_elems = fp4 ? Fmt<true>::kStageElems : Fmt<false>::kStageElems;
    DQ_CHECK_FMT(K % stage_elems == 0, "K=%d: the %s mode needs the reduction length to be a multiple of %d", K, mode, stage_elems);
    DQ_CHECK_FMT(N % 128 == 0, "N=%d: the %s mode needs a multiple of 128 output columns", N, mode);
    DQ_CHECK(a != nullptr && w != nullptr && a_sf != nullptr && w_sf != nullptr && offsets != nullptr && mtile_prefix != nullptr);
    DQ_CHECK((out != nullptr || row_dst != nullptr) && (row_dst == nullptr || !gated));
    DQ_CHECK(is_aligned(a, 16) && is_aligned(w, 16) && is_aligned(out, 16) && is_aligned(row_dst, 8) && is_aligned(a_sf, 16) &&
             is_aligned(w_sf, 16));
    if (gated) DQ_CHECK(out_sf != nullptr && is_aligned(out_sf, 16));
    if (fp4) DQ_CHECK(ga != nullptr && gw != nullptr && (!gated || gout != nullptr));
    Params p;
    p.n_rows = n;
    p.N = N;
    p.K = K;
    p.E = E;
    p.w_rows = gated ? 2 * N : N;
    p.n_tiles = gated ? ceil_div(N, kBox) : ceil_div(N, kN);
    p.tile_w_rows = gated ? kBox : kN;
    p.box2_off = gated ? N : kBox;
    p.kb_count = K / stage_elems;
    DQ_CHECK_FMT(p.w_rows % 128 == 0, "N=%d: weight rows per expert must be a multiple of 128 in the %s mode", N, mode);
    p.w_blocks = int(int64_t(E) * p.w_rows / 128);
    p.offsets = offsets;
    p.mtile_prefix = mtile_prefix;
    p.sfa = a_sf;
    p.sfb = w_sf;
    p.out = out;
    p.out_sf = out_sf;
    p.bias = bias;
    p.ga = ga;
    p.gw = gw;
    p.gout = gout;
    p.dest_to_src = dest_to_src;
    p.row_dst = static_cast<const unsigned long long*>(row_dst);
    p.status = device_status_word();
    if (p.status == nullptr) return DQMOE_ERR_CUDA;
    const uint64_t row_bytes = fp4 ? uint64_t(K) / 2 : uint64_t(K);  // both formats as byte matrices
    CUtensorMap ma, mb;
    int rc = gemm::make_map(&ma, a, 1, uint64_t(n), row_bytes, kBM);
    if (rc != DQMOE_OK) return rc;
    rc = gemm::make_map(&mb, w, 1, uint64_t(E) * p.w_rows, row_bytes, kBox);
    if (rc != DQMOE_OK) return rc;
    if (fp4) return gated ? launch<true, true>(ma, mb, p, stream) : launch<false, true>(ma, mb, p, stream);
    return gated ? launch<true, false>(ma, mb, p, stream) : launch<false, false>(ma, mb, p, stream);
}

}  // namespace gemm_mx
}  // namespace dq

extern "C" int dqmoe_grouped_gemm_mx(const void* a, const uint8_t* a_sf, const void* w, const uint8_t* w_sf,
                                     const int32_t* offsets, const int32_t* mtile_prefix, int n, int N, int K, int E,
                                     int gated, void* out, uint8_t* out_sf, const int32_t* dest_to_src,
                                     dqmoe_stream_t stream) {
    return dq::gemm_mx::grouped_gemm_mx(a, a_sf, w, w_sf, offsets, mtile_prefix, n, N, K, E, gated, out, out_sf,
                                        dest_to_src, nullptr, nullptr, false, nullptr, nullptr, nullptr,
                                        static_cast<cudaStream_t>(stream));
}

extern "C" int dqmoe_grouped_gemm_mx_rows(const void* a, const uint8_t* a_sf, const void* w, const uint8_t* w_sf,
                                          const int32_t* offsets, const int32_t* mtile_prefix, int n, int N, int K, int E,
                                          const void* row_dst, dqmoe_stream_t stream) {
    return dq::gemm_mx::grouped_gemm_mx(a, a_sf, w, w_sf, offsets, mtile_prefix, n, N, K, E, 0, nullptr, nullptr, nullptr,
                                        row_dst, nullptr, false, nullptr, nullptr, nullptr, static_cast<cudaStream_t>(stream));
}

extern "C" int dqmoe_grouped_gemm_nvfp4(const void* a, const uint8_t* a_sf, const float* a_gscale, const void* w,
                                        const uint8_t* w_sf, const float* w_gscale, const int32_t* offsets,
                                        const int32_t* mtile_prefix, int n, int N, int K, int E, int gated, void* out,
                                        uint8_t* out_sf, const float* out_gscale, const int32_t* dest_to_src,
                                        dqmoe_stream_t stream) {
    return dq::gemm_mx::grouped_gemm_mx(a, a_sf, w, w_sf, offsets, mtile_prefix, n, N, K, E, gated, out, out_sf,
                                        dest_to_src, nullptr, nullptr, true, a_gscale, w_gscale, out_gscale,
                                        static_cast<cudaStream_t>(stream));
}
