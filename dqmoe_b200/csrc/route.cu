// Routing kernels: the top-k router and the deterministic expert sort that turns
// m_indices[T, k] into per-expert row ranges and a stable permutation.
//
// The sort replaces cub::DeviceHistogram + cub::DeviceScan + the atomic-slot
// GetGroupIndex kernel of the reference (csrc/moe_kernels.h:108-127, 452-471).
// It is a counting sort in three small launches (per-chunk histograms, one scan
// block, per-chunk scatter with warp-level match ranks) or a single launch when
// the rows fit one chunk; no atomics decide the order, so the result is the
// stable order torch.where produces (test/util.py:80).
#include <mutex>

#include "common.cuh"

namespace dq {
namespace route {

constexpr int kChunk = 2048;    // rows per sort block
constexpr int kSortThreads = 256;
constexpr int kSortWarps = kSortThreads / 32;
constexpr int kRowsPerWarp = kChunk / kSortWarps;  // 256: eight passes of 32 consecutive rows
constexpr int kMaxExperts = 1024;

__device__ __forceinline__ int bucket_of(int id, int E) { return (id >= 0 && id < E) ? id : E; }

// ---------------------------------------------------------------- pass 1: chunk histograms
__global__ void __launch_bounds__(kSortThreads) sort_hist_kernel(const int* __restrict__ ids, int n, int E,
                                                                 int* __restrict__ chunk_hist /*[chunks][E+1]*/) {
    extern __shared__ int s_hist[];  // E+1
    for (int i = threadIdx.x; i <= E; i += kSortThreads) s_hist[i] = 0;
    __syncthreads();
    const int base = blockIdx.x * kChunk;
    for (int i = threadIdx.x; i < kChunk; i += kSortThreads) {
        const int r = base + i;
        if (r < n) atomicAdd(&s_hist[bucket_of(ids[r], E)], 1);  // integer counts: order-independent
    }
    __syncthreads();
    for (int i = threadIdx.x; i <= E; i += kSortThreads) chunk_hist[size_t(blockIdx.x) * (E + 1) + i] = s_hist[i];
}

// block-wide exclusive scan of s_val[0..len) in place (len <= kMaxExperts + 1), returns the total in s_val[len]
__device__ void block_exclusive_scan(int* s_val, int len, int* s_warp_tot) {
    // each thread owns a contiguous run so that the scan is one pass
    const int nthreads = blockDim.x;
    const int per = (len + nthreads - 1) / nthreads;
    const int lo = min(threadIdx.x * per, len);
    const int hi = min(lo + per, len);
    int sum = 0;
    for (int i = lo; i < hi; ++i) sum += s_val[i];
    // exclusive scan of per-thread sums across the block
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    if (lane == 31) s_warp_tot[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        const int nw = nthreads >> 5;
        int w = lane < nw ? s_warp_tot[lane] : 0;
        int wi = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, wi, o);
            if (lane >= o) wi += v;
        }
        if (lane < nw) s_warp_tot[lane] = wi - w;
        if (lane == nw - 1) s_warp_tot[32] = wi;
    }
    __syncthreads();
    int run = s_warp_tot[warp] + incl - sum;
    for (int i = lo; i < hi; ++i) {
        const int v = s_val[i];
        s_val[i] = run;
        run += v;
    }
    __syncthreads();
    if (threadIdx.x == 0) s_val[len] = s_warp_tot[32];
    __syncthreads();
}

// ---------------------------------------------------------------- pass 2: scan
// chunk_hist becomes, per chunk and bucket, the first destination row of that chunk's rows.
// kStaged: the whole table fits shared memory and is scanned there (coalesced in, coalesced out; walking the table
// bucket by bucket in global memory is a chain of strided round trips: 15.7 us at 64 chunks x 129 buckets).
template <bool kStaged>
__global__ void __launch_bounds__(1024) sort_scan_kernel(int* __restrict__ chunk_hist, int chunks, int E,
                                                         int* __restrict__ counts, int* __restrict__ offsets,
                                                         int* __restrict__ mtile_prefix) {
    extern __shared__ int s_hist[];  // kStaged: [chunks][E + 1]
    __shared__ int s_tot[kMaxExperts + 2];
    __shared__ int s_tiles[kMaxExperts + 2];
    __shared__ int s_warp_tot[33];
    const int total = chunks * (E + 1);
    int* tab = kStaged ? s_hist : chunk_hist;
    if constexpr (kStaged) {
        for (int i = threadIdx.x; i < total; i += blockDim.x) s_hist[i] = chunk_hist[i];
        __syncthreads();
    }
    // one warp per bucket, lanes over chunks: the chunk counters of a bucket are scanned 32 at a time
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    for (int b = warp; b <= E; b += nwarps) {
        int run = 0;
        for (int c0 = 0; c0 < chunks; c0 += 32) {
            const int c = c0 + lane;
            const int v = c < chunks ? tab[size_t(c) * (E + 1) + b] : 0;
            int incl = v;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int up = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += up;
            }
            if (c < chunks) tab[size_t(c) * (E + 1) + b] = run + incl - v;
            run += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) {
            s_tot[b] = run;
            s_tiles[b] = b < E ? (run + 127) / 128 : 0;
            if (b < E && counts != nullptr) counts[b] = run;
        }
    }
    __syncthreads();
    block_exclusive_scan(s_tot, E + 1, s_warp_tot);
    block_exclusive_scan(s_tiles, E + 1, s_warp_tot);
    for (int b = threadIdx.x; b <= E; b += blockDim.x) {
        offsets[b] = s_tot[b];  // offsets[E] = number of kept rows
        if (mtile_prefix != nullptr) mtile_prefix[b] = s_tiles[b];
    }
    for (int i = threadIdx.x; i < total; i += blockDim.x) chunk_hist[i] = tab[i] + s_tot[i % (E + 1)];
}

// ---------------------------------------------------------------- pass 3: scatter
// kSingle: the whole problem is one chunk; histogram, scan and scatter in one block.
template <bool kSingle>
__global__ void __launch_bounds__(kSortThreads) sort_scatter_kernel(const int* __restrict__ ids, int n, int E,
                                                                    const int* __restrict__ chunk_base,
                                                                    int* __restrict__ counts, int* __restrict__ offsets,
                                                                    int* __restrict__ mtile_prefix,
                                                                    int* __restrict__ dest_to_src,
                                                                    int* __restrict__ src_to_dest) {
    extern __shared__ int s_mem[];
    // s_warp_hist[w][E+1]: rows of bucket b seen so far by warp w, then exclusive prefix over warps
    int* s_warp_hist = s_mem;
    int* s_base = s_mem + kSortWarps * (E + 1);  // [E+2] destination of the chunk's first row per bucket
    int* s_tiles = s_base + (E + 2);             // [E+2] (kSingle only)
    __shared__ int s_warp_tot[33];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < kSortWarps * (E + 1); i += kSortThreads) s_warp_hist[i] = 0;
    __syncthreads();

    const int base = blockIdx.x * kChunk + warp * kRowsPerWarp;
    int* my_hist = s_warp_hist + warp * (E + 1);
    int bucket[kRowsPerWarp / 32];
    int rank[kRowsPerWarp / 32];
#pragma unroll
    for (int it = 0; it < kRowsPerWarp / 32; ++it) {
        const int r = base + it * 32 + lane;
        const bool live = r < n;
        const int b = live ? bucket_of(ids[r], E) : -1;
        // lanes holding the same bucket, in row order
        const unsigned peers = __match_any_sync(0xffffffffu, b);
        const int before = __popc(peers & ((1u << lane) - 1u));
        int seen = 0;
        if (live) seen = my_hist[b];
        __syncwarp();
        if (live && before == 0) my_hist[b] = seen + __popc(peers);
        __syncwarp();
        bucket[it] = b;
        rank[it] = seen + before;
    }
    __syncthreads();
    // exclusive prefix over the warps of this block, per bucket
    for (int b = threadIdx.x; b <= E; b += kSortThreads) {
        int run = 0;
#pragma unroll
        for (int w = 0; w < kSortWarps; ++w) {
            const int v = s_warp_hist[w * (E + 1) + b];
            s_warp_hist[w * (E + 1) + b] = run;
            run += v;
        }
        if constexpr (kSingle) {
            s_base[b] = run;
            s_tiles[b] = b < E ? (run + 127) / 128 : 0;
            if (b < E && counts != nullptr) counts[b] = run;
        } else {
            s_base[b] = chunk_base[size_t(blockIdx.x) * (E + 1) + b];
        }
    }
    __syncthreads();
    if constexpr (kSingle) {
        block_exclusive_scan(s_base, E + 1, s_warp_tot);
        block_exclusive_scan(s_tiles, E + 1, s_warp_tot);
        for (int b = threadIdx.x; b <= E; b += kSortThreads) {
            offsets[b] = s_base[b];
            if (mtile_prefix != nullptr) mtile_prefix[b] = s_tiles[b];
        }
    }
#pragma unroll
    for (int it = 0; it < kRowsPerWarp / 32; ++it) {
        const int r = base + it * 32 + lane;
        if (r < n) {
            const int b = bucket[it];
            const int dest = s_base[b] + my_hist[b] + rank[it];
            if (b < E) {
                dest_to_src[dest] = r;
                if (src_to_dest != nullptr) src_to_dest[r] = dest;
            } else {
                dest_to_src[dest] = -1;  // dropped rows sort behind every expert
                if (src_to_dest != nullptr) src_to_dest[r] = -1;
            }
        }
    }
}

__global__ void mtile_prefix_kernel(const int* __restrict__ offsets, int E, int* __restrict__ mtile_prefix) {
    __shared__ int s_tiles[kMaxExperts + 2];
    __shared__ int s_warp_tot[33];
    for (int b = threadIdx.x; b <= E; b += blockDim.x) s_tiles[b] = b < E ? (offsets[b + 1] - offsets[b] + 127) / 128 : 0;
    __syncthreads();
    block_exclusive_scan(s_tiles, E + 1, s_warp_tot);
    for (int b = threadIdx.x; b <= E; b += blockDim.x) mtile_prefix[b] = s_tiles[b];
}

// out[r] = values[s] for the rows r of segment s, segments laid out back to back with
// counts[s] rows each (S <= kMaxExperts). Every block rebuilds the small prefix in shared memory.
__global__ void __launch_bounds__(256) segment_ids_kernel(const int* __restrict__ counts, const int* __restrict__ values,
                                                         int S, int* __restrict__ out, int n) {
    __shared__ int s_pref[kMaxExperts + 2];
    __shared__ int s_warp_tot[33];
    for (int i = threadIdx.x; i < S; i += blockDim.x) s_pref[i] = counts[i];
    __syncthreads();
    block_exclusive_scan(s_pref, S, s_warp_tot);  // s_pref[S] = total
    for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < n; r += gridDim.x * blockDim.x) {
        int lo = 0, hi = S;  // last segment whose start is <= r and which is not empty before r
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (s_pref[mid] <= r) lo = mid; else hi = mid;
        }
        out[r] = r < s_pref[S] ? values[lo] : -1;
    }
}

size_t sort_workspace_bytes(int n, int E) {
    const int chunks = ceil_div(n > 0 ? n : 1, kChunk);
    return align_up(size_t(chunks) * (E + 1) * sizeof(int), 256);
}

int route_sort(const int* ids, int n, int E, int* counts, int* offsets, int* mtile_prefix, int* dest_to_src,
               int* src_to_dest, void* ws, size_t ws_bytes, cudaStream_t stream) {
    DQ_CHECK(n >= 0 && E > 0 && E <= kMaxExperts);
    DQ_CHECK(offsets != nullptr);
    if (n == 0) {
        DQ_CUDA(cudaMemsetAsync(offsets, 0, (E + 1) * sizeof(int), stream));
        if (counts != nullptr) DQ_CUDA(cudaMemsetAsync(counts, 0, E * sizeof(int), stream));
        if (mtile_prefix != nullptr) DQ_CUDA(cudaMemsetAsync(mtile_prefix, 0, (E + 1) * sizeof(int), stream));
        return DQMOE_OK;
    }
    DQ_CHECK(ids != nullptr && dest_to_src != nullptr);
    const int chunks = ceil_div(n, kChunk);
    const size_t smem_scatter = (size_t(kSortWarps) * (E + 1) + 2 * (E + 2)) * sizeof(int);
    // shared-memory opt-ins are per function and per device
    constexpr int kScanSmemMax = 160 * 1024;
    static std::mutex mu;
    static bool configured[64] = {};
    int dev = 0;
    DQ_CUDA(cudaGetDevice(&dev));
    DQ_CHECK(dev >= 0 && dev < 64);
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!configured[dev]) {
            DQ_CUDA(cudaFuncSetAttribute(sort_scatter_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
            DQ_CUDA(cudaFuncSetAttribute(sort_scatter_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
            DQ_CUDA(cudaFuncSetAttribute(sort_scan_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kScanSmemMax));
            configured[dev] = true;
        }
    }
    if (chunks == 1) {
        sort_scatter_kernel<true><<<1, kSortThreads, smem_scatter, stream>>>(ids, n, E, nullptr, counts, offsets,
                                                                            mtile_prefix, dest_to_src, src_to_dest);
        DQ_LAUNCH_CHECK();
        return DQMOE_OK;
    }
    if (ws == nullptr || ws_bytes < sort_workspace_bytes(n, E) || !is_aligned(ws, 16))
        return fail(DQMOE_ERR_WORKSPACE, __FILE__, __LINE__, "ws_bytes >= sort_workspace_bytes(n, E)",
                    "sort workspace %zu bytes, need %zu", ws_bytes, sort_workspace_bytes(n, E));
    int* chunk_hist = static_cast<int*>(ws);
    sort_hist_kernel<<<chunks, kSortThreads, (E + 1) * sizeof(int), stream>>>(ids, n, E, chunk_hist);
    DQ_LAUNCH_CHECK();
    const size_t smem_scan = size_t(chunks) * (E + 1) * sizeof(int);
    if (smem_scan <= size_t(kScanSmemMax))
        sort_scan_kernel<true><<<1, 1024, smem_scan, stream>>>(chunk_hist, chunks, E, counts, offsets, mtile_prefix);
    else
        sort_scan_kernel<false><<<1, 1024, 0, stream>>>(chunk_hist, chunks, E, counts, offsets, mtile_prefix);
    DQ_LAUNCH_CHECK();
    sort_scatter_kernel<false><<<chunks, kSortThreads, smem_scatter, stream>>>(ids, n, E, chunk_hist, counts, offsets,
                                                                              mtile_prefix, dest_to_src, src_to_dest);
    DQ_LAUNCH_CHECK();
    return DQMOE_OK;
}

// ---------------------------------------------------------------- top-k router
// One warp per token. Ranking is by logit (both scoring functions are monotonic),
// value descending then expert id ascending; weights are the selected scores
// normalised to sum 1. Output rows have `slots` >= k entries: entries k.. name the shared
// experts E, E+1, ... (every token, weight 1), which the layer then treats like routed ones.
template <int kPerLane>
__global__ void __launch_bounds__(256) route_topk_kernel(const float* __restrict__ logits, int T, int E, int k,
                                                         int slots, int scoring, int* __restrict__ indices,
                                                         float* __restrict__ weights) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= T) return;
    const float* row = logits + size_t(warp) * E;
    float x[kPerLane];
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
        const int e = i * 32 + lane;
        x[i] = e < E ? row[e] : -INFINITY;
        m = fmaxf(m, x[i]);
    }
    m = warp_max(m);
    float sel_score = 0.0f;  // lane j keeps the j-th selected score
    int sel_idx = 0;
    float denom = 0.0f;
    uint32_t taken = 0;      // bit i: this lane's i-th expert has been selected (an expert is chosen at most once,
                             // also when fewer than k logits are above -inf)
    for (int j = 0; j < k; ++j) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < kPerLane; ++i) {
            const int e = i * 32 + lane;
            if (e < E && ((taken >> i) & 1u) == 0u && (x[i] > bv || (x[i] == bv && e < bi))) {
                bv = x[i];
                bi = e;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) {
                bv = ov;
                bi = oi;
            }
        }
        // remove the winner from its owner lane
#pragma unroll
        for (int i = 0; i < kPerLane; ++i)
            if (i * 32 + lane == bi) taken |= 1u << i;
        const float score = scoring == DQMOE_SCORE_SIGMOID ? 1.0f / (1.0f + expf(-bv)) : expf(bv - m);
        denom += score;
        if (lane == j) {
            sel_score = score;
            sel_idx = bi;
        }
    }
    if (lane < k) {
        indices[size_t(warp) * slots + lane] = sel_idx;
        weights[size_t(warp) * slots + lane] = sel_score / denom;
    } else if (lane < slots) {
        indices[size_t(warp) * slots + lane] = E + (lane - k);
        weights[size_t(warp) * slots + lane] = 1.0f;
    }
}

int route_topk(const float* logits, int T, int E, int k, int n_shared, int scoring, int* indices, float* weights,
               cudaStream_t stream) {
    DQ_CHECK(T >= 0 && E > 0 && E <= kMaxExperts && k > 0 && k <= 32 && k <= E);
    DQ_CHECK_FMT(n_shared >= 0 && k + n_shared <= 32 && E + n_shared <= kMaxExperts, "n_shared=%d", n_shared);
    const int slots = k + n_shared;
    DQ_CHECK(scoring == DQMOE_SCORE_SOFTMAX || scoring == DQMOE_SCORE_SIGMOID);
    if (T == 0) return DQMOE_OK;
    DQ_CHECK(logits != nullptr && indices != nullptr && weights != nullptr);
    const int blocks = ceil_div(T, 8);
    if (E <= 32) route_topk_kernel<1><<<blocks, 256, 0, stream>>>(logits, T, E, k, slots, scoring, indices, weights);
    else if (E <= 64) route_topk_kernel<2><<<blocks, 256, 0, stream>>>(logits, T, E, k, slots, scoring, indices, weights);
    else if (E <= 128) route_topk_kernel<4><<<blocks, 256, 0, stream>>>(logits, T, E, k, slots, scoring, indices, weights);
    else if (E <= 256) route_topk_kernel<8><<<blocks, 256, 0, stream>>>(logits, T, E, k, slots, scoring, indices, weights);
    else if (E <= 512) route_topk_kernel<16><<<blocks, 256, 0, stream>>>(logits, T, E, k, slots, scoring, indices, weights);
    else route_topk_kernel<32><<<blocks, 256, 0, stream>>>(logits, T, E, k, slots, scoring, indices, weights);
    DQ_LAUNCH_CHECK();
    return DQMOE_OK;
}

}  // namespace route
}  // namespace dq

extern "C" {

size_t dqmoe_route_sort_workspace_bytes(int n, int E) { return dq::route::sort_workspace_bytes(n, E); }

int dqmoe_route_sort(const int32_t* expert_ids, int n, int E, int32_t* counts, int32_t* offsets,
                     int32_t* dest_to_src, int32_t* src_to_dest, void* workspace, size_t workspace_bytes,
                     dqmoe_stream_t stream) {
    return dq::route::route_sort(expert_ids, n, E, counts, offsets, nullptr, dest_to_src, src_to_dest, workspace,
                                 workspace_bytes, static_cast<cudaStream_t>(stream));
}

int dqmoe_mtile_prefix(const int32_t* offsets, int E, int32_t* mtile_prefix, dqmoe_stream_t stream) {
    DQ_CHECK(E > 0 && E <= dq::route::kMaxExperts && offsets != nullptr && mtile_prefix != nullptr);
    dq::route::mtile_prefix_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(offsets, E, mtile_prefix);
    DQ_LAUNCH_CHECK();
    return DQMOE_OK;
}

int dqmoe_segment_ids(const int32_t* counts, const int32_t* values, int S, int32_t* out, int n,
                      dqmoe_stream_t stream) {
    DQ_CHECK(S > 0 && S <= dq::route::kMaxExperts && n >= 0);
    if (n == 0) return DQMOE_OK;
    DQ_CHECK(counts != nullptr && values != nullptr && out != nullptr);
    const int blocks = dq::ceil_div(n, 256) < dq::sm_count() * 4 ? dq::ceil_div(n, 256) : dq::sm_count() * 4;
    dq::route::segment_ids_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(counts, values, S, out, n);
    DQ_LAUNCH_CHECK();
    return DQMOE_OK;
}

int dqmoe_route_topk(const float* logits, int T, int E, int k, int scoring, int32_t* indices, float* weights,
                     dqmoe_stream_t stream) {
    return dq::route::route_topk(logits, T, E, k, 0, scoring, indices, weights, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
