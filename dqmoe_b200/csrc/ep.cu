// Expert-parallel exchange over peer memory (NVLink P2P loads/stores; no NCCL on the data
// path, no multicast). Every rank maps the same set of buffers of every other rank
// ("symmetric" buffers); a layer call is
//   publish   my per-expert row counts -> every peer's count matrix, then a flag
//   plan      wait for all count rows; compute where my rows go in each owner's receive
//             buffer (already grouped by expert there) and my own receive offsets
//   dispatch  gather my rows (+ scales, + their home slot) straight into the owners' buffers
//   wait      until every source has signalled its rows
//   row_ptrs  destination address of each received row's result in its home rank's output
//   [grouped fc1 / fc2 run on the receive buffer; fc2's epilogue stores through row_ptrs]
//   signal + wait   results have landed in every home rank
// Flags carry a per-call epoch, so nothing is reset between calls. Every wait is bounded: a
// wait that gives up writes the device status word and returns (no trap, no hang).
// The reference has no multi-GPU path; this extends its layer (csrc/moe_kernels.h:770-892).
#include <atomic>

#include "common.cuh"

namespace dq {
namespace ep {

constexpr int kMaxRanks = 8;
constexpr int kMaxExperts = 1024;
constexpr long long kDefaultWaitLimit = 20000000000LL;  // cycles (~10 s): peers may be late on the host side

// Cycles a flag wait may spin before it gives up; process-wide, set by dqmoe_ep_set_wait_limit and
// handed to every kernel as an argument at launch.
static std::atomic<long long> g_wait_limit{kDefaultWaitLimit};
static long long wait_limit() { return g_wait_limit.load(std::memory_order_relaxed); }

struct Peers {
    void* p[kMaxRanks];
};

// Flags cross GPUs, so their loads and stores are system scope. System-scope fences and acquire / release accesses
// are the expensive part (measured: an exchange whose flag traffic overlaps large host copies over PCIe gets 0.3-0.4 ms
// slower per call, a device-to-device copy of the same size does nothing), so each hand-over uses exactly one fence:
// writers fence once and then store the flags relaxed, readers poll relaxed and fence once after the last flag.
__device__ __forceinline__ int ld_relaxed_sys(const int* p) {
    int v;
    asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_sys(int* p, int v) {
    asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// bounded wait until flag == epoch; false (and status written) when it gives up. The caller fences
// (__threadfence_system) after all its flags have arrived, before it reads what the flags announce.
__device__ bool wait_flag(const int* flag, int epoch, int* status, int code, long long limit) {
    const long long t0 = clock64();
    unsigned spins = 0;
    while (ld_relaxed_sys(flag) != epoch) {
        if (((++spins) & 0x3f) == 0) {
            __nanosleep(200);
            if (clock64() - t0 > limit) {
                if (status != nullptr) {
                    *reinterpret_cast<volatile int*>(status) = code;
                    __threadfence_system();
                }
                return false;
            }
        }
    }
    return true;
}

// flags: int[3][kMaxRanks] per rank: [phase][source rank]
__global__ void __launch_bounds__(256) publish_counts_kernel(const int* __restrict__ counts, int E, int me, int W,
                                                             Peers cnt, Peers flags, int epoch) {
    for (int p = 0; p < W; ++p) {
        int* dst = static_cast<int*>(cnt.p[p]) + size_t(me) * E;
        for (int e = threadIdx.x; e < E; e += blockDim.x) dst[e] = counts[e];
    }
    __threadfence();   // every thread's count stores, visible on this GPU ...
    __syncthreads();
    if (threadIdx.x < W) {
        __threadfence_system();  // ... and ordered before the flag at system scope by the flag's writer
        st_relaxed_sys(static_cast<int*>(flags.p[threadIdx.x]) + 0 * kMaxRanks + me, epoch);
    }
}

// One block. cnt: my copy of the count matrix [W][E]. Outputs (all local):
//   send_base[e]      e < E: row in the owner's receive buffer where my rows of expert e start
//   send_base[E]      (one more word) 0, or 1 when the plan is void: the counts never arrived, or some rank
//                     would receive more than `cap` rows
//   rx_offsets[El+1]  first received row of each of my experts (sum over sources), [El] = rows received
//   rx_mtiles[El+1]   cumulative 128-row tiles of my experts
// Every rank sees the same count matrix and so reaches the same verdict on the capacity: on overflow
// all ranks report status 202, dispatch sends nothing and the GEMMs see zero rows, so nothing is
// written past a receive buffer.
__device__ void plan_body(const int* __restrict__ cnt, const int* __restrict__ my_flags,
                                                   int E, int me, int W, int epoch, int cap,
                                                   int* __restrict__ send_base, int* __restrict__ rx_offsets,
                                                   int* __restrict__ rx_mtiles, int* status, long long limit) {
    __shared__ int s_tot[kMaxExperts];
    __shared__ int s_before[kMaxExperts];
    __shared__ int s_ok;
    __shared__ int s_over;
    if (threadIdx.x == 0) {
        s_ok = 1;
        s_over = 0;
    }
    __syncthreads();
    if (threadIdx.x < W) {
        if (!wait_flag(my_flags + 0 * kMaxRanks + threadIdx.x, epoch, status, 201, limit)) s_ok = 0;
        __threadfence_system();  // acquire: the counts announced by the flags
    }
    __syncthreads();
    const int El = E / W;
    if (!s_ok) {  // counts never arrived: leave a plan that moves and computes nothing
        for (int e = threadIdx.x; e <= El; e += blockDim.x) {
            rx_offsets[e] = 0;
            rx_mtiles[e] = 0;
        }
        if (threadIdx.x == 0) send_base[E] = 1;
        return;
    }
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int tot = 0, before = 0;
        for (int s = 0; s < W; ++s) {
            const int c = cnt[size_t(s) * E + e];
            if (s < me) before += c;
            tot += c;
        }
        s_tot[e] = tot;
        s_before[e] = before;
    }
    __syncthreads();
    if (threadIdx.x < W) {  // one thread per owner rank: rows it will receive
        int run = 0;
        for (int el = 0; el < El; ++el) run += s_tot[threadIdx.x * El + el];
        if (run > cap) s_over = 1;
    }
    __syncthreads();
    const bool over = s_over != 0;
    if (threadIdx.x == 0) {
        send_base[E] = over ? 1 : 0;
        if (over && status != nullptr) {
            *reinterpret_cast<volatile int*>(status) = 202;
            __threadfence_system();
        }
    }
    if (threadIdx.x < W) {  // one thread per owner rank: running base over its experts
        const int d = threadIdx.x;
        int run = 0, tiles = 0;
        for (int el = 0; el < El; ++el) {
            const int e = d * El + el;
            send_base[e] = run + s_before[e];
            if (d == me) {
                rx_offsets[el] = over ? 0 : run;
                rx_mtiles[el] = over ? 0 : tiles;
            }
            run += s_tot[e];
            tiles += (s_tot[e] + 127) / 128;
        }
        if (d == me) {
            rx_offsets[El] = over ? 0 : run;
            rx_mtiles[El] = over ? 0 : tiles;
        }
    }
}

__global__ void __launch_bounds__(256) plan_kernel(const int* __restrict__ cnt, const int* __restrict__ my_flags,
                                                   int E, int me, int W, int epoch, int cap,
                                                   int* __restrict__ send_base, int* __restrict__ rx_offsets,
                                                   int* __restrict__ rx_mtiles, int* status, long long limit) {
    plan_body(cnt, my_flags, E, me, W, epoch, cap, send_base, rx_offsets, rx_mtiles, status, limit);
}

// publish_counts and plan in one launch (one block): store my counts and flag to every rank, then wait for
// everybody's and compute the plan. Saves a launch on the path every call waits on.
__global__ void __launch_bounds__(256) publish_plan_kernel(const int* __restrict__ counts, int E, int me, int W, Peers cnt_all,
                                                           Peers flags_all, int epoch, int cap,
                                                           int* __restrict__ send_base, int* __restrict__ rx_offsets,
                                                           int* __restrict__ rx_mtiles, int* status, long long limit) {
    for (int p = 0; p < W; ++p) {
        int* dst = static_cast<int*>(cnt_all.p[p]) + size_t(me) * E;
        for (int e = threadIdx.x; e < E; e += blockDim.x) dst[e] = counts[e];
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x < W) {
        __threadfence_system();
        st_relaxed_sys(static_cast<int*>(flags_all.p[threadIdx.x]) + 0 * kMaxRanks + me, epoch);
    }
    plan_body(static_cast<const int*>(cnt_all.p[me]), static_cast<const int*>(flags_all.p[me]), E, me, W, epoch, cap, send_base,
              rx_offsets, rx_mtiles, status, limit);
}

// signal(phase) and wait(phase) in one launch: announce that the preceding kernels' stores are done, then wait for
// the same announcement from every rank.
__global__ void signal_wait_kernel(Peers flags, int phase, int me, int W, int epoch, int* status, long long limit) {
    if (threadIdx.x < W) {
        __threadfence_system();
        st_relaxed_sys(static_cast<int*>(flags.p[threadIdx.x]) + phase * kMaxRanks + me, epoch);
        wait_flag(static_cast<const int*>(flags.p[me]) + phase * kMaxRanks + threadIdx.x, epoch, status, 210 + phase, limit);
        __threadfence_system();
    }
}

__device__ __forceinline__ void copy_vecs(const uint8_t* __restrict__ src, uint8_t* dst, int vecs, int lane) {
    int i = lane;
    for (; i + 96 < vecs; i += 128) {
        const Vec16 a = ld_nc16(src + size_t(i) * 16), b = ld_nc16(src + size_t(i + 32) * 16);
        const Vec16 c = ld_nc16(src + size_t(i + 64) * 16), d = ld_nc16(src + size_t(i + 96) * 16);
        st16(dst + size_t(i) * 16, a);
        st16(dst + size_t(i + 32) * 16, b);
        st16(dst + size_t(i + 64) * 16, c);
        st16(dst + size_t(i + 96) * 16, d);
    }
    for (; i < vecs; i += 32) st16(dst + size_t(i) * 16, ld_nc16(src + size_t(i) * 16));
}

// One warp per expert-sorted local row i: a[dest_to_src[i] / k] -> owner's receive buffer.
__global__ void __launch_bounds__(256) dispatch_kernel(const uint8_t* __restrict__ a, const float* __restrict__ a_scale,
                                                       int row_vecs, int scale_cols, int k,
                                                       const int* __restrict__ offsets /*[E+1] local sort*/,
                                                       const int* __restrict__ dest_to_src,
                                                       const int* __restrict__ send_base, int E, int me, int W,
                                                       Peers rx_rows, Peers rx_scale, Peers rx_home, Peers flags,
                                                       int* done_counter, int epoch) {
    __shared__ int s_off[kMaxExperts + 1];
    for (int e = threadIdx.x; e <= E; e += blockDim.x) s_off[e] = offsets[e];
    __syncthreads();
    const int kept = send_base[E] != 0 ? 0 : s_off[E];  // the plan found a receive buffer too small: send nothing
    const int El = E / W;
    const int lane = threadIdx.x & 31;
    const int warps = gridDim.x * (blockDim.x >> 5);
    for (int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); i < kept; i += warps) {
        int lo = 0, hi = E;  // expert of sorted row i: last e with s_off[e] <= i
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (s_off[mid] <= i) lo = mid; else hi = mid;
        }
        const int e = lo;
        const int owner = e / El;
        const size_t dst_row = size_t(send_base[e] + (i - s_off[e]));
        const int slot = dest_to_src[i];
        const size_t src_row = size_t(slot / k);
        copy_vecs(a + src_row * row_vecs * 16, static_cast<uint8_t*>(rx_rows.p[owner]) + dst_row * row_vecs * 16,
                  row_vecs, lane);
        if (scale_cols > 0) {
            float* sd = static_cast<float*>(rx_scale.p[owner]) + dst_row * scale_cols;
            for (int c = lane; c < scale_cols; c += 32) sd[c] = a_scale[src_row * scale_cols + c];
        }
        // home of the result: (source rank, slot t*k+j) packed as rank * 2^27 + slot (slot < 2^27)
        if (lane == 0) static_cast<int*>(rx_home.p[owner])[dst_row] = (me << 27) | slot;
    }
    // all blocks done -> tell every owner that my rows have landed. The blocks order their row stores before the
    // counter at GPU scope; the last block, which has observed every other block's arrival, fences once at system
    // scope before it stores the flags (causality composes across the two scopes).
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int prev = atomicAdd(done_counter, 1);
        if (prev == int(gridDim.x) - 1) {
            *done_counter = 0;
            __threadfence_system();
            for (int p = 0; p < W; ++p) st_relaxed_sys(static_cast<int*>(flags.p[p]) + 1 * kMaxRanks + me, epoch);
        }
    }
}

__global__ void wait_kernel(const int* __restrict__ my_flags, int phase, int W, int epoch, int* status,
                            long long limit) {
    if (threadIdx.x < W) {
        wait_flag(my_flags + phase * kMaxRanks + threadIdx.x, epoch, status, 210 + phase, limit);
        __threadfence_system();  // acquire: what the flags announce (rows, results) is visible to the kernels that follow
    }
}

__global__ void signal_kernel(Peers flags, int phase, int me, int W, int epoch) {
    if (threadIdx.x < W) {
        __threadfence_system();  // release: the preceding kernels' stores (the fc2 epilogue's result rows)
        st_relaxed_sys(static_cast<int*>(flags.p[threadIdx.x]) + phase * kMaxRanks + me, epoch);
    }
}

// row_dst[r] = address of the home output row of received row r (0 beyond the received rows)
__global__ void __launch_bounds__(256) row_ptrs_kernel(const int* __restrict__ rx_home, const int* __restrict__ rx_offsets,
                                                       int El, Peers d_out, size_t out_row_bytes, int cap,
                                                       unsigned long long* __restrict__ row_dst) {
    const int n_recv = rx_offsets[El];
    for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < cap; r += gridDim.x * blockDim.x) {
        unsigned long long ptr = 0;
        if (r < n_recv) {
            const int h = rx_home[r];
            ptr = reinterpret_cast<unsigned long long>(static_cast<uint8_t*>(d_out.p[h >> 27]) +
                                                       size_t(h & ((1 << 27) - 1)) * out_row_bytes);
        }
        row_dst[r] = ptr;
    }
}

// wait for every source's phase-1 flag (rows landed), then row_ptrs: one launch; every block polls the W flags itself
__global__ void __launch_bounds__(256) wait_row_ptrs_kernel(const int* __restrict__ my_flags, int W, int epoch, int* status,
                                                            long long limit, const int* __restrict__ rx_home,
                                                            const int* __restrict__ rx_offsets, int El, Peers d_out,
                                                            size_t out_row_bytes, int cap,
                                                            unsigned long long* __restrict__ row_dst) {
    if (threadIdx.x < W) {
        wait_flag(my_flags + 1 * kMaxRanks + threadIdx.x, epoch, status, 211, limit);
        __threadfence_system();  // acquire: the rows the flags announce are visible to this kernel and those that follow
    }
    __syncthreads();
    const int n_recv = rx_offsets[El];
    for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < cap; r += gridDim.x * blockDim.x) {
        unsigned long long ptr = 0;
        if (r < n_recv) {
            const int h = __ldcg(rx_home + r);  // written by peers: not through the read-only path
            ptr = reinterpret_cast<unsigned long long>(static_cast<uint8_t*>(d_out.p[h >> 27]) +
                                                       size_t(h & ((1 << 27) - 1)) * out_row_bytes);
        }
        row_dst[r] = ptr;
    }
}

static int make_peers(Peers* out, const void* const* ptrs, int W) {
    DQ_CHECK(W >= 1 && W <= kMaxRanks && ptrs != nullptr);
    for (int i = 0; i < kMaxRanks; ++i) out->p[i] = i < W ? const_cast<void*>(ptrs[i]) : nullptr;
    for (int i = 0; i < W; ++i) DQ_CHECK(out->p[i] != nullptr);
    return DQMOE_OK;
}

}  // namespace ep
}  // namespace dq

using namespace dq;

extern "C" {

int dqmoe_ep_publish_counts(const int32_t* counts, int E, int me, int W, const void* const* cnt_ptrs,
                            const void* const* flag_ptrs, int epoch, dqmoe_stream_t stream) {
    DQ_CHECK(counts != nullptr && E > 0 && E <= ep::kMaxExperts && me >= 0 && me < W && E % W == 0);
    ep::Peers cnt, flags;
    int rc = ep::make_peers(&cnt, cnt_ptrs, W);
    if (rc != DQMOE_OK) return rc;
    rc = ep::make_peers(&flags, flag_ptrs, W);
    if (rc != DQMOE_OK) return rc;
    ep::publish_counts_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(counts, E, me, W, cnt, flags, epoch);
    DQ_LAUNCH_CHECK();
    return DQMOE_OK;
}

int dqmoe_ep_set_wait_limit(int64_t cycles) {
    DQ_CHECK(cycles >= 0);
    ep::g_wait_limit.store(cycles == 0 ? ep::kDefaultWaitLimit : static_cast<long long>(cycles),
                           std::memory_order_relaxed);
    return DQMOE_OK;
}

int dqmoe_ep_plan(const int32_t* cnt, const int32_t* my_flags, int E, int me, int W, int epoch, int cap,
                  int32_t* send_base, int32_t* rx_offsets, int32_t* rx_mtiles, dqmoe_stream_t stream) {
    DQ_CHECK(cnt != nullptr && my_flags != nullptr && send_base != nullptr && rx_offsets != nullptr && rx_mtiles != nullptr);
    DQ_CHECK(E > 0 && E <= ep::kMaxExperts && W >= 1 && W <= ep::kMaxRanks && me >= 0 && me < W && E % W == 0);
    DQ_CHECK(cap >= 0);
    ep::plan_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(cnt, my_flags, E, me, W, epoch, cap, send_base,
                                                                      rx_offsets, rx_mtiles, device_status_word(),
                                                                      ep::wait_limit());
    DQ_LAUNCH_CHECK();
    return DQMOE_OK;
}

int dqmoe_ep_publish_plan(const int32_t* counts, int E, int me, int W, const void* const* cnt_ptrs,
                          const void* const* flag_ptrs, int epoch, int cap, int32_t* send_base, int32_t* rx_offsets,
                          int32_t* rx_mtiles, dqmoe_stream_t stream) {
    DQ_CHECK(counts != nullptr && send_base != nullptr && rx_offsets != nullptr && rx_mtiles != nullptr);
    DQ_CHECK(E > 0 && E <= ep::kMaxExperts && W >= 1 && W <= ep::kMaxRanks && me >= 0 && me < W && E % W == 0 && cap >= 0);
    ep::Peers cnt, flags;
    int rc = ep::make_peers(&cnt, cnt_ptrs, W);
    if (rc == DQMOE_OK) rc = ep::make_peers(&flags, flag_ptrs, W);
    if (rc != DQMOE_OK) return rc;
    ep::publish_plan_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(counts, E, me, W, cnt, flags, epoch, cap, send_base,
                                                                              rx_offsets, rx_mtiles, device_status_word(),
                                                                              ep::wait_limit());
    DQ_LAUNCH_CHECK();
    return DQMOE_OK;
}

int dqmoe_ep_signal_wait(const void* const* flag_ptrs, int phase, int me, int W, int epoch, dqmoe_stream_t stream) {
    DQ_CHECK(phase >= 0 && phase < 3 && me >= 0 && me < W);
    ep::Peers flags;
    const int rc = ep::make_peers(&flags, flag_ptrs, W);
    if (rc != DQMOE_OK) return rc;
    ep::signal_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(flags, phase, me, W, epoch, device_status_word(),
                                                                            ep::wait_limit());
    DQ_LAUNCH_CHECK();
    return DQMOE_OK;
}

int dqmoe_ep_dispatch(const void* a, const float* a_scale, size_t row_bytes, int scale_cols, int k, int n,
                      const int32_t* offsets, const int32_t* dest_to_src, const int32_t* send_base, int E, int me,
                      int W, const void* const* rx_rows, const void* const* rx_scale, const void* const* rx_home,
                      const void* const* flag_ptrs, int32_t* done_counter, int epoch, dqmoe_stream_t stream) {
    DQ_CHECK(a != nullptr && offsets != nullptr && dest_to_src != nullptr && send_base != nullptr && done_counter != nullptr);
    DQ_CHECK(row_bytes % 16 == 0 && row_bytes > 0 && k > 0 && n >= 0 && scale_cols >= 0);
    DQ_CHECK(E > 0 && E <= ep::kMaxExperts && me >= 0 && me < W && E % W == 0);
    DQ_CHECK(int64_t(n) < (int64_t(1) << 27));
    ep::Peers rows, scale, home, flags;
    int rc = ep::make_peers(&rows, rx_rows, W);
    if (rc == DQMOE_OK) rc = ep::make_peers(&home, rx_home, W);
    if (rc == DQMOE_OK) rc = ep::make_peers(&flags, flag_ptrs, W);
    if (rc != DQMOE_OK) return rc;
    if (scale_cols > 0) {
        DQ_CHECK(a_scale != nullptr);
        rc = ep::make_peers(&scale, rx_scale, W);
        if (rc != DQMOE_OK) return rc;
    } else {
        for (int i = 0; i < ep::kMaxRanks; ++i) scale.p[i] = nullptr;
    }
    const int want = (n + 7) / 8;
    const int cap = sm_count() * 8;
    const int grid = want < 1 ? 1 : (want < cap ? want : cap);
    ep::dispatch_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(a), a_scale, int(row_bytes / 16), scale_cols, k, offsets, dest_to_src, send_base, E,
        me, W, rows, scale, home, flags, done_counter, epoch);
    DQ_LAUNCH_CHECK();
    return DQMOE_OK;
}

int dqmoe_ep_wait(const int32_t* my_flags, int phase, int W, int epoch, dqmoe_stream_t stream) {
    DQ_CHECK(my_flags != nullptr && phase >= 0 && phase < 3 && W >= 1 && W <= ep::kMaxRanks);
    ep::wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(my_flags, phase, W, epoch, device_status_word(),
                                                                     ep::wait_limit());
    DQ_LAUNCH_CHECK();
    return DQMOE_OK;
}

int dqmoe_ep_signal(const void* const* flag_ptrs, int phase, int me, int W, int epoch, dqmoe_stream_t stream) {
    DQ_CHECK(phase >= 0 && phase < 3 && me >= 0 && me < W);
    ep::Peers flags;
    const int rc = ep::make_peers(&flags, flag_ptrs, W);
    if (rc != DQMOE_OK) return rc;
    ep::signal_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(flags, phase, me, W, epoch);
    DQ_LAUNCH_CHECK();
    return DQMOE_OK;
}

int dqmoe_ep_wait_row_ptrs(const int32_t* my_flags, int epoch, const int32_t* rx_home, const int32_t* rx_offsets, int E_local,
                           const void* const* d_out_ptrs, int W, size_t out_row_bytes, int cap, void* row_dst,
                           dqmoe_stream_t stream) {
    DQ_CHECK(my_flags != nullptr && rx_home != nullptr && rx_offsets != nullptr && row_dst != nullptr && E_local > 0 && cap >= 0);
    ep::Peers d_out;
    const int rc = ep::make_peers(&d_out, d_out_ptrs, W);
    if (rc != DQMOE_OK) return rc;
    const int want = (cap + 255) / 256;
    const int lim = sm_count() * 4;
    ep::wait_row_ptrs_kernel<<<want < 1 ? 1 : (want < lim ? want : lim), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        my_flags, W, epoch, device_status_word(), ep::wait_limit(), rx_home, rx_offsets, E_local, d_out, out_row_bytes, cap,
        static_cast<unsigned long long*>(row_dst));
    DQ_LAUNCH_CHECK();
    return DQMOE_OK;
}

int dqmoe_ep_row_ptrs(const int32_t* rx_home, const int32_t* rx_offsets, int E_local, const void* const* d_out_ptrs,
                      int W, size_t out_row_bytes, int cap, void* row_dst, dqmoe_stream_t stream) {
    DQ_CHECK(rx_home != nullptr && rx_offsets != nullptr && row_dst != nullptr && E_local > 0 && cap >= 0);
    if (cap == 0) return DQMOE_OK;
    ep::Peers d_out;
    const int rc = ep::make_peers(&d_out, d_out_ptrs, W);
    if (rc != DQMOE_OK) return rc;
    const int want = (cap + 255) / 256;
    const int lim = sm_count() * 4;
    ep::row_ptrs_kernel<<<want < lim ? want : lim, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        rx_home, rx_offsets, E_local, d_out, out_row_bytes, cap, static_cast<unsigned long long*>(row_dst));
    DQ_LAUNCH_CHECK();
    return DQMOE_OK;
}

}  // extern "C"
