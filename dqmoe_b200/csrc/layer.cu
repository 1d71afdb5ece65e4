// Layer orchestrator: carves the caller's workspace and enqueues the MoE layer
// pipeline on one stream with no host synchronisation:
//   expert sort -> row (+scale) gather -> grouped fc1 with fused SwiGLU and
//   intermediate quantisation -> [re-quantisation pass for tensor/channel modes]
//   -> grouped fc2 with fused dequantisation and scatter into d[T, k, H].
// Replaces MoeFCRunner::getWorkspaceDeviceBufferSizes / runMoe / Gemm of the
// reference (csrc/moe_kernels.h:640-711, 770-947), which runs the same steps as
// sixteen separate launches.
#include "common.cuh"

namespace dq {
namespace route {
size_t sort_workspace_bytes(int n, int E);
int route_sort(const int* ids, int n, int E, int* counts, int* offsets, int* mtile_prefix, int* dest_to_src,
               int* src_to_dest, void* ws, size_t ws_bytes, cudaStream_t stream);
int route_topk(const float* logits, int T, int E, int k, int n_shared, int scoring, int* indices, float* weights,
               cudaStream_t stream);
}  // namespace route
namespace gemm {
int grouped_gemm(const void* a, const float* a_scale, const void* w, const float* w_scale, const int* offsets,
                 const int* mtile_prefix, int n, int N, int K, int E, int quant_mode, int gated, void* out,
                 float* out_scale, float* amax, const int* dest_to_src, const void* row_dst, cudaStream_t stream,
                 int elem = 0, const float* bias = nullptr);
enum Elem : int { kElemBf16 = 0, kElemHalf = 1, kElemF32 = 2 };  // element type of the unquantised path
}  // namespace gemm

namespace gemm_mx {
int grouped_gemm_mx(const void* a, const uint8_t* a_sf, const void* w, const uint8_t* w_sf, const int* offsets,
                    const int* mtile_prefix, int n, int N, int K, int E, int gated, void* out, uint8_t* out_sf,
                    const int* dest_to_src, const void* row_dst, const float* bias, bool fp4, const float* ga,
                    const float* gw, const float* gout, cudaStream_t stream);
}  // namespace gemm_mx

namespace decode {
int forward(const void* a, const float* a_scale, const void* b, const float* b_scale, const void* b1,
            const float* b1_scale, void* d, const int* m_indices, void* act_bf16, float* amax, int T, int H, int I,
            int E, int k, bool fp8, cudaStream_t stream);
bool eligible(int H, int I, bool fp8);  // row sizes the decode path serves (16-byte rows, activation row + ring fit shared memory)
}  // namespace decode

namespace layer {

constexpr size_t kAlign = 256;  // CUDA_MEM_ALIGN of the reference (csrc/util.h:54-59)
constexpr int kDecodeRows = 8;  // up to this many expanded rows the GEMV path of decode.cu is used (bf16, per-tensor FP8)

struct Layout {
    size_t offsets, counts, mtile_prefix, sort_ws, dest_to_src, perm_a, perm_a_scale, act, act_scale, act_bf16, amax;
    size_t total;
    size_t sort_ws_bytes;
    int perm_scale_cols;
};

static bool valid_mode(int q) {
    return q == DQMOE_QUANT_NONE || q == DQMOE_QUANT_FP8_TENSOR || q == DQMOE_QUANT_FP8_CHANNEL ||
           q == DQMOE_QUANT_FP8_BLOCK || q == DQMOE_QUANT_FP8_MX;
}

// modes the workspace can be laid out for: those of dqmoe_moe_forward plus NVFP4, which has its own entry point
static bool valid_layout_mode(int q) { return valid_mode(q) || q == DQMOE_QUANT_NVFP4; }

static Layout make_layout(int T, int H, int I, int E, int k, int quant_mode, int elem = gemm::kElemBf16) {
    Layout L{};
    const size_t n = size_t(T) * k;
    const size_t esz = quant_mode != DQMOE_QUANT_NONE ? 1 : (elem == gemm::kElemF32 ? 4 : 2);
    size_t off = 0;
    auto add = [&](size_t bytes) {
        const size_t at = off;
        off += align_up(bytes, kAlign);
        return at;
    };
    L.offsets = add((E + 1) * sizeof(int));
    L.counts = add(E * sizeof(int));
    L.mtile_prefix = add((E + 1) * sizeof(int));
    L.sort_ws_bytes = route::sort_workspace_bytes(int(n), E);
    L.sort_ws = add(L.sort_ws_bytes);
    L.dest_to_src = add(n * sizeof(int));
    const bool fp4 = quant_mode == DQMOE_QUANT_NVFP4;  // two elements per byte; scales tiled like MXFP8's, per 64 K elements
    L.perm_a = add(fp4 ? n * H / 2 : n * H * esz);
    L.perm_scale_cols = quant_mode == DQMOE_QUANT_FP8_BLOCK ? ceil_div(H, 128)
                        : quant_mode == DQMOE_QUANT_FP8_CHANNEL ? 1 : 0;
    // MX mode: UE8M0 scale bytes in the tiled layout, whole 512-byte blocks per 128-row tile of the expert sort
    const bool mx = quant_mode == DQMOE_QUANT_FP8_MX;
    L.perm_a_scale = add(fp4 ? dqmoe_mx_tiled_scale_bytes(int64_t(n), E, 2 * align_up(H, 64))
                         : mx ? dqmoe_mx_tiled_scale_bytes(int64_t(n), E, align_up(H, 128)) : n * L.perm_scale_cols * sizeof(float));
    L.act = add(fp4 ? n * I / 2 : n * I * esz);
    const size_t act_scale_elems = fp4 ? dqmoe_mx_tiled_scale_bytes(int64_t(n), E, 2 * align_up(I, 64)) / sizeof(float)
                                   : mx ? dqmoe_mx_tiled_scale_bytes(int64_t(n), E, align_up(I, 128)) / sizeof(float)
                                   : quant_mode == DQMOE_QUANT_FP8_BLOCK ? n * ceil_div(I, 128)
                                   : quant_mode == DQMOE_QUANT_FP8_CHANNEL ? n
                                   : quant_mode == DQMOE_QUANT_FP8_TENSOR ? 1 : 0;
    L.act_scale = add(act_scale_elems * sizeof(float));
    const bool two_pass = quant_mode == DQMOE_QUANT_FP8_TENSOR || quant_mode == DQMOE_QUANT_FP8_CHANNEL;
    L.act_bf16 = add(two_pass ? n * I * 2 : 0);
    L.amax = add(quant_mode == DQMOE_QUANT_FP8_CHANNEL ? n * sizeof(float)
                 : quant_mode == DQMOE_QUANT_FP8_TENSOR ? decode::kAmaxParts * sizeof(float) : 0);
    L.total = off;
    return L;
}

}  // namespace layer
}  // namespace dq

using namespace dq;

extern "C" {

size_t dqmoe_moe_workspace_bytes(int T, int H, int I, int E, int k, int quant_mode) {
    if (T < 0 || H <= 0 || I <= 0 || E <= 0 || k <= 0 || !layer::valid_layout_mode(quant_mode)) return 0;
    return layer::make_layout(T, H, I, E, k, quant_mode).total;
}

void* dqmoe_moe_workspace_ptr(void* workspace, int which, int T, int H, int I, int E, int k, int quant_mode) {
    if (workspace == nullptr || T < 0 || H <= 0 || I <= 0 || E <= 0 || k <= 0 || !layer::valid_layout_mode(quant_mode))
        return nullptr;
    const layer::Layout L = layer::make_layout(T, H, I, E, k, quant_mode);
    char* ws = static_cast<char*>(workspace);
    switch (which) {
        case 0: return ws + L.offsets;
        case 1: return ws + L.dest_to_src;
        case 2: return ws + L.perm_a;
        case 3: return ws + L.perm_a_scale;
        case 4: return ws + L.act;
        case 5: return ws + L.act_scale;
        case 6: return ws + L.counts;
        case 7: return ws + L.mtile_prefix;
        default: return nullptr;
    }
}

// elem: the operands and the output are bf16, IEEE half or fp32 (the last two with quant_mode NONE only);
// bias1 [E, 2I] / bias2 [E, H]: fp32 biases of fc1 / fc2 added to the dequantised products, or nullptr.
static int moe_forward_impl(const void* a, const float* a_scale, const void* b, const float* b_scale, const void* b1,
                            const float* b1_scale, void* d, const int32_t* m_indices, void* workspace,
                            size_t workspace_bytes, int T, int H, int I, int E, int k, int quant_mode, int elem,
                            const float* bias1, const float* bias2, cudaStream_t stream) {
    DQ_CHECK(T >= 0 && H > 0 && I > 0 && E > 0 && k > 0);
    DQ_CHECK_FMT(layer::valid_mode(quant_mode), "quant_mode_value=%d is not one of 0, 256, 512, 1024, 2048", quant_mode);
    if (quant_mode == DQMOE_QUANT_FP8_MX)
        DQ_CHECK_FMT(H % 128 == 0 && I % 128 == 0, "hidden_size=%d and inter_size=%d must be multiples of 128 in the MXFP8 mode",
                     H, I);
    if (T == 0) return DQMOE_OK;  // as csrc/pybind11_register.h:125-126
    DQ_CHECK(a != nullptr && b != nullptr && b1 != nullptr && d != nullptr && m_indices != nullptr);
    DQ_CHECK_FMT(workspace != nullptr && is_aligned(workspace, layer::kAlign), "workspace pointer %p is not aligned!",
                 workspace);
    const bool fp8 = quant_mode != DQMOE_QUANT_NONE;
    if (fp8) DQ_CHECK(a_scale != nullptr && b_scale != nullptr && b1_scale != nullptr);
    DQ_CHECK(elem == gemm::kElemBf16 || !fp8);
    const size_t esz = fp8 ? 1 : (elem == gemm::kElemF32 ? 4 : 2);
    DQ_CHECK_FMT((H * esz) % 16 == 0 && (I * esz) % 16 == 0,
                 "hidden_size=%d and inter_size=%d rows must be multiples of 16 bytes", H, I);
    DQ_CHECK(int64_t(T) * k < (int64_t(1) << 31));
    const int n = T * k;
    const layer::Layout L = layer::make_layout(T, H, I, E, k, quant_mode, elem);
    if (workspace_bytes != 0 && workspace_bytes < L.total)
        return fail(DQMOE_ERR_WORKSPACE, __FILE__, __LINE__, "workspace_bytes >= dqmoe_moe_workspace_bytes(...)",
                    "workspace has %zu bytes, the layer needs %zu", workspace_bytes, L.total);

    char* ws = static_cast<char*>(workspace);
    int* offsets = reinterpret_cast<int*>(ws + L.offsets);
    int* counts = reinterpret_cast<int*>(ws + L.counts);
    int* mtile_prefix = reinterpret_cast<int*>(ws + L.mtile_prefix);
    int* dest_to_src = reinterpret_cast<int*>(ws + L.dest_to_src);
    void* perm_a = ws + L.perm_a;
    float* perm_a_scale = reinterpret_cast<float*>(ws + L.perm_a_scale);
    void* act = ws + L.act;
    float* act_scale = reinterpret_cast<float*>(ws + L.act_scale);
    void* act_bf16 = ws + L.act_bf16;
    float* amax = reinterpret_cast<float*>(ws + L.amax);

    if (elem == gemm::kElemBf16 && bias1 == nullptr && bias2 == nullptr && n <= layer::kDecodeRows &&
        (quant_mode == DQMOE_QUANT_NONE || quant_mode == DQMOE_QUANT_FP8_TENSOR) && decode::eligible(H, I, fp8))
        return decode::forward(a, a_scale, b, b_scale, b1, b1_scale, d, m_indices, fp8 ? act_bf16 : act, amax, T, H, I,
                               E, k, fp8, stream);

    int rc = route::route_sort(m_indices, n, E, counts, offsets, mtile_prefix, dest_to_src, nullptr, ws + L.sort_ws,
                               L.sort_ws_bytes, stream);
    if (rc != DQMOE_OK) return rc;

    rc = dqmoe_permute_rows(a, size_t(H) * esz, k, dest_to_src, n, perm_a, L.perm_scale_cols ? a_scale : nullptr,
                            L.perm_scale_cols, L.perm_scale_cols ? perm_a_scale : nullptr, stream);
    if (rc != DQMOE_OK) return rc;

    if (quant_mode == DQMOE_QUANT_FP8_MX) {
        // the scale pointers address UE8M0 bytes in this mode: the activations' row-major [T, H/32], gathered here
        // into the tiled layout of the expert sort; the weights' already tiled
        rc = dqmoe_mx_tile_scales(reinterpret_cast<const uint8_t*>(a_scale), n, H, dest_to_src, k, offsets, mtile_prefix, E,
                                  reinterpret_cast<uint8_t*>(perm_a_scale), stream);
        if (rc != DQMOE_OK) return rc;
        rc = gemm_mx::grouped_gemm_mx(perm_a, reinterpret_cast<const uint8_t*>(perm_a_scale), b,
                                      reinterpret_cast<const uint8_t*>(b_scale), offsets, mtile_prefix, n, I, H, E, 1, act,
                                      reinterpret_cast<uint8_t*>(act_scale), nullptr, nullptr, bias1, false, nullptr, nullptr,
                                      nullptr, stream);
        if (rc != DQMOE_OK) return rc;
        return gemm_mx::grouped_gemm_mx(act, reinterpret_cast<const uint8_t*>(act_scale), b1,
                                        reinterpret_cast<const uint8_t*>(b1_scale), offsets, mtile_prefix, n, H, I, E, 0, d,
                                        nullptr, dest_to_src, nullptr, bias2, false, nullptr, nullptr, nullptr, stream);
    }
    const float* sa1 = quant_mode == DQMOE_QUANT_FP8_TENSOR ? a_scale : perm_a_scale;
    const bool two_pass = quant_mode == DQMOE_QUANT_FP8_TENSOR || quant_mode == DQMOE_QUANT_FP8_CHANNEL;
    if (two_pass) {
        const size_t amax_bytes = quant_mode == DQMOE_QUANT_FP8_CHANNEL ? size_t(n) * sizeof(float) : sizeof(float);
        DQ_CUDA(cudaMemsetAsync(amax, 0, amax_bytes, stream));
    }
    rc = gemm::grouped_gemm(perm_a, sa1, b, b_scale, offsets, mtile_prefix, n, I, H, E, quant_mode, 1,
                            two_pass ? act_bf16 : act, act_scale, amax, nullptr, nullptr, stream, elem, bias1);
    if (rc != DQMOE_OK) return rc;
    if (two_pass) {
        rc = dqmoe_requant_from_amax(act_bf16, n, I, amax, quant_mode == DQMOE_QUANT_FP8_CHANNEL ? 1 : 0, act,
                                     act_scale, stream);
        if (rc != DQMOE_OK) return rc;
    }
    rc = gemm::grouped_gemm(act, act_scale, b1, b1_scale, offsets, mtile_prefix, n, H, I, E, quant_mode, 0, d, nullptr,
                            nullptr, dest_to_src, nullptr, stream, elem, bias2);
    return rc;
}

int dqmoe_moe_forward(const void* a, const float* a_scale, const void* b, const float* b_scale, const void* b1,
                      const float* b1_scale, void* d, const int32_t* m_indices, void* workspace,
                      size_t workspace_bytes, int T, int H, int I, int E, int k, int quant_mode, int fused,
                      dqmoe_stream_t stream) {
    (void) fused;
    return moe_forward_impl(a, a_scale, b, b_scale, b1, b1_scale, d, m_indices, workspace, workspace_bytes, T, H, I, E, k,
                            quant_mode, gemm::kElemBf16, nullptr, nullptr, static_cast<cudaStream_t>(stream));
}

int dqmoe_moe_forward_bias(const void* a, const float* a_scale, const void* b, const float* b_scale, const void* b1,
                           const float* b1_scale, const float* bias1, const float* bias2, void* d,
                           const int32_t* m_indices, void* workspace, size_t workspace_bytes, int T, int H, int I, int E,
                           int k, int quant_mode, dqmoe_stream_t stream) {
    return moe_forward_impl(a, a_scale, b, b_scale, b1, b1_scale, d, m_indices, workspace, workspace_bytes, T, H, I, E, k,
                            quant_mode, gemm::kElemBf16, bias1, bias2, static_cast<cudaStream_t>(stream));
}

// The layer in the NVFP4 mode: expert sort, gather of the packed rows, gather of their scale bytes into the tiled
// layout of the sort, grouped fc1 (SwiGLU, re-quantisation to NVFP4 with act_gscale) and grouped fc2.
int dqmoe_moe_forward_nvfp4(const void* a, const uint8_t* a_sf, const float* a_gscale, const void* b, const uint8_t* b_sf,
                            const float* b_gscale, const void* b1, const uint8_t* b1_sf, const float* b1_gscale,
                            const float* act_gscale, const float* bias1, const float* bias2, void* d,
                            const int32_t* m_indices, void* workspace, size_t workspace_bytes, int T, int H, int I, int E,
                            int k, dqmoe_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    DQ_CHECK(T >= 0 && H > 0 && I > 0 && E > 0 && k > 0);
    DQ_CHECK_FMT(H % 256 == 0 && I % 256 == 0, "hidden_size=%d and inter_size=%d must be multiples of 256 in the NVFP4 mode", H, I);
    if (T == 0) return DQMOE_OK;
    DQ_CHECK(a != nullptr && b != nullptr && b1 != nullptr && d != nullptr && m_indices != nullptr);
    DQ_CHECK(a_sf != nullptr && b_sf != nullptr && b1_sf != nullptr && a_gscale != nullptr && b_gscale != nullptr &&
             b1_gscale != nullptr && act_gscale != nullptr);
    DQ_CHECK_FMT(workspace != nullptr && is_aligned(workspace, layer::kAlign), "workspace pointer %p is not aligned!",
                 workspace);
    DQ_CHECK(int64_t(T) * k < (int64_t(1) << 31));
    const int n = T * k;
    const layer::Layout L = layer::make_layout(T, H, I, E, k, DQMOE_QUANT_NVFP4);
    if (workspace_bytes != 0 && workspace_bytes < L.total)
        return fail(DQMOE_ERR_WORKSPACE, __FILE__, __LINE__, "workspace_bytes >= dqmoe_moe_workspace_bytes(...)",
                    "workspace has %zu bytes, the layer needs %zu", workspace_bytes, L.total);
    char* ws = static_cast<char*>(workspace);
    int* offsets = reinterpret_cast<int*>(ws + L.offsets);
    int* counts = reinterpret_cast<int*>(ws + L.counts);
    int* mtile_prefix = reinterpret_cast<int*>(ws + L.mtile_prefix);
    int* dest_to_src = reinterpret_cast<int*>(ws + L.dest_to_src);
    void* perm_a = ws + L.perm_a;
    uint8_t* perm_a_sf = reinterpret_cast<uint8_t*>(ws + L.perm_a_scale);
    void* act = ws + L.act;
    uint8_t* act_sf = reinterpret_cast<uint8_t*>(ws + L.act_scale);
    int rc = route::route_sort(m_indices, n, E, counts, offsets, mtile_prefix, dest_to_src, nullptr, ws + L.sort_ws,
                               L.sort_ws_bytes, stream);
    if (rc != DQMOE_OK) return rc;
    rc = dqmoe_permute_rows(a, size_t(H) / 2, k, dest_to_src, n, perm_a, nullptr, 0, nullptr, stream);
    if (rc != DQMOE_OK) return rc;
    // one scale byte per 16 elements: the tiling kernel sees them as the scales of a row twice as long
    rc = dqmoe_mx_tile_scales(a_sf, n, 2 * H, dest_to_src, k, offsets, mtile_prefix, E, perm_a_sf, stream);
    if (rc != DQMOE_OK) return rc;
    rc = gemm_mx::grouped_gemm_mx(perm_a, perm_a_sf, b, b_sf, offsets, mtile_prefix, n, I, H, E, 1, act, act_sf, nullptr,
                                  nullptr, bias1, true, a_gscale, b_gscale, act_gscale, stream);
    if (rc != DQMOE_OK) return rc;
    return gemm_mx::grouped_gemm_mx(act, act_sf, b1, b1_sf, offsets, mtile_prefix, n, H, I, E, 0, d, nullptr, dest_to_src,
                                    nullptr, bias2, true, act_gscale, b1_gscale, nullptr, stream);
}

int dqmoe_moe_forward_f16(const void* a, const void* b, const void* b1, void* d, const int32_t* m_indices,
                          void* workspace, size_t workspace_bytes, int T, int H, int I, int E, int k,
                          dqmoe_stream_t stream) {
    return moe_forward_impl(a, nullptr, b, nullptr, b1, nullptr, d, m_indices, workspace, workspace_bytes, T, H, I, E, k,
                            DQMOE_QUANT_NONE, gemm::kElemHalf, nullptr, nullptr, static_cast<cudaStream_t>(stream));
}

size_t dqmoe_moe_workspace_bytes_f32(int T, int H, int I, int E, int k) {
    if (T < 0 || H <= 0 || I <= 0 || E <= 0 || k <= 0) return 0;
    return layer::make_layout(T, H, I, E, k, DQMOE_QUANT_NONE, gemm::kElemF32).total;
}

int dqmoe_moe_forward_f32(const void* a, const void* b, const void* b1, const float* bias1, const float* bias2, void* d,
                          const int32_t* m_indices, void* workspace, size_t workspace_bytes, int T, int H, int I, int E,
                          int k, dqmoe_stream_t stream) {
    return moe_forward_impl(a, nullptr, b, nullptr, b1, nullptr, d, m_indices, workspace, workspace_bytes, T, H, I, E, k,
                            DQMOE_QUANT_NONE, gemm::kElemF32, bias1, bias2, static_cast<cudaStream_t>(stream));
}

int dqmoe_moe_forward_f16_bias(const void* a, const void* b, const void* b1, const float* bias1, const float* bias2,
                               void* d, const int32_t* m_indices, void* workspace, size_t workspace_bytes, int T, int H,
                               int I, int E, int k, dqmoe_stream_t stream) {
    return moe_forward_impl(a, nullptr, b, nullptr, b1, nullptr, d, m_indices, workspace, workspace_bytes, T, H, I, E, k,
                            DQMOE_QUANT_NONE, gemm::kElemHalf, bias1, bias2, static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------------------------------------
// Whole MoE block from bf16 activations: router -> expert sort -> gather fused with the dynamic
// activation quantisation -> grouped fc1/fc2 -> weighted combine over the k slots.
// Workspace = [indices T*k | weights T*k | d T*k*H bf16 | layer workspace].
struct BlockLayout {
    size_t indices, weights, d, xq, xs, xamax, layer, total;
};
static BlockLayout block_layout(int T, int H, int I, int E, int k, int quant_mode) {
    BlockLayout B{};
    size_t off = 0;
    auto add = [&](size_t bytes) {
        const size_t at = off;
        off += align_up(bytes, layer::kAlign);
        return at;
    };
    B.indices = add(size_t(T) * k * sizeof(int));
    B.weights = add(size_t(T) * k * sizeof(float));
    B.d = add(size_t(T) * k * H * 2);
    // tensor / channel modes quantise x [T, H] before the gather (block mode quantises while gathering)
    const bool pre_quant = quant_mode == DQMOE_QUANT_FP8_TENSOR || quant_mode == DQMOE_QUANT_FP8_CHANNEL;
    B.xq = add(pre_quant ? size_t(T) * H : 0);
    B.xs = add(pre_quant ? size_t(T) * sizeof(float) : 0);
    B.xamax = add(pre_quant ? sizeof(float) : 0);
    B.layer = add(layer::make_layout(T, H, I, E, k, quant_mode).total);
    B.total = off;
    return B;
}

size_t dqmoe_moe_block_workspace_bytes(int T, int H, int I, int E, int k, int quant_mode) {
    if (T < 0 || H <= 0 || I <= 0 || E <= 0 || k <= 0) return 0;
    if (!layer::valid_mode(quant_mode)) return 0;
    return block_layout(T, H, I, E, k, quant_mode).total;
}

// The block with `n_shared` shared experts: the weight tensors hold E routed experts followed by the shared ones,
// and every token gets n_shared extra slots (expert E + j, weight 1) that run through the same sort, gather,
// grouped GEMMs and weighted sum as the routed slots.
static int moe_block_impl(const void* x_bf16, const float* logits, const void* b, const float* b_scale, const void* b1,
                          const float* b1_scale, void* out_bf16, void* workspace, size_t workspace_bytes, int T, int H,
                          int I, int E_routed, int k_routed, int n_shared, int scoring, int quant_mode,
                          cudaStream_t stream) {
    DQ_CHECK(T >= 0 && H > 0 && I > 0 && E_routed > 0 && k_routed > 0 && n_shared >= 0);
    const int E = E_routed + n_shared;
    const int k = k_routed + n_shared;
    DQ_CHECK_FMT(layer::valid_mode(quant_mode), "quant_mode=%d: unknown quantisation mode", quant_mode);
    if (quant_mode == DQMOE_QUANT_FP8_MX)
        DQ_CHECK_FMT(H % 128 == 0 && I % 128 == 0, "hidden_size=%d and inter_size=%d must be multiples of 128 in the MXFP8 mode",
                     H, I);
    if (T == 0) return DQMOE_OK;
    DQ_CHECK(x_bf16 != nullptr && logits != nullptr && b != nullptr && b1 != nullptr && out_bf16 != nullptr);
    DQ_CHECK_FMT(workspace != nullptr && is_aligned(workspace, layer::kAlign), "workspace pointer %p is not aligned!",
                 workspace);
    const bool fp8 = quant_mode != DQMOE_QUANT_NONE;
    if (fp8) DQ_CHECK(b_scale != nullptr && b1_scale != nullptr);
    DQ_CHECK_FMT(H % 16 == 0 && I % 16 == 0, "hidden_size=%d and inter_size=%d must be multiples of 16", H, I);
    DQ_CHECK(int64_t(T) * k < (int64_t(1) << 31));
    const int n = T * k;
    const BlockLayout B = block_layout(T, H, I, E, k, quant_mode);
    if (workspace_bytes != 0 && workspace_bytes < B.total)
        return fail(DQMOE_ERR_WORKSPACE, __FILE__, __LINE__, "workspace_bytes >= dqmoe_moe_block_workspace_bytes(...)",
                    "workspace has %zu bytes, the block needs %zu", workspace_bytes, B.total);
    char* ws = static_cast<char*>(workspace);
    int* indices = reinterpret_cast<int*>(ws + B.indices);
    float* weights = reinterpret_cast<float*>(ws + B.weights);
    void* d = ws + B.d;
    char* lws = ws + B.layer;
    const layer::Layout L = layer::make_layout(T, H, I, E, k, quant_mode);
    int* offsets = reinterpret_cast<int*>(lws + L.offsets);
    int* counts = reinterpret_cast<int*>(lws + L.counts);
    int* mtile_prefix = reinterpret_cast<int*>(lws + L.mtile_prefix);
    int* dest_to_src = reinterpret_cast<int*>(lws + L.dest_to_src);
    void* perm_a = lws + L.perm_a;
    float* perm_a_scale = reinterpret_cast<float*>(lws + L.perm_a_scale);
    void* act = lws + L.act;
    float* act_scale = reinterpret_cast<float*>(lws + L.act_scale);

    int rc = route::route_topk(logits, T, E_routed, k_routed, n_shared, scoring, indices, weights, stream);
    if (rc != DQMOE_OK) return rc;
    if (quant_mode == DQMOE_QUANT_FP8_TENSOR || quant_mode == DQMOE_QUANT_FP8_CHANNEL) {
        // dynamic quantisation of the activations (per tensor or per token), then the layer as the drop-in call runs it
        void* xq = ws + B.xq;
        float* xs = reinterpret_cast<float*>(ws + B.xs);
        rc = quant_mode == DQMOE_QUANT_FP8_CHANNEL
                 ? dqmoe_quant_fp8_rowwise(x_bf16, T, H, xq, xs, stream)
                 : dqmoe_quant_fp8_tensor(x_bf16, 1, int64_t(T) * H, xq, xs, reinterpret_cast<float*>(ws + B.xamax), stream);
        if (rc != DQMOE_OK) return rc;
        rc = dqmoe_moe_forward(xq, xs, b, b_scale, b1, b1_scale, d, indices, lws, L.total, T, H, I, E, k, quant_mode, 1,
                               stream);
        if (rc != DQMOE_OK) return rc;
        return dqmoe_finalize_weighted(d, weights, out_bf16, T, k, H, stream);
    }
    rc = route::route_sort(indices, n, E, counts, offsets, mtile_prefix, dest_to_src, nullptr, lws + L.sort_ws,
                           L.sort_ws_bytes, stream);
    if (rc != DQMOE_OK) return rc;
    if (quant_mode == DQMOE_QUANT_FP8_MX) {  // the same fusion with 1x32 power-of-two scales
        rc = dqmoe_permute_quant_mxfp8(x_bf16, H, k, dest_to_src, n, offsets, mtile_prefix, E, perm_a,
                                       reinterpret_cast<uint8_t*>(perm_a_scale), stream);
        if (rc != DQMOE_OK) return rc;
        rc = gemm_mx::grouped_gemm_mx(perm_a, reinterpret_cast<const uint8_t*>(perm_a_scale), b,
                                      reinterpret_cast<const uint8_t*>(b_scale), offsets, mtile_prefix, n, I, H, E, 1, act,
                                      reinterpret_cast<uint8_t*>(act_scale), nullptr, nullptr, nullptr, false, nullptr, nullptr,
                                      nullptr, stream);
        if (rc != DQMOE_OK) return rc;
        rc = gemm_mx::grouped_gemm_mx(act, reinterpret_cast<const uint8_t*>(act_scale), b1,
                                      reinterpret_cast<const uint8_t*>(b1_scale), offsets, mtile_prefix, n, H, I, E, 0, d,
                                      nullptr, dest_to_src, nullptr, nullptr, false, nullptr, nullptr, nullptr, stream);
        if (rc != DQMOE_OK) return rc;
        return dqmoe_finalize_weighted(d, weights, out_bf16, T, k, H, stream);
    }
    if (fp8)  // quantise while gathering: each expanded row is read as bf16 and written as e4m3 + 1x128 scales
        rc = dqmoe_permute_quant_block_1x128(x_bf16, H, k, dest_to_src, n, perm_a, perm_a_scale, stream);
    else
        rc = dqmoe_permute_rows(x_bf16, size_t(H) * 2, k, dest_to_src, n, perm_a, nullptr, 0, nullptr, stream);
    if (rc != DQMOE_OK) return rc;
    rc = gemm::grouped_gemm(perm_a, perm_a_scale, b, b_scale, offsets, mtile_prefix, n, I, H, E, quant_mode, 1, act,
                            act_scale, nullptr, nullptr, nullptr, stream);
    if (rc != DQMOE_OK) return rc;
    rc = gemm::grouped_gemm(act, act_scale, b1, b1_scale, offsets, mtile_prefix, n, H, I, E, quant_mode, 0, d, nullptr,
                            nullptr, dest_to_src, nullptr, stream);
    if (rc != DQMOE_OK) return rc;
    return dqmoe_finalize_weighted(d, weights, out_bf16, T, k, H, stream);
}


int dqmoe_moe_block(const void* x_bf16, const float* logits, const void* b, const float* b_scale, const void* b1,
                    const float* b1_scale, void* out_bf16, void* workspace, size_t workspace_bytes, int T, int H,
                    int I, int E, int k, int scoring, int quant_mode, dqmoe_stream_t stream) {
    return moe_block_impl(x_bf16, logits, b, b_scale, b1, b1_scale, out_bf16, workspace, workspace_bytes, T, H, I, E,
                              k, 0, scoring, quant_mode, static_cast<cudaStream_t>(stream));
}

int dqmoe_moe_block_shared(const void* x_bf16, const float* logits, const void* b, const float* b_scale,
                           const void* b1, const float* b1_scale, void* out_bf16, void* workspace,
                           size_t workspace_bytes, int T, int H, int I, int E, int k, int n_shared, int scoring,
                           int quant_mode, dqmoe_stream_t stream) {
    return moe_block_impl(x_bf16, logits, b, b_scale, b1, b1_scale, out_bf16, workspace, workspace_bytes, T, H, I, E,
                              k, n_shared, scoring, quant_mode, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
