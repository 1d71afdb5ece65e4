// Plugin-shaped front end of the layer: a descriptor built from the nine creation fields of the
// reference's "mixture_of_experts" TensorRT plugin (test/trt_test.py:97-135), a workspace-size
// query, an enqueue that takes the plugin's input list in its order
// (test/trt_test.py:140-150: input, weight1, weight2, index, bias1, bias2, actscale, scale_a,
// scale_b) and one output, and a flat serialisation of the fields. It is what an
// IPluginV2DynamicExt::enqueue / getWorkspaceSize / serialize of a TensorRT build would call;
// no TensorRT type appears here.
#include <cuda_fp16.h>

#include <cstring>
#include <new>

#include "common.cuh"

struct dqmoe_plugin {
    dqmoe_plugin_fields f;
};

namespace dq {
namespace plugin {

constexpr size_t kAlign = 256;

// bf16 -> fp16 / fp32, 8 elements per thread and step
template <typename Out>
__global__ void __launch_bounds__(256) convert_kernel(const __nv_bfloat16* __restrict__ in, Out* __restrict__ out,
                                                      size_t n8) {
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n8; i += size_t(gridDim.x) * blockDim.x) {
        const Vec16 v = ld_nc16(reinterpret_cast<const uint8_t*>(in) + i * 16);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        float f[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            f[2 * j] = __uint_as_float(w[j] << 16);
            f[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
        }
        if constexpr (sizeof(Out) == 2) {
            uint32_t p[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const __half2 h = __floats2half2_rn(f[2 * j], f[2 * j + 1]);
                p[j] = *reinterpret_cast<const uint32_t*>(&h);
            }
            st16(reinterpret_cast<uint8_t*>(out) + i * 16, Vec16{p[0], p[1], p[2], p[3]});
        } else {
            uint8_t* o = reinterpret_cast<uint8_t*>(out) + i * 32;
            st16(o, Vec16{__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3])});
            st16(o + 16, Vec16{__float_as_uint(f[4]), __float_as_uint(f[5]), __float_as_uint(f[6]), __float_as_uint(f[7])});
        }
    }
}

static int validate(const dqmoe_plugin_fields& f) {
    DQ_CHECK_FMT(f.number_of_experts > 0 && f.number_of_experts <= 1024, "number_of_experts=%d", f.number_of_experts);
    DQ_CHECK_FMT(f.top_k > 0 && f.top_k <= 32, "top_k=%d", f.top_k);
    DQ_CHECK_FMT(f.expert_hidden_size > 0 && f.expert_hidden_size % 16 == 0, "expert_hidden_size=%d",
                 f.expert_hidden_size);
    DQ_CHECK_FMT(f.expert_inter_size > 0 && f.expert_inter_size % 16 == 0, "expert_inter_size=%d", f.expert_inter_size);
    DQ_CHECK_FMT(f.max_num_tokens >= 0, "max_num_tokens=%d", f.max_num_tokens);
    DQ_CHECK_FMT(f.use_bias == 0 || f.use_bias == 1, "use_bias=%d", f.use_bias);
    DQ_CHECK_FMT(f.type == DQMOE_DT_FP8 || f.type == DQMOE_DT_BF16 || f.type == DQMOE_DT_HALF || f.type == DQMOE_DT_FLOAT,
                 "type=%d: operands are FP8 (6), BF16 (7), HALF (1) or FLOAT (0)", f.type);
    DQ_CHECK_FMT(f.output_type == DQMOE_DT_BF16 || f.output_type == DQMOE_DT_HALF || f.output_type == DQMOE_DT_FLOAT,
                 "output_type=%d", f.output_type);
    if (f.type == DQMOE_DT_HALF)
        DQ_CHECK_FMT(f.output_type == DQMOE_DT_HALF, "output_type=%d: HALF operands give HALF output", f.output_type);
    if (f.type == DQMOE_DT_FLOAT)
        DQ_CHECK_FMT(f.output_type == DQMOE_DT_FLOAT, "output_type=%d: FLOAT operands give FLOAT output", f.output_type);
    if (f.type == DQMOE_DT_BF16 || f.type == DQMOE_DT_HALF || f.type == DQMOE_DT_FLOAT)
        DQ_CHECK_FMT(f.quant_mode == DQMOE_QUANT_NONE, "quant_mode=%d with unquantised operands", f.quant_mode);
    else
        DQ_CHECK_FMT(f.quant_mode == DQMOE_QUANT_FP8_TENSOR || f.quant_mode == DQMOE_QUANT_FP8_CHANNEL ||
                         f.quant_mode == DQMOE_QUANT_FP8_BLOCK || f.quant_mode == DQMOE_QUANT_FP8_MX,
                     "quant_mode=%d with FP8 operands", f.quant_mode);
    if (f.quant_mode == DQMOE_QUANT_FP8_MX)
        DQ_CHECK_FMT(f.expert_hidden_size % 128 == 0 && f.expert_inter_size % 128 == 0,
                     "expert_hidden_size=%d and expert_inter_size=%d must be multiples of 128 in the MXFP8 mode",
                     f.expert_hidden_size, f.expert_inter_size);
    return DQMOE_OK;
}

static size_t layer_bytes(const dqmoe_plugin_fields& f, int T) {
    if (f.type == DQMOE_DT_FLOAT)
        return align_up(dqmoe_moe_workspace_bytes_f32(T, f.expert_hidden_size, f.expert_inter_size, f.number_of_experts,
                                                      f.top_k),
                        kAlign);
    return align_up(dqmoe_moe_workspace_bytes(T, f.expert_hidden_size, f.expert_inter_size, f.number_of_experts, f.top_k,
                                              f.quant_mode),
                    kAlign);
}

}  // namespace plugin
}  // namespace dq

using namespace dq;

extern "C" {

int dqmoe_plugin_create(const dqmoe_plugin_fields* fields, dqmoe_plugin** out) {
    DQ_CHECK(fields != nullptr && out != nullptr);
    *out = nullptr;
    const int rc = plugin::validate(*fields);
    if (rc != DQMOE_OK) return rc;
    dqmoe_plugin* p = new (std::nothrow) dqmoe_plugin;
    DQ_CHECK(p != nullptr);
    p->f = *fields;
    *out = p;
    return DQMOE_OK;
}

void dqmoe_plugin_destroy(dqmoe_plugin* p) { delete p; }

int dqmoe_plugin_get_fields(const dqmoe_plugin* p, dqmoe_plugin_fields* out) {
    DQ_CHECK(p != nullptr && out != nullptr);
    *out = p->f;
    return DQMOE_OK;
}

size_t dqmoe_plugin_workspace_size(const dqmoe_plugin* p, int num_tokens) {
    if (p == nullptr || num_tokens < 0 || num_tokens > p->f.max_num_tokens) return 0;
    size_t bytes = plugin::layer_bytes(p->f, num_tokens);
    if (p->f.type != DQMOE_DT_HALF && p->f.type != DQMOE_DT_FLOAT && p->f.output_type != DQMOE_DT_BF16)  // bf16 result staged for conversion
        bytes += align_up(size_t(num_tokens) * p->f.top_k * p->f.expert_hidden_size * 2, plugin::kAlign);
    return bytes;
}

int dqmoe_plugin_enqueue(const dqmoe_plugin* p, int num_tokens, const void* const* inputs, void* const* outputs,
                         void* workspace, dqmoe_stream_t stream_) {
    DQ_CHECK(p != nullptr && inputs != nullptr && outputs != nullptr);
    const dqmoe_plugin_fields& f = p->f;
    DQ_CHECK_FMT(num_tokens >= 0 && num_tokens <= f.max_num_tokens, "num_tokens=%d exceeds max_num_tokens=%d", num_tokens,
                 f.max_num_tokens);
    if (num_tokens == 0) return DQMOE_OK;
    DQ_CHECK(outputs[0] != nullptr);
    DQ_CHECK_FMT(workspace != nullptr && is_aligned(workspace, plugin::kAlign), "workspace pointer %p is not aligned!",
                 workspace);
    const bool fp8 = f.quant_mode != DQMOE_QUANT_NONE;
    const int T = num_tokens, H = f.expert_hidden_size, I = f.expert_inter_size, E = f.number_of_experts, k = f.top_k;
    const size_t lbytes = plugin::layer_bytes(f, T);
    const float* bias1 = f.use_bias ? static_cast<const float*>(inputs[4]) : nullptr;
    const float* bias2 = f.use_bias ? static_cast<const float*>(inputs[5]) : nullptr;
    if (f.use_bias) DQ_CHECK(bias1 != nullptr && bias2 != nullptr);
    if (f.type == DQMOE_DT_HALF)
        return dqmoe_moe_forward_f16_bias(inputs[0], inputs[1], inputs[2], bias1, bias2, outputs[0],
                                          static_cast<const int32_t*>(inputs[3]), workspace, lbytes, T, H, I, E, k, stream_);
    if (f.type == DQMOE_DT_FLOAT)
        return dqmoe_moe_forward_f32(inputs[0], inputs[1], inputs[2], bias1, bias2, outputs[0],
                                     static_cast<const int32_t*>(inputs[3]), workspace, lbytes, T, H, I, E, k, stream_);
    void* d = f.output_type == DQMOE_DT_BF16 ? outputs[0] : static_cast<char*>(workspace) + lbytes;
    int rc = dqmoe_moe_forward_bias(inputs[0], fp8 ? static_cast<const float*>(inputs[6]) : nullptr, inputs[1],
                                    fp8 ? static_cast<const float*>(inputs[7]) : nullptr, inputs[2],
                                    fp8 ? static_cast<const float*>(inputs[8]) : nullptr, bias1, bias2, d,
                                    static_cast<const int32_t*>(inputs[3]), workspace, lbytes, T, H, I, E, k,
                                    f.quant_mode, stream_);
    if (rc != DQMOE_OK || f.output_type == DQMOE_DT_BF16) return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const size_t n8 = size_t(T) * k * H / 8;  // H is a multiple of 16
    const int blocks = int(n8 / 256 + 1 < size_t(sm_count()) * 8 ? n8 / 256 + 1 : size_t(sm_count()) * 8);
    DQ_CHECK(is_aligned(outputs[0], 16));
    if (f.output_type == DQMOE_DT_HALF)
        plugin::convert_kernel<__half><<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(d),
                                                                   static_cast<__half*>(outputs[0]), n8);
    else
        plugin::convert_kernel<float><<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(d),
                                                                  static_cast<float*>(outputs[0]), n8);
    DQ_LAUNCH_CHECK();
    return DQMOE_OK;
}

size_t dqmoe_plugin_serialization_size(void) { return sizeof(dqmoe_plugin_fields); }

int dqmoe_plugin_serialize(const dqmoe_plugin* p, void* buffer, size_t bytes) {
    DQ_CHECK(p != nullptr && buffer != nullptr && bytes >= sizeof(dqmoe_plugin_fields));
    std::memcpy(buffer, &p->f, sizeof(dqmoe_plugin_fields));
    return DQMOE_OK;
}

int dqmoe_plugin_deserialize(const void* buffer, size_t bytes, dqmoe_plugin** out) {
    DQ_CHECK(buffer != nullptr && out != nullptr);
    DQ_CHECK_FMT(bytes == sizeof(dqmoe_plugin_fields), "serialised plugin has %zu bytes, expected %zu", bytes,
                 sizeof(dqmoe_plugin_fields));
    dqmoe_plugin_fields f;
    std::memcpy(&f, buffer, sizeof(f));
    return dqmoe_plugin_create(&f, out);
}

}  // extern "C"
