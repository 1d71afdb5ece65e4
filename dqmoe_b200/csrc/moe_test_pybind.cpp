// The `moe_test` extension module of the reference (csrc/python_api.cu:9-17), rebuilt over the C ABI of
// libdqmoe_b200.so: the three functions register_apis exports (csrc/pybind11_register.h:153-163) with the
// same names, argument lists (std::pair<Tensor, Tensor> operands, `fused` defaulting to true), shape checks
// and error text, forwarding to dqmoe_moe_forward on the current torch stream. Unlike the reference it
// sets the device of `a` as current for the call (the reference assumes device 0, csrc/moe_kernels.h:633)
// and compares the workspace size with what the layer needs.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <sstream>
#include <stdexcept>
#include <string>
#include <utility>

#include "../../include/dqmoe.h"

namespace {

[[noreturn]] void fail(const char* file, int line, const std::string& cond, const std::string& info = "") {
    std::ostringstream os;  // the form of throwCheckError, csrc/util.h:143-152
    os << "[ASSERT FAILED] " << file << ":" << line << "  Condition: " << cond;
    if (!info.empty()) os << "  Info: " << info;
    throw std::runtime_error(os.str());
}
#define MT_CHECK(cond, ...) \
    do {                    \
        if (!(cond)) fail("moe_test_pybind.cpp", __LINE__, #cond, std::string(__VA_ARGS__)); \
    } while (0)

void check_rc(int rc) {
    if (rc != DQMOE_OK) throw std::runtime_error(dqmoe_last_error());
}

using TensorPair = std::pair<torch::Tensor, torch::Tensor>;

void run(const TensorPair& a, const TensorPair& b, const TensorPair& b1, const torch::Tensor& d,
         const torch::Tensor& m_indices, const torch::Tensor& workspace, int quant_mode_value, bool fused, bool fp8) {
    const torch::Tensor& a0 = a.first;
    const torch::Tensor& b0 = b.first;
    const torch::Tensor& b10 = b1.first;
    // shape checks of csrc/pybind11_register.h:108-123
    MT_CHECK(a0.dim() == 2 && b0.dim() == 3 && b10.dim() == 3 && d.dim() == 3 && m_indices.dim() == 2,
             "a [T,H], b [E,2I,H], b1 [E,H,I], d [T,k,H], m_indices [T,k]");
    const int64_t num_tokens = a0.size(0), hidden_size = a0.size(1);
    const int64_t num_groups = b0.size(0), inter_size_2 = b0.size(1), hidden_size_ = b0.size(2);
    const int64_t num_tokens_ = d.size(0), topk = d.size(1), hidden_size__ = d.size(2);
    const int64_t num_groups_ = b10.size(0), hidden_size___ = b10.size(1), inter_size = b10.size(2);
    MT_CHECK(num_tokens == num_tokens_ && num_groups == num_groups_ && hidden_size == hidden_size_ &&
             hidden_size == hidden_size__ && hidden_size == hidden_size___ && inter_size * 2 == inter_size_2);
    MT_CHECK(m_indices.size(0) == num_tokens && m_indices.size(1) == topk, "m_indices.shape == (num_tokens, topk)");
    MT_CHECK(m_indices.scalar_type() == torch::kInt);
    if (num_tokens == 0) return;  // csrc/pybind11_register.h:125-126
    const auto want = fp8 ? torch::kFloat8_e4m3fn : torch::kBFloat16;
    MT_CHECK(a0.scalar_type() == want && b0.scalar_type() == want && b10.scalar_type() == want,
             fp8 ? "a, b, b1 data tensors are float8_e4m3fn" : "a, b, b1 data tensors are bfloat16");
    MT_CHECK(d.scalar_type() == torch::kBFloat16);
    for (const torch::Tensor* t : {&a0, &b0, &b10, &d, &m_indices, &workspace}) {
        MT_CHECK(t->is_cuda(), "dqmoe_b200 has no CPU path");
        MT_CHECK(t->is_contiguous());
    }
    const float* sfa = nullptr;
    const float* sfb = nullptr;
    const float* sfb1 = nullptr;
    int mode = 0;
    if (fp8) {
        MT_CHECK(quant_mode_value == 256 || quant_mode_value == 512 || quant_mode_value == 1024 || quant_mode_value == 2048,
                 "got " + std::to_string(quant_mode_value));
        // 2048 = MXFP8, an added mode (include/dqmoe.h): its scale tensors hold UE8M0 bytes
        const auto want_s = quant_mode_value == 2048 ? torch::kByte : torch::kFloat;
        for (const torch::Tensor* s : {&a.second, &b.second, &b1.second})
            MT_CHECK(s->scalar_type() == want_s && s->is_contiguous() && s->is_cuda(),
                     "scale tensors are contiguous CUDA tensors, fp32 (UE8M0 bytes in the MXFP8 mode)");
        sfa = static_cast<const float*>(a.second.data_ptr());
        sfb = static_cast<const float*>(b.second.data_ptr());
        sfb1 = static_cast<const float*>(b1.second.data_ptr());
        mode = quant_mode_value;
    }
    // bf16: the scale halves are dummy tensors (test/util.py:232-234) and are not read
    MT_CHECK(reinterpret_cast<uintptr_t>(workspace.data_ptr()) % 256 == 0,
             "workspace pointer is not aligned!");  // csrc/pybind11_register.h:141-142
    const c10::cuda::CUDAGuard guard(a0.device());
    cudaStream_t stream = at::cuda::getCurrentCUDAStream().stream();
    check_rc(dqmoe_moe_forward(a0.data_ptr(), sfa, b0.data_ptr(), sfb, b10.data_ptr(), sfb1, d.data_ptr(),
                               m_indices.data_ptr<int32_t>(), workspace.data_ptr(),
                               static_cast<size_t>(workspace.numel()) * workspace.element_size(), int(num_tokens),
                               int(hidden_size), int(inter_size), int(num_groups), int(topk), mode, fused ? 1 : 0,
                               static_cast<dqmoe_stream_t>(stream)));
}

void m_grouped_moe_nt_contiguous_fp8_bf16(const TensorPair& a, const TensorPair& b, const TensorPair& b1,
                                          const torch::Tensor& d, const torch::Tensor& m_indices,
                                          const torch::Tensor& workspace, int quant_mode_value, bool fused) {
    run(a, b, b1, d, m_indices, workspace, quant_mode_value, fused, true);
}

void m_grouped_moe_nt_contiguous_bf16(const TensorPair& a, const TensorPair& b, const TensorPair& b1,
                                      const torch::Tensor& d, const torch::Tensor& m_indices,
                                      const torch::Tensor& workspace, int quant_mode_value, bool fused) {
    (void) quant_mode_value;  // ignored like the scale halves
    run(a, b, b1, d, m_indices, workspace, 0, fused, false);
}

// csrc/torch_help.h:37-52: the same values with MN-major strides (mn * sf_k, 1, mn); the input itself when it
// already has them. Pure tensor bookkeeping, no kernel of this library.
torch::Tensor get_mn_major_tma_aligned_tensor(const torch::Tensor& sf) {
    MT_CHECK(sf.dim() == 2 || sf.dim() == 3, "dim == 2 or dim == 3");
    MT_CHECK(sf.scalar_type() == torch::kFloat);
    const bool two = sf.dim() == 2;
    torch::Tensor batched = two ? sf.unsqueeze(0) : sf;
    const int64_t g = batched.size(0), mn = batched.size(1), sf_k = batched.size(2);
    if ((batched.stride(0) == mn * sf_k || two) && batched.stride(1) == 1 && batched.stride(2) == mn)
        return two ? batched.squeeze(0) : batched;
    torch::Tensor out = torch::empty_strided({g, mn, sf_k}, {mn * sf_k, 1, mn}, batched.options());
    out.copy_(batched);
    return two ? out.squeeze(0) : out;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "moe_test: the DQMoE operator surface over libdqmoe_b200.so (sm_100a)";
    m.def("get_mn_major_tma_aligned_tensor", &get_mn_major_tma_aligned_tensor, py::arg("sf"));
    m.def("m_grouped_moe_nt_contiguous_fp8_bf16", &m_grouped_moe_nt_contiguous_fp8_bf16, py::arg("a"), py::arg("b"),
          py::arg("b1"), py::arg("d"), py::arg("m_indices"), py::arg("workspace"), py::arg("quant_mode_value"),
          py::arg("fused") = true);
    m.def("m_grouped_moe_nt_contiguous_bf16", &m_grouped_moe_nt_contiguous_bf16, py::arg("a"), py::arg("b"),
          py::arg("b1"), py::arg("d"), py::arg("m_indices"), py::arg("workspace"), py::arg("quant_mode_value"),
          py::arg("fused") = true);
}
