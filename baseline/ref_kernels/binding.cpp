// Python bindings over the reference's kernel library (pulsarlm-core/src/kernels), compiled
// unmodified from the reference's tree. This file is this repository's own: it declares
// nothing but pass-through functions, plus one stand-in (see decode_fits below).
//
// What is bound: rmsnorm_cuda, rope_cuda, silu_mul_cuda, attn_prefill_cuda (float32 runs the
// reference's scalar kernel, bfloat16 its tensor-core kernel), rope_rotate (host) and
// gumbel_race_cuda. What is not: attn_decode_cuda and write_kv_cuda, whose file
// (src/kernels/paged_attention.cu) needs a newer host compiler than g++ 13
// ("error: 'HD' is not captured", paged_attention.cu:613); the reference asks for gcc 15.
#include <torch/extension.h>

#include <optional>

#include "pulsarlm/kernels/ops.hpp"
#include "pulsarlm/kernels/rope.hpp"

namespace pulsarlm::attn {
// Declared in the reference's attn_common.cuh (a CUDA header) and defined in paged_attention.cu, which does not compile here. It is only
// asked whether the decode kernel's tiles fit shared memory before a half-precision launch
// of either attention kernel; the shapes bound below (pages of 16 or 32, head sizes 64 and
// 128) fit on every device the reference supports, so the stand-in says yes.
bool decode_fits(int64_t, int64_t) { return true; }
}  // namespace pulsarlm::attn

namespace {

pulsarlm::rope_parameters make_rope(double theta, double partial, std::optional<std::vector<double>> llama3) {
    pulsarlm::rope_parameters rope{theta, partial, std::nullopt};
    if (llama3) {
        TORCH_CHECK(llama3->size() == 4, "llama3 scaling: factor, low, high, original_max_position_embeddings");
        rope.llama3_scaling = pulsarlm::llama3_rope_scaling{(*llama3)[0], (*llama3)[1], (*llama3)[2], (*llama3)[3]};
    }
    return rope;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("rmsnorm", [](const at::Tensor& x, const at::Tensor& w, double eps) {
        return pulsarlm::rmsnorm_cuda(x, w, eps);
    });
    m.def("rope", [](const at::Tensor& x, const at::Tensor& pos, double theta, double partial,
                     std::optional<std::vector<double>> llama3) {
        return pulsarlm::rope_cuda(x, pos, make_rope(theta, partial, llama3));
    });
    m.def("rope_rotate_host", [](const at::Tensor& x, const at::Tensor& pos, double theta, double partial,
                                 std::optional<std::vector<double>> llama3) {
        return pulsarlm::rope_rotate(x, pos, make_rope(theta, partial, llama3));
    });
    m.def("silu_mul", [](const at::Tensor& x) { return pulsarlm::silu_mul_cuda(x); });
    m.def("gumbel_race", [](const at::Tensor& scores, const at::Tensor& temperatures, const at::Tensor& draws) {
        return pulsarlm::gumbel_race_cuda(scores, temperatures, draws);
    });
    m.def("attn_prefill",
          [](const at::Tensor& q, const at::Tensor& k_pool, const at::Tensor& v_pool, const at::Tensor& page_tables,
             const at::Tensor& cu_seqlens_q, const at::Tensor& seqlens_k, const at::Tensor& page_positions,
             double theta, double partial, std::optional<std::vector<double>> llama3, double scale,
             std::optional<int64_t> sliding_window, std::optional<at::Tensor> mass_sum,
             std::optional<at::Tensor> weight_sum, std::optional<at::Tensor> cu_view_pages,
             std::optional<at::Tensor> query_weights) {
              return pulsarlm::attn_prefill_cuda(q, k_pool, v_pool, page_tables, cu_seqlens_q, seqlens_k,
                                                 page_positions, make_rope(theta, partial, llama3), scale,
                                                 sliding_window, std::nullopt, mass_sum, weight_sum, cu_view_pages,
                                                 query_weights);
          });
}
