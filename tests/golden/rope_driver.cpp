// Driver for the reference's own host RoPE code (pulsarlm-core/src/kernels/rope.cpp),
// compiled on the CPU against libtorch by make_rope_golden.py. It prints, as JSON,
// the reference's quadrants-per-position table and rope_rotate() of a fixed input
// for each parameter set the tests use.
#include "pulsarlm/kernels/rope.hpp"
#include "pulsarlm/kernels/rope_tables.hpp"

#include <ATen/ATen.h>

#include <cstdio>
#include <optional>
#include <vector>

namespace {

struct rope_case {
    const char* name;
    double theta;
    int64_t head_dim;
    std::optional<pulsarlm::llama3_rope_scaling> scaling;
};

void print_array(const at::Tensor& t) {
    auto flat = t.to(at::kDouble).contiguous().view({-1});
    std::printf("[");
    for (int64_t i = 0; i < flat.numel(); ++i) {
        std::printf("%s%.17g", i ? ", " : "", flat[i].item<double>());
    }
    std::printf("]");
}

}  // namespace

int main() {
    const std::vector<rope_case> cases = {
        {"tiny_a", 10000.0, 16, std::nullopt},
        {"tiny_b", 500000.0, 32, pulsarlm::llama3_rope_scaling{8.0, 1.0, 4.0, 64.0}},
        {"tiny_c", 10000.0, 64, pulsarlm::llama3_rope_scaling{4.0, 1.0, 4.0, 128.0}},
        {"llama31_8b", 500000.0, 128, pulsarlm::llama3_rope_scaling{8.0, 1.0, 4.0, 8192.0}},
    };
    const std::vector<int64_t> positions = {0, 1, 5, 63, 64, 1000, 4095, 131071};
    std::printf("{\n");
    for (size_t c = 0; c < cases.size(); ++c) {
        const rope_case& rc = cases[c];
        pulsarlm::rope_parameters rope{.theta = rc.theta, .partial_rotary_factor = 1.0, .llama3_scaling = rc.scaling};
        const at::Tensor quadrants = pulsarlm::rope_quadrants_per_position(rope, rc.head_dim, at::kCPU);
        // Fixed input: x[p, d] = sin(0.37 * d + 0.11 * p) in fp32.
        at::Tensor pos = at::tensor(positions, at::kLong);
        at::Tensor d = at::arange(rc.head_dim, at::kDouble);
        at::Tensor x = at::sin(0.37 * d.unsqueeze(0) + 0.11 * pos.to(at::kDouble).unsqueeze(1)).to(at::kFloat);
        at::Tensor rotated = pulsarlm::rope_rotate(x, pos, rope);
        std::printf("  \"%s\": {\"theta\": %.17g, \"head_dim\": %lld, \"quadrants_per_position\": ", rc.name,
                    rc.theta, static_cast<long long>(rc.head_dim));
        print_array(quadrants);
        std::printf(", \"positions\": ");
        print_array(pos);
        std::printf(", \"rotated\": ");
        print_array(rotated);
        std::printf("}%s\n", c + 1 < cases.size() ? "," : "");
    }
    std::printf("}\n");
    return 0;
}
