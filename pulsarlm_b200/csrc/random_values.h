// Random weights that are the same numbers wherever they are drawn.
//
// value(seed, tensor, i) is a function of a seed, a 64-bit hash of the tensor's name
// and the element's index alone: a counter-based generator. It is computed with
// integer arithmetic up to one conversion to float and one multiply (and one add for
// "1 + noise" tensors), each a single IEEE operation, so the host's copy (the host
// core, for model folders) and the device's (a kernel, for models made in place) give
// identical bits. The noise is the sum of eight 16-bit uniforms from two rounds of
// splitmix64, centred and scaled to unit variance: close to normal, within 4.9
// standard deviations. The reference draws random weights only in its tests
// (pulsarlm-core/tests/model/test_llama.cpp:47-79).
#pragma once

#include <cstdint>

#if defined(__CUDACC__)
#define PL_RANDOM_FN __host__ __device__ inline
#else
#define PL_RANDOM_FN inline
#endif

PL_RANDOM_FN uint64_t pl_splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

// The key of one tensor's stream.
PL_RANDOM_FN uint64_t pl_random_key(uint64_t seed, uint64_t tensor_hash) {
    return pl_splitmix64(pl_splitmix64(seed) ^ tensor_hash);
}

// Sum of eight 16-bit uniforms minus its mean: an integer in [-262140, 262140] with
// standard deviation sqrt(8 * (2^32 - 1) / 12).
PL_RANDOM_FN int32_t pl_random_centred_sum(uint64_t key, uint64_t index) {
    const uint64_t a = pl_splitmix64(key + index * 0xD1342543DE82EF95ull);
    const uint64_t b = pl_splitmix64(a);
    uint32_t sum = 0;
    for (int i = 0; i < 4; ++i) {
        sum += static_cast<uint32_t>((a >> (16 * i)) & 0xFFFFu) + static_cast<uint32_t>((b >> (16 * i)) & 0xFFFFu);
    }
    return static_cast<int32_t>(sum) - 262140;
}

// 1 / that standard deviation, as the float both sides multiply by.
#define PL_RANDOM_INV_STD 1.8688124e-05f

// Round-to-nearest-even of a finite float to bfloat16's bits.
PL_RANDOM_FN uint16_t pl_random_bf16_bits(float value) {
    union {
        float f;
        uint32_t u;
    } bits;
    bits.f = value;
    const uint32_t rounding = 0x7FFFu + ((bits.u >> 16) & 1u);
    return static_cast<uint16_t>((bits.u + rounding) >> 16);
}

// offset + scale * noise for element `index`, every operation rounded on its own.
PL_RANDOM_FN float pl_random_value(uint64_t key, uint64_t index, float scale, float offset) {
    const float noise = static_cast<float>(pl_random_centred_sum(key, index));
#if defined(__CUDA_ARCH__)
    const float value = __fmul_rn(noise, __fmul_rn(scale, PL_RANDOM_INV_STD));
    return offset != 0.0f ? __fadd_rn(offset, value) : value;
#else
    const volatile float factor = scale * PL_RANDOM_INV_STD;
    const volatile float value = noise * factor;
    return offset != 0.0f ? offset + value : value;
#endif
}
