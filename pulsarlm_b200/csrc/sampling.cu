// Sampling from rows of fp32 logits: argmax, temperature, top-k and top-p.
//
// One block per row. A drawing row returns argmax_i(x_i / T + Gumbel_i) over the
// kept tokens, which samples softmax(x / T) renormalised over them. The noise is
// Philox4x32-10 keyed by the row's seed with counter (i / 4, draw count), lane
// i % 4: a pure function of (seed, draw count, token index), so a row's draw does
// not depend on its neighbours in the batch. T <= 0 takes the argmax; ties go to
// the lower index. The reference's counterparts: gumbel_race_kernel,
// pulsarlm-core/src/kernels/gumbel_race.cu:17-80, and the top-k / top-p rule of
// src/engine/sampling.cpp:68-75 (a token stays while its rank is below top_k and
// the probability mass ranked above it is <= top_p). Here the kept set is found
// without sorting, by a bitwise search for the threshold value; tokens whose
// logits are exactly equal are kept or cut together.
#include "common.cuh"

namespace {

constexpr int kThreads = 1024;

__device__ __forceinline__ uint32_t ordered_bits(float v) {
    const uint32_t bits = __float_as_uint(v);
    return (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
}

__device__ __forceinline__ unsigned long long race_key(float score, int index) {
    return (static_cast<unsigned long long>(ordered_bits(score)) << 32) |
        (0xffffffffull - static_cast<uint32_t>(index));
}

__device__ __forceinline__ uint4 philox4x32_10(uint4 counter, uint2 key) {
    constexpr uint32_t kM0 = 0xD2511F53u, kM1 = 0xCD9E8D57u, kW0 = 0x9E3779B9u, kW1 = 0xBB67AE85u;
#pragma unroll
    for (int round = 0; round < 10; ++round) {
        const uint32_t hi0 = __umulhi(kM0, counter.x), lo0 = kM0 * counter.x;
        const uint32_t hi1 = __umulhi(kM1, counter.z), lo1 = kM1 * counter.z;
        counter = make_uint4(hi1 ^ counter.y ^ key.x, lo1, hi0 ^ counter.w ^ key.y, lo0);
        key.x += kW0;
        key.y += kW1;
    }
    return counter;
}

__device__ __forceinline__ float gumbel_from_bits(uint32_t bits) {
    // 23 bits keep the uniform strictly inside (0, 1), where the noise is finite.
    const float uniform = (static_cast<float>(bits >> 9) + 0.5f) * 0x1.0p-23f;
    return -logf(-logf(uniform));
}

__device__ __forceinline__ unsigned long long block_max_u64(unsigned long long v, unsigned long long* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, v, offset);
        v = other > v ? other : v;
    }
    __syncthreads();
    if (lane == 0) {
        scratch[warp] = v;
    }
    __syncthreads();
    v = lane < (kThreads >> 5) ? scratch[lane] : 0ull;
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, v, offset);
        v = other > v ? other : v;
    }
    return v;
}

__global__ void __launch_bounds__(kThreads)
sample_kernel(const float* __restrict__ logits, int64_t row_stride, int vocab, const float* __restrict__ temperature,
              const int32_t* __restrict__ top_k, const float* __restrict__ top_p,
              const unsigned long long* __restrict__ seed, const unsigned long long* __restrict__ draw_count,
              int32_t* __restrict__ out) {
    __shared__ float scratch[32];
    __shared__ unsigned long long scratch64[32];
    const int row = blockIdx.x;
    const float* x = logits + row * row_stride;
    const float temp = temperature[row];
    const int tid = threadIdx.x;

    if (!(temp > 0.0f)) {
        unsigned long long best = 0ull;
        // Four values a load where the row allows it, several loads in flight: one block
        // reads the whole row, and its time is the latency of its loads.
        const bool by_four = (reinterpret_cast<uintptr_t>(x) & 15) == 0;
        const int quads = by_four ? vocab / 4 : 0;
#pragma unroll 4
        for (int quad = tid; quad < quads; quad += kThreads) {
            const float4 v = reinterpret_cast<const float4*>(x)[quad];
            // the largest of the four, the lowest index among equals
            uint32_t top = ordered_bits(v.x);
            int at = 0;
            const uint32_t others[3] = {ordered_bits(v.y), ordered_bits(v.z), ordered_bits(v.w)};
#pragma unroll
            for (int j = 0; j < 3; ++j) {
                if (others[j] > top) {
                    top = others[j];
                    at = j + 1;
                }
            }
            const unsigned long long key = (static_cast<unsigned long long>(top) << 32) |
                (0xffffffffull - static_cast<uint32_t>(4 * quad + at));
            best = key > best ? key : best;
        }
        for (int i = 4 * quads + tid; i < vocab; i += kThreads) {
            const unsigned long long key = race_key(x[i], i);
            best = key > best ? key : best;
        }
        best = block_max_u64(best, scratch64);
        if (tid == 0) {
            out[row] = static_cast<int32_t>(0xffffffffu - static_cast<uint32_t>(best & 0xffffffffull));
        }
        return;
    }

    const float inv_temp = 1.0f / temp;
    const int k = top_k != nullptr ? top_k[row] : 0;
    const float p = top_p != nullptr ? top_p[row] : 1.0f;
    const bool keeps_k = k > 0 && k < vocab;
    const bool keeps_p = p > 0.0f && p < 1.0f;
    uint32_t threshold = 0u;  // kept: ordered_bits(x_i / T) >= threshold

    if (keeps_k) {
        uint32_t thr = 0u;
        for (int bit = 31; bit >= 0; --bit) {
            const uint32_t candidate = thr | (1u << bit);
            float count = 0.0f;
            for (int i = tid; i < vocab; i += kThreads) {
                count += ordered_bits(x[i] * inv_temp) >= candidate ? 1.0f : 0.0f;
            }
            if (pl_block_sum(count, scratch) >= static_cast<float>(k)) {
                thr = candidate;
            }
        }
        threshold = thr;  // the k-th largest value
    }
    if (keeps_p) {
        float local_max = -INFINITY;
        for (int i = tid; i < vocab; i += kThreads) {
            local_max = fmaxf(local_max, x[i] * inv_temp);
        }
        const float row_max = pl_block_max(local_max, scratch);
        float local_sum = 0.0f;
        for (int i = tid; i < vocab; i += kThreads) {
            local_sum += expf(x[i] * inv_temp - row_max);
        }
        const float total = pl_block_sum(local_sum, scratch);
        // Largest u with mass{value >= u} > top_p: tokens at or above it have at
        // most top_p ranked strictly above them.
        const float target = p * total;
        uint32_t thr = 0u;
        for (int bit = 31; bit >= 0; --bit) {
            const uint32_t candidate = thr | (1u << bit);
            float mass = 0.0f;
            for (int i = tid; i < vocab; i += kThreads) {
                const float v = x[i] * inv_temp;
                mass += ordered_bits(v) >= candidate ? expf(v - row_max) : 0.0f;
            }
            if (pl_block_sum(mass, scratch) > target) {
                thr = candidate;
            }
        }
        threshold = thr > threshold ? thr : threshold;
    }

    const unsigned long long s = seed[row], c = draw_count[row];
    const uint2 key = make_uint2(static_cast<uint32_t>(s), static_cast<uint32_t>(s >> 32));
    unsigned long long best = 0ull;
    const int quads = (vocab + 3) / 4;
    for (int quad = tid; quad < quads; quad += kThreads) {
        const uint4 random = philox4x32_10(
            make_uint4(static_cast<uint32_t>(quad), 0u, static_cast<uint32_t>(c), static_cast<uint32_t>(c >> 32)),
            key);
        const uint32_t bits[4] = {random.x, random.y, random.z, random.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int i = quad * 4 + j;
            if (i < vocab) {
                const float v = x[i] * inv_temp;
                if (ordered_bits(v) >= threshold) {
                    const unsigned long long candidate = race_key(v + gumbel_from_bits(bits[j]), i);
                    best = candidate > best ? candidate : best;
                }
            }
        }
    }
    best = block_max_u64(best, scratch64);
    if (tid == 0) {
        out[row] = static_cast<int32_t>(0xffffffffu - static_cast<uint32_t>(best & 0xffffffffull));
    }
}

}  // namespace

// logits [rows, vocab] fp32 with row_stride elements between rows. temperature
// [rows]; top_k [rows] (0 = off) and top_p [rows] (outside (0,1) = off) may be
// nullptr; seed and draw_count [rows] are 64-bit. out [rows] int32 token ids.
PL_API int pl_sample(const float* logits, int64_t row_stride, int n_rows, int vocab, const float* temperature,
                     const int32_t* top_k, const float* top_p, const unsigned long long* seed,
                     const unsigned long long* draw_count, int32_t* out, cudaStream_t stream) {
    PL_REQUIRE(n_rows >= 0 && vocab > 0 && row_stride >= vocab, "sample: bad sizes rows=%d vocab=%d stride=%lld",
               n_rows, vocab, static_cast<long long>(row_stride));
    if (n_rows == 0) {
        return 0;
    }
    sample_kernel<<<n_rows, kThreads, 0, stream>>>(logits, row_stride, vocab, temperature, top_k, top_p, seed,
                                                   draw_count, out);
    PL_CHECK_LAUNCH("sample");
    return 0;
}
