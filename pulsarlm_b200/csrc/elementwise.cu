// Embedding gather, fused residual-add + RMSNorm, and SwiGLU.
//
// The residual stream is fp32 in both engine dtypes: sums of layer outputs are
// never rounded to bfloat16. Norm statistics, the SiLU and the products are fp32
// with one rounding on store.
#include "common.cuh"

#include <algorithm>

namespace {

// x[t, :] = table[tokens[t], :] as fp32. An id outside [0, vocab) writes zeros and
// raises bit 0 of *status (the host validates ids first; this only keeps a bad id
// from reading outside the table).
template <typename scalar_t>
__global__ void embed_kernel(const scalar_t* __restrict__ table, const int32_t* __restrict__ tokens,
                             float* __restrict__ x, int hidden, int vocab, int32_t* status) {
    pl_grid_trigger();
    pl_grid_wait();
    const int t = blockIdx.x;
    const int token = tokens[t];
    float* row = x + static_cast<int64_t>(t) * hidden;
    if (token < 0 || token >= vocab) {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            row[i] = 0.0f;
        }
        if (threadIdx.x == 0 && status != nullptr) {
            atomicOr(status, 1);
        }
        return;
    }
    const scalar_t* src = table + static_cast<int64_t>(token) * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        row[i] = pl_load(src + i);
    }
}

// tokens[i] = ids[source[i]] where source[i] >= 0 (other rows keep what the host wrote).
__global__ void take_tokens_kernel(int32_t* __restrict__ tokens, const int32_t* __restrict__ source,
                                   const int32_t* __restrict__ ids, int n, int n_ids, int32_t* status) {
    pl_grid_trigger();
    pl_grid_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) {
        return;
    }
    const int from = source[i];
    if (from >= n_ids) {
        if (status != nullptr) {
            atomicOr(status, 1);  // (as a bad token id: the row keeps the host's value)
        }
    } else if (from >= 0) {
        tokens[i] = ids[from];
    }
}

// One block per output row r; source row s = rows ? rows[r] : r.
//   v = x[s] + delta[s]   (delta optional)
//   x[s] = v              (only when rows == nullptr)
//   out[r] = v * rsqrt(mean(v^2) + eps) * weight
// The block size depends on `hidden` alone, so a row's sum of squares is added in
// the same order whatever else is in the batch.
template <typename scalar_t, typename weight_t>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const scalar_t* __restrict__ delta,
                                   const weight_t* __restrict__ weight, scalar_t* __restrict__ out,
                                   const int32_t* __restrict__ rows, int hidden, float eps) {
    pl_grid_trigger();
    pl_grid_wait();
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const int64_t s = rows != nullptr ? rows[r] : r;
    float* xr = x + s * hidden;
    const scalar_t* dr = delta != nullptr ? delta + s * hidden : nullptr;
    scalar_t* outr = out + static_cast<int64_t>(r) * hidden;
    const bool write_back = rows == nullptr && dr != nullptr;

    float local = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float v = xr[i];
        if (dr != nullptr) {
            v += pl_load(dr + i);
        }
        if (write_back) {
            xr[i] = v;
        }
        local += v * v;
    }
    const float total = pl_block_sum(local, scratch);
    const float inv_rms = rsqrtf(total / static_cast<float>(hidden) + eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float v = xr[i];
        if (dr != nullptr && !write_back) {
            v += pl_load(dr + i);
        }
        pl_store(outr + i, v * inv_rms * pl_load(weight + i));
    }
}

// The same as add_rmsnorm_kernel for widths that are multiples of 4, with 16-byte
// loads and the row kept in registers between the two passes (VECS float4 per
// thread). The sum of squares is again added in an order fixed by the width.
template <typename scalar_t, typename weight_t, int VECS>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ x, const scalar_t* __restrict__ delta,
                                       const weight_t* __restrict__ weight, scalar_t* __restrict__ out,
                                       const int32_t* __restrict__ rows, int hidden, float eps) {
    pl_grid_trigger();
    __shared__ float scratch[32];
    const int n_vec = hidden / 4;
    float4 w[VECS];  // the norm's scale is a weight: read before the wait on earlier kernels
#pragma unroll
    for (int i = 0; i < VECS; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        w[i] = c < n_vec ? pl_load4(weight + 4 * c) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    pl_grid_wait();
    const int r = blockIdx.x;
    const int64_t s = rows != nullptr ? rows[r] : r;  // (rows may be written by an earlier kernel: after the wait)
    float* xr = x + s * hidden;
    const scalar_t* dr = delta != nullptr ? delta + s * hidden : nullptr;
    scalar_t* outr = out + static_cast<int64_t>(r) * hidden;
    const bool write_back = rows == nullptr && dr != nullptr;

    float4 v[VECS];
    float local = 0.0f;
#pragma unroll
    for (int i = 0; i < VECS; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < n_vec) {
            v[i] = pl_load4(xr + 4 * c);
            if (dr != nullptr) {
                const float4 d = pl_load4(dr + 4 * c);
                v[i].x += d.x;
                v[i].y += d.y;
                v[i].z += d.z;
                v[i].w += d.w;
            }
            if (write_back) {
                pl_store4(xr + 4 * c, v[i]);
            }
            local += v[i].x * v[i].x;
            local += v[i].y * v[i].y;
            local += v[i].z * v[i].z;
            local += v[i].w * v[i].w;
        }
    }
    const float total = pl_block_sum(local, scratch);
    const float inv_rms = rsqrtf(total / static_cast<float>(hidden) + eps);
#pragma unroll
    for (int i = 0; i < VECS; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < n_vec) {
            pl_store4(outr + 4 * c, make_float4(v[i].x * inv_rms * w[i].x, v[i].y * inv_rms * w[i].y,
                                                v[i].z * inv_rms * w[i].z, v[i].w * inv_rms * w[i].w));
        }
    }
}

// out[t, i..i+7] = silu(gate) * up, eight elements (16 bytes of bf16) per thread and
// two such chunks in flight. The result is rounded to bfloat16, so the exponential and
// the division are the fast forms (errors near 2^-21).
__device__ __forceinline__ uint4 swiglu8(const uint4 g, const uint4 u) {
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
    uint32_t ow[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 gf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gw[i]));
        const float2 uf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&uw[i]));
        const __nv_bfloat162 o = __floats2bfloat162_rn(__fdividef(gf.x, 1.0f + __expf(-gf.x)) * uf.x,
                                                       __fdividef(gf.y, 1.0f + __expf(-gf.y)) * uf.y);
        ow[i] = *reinterpret_cast<const uint32_t*>(&o);
    }
    return make_uint4(ow[0], ow[1], ow[2], ow[3]);
}

__global__ void swiglu_bf16x8_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out,
                                     int64_t tokens, int width) {
    pl_grid_trigger();
    pl_grid_wait();
    const int chunks = width / 8;
    const int64_t total = tokens * chunks;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    for (; idx + stride < total; idx += 2 * stride) {
        const int64_t t0 = idx / chunks, t1 = (idx + stride) / chunks;
        const int c0 = static_cast<int>(idx - t0 * chunks), c1 = static_cast<int>(idx + stride - t1 * chunks);
        const uint4 g0 = *reinterpret_cast<const uint4*>(in + t0 * 2 * width + 8 * c0);
        const uint4 u0 = *reinterpret_cast<const uint4*>(in + t0 * 2 * width + width + 8 * c0);
        const uint4 g1 = *reinterpret_cast<const uint4*>(in + t1 * 2 * width + 8 * c1);
        const uint4 u1 = *reinterpret_cast<const uint4*>(in + t1 * 2 * width + width + 8 * c1);
        *reinterpret_cast<uint4*>(out + t0 * width + 8 * c0) = swiglu8(g0, u0);
        *reinterpret_cast<uint4*>(out + t1 * width + 8 * c1) = swiglu8(g1, u1);
    }
    if (idx < total) {
        const int64_t t = idx / chunks;
        const int c = static_cast<int>(idx - t * chunks);
        const uint4 g = *reinterpret_cast<const uint4*>(in + t * 2 * width + 8 * c);
        const uint4 u = *reinterpret_cast<const uint4*>(in + t * 2 * width + width + 8 * c);
        *reinterpret_cast<uint4*>(out + t * width + 8 * c) = swiglu8(g, u);
    }
}

// out[t, i] = silu(in[t, i]) * in[t, width + i], silu(z) = z / (1 + exp(-z)).
template <typename scalar_t>
__global__ void swiglu_kernel(const scalar_t* __restrict__ in, scalar_t* __restrict__ out, int64_t tokens,
                              int width) {
    pl_grid_trigger();
    pl_grid_wait();
    const int64_t total = tokens * width;
    for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
         idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t t = idx / width;
        const int i = static_cast<int>(idx - t * width);
        const float g = pl_load(in + t * 2 * width + i);
        const float u = pl_load(in + t * 2 * width + width + i);
        pl_store(out + idx, g / (1.0f + expf(-g)) * u);
    }
}

// dst[i] = float(src[i]).
__global__ void bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ src, float* __restrict__ dst, int64_t n) {
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        dst[i] = __bfloat162float(src[i]);
    }
}

int norm_threads(int hidden) {
    int threads = 32;
    while (threads < 1024 && threads * 4 < hidden) {
        threads *= 2;
    }
    return threads;
}

}  // namespace

PL_API int pl_embed(const void* table, const int32_t* tokens, float* x, int n_tokens, int hidden, int vocab,
                    int dtype, int32_t* status, cudaStream_t stream) {
    PL_REQUIRE(n_tokens >= 0 && hidden > 0 && vocab > 0, "embed: bad sizes tokens=%d hidden=%d vocab=%d", n_tokens,
               hidden, vocab);
    if (n_tokens == 0) {
        return 0;
    }
    const int threads = hidden >= 1024 ? 256 : 128;
    PL_DISPATCH_DTYPE(dtype, "embed", {
        pl_launch_overlapped(embed_kernel<scalar_t>, n_tokens, threads, 0, stream,
                             static_cast<const scalar_t*>(table), tokens, x, hidden, vocab, status);
    });
    PL_CHECK_LAUNCH("embed");
    return 0;
}

// The tokens of entries that go on from a step still under way: tokens[i] = ids[source[i]]
// for the rows with source[i] >= 0 (ids: the int32 token ids that step is drawing, n_ids of
// them, on the device). Ordered on the stream after whatever writes ids.
PL_API int pl_take_tokens(int32_t* tokens, const int32_t* source, const int32_t* ids, int n, int n_ids,
                          int32_t* status, cudaStream_t stream) {
    PL_REQUIRE(n >= 0 && n_ids >= 0 && tokens != nullptr && source != nullptr && (ids != nullptr || n_ids == 0),
               "take_tokens: bad arguments n=%d ids=%d", n, n_ids);
    if (n == 0) {
        return 0;
    }
    pl_launch_overlapped(take_tokens_kernel, (n + 127) / 128, 128, 0, stream, tokens, source, ids, n, n_ids, status);
    PL_CHECK_LAUNCH("take_tokens");
    return 0;
}

PL_API int pl_add_rmsnorm(float* x, const void* delta, const void* weight, int weight_dtype, void* out,
                          const int32_t* rows, int n_rows, int hidden, float eps, int dtype, cudaStream_t stream) {
    PL_REQUIRE(n_rows >= 0 && hidden > 0, "add_rmsnorm: bad sizes rows=%d hidden=%d", n_rows, hidden);
    PL_REQUIRE(weight_dtype == PL_F32 || weight_dtype == dtype,
               "add_rmsnorm: weight dtype %d must be fp32 or the engine dtype %d", weight_dtype, dtype);
    if (n_rows == 0) {
        return 0;
    }
    const bool aligned = hidden % 4 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
        (reinterpret_cast<uintptr_t>(delta) & 15) == 0 && (reinterpret_cast<uintptr_t>(weight) & 15) == 0 &&
        (reinterpret_cast<uintptr_t>(out) & 15) == 0;
    if (aligned && hidden <= 16384) {
        // Widths that are multiples of 4: 16-byte loads, one pass over memory.
        const int n_vec = hidden / 4;
        int threads = 32;
        while (threads < 1024 && threads < n_vec) {
            threads *= 2;
        }
        const int vecs = (n_vec + threads - 1) / threads;
#define PL_LAUNCH_NORM(W, V)                                                                              \
    pl_launch_overlapped(add_rmsnorm_vec_kernel<scalar_t, W, V>, n_rows, threads, 0, stream, x,           \
                         static_cast<const scalar_t*>(delta), static_cast<const W*>(weight),              \
                         static_cast<scalar_t*>(out), rows, hidden, eps)
        PL_DISPATCH_DTYPE(dtype, "add_rmsnorm", {
            if (weight_dtype == PL_F32) {
                if (vecs == 1) { PL_LAUNCH_NORM(float, 1); } else if (vecs == 2) { PL_LAUNCH_NORM(float, 2); } else { PL_LAUNCH_NORM(float, 4); }
            } else {
                if (vecs == 1) { PL_LAUNCH_NORM(scalar_t, 1); } else if (vecs == 2) { PL_LAUNCH_NORM(scalar_t, 2); } else { PL_LAUNCH_NORM(scalar_t, 4); }
            }
        });
#undef PL_LAUNCH_NORM
        PL_CHECK_LAUNCH("add_rmsnorm");
        return 0;
    }
    const int threads = norm_threads(hidden);
    PL_DISPATCH_DTYPE(dtype, "add_rmsnorm", {
        if (weight_dtype == PL_F32) {
            pl_launch_overlapped(add_rmsnorm_kernel<scalar_t, float>, n_rows, threads, 0, stream, x,
                                 static_cast<const scalar_t*>(delta), static_cast<const float*>(weight),
                                 static_cast<scalar_t*>(out), rows, hidden, eps);
        } else {
            pl_launch_overlapped(add_rmsnorm_kernel<scalar_t, scalar_t>, n_rows, threads, 0, stream, x,
                                 static_cast<const scalar_t*>(delta), static_cast<const scalar_t*>(weight),
                                 static_cast<scalar_t*>(out), rows, hidden, eps);
        }
    });
    PL_CHECK_LAUNCH("add_rmsnorm");
    return 0;
}

PL_API int pl_swiglu(const void* in, void* out, int n_tokens, int width, int dtype, cudaStream_t stream) {
    PL_REQUIRE(n_tokens >= 0 && width > 0, "swiglu: bad sizes tokens=%d width=%d", n_tokens, width);
    if (n_tokens == 0) {
        return 0;
    }
    const int threads = 256;
    if (dtype == PL_BF16 && width % 8 == 0 && (reinterpret_cast<uintptr_t>(in) & 15) == 0 &&
        (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
        const int64_t chunks = static_cast<int64_t>(n_tokens) * (width / 8);
        const int blocks = static_cast<int>(std::min<int64_t>((chunks + threads - 1) / threads, 148 * 32));
        pl_launch_overlapped(swiglu_bf16x8_kernel, blocks, threads, 0, stream, static_cast<const __nv_bfloat16*>(in),
                             static_cast<__nv_bfloat16*>(out), n_tokens, width);
        PL_CHECK_LAUNCH("swiglu");
        return 0;
    }
    const int64_t total = static_cast<int64_t>(n_tokens) * width;
    const int blocks = static_cast<int>(std::min<int64_t>((total + threads - 1) / threads, 148 * 16));
    PL_DISPATCH_DTYPE(dtype, "swiglu", {
        pl_launch_overlapped(swiglu_kernel<scalar_t>, blocks, threads, 0, stream, static_cast<const scalar_t*>(in),
                             static_cast<scalar_t*>(out), n_tokens, width);
    });
    PL_CHECK_LAUNCH("swiglu");
    return 0;
}

PL_API int pl_bf16_to_f32(const void* src, float* dst, int64_t n, cudaStream_t stream) {
    if (n <= 0) {
        return 0;
    }
    const int threads = 256;
    const int blocks = static_cast<int>(std::min<int64_t>((n + threads - 1) / threads, 148 * 16));
    bf16_to_f32_kernel<<<blocks, threads, 0, stream>>>(static_cast<const __nv_bfloat16*>(src), dst, n);
    PL_CHECK_LAUNCH("bf16_to_f32");
    return 0;
}

// ---------------------------------------------------------------------------
// Random weights drawn in place (see random_values.h): out[i] = offset + scale * noise(i).
#include "random_values.h"

namespace {

template <typename scalar_t>
__global__ void fill_random_kernel(scalar_t* __restrict__ out, int64_t n, uint64_t key, float scale, float offset) {
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const float value = pl_random_value(key, static_cast<uint64_t>(i), scale, offset);
        if constexpr (sizeof(scalar_t) == 2) {
            reinterpret_cast<uint16_t*>(out)[i] = pl_random_bf16_bits(value);
        } else {
            out[i] = value;
        }
    }
}

}  // namespace

// out (fp32 or bf16, n elements) = offset + scale * noise, the noise a function of
// (seed, tensor_hash, element index) alone; the host core's plh_fill_random gives the
// same bits.
PL_API int pl_fill_random(void* out, int64_t n, int dtype, uint64_t seed, uint64_t tensor_hash, float scale,
                          float offset, cudaStream_t stream) {
    PL_REQUIRE(n >= 0, "fill_random: negative size");
    if (n == 0) {
        return 0;
    }
    const uint64_t key = pl_random_key(seed, tensor_hash);
    const int blocks = static_cast<int>(n / 1024 + 1 < 148 * 16 ? n / 1024 + 1 : 148 * 16);
    PL_DISPATCH_DTYPE(dtype, "fill_random", {
        fill_random_kernel<scalar_t><<<blocks, 256, 0, stream>>>(static_cast<scalar_t*>(out), n, key, scale, offset);
    });
    PL_CHECK_LAUNCH("fill_random");
    return 0;
}
