// Paged causal attention on CUDA cores: the float32 engine's attention, and the
// kernel that takes every head size, group size and page size in bfloat16 too.
//
// One warp per (query token, query head). The warp walks the keys of its request
// in chunks of 32 in ascending order, one key per lane for the scores, then
// accumulates the chunk's values with lane d owning output dims d, d+32, ... .
// Scores, softmax and accumulation are fp32 (expf, not the fast intrinsic). The
// walk depends only on the query's position (and the window), so a query's result
// is the same whatever else is in the batch and however the prompt was cut.
// Prefill chunks and decode tokens are the same to it: every token carries its
// position and its request's block-table row. The reference's counterpart is
// attn_scalar_kernel, pulsarlm-core/src/kernels/paged_common.cu:26-137.
#include "common.cuh"

namespace {

constexpr int kMaxAcc = 16;  // head_dim <= 512

template <typename scalar_t>
__device__ __forceinline__ float dot_row(const float* __restrict__ q, const scalar_t* __restrict__ k, int head_dim);

template <>
__device__ __forceinline__ float dot_row<float>(const float* __restrict__ q, const float* __restrict__ k,
                                                int head_dim) {
    float s = 0.0f;
    if ((head_dim & 3) == 0 && (reinterpret_cast<uintptr_t>(k) & 15) == 0) {
        const float4* k4 = reinterpret_cast<const float4*>(k);
        for (int d = 0; d < head_dim / 4; ++d) {
            const float4 kv = k4[d];
            s = fmaf(q[4 * d + 0], kv.x, s);
            s = fmaf(q[4 * d + 1], kv.y, s);
            s = fmaf(q[4 * d + 2], kv.z, s);
            s = fmaf(q[4 * d + 3], kv.w, s);
        }
    } else {
        for (int d = 0; d < head_dim; ++d) {
            s = fmaf(q[d], k[d], s);
        }
    }
    return s;
}

template <>
__device__ __forceinline__ float dot_row<__nv_bfloat16>(const float* __restrict__ q,
                                                        const __nv_bfloat16* __restrict__ k, int head_dim) {
    float s = 0.0f;
    if ((head_dim & 7) == 0 && (reinterpret_cast<uintptr_t>(k) & 15) == 0) {
        const uint4* k8 = reinterpret_cast<const uint4*>(k);
        for (int d = 0; d < head_dim / 8; ++d) {
            const uint4 raw = k8[d];
            const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                // bf16 -> fp32 is a 16-bit shift of the bit pattern.
                s = fmaf(q[8 * d + 2 * i], __uint_as_float(words[i] << 16), s);
                s = fmaf(q[8 * d + 2 * i + 1], __uint_as_float(words[i] & 0xffff0000u), s);
            }
        }
    } else {
        for (int d = 0; d < head_dim; ++d) {
            s = fmaf(q[d], __bfloat162float(k[d]), s);
        }
    }
    return s;
}

template <typename scalar_t>
__global__ void attention_simt_kernel(const scalar_t* __restrict__ q, int64_t q_row_stride,
                                      const scalar_t* __restrict__ k_pool, const scalar_t* __restrict__ v_pool,
                                      int64_t page_stride, int64_t head_stride, int page_size, int n_pages,
                                      const int32_t* __restrict__ table, int table_width,
                                      const int32_t* __restrict__ pos, const int32_t* __restrict__ entry,
                                      scalar_t* __restrict__ out, int64_t out_row_stride, int n_heads, int group,
                                      int head_dim, int window, float scale, float softcap,
                                      float* __restrict__ mass_sum, float* __restrict__ weight_sum,
                                      const float* __restrict__ query_weights, int32_t* status) {
    extern __shared__ float q_shared[];  // [warps][head_dim]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int t = blockIdx.x;
    const int kv_head = blockIdx.y;
    const int p = pos[t];
    const int first = window > 0 ? max(0, p - window + 1) : 0;
    const int32_t* row = table + static_cast<int64_t>(entry[t]) * table_width;
    float* qs = q_shared + warp * head_dim;
    const int n_acc = (head_dim + 31) / 32;

    for (int hg = warp; hg < group; hg += warps) {
        const int h = kv_head * group + hg;
        const scalar_t* qrow = q + t * q_row_stride + static_cast<int64_t>(h) * head_dim;
        __syncwarp();
        for (int d = lane; d < head_dim; d += 32) {
            qs[d] = pl_load(qrow + d);
        }
        __syncwarp();

        float m = -INFINITY, l = 0.0f;
        float acc[kMaxAcc];
#pragma unroll
        for (int i = 0; i < kMaxAcc; ++i) {
            acc[i] = 0.0f;
        }
        // Attention mass (optional): per page and head, this query's weight times its
        // largest scaled score over the page's keys it attends; per page, the weight once.
        int mass_page = -1;
        float mass_max = -INFINITY;
        auto add_mass = [&](int view_page, float page_max) {
            if (view_page < 0 || lane != 0 || !(page_max > -INFINITY)) {
                return;
            }
            const int page = row[view_page];
            if (page >= 0 && page < n_pages) {
                const float w = query_weights != nullptr ? query_weights[t] : 1.0f;
                atomicAdd(mass_sum + static_cast<int64_t>(page) * n_heads + h, w * page_max);
                if (h == 0) {
                    atomicAdd(weight_sum + page, w);
                }
            }
        };

        for (int base = (first / 32) * 32; base <= p; base += 32) {
            const int j = base + lane;
            const bool valid = j >= first && j <= p;
            int64_t offset = -1;
            float s = -INFINITY;
            if (valid) {
                const int page = row[j / page_size];
                if (page >= 0 && page < n_pages) {
                    offset = page * page_stride + kv_head * head_stride +
                        static_cast<int64_t>(j % page_size) * head_dim;
                    s = dot_row<scalar_t>(qs, k_pool + offset, head_dim) * scale;
                    if (softcap > 0.0f) {
                        s = softcap * tanhf(s / softcap);  // scores squashed into (-cap, cap) before the softmax
                    }
                } else if (status != nullptr) {
                    atomicOr(status, 4);
                }
            }
            if (mass_sum != nullptr) {
                // Largest scaled score per page; a page may span several chunks, so the
                // running maximum is flushed only when the walk leaves the page.
                const int last = min(base + 31, p);
                for (int pg = max(base, first) / page_size; pg <= last / page_size; ++pg) {
                    const float chunk_max = pl_warp_max(valid && j / page_size == pg ? s : -INFINITY);
                    if (pg != mass_page) {
                        add_mass(mass_page, mass_max);
                        mass_page = pg;
                        mass_max = chunk_max;
                    } else {
                        mass_max = fmaxf(mass_max, chunk_max);
                    }
                }
            }
            const float m_new = fmaxf(m, pl_warp_max(s));
            // m_new is -inf only if a bad block table hid every key so far.
            const bool seen = m_new > -INFINITY;
            const float corr = seen ? expf(m - m_new) : 1.0f;  // 0 on the first chunk (m = -inf)
            const float pw = offset >= 0 && seen ? expf(s - m_new) : 0.0f;
            l = l * corr + pl_warp_sum(pw);
#pragma unroll
            for (int i = 0; i < kMaxAcc; ++i) {
                if (i < n_acc) {
                    acc[i] *= corr;
                }
            }
            const int count = min(32, p - base + 1);
            for (int jj = 0; jj < count; ++jj) {
                const float pj = __shfl_sync(0xffffffffu, pw, jj);
                const int64_t oj = __shfl_sync(0xffffffffu, offset, jj);
                if (oj < 0) {
                    continue;
                }
                const scalar_t* vrow = v_pool + oj;
#pragma unroll
                for (int i = 0; i < kMaxAcc; ++i) {
                    const int d = lane + 32 * i;
                    if (i < n_acc && d < head_dim) {
                        acc[i] = fmaf(pj, pl_load(vrow + d), acc[i]);
                    }
                }
            }
            m = m_new;
        }

        if (mass_sum != nullptr) {
            add_mass(mass_page, mass_max);
        }
        const float inv = l > 0.0f ? 1.0f / l : 0.0f;
        scalar_t* orow = out + t * out_row_stride + static_cast<int64_t>(h) * head_dim;
#pragma unroll
        for (int i = 0; i < kMaxAcc; ++i) {
            const int d = lane + 32 * i;
            if (i < n_acc && d < head_dim) {
                pl_store(orow + d, acc[i] * inv);
            }
        }
    }
}

}  // namespace

// q [T, n_heads, head_dim] with q_row_stride elements between tokens; out likewise
// with out_row_stride. Token t is the query at position pos[t] of the request whose
// block-table row is table[entry[t]]; it attends keys max(0, pos - window + 1) ..
// pos (window <= 0: from 0). Pools as in pl_rope_kv_write. mass_sum [n_pages,
// n_heads] and weight_sum [n_pages] (fp32, may be nullptr) are added to: for every
// page a query attends, query_weights[t] (1 when nullptr) times the query's largest
// scaled score in the page, per head, and the weight itself once per page
// (pulsarlm-core/inc/pulsarlm/kernels/ops.hpp:150-160). softcap > 0: every scaled
// score s becomes softcap * tanh(s / softcap) before the softmax (0: off).
PL_API int pl_attention_simt(const void* q, int64_t q_row_stride, const void* k_pool, const void* v_pool,
                             int64_t page_stride, int64_t head_stride, int page_size, int n_pages,
                             const int32_t* table, int table_width, const int32_t* pos, const int32_t* entry,
                             void* out, int64_t out_row_stride, int n_tokens, int n_heads, int n_kv_heads,
                             int head_dim, int window, float scale, float softcap, int dtype, float* mass_sum,
                             float* weight_sum, const float* query_weights, int32_t* status, cudaStream_t stream) {
    PL_REQUIRE(n_tokens >= 0 && n_heads > 0 && n_kv_heads > 0 && head_dim > 0 && page_size > 0,
               "attention: bad sizes tokens=%d heads=%d kv_heads=%d head_dim=%d page=%d", n_tokens, n_heads,
               n_kv_heads, head_dim, page_size);
    PL_REQUIRE(n_heads % n_kv_heads == 0, "attention: %d query heads are not a multiple of %d kv heads", n_heads,
               n_kv_heads);
    PL_REQUIRE(head_dim <= 32 * kMaxAcc, "attention: head_dim %d exceeds the supported maximum %d", head_dim,
               32 * kMaxAcc);
    PL_REQUIRE(n_kv_heads <= 65535, "attention: %d kv heads exceed the grid limit", n_kv_heads);
    PL_REQUIRE(mass_sum == nullptr || weight_sum != nullptr, "attention: attention mass needs weight_sum too");
    if (n_tokens == 0) {
        return 0;
    }
    const int group = n_heads / n_kv_heads;
    const int warps = group < 8 ? group : 8;
    const size_t smem = static_cast<size_t>(warps) * head_dim * sizeof(float);
    const dim3 grid(n_tokens, n_kv_heads);
    PL_DISPATCH_DTYPE(dtype, "attention", {
        attention_simt_kernel<scalar_t><<<grid, warps * 32, smem, stream>>>(
            static_cast<const scalar_t*>(q), q_row_stride, static_cast<const scalar_t*>(k_pool),
            static_cast<const scalar_t*>(v_pool), page_stride, head_stride, page_size, n_pages, table, table_width,
            pos, entry, static_cast<scalar_t*>(out), out_row_stride, n_heads, group, head_dim, window, scale,
            softcap, mass_sum, weight_sum, query_weights, status);
    });
    PL_CHECK_LAUNCH("attention");
    return 0;
}
