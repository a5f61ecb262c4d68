// Rotary position encoding of q and k, and the write of k and v into cache pages.
//
// One launch per layer: q is rotated in place; k is rotated and stored, with v, at
// the token's place in the paged cache (keys are stored rotated: positions are
// absolute and never change). The angle pos * f_j is formed in fp64 from an fp64
// table, reduced to (-pi, pi] in fp64, and only then rounded to fp32 for sincosf;
// the rotation itself is fp32. Optionally each q head and each k head is first
// normalised over its head_dim (x * rsqrt(mean(x^2) + eps) * weight[d], fp32 weights
// shared by all heads; statistics and product in fp32, one rounding when the rotated
// value is stored): the per-head q/k norm some decoders of this family put before the
// rotation. The reference rotates q in
// pulsarlm-core/src/kernels/rope.cu:33-84 and writes k, v in
// src/kernels/paged_attention.cu:52-98.
#include "rope_helpers.cuh"

namespace {

// Block (t, y) handles token t and `heads_per_block` head slots from y * heads_per_block,
// where slots 0 .. n_heads-1 are q heads (rotated in place) and the next n_kv_heads are
// k heads (rotated and stored with their v head). A decode step has few tokens: many
// small blocks (four slots each), else one block per token would walk its heads one
// after the other. A prompt portion has many: one block per token, so that the
// token's angles (fp64) are formed once and not once per four heads. Rotated pairs are
// (j, j + rotary/2) for j < rotary/2; dims >= rotary pass through unchanged.
template <typename scalar_t>
__global__ void rope_kv_write_kernel(scalar_t* __restrict__ q, const scalar_t* __restrict__ k,
                                     const scalar_t* __restrict__ v, int64_t row_stride,
                                     const int32_t* __restrict__ pos, const int32_t* __restrict__ entry,
                                     const int32_t* __restrict__ table, int table_width,
                                     scalar_t* __restrict__ k_pool, scalar_t* __restrict__ v_pool,
                                     int64_t page_stride, int64_t head_stride, int page_size, int n_pages,
                                     const double* __restrict__ inv_freq, int rotary, int n_heads, int n_kv_heads,
                                     int head_dim, int heads_per_block, const float* __restrict__ q_norm,
                                     const float* __restrict__ k_norm, float norm_eps, int32_t* status) {
    extern __shared__ float sincos[];  // [rotary/2] cos, [rotary/2] sin, then [heads_per_block] norm factors
    pl_grid_trigger();  // positions are step inputs: the angles need not wait for the projection
    const int t = blockIdx.x;
    const int p = pos[t];
    const int half = rotary / 2;
    float* cs = sincos;
    float* sn = sincos + half;
    if (inv_freq != nullptr) {
        for (int j = threadIdx.x; j < half; j += blockDim.x) {
            rope_sincos(p, inv_freq[j], cs[j], sn[j]);
        }
    }
    const int n_slots = n_heads + (k_pool != nullptr ? n_kv_heads : 0);
    const int slot0 = blockIdx.y * heads_per_block;
    const int slot1 = min(slot0 + heads_per_block, n_slots);
    int page = -1;
    if (slot1 > n_heads) {  // (the block table is a step input too: looked up before the wait)
        page = table[static_cast<int64_t>(entry[t]) * table_width + p / page_size];
        if (page < 0 || page >= n_pages) {
            if (threadIdx.x == 0 && status != nullptr) {
                atomicOr(status, 2);
            }
            page = -1;
        }
    }
    pl_grid_wait();
    float* factor = sincos + rotary;  // per slot of this block: rsqrt(mean(x^2) + eps), or 1
    if (q_norm != nullptr || k_norm != nullptr) {
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
        for (int slot = slot0 + warp; slot < slot1; slot += warps) {
            const bool is_q = slot < n_heads;
            float sum = 0.0f;
            if (is_q ? q_norm != nullptr : k_norm != nullptr) {
                const scalar_t* x = is_q ? q + t * row_stride + static_cast<int64_t>(slot) * head_dim
                                         : k + t * row_stride + static_cast<int64_t>(slot - n_heads) * head_dim;
                for (int d = lane; d < head_dim; d += 32) {
                    const float value = pl_load(x + d);
                    sum = fmaf(value, value, sum);
                }
                sum = pl_warp_sum(sum);
                if (lane == 0) {
                    factor[slot - slot0] = rsqrtf(sum / static_cast<float>(head_dim) + norm_eps);
                }
            } else if (lane == 0) {
                factor[slot - slot0] = 1.0f;
            }
        }
    }
    __syncthreads();

    const int pairs = head_dim - half;  // per head: `half` rotated pairs, then the unrotated dims
    for (int idx = threadIdx.x; idx < (slot1 - slot0) * pairs; idx += blockDim.x) {
        const int slot = slot0 + idx / pairs, j = idx % pairs;
        if (slot < n_heads) {
            scalar_t* x = q + t * row_stride + static_cast<int64_t>(slot) * head_dim;
            if (q_norm != nullptr) {
                const float r = factor[slot - slot0];
                if (inv_freq == nullptr || j >= half) {  // unrotated dims: normalised only
                    const int d0 = j >= half ? j + half : j;
                    pl_store(x + d0, pl_load(x + d0) * r * q_norm[d0]);
                    if (j < half) {
                        pl_store(x + j + half, pl_load(x + j + half) * r * q_norm[j + half]);
                    }
                    continue;
                }
                const float lo = pl_load(x + j) * r * q_norm[j], hi = pl_load(x + j + half) * r * q_norm[j + half];
                pl_store(x + j, rope_lo(lo, hi, cs[j], sn[j]));
                pl_store(x + j + half, rope_hi(lo, hi, cs[j], sn[j]));
                continue;
            }
            if (inv_freq == nullptr || j >= half) {
                continue;  // q passes through
            }
            const float lo = pl_load(x + j), hi = pl_load(x + j + half);
            pl_store(x + j, rope_lo(lo, hi, cs[j], sn[j]));
            pl_store(x + j + half, rope_hi(lo, hi, cs[j], sn[j]));
        } else if (page >= 0) {
            const int h = slot - n_heads;
            const scalar_t* x = k + t * row_stride + static_cast<int64_t>(h) * head_dim;
            const scalar_t* y = v + t * row_stride + static_cast<int64_t>(h) * head_dim;
            const int64_t at = page * page_stride + h * head_stride + static_cast<int64_t>(p % page_size) * head_dim;
            const float r = k_norm != nullptr ? factor[slot - slot0] : 1.0f;
            if (j < half) {
                float lo = pl_load(x + j), hi = pl_load(x + j + half);
                if (k_norm != nullptr) {
                    lo *= r * k_norm[j];
                    hi *= r * k_norm[j + half];
                }
                if (inv_freq != nullptr) {
                    pl_store(k_pool + at + j, rope_lo(lo, hi, cs[j], sn[j]));
                    pl_store(k_pool + at + j + half, rope_hi(lo, hi, cs[j], sn[j]));
                } else if (k_norm != nullptr) {
                    pl_store(k_pool + at + j, lo);
                    pl_store(k_pool + at + j + half, hi);
                } else {
                    k_pool[at + j] = x[j];
                    k_pool[at + j + half] = x[j + half];
                }
                v_pool[at + j] = y[j];
                v_pool[at + j + half] = y[j + half];
            } else {
                const int d = j + half;  // dims rotary .. head_dim-1
                if (k_norm != nullptr) {
                    pl_store(k_pool + at + d, pl_load(x + d) * r * k_norm[d]);
                } else {
                    k_pool[at + d] = x[d];
                }
                v_pool[at + d] = y[d];
            }
        }
    }
}

// The same with four consecutive dims per thread (8- or 16-byte loads), for shapes
// where the rotated half, the unrotated tail and the row stride are multiples of 4.
template <typename scalar_t>
__global__ void rope_kv_write_vec_kernel(scalar_t* __restrict__ q, const scalar_t* __restrict__ k,
                                         const scalar_t* __restrict__ v, int64_t row_stride,
                                         const int32_t* __restrict__ pos, const int32_t* __restrict__ entry,
                                         const int32_t* __restrict__ table, int table_width,
                                         scalar_t* __restrict__ k_pool, scalar_t* __restrict__ v_pool,
                                         int64_t page_stride, int64_t head_stride, int page_size, int n_pages,
                                         const double* __restrict__ inv_freq, int rotary, int n_heads,
                                         int n_kv_heads, int head_dim, int heads_per_block,
                                         const float* __restrict__ q_norm, const float* __restrict__ k_norm,
                                         float norm_eps, int32_t* status) {
    extern __shared__ float sincos[];
    pl_grid_trigger();
    const int t = blockIdx.x;
    const int p = pos[t];
    const int half = rotary / 2;
    float* cs = sincos;
    float* sn = sincos + half;
    if (inv_freq != nullptr) {
        for (int j = threadIdx.x; j < half; j += blockDim.x) {
            rope_sincos(p, inv_freq[j], cs[j], sn[j]);
        }
    }
    const int n_slots = n_heads + (k_pool != nullptr ? n_kv_heads : 0);
    const int slot0 = blockIdx.y * heads_per_block;
    const int slot1 = min(slot0 + heads_per_block, n_slots);
    int page = -1;
    if (slot1 > n_heads) {  // (the block table is a step input too: looked up before the wait)
        page = table[static_cast<int64_t>(entry[t]) * table_width + p / page_size];
        if (page < 0 || page >= n_pages) {
            if (threadIdx.x == 0 && status != nullptr) {
                atomicOr(status, 2);
            }
            page = -1;
        }
    }
    pl_grid_wait();
    float* factor = sincos + rotary;  // per slot of this block: rsqrt(mean(x^2) + eps), or 1
    if (q_norm != nullptr || k_norm != nullptr) {
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
        for (int slot = slot0 + warp; slot < slot1; slot += warps) {
            const bool is_q = slot < n_heads;
            float sum = 0.0f;
            if (is_q ? q_norm != nullptr : k_norm != nullptr) {
                const scalar_t* x = is_q ? q + t * row_stride + static_cast<int64_t>(slot) * head_dim
                                         : k + t * row_stride + static_cast<int64_t>(slot - n_heads) * head_dim;
                for (int d = lane; d < head_dim; d += 32) {
                    const float value = pl_load(x + d);
                    sum = fmaf(value, value, sum);
                }
                sum = pl_warp_sum(sum);
                if (lane == 0) {
                    factor[slot - slot0] = rsqrtf(sum / static_cast<float>(head_dim) + norm_eps);
                }
            } else if (lane == 0) {
                factor[slot - slot0] = 1.0f;
            }
        }
    }
    __syncthreads();

    const int groups = (head_dim - half) / 4;  // per head: half/4 rotated groups, then the unrotated tail
    for (int idx = threadIdx.x; idx < (slot1 - slot0) * groups; idx += blockDim.x) {
        const int slot = slot0 + idx / groups, j = 4 * (idx % groups);
        if (slot < n_heads) {
            if (inv_freq == nullptr || j >= half) {
                continue;
            }
            scalar_t* x = q + t * row_stride + static_cast<int64_t>(slot) * head_dim;
            const float4 lo = pl_load4(x + j), hi = pl_load4(x + j + half);
            const float4 c = *reinterpret_cast<const float4*>(cs + j), s = *reinterpret_cast<const float4*>(sn + j);
            pl_store4(x + j, make_float4(rope_lo(lo.x, hi.x, c.x, s.x), rope_lo(lo.y, hi.y, c.y, s.y),
                                         rope_lo(lo.z, hi.z, c.z, s.z), rope_lo(lo.w, hi.w, c.w, s.w)));
            pl_store4(x + j + half, make_float4(rope_hi(lo.x, hi.x, c.x, s.x), rope_hi(lo.y, hi.y, c.y, s.y),
                                                rope_hi(lo.z, hi.z, c.z, s.z), rope_hi(lo.w, hi.w, c.w, s.w)));
        } else if (page >= 0) {
            const int h = slot - n_heads;
            const scalar_t* x = k + t * row_stride + static_cast<int64_t>(h) * head_dim;
            const scalar_t* y = v + t * row_stride + static_cast<int64_t>(h) * head_dim;
            const int64_t at = page * page_stride + h * head_stride + static_cast<int64_t>(p % page_size) * head_dim;
            if (j < half) {
                const float4 lo = pl_load4(x + j), hi = pl_load4(x + j + half);
                if (inv_freq != nullptr) {
                    const float4 c = *reinterpret_cast<const float4*>(cs + j);
                    const float4 s = *reinterpret_cast<const float4*>(sn + j);
                    pl_store4(k_pool + at + j, make_float4(rope_lo(lo.x, hi.x, c.x, s.x), rope_lo(lo.y, hi.y, c.y, s.y),
                                                           rope_lo(lo.z, hi.z, c.z, s.z), rope_lo(lo.w, hi.w, c.w, s.w)));
                    pl_store4(k_pool + at + j + half,
                              make_float4(rope_hi(lo.x, hi.x, c.x, s.x), rope_hi(lo.y, hi.y, c.y, s.y),
                                          rope_hi(lo.z, hi.z, c.z, s.z), rope_hi(lo.w, hi.w, c.w, s.w)));
                } else {
                    pl_store4(k_pool + at + j, lo);
                    pl_store4(k_pool + at + j + half, hi);
                }
                pl_store4(v_pool + at + j, pl_load4(y + j));
                pl_store4(v_pool + at + j + half, pl_load4(y + j + half));
            } else {
                const int d = j + half;
                pl_store4(k_pool + at + d, pl_load4(x + d));
                pl_store4(v_pool + at + d, pl_load4(y + d));
            }
        }
    }
}

}  // namespace

// q [T, n_heads, head_dim], k and v [T, n_kv_heads, head_dim], all with `row_stride`
// elements between tokens (they may be slices of one fused projection output).
// Pools: element (page, head, slot, d) of K at k_pool[page * page_stride + head *
// head_stride + slot * head_dim + d], V likewise. inv_freq == nullptr: no rotation.
// k_pool == nullptr: only q is rotated (a layer that reads another layer's cache).
// q_norm, k_norm: fp32 [head_dim] scales of a per-head RMS norm applied before the
// rotation (nullptr: none), with norm_eps inside the root.
PL_API int pl_rope_kv_write(void* q, const void* k, const void* v, int64_t row_stride, const int32_t* pos,
                            const int32_t* entry, const int32_t* table, int table_width, void* k_pool,
                            void* v_pool, int64_t page_stride, int64_t head_stride, int page_size, int n_pages,
                            const double* inv_freq, int rotary, int n_tokens, int n_heads, int n_kv_heads,
                            int head_dim, int dtype, const float* q_norm, const float* k_norm, float norm_eps,
                            int32_t* status, cudaStream_t stream) {
    PL_REQUIRE(n_tokens >= 0 && n_heads > 0 && n_kv_heads > 0 && head_dim > 0 && page_size > 0,
               "rope_kv_write: bad sizes tokens=%d heads=%d kv_heads=%d head_dim=%d page=%d", n_tokens, n_heads,
               n_kv_heads, head_dim, page_size);
    PL_REQUIRE(rotary >= 0 && rotary <= head_dim && rotary % 2 == 0,
               "rope_kv_write: rotary width %d must be even and at most head_dim %d", rotary, head_dim);
    if (n_tokens == 0) {
        return 0;
    }
    const int n_slots = n_heads + (k_pool != nullptr ? n_kv_heads : 0);
    const int heads_per_block = n_tokens >= 64 ? n_slots : 4;
    const size_t smem = static_cast<size_t>(rotary + heads_per_block) * sizeof(float);
    PL_REQUIRE(smem <= 48 * 1024, "rope_kv_write: rotary width %d and %d heads are too large", rotary, n_slots);
    PL_REQUIRE(k_norm == nullptr || k_pool != nullptr, "rope_kv_write: a k norm needs keys to write");
    const dim3 grid(n_tokens, (n_slots + heads_per_block - 1) / heads_per_block);
    PL_REQUIRE(grid.y <= 65535, "rope_kv_write: too many heads (%d)", n_slots);
    const int half = rotary / 2;
    const uintptr_t align = dtype == PL_F32 ? 15 : 7;
    const bool vec = q_norm == nullptr && k_norm == nullptr && half % 4 == 0 && (head_dim - rotary) % 4 == 0 && head_dim % 4 == 0 && row_stride % 4 == 0 &&
        page_stride % 4 == 0 && head_stride % 4 == 0 && (reinterpret_cast<uintptr_t>(q) & align) == 0 &&
        (reinterpret_cast<uintptr_t>(k) & align) == 0 && (reinterpret_cast<uintptr_t>(v) & align) == 0 &&
        (reinterpret_cast<uintptr_t>(k_pool) & align) == 0 && (reinterpret_cast<uintptr_t>(v_pool) & align) == 0;
    const int items = heads_per_block * (head_dim - half) / (vec ? 4 : 1);
    const int threads = items >= 256 ? 256 : (items >= 128 ? 128 : 64);
    PL_DISPATCH_DTYPE(dtype, "rope_kv_write", {
        auto kernel = vec ? rope_kv_write_vec_kernel<scalar_t> : rope_kv_write_kernel<scalar_t>;
        pl_launch_overlapped(
            kernel, grid, threads, smem, stream, static_cast<scalar_t*>(q), static_cast<const scalar_t*>(k), static_cast<const scalar_t*>(v), row_stride,
            pos, entry, table, table_width, static_cast<scalar_t*>(k_pool), static_cast<scalar_t*>(v_pool),
            page_stride, head_stride, page_size, n_pages, inv_freq, rotary, n_heads, n_kv_heads, head_dim,
            heads_per_block, q_norm, k_norm, norm_eps, status);
    });
    PL_CHECK_LAUNCH("rope_kv_write");
    return 0;
}
