// Paged causal attention for prompt portions in bfloat16 on tensor cores.
//
// CTA (query tile, query head): 128 consecutive query tokens of one request against
// that request's keys, 64 keys at a time. The eight warps own 16 query rows each and
// share the key and value tiles, which all threads copy from the cache pages with
// cp.async into two shared-memory stages (rows of a tile come from up to four pages
// through the block table; rows past the tile's last needed key are zero-filled, so
// a masked probability never multiplies stale memory). S = Q K^T and O += P V are
// m16n8k16 bf16 MMAs with fp32 accumulators; the softmax is online, fp32, base 2
// with the scale folded into the exponent; P is rounded to bf16 for the second
// product. A query at position p reads keys max(0, p - window + 1) .. p. Tiles are
// listed by the host, heaviest first. The order in which a query's keys are added
// depends only on its position, not on how the prompt was cut: every portion walks
// key tiles from the same 64-aligned starts.
//
// The reference's counterpart: attn_prefill_tc_kernel,
// pulsarlm-core/inc/pulsarlm/kernels/paged_prefill.cuh:58-328.
#include "mma_helpers.cuh"

namespace {

constexpr int kBM = 128;  // query rows per CTA (eight warps of 16)
constexpr int kThreads = kBM / 16 * 32;
constexpr int kBN = 64;  // keys per tile

struct PrefillParams {
    const __nv_bfloat16* q;
    int64_t q_row_stride;
    const __nv_bfloat16* k_pool;
    const __nv_bfloat16* v_pool;
    int64_t page_stride;
    int64_t head_stride;
    int page_size;
    int n_pages;
    const int32_t* table;
    int table_width;
    const int4* tiles;  // {first token row, rows, position of the first row, entry}
    __nv_bfloat16* out;
    int64_t out_row_stride;
    int group;
    int window;
    float scale_log2;
    int32_t* status;
};

template <int HD>
__global__ void __launch_bounds__(kThreads, 2) attention_prefill_kernel(const PrefillParams p) {
    // Rows in shared memory are as long as the next multiple of 64 elements, so that the swizzle
    // (which permutes a row's first eight or sixteen chunks) stays inside the row at any head size.
    constexpr int kRowBytes = padded_row_bytes(HD);
    constexpr int kChunks = HD / 8;
    constexpr int kTileBytes = kBN * kRowBytes;
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* q_s = smem;                          // [kBM][HD]
    unsigned char* kv_s = smem + kBM * kRowBytes;       // 2 stages x (K tile, V tile)

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, tig = lane & 3;
    // heads vary fastest: with the tile list sorted longest first, a wave's CTAs are of similar length
    const int4 tile = p.tiles[blockIdx.y];
    const int row0 = tile.x, n_rows = tile.y, pos0 = tile.z;
    const int head = blockIdx.x, kv_head = head / p.group;
    const int32_t* table_row = p.table + static_cast<int64_t>(tile.w) * p.table_width;

    const int last_key = pos0 + n_rows - 1;
    const int first_key = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
    const int j0 = first_key / kBN, j1 = last_key / kBN;

    // Q tile -> shared memory (zero rows past the portion's end).
    for (int c = threadIdx.x; c < kBM * kChunks; c += kThreads) {
        const int r = c / kChunks, ch = c % kChunks;
        const __nv_bfloat16* src = p.q + (row0 + min(r, n_rows - 1)) * p.q_row_stride +
            static_cast<int64_t>(head) * HD + ch * 8;
        cp_async_16_or_zero(q_s + swizzled(r, ch, kRowBytes), src, r < n_rows);
    }
    cp_async_commit();

    auto issue = [&](int j, int stage) {
        unsigned char* k_s = kv_s + stage * 2 * kTileBytes;
        unsigned char* v_s = k_s + kTileBytes;
        for (int c = threadIdx.x; c < kBN * kChunks; c += kThreads) {
            const int r = c / kChunks, ch = c % kChunks;
            const int key = j * kBN + r;
            bool valid = key <= last_key && key >= first_key;
            int64_t offset = 0;
            if (valid) {
                const int page = table_row[key / p.page_size];
                if (page < 0 || page >= p.n_pages) {
                    if (ch == 0 && p.status != nullptr) {
                        atomicOr(p.status, 4);
                    }
                    valid = false;
                } else {
                    offset = page * p.page_stride + kv_head * p.head_stride +
                        static_cast<int64_t>(key % p.page_size) * HD + ch * 8;
                }
            }
            const int dst = swizzled(r, ch, kRowBytes);
            cp_async_16_or_zero(k_s + dst, p.k_pool + offset, valid);
            cp_async_16_or_zero(v_s + dst, p.v_pool + offset, valid);
        }
        cp_async_commit();
    };

    issue(j0, 0);
    cp_async_wait<1>();  // Q has landed (the first K/V tile may still be in flight)
    __syncthreads();

    uint32_t qa[HD / 16][4];
    {
        const int mi = lane >> 3, r = lane & 7;
        const int row = warp * 16 + (mi & 1) * 8 + r;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
            ldmatrix_x4(qa[kk], q_s + swizzled(row, 2 * kk + (mi >> 1), kRowBytes));
        }
    }

    float o[HD / 8][4];
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) {
        o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;
    }
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.0f, l_hi = 0.0f;
    const int pos_lo = pos0 + warp * 16 + g, pos_hi = pos_lo + 8;
    const int first_lo = p.window > 0 ? pos_lo - p.window + 1 : 0;
    const int first_hi = p.window > 0 ? pos_hi - p.window + 1 : 0;
    const int warp_last = pos0 + warp * 16 + 15;  // the largest position among the warp's rows

    for (int j = j0; j <= j1; ++j) {
        const int stage = (j - j0) & 1;
        if (j < j1) {
            issue(j + 1, stage ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const unsigned char* k_s = kv_s + stage * 2 * kTileBytes;
        const unsigned char* v_s = k_s + kTileBytes;
        const int key0 = j * kBN;
        // A warp whose rows all come before this tile (causal) or after it (window) has nothing to add.
        const bool warp_active = key0 <= warp_last &&
            (p.window <= 0 || key0 + kBN - 1 >= pos0 + warp * 16 - p.window + 1);
        if (warp_active) {
            float s[kBN / 8][4];
#pragma unroll
            for (int n = 0; n < kBN / 8; ++n) {
                s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.0f;
            }
            {
                const int mi = lane >> 3, r = lane & 7;
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {
#pragma unroll
                    for (int np = 0; np < kBN / 16; ++np) {
                        uint32_t b[4];
                        const int key = np * 16 + (mi >> 1) * 8 + r;
                        ldmatrix_x4(b, k_s + swizzled(key, 2 * kk + (mi & 1), kRowBytes));
                        mma_bf16(s[2 * np], qa[kk], b[0], b[1]);
                        mma_bf16(s[2 * np + 1], qa[kk], b[2], b[3]);
                    }
                }
            }
            float tile_lo = -INFINITY, tile_hi = -INFINITY;
            // Only tiles that cross the diagonal or the window's edge need the mask.
            const int warp_first = pos0 + warp * 16;
            const bool edge = key0 + kBN - 1 > warp_first || (p.window > 0 && key0 < warp_last - p.window + 1);
            if (edge) {
#pragma unroll
                for (int n = 0; n < kBN / 8; ++n) {
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int key = key0 + 8 * n + 2 * tig + e;
                        s[n][e] = (key <= pos_lo && key >= first_lo) ? s[n][e] * p.scale_log2 : -INFINITY;
                        s[n][2 + e] = (key <= pos_hi && key >= first_hi) ? s[n][2 + e] * p.scale_log2 : -INFINITY;
                    }
                    tile_lo = fmaxf(tile_lo, fmaxf(s[n][0], s[n][1]));
                    tile_hi = fmaxf(tile_hi, fmaxf(s[n][2], s[n][3]));
                }
            } else {
#pragma unroll
                for (int n = 0; n < kBN / 8; ++n) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        s[n][e] *= p.scale_log2;
                    }
                    tile_lo = fmaxf(tile_lo, fmaxf(s[n][0], s[n][1]));
                    tile_hi = fmaxf(tile_hi, fmaxf(s[n][2], s[n][3]));
                }
            }
            tile_lo = fmaxf(tile_lo, __shfl_xor_sync(0xffffffffu, tile_lo, 1));
            tile_lo = fmaxf(tile_lo, __shfl_xor_sync(0xffffffffu, tile_lo, 2));
            tile_hi = fmaxf(tile_hi, __shfl_xor_sync(0xffffffffu, tile_hi, 1));
            tile_hi = fmaxf(tile_hi, __shfl_xor_sync(0xffffffffu, tile_hi, 2));
            const float new_lo = fmaxf(m_lo, tile_lo), new_hi = fmaxf(m_hi, tile_hi);
            const float base_lo = new_lo == -INFINITY ? 0.0f : new_lo;
            const float base_hi = new_hi == -INFINITY ? 0.0f : new_hi;
            const float corr_lo = exp2f(m_lo - base_lo), corr_hi = exp2f(m_hi - base_hi);
            m_lo = new_lo;
            m_hi = new_hi;
            float sum_lo = 0.0f, sum_hi = 0.0f;
#pragma unroll
            for (int n = 0; n < kBN / 8; ++n) {
                s[n][0] = fast_exp2(s[n][0] - base_lo);
                s[n][1] = fast_exp2(s[n][1] - base_lo);
                s[n][2] = fast_exp2(s[n][2] - base_hi);
                s[n][3] = fast_exp2(s[n][3] - base_hi);
                sum_lo += s[n][0] + s[n][1];
                sum_hi += s[n][2] + s[n][3];
            }
            l_lo = l_lo * corr_lo + sum_lo;
            l_hi = l_hi * corr_hi + sum_hi;
#pragma unroll
            for (int n = 0; n < HD / 8; ++n) {
                o[n][0] *= corr_lo;
                o[n][1] *= corr_lo;
                o[n][2] *= corr_hi;
                o[n][3] *= corr_hi;
            }
            {
                const int mi = lane >> 3, r = lane & 7;
#pragma unroll
                for (int ks = 0; ks < kBN / 16; ++ks) {
                    uint32_t pa[4];
                    pa[0] = pack_bf16(s[2 * ks][0], s[2 * ks][1]);
                    pa[1] = pack_bf16(s[2 * ks][2], s[2 * ks][3]);
                    pa[2] = pack_bf16(s[2 * ks + 1][0], s[2 * ks + 1][1]);
                    pa[3] = pack_bf16(s[2 * ks + 1][2], s[2 * ks + 1][3]);
                    const int key = ks * 16 + (mi & 1) * 8 + r;
#pragma unroll
                    for (int dp = 0; dp < HD / 16; ++dp) {
                        uint32_t b[4];
                        ldmatrix_x4_trans(b, v_s + swizzled(key, 2 * dp + (mi >> 1), kRowBytes));
                        mma_bf16(o[2 * dp], pa, b[0], b[1]);
                        mma_bf16(o[2 * dp + 1], pa, b[2], b[3]);
                    }
                }
            }
        }
        __syncthreads();  // everyone is done with this stage before it is refilled
    }

    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    const float inv_lo = l_lo > 0.0f ? 1.0f / l_lo : 0.0f, inv_hi = l_hi > 0.0f ? 1.0f / l_hi : 0.0f;
    const int r_lo = warp * 16 + g, r_hi = r_lo + 8;
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) {
        const int d = 8 * n + 2 * tig;
        if (r_lo < n_rows) {
            *reinterpret_cast<uint32_t*>(p.out + (row0 + r_lo) * p.out_row_stride + static_cast<int64_t>(head) * HD +
                                         d) = pack_bf16(o[n][0] * inv_lo, o[n][1] * inv_lo);
        }
        if (r_hi < n_rows) {
            *reinterpret_cast<uint32_t*>(p.out + (row0 + r_hi) * p.out_row_stride + static_cast<int64_t>(head) * HD +
                                         d) = pack_bf16(o[n][2] * inv_hi, o[n][3] * inv_hi);
        }
    }
}

template <int HD>
int launch_prefill(const PrefillParams& p, int n_tiles, int n_heads, cudaStream_t stream) {
    constexpr int smem = kBM * padded_row_bytes(HD) + 2 * 2 * kBN * padded_row_bytes(HD);
    static bool configured = false;
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(attention_prefill_kernel<HD>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (err != cudaSuccess) {
            return pl_fail(3, "attention_prefill: cannot set shared memory size: %s", cudaGetErrorString(err));
        }
        configured = true;
    }
    attention_prefill_kernel<HD><<<dim3(n_heads, n_tiles), kThreads, smem, stream>>>(p);
    PL_CHECK_LAUNCH("attention_prefill");
    return 0;
}

}  // namespace

// Query rows per tile of pl_attention_prefill's tile list.
PL_API int pl_attention_prefill_tile_rows() { return kBM; }

PL_API int pl_attention_prefill_supports(int head_dim, int page_size, int dtype) {
    return dtype == PL_BF16 && head_dim % 16 == 0 && head_dim >= 32 && head_dim <= 128 && page_size >= 1;
}

// bf16 only. tiles: int32 [n_tiles, 4] = {first token row, rows (1..128), position of
// the first row, block-table row}; a tile's rows are consecutive tokens of one
// request at consecutive positions. q and out [T, n_heads, head_dim] with row
// strides; pools and table as in pl_attention_simt.
PL_API int pl_attention_prefill(const void* q, int64_t q_row_stride, const void* k_pool, const void* v_pool,
                                int64_t page_stride, int64_t head_stride, int page_size, int n_pages,
                                const int32_t* table, int table_width, const int32_t* tiles, int n_tiles, void* out,
                                int64_t out_row_stride, int n_heads, int n_kv_heads, int head_dim, int window,
                                float scale, int32_t* status, cudaStream_t stream) {
    PL_REQUIRE(n_tiles >= 0 && n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0,
               "attention_prefill: bad sizes tiles=%d heads=%d kv_heads=%d", n_tiles, n_heads, n_kv_heads);
    PL_REQUIRE(pl_attention_prefill_supports(head_dim, page_size, PL_BF16),
               "attention_prefill: unsupported shape head_dim=%d page=%d (takes head sizes 32 to 128 in steps of 16)", head_dim,
               page_size);
    PL_REQUIRE(n_heads <= 65535, "attention_prefill: too many heads (%d)", n_heads);
    PL_REQUIRE((reinterpret_cast<uintptr_t>(q) & 15) == 0 && q_row_stride % 8 == 0 &&
                   (reinterpret_cast<uintptr_t>(out) & 3) == 0 && out_row_stride % 2 == 0,
               "attention_prefill: q must be 16-byte aligned with a row stride that is a multiple of 8 elements");
    PL_REQUIRE((reinterpret_cast<uintptr_t>(k_pool) & 15) == 0 && (reinterpret_cast<uintptr_t>(v_pool) & 15) == 0 &&
                   page_stride % 8 == 0 && head_stride % 8 == 0 && (reinterpret_cast<uintptr_t>(tiles) & 15) == 0,
               "attention_prefill: pools and the tile list must be 16-byte aligned");
    if (n_tiles == 0) {
        return 0;
    }
    PrefillParams p;
    p.q = static_cast<const __nv_bfloat16*>(q);
    p.q_row_stride = q_row_stride;
    p.k_pool = static_cast<const __nv_bfloat16*>(k_pool);
    p.v_pool = static_cast<const __nv_bfloat16*>(v_pool);
    p.page_stride = page_stride;
    p.head_stride = head_stride;
    p.page_size = page_size;
    p.n_pages = n_pages;
    p.table = table;
    p.table_width = table_width;
    p.tiles = reinterpret_cast<const int4*>(tiles);
    p.out = static_cast<__nv_bfloat16*>(out);
    p.out_row_stride = out_row_stride;
    p.group = n_heads / n_kv_heads;
    p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.status = status;
    switch (head_dim) {
        case 32: return launch_prefill<32>(p, n_tiles, n_heads, stream);
        case 48: return launch_prefill<48>(p, n_tiles, n_heads, stream);
        case 64: return launch_prefill<64>(p, n_tiles, n_heads, stream);
        case 80: return launch_prefill<80>(p, n_tiles, n_heads, stream);
        case 96: return launch_prefill<96>(p, n_tiles, n_heads, stream);
        case 112: return launch_prefill<112>(p, n_tiles, n_heads, stream);
        default: return launch_prefill<128>(p, n_tiles, n_heads, stream);
    }
}
