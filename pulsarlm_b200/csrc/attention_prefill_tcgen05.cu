// Paged causal attention for prompt portions on the 5th-generation tensor cores.
//
// CTA (query tile of 128 tokens, query head). Both products run as tcgen05 MMAs with
// M = 128 query rows and accumulators in tensor memory:
//   S  = Q K^T   M 128 x N 64 keys  x K head_dim  (Q and K tiles K-major in smem)
//   PV = P V     M 128 x N head_dim x K 64 keys   (P K-major, V as stored: N-major)
// Roles: warp 0 loads tiles with TMA (Q once; per 64-key tile the K and V rows of
// four 16-key page pieces, found through the block table), warp 1 issues the MMAs,
// warps 2-9 are two softmax warpgroups that share each query row: thread pairs
// (one per warpgroup) read the two halves of the row's S from tensor memory, agree
// on the row maximum through shared memory, do the online softmax in fp32 (base 2,
// scale folded in), write their half of P as bf16 into shared memory for the second
// product, and fold their half of each tile's PV into an fp32 output row kept in
// registers (o = o * correction + PV). Two warps per scheduler hide each other's
// latencies. S, P and PV are double-buffered, so the MMAs of tile j+1 run while the
// softmax of tile j is computed.
//
// Every mbarrier wait is bounded; on a timeout the CTA raises bit 8 of the status
// word, stops, lets loads in flight land, frees its tensor memory and returns.
//
// Takes head_dim 64 or 128 and pages that are multiples of 16 tokens in the cache
// manager's layout [page][K,V][kv head][slot][dim]; other shapes go to the mma.sync
// kernel in attention_prefill.cu. The reference's counterpart: attn_prefill_tc_kernel,
// pulsarlm-core/inc/pulsarlm/kernels/paged_prefill.cuh:58-328.
#include "tcgen05_helpers.cuh"

namespace {

constexpr int kRows = 128;     // query rows per CTA
constexpr int kKeys = 64;      // keys per tile
constexpr int kPiece = 16;     // keys per TMA box (a page, or a part of one)
constexpr int kStagesKV = 3;
constexpr int kThreadsTc = 320;  // TMA warp, MMA warp, two softmax warpgroups

struct TcPrefillParams {
    const int32_t* table;
    int table_width;
    const int4* tiles;  // {first token row, rows, position of the first row, block-table row}
    __nv_bfloat16* out;
    int64_t out_row_stride;
    int group;
    int n_kv_heads;
    int page_size;
    int n_pages;
    int window;
    float scale_log2;
    int32_t* status;
};

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Descriptor of an N-major (MN-major) operand with 128-byte swizzle: 64-element
// groups along N are `n_group_bytes` apart, groups of 8 rows along K 1024 bytes.
__device__ __forceinline__ uint64_t smem_descriptor_mn(const void* tile, uint32_t n_group_bytes) {
    const uint64_t address = (smem_u32(tile) >> 4) & 0x3FFFu;
    return address | (static_cast<uint64_t>((n_group_bytes >> 4) & 0x3FFFu) << 16) |
        (static_cast<uint64_t>(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

template <int HD>
__global__ void __launch_bounds__(kThreadsTc, 1)
attention_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                                 const __grid_constant__ CUtensorMap map_v, const TcPrefillParams p) {
    constexpr int kHalves = HD / 64;                       // 64-dim (128-byte) column groups of a row
    constexpr int kBytesQ = kRows * HD * 2;                // kHalves sub-tiles of [128 x 64]
    constexpr int kBytesK = kKeys * HD * 2;                // kHalves sub-tiles of [64 x 64]
    constexpr int kBytesStage = 2 * kBytesK;               // K then V
    constexpr int kBytesP = kRows * kKeys * 2;             // [128 x 64]
    constexpr uint32_t kColsS = kKeys, kColsPV = HD;
    constexpr uint32_t kColumns = 2 * kColsS + 2 * kColsPV <= 256 ? 256 : 512;
    // instruction descriptors: fp32 accumulate, bf16 operands, M = 128
    constexpr uint32_t kIdescS = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(kKeys >> 3) << 17) |
        (static_cast<uint32_t>(kRows >> 4) << 24);
    constexpr uint32_t kIdescPV = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) |  // B is N-major
        (static_cast<uint32_t>(HD >> 3) << 17) | (static_cast<uint32_t>(kRows >> 4) << 24);

    extern __shared__ unsigned char raw_smem[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) &
                                                           ~static_cast<uintptr_t>(1023));
    unsigned char* q_s = smem;
    unsigned char* kv_s = q_s + kBytesQ;
    unsigned char* p_s = kv_s + kStagesKV * kBytesStage;

    __shared__ __align__(8) uint64_t q_full, kv_full[kStagesKV], kv_empty[kStagesKV];
    __shared__ __align__(8) uint64_t s_full[2], s_free[2], p_full[2], p_free[2], pv_full[2], pv_free[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;
    __shared__ float half_max[2][2 * kRows];  // [tile parity][warpgroup * 128 + row]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int4 tile = p.tiles[blockIdx.x];
    const int row0 = tile.x, n_rows = tile.y, pos0 = tile.z;
    const int head = blockIdx.y, kv_head = head / p.group;
    const int last_key = pos0 + n_rows - 1;
    const int first_key = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
    const int j0 = first_key / kKeys, n_tiles = last_key / kKeys - j0 + 1;

    if (threadIdx.x == 0) {
        mbar_init(&q_full, 1);
        for (int s = 0; s < kStagesKV; ++s) {
            mbar_init(&kv_full[s], 1);
            mbar_init(&kv_empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&s_full[b], 1);
            mbar_init(&s_free[b], 8);  // one arrival per softmax warp
            mbar_init(&p_full[b], 8);
            mbar_init(&p_free[b], 1);
            mbar_init(&pv_full[b], 1);
            mbar_init(&pv_free[b], 8);
        }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        tcgen05_alloc(&tmem_base_slot, kColumns);
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    const uint32_t tmem_s = tmem_base, tmem_pv = tmem_base + 2 * kColsS;

    if (warp == 0) {
        // ------------------------------------------------ producer
        // Lane 0 waits and issues; all lanes look up block-table entries, 32 pieces
        // (eight tiles) at a time in one load each, so that the table's latency is
        // paid once per eight tiles and not once per piece.
        if (lane == 0) {
            mbar_expect_tx(&q_full, kBytesQ);
            for (int h = 0; h < kHalves; ++h) {
                tma_load_2d(q_s + h * (kRows * 128), &map_q, head * HD + h * 64, row0, &q_full);
            }
        }
        const int32_t* table_row = p.table + static_cast<int64_t>(tile.w) * p.table_width;
        constexpr int kPieces = kKeys / kPiece;  // per tile
        int my_key = 0, my_page = 0;
        for (int j = 0; j < n_tiles; ++j) {
            if (j % (32 / kPieces) == 0) {
                // Pieces outside [first_key, last_key] are never attended (masked): they
                // are filled from the nearest needed piece, whose page is held.
                my_key = (j0 + j) * kKeys + lane * kPiece;
                my_key = min(max(my_key, (first_key / kPiece) * kPiece), (last_key / kPiece) * kPiece);
                my_page = table_row[my_key / p.page_size];
                if (my_page < 0 || my_page >= p.n_pages) {
                    if (my_key <= (last_key / kPiece) * kPiece && p.status != nullptr) {
                        atomicOr(p.status, 4);
                    }
                    my_page = 0;
                }
            }
            const int stage = j % kStagesKV;
            int ok = 1;
            if (lane == 0) {
                ok = mbar_wait(&kv_empty[stage], ((j / kStagesKV) & 1) ^ 1u, &abort_flag) ? 1 : 0;
            }
            if (!__shfl_sync(0xffffffffu, ok, 0)) {
                break;
            }
            unsigned char* k_s = kv_s + stage * kBytesStage;
            unsigned char* v_s = k_s + kBytesK;
            if (lane == 0) {
                mbar_expect_tx(&kv_full[stage], kBytesStage);
            }
            // One warp instruction issues the tile's loads: lane = (piece, half, K or V).
            __syncwarp();
            {
                const int piece = lane / (2 * kHalves), h = (lane / 2) % kHalves, is_v = lane & 1;
                const int from = (j % (32 / kPieces)) * kPieces + (piece % kPieces);
                const int key = __shfl_sync(0xffffffffu, my_key, from);
                const int page = __shfl_sync(0xffffffffu, my_page, from);
                if (lane < kPieces * kHalves * 2) {
                    const int row = ((page * 2) * p.n_kv_heads + kv_head) * p.page_size + key % p.page_size;
                    const int at = h * (kKeys * 128) + piece * (kPiece * 128);
                    tma_load_2d((is_v ? v_s : k_s) + at, is_v ? &map_v : &map_k, h * 64, row, &kv_full[stage]);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer
        if (lane == 0) {
            auto issue_s = [&](int j) {  // S_j = Q K_j^T into buffer j & 1
                const unsigned char* k_s = kv_s + (j % kStagesKV) * kBytesStage;
                const uint32_t d = tmem_s + (j & 1) * kColsS;
#pragma unroll
                for (int h = 0; h < kHalves; ++h) {
                    const uint64_t da = smem_descriptor(q_s + h * (kRows * 128));
                    const uint64_t db = smem_descriptor(k_s + h * (kKeys * 128));
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        tcgen05_mma(d, da + 2 * k, db + 2 * k, kIdescS, (h > 0 || k > 0) ? 1u : 0u);
                    }
                }
                tcgen05_commit(&s_full[j & 1]);
            };
            bool ok = mbar_wait(&q_full, 0, &abort_flag) && mbar_wait(&kv_full[0], 0, &abort_flag);
            if (ok) {
                tcgen05_fence_after();
                issue_s(0);
            }
            for (int j = 0; ok && j < n_tiles; ++j) {
                if (j + 1 < n_tiles) {
                    const int next = j + 1;
                    ok = mbar_wait(&kv_full[next % kStagesKV], (next / kStagesKV) & 1, &abort_flag) &&
                        mbar_wait(&s_free[next & 1], ((next >> 1) & 1) ^ 1u, &abort_flag);
                    if (!ok) {
                        break;
                    }
                    tcgen05_fence_after();
                    issue_s(next);
                }
                const int b = j & 1;
                ok = mbar_wait(&p_full[b], (j >> 1) & 1, &abort_flag) &&
                    mbar_wait(&pv_free[b], ((j >> 1) & 1) ^ 1u, &abort_flag);
                if (!ok) {
                    break;
                }
                tcgen05_fence_after();
                const unsigned char* v_s = kv_s + (j % kStagesKV) * kBytesStage + kBytesK;
                const uint64_t da = smem_descriptor(p_s + b * kBytesP);
                const uint64_t db = smem_descriptor_mn(v_s, kKeys * 128);
#pragma unroll
                for (int k = 0; k < kKeys / 16; ++k) {
                    // 16 keys further: 32 bytes along P's rows, 16 rows of 128 bytes in V
                    tcgen05_mma(tmem_pv + b * kColsPV, da + 2 * k, db + k * ((16 * 128) >> 4), kIdescPV,
                                k > 0 ? 1u : 0u);
                }
                tcgen05_commit(&pv_full[b]);
                tcgen05_commit(&p_free[b]);
                tcgen05_commit(&kv_empty[j % kStagesKV]);
            }
        }
    } else {
        // ------------------------------------------------ softmax and output (warps 2..9)
        constexpr int kHalfKeys = kKeys / 2, kHalfDims = HD / 2;
        const int wg = (warp - 2) >> 2;        // which half of the row's keys and dims
        const int lane_group = warp & 3;       // the TMEM lanes this warp may read
        const int r = lane_group * 32 + lane;  // this thread's query row
        const uint32_t lane_bits = static_cast<uint32_t>(lane_group * 32) << 16;
        const int pos = pos0 + r;
        const int first = p.window > 0 ? pos - p.window + 1 : 0;
        float o[kHalfDims];
#pragma unroll
        for (int d = 0; d < kHalfDims; ++d) {
            o[d] = 0.0f;
        }
        float m = -INFINITY, l = 0.0f, corr_prev = 1.0f;
        bool ok = true;

        auto fold_pv = [&](int j, float corr) {  // o = o * corr + this thread's half of PV_j
            const int b = j & 1;
            if (!mbar_wait(&pv_full[b], (j >> 1) & 1, &abort_flag)) {
                return false;
            }
            tcgen05_fence_after();
            {
                // all of this thread's PV columns in flight, then one wait
                uint32_t v[kHalfDims / 32][32];
#pragma unroll
                for (int g = 0; g < kHalfDims / 32; ++g) {
                    tcgen05_ld32_nowait(tmem_pv + lane_bits + b * kColsPV + wg * kHalfDims + 32 * g, v[g]);
                }
                tcgen05_wait_ld();
#pragma unroll
                for (int g = 0; g < kHalfDims / 32; ++g) {
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        o[32 * g + c] = fmaf(o[32 * g + c], corr, __uint_as_float(v[g][c]));
                    }
                }
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&pv_free[b]);
            }
            return true;
        };

        for (int j = 0; j < n_tiles; ++j) {
            const int b = j & 1;
            if (!mbar_wait(&s_full[b], (j >> 1) & 1, &abort_flag)) {
                ok = false;
                break;
            }
            tcgen05_fence_after();
            float s[kHalfKeys];
            {
                static_assert(kHalfKeys == 32, "one 32-column load per thread");
                uint32_t v[32];
                tcgen05_ld32_nowait(tmem_s + lane_bits + b * kColsS + wg * kHalfKeys, v);
                tcgen05_wait_ld();
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    s[c] = __uint_as_float(v[c]);
                }
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&s_free[b]);
            }
            const int key0 = (j0 + j) * kKeys;
            const bool edge = key0 + kKeys - 1 > pos0 || (p.window > 0 && key0 < pos0 + kRows - p.window);
            float tile_max = -INFINITY;
            if (edge) {
#pragma unroll
                for (int c = 0; c < kHalfKeys; ++c) {
                    const int key = key0 + wg * kHalfKeys + c;
                    s[c] = (key <= pos && key >= first) ? s[c] * p.scale_log2 : -INFINITY;
                    tile_max = fmaxf(tile_max, s[c]);
                }
            } else {
#pragma unroll
                for (int c = 0; c < kHalfKeys; ++c) {
                    s[c] *= p.scale_log2;
                    tile_max = fmaxf(tile_max, s[c]);
                }
            }
            // The row's maximum over both halves: exchange through shared memory.
            half_max[b][wg * kRows + r] = tile_max;
            asm volatile("bar.sync 2, 256;" ::: "memory");
            tile_max = fmaxf(tile_max, half_max[b][(wg ^ 1) * kRows + r]);
            const float m_new = fmaxf(m, tile_max);
            const float base = m_new == -INFINITY ? 0.0f : m_new;
            const float corr = ex2(m - base);
            m = m_new;
            float sum = 0.0f;
            uint32_t packed[kHalfKeys / 2];
#pragma unroll
            for (int c = 0; c < kHalfKeys; c += 2) {
                const float p0 = ex2(s[c] - base), p1 = ex2(s[c + 1] - base);
                sum += p0 + p1;
                const __nv_bfloat162 pair = __floats2bfloat162_rn(p0, p1);
                packed[c / 2] = *reinterpret_cast<const uint32_t*>(&pair);
            }
            l = l * corr + sum;  // this thread's half of the row sum; the halves meet at the end
            // P_j into its buffer (free once PV_{j-2} has read it), row r, swizzled.
            if (!mbar_wait(&p_free[b], ((j >> 1) & 1) ^ 1u, &abort_flag)) {
                ok = false;
                break;
            }
            unsigned char* p_row = p_s + b * kBytesP + r * 128;
#pragma unroll
            for (int c = 0; c < kHalfKeys / 8; ++c) {
                const int chunk = wg * (kHalfKeys / 8) + c;
                *reinterpret_cast<uint4*>(p_row + ((chunk ^ (r & 7)) * 16)) =
                    make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&p_full[b]);
            }
            if (j > 0 && !fold_pv(j - 1, corr_prev)) {
                ok = false;
                break;
            }
            corr_prev = corr;
        }
        if (ok && n_tiles > 0) {
            ok = fold_pv(n_tiles - 1, corr_prev);
        }
        // The row sum is the sum of the two halves' sums (both followed the same maxima).
        half_max[0][wg * kRows + r] = l;
        asm volatile("bar.sync 2, 256;" ::: "memory");
        l += half_max[0][(wg ^ 1) * kRows + r];
        if (ok && r < n_rows) {
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            __nv_bfloat16* dst = p.out + (row0 + r) * p.out_row_stride + static_cast<int64_t>(head) * HD +
                wg * kHalfDims;
#pragma unroll
            for (int d = 0; d < kHalfDims; d += 8) {
                uint32_t w[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const __nv_bfloat162 pair = __floats2bfloat162_rn(o[d + 2 * i] * inv, o[d + 2 * i + 1] * inv);
                    w[i] = *reinterpret_cast<const uint32_t*>(&pair);
                }
                *reinterpret_cast<uint4*>(dst + d) = make_uint4(w[0], w[1], w[2], w[3]);
            }
        }
    }

    // ---------------------------------------------------- teardown
    __syncwarp();
    tcgen05_fence_before();
    __syncthreads();
    if (abort_flag) {
        if (threadIdx.x == 0) {
            if (p.status != nullptr) {
                atomicOr(p.status, 8);
            }
            for (uint32_t spin = 0; spin < (1u << 16); ++spin) {
                __nanosleep(64);  // lets loads that were issued land before the CTA leaves
            }
        }
        __syncthreads();
    }
    if (warp == 1) {
        tcgen05_fence_after();
        tcgen05_dealloc(tmem_base, kColumns);
    }
}

template <int HD>
int launch_tc_prefill(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const TcPrefillParams& p,
                      int n_tiles, int n_heads, cudaStream_t stream) {
    constexpr int smem = kRows * HD * 2 + kStagesKV * 2 * kKeys * HD * 2 + 2 * kRows * kKeys * 2 + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(attention_prefill_tcgen05_kernel<HD>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (err != cudaSuccess) {
            return pl_fail(3, "attention_prefill_tcgen05: cannot set shared memory size: %s",
                           cudaGetErrorString(err));
        }
        configured = true;
    }
    attention_prefill_tcgen05_kernel<HD><<<dim3(n_tiles, n_heads), kThreadsTc, smem, stream>>>(mq, mk, mv, p);
    PL_CHECK_LAUNCH("attention_prefill_tcgen05");
    return 0;
}

}  // namespace

// 1 when pl_attention_prefill_tcgen05 takes this shape and cache layout.
PL_API int pl_attention_prefill_tcgen05_supports(int head_dim, int page_size, int n_kv_heads, int64_t page_stride,
                                                 int64_t head_stride, int64_t q_row_stride, int dtype) {
    return dtype == PL_BF16 && (head_dim == 64 || head_dim == 128) && page_size % kPiece == 0 &&
        head_stride == static_cast<int64_t>(page_size) * head_dim &&
        page_stride == 2 * static_cast<int64_t>(n_kv_heads) * head_stride && q_row_stride % 8 == 0;
}

// As pl_attention_prefill (tiles of up to 128 rows), on tcgen05. The pools must be
// the two halves of one [pages][2][kv heads][page][head_dim] tensor: v_pool is
// k_pool + kv_heads * page * head_dim elements.
PL_API int pl_attention_prefill_tcgen05(const void* q, int64_t q_row_stride, int n_tokens, const void* k_pool,
                                        const void* v_pool, int64_t page_stride, int64_t head_stride, int page_size,
                                        int n_pages, const int32_t* table, int table_width, const int32_t* tiles,
                                        int n_tiles, void* out, int64_t out_row_stride, int n_heads, int n_kv_heads,
                                        int head_dim, int window, float scale, int32_t* status,
                                        cudaStream_t stream) {
    PL_REQUIRE(n_tiles >= 0 && n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0 && n_tokens > 0,
               "attention_prefill_tcgen05: bad sizes tiles=%d heads=%d kv_heads=%d tokens=%d", n_tiles, n_heads,
               n_kv_heads, n_tokens);
    PL_REQUIRE(pl_attention_prefill_tcgen05_supports(head_dim, page_size, n_kv_heads, page_stride, head_stride,
                                                     q_row_stride, PL_BF16),
               "attention_prefill_tcgen05: unsupported shape or cache layout (head_dim=%d page=%d)", head_dim,
               page_size);
    PL_REQUIRE(static_cast<const __nv_bfloat16*>(v_pool) ==
                   static_cast<const __nv_bfloat16*>(k_pool) + n_kv_heads * head_stride,
               "attention_prefill_tcgen05: v_pool must follow k_pool inside each page");
    PL_REQUIRE((reinterpret_cast<uintptr_t>(q) & 15) == 0 && (reinterpret_cast<uintptr_t>(k_pool) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(out) & 15) == 0 && out_row_stride % 8 == 0 &&
                   (reinterpret_cast<uintptr_t>(tiles) & 15) == 0,
               "attention_prefill_tcgen05: q, the pools, out and the tile list must be 16-byte aligned");
    PL_REQUIRE(n_heads <= 65535, "attention_prefill_tcgen05: too many heads (%d)", n_heads);
    if (n_tiles == 0) {
        return 0;
    }
    CUtensorMap mq, mk, mv;
    if (const int code = make_map(&mq, q, n_tokens, n_heads * head_dim, q_row_stride, kRows, 64)) {
        return code;
    }
    // Rows of the pool: (page, K or V, kv head, slot); the V map starts one K block in
    // and so has that many rows fewer.
    const int64_t rows = static_cast<int64_t>(n_pages) * 2 * n_kv_heads * page_size;
    if (const int code = make_map(&mk, k_pool, rows, head_dim, head_dim, kPiece, 64)) {
        return code;
    }
    if (const int code = make_map(&mv, v_pool, rows - static_cast<int64_t>(n_kv_heads) * page_size, head_dim,
                                  head_dim, kPiece, 64)) {
        return code;
    }
    TcPrefillParams p;
    p.table = table;
    p.table_width = table_width;
    p.tiles = reinterpret_cast<const int4*>(tiles);
    p.out = static_cast<__nv_bfloat16*>(out);
    p.out_row_stride = out_row_stride;
    p.group = n_heads / n_kv_heads;
    p.n_kv_heads = n_kv_heads;
    p.page_size = page_size;
    p.n_pages = n_pages;
    p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.status = status;
    if (head_dim == 64) {
        return launch_tc_prefill<64>(mq, mk, mv, p, n_tiles, n_heads, stream);
    }
    return launch_tc_prefill<128>(mq, mk, mv, p, n_tiles, n_heads, stream);
}
