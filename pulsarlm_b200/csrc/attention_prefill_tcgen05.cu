// Paged causal attention for prompt portions on the 5th-generation tensor cores.
//
// CTA (query tile of 128 tokens, query head). Both products run as tcgen05 MMAs with
// M = 128 query rows and accumulators in tensor memory:
//   S  = Q K^T   M 128 x N 64 keys  x K head_dim  (Q and K tiles K-major in smem)
//   PV = P V     M 128 x N head_dim x K 64 keys   (P in tensor memory, V as stored: N-major)
// Roles: warp 0 loads tiles with TMA (Q once; per 64-key tile the K and V rows of
// four 16-key page pieces, found through the block table), warp 1 issues the MMAs,
// warps 2-9 are two softmax warpgroups. When the GQA group is even a CTA takes two
// query heads of one kv head: they share every K and V tile, and each warpgroup
// does one head's softmax with one thread per query row. Otherwise a CTA takes one
// head and the warpgroups share each row (thread pairs read the two halves of the
// row's S and agree on the row maximum through shared memory). The softmax is
// online, in fp32, base 2 with the scale folded in; P goes as bf16 into tensor
// memory, over the columns its S came from (each thread stores its own row's values
// where the second product reads its A operand: lane = row, two keys per column),
// so the second product reads only V from shared memory. Its output accumulates in
// tensor memory over all tiles. The exponents' base follows the row maximum lazily: it moves only when a
// tile's maximum exceeds it by more than 2^8 (P then stays below 256, which fp32
// sums and bf16 P hold without loss), and only then is the row of O read from
// tensor memory, scaled and written back, after the previous PV has completed; most
// tiles never touch O. With two heads per CTA the heads take turns on the tensor
// pipe: Q sits in tensor memory too (each thread stores its own row there at the
// start, so the first product reads only K from shared memory), and while one
// warpgroup does the softmax of its head's tile the pipe runs the other head's PV and
// next S. With one head per CTA, S is double-buffered instead, so that S of tile j+1
// is computed while the softmax of tile j runs.
//
// Few query tiles over many keys (a short portion of a long prompt) would leave most
// SMs idle: the launch may then split every tile's keys `n_splits` ways (grid z). Each
// CTA writes its unnormalised fp32 output and each row's (exponent base, sum) to
// scratch, and a second kernel merges the splits in split order.
//
// Every mbarrier wait is bounded; on a timeout the CTA raises bit 8 of the status
// word, stops, lets loads in flight land, frees its tensor memory and returns.
//
// Takes head_dim 64 or 128 and pages that are multiples of 16 tokens in the cache
// manager's layout [page][K,V][kv head][slot][dim]; other shapes go to the mma.sync
// kernel in attention_prefill.cu. The reference's counterpart: attn_prefill_tc_kernel,
// pulsarlm-core/inc/pulsarlm/kernels/paged_prefill.cuh:58-328.
#include <type_traits>

#include "tcgen05_helpers.cuh"

namespace {

constexpr int kRows = 128;     // query rows per CTA
constexpr int kKeys = 64;      // keys per tile
constexpr int kPiece = 16;     // keys per TMA box (a page, or a part of one)
__host__ __device__ constexpr int stages_kv(int heads) { return heads == 2 ? 6 : 4; }
constexpr int kThreadsTc = 320;  // TMA warp, MMA warp, two softmax warpgroups

struct TcPrefillParams {
    const __nv_bfloat16* q;
    int64_t q_row_stride;
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
    int n_heads;
    int n_splits;     // > 1: partial results go to scratch [token][head][split]
    float* part_o;    // ... [head_dim]: unnormalised output
    float2* part_ml;  // ... (base of the exponents (log2), sum)
    // Attention mass (optional, two heads or halves per CTA only): every softmax warp adds
    // up, over its 32 query rows, weight[row] * (the row's largest scaled score among the
    // keys of a page it attends), and stores the sum at mass_part[((tile * heads + head) * 8
    // + warp slot) * mass_pages + page of the request]; a second kernel folds the sums into
    // the step's per-page accumulators in a fixed order.
    const float* query_weights;  // [tokens]
    float* mass_part;            // zero before the launch
    int mass_pages;
    float scale;
};

// What pl_attention_prefill_tcgen05 needs to measure attention mass: the rows' weights,
// zeroed scratch of n_tiles * n_heads * 8 * pages floats (pages >= the block table's
// width), the number of rows of the block table, and the step's sums step_mass [n_pages, n_heads] and step_weight [n_pages],
// which the call adds to.
struct PlPrefillMass {
    const float* query_weights;
    float* scratch;
    int pages;
    int table_rows;  // rows of the block table (requests of the step)
    float* step_mass;
    float* step_weight;
};

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// 2^x for two values at once without the special-function unit: x = n + f with n the
// nearest integer, 2^f on [-0.5, 0.5] as a cubic (relative error 7.5e-5, a thirtieth of
// the bfloat16 step the probabilities are rounded to), n added into the exponent bits.
// Values below -126 (masked keys come as -inf) give 2^-126.
__device__ __forceinline__ float2 exp2_cubic2(float2 x) {
    constexpr float kMagic = 12582912.0f;  // 1.5 * 2^23: adding it leaves n in the low mantissa bits
    x.x = fmaxf(x.x, -126.0f);
    x.y = fmaxf(x.y, -126.0f);
    const float2 shifted = __fadd2_rn(x, make_float2(kMagic, kMagic));
    const float2 whole = __fadd2_rn(shifted, make_float2(-kMagic, -kMagic));
    const float2 f = __ffma2_rn(whole, make_float2(-1.0f, -1.0f), x);
    float2 y = __ffma2_rn(make_float2(0.0551716648f, 0.0551716648f), f, make_float2(0.2426111251f, 0.2426111251f));
    y = __ffma2_rn(y, f, make_float2(0.6932609677f, 0.6932609677f));
    y = __ffma2_rn(y, f, make_float2(0.9999280572f, 0.9999280572f));
    y.x = __int_as_float(__float_as_int(y.x) + (__float_as_int(shifted.x) << 23));
    y.y = __int_as_float(__float_as_int(y.y) + (__float_as_int(shifted.y) << 23));
    return y;
}

// Descriptor of an N-major (MN-major) operand with 128-byte swizzle: 64-element
// groups along N are `n_group_bytes` apart, groups of 8 rows along K 1024 bytes.
__device__ __forceinline__ uint64_t smem_descriptor_mn(const void* tile, uint32_t n_group_bytes) {
    const uint64_t address = (smem_u32(tile) >> 4) & 0x3FFFu;
    return address | (static_cast<uint64_t>((n_group_bytes >> 4) & 0x3FFFu) << 16) |
        (static_cast<uint64_t>(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

// HEADS query heads per CTA: 2 when the GQA group is even (two heads of one kv head
// share every K and V tile, one softmax warpgroup each, one thread per query row), 1
// otherwise (the two warpgroups share each row: one takes the tile's first 32 keys
// and the first half of the output's dims, the other the rest).
//
// WIDE (with HEADS == 2, for odd groups): the two "heads" of the CTA are the two
// 128-row halves of one tile of up to 256 rows of ONE head: they share K and V just
// the same, and everything that says head `hs` below means rows 128 hs ... of it.
template <int HD, int HEADS, bool WIDE>
__global__ void __launch_bounds__(kThreadsTc, 1)
attention_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                                 const __grid_constant__ CUtensorMap map_v, const TcPrefillParams p) {
    constexpr int kHalves = HD / 64;                       // 64-dim (128-byte) column groups of a row
    constexpr int kBytesQ = kRows * HD * 2;                // per head: kHalves sub-tiles of [128 x 64]
    constexpr int kBytesK = kKeys * HD * 2;                // kHalves sub-tiles of [64 x 64]
    constexpr int kBytesStage = 2 * kBytesK;               // K then V
    constexpr int kWarpsPerHead = 8 / HEADS;               // softmax warps that arrive on a head's barriers
    constexpr bool kTurns = HEADS == 2;                    // the heads take turns: Q in tensor memory, one S buffer
    constexpr int kBuffersS = kTurns ? 1 : 2;
    constexpr int kStagesKV = stages_kv(HEADS);
    constexpr uint32_t kColsS = kKeys, kColsO = HD, kColsQ = HD / 2;  // Q: two bf16 of a row per column
    constexpr uint32_t kColumns =
        HEADS * (kBuffersS * kColsS + kColsO) + (kTurns ? HEADS * kColsQ : 0) <= 256 ? 256 : 512;
    constexpr float kLazy = 8.0f;  // the base of the exponents may lag the row maximum by this much (log2)
    // instruction descriptors: fp32 accumulate, bf16 operands, M = 128
    constexpr uint32_t kIdescS = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(kKeys >> 3) << 17) |
        (static_cast<uint32_t>(kRows >> 4) << 24);
    constexpr uint32_t kIdescPV = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) |  // B is N-major
        (static_cast<uint32_t>(HD >> 3) << 17) | (static_cast<uint32_t>(kRows >> 4) << 24);

    extern __shared__ unsigned char raw_smem[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) &
                                                           ~static_cast<uintptr_t>(1023));
    unsigned char* q_s = smem;                               // [head][half][128 rows x 128 bytes] (not with turns)
    unsigned char* kv_s = q_s + (kTurns ? 0 : HEADS * kBytesQ);

    __shared__ __align__(8) uint64_t q_full, kv_full[kStagesKV], kv_empty[kStagesKV];
    __shared__ __align__(8) uint64_t s_full[HEADS][2], s_free[HEADS][2], p_full[HEADS][2], pv_done[HEADS],
        q_ready[HEADS];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;
    __shared__ float half_max[HEADS == 1 ? 2 : 1][HEADS == 1 ? 2 * kRows : 1];  // [tile parity][warpgroup * 128 + row]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Heads vary fastest in the grid and the tile list is sorted longest first, so the
    // CTAs of a wave are of similar length and the short ones fill the end.
    const int4 tile = p.tiles[blockIdx.y];
    static_assert(!WIDE || HEADS == 2, "a wide tile is two halves that take turns");
    constexpr int kSpan = WIDE ? 2 * kRows : kRows;  // rows of a tile
    const int row0 = tile.x, n_rows = min(tile.y, kSpan), pos0 = tile.z;
    if (tile.y > kSpan && threadIdx.x == 0 && p.status != nullptr) {
        atomicOr(p.status, 4);  // a tile with more rows than this arrangement takes
    }
    const int head0 = WIDE ? blockIdx.x : blockIdx.x * HEADS, kv_head = head0 / p.group;
    const int last_key = pos0 + n_rows - 1;
    const int first_key = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
    // This CTA's share of the tile's 64-key tiles (all of them without splits).
    const int all_tiles = last_key / kKeys - first_key / kKeys + 1;
    const int per_split = (all_tiles + p.n_splits - 1) / p.n_splits;
    const int j_begin = min(all_tiles, static_cast<int>(blockIdx.z) * per_split);
    const int j0 = first_key / kKeys + j_begin, n_tiles = min(all_tiles, j_begin + per_split) - j_begin;
    if (n_tiles == 0) {
        // Nothing for this split: its rows say so (the merge skips a split whose base is -inf).
        for (int i = threadIdx.x; i < HEADS * kRows; i += kThreadsTc) {
            const int hs = i / kRows, r = WIDE ? i : i % kRows, head = head0 + (WIDE ? 0 : hs);
            if (r < n_rows) {
                p.part_ml[(static_cast<int64_t>(row0 + r) * p.n_heads + head) * p.n_splits + blockIdx.z] =
                    make_float2(-INFINITY, 0.0f);
            }
        }
        return;
    }

    if (threadIdx.x == 0) {
        mbar_init(&q_full, 1);
        for (int s = 0; s < kStagesKV; ++s) {
            mbar_init(&kv_full[s], 1);
            mbar_init(&kv_empty[s], 1);
        }
        for (int h = 0; h < HEADS; ++h) {
            for (int b = 0; b < 2; ++b) {
                mbar_init(&s_full[h][b], 1);
                mbar_init(&s_free[h][b], kWarpsPerHead);
                mbar_init(&p_full[h][b], kWarpsPerHead);
            }
            mbar_init(&pv_done[h], 1);
            mbar_init(&q_ready[h], kWarpsPerHead);
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
    const uint32_t tmem_s = tmem_base;                                // [head][buffer][64 columns]: S, then P in its first 32
    const uint32_t tmem_o = tmem_base + HEADS * kBuffersS * kColsS;   // [head][HD columns]
    const uint32_t tmem_q = tmem_o + HEADS * kColsO;                  // [head][HD / 2 columns] (with turns)

    if (warp == 0) {
        // ------------------------------------------------ producer
        // Lane 0 waits and issues; all lanes look up block-table entries, 32 pieces
        // (eight tiles) at a time in one load each, so that the table's latency is
        // paid once per eight tiles and not once per piece.
        if (lane == 0 && !kTurns) {
            mbar_expect_tx(&q_full, HEADS * kBytesQ);
            for (int hs = 0; hs < HEADS; ++hs) {
                for (int h = 0; h < kHalves; ++h) {
                    tma_load_2d(q_s + hs * kBytesQ + h * (kRows * 128), &map_q, (head0 + hs) * HD + h * 64, row0,
                                &q_full);
                }
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
        // All lanes run the loop and wait; one elected lane issues. (Descriptors and
        // counters then live in uniform registers, which the MMA instructions take.)
        if constexpr (kTurns) {
            // S_j of head hs: A = Q from tensor memory, B = K_j from shared memory, into the
            // head's one S buffer (free: the PV that read P from it was issued before).
            auto issue_s = [&](int j, int hs) {
                const unsigned char* k_s = kv_s + (j % kStagesKV) * kBytesStage;
                uint64_t db[kHalves];
#pragma unroll
                for (int h = 0; h < kHalves; ++h) {
                    db[h] = smem_descriptor(k_s + h * (kKeys * 128));
                }
                if (elect_one()) {
#pragma unroll
                    for (int k = 0; k < HD / 16; ++k) {
                        tcgen05_mma_a_tmem(tmem_s + hs * kColsS, tmem_q + hs * kColsQ + 8 * k, db[k / 4] + 2 * (k % 4),
                                           kIdescS, k > 0 ? 1u : 0u);
                    }
                    tcgen05_commit(&s_full[hs][0]);
                }
                __syncwarp();
            };
            bool ok = mbar_wait(&kv_full[0], 0, &abort_flag);
            for (int hs = 0; ok && hs < HEADS; ++hs) {
                ok = mbar_wait(&q_ready[hs], 0, &abort_flag);
                if (ok) {
                    tcgen05_fence_after();
                    issue_s(0, hs);
                }
            }
            for (int j = 0; ok && j < n_tiles; ++j) {
                const unsigned char* v_s = kv_s + (j % kStagesKV) * kBytesStage + kBytesK;
                const uint64_t db = smem_descriptor_mn(v_s, kKeys * 128);
                for (int hs = 0; ok && hs < HEADS; ++hs) {
                    // P_j of this head lies over its S_j, and its O is rescaled if its base moved
                    ok = mbar_wait(&p_full[hs][0], j & 1, &abort_flag);
                    if (!ok) {
                        break;
                    }
                    tcgen05_fence_after();
                    if (elect_one()) {
#pragma unroll
                        for (int k = 0; k < kKeys / 16; ++k) {
                            // 16 keys further: 8 columns of P, 16 rows of 128 bytes in V
                            tcgen05_mma_a_tmem(tmem_o + hs * kColsO, tmem_s + hs * kColsS + 8 * k,
                                               db + k * ((16 * 128) >> 4), kIdescPV, (j > 0 || k > 0) ? 1u : 0u);
                        }
                        tcgen05_commit(&pv_done[hs]);
                        if (hs == HEADS - 1) {
                            tcgen05_commit(&kv_empty[j % kStagesKV]);
                        }
                    }
                    __syncwarp();
                    if (j + 1 < n_tiles) {
                        // this head's next S at once: it runs while the other head's softmax does
                        if (hs == 0) {
                            ok = mbar_wait(&kv_full[(j + 1) % kStagesKV], ((j + 1) / kStagesKV) & 1, &abort_flag);
                            if (!ok) {
                                break;
                            }
                            tcgen05_fence_after();
                        }
                        issue_s(j + 1, hs);
                    }
                }
            }
        } else {
            auto issue_s = [&](int j, int hs) {  // S_j = Q K_j^T of head hs into its buffer j & 1
                const unsigned char* k_s = kv_s + (j % kStagesKV) * kBytesStage;
                const uint32_t d = tmem_s + (hs * 2 + (j & 1)) * kColsS;
                if (elect_one()) {
    #pragma unroll
                    for (int h = 0; h < kHalves; ++h) {
                        const uint64_t da = smem_descriptor(q_s + hs * kBytesQ + h * (kRows * 128));
                        const uint64_t db = smem_descriptor(k_s + h * (kKeys * 128));
    #pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            tcgen05_mma(d, da + 2 * k, db + 2 * k, kIdescS, (h > 0 || k > 0) ? 1u : 0u);
                        }
                    }
                    tcgen05_commit(&s_full[hs][j & 1]);
                }
                __syncwarp();
            };
            bool ok = mbar_wait(&q_full, 0, &abort_flag) && mbar_wait(&kv_full[0], 0, &abort_flag);
            if (ok) {
                tcgen05_fence_after();
                for (int hs = 0; hs < HEADS; ++hs) {
                    issue_s(0, hs);
                }
            }
            for (int j = 0; ok && j < n_tiles; ++j) {
                if (j + 1 < n_tiles) {
                    const int next = j + 1;
                    ok = mbar_wait(&kv_full[next % kStagesKV], (next / kStagesKV) & 1, &abort_flag);
                    for (int hs = 0; ok && hs < HEADS; ++hs) {
                        ok = mbar_wait(&s_free[hs][next & 1], ((next >> 1) & 1) ^ 1u, &abort_flag);
                        if (ok) {
                            tcgen05_fence_after();
                            issue_s(next, hs);
                        }
                    }
                    if (!ok) {
                        break;
                    }
                }
                const unsigned char* v_s = kv_s + (j % kStagesKV) * kBytesStage + kBytesK;
                const uint64_t db = smem_descriptor_mn(v_s, kKeys * 128);
                for (int hs = 0; ok && hs < HEADS; ++hs) {
                    // P_j of this head is in tensor memory, and its O rescaled if its base moved.
                    // (The buffer is written next by S_{j+2}, issued after this product: the
                    // tensor pipe runs in order, so P is read before it is overwritten.)
                    ok = mbar_wait(&p_full[hs][j & 1], (j >> 1) & 1, &abort_flag);
                    if (!ok) {
                        break;
                    }
                    tcgen05_fence_after();
                    const uint32_t pa = tmem_s + (hs * 2 + (j & 1)) * kColsS;
                    if (elect_one()) {
    #pragma unroll
                        for (int k = 0; k < kKeys / 16; ++k) {
                            // 16 keys further: 8 columns of P, 16 rows of 128 bytes in V
                            tcgen05_mma_a_tmem(tmem_o + hs * kColsO, pa + 8 * k, db + k * ((16 * 128) >> 4), kIdescPV,
                                               (j > 0 || k > 0) ? 1u : 0u);
                        }
                        tcgen05_commit(&pv_done[hs]);
                        if (hs == HEADS - 1) {
                            tcgen05_commit(&kv_empty[j % kStagesKV]);
                        }
                    }
                    __syncwarp();
                }
            }
        }
    } else {
        // ------------------------------------------------ softmax and output (warps 2..9)
        const int wg = (warp - 2) >> 2;           // warpgroup 0 or 1
        const int hs = HEADS == 2 ? wg : 0;       // the head it works on
        const int part = HEADS == 2 ? 0 : wg;     // HEADS == 1: which half of the row's keys and dims
        constexpr int kMyKeys = HEADS == 2 ? kKeys : kKeys / 2;
        constexpr int kMyDims = HEADS == 2 ? HD : HD / 2;
        const int lane_group = warp & 3;          // the TMEM lanes this warp may read
        const int r = lane_group * 32 + lane;     // this thread's query row
        const uint32_t lane_bits = static_cast<uint32_t>(lane_group * 32) << 16;
        const uint32_t my_s = tmem_s + lane_bits + hs * kBuffersS * kColsS + part * kMyKeys;
        const uint32_t my_o = tmem_o + lane_bits + hs * kColsO + part * kMyDims;
        const int rr = r + (WIDE ? hs * kRows : 0);        // this thread's row within the tile,
        const int head = head0 + (WIDE ? 0 : hs);          // and its query head
        const int pos = pos0 + rr;
        const int first = p.window > 0 ? pos - p.window + 1 : 0;
        float m = -INFINITY, l = 0.0f;  // m: the base of the exponents in use (lags the true maximum)
        bool ok = true;
        const float mass_weight = p.mass_part != nullptr && rr < n_rows ? p.query_weights[row0 + rr] : 0.0f;
        if constexpr (kTurns) {
            // This thread's row of Q into tensor memory, where the first product reads its A
            // operand: lane = row, column c = dims 2c and 2c + 1 (rows past the tile: zeros).
            const uint4* src = reinterpret_cast<const uint4*>(p.q + (row0 + rr) * p.q_row_stride +
                                                              static_cast<int64_t>(head) * HD);
#pragma unroll
            for (int g = 0; g < HD / 64; ++g) {
                uint32_t v[32];
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const uint4 four = rr < n_rows ? src[8 * g + c] : make_uint4(0u, 0u, 0u, 0u);
                    v[4 * c] = four.x;
                    v[4 * c + 1] = four.y;
                    v[4 * c + 2] = four.z;
                    v[4 * c + 3] = four.w;
                }
                tcgen05_st32_nowait(tmem_q + lane_bits + hs * kColsQ + 32 * g, v);
            }
            tcgen05_wait_st();
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&q_ready[hs]);
            }
        }

        for (int j = 0; j < n_tiles; ++j) {
            const int b = kTurns ? 0 : (j & 1);              // the S buffer of this tile,
            const uint32_t use = kTurns ? (j & 1) : ((j >> 1) & 1);  // and the parity of its use
            if (!mbar_wait(&s_full[hs][b], use, &abort_flag)) {
                ok = false;
                break;
            }
            tcgen05_fence_after();
            float s[kMyKeys];
            {
                uint32_t v[kMyKeys / 32][32];
#pragma unroll
                for (int g = 0; g < kMyKeys / 32; ++g) {
                    tcgen05_ld32_nowait(my_s + b * kColsS + 32 * g, v[g]);
                }
                tcgen05_wait_ld();
#pragma unroll
                for (int g = 0; g < kMyKeys / 32; ++g) {
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        s[32 * g + c] = __uint_as_float(v[g][c]);
                    }
                }
            }
            tcgen05_fence_before();
            __syncwarp();
            if (!kTurns && lane == 0) {
                mbar_arrive(&s_free[hs][b]);
            }
            const int key0 = (j0 + j) * kKeys + part * kMyKeys;
            const bool edge = (j0 + j) * kKeys + kKeys - 1 > pos0 ||
                (p.window > 0 && (j0 + j) * kKeys < pos0 + kSpan - p.window);
            // The tile's maximum, on the raw products (the scale is positive), four running
            // maxima side by side so that the chain of dependent instructions stays short.
            if (edge) {
#pragma unroll
                for (int c = 0; c < kMyKeys; ++c) {
                    const int key = key0 + c;
                    s[c] = (key <= pos && key >= first) ? s[c] : -INFINITY;
                }
            }
            if constexpr (kMyKeys == kKeys) {
                if (p.mass_part != nullptr) {
                    // Largest raw product per 16 keys, then per page (16, 32 or 64 keys: a page lies
                    // within the tile), weighed and added up over the warp's rows.
                    float m16[4];
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        float best = s[16 * q4];
#pragma unroll
                        for (int c = 1; c < 16; ++c) {
                            best = fmaxf(best, s[16 * q4 + c]);
                        }
                        m16[q4] = best;
                    }
                    const int per_page = p.page_size / 16;  // 1, 2 or 4 of those
                    float* dst = p.mass_part +
                        ((static_cast<int64_t>(blockIdx.y) * p.n_heads + head) * 8 + (WIDE ? hs * 4 : 0) + lane_group) *
                            p.mass_pages;
                    for (int q4 = 0; q4 < 4; q4 += per_page) {
                        float best = m16[q4];
                        for (int i = 1; i < per_page; ++i) {
                            best = fmaxf(best, m16[q4 + i]);
                        }
                        float part_sum = best > -INFINITY ? mass_weight * (best * p.scale) : 0.0f;
#pragma unroll
                        for (int offset = 16; offset > 0; offset >>= 1) {
                            part_sum += __shfl_xor_sync(0xffffffffu, part_sum, offset);
                        }
                        const int page_of_request = (key0 + 16 * q4) / p.page_size;
                        if (lane == 0 && page_of_request < p.mass_pages) {
                            dst[page_of_request] = part_sum;
                        }
                    }
                }
            }
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int c = 0; c < kMyKeys; c += 8) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    mx[i] = max3(mx[i], s[c + i], s[c + 4 + i]);
                }
            }
            float tile_max = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * p.scale_log2;
            if (HEADS == 1) {
                // The row's maximum over both halves: exchange through shared memory.
                half_max[b][wg * kRows + r] = tile_max;
                asm volatile("bar.sync 2, 256;" ::: "memory");
                tile_max = fmaxf(tile_max, half_max[b][(wg ^ 1) * kRows + r]);
            }
            // Move the base only when the tile's maximum has run away from it. (With two
            // threads to a row both see the same maximum and decide alike.)
            const bool move = tile_max > m + kLazy;
            float corr = 1.0f;
            if (move) {
                corr = ex2(m - tile_max);  // 0 when nothing was accumulated under the old base
                m = tile_max;
            }
            if (j > 0 && __any_sync(0xffffffffu, move)) {
                // Rows of this warp change base: scale their part of O where it lies. The
                // previous PV must have landed; the next one waits for this tile's P.
                if (!mbar_wait(&pv_done[hs], (j - 1) & 1, &abort_flag)) {
                    ok = false;
                    break;
                }
                tcgen05_fence_after();
#pragma unroll
                for (int g = 0; g < kMyDims / 32; ++g) {
                    uint32_t v[32];
                    tcgen05_ld32_nowait(my_o + 32 * g, v);
                    tcgen05_wait_ld();
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        v[c] = __float_as_uint(__uint_as_float(v[c]) * corr);
                    }
                    tcgen05_st32_nowait(my_o + 32 * g, v);
                }
                tcgen05_wait_st();
                tcgen05_fence_before();
            }
            const float minus_base = m == -INFINITY ? 0.0f : -m;
            // Exponentials two at a time (packed fp32 arithmetic). Of every four pairs, kCubic
            // take the cubic on the FMA pipe and the rest the special-function unit (one
            // exponential per eight cycles and warp). Measured: at head size 64, where the
            // products are short, one pair in four as a cubic is 5 % faster; at 128 the
            // cubic's extra instructions cost more than the unit's time (528 -> 561 us at
            // 8,192 tokens with one pair, 593 with two).
            constexpr int kCubic = HD == 64 ? 1 : 0;
            const float2 scale2 = make_float2(p.scale_log2, p.scale_log2), base2 = make_float2(minus_base, minus_base);
            float2 sums[4] = {};
            uint32_t packed[kMyKeys / 2];
#pragma unroll
            for (int c = 0; c < kMyKeys; c += 8) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 x = __ffma2_rn(make_float2(s[c + 2 * i], s[c + 2 * i + 1]), scale2, base2);
                    const float2 e = i < 4 - kCubic ? make_float2(ex2(x.x), ex2(x.y)) : exp2_cubic2(x);
                    sums[i] = __fadd2_rn(sums[i], e);
                    const __nv_bfloat162 pair = __floats2bfloat162_rn(e.x, e.y);
                    packed[c / 2 + i] = *reinterpret_cast<const uint32_t*>(&pair);
                }
            }
            const float2 both = __fadd2_rn(__fadd2_rn(sums[0], sums[1]), __fadd2_rn(sums[2], sums[3]));
            const float sum = both.x + both.y;
            l = l * corr + sum;  // (HEADS == 1: this thread's half of the row sum; the halves meet at the end)
            // P_j over the first columns of S_j (all of this row's S has been read: with two
            // threads to a row the exchange above came after both loads).
            if constexpr (kMyKeys == 64) {
                tcgen05_st32_nowait(tmem_s + lane_bits + (hs * kBuffersS + b) * kColsS, packed);
            } else {
                tcgen05_st16_nowait(tmem_s + lane_bits + (hs * kBuffersS + b) * kColsS + part * (kMyKeys / 2), packed);
            }
            tcgen05_wait_st();
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&p_full[hs][b]);
            }
        }
        if (HEADS == 1) {
            // The row sum is the sum of the two halves' sums (both followed the same bases).
            half_max[0][wg * kRows + r] = l;
            asm volatile("bar.sync 2, 256;" ::: "memory");
            l += half_max[0][(wg ^ 1) * kRows + r];
        }
        if (ok && n_tiles > 0) {
            ok = mbar_wait(&pv_done[hs], (n_tiles - 1) & 1, &abort_flag);
            tcgen05_fence_after();
        }
        if (ok && p.n_splits > 1) {
            // One split of several: the unnormalised row, and what the merge needs to weigh it.
            const int64_t slot = (static_cast<int64_t>(row0 + rr) * p.n_heads + head) * p.n_splits + blockIdx.z;
            float* dst = p.part_o + slot * HD + part * kMyDims;
            if (part == 0 && rr < n_rows) {
                p.part_ml[slot] = make_float2(m, l);
            }
#pragma unroll
            for (int g = 0; g < kMyDims / 32; ++g) {
                uint32_t v[32];
                tcgen05_ld32_nowait(my_o + 32 * g, v);  // all lanes take part
                tcgen05_wait_ld();
                if (rr < n_rows) {
#pragma unroll
                    for (int d = 0; d < 32; d += 4) {
                        *reinterpret_cast<uint4*>(dst + 32 * g + d) = make_uint4(v[d], v[d + 1], v[d + 2], v[d + 3]);
                    }
                }
            }
        } else if (ok) {
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            __nv_bfloat16* dst = p.out + (row0 + rr) * p.out_row_stride + static_cast<int64_t>(head) * HD +
                part * kMyDims;
#pragma unroll
            for (int g = 0; g < kMyDims / 32; ++g) {
                uint32_t v[32];
                tcgen05_ld32_nowait(my_o + 32 * g, v);  // all lanes take part
                tcgen05_wait_ld();
                if (rr < n_rows && n_tiles > 0) {
#pragma unroll
                    for (int d = 0; d < 32; d += 8) {
                        uint32_t w[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const __nv_bfloat162 pair = __floats2bfloat162_rn(
                                __uint_as_float(v[d + 2 * i]) * inv, __uint_as_float(v[d + 2 * i + 1]) * inv);
                            w[i] = *reinterpret_cast<const uint32_t*>(&pair);
                        }
                        *reinterpret_cast<uint4*>(dst + 32 * g + d) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
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

// Merges the splits of one launch: one warp per (query row, head) adds the splits'
// rows in split order, each weighed by 2^(its base - the largest base), and divides by
// the sum of the equally weighed row sums. Grid (heads, tiles, 16 groups of 8 rows).
template <int HD>
__global__ void __launch_bounds__(256) attention_prefill_merge_kernel(const TcPrefillParams p) {
    constexpr int kPer = HD / 32;  // dims per lane
    using Vec = typename std::conditional<kPer == 4, float4, float2>::type;
    const int4 tile = p.tiles[blockIdx.y];
    const int head = blockIdx.x, lane = threadIdx.x & 31;
    const int r = blockIdx.z * 8 + (threadIdx.x >> 5);
    if (r >= tile.y) {
        return;
    }
    const int64_t base = (static_cast<int64_t>(tile.x + r) * p.n_heads + head) * p.n_splits;
    const float2 ml = lane < p.n_splits ? p.part_ml[base + lane] : make_float2(-INFINITY, 0.0f);
    float top = ml.x;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, d));
    }
    const float weight = ml.x > -INFINITY ? exp2f(ml.x - top) : 0.0f;
    float acc[kPer] = {};
    float total = 0.0f;
    const float* src = p.part_o + base * HD + lane * kPer;
    for (int s0 = 0; s0 < p.n_splits; s0 += 4) {
        // four splits' rows in flight at a time; a split without keys for this row wrote none
        float w[4];
        Vec v[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            w[i] = __shfl_sync(0xffffffffu, weight, (s0 + i) & 31);
            w[i] = s0 + i < p.n_splits ? w[i] : 0.0f;
            if (w[i] > 0.0f) {
                v[i] = *reinterpret_cast<const Vec*>(src + static_cast<int64_t>(s0 + i) * HD);
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float l = __shfl_sync(0xffffffffu, ml.y, (s0 + i) & 31);
            if (w[i] > 0.0f) {
                total += w[i] * l;
                acc[0] += w[i] * v[i].x;
                acc[1] += w[i] * v[i].y;
                if constexpr (kPer == 4) {
                    acc[2] += w[i] * v[i].z;
                    acc[3] += w[i] * v[i].w;
                }
            }
        }
    }
    const float inv = total > 0.0f ? 1.0f / total : 0.0f;
    __nv_bfloat16* dst = p.out + (tile.x + r) * p.out_row_stride + static_cast<int64_t>(head) * HD + lane * kPer;
#pragma unroll
    for (int i = 0; i < kPer; i += 2) {
        *reinterpret_cast<__nv_bfloat162*>(dst + i) = __floats2bfloat162_rn(acc[i] * inv, acc[i + 1] * inv);
    }
}

// Folds the partial sums of a measuring launch into the step's accumulators. Block
// (pages of a request in chunks, block-table row e); a thread owns one (page of request e,
// head): it adds, tile after tile of e in list order, the tile's eight warp sums (in slot
// order) for that page to step_mass[physical page, head], and (head 0) the weights of the
// tile's rows that attend the page to step_weight[physical page]. A page belongs to one
// request, so no two threads write one element, and the order of additions is fixed.
__global__ void attention_mass_fold_prefill_kernel(const TcPrefillParams p, int n_tiles, int tile_rows,
                                                   float* __restrict__ step_mass, float* __restrict__ step_weight) {
    const int e = blockIdx.y;
    const int32_t* row = p.table + static_cast<int64_t>(e) * p.table_width;
    const int pages = min(p.mass_pages, p.table_width);
    for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < pages * p.n_heads; idx += gridDim.x * blockDim.x) {
        const int j = idx / p.n_heads, h = idx % p.n_heads;
        const int page = row[j];
        if (page < 0 || page >= p.n_pages) {
            continue;
        }
        const int key_lo = j * p.page_size, key_hi = key_lo + p.page_size - 1;
        float mass = 0.0f, weight = 0.0f;
        bool any = false;
        for (int ti = 0; ti < n_tiles; ++ti) {
            const int4 tile = p.tiles[ti];
            const int n_rows = min(tile.y, tile_rows);
            if (tile.w != e || key_lo > tile.z + n_rows - 1) {
                continue;
            }
            if (p.window > 0 && key_hi < tile.z - p.window + 1) {
                continue;  // behind every row's window
            }
            any = true;
            const float* part = p.mass_part + (static_cast<int64_t>(ti) * p.n_heads + h) * 8 * p.mass_pages + j;
#pragma unroll
            for (int slot = 0; slot < 8; ++slot) {
                mass += part[static_cast<int64_t>(slot) * p.mass_pages];
            }
            if (h == 0) {
                for (int r = 0; r < n_rows; ++r) {
                    const int pos = tile.z + r;
                    if (key_lo <= pos && (p.window <= 0 || key_hi >= pos - p.window + 1)) {
                        weight += p.query_weights[tile.x + r];
                    }
                }
            }
        }
        if (any) {
            step_mass[static_cast<int64_t>(page) * p.n_heads + h] += mass;
            if (h == 0) {
                step_weight[page] += weight;
            }
        }
    }
}

template <int HD, int HEADS, bool WIDE>
int launch_tc_prefill(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const TcPrefillParams& p,
                      int n_tiles, int n_heads, cudaStream_t stream) {
    constexpr int smem = (HEADS == 2 ? 0 : kRows * HD * 2) + stages_kv(HEADS) * 2 * kKeys * HD * 2 + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(attention_prefill_tcgen05_kernel<HD, HEADS, WIDE>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (err != cudaSuccess) {
            return pl_fail(3, "attention_prefill_tcgen05: cannot set shared memory size: %s",
                           cudaGetErrorString(err));
        }
        configured = true;
    }
    attention_prefill_tcgen05_kernel<HD, HEADS, WIDE>
        <<<dim3(WIDE ? n_heads : n_heads / HEADS, n_tiles, p.n_splits), kThreadsTc, smem, stream>>>(mq, mk, mv, p);
    PL_CHECK_LAUNCH("attention_prefill_tcgen05");
    if (p.n_splits > 1) {
        attention_prefill_merge_kernel<HD><<<dim3(n_heads, n_tiles, (WIDE ? 2 : 1) * kRows / 8), 256, 0, stream>>>(p);
        PL_CHECK_LAUNCH("attention_prefill_merge");
    }
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

// Rows per tile that the kernel can take for this GQA group: with an odd group a CTA
// works on one head and takes a tile twice as long (its halves share K and V the way
// two heads of an even group do).
PL_API int pl_attention_prefill_tcgen05_tile_rows(int group) { return group % 2 == 0 ? kRows : 2 * kRows; }

// Scratch floats that `n_splits` splits of the keys need for a step of `n_tokens` tokens.
PL_API int64_t pl_attention_prefill_scratch_floats(int n_tokens, int n_heads, int head_dim, int n_splits) {
    return n_splits <= 1 ? 0 : static_cast<int64_t>(n_tokens) * n_heads * n_splits * (head_dim + 2);
}

// As pl_attention_prefill (tiles of up to 128 rows), on tcgen05. The pools must be
// the two halves of one [pages][2][kv heads][page][head_dim] tensor: v_pool is
// k_pool + kv_heads * page * head_dim elements. With n_splits > 1 (at most 32) every
// tile's keys are shared out over that many CTAs and merged by a second kernel
// through `scratch` (pl_attention_prefill_scratch_floats floats, 16-byte aligned).
// `wide` (odd groups only; ignored for even ones): the tiles have up to 256 rows
// (pl_attention_prefill_tcgen05_tile_rows), else up to 128. `mass` (optional): also
// measures attention mass (see PlPrefillMass).
PL_API int pl_attention_prefill_tcgen05(const void* q, int64_t q_row_stride, int n_tokens, const void* k_pool,
                                        const void* v_pool, int64_t page_stride, int64_t head_stride, int page_size,
                                        int n_pages, const int32_t* table, int table_width, const int32_t* tiles,
                                        int n_tiles, void* out, int64_t out_row_stride, int n_heads, int n_kv_heads,
                                        int head_dim, int window, float scale, int n_splits, float* scratch,
                                        int wide, const PlPrefillMass* mass, int32_t* status, cudaStream_t stream) {
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
    PL_REQUIRE(n_tiles <= 65535, "attention_prefill_tcgen05: too many tiles in one launch (%d)", n_tiles);
    PL_REQUIRE(n_splits >= 1 && n_splits <= 32, "attention_prefill_tcgen05: 1 to 32 splits, not %d", n_splits);
    PL_REQUIRE(n_splits == 1 || (scratch != nullptr && (reinterpret_cast<uintptr_t>(scratch) & 15) == 0),
               "attention_prefill_tcgen05: %d splits need 16-byte aligned scratch memory", n_splits);
    PL_REQUIRE(scale > 0.0f, "attention_prefill_tcgen05: the scale must be positive (%g)", static_cast<double>(scale));
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
    p.q = static_cast<const __nv_bfloat16*>(q);
    p.q_row_stride = q_row_stride;
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
    p.n_heads = n_heads;
    p.n_splits = n_splits;
    p.part_o = scratch;
    p.part_ml = n_splits > 1
        ? reinterpret_cast<float2*>(scratch + static_cast<int64_t>(n_tokens) * n_heads * n_splits * head_dim)
        : nullptr;
    // Two heads of one kv head per CTA when the group is even; else one head per CTA, and
    // a tile of up to 256 rows as two halves (`wide`), or of up to 128 rows with both
    // warpgroups on it.
    const bool pairs = p.group % 2 == 0;
    p.query_weights = nullptr;
    p.mass_part = nullptr;
    p.mass_pages = 0;
    p.scale = scale;
    if (mass != nullptr) {
        PL_REQUIRE(pairs || wide, "attention_prefill_tcgen05: attention mass is measured with two heads or two halves "
                                  "of a tile per CTA (an even group, or wide tiles)");
        PL_REQUIRE(page_size == 16 || page_size == 32 || page_size == 64,
                   "attention_prefill_tcgen05: attention mass is measured for pages of 16, 32 or 64 tokens, not %d",
                   page_size);
        PL_REQUIRE(mass->query_weights != nullptr && mass->scratch != nullptr && mass->step_mass != nullptr &&
                       mass->step_weight != nullptr && mass->pages >= table_width && mass->table_rows >= 1 &&
                       mass->table_rows <= 65535,
                   "attention_prefill_tcgen05: attention mass needs weights, scratch for %d pages a row and the "
                   "step's sums",
                   table_width);
        p.query_weights = mass->query_weights;
        p.mass_part = mass->scratch;
        p.mass_pages = mass->pages;
    }
    int code;
    if (head_dim == 64) {
        code = pairs ? launch_tc_prefill<64, 2, false>(mq, mk, mv, p, n_tiles, n_heads, stream)
            : wide   ? launch_tc_prefill<64, 2, true>(mq, mk, mv, p, n_tiles, n_heads, stream)
                     : launch_tc_prefill<64, 1, false>(mq, mk, mv, p, n_tiles, n_heads, stream);
    } else {
        code = pairs ? launch_tc_prefill<128, 2, false>(mq, mk, mv, p, n_tiles, n_heads, stream)
            : wide   ? launch_tc_prefill<128, 2, true>(mq, mk, mv, p, n_tiles, n_heads, stream)
                     : launch_tc_prefill<128, 1, false>(mq, mk, mv, p, n_tiles, n_heads, stream);
    }
    if (code != 0 || mass == nullptr) {
        return code;
    }
    // Every block-table row may own tiles; rows without any find nothing to add.
    const int items = table_width * n_heads;
    const int blocks = (items + 255) / 256 > 32 ? 32 : (items + 255) / 256;
    attention_mass_fold_prefill_kernel<<<dim3(blocks, mass->table_rows), 256, 0, stream>>>(
        p, n_tiles, (!pairs && wide) ? 2 * kRows : kRows, mass->step_mass, mass->step_weight);
    PL_CHECK_LAUNCH("attention_mass_fold_prefill");
    return 0;
}
