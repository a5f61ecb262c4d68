// Paged attention for single decode tokens in bfloat16: split over the keys, the
// query heads of a GQA group packed into one tensor-core tile.
//
// A decode token reads its request's whole cache once; the kernel is bound by HBM.
// CTA (split, kv head, token) walks a contiguous share of the request's 16-key
// tiles. Its warps take tiles round-robin; each warp streams K and V tiles into its
// own ring of shared-memory stages with cp.async (16-byte chunks, XOR-swizzled so
// ldmatrix is conflict-free) and keeps the group's (<= 16) query heads as the M
// rows of m16n8k16 MMAs: S = Q K^T, online softmax in fp32 (base 2, the scale
// folded into the exponent), O += P V with P rounded to bf16. Warps are merged
// through shared memory. The splits of one (kv head, token) are merged in one of two
// ways. Up to sixteen splits form a thread-block cluster: the (head, dim) outputs are
// dealt out to the ranks in contiguous runs, every rank sends its unnormalised
// partial sums for a run to the owner's shared memory (st.async: stores that count
// their bytes on the owner's barrier) and its (m, l) to everyone, and each owner
// merges in rank order and writes its run. More splits than that write (o, m, l) to
// scratch and a second kernel merges them, in the same order with the same
// arithmetic. Split boundaries depend only on the request's length and the launch's
// split count.
//
// The reference's counterparts: attn_decode_tc_kernel and paged_decode_split /
// combine kernels, pulsarlm-core/src/kernels/paged_attention.cu:432-584.
#include "cluster_helpers.cuh"
#include "mma_helpers.cuh"
#include "rope_helpers.cuh"

PL_API int pl_attention_decode_resident_clusters(int head_dim, int group, int n_splits);

// Position encoding and the new keys' write folded into a decode attention call (see
// DecodeParams): k_new and v_new [T, n_kv_heads, head_dim] bf16 with q's row stride,
// inv_freq fp64 [rotary / 2]; only rotary == head_dim is taken.
struct PlDecodeRope {
    const void* k_new;
    const void* v_new;
    const double* inv_freq;
    int rotary;
};

namespace {

constexpr int kTile = 16;  // keys per tile

struct DecodeParams {
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
    const int32_t* pos;
    const int32_t* entry;
    __nv_bfloat16* out;
    int64_t out_row_stride;
    float* part_o;   // [tokens, heads, splits, HD]
    float* part_ml;  // [tokens, heads, splits, 2]
    int n_heads;
    int group;
    int window;
    float scale_log2;
    int n_splits;
    int cluster;  // 1: the splits are the ranks of a thread-block cluster and merge among themselves
    int32_t* status;
    // Attention mass (optional): every 16-key tile's largest masked score per head, in the
    // exponent's units (scaled score * log2 e), at [(token * heads + head) * max_tiles + tile].
    float* tile_max;
    int max_tiles;
    // Work-list mode (optional; never with `cluster`): CTA x takes item x = {token, first
    // tile, tiles, split | splits << 12} instead of an equal share of token blockIdx.z. The
    // partial results of token t's split s sit at slot token_slot[t] + s of the scratch
    // ([slot][head]); the last CTA of a (token, kv head) to finish, by counters[token *
    // kv heads + kv head] (zero before the launch and again after it), merges them.
    // Position encoding and the new key's write folded in (optional): q arrives unrotated and
    // is rotated as it is loaded; the CTA and warp whose share holds the token's own tile
    // first rotates the token's new key k_new[t] (rows of q_row_stride elements, like q) and
    // stores it with v_new[t] at the token's place in the pools. rope_freq: fp64
    // [HD / 2] radians per position (the whole head is rotated).
    const __nv_bfloat16* k_new;
    const __nv_bfloat16* v_new;
    const double* rope_freq;
    const int32_t* items;
    int n_items;
    int n_kv_heads;
    const int32_t* token_slot;
    int32_t* counters;
};

// In-cluster merge: outputs are counted in groups of four dims ("vecs"); rank r owns
// vecs [first_vec(r), first_vec(r + 1)).
__host__ __device__ constexpr int first_vec(int rank, int n_vec, int splits) {
    return (rank * n_vec + splits - 1) / splits;
}
__host__ __device__ constexpr int owned_vecs_max(int n_vec, int splits) { return (n_vec + splits - 1) / splits; }
// Bytes of the receive buffers behind the rings: partial sums [rank][vec of mine] as
// float4, then (m, l) [rank][16] as float2.
__host__ __device__ constexpr int merge_bytes(int n_vec, int splits) {
    return splits * owned_vecs_max(n_vec, splits) * 16 + splits * 16 * 8;
}

// One share of one (token, kv head): split `split` of `n_splits` equal shares, or in
// work-list mode the tiles [item_first, item_first + item_tiles).
template <int HD, int WARPS, int STAGES>
__device__ __forceinline__ void attention_decode_share(const DecodeParams& p, unsigned char* smem, const int split,
                                                       const int kv_head, const int t, const int n_splits,
                                                       const int item_first, const int item_tiles) {
    constexpr int kRowBytes = HD * 2;            // a row of the cache
    constexpr int kRowSmem = padded_row_bytes(HD);  // a row in shared memory (the swizzle stays inside it)
    constexpr int kChunks = HD / 8;              // 16-byte chunks per row
    constexpr int kTileBytes = kTile * kRowSmem;
    constexpr int kStageBytes = 2 * kTileBytes;  // K tile then V tile
    constexpr bool kFoldsRope = HD % 32 == 0;    // (a rotated pair's halves lie in whole fragments of q)

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, tig = lane & 3;

    __shared__ __align__(8) uint64_t recv_bar;
    __shared__ int abort_flag;
    const int n_vec = p.group * (HD / 4);
    const int my_first = first_vec(split, n_vec, p.n_splits);
    const int my_vecs = first_vec(split + 1, n_vec, p.n_splits) - my_first;
    if (p.cluster) {
        if (threadIdx.x == 0) {
            mbar_init(&recv_bar, 1);
            abort_flag = 0;
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            // what the other ranks will send: partial sums of my vecs, and their (m, l) of every head
            mbar_expect_tx(&recv_bar, static_cast<uint32_t>(p.n_splits - 1) * (my_vecs * 16 + p.group * 8));
        }
        __syncthreads();
        cluster_arrive_all();  // "my barrier is ready"; waited for before anything is sent
    }
    const int ctx = p.pos[t] + 1;
    const int first = p.window > 0 ? max(0, ctx - p.window) : 0;
    const int tile_first = first / kTile, tile_end = (ctx + kTile - 1) / kTile;
    const int per_split = p.items != nullptr ? item_tiles : (tile_end - tile_first + n_splits - 1) / n_splits;
    const int t0 = p.items != nullptr ? item_first : tile_first + split * per_split;
    const int t1 = min(t0 + per_split, tile_end);
    const int32_t* row = p.table + static_cast<int64_t>(p.entry[t]) * p.table_width;
    __shared__ float rope_cs[HD / 2], rope_sn[HD / 2];
    if (kFoldsRope && p.rope_freq != nullptr && threadIdx.x < HD / 2) {  // (the position is a step input: before the wait)
        rope_sincos(ctx - 1, p.rope_freq[threadIdx.x], rope_cs[threadIdx.x], rope_sn[threadIdx.x]);
    }

    unsigned char* ring = smem + warp * (STAGES * kStageBytes);
    const int my_tiles = t1 > t0 + warp ? (t1 - t0 - warp + WARPS - 1) / WARPS : 0;

    int my_page = 0;  // lane L holds the page of this warp's tile 32 * (i / 32) + L
    auto issue = [&](int i) {  // loads this warp's i-th tile into stage i % STAGES
        if (i % 32 == 0 && i < my_tiles) {
            // one coalesced look-up of the block table for the next 32 tiles
            const int mine = i + lane;
            my_page = mine < my_tiles ? row[((t0 + warp + mine * WARPS) * kTile) / p.page_size] : 0;
            if (my_page < 0 || my_page >= p.n_pages) {
                if (p.status != nullptr) {
                    atomicOr(p.status, 4);
                }
                my_page = 0;  // stay in bounds; the result is flagged as wrong
            }
        }
        if (i < my_tiles) {
            const int tile = t0 + warp + i * WARPS;
            const int key0 = tile * kTile;
            const int page = __shfl_sync(0xffffffffu, my_page, i % 32);
            const int64_t offset = page * p.page_stride + kv_head * p.head_stride +
                static_cast<int64_t>(key0 % p.page_size) * HD;
            const unsigned char* ksrc = reinterpret_cast<const unsigned char*>(p.k_pool + offset);
            const unsigned char* vsrc = reinterpret_cast<const unsigned char*>(p.v_pool + offset);
            unsigned char* stage = ring + (i % STAGES) * kStageBytes;
#pragma unroll
            for (int c = lane; c < kTile * kChunks; c += 32) {
                const int r = c / kChunks, ch = c % kChunks;
                const int dst = r * kRowSmem + ((ch ^ (r & 7)) * 16);
                cp_async_16(stage + dst, ksrc + r * kRowBytes + ch * 16);
                cp_async_16(stage + kTileBytes + dst, vsrc + r * kRowBytes + ch * 16);
            }
        }
        cp_async_commit();
    };

    float o[HD / 8][4];
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) {
        o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;
    }
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.0f, l_hi = 0.0f;

    // The first tiles are asked for before the wait on earlier kernels: they hold keys of
    // earlier steps, which no kernel of this step writes. Only the tile with the newest
    // key (the last of the request) is written in this step. By another kernel (the rotation
    // kernel, or the layer whose cache this one reads): a warp whose first tiles include it
    // waits first. By this kernel (the rotation folded in): the warp that owns the tile asks
    // for it like for any other and puts the token's own row into the tile in shared memory
    // once it has landed; no round trip through global memory, no fence.
    const bool writes_own = kFoldsRope && p.rope_freq != nullptr && p.k_new != nullptr;
    __shared__ __align__(16) __nv_bfloat16 own_kv[2][HD];  // the token's rotated key and its value
    bool patch = false;
    bool early = true;
    if (!writes_own) {
#pragma unroll
        for (int i = 0; i < STAGES - 1; ++i) {
            early = early && !(i < my_tiles && t0 + warp + i * WARPS == tile_end - 1);
        }
    }
    if (early) {
#pragma unroll
        for (int i = 0; i < STAGES - 1; ++i) {
            issue(i);
        }
    }
    pl_grid_wait();
    // Q fragments: rows g and g + 8 of the group's heads (zero past the group).
    uint32_t qa[HD / 16][4];
    const __nv_bfloat16* qbase = p.q + t * p.q_row_stride + static_cast<int64_t>(kv_head) * p.group * HD;
    const bool lo_ok = g < p.group, hi_ok = g + 8 < p.group;
    if (!kFoldsRope || p.rope_freq == nullptr) {
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
            const int d = 16 * kk + 2 * tig;
            qa[kk][0] = lo_ok ? *reinterpret_cast<const uint32_t*>(qbase + g * HD + d) : 0u;
            qa[kk][1] = hi_ok ? *reinterpret_cast<const uint32_t*>(qbase + (g + 8) * HD + d) : 0u;
            qa[kk][2] = lo_ok ? *reinterpret_cast<const uint32_t*>(qbase + g * HD + d + 8) : 0u;
            qa[kk][3] = hi_ok ? *reinterpret_cast<const uint32_t*>(qbase + (g + 8) * HD + d + 8) : 0u;
        }
    } else {
        __syncthreads();  // the angles are in place
        // Rotated as loaded: dims (d, d + HD/2) are a pair, and both lie in this thread's fragments
        // kk and kk + HD/32. Rounded to bfloat16 once, like the rotation kernel's store.
#pragma unroll
        for (int kk = 0; kk < HD / 32; ++kk) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int d = 16 * kk + 2 * tig + (e >> 1) * 8;
                const bool ok = (e & 1) ? hi_ok : lo_ok;
                const __nv_bfloat16* x = qbase + (g + (e & 1) * 8) * HD + d;
                float2 lo = make_float2(0.0f, 0.0f), hi = make_float2(0.0f, 0.0f);
                if (ok) {
                    lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(x));
                    hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(x + HD / 2));
                }
                const float c0 = rope_cs[d], s0 = rope_sn[d], c1 = rope_cs[d + 1], s1 = rope_sn[d + 1];
                qa[kk][e] = pack_bf16(rope_lo(lo.x, hi.x, c0, s0), rope_lo(lo.y, hi.y, c1, s1));
                qa[kk + HD / 32][e] = pack_bf16(rope_hi(lo.x, hi.x, c0, s0), rope_hi(lo.y, hi.y, c1, s1));
            }
        }
        // The token's own key and value: rotated and stored by the warp whose tiles end with
        // the token's tile (for later steps), and kept for that tile in shared memory.
        const int own_tile = tile_end - 1;
        if (p.k_new != nullptr && own_tile >= t0 && own_tile < t1 && (own_tile - t0) % WARPS == warp) {
            const int position = ctx - 1;
            const int page = row[position / p.page_size];
            if (page < 0 || page >= p.n_pages) {
                if (lane == 0 && p.status != nullptr) {
                    atomicOr(p.status, 2);
                }
            } else {
                const int64_t from = t * p.q_row_stride + static_cast<int64_t>(kv_head) * HD;
                const int64_t at = page * p.page_stride + kv_head * p.head_stride +
                    static_cast<int64_t>(position % p.page_size) * HD;
                __nv_bfloat16* k_out = const_cast<__nv_bfloat16*>(p.k_pool) + at;
                __nv_bfloat16* v_out = const_cast<__nv_bfloat16*>(p.v_pool) + at;
#pragma unroll
                for (int j = lane; j < HD / 2; j += 32) {
                    const float lo = __bfloat162float(p.k_new[from + j]);
                    const float hi = __bfloat162float(p.k_new[from + j + HD / 2]);
                    own_kv[0][j] = k_out[j] = __float2bfloat16_rn(rope_lo(lo, hi, rope_cs[j], rope_sn[j]));
                    own_kv[0][j + HD / 2] = k_out[j + HD / 2] =
                        __float2bfloat16_rn(rope_hi(lo, hi, rope_cs[j], rope_sn[j]));
                    own_kv[1][j] = v_out[j] = p.v_new[from + j];
                    own_kv[1][j + HD / 2] = v_out[j + HD / 2] = p.v_new[from + j + HD / 2];
                }
                patch = true;
            }
            __syncwarp();
        }
    }
    if (!early) {
#pragma unroll
        for (int i = 0; i < STAGES - 1; ++i) {
            issue(i);
        }
    }
    for (int i = 0; i < my_tiles; ++i) {
        cp_async_wait<STAGES - 2>();
        __syncwarp();
        const unsigned char* stage = ring + (i % STAGES) * kStageBytes;
        const int key0 = (t0 + warp + i * WARPS) * kTile;
        if (patch && i == my_tiles - 1) {
            // the token's own tile: its row as this warp made it, over what the copy brought
            unsigned char* tile = ring + (i % STAGES) * kStageBytes;
            const int r = (ctx - 1) % kTile;
            for (int c = lane; c < 2 * kChunks; c += 32) {
                const int which = c / kChunks, ch = c % kChunks;
                *reinterpret_cast<uint4*>(tile + which * kTileBytes + r * kRowSmem + ((ch ^ (r & 7)) * 16)) =
                    *reinterpret_cast<const uint4*>(&own_kv[which][ch * 8]);
            }
            __syncwarp();
        }

        float s[2][4] = {{0.0f, 0.0f, 0.0f, 0.0f}, {0.0f, 0.0f, 0.0f, 0.0f}};
        {
            const int mi = lane >> 3, r = lane & 7;
            const int key = (mi >> 1) * 8 + r;
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk) {
                uint32_t b[4];
                const int chunk = 2 * kk + (mi & 1);
                ldmatrix_x4(b, stage + key * kRowSmem + ((chunk ^ (key & 7)) * 16));
                mma_bf16(s[0], qa[kk], b[0], b[1]);
                mma_bf16(s[1], qa[kk], b[2], b[3]);
            }
        }
        // Mask keys outside [first, ctx); move to the base-2 exponent domain.
        float tile_lo = -INFINITY, tile_hi = -INFINITY;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = key0 + 8 * j + 2 * tig + (e & 1);
                const bool ok = key >= first && key < ctx;
                s[j][e] = ok ? s[j][e] * p.scale_log2 : -INFINITY;
            }
            tile_lo = fmaxf(tile_lo, fmaxf(s[j][0], s[j][1]));
            tile_hi = fmaxf(tile_hi, fmaxf(s[j][2], s[j][3]));
        }
        tile_lo = fmaxf(tile_lo, __shfl_xor_sync(0xffffffffu, tile_lo, 1));
        tile_lo = fmaxf(tile_lo, __shfl_xor_sync(0xffffffffu, tile_lo, 2));
        tile_hi = fmaxf(tile_hi, __shfl_xor_sync(0xffffffffu, tile_hi, 1));
        tile_hi = fmaxf(tile_hi, __shfl_xor_sync(0xffffffffu, tile_hi, 2));
        if (p.tile_max != nullptr && tig == 0) {
            // One warp of one split owns this tile: a plain store, the same whatever the split count.
            const int tile = key0 / kTile;
            const int64_t head0 = static_cast<int64_t>(t) * p.n_heads + kv_head * p.group;
            if (g < p.group) {
                p.tile_max[(head0 + g) * p.max_tiles + tile] = tile_lo;
            }
            if (g + 8 < p.group) {
                p.tile_max[(head0 + g + 8) * p.max_tiles + tile] = tile_hi;
            }
        }
        const float new_lo = fmaxf(m_lo, tile_lo), new_hi = fmaxf(m_hi, tile_hi);
        // A row that has seen no key yet keeps exponent base 0 (all its p are 0).
        const float base_lo = new_lo == -INFINITY ? 0.0f : new_lo;
        const float base_hi = new_hi == -INFINITY ? 0.0f : new_hi;
        const float corr_lo = exp2f(m_lo - base_lo), corr_hi = exp2f(m_hi - base_hi);
        m_lo = new_lo;
        m_hi = new_hi;
        uint32_t pa[4];
        {
            const float p00 = exp2f(s[0][0] - base_lo), p01 = exp2f(s[0][1] - base_lo);
            const float p02 = exp2f(s[0][2] - base_hi), p03 = exp2f(s[0][3] - base_hi);
            const float p10 = exp2f(s[1][0] - base_lo), p11 = exp2f(s[1][1] - base_lo);
            const float p12 = exp2f(s[1][2] - base_hi), p13 = exp2f(s[1][3] - base_hi);
            l_lo = l_lo * corr_lo + (p00 + p01 + p10 + p11);
            l_hi = l_hi * corr_hi + (p02 + p03 + p12 + p13);
            pa[0] = pack_bf16(p00, p01);
            pa[1] = pack_bf16(p02, p03);
            pa[2] = pack_bf16(p10, p11);
            pa[3] = pack_bf16(p12, p13);
        }
#pragma unroll
        for (int n = 0; n < HD / 8; ++n) {
            o[n][0] *= corr_lo;
            o[n][1] *= corr_lo;
            o[n][2] *= corr_hi;
            o[n][3] *= corr_hi;
        }
        {
            const int mi = lane >> 3, r = lane & 7;
            const int key = (mi & 1) * 8 + r;
            const unsigned char* vt = stage + kTileBytes;
#pragma unroll
            for (int dp = 0; dp < HD / 16; ++dp) {
                uint32_t b[4];
                const int chunk = 2 * dp + (mi >> 1);
                ldmatrix_x4_trans(b, vt + key * kRowSmem + ((chunk ^ (key & 7)) * 16));
                mma_bf16(o[2 * dp], pa, b[0], b[1]);
                mma_bf16(o[2 * dp + 1], pa, b[2], b[3]);
            }
        }
        __syncwarp();
        issue(i + STAGES - 1);
    }
    cp_async_wait<0>();
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);

    // Merge the warps through shared memory (the rings are done with).
    __syncthreads();
    float* red_o = reinterpret_cast<float*>(smem);        // [WARPS][16][HD]
    float* red_m = red_o + WARPS * 16 * HD;               // [WARPS][16]
    float* red_l = red_m + WARPS * 16;                    // [WARPS][16]
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) {
        const int d = 8 * n + 2 * tig;
        if (g < p.group) {
            red_o[(warp * 16 + g) * HD + d] = o[n][0];
            red_o[(warp * 16 + g) * HD + d + 1] = o[n][1];
        }
        if (g + 8 < p.group) {
            red_o[(warp * 16 + g + 8) * HD + d] = o[n][2];
            red_o[(warp * 16 + g + 8) * HD + d + 1] = o[n][3];
        }
    }
    if (tig == 0) {
        red_m[warp * 16 + g] = m_lo;
        red_m[warp * 16 + g + 8] = m_hi;
        red_l[warp * 16 + g] = l_lo;
        red_l[warp * 16 + g + 8] = l_hi;
    }
    __syncthreads();
    if (p.cluster) {
        float4* recv_o = reinterpret_cast<float4*>(smem + WARPS * STAGES * kStageBytes);
        const int most = owned_vecs_max(n_vec, p.n_splits);
        float2* recv_ml = reinterpret_cast<float2*>(recv_o + p.n_splits * most);
        cluster_wait_all();  // long since complete: every rank arrived at its start
        for (int vec = threadIdx.x; vec < n_vec; vec += WARPS * 32) {
            const int r = vec / (HD / 4), d = (vec % (HD / 4)) * 4;
            float m = -INFINITY;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                m = fmaxf(m, red_m[w * 16 + r]);
            }
            float l = 0.0f;
            float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (m > -INFINITY) {
#pragma unroll
                for (int w = 0; w < WARPS; ++w) {
                    const float scale = exp2f(red_m[w * 16 + r] - m);
                    const float4 part = *reinterpret_cast<const float4*>(&red_o[(w * 16 + r) * HD + d]);
                    l += red_l[w * 16 + r] * scale;
                    acc.x += part.x * scale;
                    acc.y += part.y * scale;
                    acc.z += part.z * scale;
                    acc.w += part.w * scale;
                }
            }
            const int owner = vec * p.n_splits / n_vec;
            float4* at = recv_o + split * most + (vec - first_vec(owner, n_vec, p.n_splits));
            if (owner == split) {
                *at = acc;
            } else {
                cluster_store4_counted(cluster_map(at, owner), acc, cluster_map(&recv_bar, owner));
            }
            if (d == 0) {  // this head's (m, l) goes to every rank
                float2* ml = recv_ml + split * 16 + r;
                for (int peer = 0; peer < p.n_splits; ++peer) {
                    if (peer == split) {
                        *ml = make_float2(m, l);
                    } else {
                        cluster_store2_counted(cluster_map(ml, peer), make_float2(m, l), cluster_map(&recv_bar, peer));
                    }
                }
            }
        }
        __syncthreads();  // what this rank kept for itself is in place
        if (!mbar_wait_cluster(&recv_bar, 0u, &abort_flag)) {
            if (threadIdx.x == 0 && p.status != nullptr) {
                atomicOr(p.status, 8);
            }
            return;
        }
        for (int mine = threadIdx.x; mine < my_vecs; mine += WARPS * 32) {
            const int vec = my_first + mine;
            const int r = vec / (HD / 4), d = (vec % (HD / 4)) * 4;
            float m = -INFINITY;
            for (int s = 0; s < p.n_splits; ++s) {
                m = fmaxf(m, recv_ml[s * 16 + r].x);
            }
            float l = 0.0f;
            float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (m > -INFINITY) {
                for (int s = 0; s < p.n_splits; ++s) {  // rank order, whoever arrived first
                    const float2 ml = recv_ml[s * 16 + r];
                    const float scale = exp2f(ml.x - m);
                    const float4 part = recv_o[s * most + mine];
                    l += ml.y * scale;
                    acc.x += part.x * scale;
                    acc.y += part.y * scale;
                    acc.z += part.z * scale;
                    acc.w += part.w * scale;
                }
            }
            const int h = kv_head * p.group + r;
            __nv_bfloat16* dst = p.out + t * p.out_row_stride + static_cast<int64_t>(h) * HD + d;
            if (l > 0.0f) {
                dst[0] = __float2bfloat16_rn(acc.x / l);
                dst[1] = __float2bfloat16_rn(acc.y / l);
                dst[2] = __float2bfloat16_rn(acc.z / l);
                dst[3] = __float2bfloat16_rn(acc.w / l);
            } else {
                dst[0] = dst[1] = dst[2] = dst[3] = __float2bfloat16_rn(0.0f);
            }
        }
        return;
    }
    for (int idx = threadIdx.x; idx < p.group * HD; idx += WARPS * 32) {
        const int r = idx / HD, d = idx % HD;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            m = fmaxf(m, red_m[w * 16 + r]);
        }
        float l = 0.0f, acc = 0.0f;
        if (m > -INFINITY) {
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                const float scale = exp2f(red_m[w * 16 + r] - m);
                l += red_l[w * 16 + r] * scale;
                acc += red_o[(w * 16 + r) * HD + d] * scale;
            }
        }
        const int h = kv_head * p.group + r;
        if (n_splits == 1) {
            p.out[t * p.out_row_stride + static_cast<int64_t>(h) * HD + d] =
                __float2bfloat16_rn(l > 0.0f ? acc / l : 0.0f);
        } else {
            const int64_t slot = p.items != nullptr
                ? static_cast<int64_t>(p.token_slot[t] + split) * p.n_heads + h
                : (static_cast<int64_t>(t) * p.n_heads + h) * n_splits + split;
            p.part_o[slot * HD + d] = acc;
            if (d == 0) {
                p.part_ml[slot * 2] = m;
                p.part_ml[slot * 2 + 1] = l;
            }
        }
    }
    if (p.items == nullptr || n_splits == 1) {
        return;
    }
    // Work-list mode: whoever finishes a (token, kv head) last merges its splits, in split
    // order with the merge kernel's arithmetic, and leaves the counter at zero.
    __shared__ int is_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        int32_t* counter = p.counters + 2 + static_cast<int64_t>(t) * p.n_kv_heads + kv_head;
        is_last = atomicAdd(counter, 1) == n_splits - 1;
        if (is_last) {
            *counter = 0;
        }
    }
    __syncthreads();
    if (!is_last) {
        return;
    }
    __threadfence();
    // (The rings are free: every warp passed the barriers above after its last tile.) Per head
    // the largest base, then per split its weight 2^(base - largest) and the weighed sum of the
    // row sums, through shared memory; then every thread adds up four dims of one head over the
    // splits, in split order, eight loads in flight at a time.
    const int64_t slot0 = static_cast<int64_t>(p.token_slot[t]) * p.n_heads + kv_head * p.group;
    constexpr int kChunk = 128;                                  // splits per pass
    float* weight = reinterpret_cast<float*>(smem);              // [kChunk][16]
    float* row_max = weight + kChunk * 16;                       // [16]
    float* row_sum = row_max + 16;                               // [16]
    float* partial = row_sum + 16;                               // [WARPS * 32]
    {
        // largest base per head: thread (row = tid % 16, splits tid / 16, + 8, ...)
        const int r = threadIdx.x & 15;
        float m = -INFINITY;
        if (r < p.group) {
            for (int sp = threadIdx.x >> 4; sp < n_splits; sp += (WARPS * 32) >> 4) {
                m = fmaxf(m, __ldcg(&p.part_ml[(slot0 + static_cast<int64_t>(sp) * p.n_heads + r) * 2]));
            }
        }
        partial[threadIdx.x] = m;
        __syncthreads();
        if (threadIdx.x < 16) {
            for (int i = threadIdx.x + 16; i < WARPS * 32; i += 16) {
                m = fmaxf(m, partial[i]);
            }
            row_max[threadIdx.x] = m;
            row_sum[threadIdx.x] = 0.0f;
        }
        __syncthreads();
    }
    float4 acc[(16 * (HD / 4) + WARPS * 32 - 1) / (WARPS * 32)];
#pragma unroll
    for (int i = 0; i < static_cast<int>(sizeof(acc) / sizeof(acc[0])); ++i) {
        acc[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    for (int s0 = 0; s0 < n_splits; s0 += kChunk) {
        const int count = min(kChunk, n_splits - s0);
        for (int i = threadIdx.x; i < count * 16; i += WARPS * 32) {
            const int sp = i >> 4, r = i & 15;
            float w = 0.0f;
            if (r < p.group && row_max[r] > -INFINITY) {
                w = exp2f(__ldcg(&p.part_ml[(slot0 + static_cast<int64_t>(s0 + sp) * p.n_heads + r) * 2]) - row_max[r]);
            }
            weight[i] = w;
        }
        __syncthreads();
        if (threadIdx.x < p.group) {  // the row sums, in split order
            float l = row_sum[threadIdx.x];
            for (int sp = 0; sp < count; ++sp) {
                l += __ldcg(&p.part_ml[(slot0 + static_cast<int64_t>(s0 + sp) * p.n_heads + threadIdx.x) * 2 + 1]) *
                    weight[sp * 16 + threadIdx.x];
            }
            row_sum[threadIdx.x] = l;
        }
#pragma unroll
        for (int i = 0; i < static_cast<int>(sizeof(acc) / sizeof(acc[0])); ++i) {
            const int vec = threadIdx.x + i * WARPS * 32;
            if (vec < n_vec) {
                const int r = vec / (HD / 4), d = (vec % (HD / 4)) * 4;
                const float* from = p.part_o + (slot0 + static_cast<int64_t>(s0) * p.n_heads + r) * HD + d;
                const int64_t step = static_cast<int64_t>(p.n_heads) * HD;
                int sp = 0;
                for (; sp + 8 <= count; sp += 8) {
                    float4 part[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        part[j] = __ldcg(reinterpret_cast<const float4*>(from + (sp + j) * step));
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float w = weight[(sp + j) * 16 + r];
                        acc[i].x += part[j].x * w;
                        acc[i].y += part[j].y * w;
                        acc[i].z += part[j].z * w;
                        acc[i].w += part[j].w * w;
                    }
                }
                for (; sp < count; ++sp) {
                    const float4 part = __ldcg(reinterpret_cast<const float4*>(from + sp * step));
                    const float w = weight[sp * 16 + r];
                    acc[i].x += part.x * w;
                    acc[i].y += part.y * w;
                    acc[i].z += part.z * w;
                    acc[i].w += part.w * w;
                }
            }
        }
        __syncthreads();  // the weights are rewritten by the next pass; the row sums are in place
    }
#pragma unroll
    for (int i = 0; i < static_cast<int>(sizeof(acc) / sizeof(acc[0])); ++i) {
        const int vec = threadIdx.x + i * WARPS * 32;
        if (vec < n_vec) {
            const int r = vec / (HD / 4), d = (vec % (HD / 4)) * 4;
            const float l = row_sum[r];
            __nv_bfloat16* dst = p.out + t * p.out_row_stride + static_cast<int64_t>(kv_head * p.group + r) * HD + d;
            dst[0] = __float2bfloat16_rn(l > 0.0f ? acc[i].x / l : 0.0f);
            dst[1] = __float2bfloat16_rn(l > 0.0f ? acc[i].y / l : 0.0f);
            dst[2] = __float2bfloat16_rn(l > 0.0f ? acc[i].z / l : 0.0f);
            dst[3] = __float2bfloat16_rn(l > 0.0f ? acc[i].w / l : 0.0f);
        }
    }
}

// Grid (splits, kv heads, tokens), or in work-list mode a line of CTAs that take (item, kv
// head) pairs off a queue, in list order, each as soon as it is free: counters[0] is the
// queue's head and counters[1] counts the CTAs that found it empty; the last of them puts
// both back to zero for the next launch.
template <int HD, int WARPS, int STAGES>
__global__ void __launch_bounds__(WARPS * 32, HD <= 64 ? 4 : 2) attention_decode_kernel(const DecodeParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    pl_grid_trigger();  // positions and block tables are step inputs, read before the wait
    // One loop for both modes (the share's code once, and few registers live across it): with
    // equal shares it runs once; with a work list it runs until the list's pairs are used up.
    __shared__ int next;
    int work = blockIdx.x, n_work = 1;
    bool queued = false;
    if (p.items != nullptr) {
        // Rows of no tiles are padding; the last of them says in its first field how many rows are not.
        const int4 last_row = reinterpret_cast<const int4*>(p.items)[p.n_items - 1];
        n_work = (last_row.z > 0 ? p.n_items : min(max(last_row.x, 0), p.n_items)) * p.n_kv_heads;
        queued = static_cast<int>(gridDim.x) < n_work;  // else a CTA for every pair: nobody needs the queue
        if (work >= n_work) {
            return;
        }
    }
    // (Claiming a pair ahead of the one in work, to hide the queue's answer time, measured
    // much slower: with two or three pairs per CTA the early claims leave CTAs idle.)
    while (true) {
        int split = blockIdx.x, kv_head = blockIdx.y, t = blockIdx.z, n_splits = p.n_splits, first = 0, tiles = 0;
        if (p.items != nullptr) {
            const int4 item = reinterpret_cast<const int4*>(p.items)[work / p.n_kv_heads];
            split = item.w & 4095;
            kv_head = work % p.n_kv_heads;
            t = item.x;
            n_splits = item.w >> 12;
            first = item.y;
            tiles = item.z;
        }
        attention_decode_share<HD, WARPS, STAGES>(p, smem, split, kv_head, t, n_splits, first, tiles);
        if (!queued) {
            return;
        }
        // (The counters are touched only after the kernels before this one have ended: an
        // earlier launch that shares them is among those. The share has waited for them.)
        __syncthreads();  // the next pair reuses the rings, and `next` has been read by all
        if (threadIdx.x == 0) {
            next = static_cast<int>(gridDim.x) + atomicAdd(p.counters, 1);
        }
        __syncthreads();
        work = next;
        if (work >= n_work) {
            break;
        }
    }
    if (threadIdx.x == 0) {
        if (atomicAdd(p.counters + 1, 1) == static_cast<int>(gridDim.x) - 1) {
            // Everyone has taken its last look at the queue: this launch is done with it.
            p.counters[0] = 0;
            p.counters[1] = 0;
            __threadfence();
        }
    }
}

// One block per (token, head): merges the splits' partials.
template <int HD>
__global__ void attention_decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                              __nv_bfloat16* __restrict__ out, int64_t out_row_stride, int n_heads,
                                              int n_splits) {
    pl_grid_trigger();
    pl_grid_wait();
    const int t = blockIdx.y, h = blockIdx.x;
    const int64_t base = (static_cast<int64_t>(t) * n_heads + h) * n_splits;
    float m = -INFINITY;
    for (int s = 0; s < n_splits; ++s) {
        m = fmaxf(m, part_ml[(base + s) * 2]);
    }
    for (int d = threadIdx.x; d < HD; d += blockDim.x) {
        float l = 0.0f, acc = 0.0f;
        if (m > -INFINITY) {
            for (int s = 0; s < n_splits; ++s) {
                const float scale = exp2f(part_ml[(base + s) * 2] - m);
                l += part_ml[(base + s) * 2 + 1] * scale;
                acc += part_o[(base + s) * HD + d] * scale;
            }
        }
        out[t * out_row_stride + static_cast<int64_t>(h) * HD + d] = __float2bfloat16_rn(l > 0.0f ? acc / l : 0.0f);
    }
}

constexpr int kWarps = 4;
// Ring depth per warp. (Six stages at head size 64, the same bytes as three at 128, measured slower: two CTAs
// per SM instead of four, 47.9 -> 55.4 us at batch 64 and 2,400 keys. The kernel wants warps, not depth.)
constexpr int stages_of(int) { return 3; }
// Shared memory of the warps' rings at one head size.
constexpr int ring_bytes(int head_dim) { return kWarps * stages_of(head_dim) * 2 * kTile * padded_row_bytes(head_dim); }

// `return CALL(HD);` with the head size as a constant, for the sizes the kernel is built for.
#define PL_DECODE_HEAD_SIZES(head_dim, CALL, otherwise) \
    switch (head_dim) {                                 \
        case 32: return CALL(32);                       \
        case 48: return CALL(48);                       \
        case 64: return CALL(64);                       \
        case 80: return CALL(80);                       \
        case 96: return CALL(96);                       \
        case 112: return CALL(112);                     \
        case 128: return CALL(128);                     \
        default: return otherwise;                      \
    }

constexpr int kClusterSplitsMax = 16;  // the largest cluster the part takes (above 8: opted into per kernel)

template <int HD>
int launch_decode(const DecodeParams& params, int n_tokens, int n_kv_heads, bool allow_cluster, cudaStream_t stream) {
    constexpr int rings = ring_bytes(HD);
    static_assert(rings >= kWarps * 16 * (HD + 2) * 4, "the merge buffers must fit in the rings");
    constexpr int most_merge = merge_bytes(16 * (HD / 4), kClusterSplitsMax) + 1024;
    static bool configured = false, big_clusters = false;
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(attention_decode_kernel<HD, kWarps, stages_of(HD)>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, rings + most_merge);
        if (err != cudaSuccess) {
            return pl_fail(3, "attention_decode: cannot set shared memory size: %s", cudaGetErrorString(err));
        }
        // clusters of more than eight CTAs (if the device refuses, such split counts go through scratch)
        big_clusters = cudaFuncSetAttribute(attention_decode_kernel<HD, kWarps, stages_of(HD)>,
                                            cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess;
        cudaGetLastError();
        configured = true;
    }
    DecodeParams p = params;
    p.cluster = p.items == nullptr && allow_cluster && p.n_splits >= 2 && p.n_splits <= (big_clusters ? kClusterSplitsMax : 8);
    if (p.cluster && p.n_splits > 8) {
        // a cluster this large has to find its SMs within one GPC: ask once whether any fits
        static int room[17][kClusterSplitsMax + 1] = {};
        int& known = room[p.group][p.n_splits];
        if (known == 0) {
            known = pl_attention_decode_resident_clusters(HD, p.group, p.n_splits) > 0 ? 1 : -1;
        }
        p.cluster = known > 0;
    }
    if (!p.cluster && p.n_splits > 1 && p.part_o == nullptr) {
        return pl_fail(2, "attention_decode: %d splits need scratch memory", p.n_splits);
    }
    const dim3 grid(p.n_splits, n_kv_heads, n_tokens);  // work-list mode: n_splits carries the item count here
    if (p.items != nullptr) {
        // As many CTAs as the device holds at once (or as there are items); each walks the list in strides.
        static int resident = 0;
        if (resident == 0) {
            int device = 0, sms = 0, each = 0;
            cudaGetDevice(&device);
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
            if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&each, attention_decode_kernel<HD, kWarps, stages_of(HD)>,
                                                              kWarps * 32, rings) != cudaSuccess || each < 1) {
                cudaGetLastError();
                each = 1;
            }
            resident = sms * each;
        }
        p.n_items = p.n_splits;
        p.n_splits = 1;
        p.n_kv_heads = n_kv_heads;
        // A CTA for every (token, kv head), at least as many as the device holds at once, at most one
        // per pair: requests left whole then never touch the queue, and what cutting adds goes through it.
        const int64_t n_work = static_cast<int64_t>(p.n_items) * n_kv_heads;
        int64_t ctas = static_cast<int64_t>(n_tokens) * n_kv_heads;
        ctas = ctas < resident ? resident : ctas;
        ctas = ctas > n_work ? n_work : ctas;
        pl_launch_overlapped(attention_decode_kernel<HD, kWarps, stages_of(HD)>, dim3(static_cast<int>(ctas), 1, 1),
                             kWarps * 32, rings, stream, p);
        PL_CHECK_LAUNCH("attention_decode (work list)");
        return 0;
    }
    if (p.cluster) {
        cudaLaunchConfig_t config = {};
        config.gridDim = grid;
        config.blockDim = dim3(kWarps * 32);
        config.dynamicSmemBytes = rings + merge_bytes(p.group * (HD / 4), p.n_splits);
        config.stream = stream;
        cudaLaunchAttribute attributes[2];
        attributes[0].id = cudaLaunchAttributeClusterDimension;
        attributes[0].val.clusterDim.x = p.n_splits;
        attributes[0].val.clusterDim.y = 1;
        attributes[0].val.clusterDim.z = 1;
        attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attributes[1].val.programmaticStreamSerializationAllowed = 1;
        config.attrs = attributes;
        config.numAttrs = pl_overlap_enabled() ? 2 : 1;
        const cudaError_t err = cudaLaunchKernelEx(&config, attention_decode_kernel<HD, kWarps, stages_of(HD)>, p);
        if (err != cudaSuccess) {
            return pl_fail(3, "attention_decode: launch failed: %s", cudaGetErrorString(err));
        }
        return 0;
    }
    pl_launch_overlapped(attention_decode_kernel<HD, kWarps, stages_of(HD)>, grid, kWarps * 32, rings, stream, p);
    PL_CHECK_LAUNCH("attention_decode");
    if (p.n_splits > 1) {
        pl_launch_overlapped(attention_decode_merge_kernel<HD>, dim3(p.n_heads, n_tokens), HD <= 64 ? 64 : 128, 0,
                             stream, p.part_o, p.part_ml, p.out, p.out_row_stride, p.n_heads, p.n_splits);
        PL_CHECK_LAUNCH("attention_decode_merge");
    }
    return 0;
}

}  // namespace

// 1 when pl_attention_decode takes this shape, else 0 (the caller then uses the
// CUDA-core kernel, which takes every shape).
PL_API int pl_attention_decode_supports(int head_dim, int group, int page_size, int dtype) {
    return dtype == PL_BF16 && head_dim % 16 == 0 && head_dim >= 32 && head_dim <= 128 && group >= 1 &&
        group <= 16 && page_size % kTile == 0;
}

namespace {

template <int HD>
int resident_clusters_of(int group, int n_splits) {
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(n_splits, 64, 64);
    config.blockDim = dim3(kWarps * 32);
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = n_splits;
    attribute[0].val.clusterDim.y = 1;
    attribute[0].val.clusterDim.z = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    int clusters = 0;
    constexpr int rings = ring_bytes(HD);
    cudaFuncSetAttribute(attention_decode_kernel<HD, kWarps, stages_of(HD)>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         rings + merge_bytes(16 * (HD / 4), kClusterSplitsMax) + 1024);
    cudaFuncSetAttribute(attention_decode_kernel<HD, kWarps, stages_of(HD)>,
                         cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    config.dynamicSmemBytes = rings + merge_bytes(group * (HD / 4), n_splits);
    if (cudaOccupancyMaxActiveClusters(&clusters, attention_decode_kernel<HD, kWarps, stages_of(HD)>, &config) !=
        cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return clusters;
}

template <int HD>
int ctas_per_sm_of() {
    int ctas = 0;
    constexpr int rings = ring_bytes(HD);
    cudaFuncSetAttribute(attention_decode_kernel<HD, kWarps, stages_of(HD)>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         rings + merge_bytes(16 * (HD / 4), kClusterSplitsMax) + 1024);
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&ctas, attention_decode_kernel<HD, kWarps, stages_of(HD)>,
                                                      kWarps * 32, rings) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return ctas;
}

}  // namespace

// How many clusters of `n_splits` CTAs of the decode kernel the device holds at once
// (0: unknown or not a cluster size). A launch with more (kv head, token) pairs than
// this runs its clusters in more than one wave.
PL_API int pl_attention_decode_resident_clusters(int head_dim, int group, int n_splits) {
    if (n_splits < 2 || n_splits > kClusterSplitsMax) {
        return 0;
    }
#define PL_CALL(HD) resident_clusters_of<HD>(group, n_splits)
    PL_DECODE_HEAD_SIZES(head_dim, PL_CALL, 0)
#undef PL_CALL
}

// Scratch floats needed for `n_tokens` tokens at `n_splits` splits.
PL_API int64_t pl_attention_decode_scratch_floats(int n_tokens, int n_heads, int head_dim, int n_splits) {
    return n_splits <= 1 ? 0 : static_cast<int64_t>(n_tokens) * n_heads * n_splits * (head_dim + 2);
}

namespace {

int run_attention_decode(bool allow_cluster, const void* q, int64_t q_row_stride, const void* k_pool, const void* v_pool,
                               int64_t page_stride, int64_t head_stride, int page_size, int n_pages,
                               const int32_t* table, int table_width, const int32_t* pos, const int32_t* entry,
                               void* out, int64_t out_row_stride, int n_tokens, int n_heads, int n_kv_heads,
                               int head_dim, int window, float scale, int n_splits, float* scratch,
                               int32_t* status, cudaStream_t stream, float* tile_max = nullptr, int max_tiles = 0,
                               const int32_t* items = nullptr, const int32_t* token_slot = nullptr,
                               int32_t* counters = nullptr, const PlDecodeRope* rope = nullptr) {
    PL_REQUIRE(n_tokens >= 0 && n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0,
               "attention_decode: bad sizes tokens=%d heads=%d kv_heads=%d", n_tokens, n_heads, n_kv_heads);
    const int group = n_heads / n_kv_heads;
    PL_REQUIRE(pl_attention_decode_supports(head_dim, group, page_size, PL_BF16),
               "attention_decode: unsupported shape head_dim=%d group=%d page=%d (takes head sizes 32 to 128 in steps of 16, "
               "groups of at most 16 heads, pages that are multiples of 16 tokens)",
               head_dim, group, page_size);
    PL_REQUIRE(n_splits >= 1 && n_splits <= 65535 && n_kv_heads <= 65535 && n_tokens <= 65535,
               "attention_decode: grid too large (splits=%d kv_heads=%d tokens=%d)", n_splits, n_kv_heads, n_tokens);
    PL_REQUIRE((n_splits <= 8 && allow_cluster) || n_splits == 1 || scratch != nullptr,
               "attention_decode: %d splits need scratch memory", n_splits);
    PL_REQUIRE(q_row_stride % 2 == 0 && (reinterpret_cast<uintptr_t>(q) & 3) == 0,
               "attention_decode: q must be 4-byte aligned with an even row stride");
    PL_REQUIRE((reinterpret_cast<uintptr_t>(k_pool) & 15) == 0 && (reinterpret_cast<uintptr_t>(v_pool) & 15) == 0 &&
                   page_stride % 8 == 0 && head_stride % 8 == 0,
               "attention_decode: pools must be 16-byte aligned with strides that are multiples of 8 elements");
    if (n_tokens == 0) {
        return 0;
    }
    DecodeParams p;
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
    p.pos = pos;
    p.entry = entry;
    p.out = static_cast<__nv_bfloat16*>(out);
    p.out_row_stride = out_row_stride;
    p.part_o = scratch;
    // (work-list mode: n_splits is the number of items, which bounds the slots in use)
    p.part_ml = scratch == nullptr ? nullptr
        : scratch + static_cast<int64_t>(items != nullptr ? 1 : n_tokens) * n_heads * n_splits * head_dim;
    p.items = items;
    p.n_items = 0;
    p.n_kv_heads = n_kv_heads;
    p.k_new = p.v_new = nullptr;
    p.rope_freq = nullptr;
    if (rope != nullptr) {
        PL_REQUIRE(rope->rotary == head_dim && head_dim % 32 == 0 && rope->inv_freq != nullptr &&
                       (rope->k_new == nullptr) == (rope->v_new == nullptr),
                   "attention_decode: the folded position encoding rotates the whole head (rotary %d, head_dim %d), takes "
                   "head sizes that are multiples of 32, and k and v together",
                   rope->rotary, head_dim);
        p.k_new = static_cast<const __nv_bfloat16*>(rope->k_new);
        p.v_new = static_cast<const __nv_bfloat16*>(rope->v_new);
        p.rope_freq = rope->inv_freq;
    }
    p.token_slot = token_slot;
    p.counters = counters;
    p.n_heads = n_heads;
    p.group = group;
    p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.n_splits = n_splits;
    p.status = status;
    p.tile_max = tile_max;
    p.max_tiles = max_tiles;
    PL_REQUIRE(tile_max == nullptr || max_tiles >= static_cast<int64_t>(table_width) * page_size / kTile,
               "attention_decode: %d tiles per row of tile maxima do not cover a table of %d pages", max_tiles,
               table_width);
#define PL_CALL(HD) launch_decode<HD>(p, n_tokens, n_kv_heads, allow_cluster, stream)
    PL_DECODE_HEAD_SIZES(head_dim, PL_CALL, pl_fail(2, "attention_decode: head size %d", head_dim))
#undef PL_CALL
}

}  // namespace

// bf16 only. q and out [T, n_heads, head_dim] with row strides; one query per token
// at position pos[t]; pools and table as in pl_attention_simt. scratch: at least
// pl_attention_decode_scratch_floats floats when n_splits > 8 (fewer splits merge
// inside a cluster and leave it untouched). rope (optional): q arrives unrotated and the
// call also rotates and stores the tokens' new keys and values (see PlDecodeRope).
PL_API int pl_attention_decode(const void* q, int64_t q_row_stride, const void* k_pool, const void* v_pool,
                               int64_t page_stride, int64_t head_stride, int page_size, int n_pages,
                               const int32_t* table, int table_width, const int32_t* pos, const int32_t* entry,
                               void* out, int64_t out_row_stride, int n_tokens, int n_heads, int n_kv_heads,
                               int head_dim, int window, float scale, int n_splits, float* scratch,
                               const PlDecodeRope* rope, int32_t* status, cudaStream_t stream) {
    return run_attention_decode(true, q, q_row_stride, k_pool, v_pool, page_stride, head_stride, page_size, n_pages,
                                table, table_width, pos, entry, out, out_row_stride, n_tokens, n_heads, n_kv_heads,
                                head_dim, window, scale, n_splits, scratch, status, stream, nullptr, 0, nullptr,
                                nullptr, nullptr, rope);
}

// pl_attention_decode over a work list instead of equal shares: for batches whose requests
// differ in length, or are many. items: int32 [n_items, 4] rows {token, first 16-key tile,
// tiles, split | splits << 12}; rows of no tiles are padding and come last, and the last row,
// if it is padding, holds in its first field the number of rows that are not. The pairs
// (item, kv head) go to CTAs in list order: the first by position, the rest off a queue. A token of one split writes its output itself. The splits of a token
// with more write partial results to slot token_slot[token] + split of scratch (fp32,
// n_items * n_heads * (head_dim + 2) floats; slots below n_items), and the CTA that
// finishes a (token, kv head) last merges them in split order. counters: int32 [2 + n_tokens *
// n_kv_heads], all zero before the call and again after it (the work queue's head, its
// leavers, and arrivals per token and kv head). The caller makes the items
// cover each token's tiles [first attended key / 16, ceil((pos + 1) / 16)) exactly once.
PL_API int pl_attention_decode_items(const void* q, int64_t q_row_stride, const void* k_pool, const void* v_pool,
                                     int64_t page_stride, int64_t head_stride, int page_size, int n_pages,
                                     const int32_t* table, int table_width, const int32_t* pos,
                                     const int32_t* entry, void* out, int64_t out_row_stride, int n_tokens,
                                     int n_heads, int n_kv_heads, int head_dim, int window, float scale,
                                     const int32_t* items, int n_items, const int32_t* token_slot, float* scratch,
                                     int32_t* counters, const PlDecodeRope* rope, int32_t* status,
                                     cudaStream_t stream) {
    PL_REQUIRE(items != nullptr && token_slot != nullptr && counters != nullptr && scratch != nullptr && n_items >= 1,
               "attention_decode_items: needs items, token_slot, counters and scratch");
    PL_REQUIRE((reinterpret_cast<uintptr_t>(items) & 15) == 0, "attention_decode_items: items must be 16-byte aligned");
    return run_attention_decode(false, q, q_row_stride, k_pool, v_pool, page_stride, head_stride, page_size, n_pages,
                                table, table_width, pos, entry, out, out_row_stride, n_tokens, n_heads, n_kv_heads,
                                head_dim, window, scale, n_items, scratch, status, stream, nullptr, 0, items, token_slot,
                                counters, rope);
}

// How many CTAs of the decode kernel one SM holds at once.
PL_API int pl_attention_decode_ctas_per_sm(int head_dim) {
#define PL_CALL(HD) ctas_per_sm_of<HD>()
    PL_DECODE_HEAD_SIZES(head_dim, PL_CALL, 0)
#undef PL_CALL
}

namespace {

// One thread per (page of the request, head): folds a decode step's tile maxima into the
// per-page accumulators. mass[page, head] = mass * keep + w * (largest scaled score of the
// token over the page's keys it attends), weight[page] likewise with w alone, where w =
// decay, keep = 1 - decay for pages the request already held and 0 for the page this
// token opens (it may hold a former owner's sums). Every page belongs to one request and
// a request has one token in the step: no two threads touch the same element.
__global__ void attention_mass_fold_decode_kernel(const float* __restrict__ tile_max, int max_tiles,
                                                  const int32_t* __restrict__ table, int table_width,
                                                  const int32_t* __restrict__ pos, const int32_t* __restrict__ entry,
                                                  float* __restrict__ mass, float* __restrict__ weight, int n_pages,
                                                  int n_heads, int page_size, int window, float decay) {
    pl_grid_trigger();
    pl_grid_wait();
    const int t = blockIdx.y;
    const int position = pos[t];
    const int ctx = position + 1;
    const int first = window > 0 ? max(0, ctx - window) : 0;
    const int page_first = first / page_size, page_last = position / page_size;
    const int32_t* row = table + static_cast<int64_t>(entry[t]) * table_width;
    const int tiles_per_page = page_size / kTile;
    const int items = (page_last - page_first + 1) * n_heads;
    for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < items; idx += gridDim.x * blockDim.x) {
        const int j = page_first + idx / n_heads, h = idx % n_heads;
        const int page = row[j];
        if (page < 0 || page >= n_pages) {
            continue;  // (the attention kernel has flagged it)
        }
        // the tiles of the page that hold attended keys
        const int tile0 = max(j * tiles_per_page, first / kTile);
        const int tile1 = min((j + 1) * tiles_per_page, (ctx + kTile - 1) / kTile);
        float largest = -INFINITY;
        const float* maxima = tile_max + (static_cast<int64_t>(t) * n_heads + h) * max_tiles;
        for (int tile = tile0; tile < tile1; ++tile) {
            largest = fmaxf(largest, maxima[tile]);
        }
        if (!(largest > -INFINITY)) {
            continue;
        }
        const float keep = j * page_size >= position ? 0.0f : 1.0f - decay;
        const int64_t at = static_cast<int64_t>(page) * n_heads + h;
        mass[at] = mass[at] * keep + decay * (largest * 0.6931471805599453f);  // back from base-2 units
        if (h == 0) {
            weight[page] = weight[page] * keep + decay;
        }
    }
}

}  // namespace

// pl_attention_decode that also measures attention mass: the kernel records every
// tile's largest score in tile_max (fp32 [tokens, heads, max_tiles], max_tiles >=
// table_width * page_size / 16), and a second kernel folds them into mass [pages,
// heads] and weight [pages] (see attention_mass_fold_decode_kernel). decay in (0, 1].
PL_API int pl_attention_decode_mass(const void* q, int64_t q_row_stride, const void* k_pool, const void* v_pool,
                                    int64_t page_stride, int64_t head_stride, int page_size, int n_pages,
                                    const int32_t* table, int table_width, const int32_t* pos, const int32_t* entry,
                                    void* out, int64_t out_row_stride, int n_tokens, int n_heads, int n_kv_heads,
                                    int head_dim, int window, float scale, int n_splits, float* scratch,
                                    float* tile_max, int max_tiles, float* mass, float* weight, float decay,
                                    int32_t* status, cudaStream_t stream) {
    PL_REQUIRE(tile_max != nullptr && mass != nullptr && weight != nullptr && decay > 0.0f && decay <= 1.0f,
               "attention_decode_mass: needs tile_max, mass, weight and a decay in (0, 1]");
    const int code = run_attention_decode(true, q, q_row_stride, k_pool, v_pool, page_stride, head_stride, page_size,
                                          n_pages, table, table_width, pos, entry, out, out_row_stride, n_tokens,
                                          n_heads, n_kv_heads, head_dim, window, scale, n_splits, scratch, status,
                                          stream, tile_max, max_tiles);
    if (code != 0 || n_tokens == 0) {
        return code;
    }
    const int items = table_width * n_heads;
    const dim3 grid(items < 256 ? 1 : (items + 255) / 256 > 64 ? 64 : (items + 255) / 256, n_tokens);
    pl_launch_overlapped(attention_mass_fold_decode_kernel, grid, 256, 0, stream, tile_max, max_tiles, table,
                         table_width, pos, entry, mass, weight, n_pages, n_heads, page_size, window, decay);
    PL_CHECK_LAUNCH("attention_mass_fold_decode");
    return 0;
}

// ---------------------------------------------------------------------------
// The same kernel for callers that cannot allocate: scratch from a built-in array.
// See no_alloc.h for who this is for and the rules of use.
#include "no_alloc.h"

namespace {

// In host code this name is only a stand-in for the symbol: it is not a device
// address and must not be passed to a kernel. Host code asks the runtime for the
// address (below); device code could name the array directly.
static __device__ __align__(256) float static_scratch[PL_STATIC_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;
float* static_scratch_address[kMaxDevices] = {};

// The array's address on the current device, looked up once per device.
int find_static_scratch(float** address) {
    int device = 0;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess) {
        return pl_fail(3, "attention_decode_static: cudaGetDevice failed: %s", cudaGetErrorString(err));
    }
    if (device < 0 || device >= kMaxDevices) {
        return pl_fail(2, "attention_decode_static: device index %d is beyond the %d this entry point tracks", device,
                       kMaxDevices);
    }
    if (static_scratch_address[device] == nullptr) {
        float* found = nullptr;
        err = cudaGetSymbolAddress(reinterpret_cast<void**>(&found), static_scratch);
        if (err != cudaSuccess || found == nullptr) {
            return pl_fail(3, "attention_decode_static: cannot find the built-in scratch on device %d: %s", device,
                           cudaGetErrorString(err));
        }
        static_scratch_address[device] = found;
    }
    *address = static_scratch_address[device];
    return 0;
}

}  // namespace

PL_API int64_t pl_static_scratch_floats() { return PL_STATIC_SCRATCH_FLOATS; }

PL_API int pl_attention_decode_static(const void* q, int64_t q_row_stride, const void* k_pool, const void* v_pool,
                                      int64_t page_stride, int64_t head_stride, int page_size, int n_pages,
                                      const int32_t* table, int table_width, const int32_t* pos,
                                      const int32_t* entry, void* out, int64_t out_row_stride, int n_tokens,
                                      int n_heads, int n_kv_heads, int head_dim, int window, float scale,
                                      int n_splits, int32_t* status, cudaStream_t stream) {
    // The same limits as the launcher's, checked before the sizes are multiplied: with them
    // the product below stays far inside 64 bits.
    PL_REQUIRE(n_tokens >= 0 && n_tokens <= 65535 && n_heads > 0 && n_heads <= 65535 && n_kv_heads > 0 &&
                   n_kv_heads <= 65535 && (head_dim == 64 || head_dim == 128) && n_splits >= 1 && n_splits <= 65535,
               "attention_decode_static: bad sizes tokens=%d heads=%d kv_heads=%d head_dim=%d splits=%d (at most 65535 "
               "each; head size 64 or 128)", n_tokens, n_heads, n_kv_heads, head_dim, n_splits);
    const int64_t needed = pl_attention_decode_scratch_floats(n_tokens, n_heads, head_dim, n_splits);
    PL_REQUIRE(needed <= PL_STATIC_SCRATCH_FLOATS,
               "attention_decode_static: %d tokens x %d heads x %d splits need %lld floats of scratch, the built-in "
               "array holds %lld; use fewer splits or fewer tokens per call",
               n_tokens, n_heads, n_splits, static_cast<long long>(needed),
               static_cast<long long>(PL_STATIC_SCRATCH_FLOATS));
    float* scratch = nullptr;
    if (const int code = find_static_scratch(&scratch)) {
        return code;
    }
    return run_attention_decode(false, q, q_row_stride, k_pool, v_pool, page_stride, head_stride, page_size, n_pages,
                                table, table_width, pos, entry, out, out_row_stride, n_tokens, n_heads, n_kv_heads,
                                head_dim, window, scale, n_splits, scratch, status, stream);
}
