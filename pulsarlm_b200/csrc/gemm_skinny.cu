// bfloat16 matrix product for a handful of tokens (a decode step's projections):
//   Y[T, N] = X[T, K] * W[N, K]^T,  T <= 64, fp32 accumulation.
//
// Such a product only streams weights, so the kernel is built around keeping every
// SM's loads in flight and around the time between the last byte and the result:
//
// * The weights sit on the MMA's M axis (tiles of 128 output features), the tokens
//   on its N axis (16, 32 or 64), as in the large-product kernel (gemm_pair.cu):
//   `tcgen05.mma.cta_group::1.kind::f16`, operands in shared memory through TMA with
//   128-byte swizzle, the accumulator in tensor memory.
// * One CTA computes one tile over one part of k. The grid is (splits, tiles), `splits`
//   chosen so that about one and a half CTAs per SM stream at once where the shape allows
//   (see make_skinny_plan for the rule and the measurements behind it).
// * The CTAs that share a tile form a thread-block cluster and add their partial
//   sums through distributed shared memory: the tile's 128 features are dealt out to
//   the ranks in contiguous runs; every rank stores its values for a feature into
//   the owner's shared memory, sixteen bytes at a time, with stores that count their
//   bytes on the owner's barrier (st.async), and the owner, once all the bytes it
//   expects are there, adds the parts in rank order (so the sum does not depend on
//   arrival order) and writes its features. No scratch in global memory, no
//   counters, no fences.
// * The kernel asks for its first stages of weights before it waits for the kernels
//   before it (programmatic dependent launch): they stream in under the tail of the
//   predecessor, and only the activations are loaded after the wait.
//
// Waits on barriers are bounded: after the limit the CTA raises bit 8 of the status
// word, stops, lets loads and peers' stores in flight land, frees its tensor memory
// and returns.
//
// The reference leaves these products to a library (`at::linear`,
// pulsarlm-core/src/engine/model/llama.cpp:67-69, 81, 91, 93).
#include "tcgen05_helpers.cuh"

namespace {

constexpr int kTileM = 128;
constexpr int kBlockK = 64;
constexpr int kThreads = 192;
constexpr int kSmemSmall = 110 * 1024;  // leaves room for a CTA of the next launch on the same SM
constexpr int kSmemLarge = 200 * 1024;  // deeper pipeline, for launches of few CTAs
constexpr int kMaxStages = 12;
constexpr int kMaxSplits = 8;            // the portable cluster size

struct SkinnyParams {
    void* y;  // [T, N] bf16 or fp32
    int t, n, k;
    int64_t ldy;
    int out_f32;
    int k_blocks;      // ceil(K / 64)
    int kb_per_split;  // k blocks per rank
    int stages;        // pipeline depth (shared memory given: stages * stage bytes + receive buffer)
    int32_t* status;
    // Where the activations come from. 0: x itself, through TMA. 1: x = silu(g) * u made on
    // the way in, g and u the two halves [T, K] of `gated` [T, 2K] (the gate/up projection's
    // output): the epilogue warps, idle until the accumulator is done, read g and u, form
    // the product in fp32, round it once and store it where the MMA reads its B operand
    // (same layout as a TMA tile with 128-byte swizzle). T <= 16.
    int x_mode;
    const __nv_bfloat16* gated;
    int64_t ld_gated;
};

// The receive buffer: [rank][feature of mine][token], rows of tn + 4 floats (16-byte
// aligned, and the padding spreads the rows over the banks). With `splits` ranks a
// rank owns at most ceil(128 / splits) features.
__host__ __device__ constexpr int recv_row(int tn) { return tn + 4; }
__host__ __device__ constexpr int owned_max(int splits) { return (kTileM + splits - 1) / splits; }
__host__ __device__ constexpr int recv_bytes(int tn, int splits) {
    return splits > 1 ? splits * owned_max(splits) * recv_row(tn) * 4 : 0;
}
// Features [first_feature(r), first_feature(r + 1)) belong to rank r.
__host__ __device__ constexpr int first_feature(int rank, int splits) { return (rank * kTileM + splits - 1) / splits; }
constexpr int recv_bytes_max(int tn) {
    int most = 0;
    for (int s = 2; s <= kMaxSplits; ++s) {
        most = recv_bytes(tn, s) > most ? recv_bytes(tn, s) : most;
    }
    return most;
}
__host__ __device__ constexpr int stage_bytes(int tn) { return kTileM * kBlockK * 2 + tn * kBlockK * 2; }
constexpr int stages_within(int tn, int budget) {
    const int fit = (budget - 1024 - recv_bytes_max(tn)) / stage_bytes(tn);
    return fit > kMaxStages ? kMaxStages : fit;
}

// (Two CTAs of a launch with a CTA for every SM and more share an SM: the registers must
// allow it, 168 a thread at most.)
template <int TN>
__global__ void __launch_bounds__(kThreads, 2)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                   const SkinnyParams p) {
    const int kStages = p.stages;
    constexpr int kBytesA = kTileM * kBlockK * 2;
    constexpr int kBytesB = TN * kBlockK * 2;
    constexpr int kStageBytes = kBytesA + kBytesB;
    constexpr uint32_t kColumns = TN < 32 ? 32 : TN;
    constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(TN >> 3) << 17) |
        (static_cast<uint32_t>(kTileM >> 4) << 24);

    extern __shared__ unsigned char raw_smem[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) &
                                                            ~static_cast<uintptr_t>(1023));
    float* recv = reinterpret_cast<float*>(tiles + kStages * kStageBytes);  // [rank][feature of mine][token]
    __shared__ __align__(8) uint64_t full_bar[kMaxStages];
    __shared__ __align__(8) uint64_t empty_bar[kMaxStages];
    __shared__ __align__(8) uint64_t acc_full;
    __shared__ __align__(8) uint64_t recv_bar;
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int splits = gridDim.x, rank = blockIdx.x, tile = blockIdx.y;
    pl_grid_trigger();
    // the features this rank owns, and the bytes its peers send for them (tokens in fours)
    const int my_first = first_feature(rank, splits);
    const int my_features = first_feature(rank + 1, splits) - my_first;
    const int sent_tokens = (min(p.t, TN) + 3) & ~3;
    const uint32_t expected = static_cast<uint32_t>(splits - 1) * my_features * sent_tokens * 4;
    if (threadIdx.x == 0) {
        tensormap_prefetch(&map_w);
        tensormap_prefetch(&map_x);
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full_bar[s], p.x_mode == 0 ? 1 : 2);  // (+ the warp that makes the stage's x)
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(&acc_full, 1);
        mbar_init(&recv_bar, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (expected > 0) {
            mbar_expect_tx(&recv_bar, expected);
        }
    }
    if (warp == 1) {
        tcgen05_alloc(&tmem_base_slot, kColumns);
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    if (splits > 1) {
        cluster_arrive_all();  // "my barrier is ready"; the epilogue waits for everyone's before it sends
    }

    const int kb0 = rank * p.kb_per_split;
    const int n_units = min(p.kb_per_split, p.k_blocks - kb0);
    const int n0 = tile * kTileM;

    // The producer and the issuer run their loops with all lanes of their warp, so that
    // counters, addresses and descriptors stay in uniform registers, and let one elected
    // lane issue.
    if (warp == 0) {
        // ------------------------------------------------ producer
        const int early = min(n_units, kStages);
        for (int u = 0; u < early; ++u) {  // weights: nobody writes them, no need to wait
            if (elect_one()) {
                mbar_expect_tx(&full_bar[u], p.x_mode == 0 ? kStageBytes : kBytesA);
                tma_load_2d(tiles + u * kStageBytes, &map_w, (kb0 + u) * kBlockK, n0, &full_bar[u]);
            }
            __syncwarp();
        }
        pl_grid_wait();
        for (int u = 0; u < early && p.x_mode == 0; ++u) {
            if (elect_one()) {
                tma_load_2d(tiles + u * kStageBytes + kBytesA, &map_x, (kb0 + u) * kBlockK, 0, &full_bar[u]);
            }
            __syncwarp();
        }
        int stage = early % kStages;
        uint32_t phase = early == kStages ? 1u : 0u;
        for (int u = early; u < n_units; ++u) {
            if (!mbar_wait(&empty_bar[stage], phase ^ 1u, &abort_flag)) {
                break;
            }
            unsigned char* a = tiles + stage * kStageBytes;
            if (elect_one()) {
                mbar_expect_tx(&full_bar[stage], p.x_mode == 0 ? kStageBytes : kBytesA);
                tma_load_2d(a, &map_w, (kb0 + u) * kBlockK, n0, &full_bar[stage]);
                if (p.x_mode == 0) {
                    tma_load_2d(a + kBytesA, &map_x, (kb0 + u) * kBlockK, 0, &full_bar[stage]);
                }
            }
            __syncwarp();
            if (++stage == kStages) {
                stage = 0;
                phase ^= 1u;
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer
        pl_grid_wait();  // the bounded waits below then time this kernel's own work only
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int u = 0; u < n_units; ++u) {
            if (!mbar_wait(&full_bar[stage], phase, &abort_flag)) {
                ok = false;
                break;
            }
            tcgen05_fence_after();
            const unsigned char* a = tiles + stage * kStageBytes;
            const uint64_t desc_a = smem_descriptor(a), desc_b = smem_descriptor(a + kBytesA);
            if (elect_one()) {
#pragma unroll
                for (int k = 0; k < kBlockK / 16; ++k) {
                    tcgen05_mma(tmem_base, desc_a + 2 * k, desc_b + 2 * k, kIdesc, (u > 0 || k > 0) ? 1u : 0u);
                }
                tcgen05_commit(&empty_bar[stage]);
            }
            __syncwarp();
            if (++stage == kStages) {
                stage = 0;
                phase ^= 1u;
            }
        }
        if (ok) {
            if (elect_one()) {
                tcgen05_commit(&acc_full);
            }
            __syncwarp();
        }
    }
    if (warp >= 2) {
        // ------------------------------------------------ epilogue (warps 2..5)
        const int lane_group = warp & 3;  // the tensor-memory lanes a warp may read: 32 * (warp % 4)
        const int feature = lane_group * 32 + lane;
        const int n = n0 + feature;
        const uint32_t tmem_row = tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16);
        pl_grid_wait();
        if constexpr (TN == 16) {
            if (p.x_mode == 1) {
                // These four warps make the activation tiles, each every fourth stage, so that one
                // warp's waits, fence and arrival overlap the others' arithmetic: lane (token, half
                // a row) of a 16 x 64 tile, four 16-byte chunks each. A warp asks for its next
                // stage's g and u before it works on the one it has.
                const int mine = warp - 2;                     // stages mine, mine + 4, ...
                const int token = lane >> 1, chunk0 = (lane & 1) * 4;
                const bool row_ok = token < p.t;
                const __nv_bfloat16* g_row = p.gated + static_cast<int64_t>(token) * p.ld_gated;
                uint4 g_in[2][4], u_in[2][4];
                auto fetch = [&](int u, uint4 (&g)[4], uint4 (&v)[4]) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int k = (kb0 + u) * kBlockK + (chunk0 + c) * 8;
                        if (row_ok && u < n_units && k < p.k) {  // (k is a multiple of 8, and so is p.k)
                            g[c] = *reinterpret_cast<const uint4*>(g_row + k);
                            v[c] = *reinterpret_cast<const uint4*>(g_row + p.k + k);
                        } else {
                            g[c] = make_uint4(0u, 0u, 0u, 0u);
                            v[c] = g[c];
                        }
                    }
                };
                auto make = [&](int u, const uint4 (&g_all)[4], const uint4 (&u_all)[4]) -> bool {
                    const int stage = u % kStages;
                    if (u >= kStages && !mbar_wait(&empty_bar[stage], ((u / kStages) & 1u) ^ 1u, &abort_flag)) {
                        return false;
                    }
                    unsigned char* tile = tiles + stage * kStageBytes + kBytesA + token * 128;
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g_all[c]);
                        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u_all[c]);
                        uint4 out;
                        uint32_t* o = reinterpret_cast<uint32_t*>(&out);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float2 g = __bfloat1622float2(g2[j]), v = __bfloat1622float2(u2[j]);
                            // (the SwiGLU kernel's own expression: the same bits)
                            const __nv_bfloat162 pair = __floats2bfloat162_rn(
                                __fdividef(g.x, 1.0f + __expf(-g.x)) * v.x, __fdividef(g.y, 1.0f + __expf(-g.y)) * v.y);
                            o[j] = *reinterpret_cast<const uint32_t*>(&pair);
                        }
                        *reinterpret_cast<uint4*>(tile + (((chunk0 + c) ^ (token & 7)) << 4)) = out;
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive(&full_bar[stage]);
                    }
                    return true;
                };
                fetch(mine, g_in[0], u_in[0]);
                for (int u = mine; u < n_units; u += 8) {
                    fetch(u + 4, g_in[1], u_in[1]);
                    if (!make(u, g_in[0], u_in[0])) {
                        break;
                    }
                    if (u + 4 >= n_units) {
                        break;
                    }
                    fetch(u + 8, g_in[0], u_in[0]);
                    if (!make(u + 4, g_in[1], u_in[1])) {
                        break;
                    }
                }
            }
        }
        const bool have = mbar_wait(&acc_full, 0u, &abort_flag);
        tcgen05_fence_after();
        if (have && splits == 1) {
#pragma unroll 1
            for (int c0 = 0; c0 < TN && c0 < p.t; c0 += 16) {
                float v[16];
                tcgen05_ld16(tmem_row + c0, v);
                if (n < p.n) {
#pragma unroll
                    for (int c = 0; c < 16; ++c) {
                        const int t = c0 + c;
                        if (t < p.t) {
                            if (p.out_f32) {
                                static_cast<float*>(p.y)[t * p.ldy + n] = v[c];
                            } else {
                                static_cast<__nv_bfloat16*>(p.y)[t * p.ldy + n] = __float2bfloat16_rn(v[c]);
                            }
                        }
                    }
                }
            }
        } else if (splits > 1) {
            constexpr int kRow = recv_row(TN);
            const int most = owned_max(splits);
            cluster_wait_all();  // long since complete: every rank arrived in its prologue
            if (have) {
                // all my values for this feature go to the rank that owns it: [me][feature there][token]
                const int owner = feature * splits / kTileM;
                float* row = recv + (rank * most + (feature - first_feature(owner, splits))) * kRow;
                const uint32_t remote_row = cluster_map(row, owner), remote_bar = cluster_map(&recv_bar, owner);
#pragma unroll 1
                for (int c0 = 0; c0 < TN && c0 < p.t; c0 += 16) {
                    float v[16];
                    tcgen05_ld16(tmem_row + c0, v);
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        if (c0 + 4 * q < p.t) {
                            const float4 four = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                            if (owner == rank) {
                                *reinterpret_cast<float4*>(row + c0 + 4 * q) = four;
                            } else {
                                cluster_store4_counted(remote_row + (c0 + 4 * q) * 4, four, remote_bar);
                            }
                        }
                    }
                }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");  // the parts kept here are in place
            // The features this rank owns: parts added in rank order, whoever arrived first.
            const bool arrived = expected == 0 || mbar_wait_cluster(&recv_bar, 0u, &abort_flag);
            if (arrived && have) {
                for (int item = feature; item < my_features * p.t; item += kTileM) {
                    const int mine = item % my_features, t = item / my_features;
                    float sum = 0.0f;
                    for (int s = 0; s < splits; ++s) {
                        sum += recv[(s * most + mine) * kRow + t];
                    }
                    const int at = n0 + my_first + mine;
                    if (at < p.n) {
                        if (p.out_f32) {
                            static_cast<float*>(p.y)[t * p.ldy + at] = sum;
                        } else {
                            static_cast<__nv_bfloat16*>(p.y)[t * p.ldy + at] = __float2bfloat16_rn(sum);
                        }
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
        // Something never came. Linger before the shared memory is given up, so that
        // loads and peers' stores that are still on their way land first.
        if (threadIdx.x == 0) {
            if (p.status != nullptr) {
                atomicOr(p.status, 8);
            }
            for (uint32_t spin = 0; spin < (1u << 16); ++spin) {
                __nanosleep(64);
            }
        }
        __syncthreads();
    }
    // (No meeting of the cluster here: a rank leaves only after everything sent to it
    // has arrived, and what it sent goes to ranks that cannot leave before it arrives.)
    if (warp == 1) {
        tcgen05_fence_after();
        tcgen05_dealloc(tmem_base, kColumns);
    }
}

struct SkinnyPlan {
    int tn, n_tiles, k_blocks, splits, kb_per_split, stages;
};

constexpr int smem_for(int tn, int stages) { return stages * stage_bytes(tn) + recv_bytes_max(tn) + 1024; }

template <int TN>
int configure() {
    static bool configured = false;
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(gemm_skinny_kernel<TN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               smem_for(TN, stages_within(TN, kSmemLarge)));
        if (err != cudaSuccess) {
            return pl_fail(3, "gemm_skinny: cannot configure the kernel: %s", cudaGetErrorString(err));
        }
        configured = true;
    }
    return 0;
}

// How many clusters of `splits` CTAs the device holds at once with the pipeline of the small
// (`deep` false) or the large share of shared memory (0 when it cannot say).
template <int TN>
int resident_clusters(int splits, bool deep) {
    static int known[2][kMaxSplits + 1] = {};
    int& slot = known[deep ? 1 : 0][splits];
    if (slot == 0) {
        cudaLaunchConfig_t config = {};
        config.gridDim = dim3(splits, 1024);
        config.blockDim = dim3(kThreads);
        config.dynamicSmemBytes = smem_for(TN, stages_within(TN, deep ? kSmemLarge : kSmemSmall));
        cudaLaunchAttribute attribute[1];
        attribute[0].id = cudaLaunchAttributeClusterDimension;
        attribute[0].val.clusterDim.x = splits;
        attribute[0].val.clusterDim.y = 1;
        attribute[0].val.clusterDim.z = 1;
        config.attrs = attribute;
        config.numAttrs = 1;
        int clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, gemm_skinny_kernel<TN>, &config) != cudaSuccess) {
            cudaGetLastError();
            clusters = 0;
        }
        slot = clusters > 0 ? clusters : -1;
    }
    return slot > 0 ? slot : 0;
}

// The k range of a tile is cut into parts, at most eight (the portable cluster size) and at
// most one per k block.
template <int TN>
SkinnyPlan make_skinny_plan(int n, int k) {
    SkinnyPlan plan;
    plan.tn = TN;
    plan.n_tiles = (n + kTileM - 1) / kTileM;
    plan.k_blocks = (k + kBlockK - 1) / kBlockK;
    static int sms = 0;
    if (sms == 0) {
        int device = 0;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    }
    // How many parts. Inside a decode step the products stream best with about one and a half
    // CTAs per SM (as many as the gate/up projection of the 8B shape has tiles, 224 on 148 SMs,
    // which runs at the copy bandwidth), on the smaller share of shared memory, so that two of
    // a launch's CTAs, or one and a CTA of the next launch, share an SM: the fewest parts that
    // give between 1.5 and 1.75 CTAs per SM, if there are any with at least six k blocks
    // each. Measured in the step (batch 8, one box): 8B shape q/k/v 2 -> 5 parts, o 4 -> 7, down
    // 4 -> 7: 3.357 -> 3.28 ms (3 or 6 parts for q/k/v, 144 and 288 CTAs, 3.42 - 3.54; 8 for down
    // 3.43); 13B shape 2 - 3 % faster; 1B shape gate/up 1 -> 2 parts 887 -> 858 us. Where no count
    // lands in that band (the 1B shape's other products, 16 and 24 tiles) more parts measured
    // worse (down 6 -> 8: 887 -> 984 us), and the rule is the earlier one: as many parts as still
    // lets every cluster be resident at once with the deep pipeline, which such launches, of
    // fewer CTAs than SMs, then take.
    int splits = 0;
    bool deep = false;
    for (int s = 1; s <= kMaxSplits && s <= plan.k_blocks; ++s) {
        const int total = plan.n_tiles * s;
        if (2 * total >= 3 * sms && 4 * total <= 7 * sms && plan.k_blocks / s >= 6) {
            splits = s;
            break;
        }
    }
    if (splits == 0) {
        splits = 1;
        for (int s = kMaxSplits; s > 1; --s) {
            if (s <= plan.k_blocks && plan.n_tiles <= resident_clusters<TN>(s, true)) {
                splits = s;
                break;
            }
        }
        deep = plan.n_tiles * splits < sms;
    }
    plan.kb_per_split = (plan.k_blocks + splits - 1) / splits;
    plan.splits = (plan.k_blocks + plan.kb_per_split - 1) / plan.kb_per_split;  // no rank without work
    plan.stages = stages_within(TN, deep ? kSmemLarge : kSmemSmall);
    plan.stages = plan.stages > plan.kb_per_split ? plan.kb_per_split : plan.stages;
    plan.stages = plan.stages < 2 ? 2 : plan.stages;
    return plan;
}

template <int TN>
int launch_skinny(const CUtensorMap& map_w, const CUtensorMap& map_x, const SkinnyParams& p, const SkinnyPlan& plan,
                  cudaStream_t stream) {
    const int smem = smem_for(TN, plan.stages);
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(plan.splits, plan.n_tiles);
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attributes[2];
    attributes[0].id = cudaLaunchAttributeClusterDimension;
    attributes[0].val.clusterDim.x = plan.splits;
    attributes[0].val.clusterDim.y = 1;
    attributes[0].val.clusterDim.z = 1;
    attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attributes;
    config.numAttrs = pl_overlap_enabled() ? 2 : 1;
    const cudaError_t err = cudaLaunchKernelEx(&config, gemm_skinny_kernel<TN>, map_w, map_x, p);
    if (err != cudaSuccess) {
        return pl_fail(3, "gemm_skinny: launch failed: %s", cudaGetErrorString(err));
    }
    return 0;
}

}  // namespace

// Into how many parts pl_gemm_bf16_skinny cuts k for these sizes (the cluster size).
PL_API int pl_gemm_bf16_skinny_splits(int t, int n, int k) {
    const int tn = t <= 16 ? 16 : (t <= 32 ? 32 : 64);
    if (tn == 16 ? configure<16>() : (tn == 32 ? configure<32>() : configure<64>())) {
        return -1;
    }
    return (tn == 16 ? make_skinny_plan<16>(n, k) : (tn == 32 ? make_skinny_plan<32>(n, k)
                                                               : make_skinny_plan<64>(n, k))).splits;
}

// The most tokens pl_gemm_bf16_skinny takes.
PL_API int pl_gemm_bf16_skinny_max_tokens() { return 64; }

namespace {

int run_skinny(const void* x, const void* w, void* y, int t, int n, int k, int64_t ldx, int64_t ldw, int64_t ldy,
               int out_f32, int x_mode, int32_t* status, cudaStream_t stream) {
    const int tn = t <= 16 ? 16 : (t <= 32 ? 32 : 64);
    if (const int code = tn == 16 ? configure<16>() : (tn == 32 ? configure<32>() : configure<64>())) {
        return code;
    }
    const SkinnyPlan plan = tn == 16 ? make_skinny_plan<16>(n, k)
                                     : (tn == 32 ? make_skinny_plan<32>(n, k) : make_skinny_plan<64>(n, k));
    PL_REQUIRE(plan.n_tiles <= 65535, "gemm_bf16_skinny: n=%d has too many tiles", n);
    CUtensorMap map_w, map_x;
    if (const int code = make_map(&map_w, w, n, k, ldw, kTileM, kBlockK)) {
        return code;
    }
    if (const int code = make_map(&map_x, x, t, k, ldx, plan.tn, kBlockK)) {
        return code;
    }
    SkinnyParams p;
    p.y = y;
    p.t = t;
    p.n = n;
    p.k = k;
    p.ldy = ldy;
    p.out_f32 = out_f32;
    p.k_blocks = plan.k_blocks;
    p.kb_per_split = plan.kb_per_split;
    p.stages = plan.stages;
    p.status = status;
    p.x_mode = x_mode;
    p.gated = static_cast<const __nv_bfloat16*>(x);
    p.ld_gated = ldx;
    switch (plan.tn) {
        case 16: return launch_skinny<16>(map_w, map_x, p, plan, stream);
        case 32: return launch_skinny<32>(map_w, map_x, p, plan, stream);
        default: return launch_skinny<64>(map_w, map_x, p, plan, stream);
    }
}

}  // namespace

// y[T, N] (bf16, or fp32 when out_f32) = x[T, K] w[N, K]^T with bf16 x and w, for
// T <= 64. k and the leading dimensions of x and w must be multiples of 8 (rows on
// 16-byte boundaries for TMA); N with more than 65535 tiles of 128 is refused.
PL_API int pl_gemm_bf16_skinny(const void* x, const void* w, void* y, int t, int n, int k, int64_t ldx, int64_t ldw,
                               int64_t ldy, int out_f32, int32_t* status, cudaStream_t stream) {
    PL_REQUIRE(t >= 1 && t <= 64 && n >= 1 && k >= 8 && k % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0,
               "gemm_bf16_skinny: unsupported sizes t=%d n=%d k=%d ldx=%lld ldw=%lld (t <= 64; k and the leading "
               "dimensions must be multiples of 8)",
               t, n, k, static_cast<long long>(ldx), static_cast<long long>(ldw));
    PL_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0,
               "gemm_bf16_skinny: operands must be 16-byte aligned");
    PL_REQUIRE(ldy >= n, "gemm_bf16_skinny: ldy=%lld is smaller than n=%d", static_cast<long long>(ldy), n);
    return run_skinny(x, w, y, t, n, k, ldx, ldw, ldy, out_f32, 0, status, stream);
}

// y[T, N] = (silu(g) * u)[T, K] w[N, K]^T for gated = [g | u] of [T, 2K] bf16 (a gate/up
// projection's output, rows ld_gated apart): the gated activation is formed as the product
// reads it (fp32, rounded once to bf16, as the SwiGLU kernel does) and never written. T <= 16.
PL_API int pl_gemm_bf16_skinny_gated_in(const void* gated, const void* w, void* y, int t, int n, int k,
                                        int64_t ld_gated, int64_t ldw, int64_t ldy, int out_f32, int32_t* status,
                                        cudaStream_t stream) {
    PL_REQUIRE(t >= 1 && t <= 16 && n >= 1 && k >= 8 && k % 8 == 0 && ld_gated % 8 == 0 && ldw % 8 == 0 &&
                   ld_gated >= 2 * static_cast<int64_t>(k),
               "gemm_bf16_skinny_gated_in: unsupported sizes t=%d n=%d k=%d ld=%lld ldw=%lld (t <= 16; k and the "
               "leading dimensions multiples of 8; rows of at least 2k)",
               t, n, k, static_cast<long long>(ld_gated), static_cast<long long>(ldw));
    PL_REQUIRE((reinterpret_cast<uintptr_t>(gated) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0,
               "gemm_bf16_skinny_gated_in: operands must be 16-byte aligned");
    PL_REQUIRE(ldy >= n, "gemm_bf16_skinny_gated_in: ldy=%lld is smaller than n=%d", static_cast<long long>(ldy), n);
    return run_skinny(gated, w, y, t, n, k, ld_gated, ldw, ldy, out_f32, 1, status, stream);
}
