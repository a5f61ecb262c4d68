// bfloat16 matrix product for prompts on pairs of SMs:
//   Y[T, N] = X[T, K] * W[N, K]^T,  fp32 accumulation, T in the hundreds and up.
//
// Two CTAs of a cluster work on one 256-feature x 256-token tile with
// `tcgen05.mma.cta_group::2` (M = 256 over the pair, N = 256, K = 16 per instruction).
// The weights sit on the MMA's M axis and the tokens on its N axis, as in the other
// products of this library. Each CTA loads its own 128 features of W and its own 128
// of the tile's 256 tokens of X per 64-deep k block (32 KB where a lone CTA with a
// 128 x 256 tile of its own would need 48 KB for the same number of MMA cycles: one SM
// takes in about 64 bytes a clock, which held a single-CTA kernel of that tile to 0.6 -
// 0.7 of the GEMM peak); the instruction reads both CTAs' shared memory and writes each CTA's 128 rows of the accumulator into that
// CTA's tensor memory.
//
// Roles per CTA (192 threads): warp 0 loads with TMA (`.cta_group::2` loads, whose
// bytes are counted on the barrier of the pair's first CTA); warp 1 of the first CTA
// issues the MMAs for the pair and commits them to both CTAs' barriers
// (`tcgen05.commit ... multicast::cluster`), and owns (in both CTAs) the tensor
// memory allocation; warps 2-5 read their CTA's accumulator rows and store them.
// Two accumulators let the epilogue of one tile overlap the MMAs of the next; the
// second CTA's epilogue releases an accumulator by arriving on the first CTA's barrier.
// A pair is persistent and takes every P-th whole tile (P pairs), token tiles fastest:
// the P tiles in work at one time are then neighbours that share a few weight tiles, so
// each weight tile comes from HBM once and is served to the other pairs from L2 (with a
// contiguous run of tiles per pair the pairs' weight tiles together overflow the L2 and
// every token tile re-reads its weights from HBM: 2.07 GB instead of 0.25 GB for the
// 2048 x 28672 x 4096 product).
//
// Gated mode: W holds two stacked matrices, gate over up ([2N, K]), and the kernel
// writes silu(gate x) * (up x) ([T, N]). A CTA's 128 rows are then 64 gate rows over
// the 64 up rows of the same features (two TMA boxes per stage); in the epilogue the
// warps that hold the up rows pass them through shared memory to the warps that hold
// the gate rows, which round both to bfloat16 (as a product that stored them would)
// and apply the activation.
//
// Every wait on an mbarrier is bounded: after the limit the CTA raises bit 8 of the
// status word, stops issuing work, lets what is in flight land, meets its partner,
// frees its tensor memory and returns.
//
// The reference leaves these products to a library (`at::linear`,
// pulsarlm-core/src/engine/model/llama.cpp:67-69, 81, 91, 93).
#include "tcgen05_helpers.cuh"

namespace {

constexpr int kTileM = 128;    // features per CTA, 256 per pair
constexpr int kPairN = 256;    // tokens per tile, 128 loaded by each CTA
constexpr int kBlockK = 64;
constexpr int kThreads = 192;
constexpr int kStages = 6;
constexpr int kBytesA = kTileM * kBlockK * 2;
constexpr int kBytesB = (kPairN / 2) * kBlockK * 2;
constexpr int kStageBytes = kBytesA + kBytesB;  // per CTA

struct PairParams {
    void* y;  // [T, N] bf16 or fp32
    int t, n, k;  // n: output features (gated: W has 2n rows)
    int64_t ldy;
    int out_f32;
    int n_tiles;  // tiles along N (256 features each)
    int t_tiles;  // tiles along T (256 tokens each)
    int k_blocks;
    int total_tiles;
    int32_t* status;
};

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    return rank;
}
__device__ __forceinline__ void tcgen05_alloc_pair(uint32_t* slot, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)),
                 "r"(columns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_dealloc_pair(uint32_t address, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns) : "memory");
}
// A tile load whose bytes are counted on the barrier at the same address in the pair's
// first CTA (both CTAs of the pair issue such loads for a stage).
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], "
        "[%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(cluster_map(bar, 0)), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tcgen05_mma_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                 uint32_t accumulate) {
    const uint32_t zero = 0;  // no output lanes switched off
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(zero)
        : "memory");
}
// One arrival, once the MMAs issued so far have completed, on the barrier at this
// address in both CTAs of the pair.
__device__ __forceinline__ void tcgen05_commit_pair(uint64_t* bar) {
    const uint16_t both = 3;
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(smem_u32(bar)), "h"(both)
        : "memory");
}
// One arrival on the barrier at this address in the pair's first CTA.
__device__ __forceinline__ void arrive_on_first(uint64_t* bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_map(bar, 0))
                 : "memory");
}

constexpr int kGateRow = 17;  // 16 token columns handed over per thread and chunk, padded against bank conflicts
constexpr int kGateBytes = 2 * 2 * (kTileM / 2) * kGateRow * 4;  // two buffers of [gate side, up side][64][17] floats

template <bool GATED>
__global__ void __launch_bounds__(kThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                 const PairParams p) {
    constexpr uint32_t kColumns = 2 * kPairN;  // two accumulators
    constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(kPairN >> 3) << 17) |
        (static_cast<uint32_t>((2 * kTileM) >> 4) << 24);

    extern __shared__ unsigned char raw_smem[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) &
                                                            ~static_cast<uintptr_t>(1023));
    float* handover = reinterpret_cast<float*>(tiles + kStages * kStageBytes);  // gated: [2][2][64][17]
    constexpr int kPer = GATED ? kTileM / 2 : kTileM;      // output features per CTA and tile
    __shared__ __align__(8) uint64_t full_bar[kStages];   // waited on in the first CTA only
    __shared__ __align__(8) uint64_t empty_bar[kStages];
    __shared__ __align__(8) uint64_t acc_full[2];
    __shared__ __align__(8) uint64_t acc_empty[2];         // waited on in the first CTA only
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = static_cast<int>(cluster_rank());
    const int pair = blockIdx.x >> 1;
    pl_grid_trigger();
    if (threadIdx.x == 0) {
        tensormap_prefetch(&map_w);
        tensormap_prefetch(&map_x);
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&acc_full[a], 1);
            mbar_init(&acc_empty[a], 8);  // the epilogue warps of both CTAs
        }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        tcgen05_alloc_pair(&tmem_base_slot, kColumns);
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = __shfl_sync(0xffffffffu, tmem_base_slot, 0);
    cluster_arrive_all();  // both CTAs' barriers exist before either signals the other's
    cluster_wait_all();
    pl_grid_wait();

    const int tile_begin = pair, tile_end = p.total_tiles, tile_step = gridDim.x >> 1;

    if (warp == 0) {
        // ------------------------------------------------ producer (both CTAs)
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int tile = tile_begin; ok && tile < tile_end; tile += tile_step) {
            const int n0 = (tile / p.t_tiles) * (2 * kPer) + rank * kPer;
            const int t0 = (tile % p.t_tiles) * kPairN + rank * (kPairN / 2);
            for (int kb = 0; kb < p.k_blocks; ++kb) {
                if (!mbar_wait(&empty_bar[stage], phase ^ 1u, &abort_flag)) {
                    ok = false;
                    break;
                }
                unsigned char* a = tiles + stage * kStageBytes;
                if (elect_one()) {
                    if (rank == 0) {
                        mbar_expect_tx(&full_bar[stage], 2 * kStageBytes);  // both CTAs' loads of this stage
                    }
                    tma_load_2d_pair(a, &map_w, kb * kBlockK, n0, &full_bar[stage]);
                    if (GATED) {  // the up rows of the same features under the gate rows
                        tma_load_2d_pair(a + kBytesA / 2, &map_w, kb * kBlockK, p.n + n0, &full_bar[stage]);
                    }
                    tma_load_2d_pair(a + kBytesA, &map_x, kb * kBlockK, t0, &full_bar[stage]);
                }
                __syncwarp();
                if (++stage == kStages) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
        }
    } else if (warp == 1 && rank == 0) {
        // ------------------------------------------------ MMA issuer (the pair's first CTA)
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int tile = tile_begin; ok && tile < tile_end; tile += tile_step) {
            const int run = (tile - tile_begin) / tile_step;
            const int acc = run & 1;
            if (!mbar_wait_cluster(&acc_empty[acc], ((run >> 1) & 1u) ^ 1u, &abort_flag)) {
                break;
            }
            tcgen05_fence_after();
            const uint32_t tmem_d = tmem_base + acc * kPairN;
            for (int kb = 0; kb < p.k_blocks; ++kb) {
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
                        tcgen05_mma_pair(tmem_d, desc_a + 2 * k, desc_b + 2 * k, kIdesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    tcgen05_commit_pair(&empty_bar[stage]);  // frees the stage in both CTAs
                }
                __syncwarp();
                if (++stage == kStages) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
            if (!ok) {
                break;
            }
            if (elect_one()) {
                tcgen05_commit_pair(&acc_full[acc]);  // both CTAs' epilogues may read
            }
            __syncwarp();
        }
    } else if (warp >= 2) {
        // ------------------------------------------------ epilogue (warps 2..5, both CTAs)
        const int lane_group = warp & 3;  // the tensor-memory lanes a warp may read: 32 * (warp % 4)
        const int feature = lane_group * 32 + lane;
        for (int tile = tile_begin; tile < tile_end; tile += tile_step) {
            const int run = (tile - tile_begin) / tile_step;
            const int acc = run & 1;
            if (!mbar_wait(&acc_full[acc], (run >> 1) & 1u, &abort_flag)) {
                break;
            }
            tcgen05_fence_after();
            const int n = (tile / p.t_tiles) * (2 * kPer) + rank * kPer + (GATED ? feature % kPer : feature);
            const int t0 = (tile % p.t_tiles) * kPairN;
            const uint32_t tmem_row = tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16) + acc * kPairN;
#pragma unroll 1
            for (int c0 = 0; c0 < kPairN && t0 + c0 < p.t; c0 += 32) {
                uint32_t v[32];
                tcgen05_ld32_nowait(tmem_row + c0, v);
                tcgen05_wait_ld();
                if (GATED) {
                    // Lanes 0..63 hold gate rows, lanes 64..127 the up rows of the same features.
                    // Each side hands the other half of its chunk: the gate threads then have
                    // both values for the chunk's first 16 tokens, the up threads for the last 16.
                    const bool is_up = feature >= kPer;
                    const int mine = is_up ? 16 : 0;  // the columns this thread finishes
                    float* buffer = handover + ((c0 >> 5) & 1) * (2 * kPer * kGateRow) +
                        (is_up ? 0 : kPer * kGateRow) + (feature % kPer) * kGateRow;
#pragma unroll
                    for (int c = 0; c < 16; ++c) {
                        buffer[c] = __uint_as_float(v[(16 - mine) + c]);  // the half the partner finishes
                    }
                    asm volatile("bar.sync 1, 128;" ::: "memory");  // (two buffers: one barrier per chunk is enough)
                    if (n < p.n) {
                        // (loads, arithmetic and stores in separate sweeps: a store between two
                        // loads would keep the compiler from overlapping the elements' latencies)
                        const float* theirs = handover + ((c0 >> 5) & 1) * (2 * kPer * kGateRow) +
                            (is_up ? kPer * kGateRow : 0) + (feature % kPer) * kGateRow;
                        float other[16], act[16];
#pragma unroll
                        for (int c = 0; c < 16; ++c) {
                            other[c] = theirs[c];
                        }
#pragma unroll
                        for (int c = 0; c < 16; ++c) {
                            const float own = __uint_as_float(v[mine + c]);
                            // both products rounded as a product that stored them would round them
                            const float g = __bfloat162float(__float2bfloat16_rn(is_up ? other[c] : own));
                            const float u = __bfloat162float(__float2bfloat16_rn(is_up ? own : other[c]));
                            act[c] = __fdividef(g, 1.0f + __expf(-g)) * u;
                        }
#pragma unroll
                        for (int c = 0; c < 16; ++c) {
                            const int t = t0 + c0 + mine + c;
                            if (t < p.t) {
                                if (p.out_f32) {
                                    static_cast<float*>(p.y)[t * p.ldy + n] = act[c];
                                } else {
                                    static_cast<__nv_bfloat16*>(p.y)[t * p.ldy + n] = __float2bfloat16_rn(act[c]);
                                }
                            }
                        }
                    }
                } else if (n < p.n) {
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        const int t = t0 + c0 + c;
                        if (t < p.t) {
                            if (p.out_f32) {
                                static_cast<float*>(p.y)[t * p.ldy + n] = __uint_as_float(v[c]);
                            } else {
                                static_cast<__nv_bfloat16*>(p.y)[t * p.ldy + n] =
                                    __float2bfloat16_rn(__uint_as_float(v[c]));
                            }
                        }
                    }
                }
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) {
                arrive_on_first(&acc_empty[acc]);
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
                __nanosleep(64);  // loads in flight land meanwhile
            }
        }
        __syncthreads();
    }
    // Neither CTA leaves while its partner may still read its shared memory (MMAs) or
    // arrive on its barriers.
    cluster_arrive_all();
    cluster_wait_all();
    if (warp == 1) {
        tcgen05_fence_after();
        tcgen05_dealloc_pair(tmem_base, kColumns);
    }
}

int pair_count() {
    static int pairs = 0;
    if (pairs == 0) {
        int device = 0, sms = 0;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        pairs = sms / 2;
    }
    return pairs;
}

}  // namespace

// 1 when pl_gemm_bf16_pair takes these sizes (rows of X and W on 16-byte boundaries).
PL_API int pl_gemm_bf16_pair_supports(int t, int n, int k, int64_t ldx, int64_t ldw) {
    return t >= 1 && n >= 1 && k >= 8 && k % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0;
}

namespace {

template <bool GATED>
int launch_pair(const CUtensorMap& map_w, const CUtensorMap& map_x, const PairParams& p, int used_pairs,
                cudaStream_t stream) {
    constexpr int smem = kStages * kStageBytes + (GATED ? kGateBytes : 0) + 1024;
    static bool configured = false;
    if (!configured) {
        const cudaError_t err = cudaFuncSetAttribute(gemm_pair_kernel<GATED>,
                                                     cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (err != cudaSuccess) {
            return pl_fail(3, "gemm_bf16_pair: cannot set shared memory size: %s", cudaGetErrorString(err));
        }
        configured = true;
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(2 * used_pairs);
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attributes[2];
    attributes[0].id = cudaLaunchAttributeClusterDimension;
    attributes[0].val.clusterDim.x = 2;
    attributes[0].val.clusterDim.y = 1;
    attributes[0].val.clusterDim.z = 1;
    attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attributes;
    config.numAttrs = pl_overlap_enabled() ? 2 : 1;
    const cudaError_t err = cudaLaunchKernelEx(&config, gemm_pair_kernel<GATED>, map_w, map_x, p);
    if (err != cudaSuccess) {
        return pl_fail(3, "gemm_bf16_pair: launch failed: %s", cudaGetErrorString(err));
    }
    return 0;
}

}  // namespace

// y[T, N] (bf16, or fp32 when out_f32) = x[T, K] w[N, K]^T with bf16 x and w, on
// pairs of SMs; meant for hundreds of tokens and more (a tile is 256 x 256). With
// `gated`, w is [2N, K] (a gate matrix over an up matrix) and
// y = silu(x gate^T) * (x up^T), both products rounded to bfloat16 first (a tile is
// then 128 output features x 256 tokens).
PL_API int pl_gemm_bf16_pair(const void* x, const void* w, void* y, int t, int n, int k, int64_t ldx, int64_t ldw,
                             int64_t ldy, int out_f32, int gated, int32_t* status, cudaStream_t stream) {
    PL_REQUIRE(pl_gemm_bf16_pair_supports(t, n, k, ldx, ldw),
               "gemm_bf16_pair: unsupported sizes t=%d n=%d k=%d ldx=%lld ldw=%lld (k and the leading dimensions "
               "must be multiples of 8)",
               t, n, k, static_cast<long long>(ldx), static_cast<long long>(ldw));
    PL_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0,
               "gemm_bf16_pair: operands must be 16-byte aligned");
    PL_REQUIRE(ldy >= n, "gemm_bf16_pair: ldy=%lld is smaller than n=%d", static_cast<long long>(ldy), n);
    const int per_pair = gated ? kTileM : 2 * kTileM;  // output features of a tile
    CUtensorMap map_w, map_x;
    if (const int code = make_map(&map_w, w, gated ? 2 * static_cast<int64_t>(n) : n, k, ldw,
                                  gated ? kTileM / 2 : kTileM, kBlockK)) {
        return code;
    }
    if (const int code = make_map(&map_x, x, t, k, ldx, kPairN / 2, kBlockK)) {
        return code;
    }
    PairParams p;
    p.y = y;
    p.t = t;
    p.n = n;
    p.k = k;
    p.ldy = ldy;
    p.out_f32 = out_f32;
    p.n_tiles = (n + per_pair - 1) / per_pair;
    p.t_tiles = (t + kPairN - 1) / kPairN;
    p.k_blocks = (k + kBlockK - 1) / kBlockK;
    p.total_tiles = p.n_tiles * p.t_tiles;
    const int used_pairs = p.total_tiles < pair_count() ? p.total_tiles : pair_count();
    p.status = status;
    return gated ? launch_pair<true>(map_w, map_x, p, used_pairs, stream)
                 : launch_pair<false>(map_w, map_x, p, used_pairs, stream);
}
