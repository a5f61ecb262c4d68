// bfloat16 matrix product on the 5th-generation tensor cores:
//   Y[T, N] = X[T, K] * W[N, K]^T   (W as checkpoints store it, fp32 accumulation)
//
// The weights sit on the MMA's M axis (128 output features per tile) and the tokens
// on its N axis (16 to 256 per tile), so that a decode step with a handful of tokens
// and a prompt of thousands run the same kernel: `tcgen05.mma.cta_group::1.kind::f16`
// with M = 128, N = the token tile, K = 16 per instruction, both operands in shared
// memory (K-major, 128-byte swizzle), the accumulator in tensor memory.
//
// A CTA is persistent and warp-specialised:
//   warp 0    producer: TMA loads (cp.async.bulk.tensor.2d) of a 128 x 64 weight tile
//             and a TN x 64 activation tile per stage, completion on an mbarrier;
//   warp 1    one elected thread issues the MMAs and commits them to the stage's
//             "empty" barrier and, at the end of a run, to the accumulator's "full"
//             barrier; it also owns the tensor-memory allocation;
//   warps 2-5 epilogue: tcgen05.ld of their 32 lanes, conversion, stores.
// Two accumulators in tensor memory let the epilogue of one run overlap the MMAs of
// the next.
//
// Work is cut into units of (tile, 64-wide k block) laid end to end; CTA c takes
// units [c * U, (c + 1) * U). With many tiles U is a multiple of a tile's k blocks
// and every CTA produces whole tiles. With few tiles (a decode step's projections)
// the k range of a tile is spread over several CTAs so that every SM streams
// weights; each then writes an fp32 partial to scratch and counts itself in on the
// tile's counter, and whichever CTA arrives last adds the tile's partials, in the
// order of the k range whoever it is, and writes the output (no CTA waits for
// another; the counter is left at zero for the next launch).
//
// Every wait on an mbarrier is bounded: after the limit the CTA raises bit 8 of the
// status word, stops issuing work, lets what is in flight land, frees its tensor
// memory and returns.
//
// The reference leaves these products to a library (`at::linear`,
// pulsarlm-core/src/engine/model/llama.cpp:67-69, 81, 91, 93).
#include "tcgen05_helpers.cuh"

namespace {

constexpr int kTileM = 128;   // output features per tile (MMA M)
constexpr int kBlockK = 64;   // k elements per stage: 128 bytes, one swizzle row
constexpr int kThreads = 192;

struct GemmParams {
    void* y;            // [T, N] bf16 or fp32
    float* scratch;     // partials [tiles][max_pieces][TN][128]
    int t, n, k;
    int64_t ldy;
    int out_f32;
    int n_tiles;        // tiles along N
    int t_tiles;        // tiles along T
    int k_blocks;       // ceil(K / 64)
    int units_per_cta;  // U
    int total_units;
    int max_pieces;
    int32_t* counters;  // one per tile, zero between launches
    int32_t* status;
};

__host__ __device__ constexpr int stages_for(int tn) {
    const int stage_bytes = kTileM * kBlockK * 2 + tn * kBlockK * 2;
    const int fit = (200 * 1024) / stage_bytes;
    return fit > 8 ? 8 : fit;
}

// ------------------------------------------------------------------ the kernel

template <int TN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    const GemmParams p) {
    constexpr int kStages = stages_for(TN);
    constexpr int kBytesA = kTileM * kBlockK * 2;
    constexpr int kBytesB = TN * kBlockK * 2;
    constexpr int kStageBytes = kBytesA + kBytesB;
    constexpr uint32_t kColumns = 2 * TN < 32 ? 32 : 2 * TN;  // two accumulators
    constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(TN >> 3) << 17) |
        (static_cast<uint32_t>(kTileM >> 4) << 24);

    extern __shared__ unsigned char raw_smem[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) &
                                                            ~static_cast<uintptr_t>(1023));
    __shared__ __align__(8) uint64_t full_bar[kStages];
    __shared__ __align__(8) uint64_t empty_bar[kStages];
    __shared__ __align__(8) uint64_t acc_full[2];
    __shared__ __align__(8) uint64_t acc_empty[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;
    __shared__ int last_piece;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pl_grid_trigger();
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&acc_full[a], 1);
            mbar_init(&acc_empty[a], 4);  // one arrival per epilogue warp
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

    const int unit_begin = blockIdx.x * p.units_per_cta;
    const int unit_end = min(unit_begin + p.units_per_cta, p.total_units);

    // The producer and the issuer run their loops with all lanes of their warp, so that
    // counters, addresses and descriptors stay in uniform registers, and let one elected
    // lane issue.
    if (warp == 0) {
        // ------------------------------------------------ producer
        // The first stages' weight tiles are asked for before the wait on earlier
        // kernels (no kernel writes weights): they stream in under the predecessor's
        // tail. The activation tiles of those stages follow after the wait.
        const int early_end = min(unit_end, unit_begin + kStages);
        for (int unit = unit_begin; unit < early_end; ++unit) {
            const int tile = unit / p.k_blocks, kb = unit % p.k_blocks;
            const int s = unit - unit_begin;
            if (elect_one()) {
                mbar_expect_tx(&full_bar[s], kStageBytes);
                tma_load_2d(tiles + s * kStageBytes, &map_w, kb * kBlockK, (tile % p.n_tiles) * kTileM, &full_bar[s]);
            }
            __syncwarp();
        }
        pl_grid_wait();
        for (int unit = unit_begin; unit < early_end; ++unit) {
            const int tile = unit / p.k_blocks, kb = unit % p.k_blocks;
            const int s = unit - unit_begin;
            if (elect_one()) {
                tma_load_2d(tiles + s * kStageBytes + kBytesA, &map_x, kb * kBlockK, (tile / p.n_tiles) * TN,
                            &full_bar[s]);
            }
            __syncwarp();
        }
        int stage = (early_end - unit_begin) % kStages;
        uint32_t phase = early_end - unit_begin == kStages ? 1u : 0u;
        for (int unit = early_end; unit < unit_end; ++unit) {
            const int tile = unit / p.k_blocks, kb = unit % p.k_blocks;
            const int n0 = (tile % p.n_tiles) * kTileM, t0 = (tile / p.n_tiles) * TN;
            if (!mbar_wait(&empty_bar[stage], phase ^ 1u, &abort_flag)) {
                break;
            }
            unsigned char* a = tiles + stage * kStageBytes;
            if (elect_one()) {
                mbar_expect_tx(&full_bar[stage], kStageBytes);
                tma_load_2d(a, &map_w, kb * kBlockK, n0, &full_bar[stage]);
                tma_load_2d(a + kBytesA, &map_x, kb * kBlockK, t0, &full_bar[stage]);
            }
            __syncwarp();
            if (++stage == kStages) {
                stage = 0;
                phase ^= 1u;
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer
        pl_grid_wait();  // so that the bounded waits below time this kernel's work only
        int stage = 0;
        uint32_t phase = 0;
        int run = 0;  // runs of units within one tile: accumulator run & 1
        int unit = unit_begin;
        bool ok = true;
        while (ok && unit < unit_end) {
            const int tile = unit / p.k_blocks;
            const int run_end = min(unit_end, (tile + 1) * p.k_blocks);
            const int acc = run & 1;
            const uint32_t acc_phase = (run >> 1) & 1u;
            if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1u, &abort_flag)) {
                break;
            }
            tcgen05_fence_after();
            const uint32_t tmem_d = tmem_base + acc * TN;
            for (int u = unit; u < run_end; ++u) {
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
                        // 16 k elements are 32 bytes: 2 in the descriptor's 16-byte units
                        tcgen05_mma(tmem_d, desc_a + 2 * k, desc_b + 2 * k, kIdesc, (u > unit || k > 0) ? 1u : 0u);
                    }
                    tcgen05_commit(&empty_bar[stage]);
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
                tcgen05_commit(&acc_full[acc]);
            }
            __syncwarp();
            unit = run_end;
            ++run;
        }
    } else {
        // ------------------------------------------------ epilogue (warps 2..5)
        const int lane_group = warp & 3;  // the TMEM lanes a warp may read: 32 * (warp % 4)
        const int feature = lane_group * 32 + lane;
        pl_grid_wait();  // before the first store: an earlier kernel may still read what this one overwrites
        int run = 0;
        int unit = unit_begin;
        while (unit < unit_end) {
            const int tile = unit / p.k_blocks;
            const int run_end = min(unit_end, (tile + 1) * p.k_blocks);
            const int acc = run & 1;
            const uint32_t acc_phase = (run >> 1) & 1u;
            const bool whole = unit == tile * p.k_blocks && run_end == (tile + 1) * p.k_blocks;
            if (!mbar_wait(&acc_full[acc], acc_phase, &abort_flag)) {
                break;
            }
            tcgen05_fence_after();
            const int n = (tile % p.n_tiles) * kTileM + feature, t0 = (tile / p.n_tiles) * TN;
            const uint32_t tmem_row = tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16) + acc * TN;
            float* partial = nullptr;
            int pieces = 1;
            if (!whole) {
                const int piece = unit / p.units_per_cta - (tile * p.k_blocks) / p.units_per_cta;
                pieces = ((tile + 1) * p.k_blocks - 1) / p.units_per_cta - (tile * p.k_blocks) / p.units_per_cta + 1;
                partial = p.scratch + (static_cast<int64_t>(tile) * p.max_pieces + piece) * (TN * kTileM) + feature;
            }
#pragma unroll 1
            for (int c0 = 0; c0 < TN; c0 += 16) {
                float v[16];
                tcgen05_ld16(tmem_row + c0, v);
                if (!whole) {
#pragma unroll
                    for (int c = 0; c < 16; ++c) {
                        partial[(c0 + c) * kTileM] = v[c];
                    }
                } else if (n < p.n) {
#pragma unroll
                    for (int c = 0; c < 16; ++c) {
                        const int t = t0 + c0 + c;
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
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&acc_empty[acc]);
            }
            if (!whole) {
                // Count this piece in; the CTA that completes the tile adds the pieces.
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (warp == 2 && lane == 0) {
                    const int before = atomicAdd(&p.counters[tile], 1);
                    last_piece = before == pieces - 1;
                    if (last_piece) {
                        p.counters[tile] = 0;
                    }
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (last_piece) {
                    __threadfence();
                    const float* base = p.scratch + static_cast<int64_t>(tile) * p.max_pieces * (TN * kTileM) + feature;
#pragma unroll 1
                    for (int c0 = 0; c0 < TN && t0 + c0 < p.t; c0 += 16) {
                        float sum[16];
#pragma unroll
                        for (int c = 0; c < 16; ++c) {
                            sum[c] = 0.0f;
                        }
                        for (int piece = 0; piece < pieces; ++piece) {
                            const float* src = base + (static_cast<int64_t>(piece) * TN + c0) * kTileM;
#pragma unroll
                            for (int c = 0; c < 16; ++c) {  // 16 independent loads in flight
                                sum[c] += __ldcg(src + c * kTileM);
                            }
                        }
                        if (n < p.n) {
#pragma unroll
                            for (int c = 0; c < 16; ++c) {
                                const int t = t0 + c0 + c;
                                if (t < p.t) {
                                    if (p.out_f32) {
                                        static_cast<float*>(p.y)[t * p.ldy + n] = sum[c];
                                    } else {
                                        static_cast<__nv_bfloat16*>(p.y)[t * p.ldy + n] = __float2bfloat16_rn(sum[c]);
                                    }
                                }
                            }
                        }
                    }
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");  // last_piece is reused by the next run
            }
            unit = run_end;
            ++run;
        }
    }

    // ---------------------------------------------------- teardown
    __syncwarp();
    tcgen05_fence_before();
    __syncthreads();
    if (abort_flag) {
        // Let loads that were issued land before the shared memory is given up: wait,
        // bounded, on every stage's full barrier in both phases' terms.
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
    if (warp == 1) {
        tcgen05_fence_after();
        tcgen05_dealloc(tmem_base, kColumns);
    }
}

// ------------------------------------------------------------------ host side

int sm_count() {
    static int count = 0;
    if (count == 0) {
        int device = 0;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device);
    }
    return count;
}

int token_tile(int t) {
    return t <= 16 ? 16 : t <= 32 ? 32 : t <= 64 ? 64 : t <= 128 ? 128 : 256;
}

struct Plan {
    int tn, n_tiles, t_tiles, k_blocks, total_units, units_per_cta, grid, max_pieces;
    bool partials;
};

Plan make_plan(int t, int n, int k) {
    Plan plan;
    plan.tn = token_tile(t);
    plan.n_tiles = (n + kTileM - 1) / kTileM;
    plan.t_tiles = (t + plan.tn - 1) / plan.tn;
    plan.k_blocks = (k + kBlockK - 1) / kBlockK;
    const int tiles = plan.n_tiles * plan.t_tiles;
    plan.total_units = tiles * plan.k_blocks;
    const int sms = sm_count();
    if (plan.tn >= 128 && tiles >= sms) {
        // many large tiles: whole tiles per CTA, no partials
        plan.units_per_cta = plan.k_blocks * ((tiles + sms - 1) / sms);
    } else {
        // spread k blocks over all SMs; at least 4 blocks per CTA
        const int per = (plan.total_units + sms - 1) / sms;
        plan.units_per_cta = per < 4 ? 4 : per;
    }
    plan.grid = (plan.total_units + plan.units_per_cta - 1) / plan.units_per_cta;
    plan.partials = plan.units_per_cta % plan.k_blocks != 0;
    plan.max_pieces = plan.partials ? (plan.k_blocks + plan.units_per_cta - 1) / plan.units_per_cta + 1 : 1;
    return plan;
}

template <int TN>
int launch(const CUtensorMap& map_w, const CUtensorMap& map_x, const GemmParams& p, const Plan& plan,
           cudaStream_t stream) {
    constexpr int smem = stages_for(TN) * (kTileM * kBlockK * 2 + TN * kBlockK * 2) + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(gemm_tcgen05_kernel<TN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               smem);
        if (err != cudaSuccess) {
            return pl_fail(3, "gemm_tcgen05: cannot set shared memory size: %s", cudaGetErrorString(err));
        }
        configured = true;
    }
    pl_launch_overlapped(gemm_tcgen05_kernel<TN>, plan.grid, kThreads, smem, stream, map_w, map_x, p);
    PL_CHECK_LAUNCH("gemm_tcgen05");
    return 0;
}

}  // namespace

// 1 when pl_gemm_bf16 takes these sizes: rows of X and W must start on 16 bytes
// (k and the leading dimensions multiples of 8) for TMA.
PL_API int pl_gemm_bf16_supports(int t, int n, int k, int64_t ldx, int64_t ldw) {
    return t >= 1 && n >= 1 && k >= 8 && k % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0;
}

// Floats of scratch a product of these sizes needs (0 when every tile is whole).
PL_API int64_t pl_gemm_bf16_scratch_floats(int t, int n, int k) {
    const Plan plan = make_plan(t, n, k);
    if (!plan.partials) {
        return 0;
    }
    return static_cast<int64_t>(plan.n_tiles) * plan.t_tiles * plan.max_pieces * plan.tn * kTileM;
}

// y[T, N] (bf16, or fp32 when out_f32) = x[T, K] w[N, K]^T with bf16 x and w.
// scratch: pl_gemm_bf16_scratch_floats floats. counters: n_counters int32, all zero,
// at least one per tile when scratch is needed; the kernel leaves them zero. Two
// products that overlap on the GPU must not share counters.
PL_API int pl_gemm_bf16(const void* x, const void* w, void* y, int t, int n, int k, int64_t ldx, int64_t ldw,
                        int64_t ldy, int out_f32, float* scratch, int32_t* counters, int n_counters,
                        int32_t* status, cudaStream_t stream) {
    PL_REQUIRE(pl_gemm_bf16_supports(t, n, k, ldx, ldw),
               "gemm_bf16: unsupported sizes t=%d n=%d k=%d ldx=%lld ldw=%lld (k and the leading dimensions must "
               "be multiples of 8)",
               t, n, k, static_cast<long long>(ldx), static_cast<long long>(ldw));
    PL_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0,
               "gemm_bf16: operands must be 16-byte aligned");
    PL_REQUIRE(ldy >= n, "gemm_bf16: ldy=%lld is smaller than n=%d", static_cast<long long>(ldy), n);
    const Plan plan = make_plan(t, n, k);
    PL_REQUIRE(!plan.partials || (scratch != nullptr && counters != nullptr),
               "gemm_bf16: these sizes need scratch memory and tile counters");
    PL_REQUIRE(!plan.partials || plan.n_tiles * plan.t_tiles <= n_counters,
               "gemm_bf16: %d tiles need as many counters, %d were given", plan.n_tiles * plan.t_tiles, n_counters);
    CUtensorMap map_w, map_x;
    if (const int code = make_map(&map_w, w, n, k, ldw, kTileM, kBlockK)) {
        return code;
    }
    if (const int code = make_map(&map_x, x, t, k, ldx, plan.tn, kBlockK)) {
        return code;
    }
    GemmParams p;
    p.y = y;
    p.scratch = scratch;
    p.t = t;
    p.n = n;
    p.k = k;
    p.ldy = ldy;
    p.out_f32 = out_f32;
    p.n_tiles = plan.n_tiles;
    p.t_tiles = plan.t_tiles;
    p.k_blocks = plan.k_blocks;
    p.units_per_cta = plan.units_per_cta;
    p.total_units = plan.total_units;
    p.max_pieces = plan.max_pieces;
    p.counters = counters;
    p.status = status;
    switch (plan.tn) {
        case 16: return launch<16>(map_w, map_x, p, plan, stream);
        case 32: return launch<32>(map_w, map_x, p, plan, stream);
        case 64: return launch<64>(map_w, map_x, p, plan, stream);
        case 128: return launch<128>(map_w, map_x, p, plan, stream);
        default: return launch<256>(map_w, map_x, p, plan, stream);
    }
}
