// True 32-bit matrix product for the float32 engine: C[M, N] = A[M, K] * W[N, K]^T.
//
// CUDA-core FMAs only: no tensor cores, no TF32. Each output element is one chain
// of fmaf over k = 0 .. K-1 in ascending order, whatever M is, so a token's row
// does not depend on what else is in the batch or on how a prompt was cut.
#include "common.cuh"

namespace {

constexpr int kTileM = 64;
constexpr int kTileN = 64;
constexpr int kTileK = 16;

// 256 threads; thread (ty, tx) of a 16x16 grid owns a 4x4 block of the 64x64 tile.
// Optional `accumulate`: C += product (used to add into the fp32 residual stream).
__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ a, const float* __restrict__ w, float* __restrict__ c, int m, int n,
                int k, int lda, int ldw, int ldc, int accumulate) {
    __shared__ float as[kTileK][kTileM + 1];
    __shared__ float ws[kTileK][kTileN + 1];
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const int m0 = blockIdx.y * kTileM, n0 = blockIdx.x * kTileN;

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            acc[i][j] = 0.0f;
        }
    }

    for (int k0 = 0; k0 < k; k0 += kTileK) {
        // 64 rows x 16 k of each operand: 1024 elements, 4 per thread; consecutive
        // threads read consecutive k of one row.
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = threadIdx.x + i * 256;
            const int row = e / kTileK, kk = e % kTileK;
            const int gk = k0 + kk;
            as[kk][row] = (m0 + row < m && gk < k) ? a[static_cast<int64_t>(m0 + row) * lda + gk] : 0.0f;
            ws[kk][row] = (n0 + row < n && gk < k) ? w[static_cast<int64_t>(n0 + row) * ldw + gk] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kTileK; ++kk) {
            float av[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                av[i] = as[kk][ty * 4 + i];
                wv[i] = ws[kk][tx * 4 + i];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
                }
            }
        }
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int row = m0 + ty * 4 + i;
        if (row >= m) {
            continue;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int col = n0 + tx * 4 + j;
            if (col < n) {
                float* dst = c + static_cast<int64_t>(row) * ldc + col;
                *dst = accumulate ? *dst + acc[i][j] : acc[i][j];
            }
        }
    }
}

}  // namespace

PL_API int pl_gemm_f32(const float* a, const float* w, float* c, int m, int n, int k, int lda, int ldw, int ldc,
                       int accumulate, cudaStream_t stream) {
    PL_REQUIRE(m >= 0 && n > 0 && k > 0, "gemm_f32: bad sizes m=%d n=%d k=%d", m, n, k);
    PL_REQUIRE(lda >= k && ldw >= k && ldc >= n, "gemm_f32: leading dimensions too small (lda=%d ldw=%d ldc=%d)", lda,
               ldw, ldc);
    if (m == 0) {
        return 0;
    }
    const dim3 grid((n + kTileN - 1) / kTileN, (m + kTileM - 1) / kTileM);
    PL_REQUIRE(grid.y <= 65535, "gemm_f32: m=%d is too large for one launch", m);
    gemm_f32_kernel<<<grid, 256, 0, stream>>>(a, w, c, m, n, k, lda, ldw, ldc, accumulate);
    PL_CHECK_LAUNCH("gemm_f32");
    return 0;
}
