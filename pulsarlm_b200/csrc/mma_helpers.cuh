// Warp-level building blocks of the bfloat16 attention kernels: 16-byte async
// copies into shared memory, ldmatrix loads, the m16n8k16 bf16 MMA with fp32
// accumulators, and the XOR swizzle that keeps ldmatrix free of bank conflicts
// (16-byte chunk c of row r is stored at chunk c ^ (r & 7)).
#pragma once

#include "common.cuh"

__device__ __forceinline__ void cp_async_16(void* smem, const void* global) {
    const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(global));
}
// Copies 16 bytes when `valid`, else fills the 16 bytes with zeros (nothing is read).
__device__ __forceinline__ void cp_async_16_or_zero(void* smem, const void* global, bool valid) {
    const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(global), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
    const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
    const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// 2^x by the hardware's approximation (2 ulp; -inf gives 0). The probabilities it
// makes are rounded to bfloat16 right after, so the fp32 engine never uses it.
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Bytes of a shared-memory row that holds `head_dim` bfloat16 values: a multiple of 128,
// so that `swizzled` never leaves the row.
__host__ __device__ constexpr int padded_row_bytes(int head_dim) { return (head_dim + 63) / 64 * 128; }

// Byte offset of 16-byte chunk `chunk` of row `row` in a swizzled tile whose rows
// are `row_bytes` long (a multiple of 128).
__device__ __forceinline__ int swizzled(int row, int chunk, int row_bytes) {
    return row * row_bytes + ((chunk ^ (row & 7)) * 16);
}
