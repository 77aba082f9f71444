// tcgen05 (5th-generation tensor core) building blocks shared by the tensor-core kernels: the
// 128-byte-swizzled K-major operand tile, TF32 splitting, shared-memory and instruction descriptors,
// MMA issue, commit and the tcgen05 fences.
#pragma once
#include "oeq_common.cuh"

namespace oeq {

// byte offset of element (row, col) inside a [rows x 32 tf32] K-major tile with the 128-byte swizzle
__host__ __device__ __forceinline__ int tc_swizzle(int row, int col) {
    return (row >> 3) * 1024 + (row & 7) * 128 + ((((col >> 2) ^ (row & 7)) & 7) << 4) + ((col & 3) << 2);
}

__device__ __forceinline__ float tf32_round(float x) {
    unsigned r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}
// The same rounding (to nearest, ties away from zero, 10 mantissa bits kept) with two integer
// instructions: conversion instructions issue at a fraction of the integer rate, and the operand tiles
// are rebuilt for every edge / batch tile.  Finite inputs only.
__device__ __forceinline__ float tf32_hi(float x) {
    return __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xffffe000u);
}

// shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ unsigned long long tc_smem_desc(unsigned smem_addr) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_addr >> 4) & 0x3fff);        // start address
    d |= (unsigned long long)1 << 16;                             // leading byte offset (16 B units)
    d |= (unsigned long long)(1024 >> 4) << 32;                   // stride byte offset
    d |= (unsigned long long)1 << 46;                             // descriptor version
    d |= (unsigned long long)2 << 61;                             // SWIZZLE_128B
    return d;
}
// instruction descriptor: TF32 x TF32 -> F32, both operands K-major, M = 128, N = n
__host__ __device__ constexpr unsigned tc_instr_desc(int n) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((unsigned)(n >> 3) << 17) | ((unsigned)(128 >> 4) << 24);
}
__device__ __forceinline__ void tc_mma(unsigned tmem_d, unsigned long long a, unsigned long long b, unsigned idesc,
                                       unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void tc_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
// 16 consecutive accumulator columns of the calling warp's 32 TMEM lanes (wait with tcgen05.wait::ld)
__device__ __forceinline__ void tc_load16(unsigned taddr, unsigned* v) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr));
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

}  // namespace oeq
