// mma.sync pieces shared by the few-token kernels (rns_small_sm100.cu, rns_stream_sm100.cu).
#pragma once

#include <cstdint>

namespace rns {

__device__ __forceinline__ void mma_s8(int (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// Shared memory: residues of the CTA's 16 tokens, per channel and K step of 32 bytes, as
// [half of the K step][token row][16 bytes] (512 bytes): a lane's fragment words are then
// 32 consecutive words across the warp (no bank conflicts).
__device__ __forceinline__ int small_a_offset(int channel, int kstep, int ksteps, int row, int byte_in_step) {
    const int half = byte_in_step >> 4;
    return ((channel * ksteps + kstep) * 2 + half) * 256 + row * 16 + (byte_in_step & 15);
}

}  // namespace rns
