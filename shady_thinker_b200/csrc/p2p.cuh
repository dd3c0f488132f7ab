// Exchange-buffer layouts and system-scope flag accesses shared by the cross-GPU kernels.
#pragma once
#include "common.cuh"

namespace shady {

constexpr uint32_t kP2PMaxWorld = 16;
constexpr uint32_t kP2PChunk = 64;            // head dims per CTA of the fused merge + exchange kernel
constexpr uint32_t kP2PSlotFloats = kP2PChunk + 2;   // 64 values, the head's log-sum-exp, one unused

// Whole-record layout (p2p_combine_kernel): flags [2 parities][world][nh] u32 (padded to 256 B), then records
// [2][world][nh][hd+2] f32.
__host__ __device__ inline unsigned long long p2p_flags_bytes(uint32_t world, uint32_t nh) {
    return ((unsigned long long)2 * world * nh * sizeof(uint32_t) + 255ull) / 256ull * 256ull;
}
// Chunked layout (shard_merge_p2p_kernel): flags [2][world][nh][chunks] u32 (padded to 256 B), then slots
// [2][world][nh][chunks][66] f32; chunks = ceil(hd / 64).  One buffer is sized for either layout; a buffer is used
// with one of the two kernels only.
__host__ __device__ inline uint32_t p2p_chunks(uint32_t hd) { return (hd + kP2PChunk - 1) / kP2PChunk; }
__host__ __device__ inline unsigned long long p2p_chunk_flags_bytes(uint32_t world, uint32_t nh, uint32_t hd) {
    return ((unsigned long long)2 * world * nh * p2p_chunks(hd) * sizeof(uint32_t) + 255ull) / 256ull * 256ull;
}

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

}  // namespace shady
