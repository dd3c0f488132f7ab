// The per-head arithmetic of fused_split_qknorm_kvstore.wgsl:139-166 / 195-218 for one warp: RMSNorm with (1 + w)
// bf16 weights, then partial (m)RoPE, on a head vector held in shared memory.  Shared by the stand-alone append
// kernel and by the projection kernel that appends in its epilogue.
#pragma once
#include <math.h>

#include "common.cuh"

namespace shady {

struct RopeSpec {
    uint32_t rd, s1, s2, interleaved;   // PARTIAL_DIM, MROPE_S1_LIMIT, MROPE_S2_LIMIT, MROPE_INTERLEAVED (model.rs:32-54)
    float eps;
};

// vals[hd] in shared memory, written by this warp (the caller has synchronised the warp).  w: bf16 bits of the norm
// weights of this head kind (q or k), or NULL.  inv_freq[rd/2] as the host computed it (1/powf(theta, 2i/rd)).
__device__ __forceinline__ void warp_norm_rope(float *vals, uint32_t lane, uint32_t hd, const uint16_t *w, const RopeSpec &r,
                                               const float *inv_freq, uint32_t p_t, uint32_t p_h, uint32_t p_w) {
    if (w) {   // wgsl:150-160 / :205-212
        float ssq = 0.f;
        for (uint32_t d = lane; d < hd; d += 32) ssq += vals[d] * vals[d];
        ssq = warp_sum(ssq);
        const float rms = 1.0f / sqrtf(ssq / (float)hd + r.eps);
        for (uint32_t d = lane; d < hd; d += 32) {
            const float wf = __uint_as_float(((uint32_t)w[d]) << 16);
            vals[d] = vals[d] * rms * (1.0f + wf);
        }
    }
    __syncwarp();
    // (m)RoPE on the first rd dims (wgsl:56-104); cos/sin by the accurate sincosf: the shader takes them of up to
    // 131071 radians in f32
    const uint32_t half = r.rd / 2;
    for (uint32_t i = lane; i < half; i += 32) {
        uint32_t pos = p_t;
        if ((i % 3u) == 1u && i < r.s1) pos = p_h;
        else if ((i % 3u) == 2u && i < r.s2) pos = p_w;
        const float angle = (float)pos * inv_freq[i];
        float sn, cs;
        sincosf(angle, &sn, &cs);
        const uint32_t ia = r.interleaved ? 2 * i : i;
        const uint32_t ib = r.interleaved ? 2 * i + 1 : i + half;
        const float x = vals[ia], y = vals[ib];
        vals[ia] = x * cs - y * sn;
        vals[ib] = y * cs + x * sn;
    }
    __syncwarp();
}

}  // namespace shady
