// Cross-GPU merge of a row-sharded decode over NVLink peer memory — exchange and merge in ONE kernel.
//
// Each rank has decoded its rows of the sequence(s) into records [nh][hd+2] (output, log-sum-exp, unused;
// the layout of gqa_attention_head.wgsl:112-123).  Instead of an NCCL all-gather followed by a merge kernel,
// one CTA per query head
//   1. stores this rank's record of its head into every peer's receive buffer with plain peer stores
//      (no TMA, no multicast), fences at system scope and raises one flag per (rank, head) on every peer;
//   2. waits — bounded — until the flags of all ranks for its head have arrived in its own buffer;
//   3. merges the `world` records with the gqa_reduce.wgsl:33-64 math and writes the final rows.
// Receive buffers and flags are double-buffered by the parity of the call's epoch: a rank can be at most one
// call ahead of its slowest peer (it needs that peer's flags of the current call to finish), so the buffer it
// overwrites is never the one a peer is still merging.  Every wait has an iteration limit (shady_ctx_set_wait_limits);
// on expiry the kernel records a code in the context's status words and returns, and the next shady_synchronize
// reports SHADY_ERR_TIMEOUT.
#include "p2p.cuh"

namespace shady {

struct P2PArgs {
    char *const *peer_bases;   // device array [world]: every rank's shared buffer as mapped into this process
    const float *rec;          // this rank's records [nh][hd+2]
    void *out;
    const float *gate;
    StatusRef status;
    uint32_t wait_peer;        // poll limit of the flag wait
    uint32_t rank, world, nh, hd, epoch, out_dtype;
    unsigned long long flags_bytes;   // size of the flag region at the head of a shared buffer
};

unsigned long long p2p_buffer_bytes(uint32_t world, uint32_t nh, uint32_t hd) {
    const unsigned long long whole = p2p_flags_bytes(world, nh) + (unsigned long long)2 * world * nh * (hd + 2) * sizeof(float);
    const unsigned long long chunked = p2p_chunk_flags_bytes(world, nh, hd) +
                                       (unsigned long long)2 * world * nh * p2p_chunks(hd) * kP2PSlotFloats * sizeof(float);
    return whole > chunked ? whole : chunked;
}

__global__ void __launch_bounds__(128) p2p_combine_kernel(const P2PArgs a) {
    const uint32_t h = blockIdx.x, tid = threadIdx.x;
    const uint32_t rs = a.hd + 2, par = a.epoch & 1u;
    __shared__ float sm_lse[kP2PMaxWorld];
    __shared__ int sm_fail;
    if (tid == 0) sm_fail = 0;
    // ---- 1. my record of head h -> every rank's receive slot [par][my rank][h] ----
    const float *src = a.rec + (size_t)h * rs;
    for (uint32_t r = 0; r < a.world; ++r) {
        float *dst = reinterpret_cast<float *>(a.peer_bases[r] + a.flags_bytes) +
                     (((size_t)par * a.world + a.rank) * a.nh + h) * rs;
        for (uint32_t d = tid; d < rs; d += blockDim.x) dst[d] = src[d];
    }
    __threadfence_system();
    __syncthreads();
    if (tid < a.world) {
        uint32_t *flag = reinterpret_cast<uint32_t *>(a.peer_bases[tid]) + ((size_t)par * a.world + a.rank) * a.nh + h;
        st_release_sys(flag, a.epoch);
    }
    // ---- 2. bounded wait for every rank's flag of this head in my own buffer ----
    if (tid < a.world) {
        const uint32_t *flag = reinterpret_cast<const uint32_t *>(a.peer_bases[a.rank]) + ((size_t)par * a.world + tid) * a.nh + h;
        bool ok = false;
        for (uint32_t i = 0; i < a.wait_peer; ++i) {
            if ((int32_t)(ld_acquire_sys(flag) - a.epoch) >= 0) { ok = true; break; }
            if ((i & 4095u) == 4095u && gave_up(a.status)) break;   // somebody already gave up
        }
        if (!ok) {
            sm_fail = 1;
            report_timeout(a.status, 100 + (int)tid);
        }
    }
    __syncthreads();
    if (sm_fail) return;
    // ---- 3. merge the world records of head h (gqa_reduce.wgsl:33-64; empty shards weigh nothing) ----
    const float *mine = reinterpret_cast<const float *>(a.peer_bases[a.rank] + a.flags_bytes) + ((size_t)par * a.world * a.nh) * rs;
    if (tid < a.world) sm_lse[tid] = __ldcg(mine + ((size_t)tid * a.nh + h) * rs + a.hd);
    __syncthreads();
    float gmax = -INFINITY;
    for (uint32_t r = 0; r < a.world; ++r)
        if (sm_lse[r] > -INFINITY) gmax = fmaxf(gmax, sm_lse[r]);
    for (uint32_t d = tid; d < a.hd; d += blockDim.x) {
        float acc = 0.f, wsum = 0.f;
        for (uint32_t r = 0; r < a.world; ++r) {
            const float l = sm_lse[r];
            if (!(l > -INFINITY)) continue;
            const float w = expf(l - gmax);
            acc += w * __ldcg(mine + ((size_t)r * a.nh + h) * rs + d);
            wsum += w;
        }
        float val = wsum > 0.f ? acc / wsum : 0.f;
        const size_t oi = (size_t)h * a.hd + d;
        if (a.gate) val *= sigmoidf_ref(a.gate[oi]);
        store_from_f32(a.out, oi, a.out_dtype, val);
    }
}

int launch_combine_p2p(shady_ctx *ctx, uint32_t world, uint32_t rank, uint32_t nh, uint32_t hd, uint32_t epoch,
                       void *const *d_peer_table, const float *d_rec, void *d_out, uint32_t out_dtype, const float *d_gate) {
    SHADY_REQUIRE(ctx, d_peer_table && d_rec && d_out && nh && hd, SHADY_ERR_BAD_ARG, "combine_p2p: null or zero argument");
    SHADY_REQUIRE(ctx, world >= 1 && world <= kP2PMaxWorld && rank < world, SHADY_ERR_BAD_ARG, "combine_p2p: bad world/rank");
    SHADY_REQUIRE(ctx, epoch != 0, SHADY_ERR_BAD_ARG, "combine_p2p: epoch must start at 1 (flags start at 0)");
    SHADY_REQUIRE(ctx, out_dtype <= SHADY_BF16, SHADY_ERR_BAD_ARG, "combine_p2p: bad out dtype");
    if (const int st = pending_timeout(ctx, "combine_p2p")) return st;
    P2PArgs a{};
    a.peer_bases = reinterpret_cast<char *const *>(d_peer_table);
    a.rec = d_rec; a.out = d_out; a.gate = d_gate; a.status = status_ref(ctx); a.wait_peer = ctx->wait_peer;
    a.rank = rank; a.world = world; a.nh = nh; a.hd = hd; a.epoch = epoch; a.out_dtype = out_dtype;
    a.flags_bytes = p2p_flags_bytes(world, nh);
    p2p_combine_kernel<<<nh, 128, 0, ctx->stream>>>(a);
    ctx->launches++;
    SHADY_CUDA_OK(ctx, cudaGetLastError());
    return SHADY_OK;
}

}  // namespace shady
