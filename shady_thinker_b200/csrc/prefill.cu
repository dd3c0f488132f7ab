// Causal prefill attention (placeholder until the tcgen05 kernel lands in this file).
#include "common.cuh"

namespace shady {
int launch_prefill(shady_ctx *ctx, const shady_prefill_params *, const void *, const shady_kv_cache *, void *) {
    return fail(ctx, SHADY_ERR_UNSUPPORTED, "attn_prefill: not built yet");
}
}  // namespace shady
