// Causal prefill attention (placeholder until the tensor-core kernel lands).
#include "common.cuh"

int flare_launch_prefill(flare_attn_ctx* ctx, const PrefillArgs& a) {
    (void)a;
    return flare_set_error(ctx, FLARE_ERR_UNSUPPORTED, "prefill attention kernel is not built yet");
}
