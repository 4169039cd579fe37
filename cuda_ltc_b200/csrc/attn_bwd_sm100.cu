// Attention backward on the sm_100a tensor pipe (placeholder translation unit while the kernel
// is brought up: every problem is routed to the fp32 backward).
#include "host_common.h"

namespace ltca {

bool attn_bwd_sm100_supported(const ltca_attn_params*) { return false; }
size_t attn_bwd_sm100_workspace(const ltca_attn_params*) { return 0; }
int launch_attn_bwd_sm100(ltca_ctx* ctx, const ltca_attn_params*) {
    return fail(ctx, LTCA_ERR_UNSUPPORTED, "tensor-pipe backward not available");
}

}  // namespace ltca
