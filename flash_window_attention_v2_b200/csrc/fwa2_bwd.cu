// Backward kernel (placeholder until the kernel lands): the entry points exist so that the
// library exports its full ABI, and fail loudly.
#include "../../include/fwa2.h"

extern "C" size_t fwa2_bwd_workspace_bytes(int32_t, int32_t, int32_t, int32_t, int32_t, int32_t) { return 0; }
extern "C" int fwa2_backward(const fwa2_bwd_args*, void*) { return FWA2_ERR_LAUNCH; }
