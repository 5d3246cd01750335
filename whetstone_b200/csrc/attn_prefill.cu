#include "attn_prefill.cuh"

namespace wst {

bool prefill_kernel_supports(int, int, int, int) { return false; }

wst_status_t launch_prefill(const PrefillLaunch &P) {
  return fail(WST_ERR_SHAPE, "%s: prefill kernel not built", P.name);
}

}  // namespace wst
