// tcgen05 prefill kernel (placeholder translation unit until the kernel lands).
#include "tc5_api.cuh"

namespace fa {

bool tc5_eligible(const fa_fwd_params&, bool, bool, int) { return false; }
void tc5_fill_plan(const fa_fwd_params&, fa_fwd_plan*) {}
int tc5_launch(const fa_fwd_params&, const fa_fwd_plan&, cudaStream_t, std::string* err) {
  *err = "tcgen05 kernel not built";
  return FA_ERR_UNSUPPORTED;
}

}  // namespace fa
