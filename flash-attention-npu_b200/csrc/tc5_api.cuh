// Interface between the host planner and the tcgen05 / TMEM / TMA prefill kernel.
#pragma once

#include <cuda_runtime.h>

#include <string>

#include "fa_b200.h"

namespace fa {

// True when the tcgen05 kernel covers this problem (dense or varlen prefill without paging,
// append, alibi or softcap, head dim 64 or 128).
bool tc5_eligible(const fa_fwd_params& a, bool is_causal, bool is_local, int wl_on_device);
// Overwrites the tile fields of the plan for the tcgen05 kernel.
void tc5_fill_plan(const fa_fwd_params& a, fa_fwd_plan* pl);
int tc5_launch(const fa_fwd_params& a, const fa_fwd_plan& pl, cudaStream_t st, std::string* err);
// Synchronises the stream, then returns and clears the device status word (0 = every wait completed).
int tc5_read_status(cudaStream_t st);

}  // namespace fa
