// Launcher of the append / rotary prologue that precedes the tcgen05 prefill kernel (kv_prologue.cu).
#pragma once

#include <cuda_runtime.h>

#include "common.cuh"

namespace fa {

// Appends k_new / v_new to the cache (k rotated when rotary tables are given) and, when q_rot is not
// null, writes the rotated q there as a contiguous (b, s_q, h, d) tensor.  rot_per_token: query
// token i is rotated at position cache_seqlens + i (causal / local), else all at cache_seqlens.
cudaError_t launch_kv_prologue(const KParams& p, void* q_rot, bool rot_per_token, cudaStream_t st);

}  // namespace fa
