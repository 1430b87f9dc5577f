// Interface between the host planner and the tcgen05 / TMEM / TMA prefill kernel.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <string>

#include "fa_b200.h"

namespace fa {

// True when the tcgen05 kernel covers this problem (head dim up to 256, at least 128 query rows; dense,
// packed varlen, or a KV cache with per-entry lengths, paged or not; no alibi).
bool tc5_eligible(const fa_fwd_params& a, bool is_causal, bool is_local, int wl_on_device);
// Overwrites the tile fields of the plan for the tcgen05 kernel.
void tc5_fill_plan(const fa_fwd_params& a, fa_fwd_plan* pl);
int tc5_launch(const fa_fwd_params& a, const fa_fwd_plan& pl, cudaStream_t st, std::string* err);
// Synchronises the stream, then returns and clears the device status word (0 = every wait completed).
int tc5_read_status(cudaStream_t st);
// 4-D TMA descriptor (d, heads, rows, outer) over a 16-bit tensor with element strides; box =
// 64 columns x 1 head x box_rows rows x 1, 128-byte swizzle.  Returns false when the driver refuses.
bool tma_encode_rows(CUtensorMap* m, const void* ptr, int dtype, int d, int heads, int64_t rows, int64_t outer,
                     int64_t head_stride, int64_t row_stride, int64_t outer_stride, int box_rows);
// Device word shared by all kernels with bounded waits (allocated on first use, one per device).
int32_t* device_status_word();

}  // namespace fa
