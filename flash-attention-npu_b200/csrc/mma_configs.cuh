// Tile configurations of the register-accumulator kernel, per padded head dim.
//   X(index, MT, WM, WN, BN, STAGES)
// index 0: <= 16 packed rows (decode)      index 1: <= 32 packed rows (speculative decode)
// (for head dim 128 these two keep two CTAs resident per SM: measured 1.5x faster than one CTA
//  with 128-token stages, the kernel being latency- rather than bandwidth-limited)
// index 2: larger packed-GQA tiles          index 3: one query head per tile (prefill fallback)
#pragma once

#include "fwd_mma.cuh"

#define FA_MMA_CONFIGS_64(X) X(0, 1, 1, 4, 128, 4) X(1, 2, 1, 4, 128, 4) X(2, 2, 2, 2, 64, 4) X(3, 1, 4, 1, 64, 3)
#define FA_MMA_CONFIGS_128(X) X(0, 1, 1, 4, 64, 3) X(1, 2, 1, 4, 64, 3) X(2, 2, 2, 2, 64, 3) X(3, 1, 4, 1, 64, 2)
#define FA_MMA_CONFIGS_256(X) X(0, 1, 1, 4, 64, 3) X(1, 1, 2, 2, 64, 2) X(2, 1, 4, 1, 64, 2) X(3, 1, 4, 1, 64, 2)

namespace fa {

struct MmaConfigInfo {
  int block_m, block_n, threads, smem_bytes;
};

inline bool mma_config_info(int hd, int cfg, MmaConfigInfo* out) {
#define FA_X(I_, MT_, WM_, WN_, BN_, ST_)                                                   \
  if (cfg == I_) {                                                                     \
    using Tr = MmaTraits<FA_HD_, __nv_bfloat16, MT_, WM_, WN_, BN_, ST_>;                  \
    *out = MmaConfigInfo{Tr::BM, Tr::BN, Tr::NTHREADS, Tr::SMEM_BYTES};               \
    return true;                                                                      \
  }
  if (hd == 64) {
#define FA_HD_ 64
    FA_MMA_CONFIGS_64(FA_X)
#undef FA_HD_
  } else if (hd == 128) {
#define FA_HD_ 128
    FA_MMA_CONFIGS_128(FA_X)
#undef FA_HD_
  } else if (hd == 256) {
#define FA_HD_ 256
    FA_MMA_CONFIGS_256(FA_X)
#undef FA_HD_
  }
#undef FA_X
  return false;
}

// Defined in mma_inst_<hd>_<dtype>.cu (one translation unit each so they compile in parallel).
cudaError_t launch_mma_64_bf16(int cfg, const KParams& p, int grid, cudaStream_t st);
cudaError_t launch_mma_64_fp16(int cfg, const KParams& p, int grid, cudaStream_t st);
cudaError_t launch_mma_128_bf16(int cfg, const KParams& p, int grid, cudaStream_t st);
cudaError_t launch_mma_128_fp16(int cfg, const KParams& p, int grid, cudaStream_t st);
cudaError_t launch_mma_256_bf16(int cfg, const KParams& p, int grid, cudaStream_t st);
cudaError_t launch_mma_256_fp16(int cfg, const KParams& p, int grid, cudaStream_t st);

}  // namespace fa
