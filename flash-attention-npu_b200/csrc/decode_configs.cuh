// Tile configurations of the producer / consumer decode kernel (head dim padded to 128).
//   X(index, MT, WM, WN, BN, STAGES, SR)   rows per CTA = 16 * MT * WM, consumer warps = WM * WN;
//   SR = 1: the merge slab lies over the ring (never with persistent CTAs)
#pragma once

#include <cuda.h>

#include "fwd_decode.cuh"

// Only the configurations the planner can choose are built (measured against the others on the benchmark shapes):
//   3   up to 16 packed rows: two resident CTAs of 1 x 4 consumer warps, 64-key stages
//   5   17-32 rows, long key ranges or persistent launches: one CTA of 2 x 4 warps, 128-key stages
//   11  17-32 rows, short key ranges (a sliding window): two resident CTAs of 2 x 2 warps, slab over the ring
#define FA_DECODE_CONFIGS_128(X) X(3, 1, 1, 4, 64, 3, 0) X(5, 1, 2, 4, 128, 3, 0) X(11, 1, 2, 2, 64, 3, 1)

namespace fa {

struct DecodeConfigInfo {
  int block_m, block_n, threads, smem_bytes;
  bool slab_in_ring;
};

inline bool decode_config_info(int hd, int cfg, DecodeConfigInfo* out) {
  if (hd != 128) return false;
#define FA_X(I_, MT_, WM_, WN_, BN_, ST_, SR_)                                              \
  if (cfg == I_) {                                                                    \
    using Tr = DecTraits<128, __nv_bfloat16, MT_, WM_, WN_, BN_, ST_, SR_>;                \
    *out = DecodeConfigInfo{Tr::BM, Tr::BN, Tr::NTHREADS, Tr::SMEM_BYTES, Tr::SLAB_IN_RING}; \
    return true;                                                                      \
  }
  FA_DECODE_CONFIGS_128(FA_X)
#undef FA_X
  return false;
}

cudaError_t launch_decode_128_bf16(int cfg, const KParams& p, const CUtensorMap& tm_k, const CUtensorMap& tm_v, int grid,
                                   cudaStream_t st);
cudaError_t launch_decode_128_fp16(int cfg, const KParams& p, const CUtensorMap& tm_k, const CUtensorMap& tm_v, int grid,
                                   cudaStream_t st);

}  // namespace fa
