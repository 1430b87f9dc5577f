// Split-KV merge (one warp per output row):
//   m = max_i lse_i;  w_i = exp(lse_i - m);  O = sum_i w_i O_i / sum_i w_i;  LSE = m + ln sum_i w_i
// the same arithmetic as CombineScale (csrc/arch22/flash_attn_npu_v2/CombineScale.hpp:165-309).
// An empty partial carries lse = -inf (weight 0, its O is never read).  A row whose every
// partial is empty yields O = 0 and LSE = +inf (the API convention for a row without visible
// keys, rescale_o.hpp:57) -- or -inf when the result is itself a partial.
#pragma once

#include "common.cuh"

namespace fa {

constexpr int kCombineWarps = 4;

template <typename OutT>
__device__ __forceinline__ void store4(OutT* dst, float4 v);
template <>
__device__ __forceinline__ void store4<float>(float* dst, float4 v) { *reinterpret_cast<float4*>(dst) = v; }
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* dst, float4 v) {
  uint2 w;
  w.x = pack2<__nv_bfloat16>(v.x, v.y);
  w.y = pack2<__nv_bfloat16>(v.z, v.w);
  *reinterpret_cast<uint2*>(dst) = w;
}
template <>
__device__ __forceinline__ void store4<__half>(__half* dst, float4 v) {
  uint2 w;
  w.x = pack2<__half>(v.x, v.y);
  w.y = pack2<__half>(v.z, v.w);
  *reinterpret_cast<uint2*>(dst) = w;
}

// One row's merge weights for n <= 32 partials, one partial per lane: lane i loads LSE_i (one round trip for all of
// them instead of a chain of dependent loads), the maximum and the sum go through the warp.  Returns this lane's LSE
// and weight exp(LSE_i - m) / sum; m, tot and dead are the row's.  The arithmetic and its order are those of the
// sequential form below (lane i contributes term i, the same xor tree adds them up).
template <typename LoadLse>
__device__ __forceinline__ void merge_weights(int n, int lane, LoadLse lse_of, float& l_mine, float& w_mine, float& m, float& tot,
                                              bool& dead) {
  l_mine = lane < n ? lse_of(lane) : -INFINITY;
  m = l_mine;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  dead = (m == -INFINITY);
  tot = (!dead && lane < n) ? __expf(l_mine - m) : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
  const float inv = dead ? 0.f : 1.f / tot;
  w_mine = (dead || l_mine == -INFINITY) ? 0.f : __expf(l_mine - m) * inv;
}

// Weighted sum of 4 columns over n <= 32 partials in their order; the loads of eight partials are issued together.
// Partials whose LSE is -inf are skipped (their O may be anything).
template <typename LoadX>
__device__ __forceinline__ float4 merge_columns(int n, float l_mine, float w_mine, LoadX x_of) {
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int i0 = 0; i0 < n; i0 += 8) {
    float4 x[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) x[k] = (i0 + k < n) ? x_of(i0 + k) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float w = __shfl_sync(0xffffffffu, w_mine, (i0 + k) & 31), l = __shfl_sync(0xffffffffu, l_mine, (i0 + k) & 31);
      if (i0 + k < n && l != -INFINITY) {
        acc.x += w * x[k].x; acc.y += w * x[k].y; acc.z += w * x[k].z; acc.w += w * x[k].w;
      }
    }
  }
  return acc;
}

template <typename OutT>
__global__ void __launch_bounds__(kCombineWarps * 32) combine_kernel(const __grid_constant__ fa_combine_params p) {
  // The merge is launched as a programmatic dependent of the kernel in front of it (launch_combine): its CTAs may
  // become resident while that kernel still runs and wait here until it has completed and its writes are visible.
  // Without such a kernel in front this returns at once.
  asm volatile("griddepcontrol.wait;\n" ::: "memory");
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kCombineWarps + (threadIdx.x >> 5);
  const int64_t n_rows = (int64_t)p.b * p.s * p.h;
  if (row >= n_rows) return;
  // row -> (b, s, h), h fastest
  const int hh = (int)(row % p.h);
  const int ss = (int)((row / p.h) % p.s);
  const int bb = (int)(row / ((int64_t)p.h * p.s));
  const float* lp = p.lse_partial + bb * p.lp_batch_stride + ss * p.lp_row_stride + hh * p.lp_head_stride;
  const float* op = p.o_partial + bb * p.op_batch_stride + ss * p.op_row_stride + hh * p.op_head_stride;

  float m, tot;
  bool dead;
  OutT* out = reinterpret_cast<OutT*>(p.o) + bb * p.o_batch_stride + ss * p.o_row_stride + hh * p.o_head_stride;
  if (p.num_splits <= 32) {
    float l_mine, w_mine;
    merge_weights(p.num_splits, lane, [&](int i) { return lp[(int64_t)i * p.lp_split_stride]; }, l_mine, w_mine, m, tot, dead);
    for (int c0 = 0; c0 < p.d; c0 += 128) {  // every lane takes part in the shuffles, also one without columns
      const int c = c0 + lane * 4;
      const bool on = c < p.d;
      const float4 acc = merge_columns(p.num_splits, l_mine, w_mine, [&](int i) {
        return on ? *reinterpret_cast<const float4*>(op + (int64_t)i * p.op_split_stride + c) : make_float4(0.f, 0.f, 0.f, 0.f);
      });
      if (on) store4<OutT>(out + c, acc);
    }
  } else {
    m = -INFINITY;
    for (int i = lane; i < p.num_splits; i += 32) m = fmaxf(m, lp[(int64_t)i * p.lp_split_stride]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    dead = (m == -INFINITY);
    tot = 0.f;
    if (!dead)
      for (int i = lane; i < p.num_splits; i += 32) tot += __expf(lp[(int64_t)i * p.lp_split_stride] - m);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
    const float inv = dead ? 0.f : 1.f / tot;
    for (int c = lane * 4; c < p.d; c += 128) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      if (!dead) {
        for (int i = 0; i < p.num_splits; ++i) {
          const float l = lp[(int64_t)i * p.lp_split_stride];
          if (l == -INFINITY) continue;
          const float w = __expf(l - m) * inv;
          const float4 x = *reinterpret_cast<const float4*>(op + (int64_t)i * p.op_split_stride + c);
          acc.x += w * x.x; acc.y += w * x.y; acc.z += w * x.z; acc.w += w * x.w;
        }
      }
      store4<OutT>(out + c, acc);
    }
  }
  if (p.lse && lane == 0) {
    float v = dead ? (p.partial_out ? -INFINITY : INFINITY) : m + logf(tot);
    p.lse[bb * p.lse_batch_stride + ss * p.lse_row_stride + hh * p.lse_head_stride] = v;
  }
}

}  // namespace fa
