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

  float m = -INFINITY;
  for (int i = lane; i < p.num_splits; i += 32) m = fmaxf(m, lp[(int64_t)i * p.lp_split_stride]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  const bool dead = (m == -INFINITY);
  float tot = 0.f;
  if (!dead)
    for (int i = lane; i < p.num_splits; i += 32) tot += __expf(lp[(int64_t)i * p.lp_split_stride] - m);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
  const float inv = dead ? 0.f : 1.f / tot;

  OutT* out = reinterpret_cast<OutT*>(p.o) + bb * p.o_batch_stride + ss * p.o_row_stride + hh * p.o_head_stride;
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
  if (p.lse && lane == 0) {
    float v = dead ? (p.partial_out ? -INFINITY : INFINITY) : m + logf(tot);
    p.lse[bb * p.lse_batch_stride + ss * p.lse_row_stride + hh * p.lse_head_stride] = v;
  }
}

}  // namespace fa
