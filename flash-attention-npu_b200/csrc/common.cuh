// Shared device helpers and the kernel-side parameter block.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "fa_b200.h"

namespace fa {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// What a kernel receives: the caller's parameters plus everything the host planner derived.
struct KParams {
  fa_fwd_params a;
  // host-normalised mask state; when wl_on_device != 0 the left-window rule
  // (wl >= max_k - 1 -> -1) is finished on the device from seqused_k.
  int32_t causal_in, wl, wr, wl_on_device;
  int32_t group;      // h / h_k
  int32_t gp;         // query heads packed into one tile (group or 1)
  int32_t heads_eff;  // h / gp
  int32_t m_blocks;
  int32_t num_splits, blocks_per_split;
  int32_t persistent;  // decode kernel: persistent CTAs with equal shares of the KV blocks; num_splits = partial slots
  float scale_log2;   // softmax_scale * log2(e)   (softcap: log2(e) only, see kernel)
  float* o_partial;   // [split][lse_index][d] fp32 (num_splits > 1)
  float* lse_partial; // [split][lse_index]
  int64_t lse_elems;  // elements of the LSE tensor
  int32_t* status;    // device status word (bounded waits that gave up), may be null
};

__host__ __device__ inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// ---- index tensors are never trusted ----
// A stale block_table / cache_batch_idx entry or a cache length beyond the cache's capacity must not become a wild
// access: the value is clamped (plain loads / stores) or handed to the TMA unit, whose tensor maps carry the true
// extents and return zeros outside them, and this bit is raised in the device status word for
// fa_b200_check_status.  The reference validates these on the host after a device-to-host copy
// (csrc/arch22/flash_attn_npu_v2/flash_api.cpp:459); here the lengths stay on the device.
constexpr int kStatusBadIndex = 0x10000000;
__device__ __forceinline__ void raise_bad_index(int32_t* status) {
  if (status) atomicOr(status, kStatusBadIndex);
}
// Keys already held by batch entry bi of a KV cache, clamped to [0, capacity - s_new].
__device__ __forceinline__ int cache_len(const fa_fwd_params& a, int bi, int32_t* status) {
  int l = a.seqused_k[bi];
  const int cap = max(a.seqlen_k - a.seqlen_new, 0);
  if (l < 0 || l > cap) {
    raise_bad_index(status);
    l = min(max(l, 0), cap);
  }
  return l;
}
// Outermost k / v index (page or cache row) clamped into [0, kv_outer) for code that forms addresses from it.
__device__ __forceinline__ int outer_index(const fa_fwd_params& a, int idx, int32_t* status) {
  const int n = a.kv_outer > 0 ? a.kv_outer : a.b;
  if ((unsigned)idx >= (unsigned)n) {
    raise_bad_index(status);
    idx = min(max(idx, 0), n - 1);
  }
  return idx;
}
// Same check for an index that goes into a TMA coordinate: out-of-range values are kept (the copy then
// returns zeros), only the status bit is raised.
__device__ __forceinline__ void check_outer_index(const fa_fwd_params& a, int idx, int32_t* status) {
  const int n = a.kv_outer > 0 ? a.kv_outer : a.b;
  if ((unsigned)idx >= (unsigned)n) raise_bad_index(status);
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, bool valid) {
  int sz = valid ? 16 : 0;  // src-size 0: nothing is read, 16 zero bytes are written
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(sz));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3,
                                                  uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}

template <typename T>
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma_16816<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma_16816<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Two fp32 -> packed 16-bit pair (round to nearest even), low half = first value.
template <typename T>
__device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <typename T>
__device__ __forceinline__ float to_f32(T x);
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <>
__device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }
template <typename T>
__device__ __forceinline__ T from_f32(float x);
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <>
__device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

union Vec16 {
  uint4 u;
  __nv_bfloat16 b[8];
  __half h[8];
};

// Rotary embedding of one 16-byte chunk (8 elements) of a row of x.
//   own     : the chunk at element offset c8 of the row
//   row_ptr : start of the row (to fetch the partner chunk in the non-interleaved layout)
//   cosr/sinr : the (rotary_dim / 2)-long cos / sin rows of this token's position
// Arithmetic: fp32 products rounded separately (no fused multiply-add), the difference / sum
// rounded once more, then round-to-nearest-even to T -- the same sequence of roundings as
// x1 * cos - x2 * sin evaluated on fp32 tensors on the host.
template <typename T>
__device__ __forceinline__ uint4 rotary_chunk(uint4 own_u, const T* row_ptr, int c8, const T* cosr, const T* sinr,
                                              int rotary_dim, bool interleaved) {
  if (c8 >= rotary_dim) return own_u;
  Vec16 own, out;
  own.u = own_u;
  const T* ownv = reinterpret_cast<const T*>(&own);
  T* outv = reinterpret_cast<T*>(&out);
  const int half = rotary_dim >> 1;
  if (interleaved) {
    const int j0 = c8 >> 1;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float x1 = to_f32<T>(ownv[2 * e]), x2 = to_f32<T>(ownv[2 * e + 1]);
      float c = to_f32<T>(cosr[j0 + e]), s = to_f32<T>(sinr[j0 + e]);
      outv[2 * e] = from_f32<T>(__fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, s)));
      outv[2 * e + 1] = from_f32<T>(__fadd_rn(__fmul_rn(x1, s), __fmul_rn(x2, c)));
    }
  } else {
    const bool first = c8 < half;
    Vec16 other;
    other.u = *reinterpret_cast<const uint4*>(row_ptr + (first ? c8 + half : c8 - half));
    const T* othv = reinterpret_cast<const T*>(&other);
    const int j0 = first ? c8 : c8 - half;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float c = to_f32<T>(cosr[j0 + e]), s = to_f32<T>(sinr[j0 + e]);
      if (first) {
        float x1 = to_f32<T>(ownv[e]), x2 = to_f32<T>(othv[e]);
        outv[e] = from_f32<T>(__fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, s)));
      } else {
        float x1 = to_f32<T>(othv[e]), x2 = to_f32<T>(ownv[e]);
        outv[e] = from_f32<T>(__fadd_rn(__fmul_rn(x1, s), __fmul_rn(x2, c)));
      }
    }
  }
  return out.u;
}

}  // namespace fa
