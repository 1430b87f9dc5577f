// Softmax + epilogue role of the tcgen05 prefill kernel: 128 threads per query sub-tile, one
// thread per query row (TMEM lane).  Restates the arithmetic of the reference's OnlineSoftmax and
// RescaleO epilogues (csrc/arch22/flash_attn_npu_v2/online_softmax.hpp:479-803,
// rescale_o.hpp:299-534) in the log2 domain: P = exp2(S * scale*log2e - m * scale*log2e), P rounded
// to the input dtype before P.V, O rescaled only when the running max moved (by more than an optional threshold),
// final O / l and LSE = m * scale + ln(l).
#pragma once

#include "fwd_tc5_kernel.cuh"

namespace fa {
namespace tc5 {

template <typename T>
__device__ __forceinline__ void softmax_loop(const Tc5Params& p, Barriers* bar, uint32_t tmem, int t, int warp_in_wg,
                                             int lane) {
  volatile int* abort_flag = &bar->abort_flag;
  const int row = warp_in_wg * 32 + lane;
  const uint32_t lane_addr = (uint32_t)(warp_in_wg * 32) << 16;
  const uint32_t s_tmem = tmem + lane_addr + t * 128;
  const uint32_t o_tmem = tmem + lane_addr + 256 + t * 128;
  uint32_t s_cnt = 0, od_cnt = 0;
  const float scale_log2 = p.scale_log2;

  for (int n = blockIdx.x; n < p.total_tiles; n += gridDim.x) {
    TileInfo ti;
    tile_info(p, n, ti);
    if (ti.row0[t] >= ti.q_len) continue;
    const int i = ti.row0[t] + row;
    const bool row_valid = i < ti.q_len;
    T* o_ptr = reinterpret_cast<T*>(p.a.o) + (int64_t)ti.bi * p.a.o_batch_stride +
               (int64_t)(ti.q_row0 + i) * p.a.o_row_stride + (int64_t)ti.hh * p.a.o_head_stride;
    float* lse_ptr = p.a.lse + (int64_t)ti.bi * p.a.lse_batch_stride + (int64_t)ti.hh * p.a.lse_head_stride +
                     ti.q_row0 + i;
    if (!ti.has[t]) {  // no visible key for the whole sub-tile
      if (row_valid) {
        for (int c = 0; c < p.a.d; c += 8) *reinterpret_cast<uint4*>(o_ptr + c) = make_uint4(0, 0, 0, 0);
        *lse_ptr = INFINITY;
      }
      continue;
    }
    int lo = 0, hi = ti.k_len - 1;
    if (p.is_causal) hi = min(hi, i + ti.koff);
    if (p.is_local) {
      hi = min(hi, i + ti.koff + p.wr);
      lo = max(0, i + ti.koff - p.wl);
    }
    const int i_min = ti.row0[t], i_max = min(ti.q_len, ti.row0[t] + kBlockM) - 1;
    float m_run = -INFINITY, l_run = 0.f;

    for (int j = ti.jlo[t]; j < ti.jhi[t]; ++j) {
      if (!mbar_wait(smem_addr(&bar->s_full[t]), s_cnt & 1, abort_flag)) return;
      ++s_cnt;
      tc_fence_after();
      uint32_t s[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(s_tmem + c * 32, s[c]);
      tmem_wait_ld();

      const int col0 = j * kBlockN;
      bool need_mask = col0 + kBlockN > ti.k_len;
      if (p.is_causal || p.is_local) need_mask = need_mask || (col0 + kBlockN - 1 > i_min + ti.koff + (p.is_local ? p.wr : 0));
      if (p.is_local) need_mask = need_mask || (col0 < i_max + ti.koff - p.wl);
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const int col = col0 + c * 32 + e;
            if (col < lo || col > hi) s[c][e] = 0xff800000u;  // -inf
          }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int e = 0; e < 32; e += 4) {
          mx0 = fmaxf(mx0, __uint_as_float(s[c][e]));
          mx1 = fmaxf(mx1, __uint_as_float(s[c][e + 1]));
          mx2 = fmaxf(mx2, __uint_as_float(s[c][e + 2]));
          mx3 = fmaxf(mx3, __uint_as_float(s[c][e + 3]));
        }
      const float blk_max = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      float m_new = fmaxf(m_run, blk_max);
      // optional lazy update: keep the old reference max while the true max is within the threshold
      // (numerator and denominator use the same reference, so the result stays consistent)
      if (m_run != -INFINITY && (m_new - m_run) * scale_log2 <= p.rescale_threshold) m_new = m_run;
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float corr = fast_exp2((m_run - m_use) * scale_log2);  // 0 when m_run = -inf
      const bool rescale = (m_new != m_run) && (j > ti.jlo[t]);
      m_run = m_new;
      const float neg_ms = -m_use * scale_log2;

      float sum0 = 0.f, sum1 = 0.f;
      uint32_t pk[2][32];
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          const float p0 = fast_exp2(fmaf(__uint_as_float(s[c][e]), scale_log2, neg_ms));
          const float p1 = fast_exp2(fmaf(__uint_as_float(s[c][e + 1]), scale_log2, neg_ms));
          sum0 += p0;
          sum1 += p1;
          pk[c >> 1][(c & 1) * 16 + (e >> 1)] = pack2<T>(p0, p1);
        }
      l_run = l_run * corr + (sum0 + sum1);

      if (j > ti.jlo[t]) {  // P.V of the previous block has finished accumulating into O_t
        if (!mbar_wait(smem_addr(&bar->o_done[t]), od_cnt & 1, abort_flag)) return;
        ++od_cnt;
        if (__any_sync(0xffffffffu, rescale)) {
          tc_fence_after();
          const float f = rescale ? corr : 1.f;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t o[32];
            tmem_ld32(o_tmem + c * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * f);
            tmem_st32(o_tmem + c * 32, o);
          }
        }
      }
      tmem_st32(s_tmem, pk[0]);
      tmem_st32(s_tmem + 32, pk[1]);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_addr(&bar->p_full[t]));
    }

    // ---- epilogue: O_t / l -> global, LSE ----
    if (!mbar_wait(smem_addr(&bar->o_done[t]), od_cnt & 1, abort_flag)) return;
    ++od_cnt;
    tc_fence_after();
    const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t o[32];
      tmem_ld32(o_tmem + c * 32, o);
      tmem_wait_ld();
      if (row_valid) {
#pragma unroll
        for (int e = 0; e < 32; e += 8) {
          uint4 w;
          w.x = pack2<T>(__uint_as_float(o[e]) * inv, __uint_as_float(o[e + 1]) * inv);
          w.y = pack2<T>(__uint_as_float(o[e + 2]) * inv, __uint_as_float(o[e + 3]) * inv);
          w.z = pack2<T>(__uint_as_float(o[e + 4]) * inv, __uint_as_float(o[e + 5]) * inv);
          w.w = pack2<T>(__uint_as_float(o[e + 6]) * inv, __uint_as_float(o[e + 7]) * inv);
          *reinterpret_cast<uint4*>(o_ptr + c * 32 + e) = w;
        }
      }
    }
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_addr(&bar->o_free[t]));
    if (row_valid) *lse_ptr = l_run > 0.f ? (m_run * p.a.softmax_scale + __logf(l_run)) : INFINITY;
  }
}

}  // namespace tc5
}  // namespace fa
