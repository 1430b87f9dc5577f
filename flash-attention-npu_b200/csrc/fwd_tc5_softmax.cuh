// Softmax role and correction / epilogue role of the tcgen05 prefill kernel.
//
// Softmax: 128 threads per query sub-tile, one thread per query row (TMEM lane).  It restates the
// arithmetic of the reference's OnlineSoftmax epilogue
// (csrc/arch22/flash_attn_npu_v2/online_softmax.hpp:479-803) in the log2 domain:
//   P = exp2(S * scale*log2e - m * scale*log2e), rounded to the input dtype before P.V.
// The 128 scores of a row are held in registers (the softmax warps raise their register budget
// with setmaxnreg, the other roles lower theirs).
//
// P leaves the thread as 16-byte chunks of 8 keys written to shared memory in the layout the MMA
// reads an A operand in (128-byte rows, 128-byte swizzle, two 64-key halves).  At the end of a tile
// the thread writes LSE = m*scale + ln(l) and hands 1 / l to the correction warps.
//
// Correction: 128 threads serving both sub-tiles.  When a row maximum moved it multiplies O (in
// TMEM) by exp2((m_old - m_new) * scale*log2e) between two P.V accumulations, off the softmax
// threads' critical path, and at the end of a tile writes O / l
// (RescaleO, csrc/arch22/flash_attn_npu_v2/rescale_o.hpp:299-534).
#pragma once

#include "fwd_tc5_kernel.cuh"

namespace fa {
namespace tc5 {

__device__ __forceinline__ float chunk_max(const uint32_t (&a)[32], float m) {
  float m0 = m, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
  for (int e = 0; e < 32; e += 8) {
    m0 = max3(m0, __uint_as_float(a[e]), __uint_as_float(a[e + 1]));
    m1 = max3(m1, __uint_as_float(a[e + 2]), __uint_as_float(a[e + 3]));
    m2 = max3(m2, __uint_as_float(a[e + 4]), __uint_as_float(a[e + 5]));
    m3 = max3(m3, __uint_as_float(a[e + 6]), __uint_as_float(a[e + 7]));
  }
  return fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
}

// Columns outside [lo, hi] become -inf.  The valid columns of the chunk form one bit mask, so an
// element costs a bit test and a select (per-element range compares were several times slower).
__device__ __forceinline__ void chunk_mask(uint32_t (&a)[32], int col_first, int lo, int hi) {
  const int n_lo = min(max(lo - col_first, 0), 32);       // first valid element of the chunk
  const int n_hi = min(max(hi - col_first + 1, 0), 32);   // one past the last valid element
  const uint32_t below_hi = n_hi >= 32 ? 0xffffffffu : ((1u << n_hi) - 1u);
  const uint32_t below_lo = n_lo >= 32 ? 0xffffffffu : ((1u << n_lo) - 1u);
  const uint32_t valid = below_hi & ~below_lo;
#pragma unroll
  for (int e = 0; e < 32; ++e)
    if (!((valid >> e) & 1u)) a[e] = 0xff800000u;  // -inf
}

// softcap: s -> softcap * tanh(s * scale / softcap), here straight into the log2 domain (tests/test_flash_attn_npu_v2.py:
// the golden applies it to the scaled scores before the mask).  tanh.approx has a relative error of 2^-11.
__device__ __forceinline__ void chunk_softcap(uint32_t (&a)[32], float mul, float cap_l2) {
#pragma unroll
  for (int e = 0; e < 32; ++e) {
    float th;
    asm("tanh.approx.f32 %0, %1;\n" : "=f"(th) : "f"(__uint_as_float(a[e]) * mul));
    a[e] = __float_as_uint(th * cap_l2);
  }
}

// Build-time tuning constants of the softmax role.
#ifndef FA_TC5_POLY
#define FA_TC5_POLY 0
#endif
#ifndef FA_TC5_RESCALE_THRESHOLD
#define FA_TC5_RESCALE_THRESHOLD 0.f
#endif
constexpr int kPolyPairs = FA_TC5_POLY;  // of every 4 pairs of exponentials, how many use the polynomial
constexpr float kRescaleThreshold = FA_TC5_RESCALE_THRESHOLD;

// 32 scores -> 16 packed 16-bit pairs of P, accumulating the fp32 row sum (two partial sums).
// POLY of every 4 pairs use the polynomial, the others the special-function unit.
template <typename T, int POLY>
__device__ __forceinline__ void chunk_exp(const uint32_t (&a)[32], uint64_t scale2, uint64_t negms2, uint64_t (&sum2)[4],
                                          uint32_t (&pk)[16]) {
#pragma unroll
  for (int e = 0; e < 32; e += 2) {
    const uint64_t x2 = fma_f32x2(pack_f32x2(__uint_as_float(a[e]), __uint_as_float(a[e + 1])), scale2, negms2);
    float p0, p1;
    if (((e >> 1) & 3) < POLY) {
      poly_exp2_x2(x2, p0, p1);
    } else {
      float x0, x1;
      unpack_f32x2(x2, x0, x1);
      p0 = fast_exp2(x0);
      p1 = fast_exp2(x1);
    }
    sum2[(e >> 1) & 3] = add_f32x2(sum2[(e >> 1) & 3], pack_f32x2(p0, p1));  // four independent chains
    pk[e >> 1] = pack2<T>(p0, p1);
  }
}

// 32 keys of P (16 packed pairs = four 16-byte chunks) of one row into the swizzled A-operand tile.
__device__ __forceinline__ void store_p_chunk(uint32_t p_row, uint32_t p_xor, int c, const uint32_t (&pk)[16]) {
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const uint32_t kc = (uint32_t)(c * 4 + q);
    const uint32_t addr = p_row + (kc >> 3) * kHalfBytes + (((kc & 7) ^ p_xor) << 4);
    asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(addr), "r"(pk[4 * q]), "r"(pk[4 * q + 1]),
                 "r"(pk[4 * q + 2]), "r"(pk[4 * q + 3])
                 : "memory");
  }
}

template <typename T, bool SOFTCAP, int ROWS>
__device__ __forceinline__ void softmax_loop(const Tc5Params& p, Barriers* bar, uint32_t tmem, uint32_t p_smem, int t,
                                             int warp_in_wg, int lane) {
  volatile int* abort_flag = &bar->abort_flag;
  const int row = warp_in_wg * 32 + lane;
  const uint32_t lane_addr = (uint32_t)(warp_in_wg * 32) << 16;
  const uint32_t s_tmem = tmem + lane_addr + t * 128;
  uint32_t s_cnt = 0, cr_cnt = 0, st_cnt = 0;
  // this row of P_t: chunk kc (8 keys) of the row lives at  half(kc) + row * 128 + ((kc ^ row) & 7) * 16
  const uint32_t p_row = p_smem + t * kTileBytes + row * 128;
  const uint32_t p_xor = (uint32_t)(row & 7);
  const uint32_t bar_sfree = smem_addr(&bar->s_free[t]), bar_odone = smem_addr(&bar->o_done[t]);
  const uint32_t bar_oready = smem_addr(&bar->o_ready[t]), bar_ofree = smem_addr(&bar->o_free[t]);
  // with softcap the scores are in the log2 domain once they have been capped: the scale is part of the cap
  const float scale_log2 = SOFTCAP ? 1.f : p.scale_log2;
  const float lse_scale = SOFTCAP ? 0.6931471805599453f : p.a.softmax_scale;  // running maximum -> natural log
  const uint64_t scale2 = pack_f32x2(scale_log2, scale_log2);

  TileSched sched(p);
  for (int n = sched.first(); n < p.total_tiles; n = sched.next()) {
    TileInfo ti;
    tile_info<ROWS>(p, n, ti);
    if (ti.row0[t] >= ti.q_len) continue;
    const int i = ti.row0[t] + row;
    if (!ti.has[t]) {  // no visible key for the whole sub-tile: O = 0, LSE = +inf
      if (i < ti.q_len) {
        T* o_ptr = reinterpret_cast<T*>(p.a.o) + (int64_t)ti.bi * p.a.o_batch_stride +
                   (int64_t)(ti.q_row0 + i) * p.a.o_row_stride + (int64_t)ti.hh * p.a.o_head_stride;
        for (int c = 0; c < p.a.d; c += 8) *reinterpret_cast<uint4*>(o_ptr + c) = make_uint4(0, 0, 0, 0);
        p.a.lse[(int64_t)ti.bi * p.a.lse_batch_stride + (int64_t)ti.hh * p.a.lse_head_stride + ti.q_row0 + i] = INFINITY;
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
      const int col0 = j * kBlockN;
      bool need_mask = col0 + kBlockN > ti.k_len;
      if (p.is_causal || p.is_local) need_mask = need_mask || (col0 + kBlockN - 1 > i_min + ti.koff + (p.is_local ? p.wr : 0));
      if (p.is_local) need_mask = need_mask || (col0 < i_max + ti.koff - p.wl);

      if (!mbar_wait(smem_addr(&bar->s_full[t]), s_cnt & 1, abort_flag, 41)) return;
      const uint32_t blk = s_cnt;  // running number of this block (all tiles of this CTA)
      ++s_cnt;
      tc_fence_after();
      // ---- all 128 scores of the row into registers (one TMEM round trip) ----
      uint32_t sc[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(s_tmem + c * 32, sc[c]);
      tmem_wait_ld();
      // the S columns are free: Q.K^T of the next block may overwrite them
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_sfree);
      if (SOFTCAP) {
#pragma unroll
        for (int c = 0; c < 4; ++c) chunk_softcap(sc[c], p.softcap_mul, p.softcap_l2);
      }
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < 4; ++c) chunk_mask(sc[c], col0 + c * 32, lo, hi);
      }
      float blk_max = chunk_max(sc[0], -INFINITY);
#pragma unroll
      for (int c = 1; c < 4; ++c) blk_max = chunk_max(sc[c], blk_max);

      float m_new = fmaxf(m_run, blk_max);
      // The running maximum follows every increase (P <= 1, and the row maximum has P = 1 exactly, like the
      // reference's golden).  kRescaleThreshold > 0 (log2 units) would keep the old maximum while the new one is
      // within the threshold: fewer O rescales for a few ulps of P rounding on sharply peaked rows.
      if (kRescaleThreshold > 0.f && m_run != -INFINITY && (m_new - m_run) * scale_log2 <= kRescaleThreshold) m_new = m_run;
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float corr = fast_exp2((m_run - m_use) * scale_log2);  // 0 when m_run = -inf
      if (j > ti.jlo[t]) {
        // The correction warps must have consumed the previous factors: this thread can be a whole
        // block ahead of them, and neither the factor array nor the barrier phase may be reused early.
        if (cr_cnt > 0 && !mbar_wait(bar_oready, (cr_cnt - 1) & 1, abort_flag, 47)) return;
        ++cr_cnt;
        bar->corr[t][row] = (m_new != m_run) ? corr : 1.f;
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_addr(&bar->corr_ready[t]));
      }
      m_run = m_new;
      const float neg_ms = -m_use * scale_log2;
      const uint64_t negms2 = pack_f32x2(neg_ms, neg_ms);

      // ---- exponentials, P -> shared memory ----
      uint64_t sum2[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) sum2[q] = pack_f32x2(0.f, 0.f);
      uint32_t pk[16];
      chunk_exp<T, kPolyPairs>(sc[0], scale2, negms2, sum2, pk);
      // P.V of the previous block must have read P_t before it is overwritten
      if (blk > 0 && !mbar_wait(bar_odone, (blk - 1) & 1, abort_flag, 42)) return;
      store_p_chunk(p_row, p_xor, 0, pk);
      chunk_exp<T, kPolyPairs>(sc[1], scale2, negms2, sum2, pk);
      store_p_chunk(p_row, p_xor, 1, pk);
      fence_proxy_async();  // generic-proxy stores -> visible to the MMA (async proxy)
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_addr(&bar->p_full[t][0]));  // first 64 keys of P are ready
      chunk_exp<T, kPolyPairs>(sc[2], scale2, negms2, sum2, pk);
      store_p_chunk(p_row, p_xor, 2, pk);
      chunk_exp<T, kPolyPairs>(sc[3], scale2, negms2, sum2, pk);
      store_p_chunk(p_row, p_xor, 3, pk);
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_addr(&bar->p_full[t][1]));  // last 64 keys
      float s0, s1;
      unpack_f32x2(add_f32x2(add_f32x2(sum2[0], sum2[1]), add_f32x2(sum2[2], sum2[3])), s0, s1);
      l_run = l_run * corr + (s0 + s1);
    }
    // 1 / l for the epilogue, LSE from here.  The previous tile's epilogue must have read its 1 / l
    // (a tile of a single block does not wait for anything else the epilogue does).
    if (st_cnt > 0 && !mbar_wait(bar_ofree, (st_cnt - 1) & 1, abort_flag, 48)) return;
    ++st_cnt;
    bar->row_inv[t][row] = l_run > 0.f ? 1.f / l_run : 0.f;
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_addr(&bar->stats_ready[t]));
    if (i < ti.q_len)
      p.a.lse[(int64_t)ti.bi * p.a.lse_batch_stride + (int64_t)ti.hh * p.a.lse_head_stride + ti.q_row0 + i] =
          l_run > 0.f ? (m_run * lse_scale + __logf(l_run)) : INFINITY;
  }
}

// Multiplies the HD fp32 columns of one TMEM lane by f (two chunks in flight).
template <int HD>
__device__ __forceinline__ void rescale_o(uint32_t o_tmem, float f) {
  const uint64_t f2 = pack_f32x2(f, f);
  uint32_t a[32], b[32];
  tmem_ld32(o_tmem, a);
  tmem_ld32(o_tmem + 32, b);
  tmem_wait_ld();
#pragma unroll
  for (int half = 0; half < HD / 64; ++half) {
#pragma unroll
    for (int e = 0; e < 32; e += 2) {
      float x0, x1;
      unpack_f32x2(mul_f32x2(pack_f32x2(__uint_as_float(a[e]), __uint_as_float(a[e + 1])), f2), x0, x1);
      a[e] = __float_as_uint(x0);
      a[e + 1] = __float_as_uint(x1);
      unpack_f32x2(mul_f32x2(pack_f32x2(__uint_as_float(b[e]), __uint_as_float(b[e + 1])), f2), x0, x1);
      b[e] = __float_as_uint(x0);
      b[e + 1] = __float_as_uint(x1);
    }
    tmem_st32(o_tmem + half * 64, a);
    tmem_st32(o_tmem + half * 64 + 32, b);
    if (half + 1 < HD / 64) {
      tmem_ld32(o_tmem + (half + 1) * 64, a);
      tmem_ld32(o_tmem + (half + 1) * 64 + 32, b);
      tmem_wait_ld();
    }
  }
  tmem_wait_st();
}

template <typename T, int HD>
__device__ __forceinline__ void correction_loop(const Tc5Params& p, Barriers* bar, uint32_t tmem, int warp_in_wg,
                                                int lane) {
  volatile int* abort_flag = &bar->abort_flag;
  const int row = warp_in_wg * 32 + lane;
  const uint32_t lane_addr = (uint32_t)(warp_in_wg * 32) << 16;
  uint32_t cr_cnt[2] = {0, 0}, od_cnt[2] = {0, 0}, st_cnt[2] = {0, 0};
  const int d_cols = p.a.d;

  TileSched sched(p);
  for (int n = sched.first(); n < p.total_tiles; n = sched.next()) {
    TileInfo ti;
    tile_info<Geo<HD>::kRows>(p, n, ti);
    if (ti.uhi <= ti.ulo) continue;
    for (int j = ti.ulo; j < ti.uhi; ++j) {
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        if (!(ti.has[t] && j > ti.jlo[t] && j < ti.jhi[t])) continue;
        if (!mbar_wait(smem_addr(&bar->corr_ready[t]), cr_cnt[t] & 1, abort_flag, 43)) return;
        ++cr_cnt[t];
        const float f = bar->corr[t][row];
        if (!mbar_wait(smem_addr(&bar->o_done[t]), od_cnt[t] & 1, abort_flag, 44)) return;  // P.V of block j-1 done
        ++od_cnt[t];
        if (__any_sync(0xffffffffu, f != 1.f)) {
          tc_fence_after();
          rescale_o<HD>(tmem + lane_addr + 256 + t * 128, f);
          tc_fence_before();
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_addr(&bar->o_ready[t]));
      }
    }
    // ---- epilogue of both sub-tiles ----
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      if (!ti.has[t]) continue;
      if (!mbar_wait(smem_addr(&bar->stats_ready[t]), st_cnt[t] & 1, abort_flag, 45)) return;
      ++st_cnt[t];
      const float inv = bar->row_inv[t][row];
      if (!mbar_wait(smem_addr(&bar->o_done[t]), od_cnt[t] & 1, abort_flag, 46)) return;  // last P.V done
      ++od_cnt[t];
      tc_fence_after();
      const int i = ti.row0[t] + row;
      const bool row_valid = i < ti.q_len;
      T* o_ptr = reinterpret_cast<T*>(p.a.o) + (int64_t)ti.bi * p.a.o_batch_stride +
                 (int64_t)(ti.q_row0 + i) * p.a.o_row_stride + (int64_t)ti.hh * p.a.o_head_stride;
      const uint32_t o_tmem = tmem + lane_addr + 256 + t * 128;
      uint32_t a[32], b[32];
      tmem_ld32(o_tmem, a);
      tmem_ld32(o_tmem + 32, b);
#pragma unroll
      for (int half = 0; half < HD / 64; ++half) {
        tmem_wait_ld();
        if (row_valid) {
#pragma unroll
          for (int e = 0; e < 32; e += 8) {
            uint4 w;
            w.x = pack2<T>(__uint_as_float(a[e]) * inv, __uint_as_float(a[e + 1]) * inv);
            w.y = pack2<T>(__uint_as_float(a[e + 2]) * inv, __uint_as_float(a[e + 3]) * inv);
            w.z = pack2<T>(__uint_as_float(a[e + 4]) * inv, __uint_as_float(a[e + 5]) * inv);
            w.w = pack2<T>(__uint_as_float(a[e + 6]) * inv, __uint_as_float(a[e + 7]) * inv);
            // written once, read by nobody here: streaming.  Head dims between the two tile widths: the tiles' columns
            // beyond the head dim are the zeros the TMA unit fills in, and are not stored.
            if (half * 64 + e < d_cols) __stcs(reinterpret_cast<uint4*>(o_ptr + half * 64 + e), w);
          }
#pragma unroll
          for (int e = 0; e < 32; e += 8) {
            uint4 w;
            w.x = pack2<T>(__uint_as_float(b[e]) * inv, __uint_as_float(b[e + 1]) * inv);
            w.y = pack2<T>(__uint_as_float(b[e + 2]) * inv, __uint_as_float(b[e + 3]) * inv);
            w.z = pack2<T>(__uint_as_float(b[e + 4]) * inv, __uint_as_float(b[e + 5]) * inv);
            w.w = pack2<T>(__uint_as_float(b[e + 6]) * inv, __uint_as_float(b[e + 7]) * inv);
            if (half * 64 + 32 + e < d_cols) __stcs(reinterpret_cast<uint4*>(o_ptr + half * 64 + 32 + e), w);
          }
        }
        if (half + 1 < HD / 64) {
          tmem_ld32(o_tmem + (half + 1) * 64, a);
          tmem_ld32(o_tmem + (half + 1) * 64 + 32, b);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_addr(&bar->o_free[t]));
    }
  }
}

}  // namespace tc5
}  // namespace fa
