// Attention backward (dQ, dK, dV) for dense and packed-varlen inputs.
//
// It replaces the reference's mha_bwd / mha_varlen_bwd host functions and FAG kernels
// (csrc/arch22/flash_attn_npu_v2/flash_api.cpp, pybind names bwd / varlen_bwd at :1301-1309) and
// follows the arithmetic of the reference's golden (tests/fa_small_op_golden.py:160-353):
//   P  = exp(S * scale - LSE)            with the forward's own LSE, masked entries 0
//   dV = P^T dO        dP = dO V^T       D_i = sum_d dO_id O_id  (= rowsum(dP o P))
//   dS = P o (dP - D) * scale            dQ = dS K        dK = dS^T Q
// (with softcap: S' = c tanh(S scale / c) replaces S scale, and dS gets the factor 1 - tanh^2)
// P and dS are rounded to the input dtype before the second matmuls (as the tensor cores need),
// all accumulation is fp32.
//
// One CTA owns 64 keys of one (batch entry, kv head): dK and dV of those keys stay in registers
// while the CTA walks over the query heads of the group and the 64-row query blocks that can see
// the keys; dQ contributions go to an fp32 accumulator in global memory with atomic adds (converted
// to the output dtype by bwd_convert_kernel).  mma.sync m16n8k16 with fp32 accumulators.
#pragma once

#include "common.cuh"

namespace fa {

struct BwdParams {
  const void *q, *k, *v, *o, *dout;
  const float* lse;
  void *dq, *dk, *dv;
  float* dq_accum;  // (rows of q, h, d_pad) fp32, zeroed
  float* delta;     // same indexing as lse
  const int32_t *cu_seqlens_q, *cu_seqlens_k;
  int64_t q_batch_stride, q_row_stride, q_head_stride;
  int64_t k_batch_stride, k_row_stride, k_head_stride;
  int64_t v_batch_stride, v_row_stride, v_head_stride;
  int64_t o_batch_stride, o_row_stride, o_head_stride;
  int64_t do_batch_stride, do_row_stride, do_head_stride;
  int64_t dq_batch_stride, dq_row_stride, dq_head_stride;
  int64_t dk_batch_stride, dk_row_stride, dk_head_stride;
  int64_t dv_batch_stride, dv_row_stride, dv_head_stride;
  int64_t lse_batch_stride, lse_head_stride;
  int32_t b, seqlen_q, seqlen_k, h, h_k, d, d_pad, total_q;
  int32_t is_causal, is_local, wl, wr;
  float softmax_scale, scale_log2;
  float softcap;  // 0 = off; scores become softcap * tanh(S * scale / softcap) (tests/fa_small_op_golden.py:80-89,124-125)
};

constexpr int kBwdBM = 64, kBwdBN = 64, kBwdThreads = 128;

template <int HD>
struct BwdSmem {
  static constexpr int PITCH = HD * 2 + 16;      // bytes per row of a [64 x HD] 16-bit tile
  static constexpr int PPITCH = kBwdBN * 2 + 16;  // bytes per row of the [64 x 64] P / dS tiles
  static constexpr int TILE = 64 * PITCH;
  static constexpr int K_OFF = 0, V_OFF = TILE, Q_OFF = 2 * TILE, DO_OFF = 3 * TILE;
  static constexpr int P_OFF = 4 * TILE, DS_OFF = P_OFF + 64 * PPITCH;
  static constexpr int LSE_OFF = DS_OFF + 64 * PPITCH, DELTA_OFF = LSE_OFF + 64 * 4;
  static constexpr int BYTES = DELTA_OFF + 64 * 4;
};

// D_i = sum_d dO_id * O_id.  Half a warp per (row, head): 16 lanes x 16 bytes cover 128 columns per step, so a row of
// O and of dO is one 256-byte transaction each (the head dim is a multiple of 8, rows are 16-byte aligned).
template <typename T>
__global__ void __launch_bounds__(128) bwd_delta_kernel(const __grid_constant__ BwdParams p) {
  const int lane = threadIdx.x & 31, l16 = lane & 15;
  const int64_t idx = ((int64_t)blockIdx.x * 4 + (threadIdx.x >> 5)) * 2 + (lane >> 4);
  const bool varlen = p.cu_seqlens_q != nullptr;
  const int64_t rows = varlen ? p.total_q : (int64_t)p.b * p.seqlen_q;
  const bool live = idx < rows * p.h;
  const int head = live ? (int)(idx % p.h) : 0;
  const int64_t row = live ? idx / p.h : 0;
  const int bi = varlen ? 0 : (int)(row / p.seqlen_q);
  const int64_t i = varlen ? row : row % p.seqlen_q;
  const T* o = reinterpret_cast<const T*>(p.o) + bi * p.o_batch_stride + i * p.o_row_stride + head * p.o_head_stride;
  const T* g = reinterpret_cast<const T*>(p.dout) + bi * p.do_batch_stride + i * p.do_row_stride + head * p.do_head_stride;
  float acc = 0.f;
  if (live) {
    for (int c = l16 * 8; c < p.d; c += 128) {
      Vec16 a, b;
      a.u = *reinterpret_cast<const uint4*>(o + c);
      b.u = *reinterpret_cast<const uint4*>(g + c);
      const T* av = reinterpret_cast<const T*>(&a);
      const T* bv = reinterpret_cast<const T*>(&b);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc += to_f32<T>(av[e]) * to_f32<T>(bv[e]);
    }
  }
#pragma unroll
  for (int s = 8; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
  if (live && l16 == 0) p.delta[bi * p.lse_batch_stride + head * p.lse_head_stride + i] = acc;
}

// fp32 dQ accumulator -> dq in the output dtype.
template <typename T>
__global__ void __launch_bounds__(256) bwd_convert_kernel(const __grid_constant__ BwdParams p) {
  const bool varlen = p.cu_seqlens_q != nullptr;
  const int64_t rows = varlen ? p.total_q : (int64_t)p.b * p.seqlen_q;
  const int chunks = p.d_pad / 4;
  const int64_t n = rows * p.h * chunks;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (int64_t)gridDim.x * blockDim.x) {
    const int c4 = (int)(idx % chunks) * 4;
    const int64_t rh = idx / chunks;
    const int head = (int)(rh % p.h);
    const int64_t row = rh / p.h;
    if (c4 >= p.d) continue;
    const int bi = varlen ? 0 : (int)(row / p.seqlen_q);
    const int64_t i = varlen ? row : row % p.seqlen_q;
    const float4 a = *reinterpret_cast<const float4*>(p.dq_accum + (row * p.h + head) * p.d_pad + c4);
    T* dst = reinterpret_cast<T*>(p.dq) + bi * p.dq_batch_stride + i * p.dq_row_stride + head * p.dq_head_stride + c4;
    uint2 w;
    w.x = pack2<T>(a.x, a.y);
    w.y = pack2<T>(a.z, a.w);
    *reinterpret_cast<uint2*>(dst) = w;
  }
}

// 64 rows x HD columns of a 16-bit matrix -> shared memory tile (rows >= n_rows and columns >= d are zero).
template <int HD, typename T>
__device__ __forceinline__ void bwd_load_tile(uint32_t dst, const T* src, int64_t row_stride, int n_rows, int d, int tid) {
  constexpr int CH = HD / 8;
  for (int c = tid; c < 64 * CH; c += kBwdThreads) {
    const int row = c / CH, ch = c % CH;
    const bool ok = row < n_rows && ch * 8 < d;
    const T* g = ok ? src + (int64_t)row * row_stride + ch * 8 : src;
    cp_async_16(dst + row * BwdSmem<HD>::PITCH + ch * 16, g, ok);
  }
}

template <int HD, typename T>
__global__ void __launch_bounds__(kBwdThreads) bwd_kernel(const __grid_constant__ BwdParams p) {
  using S = BwdSmem<HD>;
  // dK / dV accumulators cover at most 128 columns of the head dim at a time (register budget): a head dim of 256
  // takes two passes over the query blocks, each recomputing S, P, dP, dS; dQ is produced in the first pass only.
  constexpr int KS = HD / 16, DW = HD > 128 ? 128 : HD, DT = DW / 8, NPASS = HD / DW;
  constexpr int DQW = HD >= 128 ? 64 : 32, DH = DQW / 8, NQ = HD / DQW;  // dQ in slices of DQW columns
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t sb = smem_u32(smem);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g8 = lane >> 2, t4 = lane & 3;
  const int lm = lane >> 3, lr = lane & 7;  // ldmatrix: matrix index and row within it

  const int nb = blockIdx.x, hk = blockIdx.y, bi = blockIdx.z;
  int q_row0 = 0, q_len = p.seqlen_q, k_row0 = 0, k_len = p.seqlen_k;
  if (p.cu_seqlens_q) {
    q_row0 = p.cu_seqlens_q[bi];
    q_len = p.cu_seqlens_q[bi + 1] - q_row0;
    k_row0 = p.cu_seqlens_k[bi];
    k_len = p.cu_seqlens_k[bi + 1] - k_row0;
  }
  const int key0 = nb * kBwdBN;
  if (key0 >= k_len) return;
  const int n_keys = min(kBwdBN, k_len - key0);
  const int bq = p.cu_seqlens_q ? 0 : bi;
  const int koff = k_len - q_len;
  const int group = p.h / p.h_k;

  // K, V tiles of this CTA
  const T* kg = reinterpret_cast<const T*>(p.k) + (int64_t)bq * p.k_batch_stride + (int64_t)(k_row0 + key0) * p.k_row_stride +
                (int64_t)hk * p.k_head_stride;
  const T* vg = reinterpret_cast<const T*>(p.v) + (int64_t)bq * p.v_batch_stride + (int64_t)(k_row0 + key0) * p.v_row_stride +
                (int64_t)hk * p.v_head_stride;
  bwd_load_tile<HD, T>(sb + S::K_OFF, kg, p.k_row_stride, n_keys, p.d, tid);
  bwd_load_tile<HD, T>(sb + S::V_OFF, vg, p.v_row_stride, n_keys, p.d, tid);
  cp_async_commit();

  // query rows that can see at least one key of this block: i in [i_lo, i_hi)
  int i_lo = 0, i_hi = q_len;
  if (p.is_causal) i_lo = max(0, key0 - koff);
  if (p.is_local) {  // a negative side is unbounded (make_window_atten_mask, tests/fa_small_op_golden.py:36-58)
    if (p.wr >= 0) i_lo = max(0, key0 - koff - p.wr);
    if (p.wl >= 0) i_hi = min(q_len, key0 + n_keys - 1 - koff + p.wl + 1);
  }
  const int m_lo = i_lo / kBwdBM, m_hi = i_hi > i_lo ? ceil_div(i_hi, kBwdBM) : m_lo;

  float* lse_s = reinterpret_cast<float*>(smem + S::LSE_OFF);
  float* delta_s = reinterpret_cast<float*>(smem + S::DELTA_OFF);

#pragma unroll 1
  for (int pass = 0; pass < NPASS; ++pass) {
  float dk_acc[DT][4], dv_acc[DT][4];
#pragma unroll
  for (int dt = 0; dt < DT; ++dt)
#pragma unroll
    for (int e = 0; e < 4; ++e) dk_acc[dt][e] = dv_acc[dt][e] = 0.f;

  for (int hg = 0; hg < group; ++hg) {
    const int head = hk * group + hg;
    for (int mb = m_lo; mb < m_hi; ++mb) {
      const int row0 = mb * kBwdBM;
      const int n_rows = min(kBwdBM, q_len - row0);
      const T* qg = reinterpret_cast<const T*>(p.q) + (int64_t)bq * p.q_batch_stride + (int64_t)(q_row0 + row0) * p.q_row_stride +
                    (int64_t)head * p.q_head_stride;
      const T* dog = reinterpret_cast<const T*>(p.dout) + (int64_t)bq * p.do_batch_stride +
                     (int64_t)(q_row0 + row0) * p.do_row_stride + (int64_t)head * p.do_head_stride;
      __syncthreads();  // the previous iteration is done with Q, dO, P, dS, lse, delta
      bwd_load_tile<HD, T>(sb + S::Q_OFF, qg, p.q_row_stride, n_rows, p.d, tid);
      bwd_load_tile<HD, T>(sb + S::DO_OFF, dog, p.do_row_stride, n_rows, p.d, tid);
      cp_async_commit();
      if (tid < kBwdBM) {
        const int i = row0 + tid;
        const int64_t li = (int64_t)bq * p.lse_batch_stride + (int64_t)head * p.lse_head_stride + q_row0 + i;
        lse_s[tid] = i < q_len ? p.lse[li] * kLog2e : INFINITY;  // rows beyond the sequence: P = 0
        delta_s[tid] = i < q_len ? p.delta[li] : 0.f;
      }
      cp_async_wait<0>();
      __syncthreads();

      // ---- S = Q K^T and dP = dO V^T for this warp's 16 rows x 64 keys ----
      float s_acc[8][4], dp_acc[8][4];
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) s_acc[nt][e] = dp_acc[nt][e] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        uint32_t aq[4], ad[4];
        const int arow = warp * 16 + (lm & 1) * 8 + lr;
        const uint32_t aoff = arow * S::PITCH + (ks * 2 + (lm >> 1)) * 16;
        ldmatrix_x4(aq[0], aq[1], aq[2], aq[3], sb + S::Q_OFF + aoff);
        ldmatrix_x4(ad[0], ad[1], ad[2], ad[3], sb + S::DO_OFF + aoff);
#pragma unroll
        for (int np = 0; np < 4; ++np) {
          const int brow = np * 16 + (lm >> 1) * 8 + lr;
          const uint32_t boff = brow * S::PITCH + (ks * 2 + (lm & 1)) * 16;
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4(b0, b1, b2, b3, sb + S::K_OFF + boff);
          mma_16816<T>(s_acc[2 * np], aq, b0, b1);
          mma_16816<T>(s_acc[2 * np + 1], aq, b2, b3);
          ldmatrix_x4(b0, b1, b2, b3, sb + S::V_OFF + boff);
          mma_16816<T>(dp_acc[2 * np], ad, b0, b1);
          mma_16816<T>(dp_acc[2 * np + 1], ad, b2, b3);
        }
      }

      // ---- P, dS (fp32 in registers), rounded copies to shared memory ----
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int r = warp * 16 + g8 + 8 * hf;
        const int i = row0 + r;
        int lo = 0, hi = k_len - 1;
        if (p.is_causal) hi = min(hi, i + koff);
        if (p.is_local) {
          if (p.wr >= 0) hi = min(hi, i + koff + p.wr);
          if (p.wl >= 0) lo = max(0, i + koff - p.wl);
        }
        const float lse2 = lse_s[r], dl = delta_s[r];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int j = key0 + nt * 8 + 2 * t4 + e;
            float pv = 0.f, fac = p.softmax_scale;
            if (j >= lo && j <= hi) {
              if (p.softcap > 0.f) {  // d/dS of softcap * tanh(S * scale / softcap) = scale * (1 - tanh^2)
                const float th = tanhf(s_acc[nt][hf * 2 + e] * p.softmax_scale / p.softcap);
                pv = fast_exp2(p.softcap * th * kLog2e - lse2);
                fac = p.softmax_scale * (1.f - th * th);
              } else {
                pv = fast_exp2(s_acc[nt][hf * 2 + e] * p.scale_log2 - lse2);
              }
            }
            s_acc[nt][hf * 2 + e] = pv;
            dp_acc[nt][hf * 2 + e] = pv * (dp_acc[nt][hf * 2 + e] - dl) * fac;
          }
          const uint32_t off = r * S::PPITCH + (nt * 8 + 2 * t4) * 2;
          *reinterpret_cast<uint32_t*>(smem + S::P_OFF + off) = pack2<T>(s_acc[nt][hf * 2], s_acc[nt][hf * 2 + 1]);
          *reinterpret_cast<uint32_t*>(smem + S::DS_OFF + off) = pack2<T>(dp_acc[nt][hf * 2], dp_acc[nt][hf * 2 + 1]);
        }
      }

      // ---- dQ (this warp's 16 rows) += dS K, in slices of the head dim to bound the registers ----
      if (pass == 0) {
#pragma unroll
      for (int half = 0; half < NQ; ++half) {
        float dq_acc[DH][4];
#pragma unroll
        for (int dt = 0; dt < DH; ++dt)
#pragma unroll
          for (int e = 0; e < 4; ++e) dq_acc[dt][e] = 0.f;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {  // 16 keys per step
          uint32_t a[4];
          a[0] = pack2<T>(dp_acc[2 * kk][0], dp_acc[2 * kk][1]);
          a[1] = pack2<T>(dp_acc[2 * kk][2], dp_acc[2 * kk][3]);
          a[2] = pack2<T>(dp_acc[2 * kk + 1][0], dp_acc[2 * kk + 1][1]);
          a[3] = pack2<T>(dp_acc[2 * kk + 1][2], dp_acc[2 * kk + 1][3]);
#pragma unroll
          for (int dp = 0; dp < DH / 2; ++dp) {
            const int krow = kk * 16 + (lm & 1) * 8 + lr;
            const int dch = (half * DH + dp * 2) + (lm >> 1);
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4_trans(b0, b1, b2, b3, sb + S::K_OFF + krow * S::PITCH + dch * 16);
            mma_16816<T>(dq_acc[2 * dp], a, b0, b1);
            mma_16816<T>(dq_acc[2 * dp + 1], a, b2, b3);
          }
        }
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          const int i = row0 + warp * 16 + g8 + 8 * hf;
          if (i < q_len) {
            const int64_t grow = p.cu_seqlens_q ? (int64_t)q_row0 + i : (int64_t)bi * p.seqlen_q + i;  // row of q
            float* dst = p.dq_accum + (grow * p.h + head) * p.d_pad + half * DH * 8;
#pragma unroll
            for (int dt = 0; dt < DH; ++dt) {
              asm volatile("red.global.add.v2.f32 [%0], {%1, %2};\n" ::"l"(dst + dt * 8 + 2 * t4), "f"(dq_acc[dt][hf * 2]),
                           "f"(dq_acc[dt][hf * 2 + 1])
                           : "memory");
            }
          }
        }
      }
      }
      __syncthreads();  // P and dS of all four warps are in shared memory

      // ---- dV (this warp's 16 keys) += P^T dO,  dK += dS^T Q : contraction over the 64 rows ----
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {  // 16 rows per step
        uint32_t ap[4], as[4];
        const int prow = kk * 16 + (lm >> 1) * 8 + lr;
        const uint32_t poff = prow * S::PPITCH + (warp * 16 + (lm & 1) * 8) * 2;
        ldmatrix_x4_trans(ap[0], ap[1], ap[2], ap[3], sb + S::P_OFF + poff);
        ldmatrix_x4_trans(as[0], as[1], as[2], as[3], sb + S::DS_OFF + poff);
#pragma unroll
        for (int dp = 0; dp < DT / 2; ++dp) {
          const int brow = kk * 16 + (lm & 1) * 8 + lr;
          const uint32_t boff = brow * S::PITCH + (pass * (DW / 8) + dp * 2 + (lm >> 1)) * 16;
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4_trans(b0, b1, b2, b3, sb + S::DO_OFF + boff);
          mma_16816<T>(dv_acc[2 * dp], ap, b0, b1);
          mma_16816<T>(dv_acc[2 * dp + 1], ap, b2, b3);
          ldmatrix_x4_trans(b0, b1, b2, b3, sb + S::Q_OFF + boff);
          mma_16816<T>(dk_acc[2 * dp], as, b0, b1);
          mma_16816<T>(dk_acc[2 * dp + 1], as, b2, b3);
        }
      }
    }
  }

  // ---- dK, dV of this warp's 16 keys (columns of this pass) ----
  cp_async_wait<0>();
#pragma unroll
  for (int hf = 0; hf < 2; ++hf) {
    const int kr = warp * 16 + g8 + 8 * hf;
    if (kr >= n_keys) continue;
    T* dkg = reinterpret_cast<T*>(p.dk) + (int64_t)bq * p.dk_batch_stride + (int64_t)(k_row0 + key0 + kr) * p.dk_row_stride +
             (int64_t)hk * p.dk_head_stride;
    T* dvg = reinterpret_cast<T*>(p.dv) + (int64_t)bq * p.dv_batch_stride + (int64_t)(k_row0 + key0 + kr) * p.dv_row_stride +
             (int64_t)hk * p.dv_head_stride;
#pragma unroll
    for (int dt = 0; dt < DT; ++dt) {
      const int c = pass * DW + dt * 8 + 2 * t4;
      if (c < p.d) {
        *reinterpret_cast<uint32_t*>(dkg + c) = pack2<T>(dk_acc[dt][hf * 2], dk_acc[dt][hf * 2 + 1]);
        *reinterpret_cast<uint32_t*>(dvg + c) = pack2<T>(dv_acc[dt][hf * 2], dv_acc[dt][hf * 2 + 1]);
      }
    }
  }
  }  // pass
}

}  // namespace fa
