// Main body of the register-accumulator forward kernel (see fwd_mma.cuh for the overview).
#pragma once

#include "fwd_mma.cuh"

namespace fa {

template <class Tr>
__global__ void __launch_bounds__(Tr::NTHREADS) fwd_mma_kernel(const __grid_constant__ KParams p) {
  using T = typename Tr::T;
  constexpr int MT = Tr::MT, NT = Tr::NT, DT = Tr::DT, KS = Tr::KS, BN = Tr::BN, BM = Tr::BM, ST = Tr::ST;
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ int s_red[32];
  __shared__ float s_lse[Tr::BM];

  // A merge kernel queued behind this one may start launching its CTAs now (they wait for this grid to complete).
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wm = warp / Tr::WN, wn = warp % Tr::WN;
  const int g8 = lane >> 2, t4 = lane & 3;

  // ---- which tile ----
  // Heads vary fastest: the CTAs that run together read the same token rows of the (.., h_k, d)
  // cache, i.e. neighbouring 2 * d-byte pieces of the same DRAM pages.
  int idx = blockIdx.x;
  const int hh = idx % p.heads_eff;
  idx /= p.heads_eff;
  const int split = idx % p.num_splits;
  idx /= p.num_splits;
  const int bi = idx % p.a.b;
  const int mb = p.m_blocks - 1 - idx / p.a.b;  // heavy (late) causal tiles first
  const int hk = (hh * p.gp) / p.group;

  // ---- sequence view ----
  SeqView<T> sv;
  {
    int q_row0 = 0;
    sv.q_len = p.a.seqlen_q;
    if (p.a.cu_seqlens_q) {
      q_row0 = p.a.cu_seqlens_q[bi];
      sv.q_len = p.a.cu_seqlens_q[bi + 1] - q_row0;
    }
    sv.q_row0 = q_row0;
    sv.q = reinterpret_cast<const T*>(p.a.q) + (int64_t)bi * p.a.q_batch_stride + (int64_t)q_row0 * p.a.q_row_stride;
    int k_row0 = 0;
    sv.l_cache = p.a.seqlen_k;
    if (p.a.cu_seqlens_k) {
      k_row0 = p.a.cu_seqlens_k[bi];
      sv.l_cache = p.a.cu_seqlens_k[bi + 1] - k_row0;
    }
    if (p.a.seqused_k) sv.l_cache = cache_len(p.a, bi, p.status);
    sv.k_len = sv.l_cache + p.a.seqlen_new;
    const T* kb = reinterpret_cast<const T*>(p.a.k) + (int64_t)hk * p.a.k_head_stride;
    const T* vb = reinterpret_cast<const T*>(p.a.v) + (int64_t)hk * p.a.v_head_stride;
    sv.pages = nullptr;
    if (p.a.block_table) {
      sv.pages = p.a.block_table + (int64_t)bi * p.a.block_table_batch_stride;
    } else {
      const int64_t row = p.a.cache_batch_idx ? outer_index(p.a, p.a.cache_batch_idx[bi], p.status) : bi;
      kb += row * p.a.k_batch_stride + (int64_t)k_row0 * p.a.k_row_stride;
      vb += row * p.a.v_batch_stride + (int64_t)k_row0 * p.a.v_row_stride;
    }
    sv.k = kb;
    sv.v = vb;
    sv.knew = sv.vnew = nullptr;
    if (p.a.k_new) {
      sv.knew = reinterpret_cast<const T*>(p.a.k_new) + (int64_t)bi * p.a.knew_batch_stride +
                (int64_t)hk * p.a.knew_head_stride;
      sv.vnew = reinterpret_cast<const T*>(p.a.v_new) + (int64_t)bi * p.a.vnew_batch_stride +
                (int64_t)hk * p.a.vnew_head_stride;
    }
  }
  const int rows_total = sv.q_len * p.gp;
  const int row0 = mb * BM;
  // ---- append duty: one CTA per (batch, kv head) writes the new tokens into the cache ----
  if (sv.knew && split == 0 && mb == 0 && (hh * p.gp) % p.group == 0) append_to_cache<Tr>(p, sv, tid);
  if (row0 >= rows_total) return;

  // ---- mask mode: finish the left-window rule on the device when the host could not ----
  int wl = p.wl;
  const int wr = p.wr;
  if (p.wl_on_device) {
    int mx = 0;
    for (int i = tid; i < p.a.b; i += Tr::NTHREADS) mx = max(mx, p.a.seqused_k[i] + p.a.seqlen_new);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) s_red[warp] = mx;
    __syncthreads();
    mx = 0;
    for (int w = 0; w < Tr::NTHREADS / 32; ++w) mx = max(mx, s_red[w]);
    if (mx > 0 && wl >= mx - 1) wl = -1;
  }
  const bool is_causal = wl < 0 && wr == 0;
  const bool is_local = (wl >= 0 || wr >= 0) && !is_causal;

  // ---- KV range of this tile and split ----
  const int koff = (p.a.kv_total > 0 ? p.a.kv_total - p.a.kv_pos_offset : sv.k_len) - sv.q_len;  // j <= i + koff
  const int i_min = row0 / p.gp;
  const int i_max = (min(rows_total, row0 + BM) - 1) / p.gp;
  int j_lo = 0, j_hi = sv.k_len;
  if (is_causal) j_hi = min(sv.k_len, i_max + koff + 1);
  if (is_local) {
    j_hi = min(sv.k_len, i_max + koff + wr + 1);
    j_lo = max(0, i_min + koff - wl);
  }
  int nb_lo = j_lo / BN;
  int nb_hi = j_hi > j_lo ? ceil_div(j_hi, BN) : nb_lo;
  int my_lo = nb_lo + split * p.blocks_per_split;
  int my_hi = min(nb_hi, my_lo + p.blocks_per_split);
  if (p.num_splits == 1) { my_lo = nb_lo; my_hi = nb_hi; }
  const int n_blocks = max(0, my_hi - my_lo);

  const uint32_t q_base = smem_u32(smem);
  const uint32_t pipe_base = q_base + Tr::Q_BYTES;

  // ---- prologue: Q + first stages ----
  load_q_tile<Tr>(p, sv, q_base, row0, hh, is_causal || is_local, tid);
#pragma unroll
  for (int s = 0; s < ST - 1; ++s) {
    if (s < n_blocks) load_kv_block<Tr>(p, sv, pipe_base + s * Tr::STAGE_BYTES, my_lo + s, tid);
    cp_async_commit();
  }

  // ---- per-thread row bounds: thread owns rows (mt, half) -> tile row (wm*MT+mt)*16 + g8 + 8*half ----
  int row_lo[MT][2], row_hi[MT][2];
  float slope_l2[MT][2];
  int row_i[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const int r = row0 + (wm * MT + mt) * 16 + g8 + 8 * hf;
      const int i = r / p.gp;
      row_i[mt][hf] = i;
      int lo = 0, hi = sv.k_len - 1;
      if (is_causal) hi = min(hi, i + koff);
      if (is_local) {
        hi = min(hi, i + koff + wr);
        lo = max(0, i + koff - wl);
      }
      if (r >= rows_total) hi = -1;
      row_lo[mt][hf] = lo;
      row_hi[mt][hf] = hi;
      slope_l2[mt][hf] = 0.f;
      if (p.a.alibi_slopes && r < rows_total) {
        const int head = hh * p.gp + (r - i * p.gp);
        slope_l2[mt][hf] = p.a.alibi_slopes[(int64_t)bi * p.a.alibi_batch_stride + head] * kLog2e;
      }
    }
  const bool has_alibi = p.a.alibi_slopes != nullptr;
  const bool has_softcap = p.a.softcap > 0.f;
  // score -> log2 domain: x = s * scale_log2; with softcap: x = cap*log2e * tanh(s * scale / cap)
  const float sc_mul = has_softcap ? p.a.softmax_scale / p.a.softcap : p.scale_log2;
  const float cap_l2 = p.a.softcap * kLog2e;

  float o_acc[MT][DT][4];
  float m_run[MT][2], l_run[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
    for (int dt = 0; dt < DT; ++dt)
#pragma unroll
      for (int e = 0; e < 4; ++e) o_acc[mt][dt][e] = 0.f;
    m_run[mt][0] = m_run[mt][1] = -INFINITY;
    l_run[mt][0] = l_run[mt][1] = 0.f;
  }

  // ---- main loop ----
  for (int it = 0; it < n_blocks; ++it) {
    cp_async_wait<ST - 2>();
    __syncthreads();
    {
      const int nx = it + ST - 1;
      if (nx < n_blocks) load_kv_block<Tr>(p, sv, pipe_base + (nx % ST) * Tr::STAGE_BYTES, my_lo + nx, tid);
      cp_async_commit();
    }
    const uint32_t k_base = pipe_base + (it % ST) * Tr::STAGE_BYTES;
    const uint32_t v_base = k_base + Tr::KV_BYTES;
    const int nb = my_lo + it;
    const int col0 = nb * BN + wn * Tr::NW;  // first key of this warp's slice

    // S = Q K^T
    float s_acc[MT][NT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) s_acc[mt][nt][e] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      uint32_t a[MT][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const int m = lane >> 3, r = lane & 7;
        const int row = (wm * MT + mt) * 16 + (m & 1) * 8 + r;
        ldmatrix_x4(a[mt][0], a[mt][1], a[mt][2], a[mt][3], tile_addr<Tr::ROW_BYTES>(q_base, row, ks * 2 + (m >> 1)));
      }
#pragma unroll
      for (int np = 0; np < NT / 2; ++np) {
        uint32_t b0, b1, b2, b3;
        const int m = lane >> 3, r = lane & 7;
        const int row = wn * Tr::NW + np * 16 + (m >> 1) * 8 + r;
        ldmatrix_x4(b0, b1, b2, b3, tile_addr<Tr::ROW_BYTES>(k_base, row, ks * 2 + (m & 1)));
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          mma_16816<T>(s_acc[mt][2 * np], a[mt], b0, b1);
          mma_16816<T>(s_acc[mt][2 * np + 1], a[mt], b2, b3);
        }
      }
    }

    // ---- online softmax on this warp's slice ----
    // Elementwise masking is only needed when the block touches a boundary.
    bool need_mask = has_alibi || (nb * BN + BN > sv.k_len);
    if (is_causal || is_local) need_mask = need_mask || (nb * BN + BN - 1 > i_min + koff + (is_local ? wr : 0));
    if (is_local) need_mask = need_mask || (nb * BN < i_max + koff - wl);
    need_mask = need_mask || (row0 + BM > rows_total);
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        float mx = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            float x = s_acc[mt][nt][hf * 2 + e] * sc_mul;
            if (has_softcap) {
              // cap * tanh(y) = cap * (1 - 2 / (exp(2y) + 1))
              const float ex = __expf(2.f * x);
              x = cap_l2 * (1.f - __fdividef(2.f, ex + 1.f));
            }
            if (need_mask) {
              const int j = col0 + nt * 8 + 2 * t4 + e;
              if (has_alibi) x -= slope_l2[mt][hf] * fabsf((float)(row_i[mt][hf] + koff - j));
              if (j < row_lo[mt][hf] || j > row_hi[mt][hf]) x = -INFINITY;
            }
            s_acc[mt][nt][hf * 2 + e] = x;
            mx = fmaxf(mx, x);
          }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run[mt][hf], mx);
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        const float corr = fast_exp2(m_run[mt][hf] - m_use);
        m_run[mt][hf] = m_new;
        float sum = 0.f;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float pv = fast_exp2(s_acc[mt][nt][hf * 2 + e] - m_use);
            s_acc[mt][nt][hf * 2 + e] = pv;
            sum += pv;
          }
        l_run[mt][hf] = l_run[mt][hf] * corr + sum;
#pragma unroll
        for (int dt = 0; dt < DT; ++dt) {
          o_acc[mt][dt][hf * 2] *= corr;
          o_acc[mt][dt][hf * 2 + 1] *= corr;
        }
      }
    }

    // ---- O += P V  (P rounded to T first, as the golden and DownCastP do) ----
#pragma unroll
    for (int kk = 0; kk < Tr::NW / 16; ++kk) {
      uint32_t a[MT][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        a[mt][0] = pack2<T>(s_acc[mt][2 * kk][0], s_acc[mt][2 * kk][1]);
        a[mt][1] = pack2<T>(s_acc[mt][2 * kk][2], s_acc[mt][2 * kk][3]);
        a[mt][2] = pack2<T>(s_acc[mt][2 * kk + 1][0], s_acc[mt][2 * kk + 1][1]);
        a[mt][3] = pack2<T>(s_acc[mt][2 * kk + 1][2], s_acc[mt][2 * kk + 1][3]);
      }
#pragma unroll
      for (int dp = 0; dp < DT / 2; ++dp) {
        uint32_t b0, b1, b2, b3;
        const int m = lane >> 3, r = lane & 7;
        const int row = wn * Tr::NW + kk * 16 + (m & 1) * 8 + r;
        ldmatrix_x4_trans(b0, b1, b2, b3, tile_addr<Tr::ROW_BYTES>(v_base, row, dp * 2 + (m >> 1)));
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          mma_16816<T>(o_acc[mt][2 * dp], a[mt], b0, b1);
          mma_16816<T>(o_acc[mt][2 * dp + 1], a[mt], b2, b3);
        }
      }
    }
  }

  // ================= epilogue =================
  cp_async_wait<0>();
  __syncthreads();
  float* slab = reinterpret_cast<float*>(smem + Tr::Q_BYTES);
  float2* ml = reinterpret_cast<float2*>(smem + Tr::SMEM_BYTES - Tr::ML_BYTES);  // [WN][BM] (m, l)
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      float l = l_run[mt][hf];
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      l_run[mt][hf] = l;
      if (t4 == 0) ml[wn * BM + (wm * MT + mt) * 16 + g8 + 8 * hf] = make_float2(m_run[mt][hf], l);
    }
  __syncthreads();
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const int trow = (wm * MT + mt) * 16 + g8 + 8 * hf;
      float m_all = -INFINITY;
#pragma unroll
      for (int w = 0; w < Tr::WN; ++w) m_all = fmaxf(m_all, ml[w * BM + trow].x);
      const float m_use = (m_all == -INFINITY) ? 0.f : m_all;
      float l_all = 0.f;
#pragma unroll
      for (int w = 0; w < Tr::WN; ++w) {
        const float2 x = ml[w * BM + trow];
        l_all += x.y * fast_exp2(x.x - m_use);
      }
      const float f = (l_all > 0.f) ? fast_exp2(m_run[mt][hf] - m_use) / l_all : 0.f;
      float* dst = slab + (size_t)(wn * BM + trow) * Tr::SLAB_LD;
#pragma unroll
      for (int dt = 0; dt < DT; ++dt)
        *reinterpret_cast<float2*>(dst + dt * 8 + 2 * t4) =
            make_float2(o_acc[mt][dt][hf * 2] * f, o_acc[mt][dt][hf * 2 + 1] * f);
    }
  __syncthreads();

  const bool to_partial = p.num_splits > 1;
  const bool f32_out = to_partial || p.a.partial_out;
  for (int trow = tid; trow < BM; trow += Tr::NTHREADS) {
    float m_all = -INFINITY, l_all = 0.f;
    for (int w = 0; w < Tr::WN; ++w) m_all = fmaxf(m_all, ml[w * BM + trow].x);
    const float m_use = (m_all == -INFINITY) ? 0.f : m_all;
    for (int w = 0; w < Tr::WN; ++w) {
      const float2 x = ml[w * BM + trow];
      l_all += x.y * fast_exp2(x.x - m_use);
    }
    s_lse[trow] = (l_all > 0.f) ? (m_use + log2f(l_all)) * kLn2 : -INFINITY;
  }
  __syncthreads();
  // one pass over (row, 4 columns)
  for (int c = tid; c < BM * (Tr::HD / 4); c += Tr::NTHREADS) {
    const int trow = c / (Tr::HD / 4), c4 = (c % (Tr::HD / 4)) * 4;
    const int r = row0 + trow;
    if (r >= rows_total) continue;
    const int i = r / p.gp, head = hh * p.gp + (r - i * p.gp);
    const int64_t lse_idx = (int64_t)bi * p.a.lse_batch_stride + (int64_t)head * p.a.lse_head_stride + sv.q_row0 + i;
    const float lse_row = s_lse[trow];
    const bool dead = lse_row == -INFINITY;
    if (c4 == 0) {
      if (to_partial) p.lse_partial[(int64_t)split * p.lse_elems + lse_idx] = lse_row;
      else p.a.lse[lse_idx] = (dead && !p.a.partial_out) ? INFINITY : lse_row;
    }
    if (c4 >= p.a.d || (dead && to_partial)) continue;  // the merge never reads an empty partial's O
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w = 0; w < Tr::WN; ++w) {
      const float4 x = *reinterpret_cast<const float4*>(slab + (size_t)(w * BM + trow) * Tr::SLAB_LD + c4);
      acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
    }
    if (to_partial) {
      *reinterpret_cast<float4*>(p.o_partial + ((int64_t)split * p.lse_elems + lse_idx) * p.a.d + c4) = acc;
    } else {
      const int64_t off = (int64_t)bi * p.a.o_batch_stride + (int64_t)(sv.q_row0 + i) * p.a.o_row_stride +
                          (int64_t)head * p.a.o_head_stride + c4;
      if (f32_out) {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.a.o) + off) = acc;
      } else {
        uint2 w2;
        w2.x = pack2<T>(acc.x, acc.y);
        w2.y = pack2<T>(acc.z, acc.w);
        *reinterpret_cast<uint2*>(reinterpret_cast<T*>(p.a.o) + off) = w2;
      }
    }
  }
}

}  // namespace fa
