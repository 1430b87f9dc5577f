// Body of the producer / consumer split-KV decode kernel (overview in fwd_decode.cuh).
#pragma once

#include "fwd_decode.cuh"

namespace fa {

template <class Tr>
__global__ void __launch_bounds__(Tr::NTHREADS)
fwd_decode_kernel(const __grid_constant__ KParams p, const __grid_constant__ CUtensorMap tm_k,
                  const __grid_constant__ CUtensorMap tm_v) {
  using T = typename Tr::T;
  constexpr int MT = Tr::MT, NT = Tr::NT, DT = Tr::DT, KS = Tr::KS, BN = Tr::BN, BM = Tr::BM, ST = Tr::ST;
  constexpr int NCW = Tr::NCW, WN = Tr::WN, PITCH = Tr::PITCH;
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ float s_lse[Tr::BM];
  __shared__ int s_abort;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g8 = lane >> 2, t4 = lane & 3;
  const int wm = (warp < Tr::NCW) ? warp / Tr::WN : 0;  // row group of a consumer warp

  // ---- which tile (same enumeration as fwd_mma_kernel; m_blocks == 1 here) ----
  int idx = blockIdx.x;
  const int hh = idx % p.heads_eff;
  idx /= p.heads_eff;
  const int split = idx % p.num_splits;
  idx /= p.num_splits;
  const int bi = idx % p.a.b;
  const int hk = (hh * p.gp) / p.group;

  SeqView<T> sv;
  int batch_row = 0;
  {
    int q_row0 = 0;
    sv.q_len = p.a.seqlen_q;
    if (p.a.cu_seqlens_q) {
      q_row0 = p.a.cu_seqlens_q[bi];
      sv.q_len = p.a.cu_seqlens_q[bi + 1] - q_row0;
    }
    sv.q_row0 = q_row0;
    sv.q = reinterpret_cast<const T*>(p.a.q) + (int64_t)bi * p.a.q_batch_stride + (int64_t)q_row0 * p.a.q_row_stride;
    sv.l_cache = p.a.seqused_k ? p.a.seqused_k[bi] : p.a.seqlen_k;
    sv.k_len = sv.l_cache + p.a.seqlen_new;
    const T* kb = reinterpret_cast<const T*>(p.a.k) + (int64_t)hk * p.a.k_head_stride;
    const T* vb = reinterpret_cast<const T*>(p.a.v) + (int64_t)hk * p.a.v_head_stride;
    sv.pages = nullptr;
    if (p.a.block_table) {
      sv.pages = p.a.block_table + (int64_t)bi * p.a.block_table_batch_stride;
    } else {
      batch_row = p.a.cache_batch_idx ? p.a.cache_batch_idx[bi] : bi;
      kb += (int64_t)batch_row * p.a.k_batch_stride;
      vb += (int64_t)batch_row * p.a.v_batch_stride;
    }
    sv.k = kb;
    sv.v = vb;
    sv.knew = sv.vnew = nullptr;
    if (p.a.k_new) {
      sv.knew = reinterpret_cast<const T*>(p.a.k_new) + (int64_t)bi * p.a.knew_batch_stride + (int64_t)hk * p.a.knew_head_stride;
      sv.vnew = reinterpret_cast<const T*>(p.a.v_new) + (int64_t)bi * p.a.vnew_batch_stride + (int64_t)hk * p.a.vnew_head_stride;
    }
  }
  const int rows_total = sv.q_len * p.gp;
  if (sv.knew && split == 0 && (hh * p.gp) % p.group == 0) append_to_cache<Tr>(p, sv, tid);
  if (rows_total <= 0) return;

  int wl = p.wl;
  const int wr = p.wr;
  if (p.wl_on_device) {  // every warp reduces the batch maximum of the key lengths by itself (no block barrier)
    int mx = 0;
    for (int i = lane; i < p.a.b; i += 32) mx = max(mx, p.a.seqused_k[i] + p.a.seqlen_new);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (mx > 0 && wl >= mx - 1) wl = -1;
  }
  const bool is_causal = wl < 0 && wr == 0;
  const bool is_local = (wl >= 0 || wr >= 0) && !is_causal;

  const int koff = (p.a.kv_total > 0 ? p.a.kv_total - p.a.kv_pos_offset : sv.k_len) - sv.q_len;
  const int i_max = (rows_total - 1) / p.gp;
  int j_lo = 0, j_hi = sv.k_len;
  if (is_causal) j_hi = min(sv.k_len, i_max + koff + 1);
  if (is_local) {
    j_hi = min(sv.k_len, i_max + koff + wr + 1);
    j_lo = max(0, koff - wl);
  }
  const int nb_lo = j_lo / BN;
  const int nb_hi = j_hi > j_lo ? ceil_div(j_hi, BN) : nb_lo;
  int my_lo = nb_lo + split * p.blocks_per_split;
  int my_hi = min(nb_hi, my_lo + p.blocks_per_split);
  if (p.num_splits == 1) { my_lo = nb_lo; my_hi = nb_hi; }
  const int n_blocks = max(0, my_hi - my_lo);

  const uint32_t raw = smem_u32(smem);
  const uint32_t pipe_base = (raw + 1023u) & ~1023u;  // 128-byte-swizzled tiles need 1024-byte aligned bases
  uint8_t* smem_al = smem + (pipe_base - raw);
  const uint32_t q_base = pipe_base + Tr::MAIN_BYTES;
  const uint32_t full0 = q_base + Tr::Q_BYTES + Tr::ML_BYTES, empty0 = full0 + ST * 8;
  if (tid == 0) {
    for (int s = 0; s < ST; ++s) {
      tc5::mbar_init(full0 + s * 8, 1);     // the producer's arrival with the stage's byte count
      tc5::mbar_init(empty0 + s * 8, NCW);  // one arrival per consumer warp
    }
    s_abort = 0;
    tc5::fence_barrier_init();
  }
  __syncthreads();  // barriers initialised; from here the producer warp runs ahead of the consumers
  // ---- Q tile -> shared memory by the consumer warps (rotated when rotary tables are given);
  //      padded rows, no swizzle.  The producer is already fetching the first K / V stages. ----
  if (warp < NCW) {
    const bool rot_per_token = is_causal || is_local;
    for (int c = tid; c < BM * Tr::CHUNKS; c += NCW * 32) {
      const int row = c / Tr::CHUNKS, ch = c % Tr::CHUNKS;
      uint4 q4 = make_uint4(0, 0, 0, 0);
      if (row < rows_total && ch * 8 < p.a.d) {
        const int i = row / p.gp, g = row - i * p.gp;
        const T* qrow = sv.q + (int64_t)i * p.a.q_row_stride + (int64_t)(hh * p.gp + g) * p.a.q_head_stride;
        q4 = *reinterpret_cast<const uint4*>(qrow + ch * 8);
        if (p.a.rotary_cos) {
          const int pos = sv.l_cache + p.a.kv_pos_offset + (rot_per_token ? i : 0);
          const T* cosr = reinterpret_cast<const T*>(p.a.rotary_cos) + (int64_t)pos * (p.a.rotary_dim >> 1);
          const T* sinr = reinterpret_cast<const T*>(p.a.rotary_sin) + (int64_t)pos * (p.a.rotary_dim >> 1);
          q4 = rotary_chunk<T>(q4, qrow, ch * 8, cosr, sinr, p.a.rotary_dim, p.a.rotary_interleaved != 0);
        }
      }
      asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(q_base + row * PITCH + ch * 16), "r"(q4.x), "r"(q4.y), "r"(q4.z), "r"(q4.w));
    }
    asm volatile("bar.sync 1, %0;\n" ::"n"(NCW * 32));  // consumer warps only
  }

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

  if (warp == NCW) {
    if (lane == 0) { tc5::tma_prefetch_desc(&tm_k); tc5::tma_prefetch_desc(&tm_v); }
    decode_producer<Tr>(p, sv, &tm_k, &tm_v, pipe_base, full0, empty0, my_lo, n_blocks, hk, batch_row, &s_abort);
  } else {
    const int wn = warp % WN;
    // per-thread row bounds (thread owns rows g8 and g8 + 8 of each m-tile)
    int row_lo[MT][2], row_hi[MT][2], row_i[MT][2];
    float slope_l2[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int r = (wm * MT + mt) * 16 + g8 + 8 * hf;
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
        if (p.a.alibi_slopes && r < rows_total)
          slope_l2[mt][hf] = p.a.alibi_slopes[(int64_t)bi * p.a.alibi_batch_stride + hh * p.gp + (r - i * p.gp)] * kLog2e;
      }
    const bool has_alibi = p.a.alibi_slopes != nullptr;
    const bool has_softcap = p.a.softcap > 0.f;
    const float sc_mul = has_softcap ? p.a.softmax_scale / p.a.softcap : p.scale_log2;
    const float cap_l2 = p.a.softcap * kLog2e;

    uint32_t qf[Tr::Q_IN_REGS ? MT : 1][Tr::Q_IN_REGS ? KS : 1][4];
    if (Tr::Q_IN_REGS) {
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
          const int m = lane >> 3, r = lane & 7;
          const int row = (wm * MT + mt) * 16 + (m & 1) * 8 + r;
          ldmatrix_x4(qf[mt][ks][0], qf[mt][ks][1], qf[mt][ks][2], qf[mt][ks][3],
                      q_base + row * PITCH + (ks * 2 + (m >> 1)) * 16);
        }
    }

    for (int it = 0; it < n_blocks; ++it) {
      const int stage = it % ST;
      if (!tc5::mbar_wait(full0 + stage * 8, (it / ST) & 1, &s_abort)) break;
      const uint32_t k_base = pipe_base + stage * Tr::STAGE_BYTES, v_base = k_base + Tr::KV_BYTES;
      const int nb = my_lo + it;
      const int col0 = nb * BN + wn * Tr::NW;
      if (nb * BN + BN > sv.l_cache) decode_fix_rows<Tr>(p, sv, k_base, v_base, nb * BN, wn, lane);

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
          if (Tr::Q_IN_REGS) {
#pragma unroll
            for (int e = 0; e < 4; ++e) a[mt][e] = qf[mt][ks][e];
          } else {
            const int m = lane >> 3, r = lane & 7;
            const int row = (wm * MT + mt) * 16 + (m & 1) * 8 + r;
            ldmatrix_x4(a[mt][0], a[mt][1], a[mt][2], a[mt][3], q_base + row * PITCH + (ks * 2 + (m >> 1)) * 16);
          }
        }
#pragma unroll
        for (int np = 0; np < NT / 2; ++np) {
          uint32_t b0, b1, b2, b3;
          const int m = lane >> 3, r = lane & 7;
          const int row = wn * Tr::NW + np * 16 + (m >> 1) * 8 + r;
          ldmatrix_x4(b0, b1, b2, b3, kv_chunk_addr<Tr>(k_base, row, ks * 2 + (m & 1)));
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            mma_16816<T>(s_acc[mt][2 * np], a[mt], b0, b1);
            mma_16816<T>(s_acc[mt][2 * np + 1], a[mt], b2, b3);
          }
        }
      }

      bool need_mask = has_alibi || (nb * BN + BN > sv.k_len) || (BM > rows_total);
      if (is_causal || is_local) need_mask = need_mask || (nb * BN + BN - 1 > koff + (is_local ? wr : 0));
      if (is_local) need_mask = need_mask || (nb * BN < i_max + koff - wl);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          float mx = -INFINITY;
          if (!need_mask && !has_softcap) {  // interior block: scale only
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                const float x = s_acc[mt][nt][hf * 2 + e] * sc_mul;
                s_acc[mt][nt][hf * 2 + e] = x;
                mx = fmaxf(mx, x);
              }
          } else {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                float x = s_acc[mt][nt][hf * 2 + e] * sc_mul;
                if (has_softcap) {
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
          if (corr != 1.f) {
#pragma unroll
            for (int dt = 0; dt < DT; ++dt) {
              o_acc[mt][dt][hf * 2] *= corr;
              o_acc[mt][dt][hf * 2 + 1] *= corr;
            }
          }
        }
      }

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
          ldmatrix_x4_trans(b0, b1, b2, b3, kv_chunk_addr<Tr>(v_base, row, dp * 2 + (m >> 1)));
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            mma_16816<T>(o_acc[mt][2 * dp], a[mt], b0, b1);
            mma_16816<T>(o_acc[mt][2 * dp + 1], a[mt], b2, b3);
          }
        }
      }
      __syncwarp();
      if (lane == 0) tc5::mbar_arrive(empty0 + stage * 8);
    }
  }

  // ================= epilogue (all warps) =================
  __syncthreads();
  if (s_abort) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);  // let copies in flight land before the CTA retires
    if (tid == 0 && p.status) atomicExch(p.status, 0x40000000 | (int)blockIdx.x);
    __syncthreads();
  }
  float* slab = reinterpret_cast<float*>(smem_al);
  float2* ml = reinterpret_cast<float2*>(smem_al + Tr::MAIN_BYTES + Tr::Q_BYTES);
  if (warp < NCW) {
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        float l = l_run[mt][hf];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        l_run[mt][hf] = l;
        if (t4 == 0) ml[(warp % WN) * BM + (wm * MT + mt) * 16 + g8 + 8 * hf] = make_float2(m_run[mt][hf], l);
      }
  }
  __syncthreads();
  if (warp < NCW) {
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int trow = (wm * MT + mt) * 16 + g8 + 8 * hf;
        float m_all = -INFINITY;
#pragma unroll
        for (int w = 0; w < WN; ++w) m_all = fmaxf(m_all, ml[w * BM + trow].x);
        const float m_use = (m_all == -INFINITY) ? 0.f : m_all;
        float l_all = 0.f;
#pragma unroll
        for (int w = 0; w < WN; ++w) {
          const float2 x = ml[w * BM + trow];
          l_all += x.y * fast_exp2(x.x - m_use);
        }
        const float f = (l_all > 0.f) ? fast_exp2(m_run[mt][hf] - m_use) / l_all : 0.f;
        float* dst = slab + (size_t)((warp % WN) * BM + trow) * Tr::SLAB_LD;
#pragma unroll
        for (int dt = 0; dt < DT; ++dt)
          *reinterpret_cast<float2*>(dst + dt * 8 + 2 * t4) = make_float2(o_acc[mt][dt][hf * 2] * f, o_acc[mt][dt][hf * 2 + 1] * f);
      }
  }
  for (int trow = tid; trow < BM; trow += Tr::NTHREADS) {
    float m_all = -INFINITY, l_all = 0.f;
    for (int w = 0; w < WN; ++w) m_all = fmaxf(m_all, ml[w * BM + trow].x);
    const float m_use = (m_all == -INFINITY) ? 0.f : m_all;
    for (int w = 0; w < WN; ++w) {
      const float2 x = ml[w * BM + trow];
      l_all += x.y * fast_exp2(x.x - m_use);
    }
    s_lse[trow] = (l_all > 0.f) ? (m_use + log2f(l_all)) * kLn2 : -INFINITY;
  }
  __syncthreads();

  const bool to_partial = p.num_splits > 1;
  const bool f32_out = to_partial || p.a.partial_out;
  for (int c = tid; c < BM * (Tr::HD / 4); c += Tr::NTHREADS) {
    const int trow = c / (Tr::HD / 4), c4 = (c % (Tr::HD / 4)) * 4;
    if (trow >= rows_total) continue;
    const int i = trow / p.gp, head = hh * p.gp + (trow - i * p.gp);
    const int64_t lse_idx = (int64_t)bi * p.a.lse_batch_stride + (int64_t)head * p.a.lse_head_stride + sv.q_row0 + i;
    const float lse_row = s_lse[trow];
    const bool dead = lse_row == -INFINITY;
    if (c4 == 0) {
      if (to_partial) p.lse_partial[(int64_t)split * p.lse_elems + lse_idx] = lse_row;
      else p.a.lse[lse_idx] = (dead && !p.a.partial_out) ? INFINITY : lse_row;
    }
    if (c4 >= p.a.d || (dead && to_partial)) continue;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w = 0; w < WN; ++w) {
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
