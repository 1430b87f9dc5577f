// Body of the producer / consumer split-KV decode kernel (overview in fwd_decode.cuh).
#pragma once

#include "fwd_decode.cuh"

namespace fa {

// A CTA works through a list of segments: (batch entry, packed head group, KV block range).
struct DecSeg {
  int bi, hh, my_lo, cnt, slot, fill_from, first, force_mask;
  int valid;  // 0: no more work; 1: run; 2: nothing to run here (only the fixed part of a unit), take the next
};
// Cursor of the persistent mode (see dec_walk_first).
struct DecWalk {
  int bi, hh, nb_lo, nb_hi, n_b, quota, cur, g1, ustart;
};

template <class Tr>
__global__ void __launch_bounds__(Tr::NTHREADS, Tr::MIN_CTAS)
fwd_decode_kernel(const __grid_constant__ KParams p, const __grid_constant__ CUtensorMap tm_k,
                  const __grid_constant__ CUtensorMap tm_v) {
  using T = typename Tr::T;
  constexpr int MT = Tr::MT, NT = Tr::NT, DT = Tr::DT, KS = Tr::KS, BN = Tr::BN, BM = Tr::BM, ST = Tr::ST;
  constexpr int NCW = Tr::NCW, WN = Tr::WN, PITCH = Tr::PITCH, NCT = Tr::NCW * 32;
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ float s_lse[Tr::BM];
  __shared__ int s_abort;
  __shared__ DecSeg s_seg;
  __shared__ DecWalk s_walk;

  // A merge kernel queued behind this one may start launching its CTAs now (they wait for this grid to complete).
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g8 = lane >> 2, t4 = lane & 3;
  const int wm = (warp < Tr::NCW) ? warp / Tr::WN : 0;  // row group of a consumer warp

  // Mask state is the same for every unit of the launch.
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

  // KV block range [nb_lo, nb_hi) that the queries of batch entry bi can see (all heads alike).
  auto batch_range = [&](int bi, int q_len, int& nb_lo, int& nb_hi) {
    const int l_cache = p.a.seqused_k ? cache_len(p.a, bi, p.status) : p.a.seqlen_k;
    const int k_len = l_cache + p.a.seqlen_new;
    const int koff = (p.a.kv_total > 0 ? p.a.kv_total - p.a.kv_pos_offset : k_len) - q_len;
    const int i_max = q_len - 1;
    int j_lo = 0, j_hi = k_len;
    if (is_causal) j_hi = min(k_len, i_max + koff + 1);
    if (is_local) {
      j_hi = min(k_len, i_max + koff + wr + 1);
      j_lo = max(0, koff - wl);
    }
    nb_lo = j_lo / BN;
    nb_hi = j_hi > j_lo ? ceil_div(j_hi, BN) : nb_lo;
  };

  // ---- which segments this CTA runs ----
  // One tile per CTA (same enumeration as fwd_mma_kernel; m_blocks == 1 here), or persistent CTAs
  // with equal shares of the work of the whole launch.  Persistent mode: a unit (batch entry, head
  // group) costs its KV blocks plus a fixed part (Q load, merge of the consumer warps, partial store:
  // a few microseconds, measured) worth kOvh blocks; units are laid end to end, the fixed part as kOvh
  // virtual blocks in front of the real ones (a unit without visible keys counts one fully masked
  // block, so that its rows are written); CTA c takes virtual blocks [c * quota, (c + 1) * quota).
  // A unit cut by CTA boundaries leaves one partial per CTA in consecutive slots; the merge kernel
  // finishes it.  quota is raised when the longest unit would otherwise need more slots than there are.
  // The producer warp and the consumer warps walk the same list independently: the producer is
  // never held back by the consumers' merge and output phase, only by the ring.
  constexpr int kOvh = 512 / BN;
  const int nbat = p.a.b, he = p.heads_eff;
  // next segment off the cursor (persistent mode; no collective operation inside)
  auto walk_next = [&](DecWalk& w, DecSeg& sg) {
    if (!p.persistent || w.cur >= w.g1 || w.bi >= nbat) {
      sg.valid = 0;
      return;
    }
    // [seg_lo, seg_hi): this CTA's part of the unit in virtual blocks; real blocks start at kOvh
    const int seg_lo = w.cur - w.ustart, seg_hi = min(w.n_b, w.g1 - w.ustart);
    const int lo = max(seg_lo - kOvh, 0), hi = max(seg_hi - kOvh, 0);
    const int first_cta = (w.ustart + kOvh) / w.quota;  // the CTA that holds the first real block
    const bool first = lo == 0 && hi > 0;
    sg = DecSeg{w.bi, w.hh, w.nb_lo + lo, hi - lo, (int)blockIdx.x - first_cta,
                first ? (w.ustart + w.n_b - 1) / w.quota - first_cta + 1 : p.num_splits, first, w.nb_hi <= w.nb_lo,
                hi > lo ? 1 : 2};
    w.cur = w.ustart + seg_hi;
    if (seg_hi == w.n_b) {  // the cursor moves on to the next unit
      w.ustart += w.n_b;
      if (++w.hh == he) {
        w.hh = 0;
        if (++w.bi < nbat) {
          batch_range(w.bi, p.a.seqlen_q, w.nb_lo, w.nb_hi);
          w.n_b = max(1, w.nb_hi - w.nb_lo) + kOvh;
        }
      }
    }
  };

  // warp-collective: first segment of this CTA (and the cursor, persistent mode)
  auto walk_first = [&](DecWalk& w, DecSeg& sg) {
    w = DecWalk{0, 0, 0, 0, 1, 1, 0, 0, 0};
    if (!p.persistent) {
      int idx = blockIdx.x;
      const int hh = idx % he;
      idx /= he;
      const int split = idx % p.num_splits;
      const int bi = (idx / p.num_splits) % nbat;
      int q_len = p.a.seqlen_q;
      if (p.a.cu_seqlens_q) q_len = p.a.cu_seqlens_q[bi + 1] - p.a.cu_seqlens_q[bi];
      int nb_lo, nb_hi;
      batch_range(bi, q_len, nb_lo, nb_hi);
      if (p.num_splits > 1) {
        const int lo = nb_lo + split * p.blocks_per_split;
        nb_hi = min(nb_hi, lo + p.blocks_per_split);
        nb_lo = lo;
      }
      sg = DecSeg{bi, hh, nb_lo, max(0, nb_hi - nb_lo), split, p.num_splits, split == 0, 0, 1};
      return;
    }
    int total = 0, n_max = 1;
    for (int b0 = 0; b0 < nbat; b0 += 32) {
      int n = 0;
      if (b0 + lane < nbat) {
        int lo, hi;
        batch_range(b0 + lane, p.a.seqlen_q, lo, hi);
        n = max(1, hi - lo) + kOvh;
      }
      int mx = n, sm = n;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        sm += __shfl_xor_sync(0xffffffffu, sm, o);
      }
      n_max = max(n_max, mx);
      total += sm * he;
    }
    w.quota = max(ceil_div(total, (int)gridDim.x), ceil_div(n_max - kOvh, p.num_splits - 1));
    w.cur = (int)blockIdx.x * w.quota;
    w.g1 = min(total, w.cur + w.quota);
    w.bi = nbat;
    if (w.cur < w.g1) {
      // the batch entry that holds virtual block `cur`: prefix sums 32 entries at a time (a serial
      // walk paid one global-memory latency per entry)
      for (int b0 = 0; b0 < nbat && w.bi == nbat; b0 += 32) {
        int lo = 0, hi = 0, n = 0;
        if (b0 + lane < nbat) {
          batch_range(b0 + lane, p.a.seqlen_q, lo, hi);
          n = max(1, hi - lo) + kOvh;
        }
        int incl = n * he;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int y = __shfl_up_sync(0xffffffffu, incl, o);
          if (lane >= o) incl += y;
        }
        const unsigned hit = __ballot_sync(0xffffffffu, b0 + lane < nbat && w.ustart + incl > w.cur);
        if (hit) {
          const int src = __ffs(hit) - 1;
          w.bi = b0 + src;
          w.ustart += __shfl_sync(0xffffffffu, incl - n * he, src);
          w.nb_lo = __shfl_sync(0xffffffffu, lo, src);
          w.nb_hi = __shfl_sync(0xffffffffu, hi, src);
          w.n_b = __shfl_sync(0xffffffffu, n, src);
        } else {
          w.ustart += __shfl_sync(0xffffffffu, incl, 31);
        }
      }
      w.hh = (w.cur - w.ustart) / w.n_b;
      w.ustart += w.hh * w.n_b;
    }
    walk_next(w, sg);
  };
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
  if (warp == NCW && lane == 0) { tc5::tma_prefetch_desc(&tm_k); tc5::tma_prefetch_desc(&tm_v); }
  __syncthreads();  // barriers initialised; from here the producer warp runs ahead of the consumers

  // what both roles need of a unit
  auto seq_view = [&](int bi, int hh, SeqView<T>& sv, int& hk, int& batch_row) {
    hk = (hh * p.gp) / p.group;
    batch_row = 0;
    int q_row0 = 0;
    sv.q_len = p.a.seqlen_q;
    if (p.a.cu_seqlens_q) {
      q_row0 = p.a.cu_seqlens_q[bi];
      sv.q_len = p.a.cu_seqlens_q[bi + 1] - q_row0;
    }
    sv.q_row0 = q_row0;
    sv.q = reinterpret_cast<const T*>(p.a.q) + (int64_t)bi * p.a.q_batch_stride + (int64_t)q_row0 * p.a.q_row_stride;
    sv.l_cache = p.a.seqused_k ? cache_len(p.a, bi, p.status) : p.a.seqlen_k;
    sv.k_len = sv.l_cache + p.a.seqlen_new;
    const T* kb = reinterpret_cast<const T*>(p.a.k) + (int64_t)hk * p.a.k_head_stride;
    const T* vb = reinterpret_cast<const T*>(p.a.v) + (int64_t)hk * p.a.v_head_stride;
    sv.pages = nullptr;
    if (p.a.block_table) {
      sv.pages = p.a.block_table + (int64_t)bi * p.a.block_table_batch_stride;
    } else {
      batch_row = p.a.cache_batch_idx ? outer_index(p.a, p.a.cache_batch_idx[bi], p.status) : bi;
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
  };

  if (warp == NCW) {
    // ================= producer warp =================
    DecWalk w;
    DecSeg sg;
    walk_first(w, sg);
    uint32_t it_base = 0;  // stages filled so far: ring position and barrier parity
    while (sg.valid) {
      if (sg.valid == 1) {
        SeqView<T> sv;
        int hk, batch_row;
        seq_view(sg.bi, sg.hh, sv, hk, batch_row);
        if (sv.q_len * p.gp > 0) {
          if (!decode_producer<Tr>(p, sv, &tm_k, &tm_v, pipe_base, full0, empty0, sg.my_lo, sg.cnt, it_base, hk, batch_row,
                                   &s_abort))
            break;
          it_base += (uint32_t)sg.cnt;
        }
      }
      walk_next(w, sg);
    }
  } else {
    // ================= consumer warps =================
    if (warp == 0) {
      DecWalk w;
      DecSeg sg;
      walk_first(w, sg);
      if (lane == 0) { s_walk = w; s_seg = sg; }
    }
    uint32_t it_base = 0;  // stages consumed so far
    for (;;) {
      asm volatile("bar.sync 1, %0;\n" ::"n"(NCT));  // the segment descriptor is published
      const DecSeg sg = s_seg;
      asm volatile("bar.sync 1, %0;\n" ::"n"(NCT));  // ... and read by everybody: thread 0 may replace it
      if (!sg.valid || s_abort) break;
      if (sg.valid == 1) {
        const int bi = sg.bi, hh = sg.hh, my_lo = sg.my_lo, n_blocks = sg.cnt, split = sg.slot, fill_from = sg.fill_from;
        const bool to_partial = p.persistent || p.num_splits > 1, force_mask = sg.force_mask != 0;
        SeqView<T> sv;
        int hk, batch_row;
        seq_view(bi, hh, sv, hk, batch_row);
        const int rows_total = sv.q_len * p.gp;
        if (sv.knew && sg.first && (hh * p.gp) % p.group == 0) append_to_cache<Tr>(p, sv, tid, NCT);
        if (rows_total > 0) {
          const int koff = (p.a.kv_total > 0 ? p.a.kv_total - p.a.kv_pos_offset : sv.k_len) - sv.q_len;
          const int i_max = (rows_total - 1) / p.gp;
          // ---- Q tile -> shared memory (rotated when rotary tables are given); padded rows, no swizzle.
          //      The producer is already fetching the first K / V stages. ----
          {
            const bool rot_per_token = is_causal || is_local;
            for (int c = tid; c < BM * Tr::CHUNKS; c += NCT) {
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
            asm volatile("bar.sync 1, %0;\n" ::"n"(NCT));
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
            const uint32_t git = it_base + (uint32_t)it;  // stages this CTA has consumed so far: ring position and parity
            const int stage = (int)(git % ST);
            if (!tc5::mbar_wait(full0 + stage * 8, (git / ST) & 1, &s_abort)) break;
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

            bool need_mask = has_alibi || (nb * BN + BN > sv.k_len) || (BM > rows_total) || force_mask;
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
          it_base += (uint32_t)n_blocks;

          // ---- merge of the WN key slices and output (consumer warps only; the slab is not part of the ring) ----
          float* slab = reinterpret_cast<float*>(smem_al + Tr::SLAB_OFF);
          float2* ml = reinterpret_cast<float2*>(smem_al + Tr::MAIN_BYTES + Tr::Q_BYTES);
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
          asm volatile("bar.sync 1, %0;\n" ::"n"(NCT));
          float f_row[MT][2];
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
              f_row[mt][hf] = (l_all > 0.f) ? fast_exp2(m_run[mt][hf] - m_use) / l_all : 0.f;
              if (wn == 0 && t4 == 0) s_lse[trow] = (l_all > 0.f) ? (m_use + log2f(l_all)) * kLn2 : -INFINITY;
            }
          // slice 0 stores, slices 1 .. WN-1 add in turn: a fixed order, so the result does not depend on timing
#pragma unroll 1
          for (int turn = 0; turn < WN; ++turn) {
            if (wn == turn) {
#pragma unroll
              for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                  const int trow = (wm * MT + mt) * 16 + g8 + 8 * hf;
                  float* dst = slab + (size_t)trow * Tr::SLAB_LD;
                  const float f = f_row[mt][hf];
#pragma unroll
                  for (int dt = 0; dt < DT; ++dt) {
                    float2* q2 = reinterpret_cast<float2*>(dst + dt * 8 + 2 * t4);
                    float2 v = make_float2(o_acc[mt][dt][hf * 2] * f, o_acc[mt][dt][hf * 2 + 1] * f);
                    if (turn > 0) {
                      const float2 old = *q2;
                      v.x += old.x;
                      v.y += old.y;
                    }
                    *q2 = v;
                  }
                }
            }
            asm volatile("bar.sync 1, %0;\n" ::"n"(NCT));
          }

          const bool f32_out = to_partial || p.a.partial_out;
          for (int c = tid; c < BM * (Tr::HD / 4); c += NCT) {
            const int trow = c / (Tr::HD / 4), c4 = (c % (Tr::HD / 4)) * 4;
            if (trow >= rows_total) continue;
            const int i = trow / p.gp, head = hh * p.gp + (trow - i * p.gp);
            const int64_t lse_idx = (int64_t)bi * p.a.lse_batch_stride + (int64_t)head * p.a.lse_head_stride + sv.q_row0 + i;
            const float lse_row = s_lse[trow];
            const bool dead = lse_row == -INFINITY;
            if (c4 == 0) {
              if (to_partial) {
                p.lse_partial[(int64_t)split * p.lse_elems + lse_idx] = lse_row;
                for (int sl = fill_from; sl < p.num_splits; ++sl) p.lse_partial[(int64_t)sl * p.lse_elems + lse_idx] = -INFINITY;
              } else {
                p.a.lse[lse_idx] = (dead && !p.a.partial_out) ? INFINITY : lse_row;
              }
            }
            if (c4 >= p.a.d || (dead && to_partial)) continue;
            const float4 acc = *reinterpret_cast<const float4*>(slab + (size_t)trow * Tr::SLAB_LD + c4);
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
      }
      if (!p.persistent) break;
      if (tid == 0) {
        DecWalk w = s_walk;
        DecSeg nx;
        walk_next(w, nx);
        s_walk = w;
        s_seg = nx;
      }
    }
  }

  __syncthreads();
  if (s_abort) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);  // let copies in flight land before the CTA retires
    if (tid == 0 && p.status) atomicExch(p.status, 0x40000000 | (int)blockIdx.x);
  }
}

}  // namespace fa
