// The two single-thread roles of the tcgen05 prefill kernel: TMA producer and MMA issuer.
#pragma once

#include "fwd_tc5_kernel.cuh"

namespace fa {
namespace tc5 {

// Both single-thread roles walk the K / V tiles of a CTA tile in the order the tensor pipe needs them:
//   K_lo | K_lo+1 V_lo | K_lo+2 V_lo+1 | ... | V_hi-1
// (Q.K^T of block j+1 is issued before P.V of block j).  Ring slot and parity follow from a running count.
// (Carrying the order across tile boundaries -- Q.K^T of the next tile's first block before P.V of this tile's last
// one -- lets one sub-tile run a block ahead of the other, and then the two need four K / V tiles at a time where the
// ring has three: measured 8 % slower on causal 4K.)
template <int SLOTS>
struct RingPos {
  uint32_t cnt = 0;
  __device__ __forceinline__ void next(uint32_t& slot, uint32_t& par) {
    slot = cnt % SLOTS;
    par = (cnt / SLOTS) & 1;
    ++cnt;
  }
};

// ---------------------------------------------------------------------------------------------
// TMA producer: Q sub-tiles once per CTA tile, then the K / V tiles into the ring.
// Tensor maps are 4-D (d, head, row, batch); a [128 x 128] tile arrives as two 64-column boxes
// (128-byte rows, 128-byte swizzle), each 16 KiB.  A paged cache is (d, head, row in page, page):
// pages hold whole 128-key blocks, the page of a block comes from the block table (the warp keeps
// 32 consecutive entries in registers, one per lane).
// ---------------------------------------------------------------------------------------------
// HD (64 or 128) is the head dim: with 64 a Q / K / V tile is the first 64-column half of its 32 KiB slot only.
template <bool FIX, int HD>
__device__ __forceinline__ void producer_loop(const Tc5Params& p, const CUtensorMap* tm_q, const CUtensorMap* tm_k,
                                              const CUtensorMap* tm_v, Barriers* bar, uint32_t q_smem, uint32_t kv_smem) {
  volatile int* abort_flag = &bar->abort_flag;
  using G = Geo<HD>;
  RingPos<G::kRing> ring;
  uint32_t q_cnt[2] = {0, 0};
  const bool varlen_q = p.a.cu_seqlens_q != nullptr, varlen_k = p.a.cu_seqlens_k != nullptr;
  const int lane = threadIdx.x & 31;
  const uint64_t q_policy = l2_policy_evict_first();  // Q is read once
  const int pages_per_seq = p.a.block_table ? ceil_div(p.a.seqlen_k, p.a.page_size) : 0;  // entries per block-table row
  TileSched sched(p);
  for (int n = sched.first(); n < p.total_tiles; n = sched.next()) {
    TileInfo ti;
    tile_info<G::kRows>(p, n, ti);
    if (ti.uhi <= ti.ulo) continue;
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      if (!ti.has[t]) continue;
      if (!mbar_wait(smem_addr(&bar->q_empty[t]), (q_cnt[t] & 1) ^ 1, abort_flag, 11)) return;
      ++q_cnt[t];
      const uint32_t full = smem_addr(&bar->q_full[t]);
      const int row = ti.q_row0 + ti.row0[t];
      const int bq = varlen_q ? 0 : ti.bi;
      if (elect_one()) {
        mbar_arrive_expect_tx(full, G::kHalves * kHalfBytes);
#pragma unroll
        for (int hf = 0; hf < G::kHalves; ++hf)
          tma_load_4d_hint(q_smem + t * kTileBytes + hf * kHalfBytes, tm_q, full, 64 * hf, ti.hh, row, bq, q_policy);
      }
      __syncwarp();
    }
    const int bk = varlen_k ? 0 : ti.bk;
    if (FIX && lane == 0 && p.a.seqused_k) {  // every role clamps these silently (tile_info); this one reports them
      cache_len(p.a, ti.bi, p.status);
      if (p.a.cache_batch_idx && !p.a.block_table) check_outer_index(p.a, bk, p.status);
    }
    const int32_t* pages = p.a.block_table ? p.a.block_table + (int64_t)ti.bi * p.a.block_table_batch_stride : nullptr;
    int pg_base = -1, pg_reg = 0;  // block-table entries pg_base .. pg_base + 31 of this batch entry, one per lane
    auto load = [&](const CUtensorMap* tm, int j) -> bool {
      uint32_t slot, par;
      ring.next(slot, par);
      int row = ti.k_row0 + j * kBlockN, outer = bk;
      if (pages) {
        const int pg = (j * kBlockN) / p.a.page_size;
        if (pg_base < 0 || pg < pg_base || pg >= pg_base + 32) {
          pg_base = pg;
          const int idx = pg + lane;
          pg_reg = idx < pages_per_seq ? pages[idx] : 0;
        }
        outer = __shfl_sync(0xffffffffu, pg_reg, pg - pg_base);
        if (FIX && lane == 0) check_outer_index(p.a, outer, p.status);  // out of range: the TMA returns zeros
        row = j * kBlockN - pg * p.a.page_size;
      }
      if (!mbar_wait(smem_addr(&bar->kv_empty[slot]), par ^ 1, abort_flag, 12)) return false;
      const uint32_t full = smem_addr(&bar->kv_full[slot]);
      if (elect_one()) {
        mbar_arrive_expect_tx(full, G::kHalves * kHalfBytes);
#pragma unroll
        for (int hf = 0; hf < G::kHalves; ++hf)
          tma_load_4d(kv_smem + slot * G::kSlotBytes + hf * kHalfBytes, tm, full, 64 * hf, ti.hk, row, outer);
      }
      __syncwarp();
      return true;
    };
    if (!load(tm_k, ti.ulo)) return;
    for (int j = ti.ulo; j < ti.uhi; ++j) {
      if (j + 1 < ti.uhi && !load(tm_k, j + 1)) return;
      if (!load(tm_v, j)) return;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Warp 15: the rows of the last V tile that lie behind the last key of the sequence.  For dense input they are
// outside the tensor and arrive as zeros; in a KV cache, a page or a packed tensor they hold whatever is there
// (an uninitialised tail, a recycled page, the next sequence).  The mask makes P exactly 0 for those keys, but
// 0 x NaN = NaN in P.V, so the rows are cleared in shared memory before the tile is used -- what the reference
// gets from copying only the valid rows of a page (csrc/arch22/flash_attn_npu_v2/pv_matmul.hpp:137-142,188-206).
// K needs no repair: a score of a masked key is replaced, whatever it was.
// Hand-shake: the issuing warps arrive on fix_req once the tile has landed (at least one of them uses it and has
// waited for it), this warp clears the rows and arrives on v_fixed, which both issuing warps wait for.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ bool tile_needs_tail_fix(const Tc5Params& p, const TileInfo& ti) {
  return p.fix_tail && ti.uhi > ti.ulo && ti.uhi * kBlockN > ti.k_len;
}

template <int HD>
__device__ __forceinline__ void tail_fix_loop(const Tc5Params& p, Barriers* bar, uint32_t kv_smem, int lane) {
  if (!p.fix_tail) return;
  volatile int* abort_flag = &bar->abort_flag;
  uint32_t fix_cnt = 0;  // tails cleared so far
  TileSched sched(p);
  for (int n = sched.first(); n < p.total_tiles; n = sched.next()) {
    TileInfo ti;
    tile_info<Geo<HD>::kRows>(p, n, ti);
    if (!tile_needs_tail_fix(p, ti)) continue;
    if (!mbar_wait_patient(smem_addr(&bar->fix_req), fix_cnt & 1, abort_flag, 51)) return;
    ++fix_cnt;
    const uint32_t slot = bar->fix_slot;  // written by the issuing warps before they arrived
    const int r0 = ti.k_len - (ti.uhi - 1) * kBlockN;  // first row without a key, 1 .. 127
    // a row is 128 bytes in each 64-column half of the tile (the swizzle only permutes inside a row)
#pragma unroll
    for (int half = 0; half < HD / 64; ++half) {
      const uint32_t base = kv_smem + slot * Geo<HD>::kSlotBytes + half * kHalfBytes;
      for (int off = r0 * 128 + lane * 16; off < kHalfBytes; off += 32 * 16)
        asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};\n" ::"r"(base + off), "r"(0) : "memory");
    }
    fence_proxy_async();  // generic-proxy stores -> visible to the MMA (async proxy)
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_addr(&bar->v_fixed));
  }
}

// ---------------------------------------------------------------------------------------------
// MMA issuer of sub-tile t (one warp per sub-tile, one elected lane each).  Per KV block j:
//   S_t = Q_t K_j^T (both operands in shared memory),
//   O_t += P_t V_j  (P_t from shared memory, V_j as an N-contiguous operand).
// Issue order  QK(j0) | QK(j+1) PV(j) | ... : Q.K^T of the next block only waits for the softmax
// threads to have copied S_t into registers, so it runs under this block's exponentials.
// A K / V slot is released by two arrivals: one per sub-tile, or both from the only user.
// ---------------------------------------------------------------------------------------------
template <uint32_t AB_FMT, bool FIX, int HD>
__device__ __forceinline__ void mma_loop(const Tc5Params& p, Barriers* bar, uint32_t q_smem, uint32_t p_smem,
                                         uint32_t kv_smem, uint32_t tmem, const int t) {
  volatile int* abort_flag = &bar->abort_flag;
  constexpr uint32_t idesc_qk = make_idesc(AB_FMT, kBlockM, kBlockN, 0);
  constexpr uint32_t idesc_pv = make_idesc(AB_FMT, kBlockM, HD, 1);
  using G = Geo<HD>;
  RingPos<G::kRing> ring;
  uint32_t q_cnt = 0, qk_cnt = 0, p_cnt = 0, ofree_cnt = 0, oready_cnt = 0;
  // Descriptor bases are built once; inside the loops a descriptor is base + a small constant.
  const uint64_t q_desc = make_smem_desc(q_smem + t * kTileBytes, 16, 1024);
  const uint64_t p_desc = make_smem_desc(p_smem + t * kTileBytes, 16, 1024);
  const uint64_t k_desc0 = make_smem_desc(kv_smem, 16, 1024);          // K-major operand (K)
  const uint64_t v_desc0 = make_smem_desc(kv_smem, kHalfBytes, 1024);  // N-contiguous operand (V)
  constexpr uint64_t kSlotStep = G::kSlotBytes >> 4;
  // K-major operands: 16 columns per k-step = 32 bytes inside the 128-byte swizzle span
  auto k_off = [](int ks) { return (uint64_t)(((ks >> 2) * kHalfBytes + (ks & 3) * 32) >> 4); };
  const uint32_t s_tmem = tmem + t * 128, o_tmem = tmem + 256 + t * 128;
  const uint32_t bar_pfull0 = smem_addr(&bar->p_full[t][0]), bar_pfull1 = smem_addr(&bar->p_full[t][1]);
  const uint32_t bar_ofree = smem_addr(&bar->o_free[t]), bar_oready = smem_addr(&bar->o_ready[t]);
  const uint32_t bar_odone = smem_addr(&bar->o_done[t]), bar_sfull = smem_addr(&bar->s_full[t]);
  const uint32_t bar_sfree = smem_addr(&bar->s_free[t]);
  const uint32_t bar_kvfull0 = smem_addr(&bar->kv_full[0]), bar_kvempty0 = smem_addr(&bar->kv_empty[0]);
  const int o = 1 - t;

  // Tail of the last V tile of a CTA tile (tail_fix_loop): both issuing warps ask for it and wait for it, also the
  // one that does not use the tile, so that every phase of the two barriers is seen by everybody.  (The phase count
  // lives in shared memory: this warp has 40 registers and needs it once in many tiles.)
  auto tail_fix = [&](uint32_t slot) -> bool {
    const uint32_t n = bar->fix_seen[t];
    __syncwarp();
    if (elect_one()) {
      bar->fix_seen[t] = n + 1;
      bar->fix_slot = slot;  // both warps write the same value
      mbar_arrive(smem_addr(&bar->fix_req));
    }
    __syncwarp();
    return mbar_wait(smem_addr(&bar->v_fixed), n & 1, abort_flag, 22);
  };

  TileSched sched(p);
  for (int n = sched.first(); n < p.total_tiles; n = sched.next()) {
    TileInfo ti;
    tile_info<G::kRows>(p, n, ti);
    if (ti.uhi <= ti.ulo) continue;
    if (ti.has[t]) {
      if (!mbar_wait(smem_addr(&bar->q_full[t]), q_cnt & 1, abort_flag, 13)) return;
      ++q_cnt;
    }
    const int jlo_t = ti.has[t] ? ti.jlo[t] : 0, jhi_t = ti.has[t] ? ti.jhi[t] : 0;
    const int jlo_o = ti.has[o] ? ti.jlo[o] : 0, jhi_o = ti.has[o] ? ti.jhi[o] : 0;
    const int fix_j = (FIX && tile_needs_tail_fix(p, ti)) ? ti.uhi - 1 : -1;  // the block whose V tile needs its tail cleared

    // S_t = Q_t K_j^T.  Tiles only the other sub-tile uses need no arrival from this warp (that warp
    // arrives twice); tiles nobody uses cannot occur (the union of two touching intervals has no hole).
    auto issue_qk = [&](int j) -> bool {
      uint32_t slot, par;
      ring.next(slot, par);
      if (j < jlo_t || j >= jhi_t) return true;
      const uint64_t k_desc = k_desc0 + slot * kSlotStep;
      if (!mbar_wait(bar_kvfull0 + slot * 8, par, abort_flag, 14)) return false;
      // the softmax threads must have copied the previous S_t out of TMEM
      if (qk_cnt > 0 && !mbar_wait(bar_sfree, (qk_cnt - 1) & 1, abort_flag, 15)) return false;
      ++qk_cnt;
      tc_fence_after();
      const bool other = j >= jlo_o && j < jhi_o;
      if (elect_one()) {
        mma_ss_c<false>(s_tmem, q_desc, k_desc, idesc_qk);
#pragma unroll
        for (int ks = 1; ks < HD / 16; ++ks) mma_ss_c<true>(s_tmem, q_desc + k_off(ks), k_desc + k_off(ks), idesc_qk);
        mma_commit(bar_sfull);
        if (j == jhi_t - 1) mma_commit(smem_addr(&bar->q_empty[t]));
        mma_commit(bar_kvempty0 + slot * 8);
        if (!other) mma_commit(bar_kvempty0 + slot * 8);
      }
      __syncwarp();
      return true;
    };

    // O_t (+)= P_t V_j, in two halves of 64 keys so that the first starts while the softmax threads
    // still work on the second.
    auto issue_pv = [&](int j) -> bool {
      uint32_t slot, par;
      ring.next(slot, par);
      if (j < jlo_t || j >= jhi_t) return !FIX || j != fix_j || tail_fix(slot);
      const bool first_pv = j == jlo_t;
      if (first_pv) {  // the previous tile's epilogue must have read O_t
        if (!mbar_wait(bar_ofree, (ofree_cnt & 1) ^ 1, abort_flag, 16)) return false;
        ++ofree_cnt;
      } else {         // the correction warps must have rescaled O_t for this block
        if (!mbar_wait(bar_oready, oready_cnt & 1, abort_flag, 17)) return false;
        ++oready_cnt;
      }
      if (!mbar_wait(bar_kvfull0 + slot * 8, par, abort_flag, 18)) return false;
      if (FIX && j == fix_j && !tail_fix(slot)) return false;
      const uint64_t v_desc = v_desc0 + slot * kSlotStep;
      if (!mbar_wait(bar_pfull0, p_cnt & 1, abort_flag, 19)) return false;  // first 64 keys of P
      tc_fence_after();
      if (elect_one()) {
        if (first_pv) mma_ss_c<false>(o_tmem, p_desc, v_desc, idesc_pv);
        else mma_ss_c<true>(o_tmem, p_desc, v_desc, idesc_pv);
#pragma unroll
        for (int ks = 1; ks < 4; ++ks) mma_ss_c<true>(o_tmem, p_desc + k_off(ks), v_desc + (uint64_t)(ks * (2048 >> 4)), idesc_pv);
      }
      if (!mbar_wait(bar_pfull1, p_cnt & 1, abort_flag, 20)) return false;  // last 64 keys
      tc_fence_after();
      const bool other = j >= jlo_o && j < jhi_o;
      if (elect_one()) {
#pragma unroll
        for (int ks = 4; ks < 8; ++ks) mma_ss_c<true>(o_tmem, p_desc + k_off(ks), v_desc + (uint64_t)(ks * (2048 >> 4)), idesc_pv);
        mma_commit(bar_odone);
        mma_commit(bar_kvempty0 + slot * 8);
        if (!other) mma_commit(bar_kvempty0 + slot * 8);
      }
      __syncwarp();
      ++p_cnt;
      return true;
    };

    if (!issue_qk(ti.ulo)) return;
    for (int j = ti.ulo; j < ti.uhi; ++j) {
      if (j + 1 < ti.uhi && !issue_qk(j + 1)) return;
      if (!issue_pv(j)) return;
    }
  }
}

}  // namespace tc5
}  // namespace fa
