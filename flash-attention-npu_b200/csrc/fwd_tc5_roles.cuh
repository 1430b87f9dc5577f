// The two single-thread roles of the tcgen05 prefill kernel: TMA producer and MMA issuer.
#pragma once

#include "fwd_tc5_kernel.cuh"

namespace fa {
namespace tc5 {

// Both roles walk the K / V tiles of a CTA tile in the order the tensor pipe needs them:
//   K_lo | K_lo+1 V_lo | K_lo+2 V_lo+1 | ... | V_hi-1
// (Q.K^T of block j+1 is issued before P.V of block j).  Ring slot and parity follow from a running count.
struct RingPos {
  uint32_t cnt = 0;
  __device__ __forceinline__ void next(uint32_t& slot, uint32_t& par) {
    slot = cnt % kSlots;
    par = (cnt / kSlots) & 1;
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
__device__ __forceinline__ void producer_loop(const Tc5Params& p, const CUtensorMap* tm_q, const CUtensorMap* tm_k,
                                              const CUtensorMap* tm_v, Barriers* bar, uint32_t q_smem, uint32_t kv_smem) {
  volatile int* abort_flag = &bar->abort_flag;
  RingPos ring;
  Tracer tr(p, 5, (threadIdx.x & 31) == 0);
  uint32_t q_cnt[2] = {0, 0};
  const bool varlen_q = p.a.cu_seqlens_q != nullptr, varlen_k = p.a.cu_seqlens_k != nullptr;
  const int lane = threadIdx.x & 31;
  const uint64_t q_policy = l2_policy_evict_first();  // Q is read once
  const int pages_per_seq = p.a.block_table ? ceil_div(p.a.seqlen_k, p.a.page_size) : 0;  // entries per block-table row
  TileSched sched(p);
  for (int n = sched.first(); n < p.total_tiles; n = sched.next()) {
    TileInfo ti;
    tile_info(p, n, ti);
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
        mbar_arrive_expect_tx(full, kTileBytes);
        tma_load_4d_hint(q_smem + t * kTileBytes, tm_q, full, 0, ti.hh, row, bq, q_policy);
        tma_load_4d_hint(q_smem + t * kTileBytes + kHalfBytes, tm_q, full, 64, ti.hh, row, bq, q_policy);
      }
      __syncwarp();
      FA_TR(tr, 40 + t);
    }
    const int bk = varlen_k ? 0 : ti.bk;
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
        row = j * kBlockN - pg * p.a.page_size;
      }
      if (!mbar_wait(smem_addr(&bar->kv_empty[slot]), par ^ 1, abort_flag, 12)) return false;
      const uint32_t full = smem_addr(&bar->kv_full[slot]);
      if (elect_one()) {
        mbar_arrive_expect_tx(full, kTileBytes);
        tma_load_4d(kv_smem + slot * kTileBytes, tm, full, 0, ti.hk, row, outer);
        tma_load_4d(kv_smem + slot * kTileBytes + kHalfBytes, tm, full, 64, ti.hk, row, outer);
      }
      __syncwarp();
      FA_TR(tr, tm == tm_k ? 42 : 43);
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
// MMA issuer of sub-tile t (one warp per sub-tile, one elected lane each).  Per KV block j:
//   S_t = Q_t K_j^T (both operands in shared memory),
//   O_t += P_t V_j  (P_t from shared memory, V_j as an N-contiguous operand).
// Issue order  QK(j0) | QK(j+1) PV(j) | ... : Q.K^T of the next block only waits for the softmax
// threads to have copied S_t into registers, so it runs under this block's exponentials.
// A K / V slot is released by two arrivals: one per sub-tile, or both from the only user.
// ---------------------------------------------------------------------------------------------
template <uint32_t AB_FMT>
__device__ __forceinline__ void mma_loop(const Tc5Params& p, Barriers* bar, uint32_t q_smem, uint32_t p_smem,
                                         uint32_t kv_smem, uint32_t tmem, const int t) {
  volatile int* abort_flag = &bar->abort_flag;
  constexpr uint32_t idesc_qk = make_idesc(AB_FMT, kBlockM, kBlockN, 0);
  constexpr uint32_t idesc_pv = make_idesc(AB_FMT, kBlockM, 128, 1);
  RingPos ring;
  uint32_t q_cnt = 0, qk_cnt = 0, p_cnt = 0, ofree_cnt = 0, oready_cnt = 0;
  Tracer tr(p, 3 + t, (threadIdx.x & 31) == 0);
  // Descriptor bases are built once; inside the loops a descriptor is base + a small constant.
  const uint64_t q_desc = make_smem_desc(q_smem + t * kTileBytes, 16, 1024);
  const uint64_t p_desc = make_smem_desc(p_smem + t * kTileBytes, 16, 1024);
  const uint64_t k_desc0 = make_smem_desc(kv_smem, 16, 1024);          // K-major operand (K)
  const uint64_t v_desc0 = make_smem_desc(kv_smem, kHalfBytes, 1024);  // N-contiguous operand (V)
  constexpr uint64_t kSlotStep = kTileBytes >> 4;
  // K-major operands: 16 columns per k-step = 32 bytes inside the 128-byte swizzle span
  auto k_off = [](int ks) { return (uint64_t)(((ks >> 2) * kHalfBytes + (ks & 3) * 32) >> 4); };
  const uint32_t s_tmem = tmem + t * 128, o_tmem = tmem + 256 + t * 128;
  const uint32_t bar_pfull0 = smem_addr(&bar->p_full[t][0]), bar_pfull1 = smem_addr(&bar->p_full[t][1]);
  const uint32_t bar_ofree = smem_addr(&bar->o_free[t]), bar_oready = smem_addr(&bar->o_ready[t]);
  const uint32_t bar_odone = smem_addr(&bar->o_done[t]), bar_sfull = smem_addr(&bar->s_full[t]);
  const uint32_t bar_sfree = smem_addr(&bar->s_free[t]);
  const uint32_t bar_kvfull0 = smem_addr(&bar->kv_full[0]), bar_kvempty0 = smem_addr(&bar->kv_empty[0]);
  const int o = 1 - t;

  TileSched sched(p);
  for (int n = sched.first(); n < p.total_tiles; n = sched.next()) {
    TileInfo ti;
    tile_info(p, n, ti);
    if (ti.uhi <= ti.ulo) continue;
    if (ti.has[t]) {
      if (!mbar_wait(smem_addr(&bar->q_full[t]), q_cnt & 1, abort_flag, 13)) return;
      ++q_cnt;
    }
    const int jlo_t = ti.has[t] ? ti.jlo[t] : 0, jhi_t = ti.has[t] ? ti.jhi[t] : 0;
    const int jlo_o = ti.has[o] ? ti.jlo[o] : 0, jhi_o = ti.has[o] ? ti.jhi[o] : 0;

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
        for (int ks = 1; ks < 8; ++ks) mma_ss_c<true>(s_tmem, q_desc + k_off(ks), k_desc + k_off(ks), idesc_qk);
        mma_commit(bar_sfull);
        if (j == jhi_t - 1) mma_commit(smem_addr(&bar->q_empty[t]));
        mma_commit(bar_kvempty0 + slot * 8);
        if (!other) mma_commit(bar_kvempty0 + slot * 8);
      }
      __syncwarp();
      FA_TR(tr, 30);
      return true;
    };

    // O_t (+)= P_t V_j, in two halves of 64 keys so that the first starts while the softmax threads
    // still work on the second.
    auto issue_pv = [&](int j) -> bool {
      uint32_t slot, par;
      ring.next(slot, par);
      if (j < jlo_t || j >= jhi_t) return true;
      FA_TR(tr, 20);
      const bool first_pv = j == jlo_t;
      if (first_pv) {  // the previous tile's epilogue must have read O_t
        if (!mbar_wait(bar_ofree, (ofree_cnt & 1) ^ 1, abort_flag, 16)) return false;
        ++ofree_cnt;
      } else {         // the correction warps must have rescaled O_t for this block
        if (!mbar_wait(bar_oready, oready_cnt & 1, abort_flag, 17)) return false;
        ++oready_cnt;
      }
      if (!mbar_wait(bar_kvfull0 + slot * 8, par, abort_flag, 18)) return false;
      const uint64_t v_desc = v_desc0 + slot * kSlotStep;
      if (!mbar_wait(bar_pfull0, p_cnt & 1, abort_flag, 19)) return false;  // first 64 keys of P
      FA_TR(tr, 24);
      tc_fence_after();
      if (elect_one()) {
        if (first_pv) mma_ss_c<false>(o_tmem, p_desc, v_desc, idesc_pv);
        else mma_ss_c<true>(o_tmem, p_desc, v_desc, idesc_pv);
#pragma unroll
        for (int ks = 1; ks < 4; ++ks) mma_ss_c<true>(o_tmem, p_desc + k_off(ks), v_desc + (uint64_t)(ks * (2048 >> 4)), idesc_pv);
      }
      if (!mbar_wait(bar_pfull1, p_cnt & 1, abort_flag, 20)) return false;  // last 64 keys
      FA_TR(tr, 26);
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
      FA_TR(tr, 28);
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
