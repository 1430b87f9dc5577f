// The two single-thread roles of the tcgen05 prefill kernel: TMA producer and MMA issuer.
#pragma once

#include "fwd_tc5_kernel.cuh"

namespace fa {
namespace tc5 {

// ---------------------------------------------------------------------------------------------
// TMA producer: Q sub-tiles once per CTA tile, then K_j, V_j, K_j+1, V_j+1 ... into the ring.
// Tensor maps are 4-D (d, head, row, batch); a [128 x 128] tile arrives as two 64-column boxes
// (128-byte rows, 128-byte swizzle), each 16 KiB.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void producer_loop(const Tc5Params& p, const CUtensorMap* tm_q, const CUtensorMap* tm_k,
                                              const CUtensorMap* tm_v, Barriers* bar, uint32_t q_smem, uint32_t kv_smem) {
  volatile int* abort_flag = &bar->abort_flag;
  uint32_t kv_cnt = 0, q_cnt[2] = {0, 0};
  const bool varlen_q = p.a.cu_seqlens_q != nullptr, varlen_k = p.a.cu_seqlens_k != nullptr;
  for (int n = blockIdx.x; n < p.total_tiles; n += gridDim.x) {
    TileInfo ti;
    tile_info(p, n, ti);
    if (ti.uhi <= ti.ulo) continue;
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      if (!ti.has[t]) continue;
      if (!mbar_wait(smem_addr(&bar->q_empty[t]), (q_cnt[t] & 1) ^ 1, abort_flag)) return;
      ++q_cnt[t];
      const uint32_t full = smem_addr(&bar->q_full[t]);
      mbar_arrive_expect_tx(full, kTileBytes);
      const int row = ti.q_row0 + ti.row0[t];
      const int bq = varlen_q ? 0 : ti.bi;
      tma_load_4d(q_smem + t * kTileBytes, tm_q, full, 0, ti.hh, row, bq);
      tma_load_4d(q_smem + t * kTileBytes + kHalfBytes, tm_q, full, 64, ti.hh, row, bq);
    }
    const int bk = varlen_k ? 0 : ti.bi;
    for (int j = ti.ulo; j < ti.uhi; ++j) {
      const int row = ti.k_row0 + j * kBlockN;
#pragma unroll
      for (int kv = 0; kv < 2; ++kv) {
        const uint32_t slot = kv_cnt % kSlots, par = ((kv_cnt / kSlots) & 1) ^ 1;
        ++kv_cnt;
        if (!mbar_wait(smem_addr(&bar->kv_empty[slot]), par, abort_flag)) return;
        const uint32_t full = smem_addr(&bar->kv_full[slot]);
        mbar_arrive_expect_tx(full, kTileBytes);
        const CUtensorMap* tm = kv == 0 ? tm_k : tm_v;
        tma_load_4d(kv_smem + slot * kTileBytes, tm, full, 0, ti.hk, row, bk);
        tma_load_4d(kv_smem + slot * kTileBytes + kHalfBytes, tm, full, 64, ti.hk, row, bk);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// MMA issuer.  Per KV block j and sub-tile t:  S_t = Q_t K_j^T (operands in shared memory),
// O_t += P_t V_j (P from TMEM, V from shared memory as an N-contiguous operand).
// Issue order  QK(0,j0) QK(1,j0) | PV(0,j) QK(0,j+1) | PV(1,j) QK(1,j+1) | ...  : MMAs of one
// thread execute in issue order, so QK(t,j+1) may overwrite the S_t / P_t columns right after
// PV(t,j) that read them.
// ---------------------------------------------------------------------------------------------
template <uint32_t AB_FMT>
__device__ __forceinline__ void mma_loop(const Tc5Params& p, Barriers* bar, uint32_t q_smem, uint32_t kv_smem,
                                         uint32_t tmem) {
  volatile int* abort_flag = &bar->abort_flag;
  constexpr uint32_t idesc_qk = make_idesc(AB_FMT, kBlockM, kBlockN, 0);
  constexpr uint32_t idesc_pv = make_idesc(AB_FMT, kBlockM, 128, 1);
  uint32_t kv_cnt = 0, q_cnt[2] = {0, 0}, p_cnt[2] = {0, 0}, ofree_cnt[2] = {0, 0}, oready_cnt[2] = {0, 0};

  for (int n = blockIdx.x; n < p.total_tiles; n += gridDim.x) {
    TileInfo ti;
    tile_info(p, n, ti);
    if (ti.uhi <= ti.ulo) continue;
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      if (!ti.has[t]) continue;
      if (!mbar_wait(smem_addr(&bar->q_full[t]), q_cnt[t] & 1, abort_flag)) return;
      ++q_cnt[t];
    }
    int pend_j[2] = {-1, -1};
    uint32_t pend_slot[2] = {0, 0}, pend_par[2] = {0, 0};
    bool first_pv[2] = {true, true};

    auto issue_pv = [&](int t) -> bool {
      const int j = pend_j[t];
      pend_j[t] = -1;
      if (first_pv[t]) {  // the previous tile's epilogue must have read O_t
        if (!mbar_wait(smem_addr(&bar->o_free[t]), (ofree_cnt[t] & 1) ^ 1, abort_flag)) return false;
        ++ofree_cnt[t];
      } else {            // the correction warps must have rescaled O_t for this block
        if (!mbar_wait(smem_addr(&bar->o_ready[t]), oready_cnt[t] & 1, abort_flag)) return false;
        ++oready_cnt[t];
      }
      if (!mbar_wait(smem_addr(&bar->kv_full[pend_slot[t]]), pend_par[t], abort_flag)) return false;
      const uint32_t v_base = kv_smem + pend_slot[t] * kTileBytes;
      const uint32_t d_tmem = tmem + 256 + t * 128;
      const uint32_t a_tmem = tmem + t * 128;
#pragma unroll
      for (int half = 0; half < 2; ++half) {  // P arrives in two halves of 64 keys
        if (!mbar_wait(smem_addr(&bar->p_full[t][half]), p_cnt[t] & 1, abort_flag)) return false;
        tc_fence_after();
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4) {
          const int ks = half * 4 + k4;
          // V tile: [half][128 keys][64 cols]: 16 keys per step = 2 KiB; N chunks of 64 columns 16 KiB apart
          const uint64_t b_desc = make_smem_desc(v_base + ks * 2048, kHalfBytes, 1024);
          mma_ts(d_tmem, a_tmem + ks * 8, b_desc, idesc_pv, (first_pv[t] && ks == 0) ? 0u : 1u);
        }
      }
      ++p_cnt[t];
      first_pv[t] = false;
      mma_commit(smem_addr(&bar->o_done[t]));
      const bool other_uses = (t == 0) && ti.has[1] && j >= ti.jlo[1] && j < ti.jhi[1];
      if (!other_uses) mma_commit(smem_addr(&bar->kv_empty[pend_slot[t]]));
      return true;
    };

    for (int j = ti.ulo; j < ti.uhi; ++j) {
      const uint32_t kslot = kv_cnt % kSlots, kpar = (kv_cnt / kSlots) & 1;
      ++kv_cnt;
      const uint32_t vslot = kv_cnt % kSlots, vpar = (kv_cnt / kSlots) & 1;
      ++kv_cnt;
      const bool act0 = ti.has[0] && j >= ti.jlo[0] && j < ti.jhi[0];
      const bool act1 = ti.has[1] && j >= ti.jlo[1] && j < ti.jhi[1];
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        if (pend_j[t] >= 0 && !issue_pv(t)) return;
        const bool act = t == 0 ? act0 : act1;
        if (!act) continue;
        if (!mbar_wait(smem_addr(&bar->kv_full[kslot]), kpar, abort_flag)) return;
        tc_fence_after();
        const uint32_t q_base = q_smem + t * kTileBytes, k_base = kv_smem + kslot * kTileBytes;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          // K-major operands: 16 columns per step = 32 bytes inside the 128-byte swizzle span
          const uint32_t off = (ks >> 2) * kHalfBytes + (ks & 3) * 32;
          mma_ss(tmem + t * 128, make_smem_desc(q_base + off, 16, 1024), make_smem_desc(k_base + off, 16, 1024),
                 idesc_qk, ks > 0 ? 1u : 0u);
        }
        mma_commit(smem_addr(&bar->s_full[t]));
        if (j == ti.jhi[t] - 1) mma_commit(smem_addr(&bar->q_empty[t]));
        if (t == 1 || !act1) mma_commit(smem_addr(&bar->kv_empty[kslot]));
        pend_j[t] = j;
        pend_slot[t] = vslot;
        pend_par[t] = vpar;
      }
      if (!act0 && !act1) {  // cannot happen for a union range of two intervals that touch; keep the ring consistent
        mma_commit(smem_addr(&bar->kv_empty[kslot]));
        mma_commit(smem_addr(&bar->kv_empty[vslot]));
      }
    }
#pragma unroll
    for (int t = 0; t < 2; ++t)
      if (pend_j[t] >= 0 && !issue_pv(t)) return;
  }
}

}  // namespace tc5
}  // namespace fa
