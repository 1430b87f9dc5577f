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
      const int row = ti.q_row0 + ti.row0[t];
      const int bq = varlen_q ? 0 : ti.bi;
      if (elect_one()) {
        mbar_arrive_expect_tx(full, kTileBytes);
        tma_load_4d(q_smem + t * kTileBytes, tm_q, full, 0, ti.hh, row, bq);
        tma_load_4d(q_smem + t * kTileBytes + kHalfBytes, tm_q, full, 64, ti.hh, row, bq);
      }
      __syncwarp();
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
        const CUtensorMap* tm = kv == 0 ? tm_k : tm_v;
        if (elect_one()) {
          mbar_arrive_expect_tx(full, kTileBytes);
          tma_load_4d(kv_smem + slot * kTileBytes, tm, full, 0, ti.hk, row, bk);
          tma_load_4d(kv_smem + slot * kTileBytes + kHalfBytes, tm, full, 64, ti.hk, row, bk);
        }
        __syncwarp();
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// MMA issuer of sub-tile t (one warp per sub-tile, one elected lane each).  Per KV block j:
//   S_t = Q_t K_j^T (operands in shared memory),  O_t += P_t V_j (P from TMEM, V from shared memory
//   as an N-contiguous operand).
// Issue order  QK(t,j0) | PV(t,j) QK(t,j+1) | ... : MMAs of one thread execute in issue order, so
// QK(t,j+1) may overwrite the S_t / P_t columns right after PV(t,j) that read them.  Two issuing
// warps keep the tensor pipe fed while the other one is busy with barrier waits and bookkeeping
// (a single thread's instruction latency was measured to leave the pipe idle half of the time).
// A K / V slot is released by two arrivals: one per sub-tile, or both from the only user.
// ---------------------------------------------------------------------------------------------
template <uint32_t AB_FMT>
__device__ __forceinline__ void mma_loop(const Tc5Params& p, Barriers* bar, uint32_t q_smem, uint32_t kv_smem,
                                         uint32_t tmem, const int t) {
  volatile int* abort_flag = &bar->abort_flag;
  constexpr uint32_t idesc_qk = make_idesc(AB_FMT, kBlockM, kBlockN, 0);
  constexpr uint32_t idesc_pv = make_idesc(AB_FMT, kBlockM, 128, 1);
  uint32_t kv_cnt = 0, q_cnt = 0, p_cnt = 0, ofree_cnt = 0, oready_cnt = 0, turn_cnt = 0;
  Tracer tr(p, 3 + t, (threadIdx.x & 31) == 0);
  // The two issuing warps take turns (sub-tile 0, then 1, per KV block) so that the sub-tiles stay
  // half a period apart: one is in its softmax while the tensor pipe works on the other.  Without
  // the token both drift into lockstep and the pipe idles during both softmaxes.
  const uint32_t bar_turn_mine = smem_addr(&bar->mma_turn[t]), bar_turn_other = smem_addr(&bar->mma_turn[1 - t]);
  const uint32_t turn_flip = t == 0 ? 1u : 0u;
  // Descriptor bases are built once; inside the loops a descriptor is base + a small constant.
  const uint64_t q_desc = make_smem_desc(q_smem + t * kTileBytes, 16, 1024);
  const uint64_t k_desc0 = make_smem_desc(kv_smem, 16, 1024);          // K-major operand (K)
  const uint64_t v_desc0 = make_smem_desc(kv_smem, kHalfBytes, 1024);  // N-contiguous operand (V)
  constexpr uint64_t kSlotStep = kTileBytes >> 4;
  // K-major operands: 16 columns per k-step = 32 bytes inside the 128-byte swizzle span
  uint64_t kOff[8], qd[8];
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    kOff[ks] = (uint64_t)(((ks >> 2) * kHalfBytes + (ks & 3) * 32) >> 4);
    qd[ks] = q_desc + kOff[ks];
  }
  const uint32_t s_tmem = tmem + t * 128, o_tmem = tmem + 256 + t * 128;
  const uint32_t bar_pfull0 = smem_addr(&bar->p_full[t][0]), bar_pfull1 = smem_addr(&bar->p_full[t][1]);
  const uint32_t bar_ofree = smem_addr(&bar->o_free[t]), bar_oready = smem_addr(&bar->o_ready[t]);
  const uint32_t bar_odone = smem_addr(&bar->o_done[t]), bar_sfull = smem_addr(&bar->s_full[t]);
  const uint32_t bar_kvfull0 = smem_addr(&bar->kv_full[0]), bar_kvempty0 = smem_addr(&bar->kv_empty[0]);

  for (int n = blockIdx.x; n < p.total_tiles; n += gridDim.x) {
    TileInfo ti;
    tile_info(p, n, ti);
    if (ti.uhi <= ti.ulo) continue;
    const int o = 1 - t;
    if (ti.has[t]) {
      if (!mbar_wait(smem_addr(&bar->q_full[t]), q_cnt & 1, abort_flag)) return;
      ++q_cnt;
    }
    int pend_j = -1;
    uint32_t pend_slot = 0, pend_par = 0;
    bool first_pv = true, have_turn = false;
    auto take_turn = [&]() -> bool {
      if (have_turn) return true;
      have_turn = true;
      return mbar_wait(bar_turn_mine, (turn_cnt & 1) ^ turn_flip, abort_flag);
    };
    auto pass_turn = [&]() {
      if (elect_one()) mbar_arrive(bar_turn_other);
      ++turn_cnt;
      have_turn = false;
    };

    auto issue_pv = [&]() -> bool {
      const int j = pend_j;
      pend_j = -1;
      FA_TR(tr, 20);
      if (first_pv) {  // the previous tile's epilogue must have read O_t
        if (!mbar_wait(bar_ofree, (ofree_cnt & 1) ^ 1, abort_flag)) return false;
        ++ofree_cnt;
      } else {         // the correction warps must have rescaled O_t for this block
        if (!mbar_wait(bar_oready, oready_cnt & 1, abort_flag)) return false;
        ++oready_cnt;
      }
      if (!mbar_wait(bar_kvfull0 + pend_slot * 8, pend_par, abort_flag)) return false;
      const uint64_t v_desc = v_desc0 + pend_slot * kSlotStep;
      uint64_t vd[8];  // all operands of the burst are ready before the last wait
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) vd[ks] = v_desc + (uint64_t)(ks * (2048 >> 4));
      if (!mbar_wait(bar_pfull0, p_cnt & 1, abort_flag)) return false;  // first 64 keys of P
      if (p.tune_wait_full_p && !mbar_wait(bar_pfull1, p_cnt & 1, abort_flag)) return false;
      if (!mbar_wait(bar_turn_mine, (turn_cnt & 1) ^ turn_flip, abort_flag)) return false;
      have_turn = true;
      FA_TR(tr, 24);
      tc_fence_after();
      if (elect_one()) {
        if (first_pv) mma_ts_c<false>(o_tmem, s_tmem, vd[0], idesc_pv);
        else mma_ts_c<true>(o_tmem, s_tmem, vd[0], idesc_pv);
#pragma unroll
        for (int ks = 1; ks < 4; ++ks) mma_ts_c<true>(o_tmem, s_tmem + ks * 8, vd[ks], idesc_pv);
      }
      if (!mbar_wait(bar_pfull1, p_cnt & 1, abort_flag)) return false;  // last 64 keys
      FA_TR(tr, 26);
      tc_fence_after();
      const bool other_v = ti.has[o] && j >= ti.jlo[o] && j < ti.jhi[o];
      if (elect_one()) {
#pragma unroll
        for (int ks = 4; ks < 8; ++ks) mma_ts_c<true>(o_tmem, s_tmem + ks * 8, vd[ks], idesc_pv);
        mma_commit(bar_odone);
        mma_commit(bar_kvempty0 + pend_slot * 8);
        if (!other_v) mma_commit(bar_kvempty0 + pend_slot * 8);
      }
      __syncwarp();
      ++p_cnt;
      first_pv = false;
      return true;
    };

    for (int j = ti.ulo; j < ti.uhi; ++j) {
      const uint32_t kslot = kv_cnt % kSlots, kpar = (kv_cnt / kSlots) & 1;
      ++kv_cnt;
      const uint32_t vslot = kv_cnt % kSlots, vpar = (kv_cnt / kSlots) & 1;
      ++kv_cnt;
      const bool act = ti.has[t] && j >= ti.jlo[t] && j < ti.jhi[t];
      const bool act_o = ti.has[o] && j >= ti.jlo[o] && j < ti.jhi[o];
      if (pend_j >= 0 && !issue_pv()) return;
      if (!act) {
        // blocks only the other sub-tile uses need no arrival from this warp (that warp arrives twice);
        // blocks nobody uses cannot occur (the union of two touching intervals has no hole)
        if (!take_turn()) return;
        pass_turn();
        continue;
      }
      const uint64_t k_desc = k_desc0 + kslot * kSlotStep;
      uint64_t kd[8];
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) kd[ks] = k_desc + kOff[ks];
      if (!mbar_wait(bar_kvfull0 + kslot * 8, kpar, abort_flag)) return;
      if (!take_turn()) return;
      tc_fence_after();
      if (elect_one()) {
        mma_ss_c<false>(s_tmem, qd[0], kd[0], idesc_qk);
#pragma unroll
        for (int ks = 1; ks < 8; ++ks) mma_ss_c<true>(s_tmem, qd[ks], kd[ks], idesc_qk);
        mma_commit(bar_sfull);
        if (j == ti.jhi[t] - 1) mma_commit(smem_addr(&bar->q_empty[t]));
        mma_commit(bar_kvempty0 + kslot * 8);
        if (!act_o) mma_commit(bar_kvempty0 + kslot * 8);
      }
      __syncwarp();
      FA_TR(tr, 30);
      pend_j = j;
      pend_slot = vslot;
      pend_par = vpar;
      pass_turn();
    }
    // flush step
    if (pend_j >= 0 && !issue_pv()) return;
    if (!take_turn()) return;
    pass_turn();
  }
}

}  // namespace tc5
}  // namespace fa
