// Split-KV decode kernel with a dedicated producer warp (HBM-bound path).
//
// Same arithmetic and tile / split scheme as fwd_mma_kernel (see fwd_mma.cuh), restructured so
// that the streaming of K / V never competes with the math for issue slots:
//   * one producer warp moves a whole stage (BN keys of K and of V) with four tiled TMA loads
//     (a first version issued one bulk copy per 256-byte row: the per-copy issue rate, about one
//     per 60 cycles per SM, capped it at 1.1 TB/s).  Paged caches work through a 4-D tensor map
//     (d, kv head, row in page, page) when page_size is a multiple of BN;
//   * NCW consumer warps each own a slice of the stage's keys (own running max / sum / O, merged
//     once at the end through a slab that is not part of the ring) and only wait on the stage's
//     "full" barrier; they release it through the "empty" barrier.  The producer never synchronises
//     with the consumers except through the ring, also across the units a persistent CTA works on.
// K / V tiles use the TMA 128-byte swizzle (conflict-free ldmatrix).
// Rows of the appended range come from k_new / v_new (k rotated on the fly), rows past the end
// are zero-filled; each consumer warp repairs the rows of its own key slice after the TMA landed.
#pragma once

#include "fwd_mma.cuh"
#include "tc5_ptx.cuh"

namespace fa {

// Consumer warps form a WM x WN grid: WM splits the packed query rows (16 * MT rows per warp), WN
// splits the keys of a stage.
template <int HD_, typename T_, int MT_, int WM_, int WN_, int BN_, int ST_, int SR_ = 0>
struct DecTraits {
  using T = T_;
  static constexpr int HD = HD_, MT = MT_, WM = WM_, WN = WN_, NCW = WM_ * WN_, BN = BN_, ST = ST_;
  static_assert(HD == 128, "K / V tiles arrive as two 64-column TMA boxes");
  static constexpr int BM = 16 * MT * WM;
  static constexpr int NTHREADS = 32 * (NCW + 1);
  static constexpr int NW = BN / WN;
  static constexpr int NT = NW / 8;
  static constexpr int KS = HD / 16;
  static constexpr int DT = HD / 8;
  static constexpr int CHUNKS = HD / 8;
  static constexpr int PITCH = HD * 2 + 16;      // Q rows: padded pitch, no swizzle
  static constexpr int HALF_BYTES = BN * 128;    // one 64-column half of a K or V tile (128-byte swizzled rows)
  static constexpr int KV_BYTES = 2 * HALF_BYTES;
  static constexpr int STAGE_BYTES = 2 * KV_BYTES;
  static constexpr int PIPE_BYTES = ST * STAGE_BYTES;
  static constexpr int SLAB_LD = HD + 4;
  static constexpr int SLAB_BYTES = BM * SLAB_LD * 4;  // merged output rows of the tile (fp32)
  // The slab normally lies behind the ring, so that the producer of a persistent CTA can fill the
  // ring for the next segment while the consumers merge.  SR_ = 1 puts it over the first stages
  // instead (one segment per CTA only: the ring is dead when the merge starts), which lets two
  // CTAs of 32 rows share an SM.
  static constexpr bool SLAB_IN_RING = SR_ != 0;
  static_assert(!SLAB_IN_RING || SLAB_BYTES <= PIPE_BYTES, "the slab must fit into the ring");
  static constexpr int SLAB_OFF = SLAB_IN_RING ? 0 : PIPE_BYTES;
  static constexpr int MAIN_BYTES = SLAB_IN_RING ? PIPE_BYTES : PIPE_BYTES + SLAB_BYTES;
  static constexpr int Q_BYTES = BM * PITCH;
  static constexpr int ML_BYTES = WN * BM * 8;
  static constexpr int BAR_BYTES = 128 + 2 * ST * 8;
  // [pipeline | slab | Q | (m, l) | barriers], the pipeline at a 1024-byte aligned base
  static constexpr int SMEM_BYTES = 1024 + MAIN_BYTES + Q_BYTES + ML_BYTES + BAR_BYTES;
  static constexpr bool Q_IN_REGS = (MT == 1);
  static constexpr int MIN_CTAS = SLAB_IN_RING ? 2 : 0;  // resident CTAs per SM the register count must allow (0: no constraint)
  static_assert(NW % 16 == 0, "each consumer warp needs a multiple of 16 keys");
};

// Address of 16-byte chunk `ch` (0..15) of row `row` in a K / V tile laid out by two TMA boxes of
// 64 columns with the 128-byte swizzle (chunk index XOR row % 8 inside each 128-byte row).
template <class Tr>
__device__ __forceinline__ uint32_t kv_chunk_addr(uint32_t tile_base, int row, int ch) {
  return tile_base + (ch >> 3) * Tr::HALF_BYTES + row * 128 + ((((ch & 7) ^ (row & 7))) << 4);
}

// Rows of the stage that the cache does not hold (yet): the appended tokens come from k_new / v_new
// (k rotated on the fly, never read back from the cache another CTA is writing), rows past the end
// are zeroed (V must be finite where P == 0).  Each consumer warp repairs the rows of its own slice.
template <class Tr>
__device__ __forceinline__ void decode_fix_rows(const KParams& p, const SeqView<typename Tr::T>& sv, uint32_t k_base,
                                                uint32_t v_base, int t0, int wn, int lane) {
  using T = typename Tr::T;
  for (int c = lane; c < Tr::NW * Tr::CHUNKS; c += 32) {
    const int row = wn * Tr::NW + c / Tr::CHUNKS, ch = c % Tr::CHUNKS;
    const int t = t0 + row;
    if (t < sv.l_cache) continue;
    uint4 kv4 = make_uint4(0, 0, 0, 0), vv4 = make_uint4(0, 0, 0, 0);
    if (t < sv.k_len) {
      const int tn = t - sv.l_cache;
      const T* krow = sv.knew + (int64_t)tn * p.a.knew_row_stride;
      kv4 = *reinterpret_cast<const uint4*>(krow + ch * 8);
      if (p.a.rotary_cos) {
        const int pos = t + p.a.kv_pos_offset;
        const T* cosr = reinterpret_cast<const T*>(p.a.rotary_cos) + (int64_t)pos * (p.a.rotary_dim >> 1);
        const T* sinr = reinterpret_cast<const T*>(p.a.rotary_sin) + (int64_t)pos * (p.a.rotary_dim >> 1);
        kv4 = rotary_chunk<T>(kv4, krow, ch * 8, cosr, sinr, p.a.rotary_dim, p.a.rotary_interleaved != 0);
      }
      vv4 = *reinterpret_cast<const uint4*>(sv.vnew + (int64_t)tn * p.a.vnew_row_stride + ch * 8);
    }
    const uint32_t kd = kv_chunk_addr<Tr>(k_base, row, ch), vd = kv_chunk_addr<Tr>(v_base, row, ch);
    asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(kd), "r"(kv4.x), "r"(kv4.y), "r"(kv4.z), "r"(kv4.w));
    asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(vd), "r"(vv4.x), "r"(vv4.y), "r"(vv4.z), "r"(vv4.w));
  }
  tc5::fence_proxy_async();  // the stage is refilled by TMA (async proxy) later
  __syncwarp();
}

// Producer: one elected lane issues four tiled TMA loads per stage (K and V, two 64-column halves
// each).  Tensor maps are 4-D (d, kv head, row, batch-or-page); every load targets the issuing CTA only.
template <class Tr>
__device__ __forceinline__ bool decode_producer(const KParams& p, const SeqView<typename Tr::T>& sv,
                                                const CUtensorMap* tm_k, const CUtensorMap* tm_v, uint32_t pipe_base,
                                                uint32_t full0, uint32_t empty0, int my_lo, int n_blocks,
                                                uint32_t it_base, int hk, int batch_row, volatile int* abort_flag) {
  for (int it = 0; it < n_blocks; ++it) {
    const uint32_t git = it_base + (uint32_t)it;  // stages this CTA has filled so far: ring position and parity
    const int stage = (int)(git % Tr::ST);
    if (git >= (uint32_t)Tr::ST && !tc5::mbar_wait(empty0 + stage * 8, ((git / Tr::ST) - 1) & 1, abort_flag)) return false;
    const uint32_t k_base = pipe_base + stage * Tr::STAGE_BYTES, v_base = k_base + Tr::KV_BYTES;
    const uint32_t full = full0 + stage * 8;
    const int t0 = (my_lo + it) * Tr::BN;
    int row = t0, outer = batch_row;
    if (sv.pages) {  // a block never straddles pages (page_size is a multiple of BN)
      const int pg = t0 / p.a.page_size;
      row = t0 - pg * p.a.page_size;
      outer = __ldg(sv.pages + pg);
      check_outer_index(p.a, outer, p.status);  // out of range: the TMA returns zeros, the status word says so
    }
    if (tc5::elect_one()) {
      tc5::mbar_arrive_expect_tx(full, Tr::STAGE_BYTES);
      tc5::tma_load_4d(k_base, tm_k, full, 0, hk, row, outer);
      tc5::tma_load_4d(k_base + Tr::HALF_BYTES, tm_k, full, 64, hk, row, outer);
      tc5::tma_load_4d(v_base, tm_v, full, 0, hk, row, outer);
      tc5::tma_load_4d(v_base + Tr::HALF_BYTES, tm_v, full, 64, hk, row, outer);
    }
    __syncwarp();
  }
  return true;
}

}  // namespace fa
