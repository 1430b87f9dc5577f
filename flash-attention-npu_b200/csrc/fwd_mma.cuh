// Register-accumulator attention-forward kernel (mma.sync m16n8k16, cp.async pipeline).
//
// One CTA owns a tile of BM "packed" query rows of one (batch, head-group) and a
// contiguous range of KV blocks (a split).  Packed row r -> query token r / gp, query head
// hh * gp + r % gp, so with gp = h / h_k all query heads of a kv head share each K/V byte
// (same idea as GetQNBlockTile, csrc/arch22/flash_attn_npu_v2/kernel_common.hpp:85-92).
// Warps form a WM x WN grid: WM splits the rows, WN splits the columns of every KV block
// (each warp keeps its own running max / sum / O and they are merged once at the end), which
// is what keeps all four tensor pipes busy when there are only 4..32 rows (decode).
//
// Functionally this replaces FAInferKernel::runMainLoop
// (csrc/arch22/flash_attn_npu_v2/mha_fwd_kvcache.cpp:436-966): QK^T (qk_matmul.hpp), online
// softmax (online_softmax.hpp:479-803), PV (pv_matmul.hpp), rescale + final normalise + LSE
// (rescale_o.hpp:299-534), paged gather (qk_matmul.hpp:177-182,233-251), split partials
// (rescale_o.hpp:226-262).  Added beyond the reference: fused KV append + rotary, alibi.
#pragma once

#include "common.cuh"

namespace fa {

template <int HD_, typename T_, int MT_, int WM_, int WN_, int BN_, int ST_>
struct MmaTraits {
  using T = T_;
  static constexpr int HD = HD_, MT = MT_, WM = WM_, WN = WN_, BN = BN_, ST = ST_;
  static constexpr int BM = 16 * MT * WM;
  static constexpr int NTHREADS = 32 * WM * WN;
  static constexpr int NW = BN / WN;   // KV columns of one block handled by one warp
  static constexpr int NT = NW / 8;    // score n-tiles per warp
  static constexpr int KS = HD / 16;   // k-steps of QK^T
  static constexpr int DT = HD / 8;    // output n-tiles
  static constexpr int CHUNKS = HD / 8;  // 16-byte chunks per row
  static constexpr int ROW_BYTES = HD * 2;
  static constexpr int Q_BYTES = BM * ROW_BYTES;
  static constexpr int KV_BYTES = BN * ROW_BYTES;       // one of K or V
  static constexpr int STAGE_BYTES = 2 * KV_BYTES;
  static constexpr int SLAB_LD = HD + 4;                // fp32 row pitch of the epilogue slab
  static constexpr int SLAB_BYTES = WN * BM * SLAB_LD * 4;
  static constexpr int ML_BYTES = WN * BM * 8;
  static constexpr int PIPE_BYTES = ST * STAGE_BYTES;
  static constexpr int SMEM_BYTES = Q_BYTES + (PIPE_BYTES > SLAB_BYTES ? PIPE_BYTES : SLAB_BYTES) + ML_BYTES;
  static_assert(NW % 16 == 0, "each warp needs a multiple of 16 KV columns");
  static_assert(HD % 64 == 0, "head dim is padded to a multiple of 64");
};

// Address of row `row`, 16-byte chunk `ch` in a [rows][HD] 16-bit tile whose chunks are
// XOR-swizzled with the low 3 bits of the row (conflict-free ldmatrix).
template <int ROW_BYTES>
__device__ __forceinline__ uint32_t tile_addr(uint32_t base, int row, int ch) {
  return base + row * ROW_BYTES + (((ch) ^ (row & 7)) << 4);
}

// Per-CTA view of its sequence.
template <typename T>
struct SeqView {
  const T* q;      // first query row of this sequence, head 0
  const T* k;      // contiguous: row 0 of this sequence / cache row, kv head hk; paged: pool base + head offset
  const T* v;
  const T* knew;   // (s_new, d) of this sequence and kv head, or nullptr
  const T* vnew;
  const int32_t* pages;  // block_table row or nullptr
  int q_len, l_cache, k_len, q_row0;
};

template <class Tr>
__device__ __forceinline__ const typename Tr::T* kv_row_ptr(const KParams& p, const typename Tr::T* base,
                                                            const int32_t* pages, int64_t page_stride,
                                                            int64_t row_stride, int t) {
  if (pages) {
    int pg = t / p.a.page_size;
    int in = t - pg * p.a.page_size;
    return base + (int64_t)outer_index(p.a, __ldg(pages + pg), p.status) * page_stride + (int64_t)in * row_stride;
  }
  return base + (int64_t)t * row_stride;
}

// Loads KV block `nb` (BN tokens) of K and V into one pipeline stage.  Tokens already in the
// cache come through cp.async; tokens of the appended range [l_cache, k_len) are produced from
// k_new / v_new (k rotated on the fly), so no CTA ever reads a cache row that the append writes;
// tokens >= k_len are zero-filled (V must be finite where P == 0).
template <class Tr>
__device__ __forceinline__ void load_kv_block(const KParams& p, const SeqView<typename Tr::T>& sv, uint32_t stage_base,
                                              int nb, int tid) {
  using T = typename Tr::T;
  constexpr int ITER = Tr::BN * Tr::CHUNKS / Tr::NTHREADS;
  static_assert(Tr::BN * Tr::CHUNKS % Tr::NTHREADS == 0, "");
  const int d = p.a.d;
#pragma unroll 4
  for (int it = 0; it < ITER; ++it) {
    const int c = tid + it * Tr::NTHREADS;
    const int row = c / Tr::CHUNKS, ch = c % Tr::CHUNKS;
    const int t = nb * Tr::BN + row;
    const uint32_t kd = tile_addr<Tr::ROW_BYTES>(stage_base, row, ch);
    const uint32_t vd = kd + Tr::KV_BYTES;
    const bool in_d = ch * 8 < d;
    if (t < sv.l_cache || !in_d || t >= sv.k_len) {
      const bool valid = in_d && t < sv.l_cache;
      const T* kp = sv.k;
      const T* vp = sv.v;
      if (valid) {
        kp = kv_row_ptr<Tr>(p, sv.k, sv.pages, p.a.k_batch_stride, p.a.k_row_stride, t) + ch * 8;
        vp = kv_row_ptr<Tr>(p, sv.v, sv.pages, p.a.v_batch_stride, p.a.v_row_stride, t) + ch * 8;
      }
      cp_async_16(kd, kp, valid);
      cp_async_16(vd, vp, valid);
    } else {
      const int tn = t - sv.l_cache;  // index into the new tokens
      const T* krow = sv.knew + (int64_t)tn * p.a.knew_row_stride;
      uint4 kv4 = *reinterpret_cast<const uint4*>(krow + ch * 8);
      if (p.a.rotary_cos) {
        const int pos = t + p.a.kv_pos_offset;
        const T* cosr = reinterpret_cast<const T*>(p.a.rotary_cos) + (int64_t)pos * (p.a.rotary_dim >> 1);
        const T* sinr = reinterpret_cast<const T*>(p.a.rotary_sin) + (int64_t)pos * (p.a.rotary_dim >> 1);
        kv4 = rotary_chunk<T>(kv4, krow, ch * 8, cosr, sinr, p.a.rotary_dim, p.a.rotary_interleaved != 0);
      }
      uint4 vv4 = *reinterpret_cast<const uint4*>(sv.vnew + (int64_t)tn * p.a.vnew_row_stride + ch * 8);
      asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(kd), "r"(kv4.x), "r"(kv4.y), "r"(kv4.z), "r"(kv4.w));
      asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(vd), "r"(vv4.x), "r"(vv4.y), "r"(vv4.z), "r"(vv4.w));
    }
  }
}

// The designated CTA of a (batch, kv head) writes the appended tokens into the cache
// (k rotated, v copied).  Bit-exact with the host formula documented at rotary_chunk.
template <class Tr>
__device__ __forceinline__ void append_to_cache(const KParams& p, const SeqView<typename Tr::T>& sv, int tid,
                                                int nthreads = Tr::NTHREADS) {
  using T = typename Tr::T;
  const int chunks = p.a.d >> 3;
  const int total = p.a.seqlen_new * chunks;
  for (int c = tid; c < total; c += nthreads) {
    const int tn = c / chunks, ch = c - tn * chunks;
    const int t = sv.l_cache + tn;
    const T* krow = sv.knew + (int64_t)tn * p.a.knew_row_stride;
    uint4 kv4 = *reinterpret_cast<const uint4*>(krow + ch * 8);
    if (p.a.rotary_cos) {
      const int pos = t + p.a.kv_pos_offset;
      const T* cosr = reinterpret_cast<const T*>(p.a.rotary_cos) + (int64_t)pos * (p.a.rotary_dim >> 1);
      const T* sinr = reinterpret_cast<const T*>(p.a.rotary_sin) + (int64_t)pos * (p.a.rotary_dim >> 1);
      kv4 = rotary_chunk<T>(kv4, krow, ch * 8, cosr, sinr, p.a.rotary_dim, p.a.rotary_interleaved != 0);
    }
    uint4 vv4 = *reinterpret_cast<const uint4*>(sv.vnew + (int64_t)tn * p.a.vnew_row_stride + ch * 8);
    T* kdst = const_cast<T*>(kv_row_ptr<Tr>(p, sv.k, sv.pages, p.a.k_batch_stride, p.a.k_row_stride, t)) + ch * 8;
    T* vdst = const_cast<T*>(kv_row_ptr<Tr>(p, sv.v, sv.pages, p.a.v_batch_stride, p.a.v_row_stride, t)) + ch * 8;
    *reinterpret_cast<uint4*>(kdst) = kv4;
    *reinterpret_cast<uint4*>(vdst) = vv4;
  }
}

// Q tile -> shared memory (rotated when rotary tables are given).  Rows beyond the sequence are zero.
template <class Tr>
__device__ __forceinline__ void load_q_tile(const KParams& p, const SeqView<typename Tr::T>& sv, uint32_t q_base,
                                            int row0, int hh, bool rot_per_token, int tid) {
  using T = typename Tr::T;
  const int rows_total = sv.q_len * p.gp;
  for (int c = tid; c < Tr::BM * Tr::CHUNKS; c += Tr::NTHREADS) {
    const int row = c / Tr::CHUNKS, ch = c % Tr::CHUNKS;
    const int r = row0 + row;
    const uint32_t dst = tile_addr<Tr::ROW_BYTES>(q_base, row, ch);
    const bool valid = r < rows_total && ch * 8 < p.a.d;
    const int i = r / p.gp, g = r - i * p.gp;
    const T* qrow = sv.q + (int64_t)i * p.a.q_row_stride + (int64_t)(hh * p.gp + g) * p.a.q_head_stride;
    if (!valid || !p.a.rotary_cos) {
      cp_async_16(dst, valid ? qrow + ch * 8 : sv.q, valid);
    } else {
      const int pos = sv.l_cache + p.a.kv_pos_offset + (rot_per_token ? i : 0);
      const T* cosr = reinterpret_cast<const T*>(p.a.rotary_cos) + (int64_t)pos * (p.a.rotary_dim >> 1);
      const T* sinr = reinterpret_cast<const T*>(p.a.rotary_sin) + (int64_t)pos * (p.a.rotary_dim >> 1);
      uint4 q4 = *reinterpret_cast<const uint4*>(qrow + ch * 8);
      q4 = rotary_chunk<T>(q4, qrow, ch * 8, cosr, sinr, p.a.rotary_dim, p.a.rotary_interleaved != 0);
      asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(dst), "r"(q4.x), "r"(q4.y), "r"(q4.z), "r"(q4.w));
    }
  }
}

}  // namespace fa
