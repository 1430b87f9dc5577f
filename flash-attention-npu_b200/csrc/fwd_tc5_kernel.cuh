// Prefill attention-forward kernel for sm_100a: tcgen05 MMA with accumulators in TMEM, K/V tiles
// streamed by TMA through a shared-memory ring, online softmax in registers (one thread per
// query row), persistent CTAs.
//
// It replaces, for prefill (dense, packed varlen, or many query tokens against a KV cache, paged or
// not), the cube+vector pipeline of the reference kernel
// (csrc/arch22/flash_attn_npu_v2/mha_fwd_kvcache.cpp:632-965: QK -> online softmax -> PV ->
// rescale O, with S / P / O_tmp round-tripping through a global workspace).  Here S, P and O never
// leave the SM: S and O live in TMEM, P goes through shared memory (16-bit, the layout of an MMA
// A operand) into the second MMA.
//
// CTA = 16 warps:  warps 0-3    softmax of query sub-tile 0 (128 rows, one thread per row)
//                  warps 4-7    softmax of query sub-tile 1
//                  warps 8-11   correction (rescale of O in TMEM when a row maximum moved) and
//                               epilogue (O / l -> global) for both sub-tiles
//                  warps 12-13  MMA issuers, one per sub-tile (one elected lane each)
//                  warp  14     TMA producer (one elected lane)
//                  warp  15     clears the V rows past the end of a sequence (KV caches, packed input)
// TMEM (512 columns): S0 [0,128)  S1 [128,256)  O0 [256,384)  O1 [384,512).
// Shared memory: Q0 Q1 | P0 P1 | ring of K / V tiles (32 KiB each).
// Dependency chain per sub-tile: a softmax thread copies its row of S into registers and frees the
// S columns at once, so Q.K^T of the next KV block runs while this block's exponentials are
// computed; P.V follows when P is in shared memory.  The softmax warps therefore never wait for the
// tensor pipe in steady state, and the tensor pipe has two sub-tiles' worth of independent work.
#pragma once

#include "common.cuh"
#include "tc5_ptx.cuh"

namespace fa {
namespace tc5 {

constexpr int kBlockM = 128;          // rows of one query sub-tile
constexpr int kTileM = 2 * kBlockM;   // rows of one CTA tile
constexpr int kBlockN = 128;          // keys per KV block
constexpr int kSlots = 3;             // ring of 32 KiB K / V buffers
constexpr int kThreads = 512;
constexpr int kMmaWarp = 12 /* and 13: one per sub-tile */, kTmaWarp = 14;
// Registers per thread after the roles have re-balanced them (setmaxnreg, one value per warpgroup).
// A CTA can only re-distribute the registers it was launched with (512 threads x 128), never more:
// a setmaxnreg.inc that the other warpgroups' releases cannot cover would block for ever.
#ifndef FA_TC5_REGS_SOFTMAX
#define FA_TC5_REGS_SOFTMAX 192
#define FA_TC5_REGS_CORR 88
#define FA_TC5_REGS_MMA 40
#endif
constexpr int kRegsSoftmax = FA_TC5_REGS_SOFTMAX, kRegsCorr = FA_TC5_REGS_CORR, kRegsMma = FA_TC5_REGS_MMA;
static_assert(256 * kRegsSoftmax + 128 * (kRegsCorr + kRegsMma) <= kThreads * 128, "more registers than the CTA was launched with");
constexpr int kHalfBytes = kBlockN * 128;   // one 64-column half of a [128 x 128] 16-bit tile (128-byte rows)
constexpr int kTileBytes = 2 * kHalfBytes;  // 32 KiB
constexpr int kBarBytes = 3072;  // barriers, per-row rescale factors and 1 / l
// Q0 Q1 | P0 P1 | ring | barriers.  The dynamic shared memory base must be 1024-byte aligned (the
// kernel checks it): there is no room left for a round-up.
constexpr int kSmemBytes = 4 * kTileBytes + kSlots * kTileBytes + kBarBytes;
static_assert(kSmemBytes <= 232448, "more than the 227 KiB a CTA can have");

// Geometry by tile width HD (64, 128 or 256 columns; the head dim is at most HD).  Up to 128 a CTA tile is two
// 128-row sub-tiles and a K / V tile fills one 32 KiB ring slot (its first half only for 64).  For 256 the 256 fp32
// columns of O leave TMEM room for one sub-tile only: the CTA tile is 128 rows, Q takes both Q slots (64 KiB), the
// second P slot joins the ring, and the ring is two slots of 64 KiB.
template <int HD>
struct Geo {
  static_assert(HD == 64 || HD == 128 || HD == 256, "tile widths");
  static constexpr int kHalves = HD / 64;                                      // 64-column halves of a Q / K / V tile
  static constexpr bool kWide = HD > 128;
  static constexpr int kRows = kWide ? kBlockM : kTileM;                       // query rows of a CTA tile
  static constexpr int kSlotBytes = kWide ? 2 * kTileBytes : kTileBytes;
  static constexpr int kRing = kWide ? 2 : kSlots;
  static constexpr int kRingOff = kWide ? 3 * kTileBytes : 4 * kTileBytes;     // Q0 Q1 | P0 [P1] | ring
  static_assert(kRingOff + kRing * kSlotBytes + kBarBytes <= kSmemBytes, "shared memory layout");
};

struct Tc5Params {
  fa_fwd_params a;
  int32_t is_causal, is_local, wl, wr;
  int32_t group;    // h / h_k
  int32_t m_tiles;  // ceil(max seqlen_q / 256)
  int32_t total_tiles;
  float scale_log2;
  float softcap_mul, softcap_l2;  // softcap: scores become softcap_l2 * tanh(s * softcap_mul) in the log2 domain (scale / softcap, softcap * log2 e)
  int32_t chunk_bh;          // (batch, head) pairs per L2 chunk of the tile order (tile_info)
  // 1: the rows behind the last key of a sequence hold foreign data (the unused tail of a KV cache or of a page,
  // the next sequence of a packed tensor) and must be cleared in V before P.V: P is 0 there, but 0 x NaN is NaN.
  // 0: dense input, those rows lie outside the tensor and the TMA unit already returns zeros for them.
  int32_t fix_tail;
  int32_t* status;  // device word: 0 ok, otherwise the wait that gave up
};


struct TileInfo {
  int bi, hh, hk, q_row0, q_len, k_row0, k_len, koff;
  int bk;  // batch row of K / V (cache_batch_idx for a contiguous cache)
  int row0[2];  // first row (within the sequence) of each sub-tile
  int jlo[2], jhi[2];
  bool has[2];
  int ulo, uhi;  // union of the block ranges
};

// Tile order: the (batch, head) pairs are cut into chunks whose K / V fit in L2 together; inside a
// chunk all pairs run their last (heaviest, causal) query tile first, then the one before, and so
// on, so the K / V prefixes a chunk re-reads tile after tile come from L2 and not from HBM.  The
// chunk length makes a chunk a whole even number of rounds of the grid (TileSched), which keeps the
// per-CTA sums as even as one chunk over everything would.
template <int ROWS>  // query rows of a CTA tile: 256 (two sub-tiles) or 128 (sub-tile 0 only)
__device__ __forceinline__ void tile_info(const Tc5Params& p, int n, TileInfo& ti) {
  const int per_m = p.a.b * p.a.h;
  const int per_chunk = p.chunk_bh * p.m_tiles;
  const int ck = n / per_chunk, r = n - ck * per_chunk;
  const int cnt = min(p.chunk_bh, per_m - ck * p.chunk_bh);  // pairs in this chunk (the last one may be short)
  const int mt = p.m_tiles - 1 - r / cnt;  // heavy (late, causal) tiles first
  const int rem = ck * p.chunk_bh + r % cnt;
  ti.bi = rem / p.a.h;
  ti.hh = rem % p.a.h;
  ti.hk = ti.hh / p.group;
  ti.q_row0 = 0;
  ti.q_len = p.a.seqlen_q;
  ti.k_row0 = 0;
  ti.k_len = p.a.seqlen_k;
  if (p.a.cu_seqlens_q) {
    ti.q_row0 = p.a.cu_seqlens_q[ti.bi];
    ti.q_len = p.a.cu_seqlens_q[ti.bi + 1] - ti.q_row0;
  }
  if (p.a.cu_seqlens_k) {
    ti.k_row0 = p.a.cu_seqlens_k[ti.bi];
    ti.k_len = p.a.cu_seqlens_k[ti.bi + 1] - ti.k_row0;
  }
  ti.bk = (p.a.cache_batch_idx && !p.a.block_table) ? p.a.cache_batch_idx[ti.bi] : ti.bi;
  // KV cache (contiguous or paged): keys in use per batch entry, plus the tokens the prologue appended
  if (p.a.seqused_k) ti.k_len = cache_len(p.a, ti.bi, nullptr) + p.a.seqlen_new;  // clamped; the producer reports it
  ti.koff = ti.k_len - ti.q_len;
  ti.ulo = 0x7fffffff;
  ti.uhi = 0;
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int r0 = (ROWS == kBlockM && t == 1) ? 0x3fffffff : mt * ROWS + t * kBlockM;  // no second sub-tile in 128-row tiles
    ti.row0[t] = r0;
    ti.jlo[t] = ti.jhi[t] = 0;
    ti.has[t] = false;
    if (r0 < ti.q_len) {
      const int i_min = r0, i_max = min(ti.q_len, r0 + kBlockM) - 1;
      int j_lo = 0, j_hi = ti.k_len;
      if (p.is_causal) j_hi = min(ti.k_len, i_max + ti.koff + 1);
      if (p.is_local) {
        j_hi = min(ti.k_len, i_max + ti.koff + p.wr + 1);
        j_lo = max(0, i_min + ti.koff - p.wl);
      }
      if (j_hi > j_lo) {
        ti.jlo[t] = j_lo / kBlockN;
        ti.jhi[t] = ceil_div(j_hi, kBlockN);
        ti.has[t] = true;
        ti.ulo = min(ti.ulo, ti.jlo[t]);
        ti.uhi = max(ti.uhi, ti.jhi[t]);
      }
    }
  }
  if (ti.uhi == 0) ti.ulo = 0;
}

// Static tile schedule.  tile_info orders tiles heaviest first; CTA c of G takes tiles
// c, 2G-1-c, 2G+c, 4G-1-c, ... (serpentine), which evens out the per-CTA sums of a decreasing
// sequence (causal, 4K: 1 % spread instead of 6 % with a plain stride).
struct TileSched {
  int round, total;
  __device__ explicit TileSched(const Tc5Params& p) : round(0), total(p.total_tiles) {}
  __device__ __forceinline__ int cur() const {
    const int g = (int)gridDim.x, c = (int)blockIdx.x;
    if (round * g >= total) return total;
    const int n = round * g + ((round & 1) ? g - 1 - c : c);
    return n < total ? n : total;
  }
  __device__ __forceinline__ int first() { return cur(); }
  __device__ __forceinline__ int next() {
    ++round;
    return cur();
  }
};

struct Barriers {
  uint64_t q_full[2], q_empty[2], kv_full[kSlots], kv_empty[kSlots];
  uint64_t s_full[2];      // MMA -> softmax: S_t = Q_t K_j^T is in TMEM
  uint64_t s_free[2];      // softmax -> MMA: every row of S_t has been copied into registers
  // softmax -> MMA: half h (64 keys) of P_t is in shared memory.  One barrier per half: a waiter must
  // never fall two phases behind a barrier, which two arrivals per block on one barrier would allow.
  uint64_t p_full[2][2];
  uint64_t corr_ready[2];  // softmax -> correction: rescale factors of block j are in shared memory
  uint64_t o_ready[2];     // correction -> MMA: O_t has been rescaled, P.V of block j may accumulate
  uint64_t o_done[2];      // MMA -> correction, softmax: P.V of a block has completed (O_t updated, P_t read)
  uint64_t stats_ready[2]; // softmax -> correction: 1 / l of the tile's rows is in shared memory
  uint64_t o_free[2];      // correction -> MMA: the epilogue has read O_t
  uint64_t fix_req;        // MMA (both warps) -> warp 15: the last V tile of the CTA tile has landed and needs its tail cleared
  uint64_t v_fixed;        // warp 15 -> MMA (both warps): done
  uint32_t tmem_base;
  int abort_flag;
  uint32_t fix_seen[2];    // tail repairs each issuing warp has been through (phase of fix_req / v_fixed)
  uint32_t fix_slot;       // ring slot of the V tile to repair
  float corr[2][kBlockM];
  float row_inv[2][kBlockM];
};
static_assert(sizeof(Barriers) <= kBarBytes, "barrier block does not fit");

}  // namespace tc5
}  // namespace fa
