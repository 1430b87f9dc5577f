// Attention backward on the Blackwell tensor cores (tcgen05.mma, accumulators and the P / dS operands in TMEM,
// Q / K / V / dO tiles by TMA), head dims up to 128, dense and packed-varlen input, optional softcap.
//
// Same arithmetic as bwd_kernel.cuh, which follows the reference's golden (tests/fa_small_op_golden.py:160-353) and
// replaces its FAG kernels (csrc/arch22/flash_attn_npu_v3/fag_kernel.cpp):
//   P = exp(S scale - LSE)   dP = dO V^T   dS = P o (dP - D) scale   dV = P^T dO   dK = dS^T Q   dQ = dS K
// with P and dS rounded to the input dtype before the second matrix products and fp32 accumulation.
//
// Two persistent kernels (one CTA per SM; work items drawn from a global counter, a head's blocks neighbours in the
// order, its heavy blocks first), no atomics (the results do not depend on any order of arrival):
//   bwd_dkv_kernel  one CTA per 128 keys of a (batch entry, kv head).  K and V stay in shared memory, the query
//                   rows that see the keys (of every query head of the group) stream through a ring, 64 at a time.
//                   It computes the TRANSPOSED products S^T = K Q^T and dP^T = V dO^T, so that a TMEM lane is a key:
//                   P^T and dS^T, written back into the TMEM columns their fp32 sources came from, are the A
//                   operands of dV += P^T dO and dK += dS^T Q (dO and Q as N-contiguous B operands from the same
//                   tiles).  TMEM: two buffers of S^T | dP^T (64 rows each), dV, dK.
//   bwd_dq_kernel   one CTA per 128 query rows of a (batch entry, head).  Q and dO stay in shared memory, K and V
//                   stream through a ring; S = Q K^T, dP = dO V^T, dS (16-bit) goes to TMEM columns of its own and
//                   is the A operand of dQ += dS K (K as an N-contiguous B operand from the tile S was computed
//                   from).  S and dP are free as soon as they are in registers, so the products of the next block
//                   run under this block's exponentials.  TMEM: S | dP | dQ | dS.
// The elementwise work has no row reduction (LSE and D are inputs), so it is split by columns over 16 warps: a
// thread owns one TMEM lane and 32 columns (of a block's 128 in the dQ kernel, of a unit's 64 in the dK / dV kernel,
// where warps 0-7 and 8-15 take alternate units).
// Warps 0-15 elementwise + epilogue; warps 16-18 issue the MMAs (one elected lane each), each its own chain of
// products: S^T then dV, and dP^T then dK (each chain's TMEM hazards stay inside one in-order issuer), or S, dP and
// dQ (spreading the issue over warps did not change the speed by itself); warp 19 is the TMA producer.
// A CTA walks over its work items without tearing anything down: barrier phases and ring positions run on, the next
// item's tiles are requested as soon as the current item's last product has read the old ones, and the epilogue hands
// the accumulators back (acc_free) as soon as they are in registers, so its global stores lie under the next item's
// first products.  (One CTA per item cost ~15 000 cycles of fill, drain and launch per item against ~40 000 of work.)
// Every wait is bounded; a wait that gives up raises the CTA's abort flag and ends in the device status word.
#pragma once

#include <type_traits>

#include "bwd_kernel.cuh"
#include "tc5_ptx.cuh"

namespace fa {
namespace btc5 {

using namespace tc5;

constexpr int kBlk = 128;                 // rows of a query block = keys of a key block
constexpr int kHalfBytes = kBlk * 128;    // one 64-column half of a [128 x 128] 16-bit tile (128-byte rows)
constexpr int kTileBytes = 2 * kHalfBytes;
constexpr int kEwWarps = 16, kMmaWarp = 16 /* .. 18 */, kTmaWarp = 19;
constexpr int kThreads = 20 * 32;
constexpr int kBarBytes = 3072;
constexpr int kDqSlots = 5, kDqKSlots = 3;  // rings of bwd_dq_kernel: three K tiles (slots 0-2), two V tiles (slots 3-4)
constexpr int kSmemBytes = 7 * kTileBytes + kBarBytes;   // dQ: 2 resident tiles + 5 ring tiles; dK / dV: 2 + 4 stages of 32 KiB (6 tiles' worth)
static_assert(kSmemBytes <= 232448, "more than the 227 KiB a CTA can have");

// 16 columns / 8 columns of one TMEM lane per thread
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};\n" ::"r"(taddr), "r"(r[0]), "r"(r[1]),
               "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}

// Bit e set: element (first + e) lies in [lo, hi].
__device__ __forceinline__ uint32_t range_bits(int first, int lo, int hi) {
  const int n_lo = min(max(lo - first, 0), 32);
  const int n_hi = min(max(hi - first + 1, 0), 32);
  const uint32_t below_hi = n_hi >= 32 ? 0xffffffffu : ((1u << n_hi) - 1u);
  const uint32_t below_lo = n_lo >= 32 ? 0xffffffffu : ((1u << n_lo) - 1u);
  return below_hi & ~below_lo;
}

// Build-time constant: of every 4 pairs of exponentials, how many are evaluated by polynomial on the FMA pipe instead
// of the special-function unit (whose 16 results per clock per SM are what bounds the elementwise phase otherwise).
#ifndef FA_BWD_POLY
#define FA_BWD_POLY 0
#endif
constexpr int kPolyPairs = FA_BWD_POLY;

// Two elements:  P = exp2(s * scale_log2 - lse2)  (0 where masked),  dS = P * (dP - D) * scale, both as packed 16-bit
// pairs.  nlse2 = -lse2 and ndls2 = -D * scale per element, so the arithmetic is two packed fused multiply-adds, two
// exponentials and one packed multiply.  With softcap the capped score c * tanh(s * scale / c) replaces s * scale and
// dS gets the factor 1 - tanh^2 (tests/fa_small_op_golden.py:80-89,124-125); a2 is then scale / c instead of
// scale * log2(e), cap2 = c * log2(e).
// (poly is a constant after unrolling: pair number & 3 < kPolyPairs)
template <typename T, bool MASK, bool SOFTCAP>
__device__ __forceinline__ void ew_pair(const bool poly, uint32_t s0, uint32_t s1, uint32_t d0, uint32_t d1, uint64_t a2,
                                        uint64_t cap2, uint64_t nlse2, uint64_t scale2, uint64_t ndls2, uint32_t bits, int e,
                                        uint32_t& pk_p, uint32_t& pk_ds) {
  uint64_t x2, g2 = 0;
  if (SOFTCAP) {
    float y0, y1, t0, t1;
    unpack_f32x2(mul_f32x2(pack_f32x2(__uint_as_float(s0), __uint_as_float(s1)), a2), y0, y1);
    asm("tanh.approx.f32 %0, %1;\n" : "=f"(t0) : "f"(y0));
    asm("tanh.approx.f32 %0, %1;\n" : "=f"(t1) : "f"(y1));
    const uint64_t th2 = pack_f32x2(t0, t1);
    x2 = fma_f32x2(th2, cap2, nlse2);
    g2 = fma_f32x2(th2, pack_f32x2(-t0, -t1), pack_f32x2(1.f, 1.f));  // 1 - tanh^2
  } else {
    x2 = fma_f32x2(pack_f32x2(__uint_as_float(s0), __uint_as_float(s1)), a2, nlse2);
  }
  float p0, p1;
  if (poly) {
    poly_exp2_x2(x2, p0, p1);
  } else {
    float x0, x1;
    unpack_f32x2(x2, x0, x1);
    p0 = fast_exp2(x0);
    p1 = fast_exp2(x1);
  }
  if (MASK) {
    p0 = ((bits >> e) & 1u) ? p0 : 0.f;
    p1 = ((bits >> (e + 1)) & 1u) ? p1 : 0.f;
  }
  uint64_t t2 = fma_f32x2(pack_f32x2(__uint_as_float(d0), __uint_as_float(d1)), scale2, ndls2);
  if (SOFTCAP) t2 = mul_f32x2(t2, g2);
  float ds0, ds1;
  unpack_f32x2(mul_f32x2(pack_f32x2(p0, p1), t2), ds0, ds1);
  pk_p = pack2<T>(p0, p1);
  pk_ds = pack2<T>(ds0, ds1);
}

// Work items are handed out dynamically: the producer warp draws the next item number from a global counter and
// publishes it to the other roles of its CTA through a small ring in shared memory (slot k % 8 for the CTA's k-th
// published item, -1 = no more items).  Items without work (keys nobody sees, rows that see no key) are not
// published: the producer warp writes their zeros itself.  The ring needs no "empty" barrier: for items with work the
// producer cannot be more than two items ahead of any other role (it waits for the previous item's last read of the
// resident tiles, the issuing warps wait for the epilogue of the item before that), and the ring has eight slots.
constexpr int kQueue = 8;
struct ItemQueue {
  uint64_t full[kQueue];
  int32_t item[kQueue];
};
__device__ __forceinline__ int queue_draw(int32_t* counter, int n_items, int lane) {
  int t = 0;
  if (lane == 0) {
    t = atomicAdd(counter, 1);
    if (t >= n_items) t = -1;
  }
  return __shfl_sync(0xffffffffu, t, 0);
}
__device__ __forceinline__ void queue_publish(ItemQueue* q, uint32_t k, int t, int lane) {
  if (lane == 0) {
    q->item[k % kQueue] = t;
    mbar_arrive(smem_addr(&q->full[k % kQueue]));
  }
  __syncwarp();
}
__device__ __forceinline__ int queue_get(ItemQueue* q, uint32_t k, volatile int* abort_flag) {
  if (!mbar_wait(smem_addr(&q->full[k % kQueue]), (k / kQueue) & 1, abort_flag, 59)) return -1;
  return q->item[k % kQueue];
}

// K-major operand tile (two 64-column halves, 128-byte swizzle): byte offset of k-step ks (16 columns), >> 4
__device__ __forceinline__ uint64_t kmaj_off(int ks) { return (uint64_t)(((ks >> 2) * kHalfBytes + (ks & 3) * 32) >> 4); }
// the same tile read as an N-contiguous B operand: k-step ks = 16 rows of 128 bytes
__device__ __forceinline__ uint64_t nmaj_off(int ks) { return (uint64_t)((ks * 2048) >> 4); }

struct SeqInfo {
  int q_row0, q_len, k_row0, k_len, koff, bq;
  int wl, wr;  // window sides in force; negative = unbounded
};
__device__ __forceinline__ SeqInfo seq_info(const BwdParams& p, int bi) {
  SeqInfo s;
  s.q_row0 = 0; s.q_len = p.seqlen_q; s.k_row0 = 0; s.k_len = p.seqlen_k;
  if (p.cu_seqlens_q) {
    s.q_row0 = p.cu_seqlens_q[bi];
    s.q_len = p.cu_seqlens_q[bi + 1] - s.q_row0;
    s.k_row0 = p.cu_seqlens_k[bi];
    s.k_len = p.cu_seqlens_k[bi + 1] - s.k_row0;
  }
  s.bq = p.cu_seqlens_q ? 0 : bi;
  s.koff = s.k_len - s.q_len;
  // a negative side is unbounded (make_window_atten_mask, tests/fa_small_op_golden.py:36-58)
  s.wr = p.is_causal ? 0 : ((p.is_local && p.wr >= 0) ? p.wr : -1);
  s.wl = (p.is_local && p.wl >= 0) ? p.wl : -1;
  return s;
}

// 32 columns of a row, of which the first n_cols (a multiple of 8, possibly <= 0) exist
template <typename T>
__device__ __forceinline__ void store_slice(T* dst, const uint32_t (&a)[32], int n_cols) {
#pragma unroll
  for (int e = 0; e < 32; e += 8) {
    if (e >= n_cols) break;
    uint4 w;
    w.x = pack2<T>(__uint_as_float(a[e]), __uint_as_float(a[e + 1]));
    w.y = pack2<T>(__uint_as_float(a[e + 2]), __uint_as_float(a[e + 3]));
    w.z = pack2<T>(__uint_as_float(a[e + 4]), __uint_as_float(a[e + 5]));
    w.w = pack2<T>(__uint_as_float(a[e + 6]), __uint_as_float(a[e + 7]));
    *reinterpret_cast<uint4*>(dst + e) = w;
  }
}

__device__ __forceinline__ void finish(int32_t* status, int aborted, int tid) {
  if (aborted) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);  // copies in flight may still land in this CTA's shared memory
    if (tid == 0) atomicExch(status, (aborted << 16) | (1 + (blockIdx.x & 0xffff)));
    __syncthreads();
  }
}

// =================================================================================================
// dK, dV.  The query rows stream through in units of 64; S^T / dP^T of a unit are 64 TMEM columns each and there are
// two such buffers, so the products of unit u + 1 run while the elementwise warps work on unit u.
// TMEM: buffer 0 [S^T 0-63 | dP^T 64-127]  buffer 1 [128-255]  dV 256-383  dK 384-511.
// =================================================================================================
constexpr int kUnit = 64;                    // query rows per unit
constexpr int kUnitHalf = kUnit * 128;       // one 64-column half of a [64 x 128] 16-bit tile: 8 KiB
constexpr int kUnitTile = 2 * kUnitHalf;     // 16 KiB
constexpr int kStages = 4;                   // ring stages, each Q (16 KiB) then dO (16 KiB)

struct BarA {
  uint64_t kv_full, kv_empty;  // K / V of the item have landed; the item's last S^T / dP^T have read them
  uint64_t qdo_full[kStages], qdo_empty[kStages];
  uint64_t st_full[2];   // MMA -> elementwise: S^T and dP^T of the buffer are in TMEM
  uint64_t pds_full[2];  // elementwise -> MMA: P^T and dS^T of the buffer are in TMEM
  uint64_t acc_done;     // MMA -> epilogue: dV, dK of the item are complete
  uint64_t acc_free;     // epilogue -> MMA: dV, dK are in registers
  ItemQueue queue;
  uint32_t tmem_base;
  int abort_flag;
  alignas(16) float nlse2[kStages][kUnit];  // per ring stage: -LSE * log2(e) and -D * scale of the unit's query rows (read 4 at a time)
  alignas(16) float ndls[kStages][kUnit];
};
static_assert(sizeof(BarA) <= kBarBytes, "barrier block does not fit");

// Work item t of the dK / dV kernel: 128 keys of one (kv head, batch entry).  The key blocks of a pair are
// neighbours in the order, so the CTAs running at one time stream the same few heads' Q / dO and find them in L2
// (with one key block index across all pairs at a time every item read its Q / dO from HBM: 2.3 ms against 1.8 on the
// 4 K causal case); block 0 first: under a causal mask it has the most work, and the launch ends on light items.
struct ItemA {
  SeqInfo sq;
  int hk, bi, key0, u_lo, nu, iters;  // iters = units x query heads of the group; 0 = nobody sees the keys
  bool live;                          // false: the sequence has no such keys, nothing to write
};
__device__ __forceinline__ ItemA item_a(const BwdParams& p, int t) {
  ItemA w;
  const int n_kblocks = ceil_div(p.seqlen_k, kBlk);
  const int pair = t / n_kblocks, nb = t - pair * n_kblocks;
  w.hk = pair % p.h_k;
  w.bi = pair / p.h_k;
  w.sq = seq_info(p, w.bi);
  w.key0 = nb * kBlk;
  w.live = w.key0 < w.sq.k_len;
  w.u_lo = w.nu = w.iters = 0;
  if (w.live) {
    // query rows that see at least one key of the block
    const int k1 = min(w.sq.k_len, w.key0 + kBlk) - 1;
    const int i_lo = w.sq.wr >= 0 ? max(0, w.key0 - w.sq.koff - w.sq.wr) : 0;
    const int i_hi = w.sq.wl >= 0 ? min(w.sq.q_len - 1, k1 - w.sq.koff + w.sq.wl) : w.sq.q_len - 1;  // inclusive
    w.u_lo = i_lo / kUnit;
    w.nu = i_hi >= i_lo ? i_hi / kUnit + 1 - w.u_lo : 0;
    w.iters = w.nu * (p.h / p.h_k);
  }
  return w;
}

// HD (64 or 128): width of the tiles; a head dim below it leaves zero columns (filled in by the TMA unit) that are not stored.
template <typename T, uint32_t AB_FMT, bool SOFTCAP, int HD>
__global__ void __launch_bounds__(kThreads, 1)
bwd_dkv_kernel(const __grid_constant__ BwdParams p, const __grid_constant__ CUtensorMap tm_q,
               const __grid_constant__ CUtensorMap tm_do, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v, int32_t* status, int32_t* counter) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t base = smem_addr(smem);
  const int tid = threadIdx.x, lane = tid & 31;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
  if ((base & 1023u) != 0) {
    if (tid == 0) atomicExch(status, 0x20000000);
    return;
  }
  const int group = p.h / p.h_k;
  const int n_items = ceil_div(p.seqlen_k, kBlk) * p.h_k * p.b;
  const uint32_t k_smem = base, v_smem = base + kTileBytes, ring = base + 2 * kTileBytes;  // stage s: Q at ring + s * 32 KiB, dO behind it
  BarA* bar = reinterpret_cast<BarA*>(smem + 7 * kTileBytes);
  if (tid == 0) {
    mbar_init(smem_addr(&bar->kv_full), 1);
    mbar_init(smem_addr(&bar->kv_empty), 2);        // one commit per issuing warp
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_addr(&bar->qdo_full[s]), 1);
      mbar_init(smem_addr(&bar->qdo_empty[s]), 2);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_addr(&bar->st_full[b]), 2);
      mbar_init(smem_addr(&bar->pds_full[b]), kEwWarps / 2);  // the half of the elementwise warps that owns the buffer
    }
    mbar_init(smem_addr(&bar->acc_done), 2);
    mbar_init(smem_addr(&bar->acc_free), kEwWarps);
    for (int k = 0; k < kQueue; ++k) mbar_init(smem_addr(&bar->queue.full[k]), 1);
    bar->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_addr(&bar->tmem_base), 512);
    tmem_relinquish();
  }
  if (warp == kTmaWarp && lane == 0) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_do);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = __shfl_sync(0xffffffffu, bar->tmem_base, 0);
  volatile int* abort_flag = &bar->abort_flag;
  // Every role walks over the same items and keeps the same two counters: wi = items with work so far (phase of the
  // per-item barriers), gu = units so far (ring stage, TMEM buffer and their phases).
  uint32_t wi = 0, gu = 0;

  if (warp == kTmaWarp) {
    // ------------------------------------------------------------------ producer
    bool ok = true;
    while (ok) {
      const int t = queue_draw(counter, n_items, lane);
      if (t < 0) break;
      const ItemA w = item_a(p, t);
      if (!w.live) continue;
      const SeqInfo& sq = w.sq;
      if (w.iters == 0) {  // nobody sees these keys: dK = dV = 0
        T* dk0 = reinterpret_cast<T*>(p.dk) + (int64_t)sq.bq * p.dk_batch_stride + (int64_t)(sq.k_row0 + w.key0) * p.dk_row_stride +
                 (int64_t)w.hk * p.dk_head_stride;
        T* dv0 = reinterpret_cast<T*>(p.dv) + (int64_t)sq.bq * p.dv_batch_stride + (int64_t)(sq.k_row0 + w.key0) * p.dv_row_stride +
                 (int64_t)w.hk * p.dv_head_stride;
        for (int c = lane; c < kBlk * 16; c += 32) {
          const int r = c >> 4, ch = c & 15;
          if (w.key0 + r < sq.k_len && ch * 8 < p.d) {
            *reinterpret_cast<uint4*>(dk0 + (int64_t)r * p.dk_row_stride + ch * 8) = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(dv0 + (int64_t)r * p.dv_row_stride + ch * 8) = make_uint4(0, 0, 0, 0);
          }
        }
        continue;
      }
      queue_publish(&bar->queue, wi, t, lane);
      if (!mbar_wait(smem_addr(&bar->kv_empty), (wi & 1) ^ 1, abort_flag, 60)) break;
      if (elect_one()) {
        const uint32_t full = smem_addr(&bar->kv_full);
        mbar_arrive_expect_tx(full, 2 * (HD / 64) * kHalfBytes);
        tma_load_4d(k_smem, &tm_k, full, 0, w.hk, sq.k_row0 + w.key0, sq.bq);
        if (HD > 64) tma_load_4d(k_smem + kHalfBytes, &tm_k, full, 64, w.hk, sq.k_row0 + w.key0, sq.bq);
        tma_load_4d(v_smem, &tm_v, full, 0, w.hk, sq.k_row0 + w.key0, sq.bq);
        if (HD > 64) tma_load_4d(v_smem + kHalfBytes, &tm_v, full, 64, w.hk, sq.k_row0 + w.key0, sq.bq);
      }
      __syncwarp();
      for (int it = 0; it < w.iters; ++it) {
        const uint32_t g = gu + it;
        const int s = g % kStages, head = w.hk * group + it / w.nu, row0 = (w.u_lo + it % w.nu) * kUnit;
        if (!mbar_wait(smem_addr(&bar->qdo_empty[s]), ((g / kStages) & 1) ^ 1, abort_flag, 61)) { ok = false; break; }
        for (int r = lane; r < kUnit; r += 32) {
          const int i = row0 + r;
          const int64_t li = (int64_t)sq.bq * p.lse_batch_stride + (int64_t)head * p.lse_head_stride + sq.q_row0 + i;
          bar->nlse2[s][r] = i < sq.q_len ? -p.lse[li] * kLog2e : -INFINITY;  // rows beyond the sequence: P = 0
          bar->ndls[s][r] = i < sq.q_len ? -p.delta[li] * p.softmax_scale : 0.f;
        }
        __syncwarp();
        if (elect_one()) {
          const uint32_t full = smem_addr(&bar->qdo_full[s]);
          const uint32_t q_dst = ring + s * 2 * kUnitTile, do_dst = q_dst + kUnitTile;
          mbar_arrive_expect_tx(full, 2 * (HD / 64) * kUnitHalf);
          tma_load_4d(q_dst, &tm_q, full, 0, head, sq.q_row0 + row0, sq.bq);
          if (HD > 64) tma_load_4d(q_dst + kUnitHalf, &tm_q, full, 64, head, sq.q_row0 + row0, sq.bq);
          tma_load_4d(do_dst, &tm_do, full, 0, head, sq.q_row0 + row0, sq.bq);
          if (HD > 64) tma_load_4d(do_dst + kUnitHalf, &tm_do, full, 64, head, sq.q_row0 + row0, sq.bq);
        }
        __syncwarp();
      }
      ++wi;
      gu += w.iters;
    }
    queue_publish(&bar->queue, wi, -1, lane);  // (after an abort too: the others are leaving through the abort flag anyway)
  } else if (warp == kMmaWarp || warp == kMmaWarp + 1) {
    // ------------------------------------------------------------------ MMA issuers: chain 0 = S^T, dV; chain 1 = dP^T, dK
    // Issue order of a chain:  ST(0) | ST(1) DV(0) | ST(2) DV(1) | ...  ST(u + 2) overwrites the buffer whose P^T / dS^T
    // DV(u) reads: both come from this warp, in this order, and the tensor pipe keeps the order.
    const int r = warp - kMmaWarp;
    constexpr uint32_t idesc_st = make_idesc(AB_FMT, kBlk, kUnit, 0);  // [128 keys] x [64 rows], both operands K-major
    constexpr uint32_t idesc_acc = make_idesc(AB_FMT, kBlk, HD, 1);    // [128 keys] x [head dim], B N-contiguous
    const uint64_t a_desc = make_smem_desc(r ? v_smem : k_smem, 16, 1024);                    // K (S^T = K Q^T) or V (dP^T = V dO^T)
    const uint64_t b_desc0 = make_smem_desc(ring + (r ? kUnitTile : 0), 16, 1024);            // Q or dO of stage 0, K-major
    const uint64_t b_nd0 = make_smem_desc(ring + (r ? 0 : kUnitTile), kUnitHalf, 1024);       // dO (dV += P^T dO) or Q (dK += dS^T Q), N-contiguous
    constexpr uint64_t kStageStep = (2 * kUnitTile) >> 4;
    // K-major unit tile: k-step ks (16 columns) at (ks >> 2) * 8 KiB + (ks & 3) * 32 bytes
    auto unit_off = [](int ks) { return (uint64_t)(((ks >> 2) * kUnitHalf + (ks & 3) * 32) >> 4); };
    const uint32_t acc_tmem = tmem + 256 + 128 * r;
    const uint32_t bar_stfull0 = smem_addr(&bar->st_full[0]), bar_pds0 = smem_addr(&bar->pds_full[0]);
    const uint32_t bar_full0 = smem_addr(&bar->qdo_full[0]), bar_empty0 = smem_addr(&bar->qdo_empty[0]);
    const uint32_t bar_kvempty = smem_addr(&bar->kv_empty), bar_accdone = smem_addr(&bar->acc_done);
    bool ok = true;
    while (ok) {
      const int t = queue_get(&bar->queue, wi, abort_flag);
      if (t < 0) break;
      const ItemA w = item_a(p, t);
      const int iters = w.iters;
      auto issue_st = [&](int u) -> bool {
        const uint32_t g = gu + u;
        const int s = g % kStages, b = g & 1;
        if (!mbar_wait(bar_full0 + 8 * s, (g / kStages) & 1, abort_flag, 63)) return false;
        tc_fence_after();
        if (elect_one()) {
          const uint64_t b_desc = b_desc0 + (uint64_t)s * kStageStep;
          const uint32_t d_tmem = tmem + 128 * b + 64 * r;
          mma_ss_c<false>(d_tmem, a_desc, b_desc, idesc_st);
#pragma unroll
          for (int ks = 1; ks < HD / 16; ++ks) mma_ss_c<true>(d_tmem, a_desc + kmaj_off(ks), b_desc + unit_off(ks), idesc_st);
          mma_commit(bar_stfull0 + 8 * b);
          if (u == iters - 1) mma_commit(bar_kvempty);  // the item's last reader of K / V
        }
        __syncwarp();
        return true;
      };
      if (!mbar_wait(smem_addr(&bar->kv_full), wi & 1, abort_flag, 62)) break;
      if (!issue_st(0)) break;
      for (int u = 0; u < iters; ++u) {
        if (u + 1 < iters && !issue_st(u + 1)) { ok = false; break; }
        const uint32_t g = gu + u;
        const int s = g % kStages, b = g & 1;
        if (!mbar_wait(bar_pds0 + 8 * b, (g >> 1) & 1, abort_flag, 64)) { ok = false; break; }
        // the epilogue of the previous item must have the accumulators in registers
        if (u == 0 && !mbar_wait(smem_addr(&bar->acc_free), (wi & 1) ^ 1, abort_flag, 68)) { ok = false; break; }
        tc_fence_after();
        if (elect_one()) {
          const uint64_t b_nd = b_nd0 + (uint64_t)s * kStageStep;
          const uint32_t src = tmem + 128 * b + 64 * r;
          // k-step ks = query rows 16 ks .. 16 ks + 15 of the unit: the 8 packed columns their thread wrote inside its own 32
          if (u == 0) mma_ts_c<false>(acc_tmem, src, b_nd, idesc_acc);
          else mma_ts_c<true>(acc_tmem, src, b_nd, idesc_acc);
#pragma unroll
          for (int ks = 1; ks < 4; ++ks) mma_ts_c<true>(acc_tmem, src + 32 * (ks >> 1) + 8 * (ks & 1), b_nd + nmaj_off(ks), idesc_acc);
          mma_commit(bar_empty0 + 8 * s);
          if (u == iters - 1) mma_commit(bar_accdone);
        }
        __syncwarp();
      }
      ++wi;
      gu += iters;
    }
  } else if (warp > kMmaWarp + 1) {
    // spare issuing warp of the dQ kernel's layout: nothing to do here
  } else {
    // ------------------------------------------------------------------ elementwise: lane = key, 32 query rows per thread
    // Warps 0-7 take the even units (buffer 0), warps 8-15 the odd ones (buffer 1): two independent chains of
    // wait / load / compute / store / signal, so that one's latencies lie under the other's arithmetic.
    const int kr = (warp & 3) * 32 + lane, q2 = (warp >> 2) & 1, grp = warp >> 3, q4 = warp >> 2;
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const float a1 = SOFTCAP ? p.softmax_scale / p.softcap : p.scale_log2, cap1 = p.softcap * kLog2e;
    const uint64_t sl2 = pack_f32x2(a1, a1), cap2 = pack_f32x2(cap1, cap1), sc2 = pack_f32x2(p.softmax_scale, p.softmax_scale);
    const uint32_t st_tmem = tmem + lane_addr + 128 * grp + 32 * q2;  // this thread's 32 columns of S^T; dP^T 64 columns on
    auto unit = [&](auto mask_tag, int s, uint32_t bits) {
      constexpr bool MASK = decltype(mask_tag)::value;
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        uint32_t sv[16], dv[16];
        tmem_ld16(st_tmem + 16 * hf, sv);
        tmem_ld16(st_tmem + 64 + 16 * hf, dv);
        tmem_wait_ld();
        uint32_t pk_p[8], pk_ds[8];
#pragma unroll
        for (int e4 = 0; e4 < 16; e4 += 4) {
          const float4 l4 = *reinterpret_cast<const float4*>(&bar->nlse2[s][32 * q2 + 16 * hf + e4]);
          const float4 d4 = *reinterpret_cast<const float4*>(&bar->ndls[s][32 * q2 + 16 * hf + e4]);
          ew_pair<T, MASK, SOFTCAP>(((e4 >> 1) & 3) < kPolyPairs, sv[e4], sv[e4 + 1], dv[e4], dv[e4 + 1], sl2, cap2, pack_f32x2(l4.x, l4.y), sc2,
                           pack_f32x2(d4.x, d4.y), bits, 16 * hf + e4, pk_p[e4 >> 1], pk_ds[e4 >> 1]);
          ew_pair<T, MASK, SOFTCAP>((((e4 >> 1) + 1) & 3) < kPolyPairs, sv[e4 + 2], sv[e4 + 3], dv[e4 + 2], dv[e4 + 3], sl2, cap2,
                           pack_f32x2(l4.z, l4.w), sc2, pack_f32x2(d4.z, d4.w), bits, 16 * hf + e4 + 2, pk_p[(e4 >> 1) + 1],
                           pk_ds[(e4 >> 1) + 1]);
        }
        // into the columns this thread has already read (the first 16 of its 32): nobody else's data
        tmem_st8(st_tmem + 8 * hf, pk_p);
        tmem_st8(st_tmem + 64 + 8 * hf, pk_ds);
      }
    };
    bool ok = true;
    while (ok) {
      const int t = queue_get(&bar->queue, wi, abort_flag);
      if (t < 0) break;
      const ItemA w = item_a(p, t);
      const SeqInfo& sq = w.sq;
      const int key0 = w.key0, jk = key0 + kr;
      T* dk_row = reinterpret_cast<T*>(p.dk) + (int64_t)sq.bq * p.dk_batch_stride + (int64_t)(sq.k_row0 + jk) * p.dk_row_stride +
                  (int64_t)w.hk * p.dk_head_stride + 32 * q4;
      T* dv_row = reinterpret_cast<T*>(p.dv) + (int64_t)sq.bq * p.dv_batch_stride + (int64_t)(sq.k_row0 + jk) * p.dv_row_stride +
                  (int64_t)w.hk * p.dv_head_stride + 32 * q4;
      // query rows that see this key
      const int vis_lo = sq.wr >= 0 ? jk - sq.koff - sq.wr : -0x40000000;
      const int vis_hi = jk < sq.k_len ? (sq.wl >= 0 ? jk - sq.koff + sq.wl : 0x40000000) : -0x40000001;
      for (int u = (int)((grp - gu) & 1u); u < w.iters; u += 2) {  // the units whose running number has this group's parity
        const uint32_t g = gu + u;
        const int s = g % kStages, r0 = (w.u_lo + u % w.nu) * kUnit, i0 = r0 + 32 * q2;
        if (!mbar_wait(smem_addr(&bar->qdo_full[s]), (g / kStages) & 1, abort_flag, 65)) { ok = false; break; }  // LSE / D of the stage
        if (!mbar_wait(smem_addr(&bar->st_full[grp]), (g >> 1) & 1, abort_flag, 66)) { ok = false; break; }
        tc_fence_after();
        // does any (key of the block, query row of the unit) pair fall outside the mask?  (the same answer in every thread;
        // rows beyond the sequence need no mask: their -LSE is -inf)
        bool need_mask = key0 + kBlk > sq.k_len;
        if (sq.wr >= 0) need_mask = need_mask || (key0 + kBlk - 1 > r0 + sq.koff + sq.wr);
        if (sq.wl >= 0) need_mask = need_mask || (key0 < min(sq.q_len, r0 + kUnit) - 1 + sq.koff - sq.wl);
        if (need_mask) unit(std::true_type{}, s, range_bits(i0, vis_lo, vis_hi));
        else unit(std::false_type{}, s, 0xffffffffu);
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_addr(&bar->pds_full[grp]));
      }
      if (!ok) break;
      // ---- epilogue: dV, dK of this key, 32 columns of the head dim; the accumulators are handed back once they are in
      // registers, the stores run under the next item's first products
      if (!mbar_wait(smem_addr(&bar->acc_done), wi & 1, abort_flag, 67)) break;
      tc_fence_after();
      uint32_t av[32], ak[32];
      tmem_ld32(tmem + lane_addr + 256 + 32 * q4, av);
      tmem_ld32(tmem + lane_addr + 384 + 32 * q4, ak);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_addr(&bar->acc_free));
      if (jk < sq.k_len) {
        store_slice<T>(dv_row, av, p.d - 32 * q4);
        store_slice<T>(dk_row, ak, p.d - 32 * q4);
      }
      ++wi;
      gu += w.iters;
    }
  }

  tc_fence_before();
  __syncthreads();
  finish(status, bar->abort_flag, tid);
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// =================================================================================================
// dQ
// =================================================================================================
struct BarB {
  uint64_t qdo_full, qdo_empty;  // Q / dO of the item have landed; the item's last S / dP have read them
  uint64_t kv_full[kDqSlots], kv_empty[kDqSlots];
  uint64_t s_full;    // MMA -> elementwise: S and dP are in TMEM
  uint64_t s_free;    // elementwise -> MMA: S and dP are in registers
  uint64_t ds_full;   // elementwise -> MMA: dS is in TMEM
  uint64_t ds_free;   // MMA -> elementwise: dQ += dS K has read dS
  uint64_t acc_done;  // MMA -> epilogue: dQ of the item is complete
  uint64_t acc_free;  // epilogue -> MMA: dQ is in registers
  ItemQueue queue;
  uint32_t tmem_base;
  int abort_flag;
  float nlse2[2][kBlk], ndls[2][kBlk];  // by item parity: -LSE * log2(e) and -D * scale of the block's query rows
};
static_assert(sizeof(BarB) <= kBarBytes, "barrier block does not fit");

// Work item t of the dQ kernel: 128 query rows of one (head, batch entry); the query blocks of a pair are neighbours
// in the order (they stream the same K / V), the last one (under a causal mask: the heaviest) first.
struct ItemB {
  SeqInfo sq;
  int head, hk, bi, row0, j_lo, iters;  // iters = key blocks; 0 = the rows see no key
  bool live;
};
__device__ __forceinline__ ItemB item_b(const BwdParams& p, int t) {
  ItemB w;
  const int m_blocks = ceil_div(p.seqlen_q, kBlk);
  const int pair = t / m_blocks, mi = t - pair * m_blocks;
  w.head = pair % p.h;
  w.bi = pair / p.h;
  w.hk = w.head / (p.h / p.h_k);
  w.sq = seq_info(p, w.bi);
  w.row0 = (m_blocks - 1 - mi) * kBlk;
  w.live = w.row0 < w.sq.q_len;
  w.j_lo = w.iters = 0;
  if (w.live) {
    // keys that at least one row of the block sees
    const int r1 = min(w.sq.q_len, w.row0 + kBlk) - 1;
    const int k_hi = w.sq.wr >= 0 ? min(w.sq.k_len - 1, r1 + w.sq.koff + w.sq.wr) : w.sq.k_len - 1;  // inclusive
    const int k_lo = w.sq.wl >= 0 ? max(0, w.row0 + w.sq.koff - w.sq.wl) : 0;
    w.j_lo = k_lo / kBlk;
    w.iters = k_hi >= k_lo ? k_hi / kBlk + 1 - w.j_lo : 0;
  }
  return w;
}

template <typename T, uint32_t AB_FMT, bool SOFTCAP, int HD>
__global__ void __launch_bounds__(kThreads, 1)
bwd_dq_kernel(const __grid_constant__ BwdParams p, const __grid_constant__ CUtensorMap tm_q,
              const __grid_constant__ CUtensorMap tm_do, const __grid_constant__ CUtensorMap tm_k,
              const __grid_constant__ CUtensorMap tm_v, int32_t* status, int32_t* counter) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t base = smem_addr(smem);
  const int tid = threadIdx.x, lane = tid & 31;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
  if ((base & 1023u) != 0) {
    if (tid == 0) atomicExch(status, 0x20000000);
    return;
  }
  const int n_items = ceil_div(p.seqlen_q, kBlk) * p.h * p.b;
  const uint32_t q_smem = base, do_smem = base + kTileBytes, ring = base + 2 * kTileBytes;
  BarB* bar = reinterpret_cast<BarB*>(smem + 7 * kTileBytes);
  if (tid == 0) {
    mbar_init(smem_addr(&bar->qdo_full), 1);
    mbar_init(smem_addr(&bar->qdo_empty), 2);      // the S and the dP issuer
    for (int s = 0; s < kDqSlots; ++s) {
      mbar_init(smem_addr(&bar->kv_full[s]), 1);
      mbar_init(smem_addr(&bar->kv_empty[s]), 2);  // K: the S and the dQ issuer; V: the dP issuer, twice
    }
    mbar_init(smem_addr(&bar->s_full), 2);           // S and dP
    mbar_init(smem_addr(&bar->s_free), kEwWarps);
    mbar_init(smem_addr(&bar->ds_full), kEwWarps);
    mbar_init(smem_addr(&bar->ds_free), 1);
    mbar_init(smem_addr(&bar->acc_done), 1);
    mbar_init(smem_addr(&bar->acc_free), kEwWarps);
    for (int k = 0; k < kQueue; ++k) mbar_init(smem_addr(&bar->queue.full[k]), 1);
    bar->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_addr(&bar->tmem_base), 512);
    tmem_relinquish();
  }
  if (warp == kTmaWarp && lane == 0) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_do);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = __shfl_sync(0xffffffffu, bar->tmem_base, 0);
  volatile int* abort_flag = &bar->abort_flag;
  // wi = items with work so far (phase of the per-item barriers), gj = key blocks so far (ring slots and the phases of
  // the per-block barriers): the same in every role
  uint32_t wi = 0, gj = 0;

  if (warp == kTmaWarp) {
    // ------------------------------------------------------------------ producer
    bool ok = true;
    while (ok) {
      const int t = queue_draw(counter, n_items, lane);
      if (t < 0) break;
      const ItemB w = item_b(p, t);
      if (!w.live) continue;
      const SeqInfo& sq = w.sq;
      if (w.iters == 0) {  // these rows see no key: dQ = 0
        T* dq0 = reinterpret_cast<T*>(p.dq) + (int64_t)sq.bq * p.dq_batch_stride + (int64_t)(sq.q_row0 + w.row0) * p.dq_row_stride +
                 (int64_t)w.head * p.dq_head_stride;
        for (int c = lane; c < kBlk * 16; c += 32) {
          const int r = c >> 4, ch = c & 15;
          if (w.row0 + r < sq.q_len && ch * 8 < p.d) *reinterpret_cast<uint4*>(dq0 + (int64_t)r * p.dq_row_stride + ch * 8) = make_uint4(0, 0, 0, 0);
        }
        continue;
      }
      queue_publish(&bar->queue, wi, t, lane);
      if (!mbar_wait(smem_addr(&bar->qdo_empty), (wi & 1) ^ 1, abort_flag, 70)) break;
      for (int r = lane; r < kBlk; r += 32) {
        const int i = w.row0 + r;
        const int64_t li = (int64_t)sq.bq * p.lse_batch_stride + (int64_t)w.head * p.lse_head_stride + sq.q_row0 + i;
        bar->nlse2[wi & 1][r] = i < sq.q_len ? -p.lse[li] * kLog2e : -INFINITY;
        bar->ndls[wi & 1][r] = i < sq.q_len ? -p.delta[li] * p.softmax_scale : 0.f;
      }
      __syncwarp();
      if (elect_one()) {
        const uint32_t full = smem_addr(&bar->qdo_full);
        mbar_arrive_expect_tx(full, 2 * (HD / 64) * kHalfBytes);
        tma_load_4d(q_smem, &tm_q, full, 0, w.head, sq.q_row0 + w.row0, sq.bq);
        if (HD > 64) tma_load_4d(q_smem + kHalfBytes, &tm_q, full, 64, w.head, sq.q_row0 + w.row0, sq.bq);
        tma_load_4d(do_smem, &tm_do, full, 0, w.head, sq.q_row0 + w.row0, sq.bq);
        if (HD > 64) tma_load_4d(do_smem + kHalfBytes, &tm_do, full, 64, w.head, sq.q_row0 + w.row0, sq.bq);
      }
      __syncwarp();
      // K(j) lives in slot j % 3 and is held until dQ += dS K of its block has run; V(j) in slot 3 + j % 2 until dP has
      for (int it = 0; it < 2 * w.iters; ++it) {  // K(j), V(j), K(j + 1), ...
        const uint32_t g = gj + (it >> 1);
        const int is_v = it & 1;
        const uint32_t slot = is_v ? kDqKSlots + (g & 1) : g % kDqKSlots;
        const uint32_t par = is_v ? (g >> 1) & 1 : (g / kDqKSlots) & 1;
        const int krow = sq.k_row0 + (w.j_lo + (it >> 1)) * kBlk;
        const CUtensorMap* tm = is_v ? &tm_v : &tm_k;
        if (!mbar_wait(smem_addr(&bar->kv_empty[slot]), par ^ 1, abort_flag, 71)) { ok = false; break; }
        if (elect_one()) {
          const uint32_t full = smem_addr(&bar->kv_full[slot]);
          mbar_arrive_expect_tx(full, (HD / 64) * kHalfBytes);
          tma_load_4d(ring + slot * kTileBytes, tm, full, 0, w.hk, krow, sq.bq);
          if (HD > 64) tma_load_4d(ring + slot * kTileBytes + kHalfBytes, tm, full, 64, w.hk, krow, sq.bq);
        }
        __syncwarp();
      }
      ++wi;
      gj += w.iters;
    }
    queue_publish(&bar->queue, wi, -1, lane);
  } else if (warp == kMmaWarp || warp == kMmaWarp + 1) {
    // ------------------------------------------------------------------ MMA issuers 0 / 1: S = Q K^T / dP = dO V^T
    const int r = warp - kMmaWarp;
    constexpr uint32_t idesc_kk = make_idesc(AB_FMT, kBlk, kBlk, 0);
    const uint64_t a_desc = make_smem_desc(r ? do_smem : q_smem, 16, 1024);
    const uint64_t ring_kd = make_smem_desc(ring, 16, 1024);
    constexpr uint64_t kSlotStep = kTileBytes >> 4;
    const uint32_t bar_full0 = smem_addr(&bar->kv_full[0]), bar_empty0 = smem_addr(&bar->kv_empty[0]);
    const uint32_t bar_sfull = smem_addr(&bar->s_full), bar_sfree = smem_addr(&bar->s_free);
    const uint32_t bar_qdoempty = smem_addr(&bar->qdo_empty);
    const uint32_t d_tmem = tmem + 128 * r;
    bool ok = true;
    while (ok) {
      const int t = queue_get(&bar->queue, wi, abort_flag);
      if (t < 0) break;
      const ItemB w = item_b(p, t);
      if (!mbar_wait(smem_addr(&bar->qdo_full), wi & 1, abort_flag, 73)) break;
      for (int it = 0; it < w.iters; ++it) {
        const uint32_t g = gj + it;
        const uint32_t slot = r ? kDqKSlots + (g & 1) : g % kDqKSlots;  // V(g) or K(g)
        const uint32_t par = r ? (g >> 1) & 1 : (g / kDqKSlots) & 1;
        if (!mbar_wait(bar_full0 + 8 * slot, par, abort_flag, 74)) { ok = false; break; }
        if (g > 0 && !mbar_wait(bar_sfree, (g - 1) & 1, abort_flag, 76)) { ok = false; break; }
        tc_fence_after();
        if (elect_one()) {
          const uint64_t b_desc = ring_kd + slot * kSlotStep;
          mma_ss_c<false>(d_tmem, a_desc, b_desc, idesc_kk);
#pragma unroll
          for (int ks = 1; ks < HD / 16; ++ks) mma_ss_c<true>(d_tmem, a_desc + kmaj_off(ks), b_desc + kmaj_off(ks), idesc_kk);
          mma_commit(bar_sfull);
          mma_commit(bar_empty0 + 8 * slot);
          if (r) mma_commit(bar_empty0 + 8 * slot);        // nobody else reads the V tile
          if (it == w.iters - 1) mma_commit(bar_qdoempty);   // the item's last reader of Q / dO
        }
        __syncwarp();
      }
      ++wi;
      gj += w.iters;
    }
  } else if (warp == kMmaWarp + 2) {
    // ------------------------------------------------------------------ MMA issuer 2: dQ += dS K
    constexpr uint32_t idesc_nn = make_idesc(AB_FMT, kBlk, HD, 1);  // [128 rows] x [head dim]
    const uint64_t ring_nd = make_smem_desc(ring, kHalfBytes, 1024);
    constexpr uint64_t kSlotStep = kTileBytes >> 4;
    const uint32_t bar_full0 = smem_addr(&bar->kv_full[0]), bar_empty0 = smem_addr(&bar->kv_empty[0]);
    const uint32_t bar_dsfull = smem_addr(&bar->ds_full), bar_dsfree = smem_addr(&bar->ds_free);
    bool ok = true;
    while (ok) {
      const int t = queue_get(&bar->queue, wi, abort_flag);
      if (t < 0) break;
      const ItemB w = item_b(p, t);
      for (int it = 0; it < w.iters; ++it) {
        const uint32_t g = gj + it;
        const uint32_t slot = g % kDqKSlots, par = (g / kDqKSlots) & 1;
        if (!mbar_wait(bar_full0 + 8 * slot, par, abort_flag, 75)) { ok = false; break; }  // long complete: S of this block has used the tile
        if (!mbar_wait(bar_dsfull, g & 1, abort_flag, 72)) { ok = false; break; }
        // the epilogue of the previous item must have the accumulator in registers
        if (it == 0 && !mbar_wait(smem_addr(&bar->acc_free), (wi & 1) ^ 1, abort_flag, 69)) { ok = false; break; }
        tc_fence_after();
        if (elect_one()) {
          const uint64_t k_nd = ring_nd + slot * kSlotStep;
          if (it == 0) mma_ts_c<false>(tmem + 256, tmem + 384, k_nd, idesc_nn);
          else mma_ts_c<true>(tmem + 256, tmem + 384, k_nd, idesc_nn);
#pragma unroll
          for (int ks = 1; ks < 8; ++ks) mma_ts_c<true>(tmem + 256, tmem + 384 + 8 * ks, k_nd + nmaj_off(ks), idesc_nn);
          mma_commit(bar_dsfree);
          mma_commit(bar_empty0 + 8 * slot);
          if (it == w.iters - 1) mma_commit(smem_addr(&bar->acc_done));
        }
        __syncwarp();
      }
      ++wi;
      gj += w.iters;
    }
  } else {
    // ------------------------------------------------------------------ elementwise: lane = query row, 32 keys per thread
    const int r = (warp & 3) * 32 + lane, q4 = warp >> 2;
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const float a1 = SOFTCAP ? p.softmax_scale / p.softcap : p.scale_log2, cap1 = p.softcap * kLog2e;
    const uint64_t sl2 = pack_f32x2(a1, a1), cap2 = pack_f32x2(cap1, cap1), sc2 = pack_f32x2(p.softmax_scale, p.softmax_scale);
    bool ok = true;
    while (ok) {
      const int t = queue_get(&bar->queue, wi, abort_flag);
      if (t < 0) break;
      const ItemB w = item_b(p, t);
      const SeqInfo& sq = w.sq;
      const int row0 = w.row0, i = row0 + r;
      T* dq_row = reinterpret_cast<T*>(p.dq) + (int64_t)sq.bq * p.dq_batch_stride + (int64_t)(sq.q_row0 + i) * p.dq_row_stride +
                  (int64_t)w.head * p.dq_head_stride + 32 * q4;
      int hi = sq.k_len - 1, lo = 0;
      if (sq.wr >= 0) hi = min(hi, i + sq.koff + sq.wr);
      if (sq.wl >= 0) lo = max(0, i + sq.koff - sq.wl);
      if (!mbar_wait(smem_addr(&bar->qdo_full), wi & 1, abort_flag, 77)) break;
      const float nl = bar->nlse2[wi & 1][r], nd = bar->ndls[wi & 1][r];
      const uint64_t nlse2 = pack_f32x2(nl, nl), ndls2 = pack_f32x2(nd, nd);
      const int i_max = min(sq.q_len, row0 + kBlk) - 1;
      for (int it = 0; it < w.iters; ++it) {
        const uint32_t g = gj + it;
        if (!mbar_wait(smem_addr(&bar->s_full), g & 1, abort_flag, 78)) { ok = false; break; }
        tc_fence_after();
        uint32_t sv[32], dv[32];
        tmem_ld32(tmem + lane_addr + 32 * q4, sv);
        tmem_ld32(tmem + lane_addr + 128 + 32 * q4, dv);
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_addr(&bar->s_free));  // the products of the next block may overwrite S and dP
        const int c0 = (w.j_lo + it) * kBlk;
        // does any (row of the block, key of the block) pair fall outside the mask?  (the same answer in every thread)
        bool need_mask = c0 + kBlk > sq.k_len;
        if (sq.wr >= 0) need_mask = need_mask || (c0 + kBlk - 1 > row0 + sq.koff + sq.wr);
        if (sq.wl >= 0) need_mask = need_mask || (c0 < i_max + sq.koff - sq.wl);
        uint32_t pk[16], unused;
        if (need_mask) {
          const uint32_t bits = range_bits(c0 + 32 * q4, lo, hi);
#pragma unroll
          for (int e = 0; e < 32; e += 2)
            ew_pair<T, true, SOFTCAP>(((e >> 1) & 3) < kPolyPairs, sv[e], sv[e + 1], dv[e], dv[e + 1], sl2, cap2, nlse2, sc2, ndls2, bits, e, unused, pk[e >> 1]);
        } else {
#pragma unroll
          for (int e = 0; e < 32; e += 2)
            ew_pair<T, false, SOFTCAP>(((e >> 1) & 3) < kPolyPairs, sv[e], sv[e + 1], dv[e], dv[e + 1], sl2, cap2, nlse2, sc2, ndls2, 0u, e, unused, pk[e >> 1]);
        }
        if (g > 0 && !mbar_wait(smem_addr(&bar->ds_free), (g - 1) & 1, abort_flag, 79)) { ok = false; break; }
        tc_fence_after();
        tmem_st16(tmem + lane_addr + 384 + 16 * q4, pk);
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_addr(&bar->ds_full));
      }
      if (!ok) break;
      // ---- epilogue: the accumulator is handed back once it is in registers
      if (!mbar_wait(smem_addr(&bar->acc_done), wi & 1, abort_flag, 80)) break;
      tc_fence_after();
      uint32_t a[32];
      tmem_ld32(tmem + lane_addr + 256 + 32 * q4, a);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_addr(&bar->acc_free));
      if (i < sq.q_len) store_slice<T>(dq_row, a, p.d - 32 * q4);
      ++wi;
      gj += w.iters;
    }
  }

  tc_fence_before();
  __syncthreads();
  finish(status, bar->abort_flag, tid);
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace btc5
}  // namespace fa
