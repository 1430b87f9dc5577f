// tcgen05 / TMEM / TMA prefill kernel: entry point, TMA descriptors, launch.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <type_traits>

#include "fwd_tc5_roles.cuh"
#include "fwd_tc5_softmax.cuh"
#include "tc5_api.cuh"

namespace fa {
namespace tc5 {

// FIX: the input is a KV cache or packed sequences, where the rows behind the last key of a sequence hold foreign
// data: warp 15 clears them in the last V tile (tail_fix_loop) and the producer checks the index tensors.  Dense
// input needs neither, and its instance carries none of that code (the issuing warps' instruction stream is on
// the kernel's critical path: measured 3-8 % on causal 4K).
template <typename T, uint32_t AB_FMT, bool FIX, bool SOFTCAP, int HD>
__global__ void __launch_bounds__(kThreads, 1)
fwd_tc5_kernel(const __grid_constant__ Tc5Params p, const __grid_constant__ CUtensorMap tm_q,
               const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v) {
  // 128-byte-swizzled tiles need 1024-byte aligned bases; the whole 227 KiB are in use, so the base
  // itself must be aligned (checked below) instead of being rounded up.
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t base = smem_addr(smem);
  if ((base & 1023u) != 0) {
    if (threadIdx.x == 0) atomicExch(p.status, 0x20000000);
    return;
  }
  const uint32_t q_smem = base;
  const uint32_t p_smem = base + 2 * kTileBytes;
  const uint32_t kv_smem = base + Geo<HD>::kRingOff;
  Barriers* bar = reinterpret_cast<Barriers*>(smem + 4 * kTileBytes + kSlots * kTileBytes);

  // The warp index and the TMEM base are broadcast from lane 0 so that the compiler knows they are
  // warp-uniform: everything the MMA / TMA roles derive from them (barrier addresses, descriptors,
  // TMEM addresses) can then live on the uniform datapath, which is what tcgen05.mma reads.
  const int tid = threadIdx.x, lane = tid & 31;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
  if (tid == 0) {
    for (int t = 0; t < 2; ++t) {
      mbar_init(smem_addr(&bar->q_full[t]), 1);
      mbar_init(smem_addr(&bar->q_empty[t]), 1);
      mbar_init(smem_addr(&bar->s_full[t]), 1);
      mbar_init(smem_addr(&bar->s_free[t]), 4);
      mbar_init(smem_addr(&bar->p_full[t][0]), 4);
      mbar_init(smem_addr(&bar->p_full[t][1]), 4);
      mbar_init(smem_addr(&bar->corr_ready[t]), 4);
      mbar_init(smem_addr(&bar->o_ready[t]), 4);
      mbar_init(smem_addr(&bar->o_done[t]), 1);
      mbar_init(smem_addr(&bar->stats_ready[t]), 4);
      mbar_init(smem_addr(&bar->o_free[t]), 4);
    }
    for (int s = 0; s < kSlots; ++s) {
      mbar_init(smem_addr(&bar->kv_full[s]), 1);
      mbar_init(smem_addr(&bar->kv_empty[s]), 2);
    }
    mbar_init(smem_addr(&bar->fix_req), 2);
    mbar_init(smem_addr(&bar->v_fixed), 1);
    bar->abort_flag = 0;
    bar->fix_seen[0] = bar->fix_seen[1] = 0;
    fence_barrier_init();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_addr(&bar->tmem_base), 512);
    tmem_relinquish();
  }
  if (warp == kTmaWarp && lane == 0) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = __shfl_sync(0xffffffffu, bar->tmem_base, 0);

  // Register budget: 512 threads start with 128 registers each; the softmax warps need the 128
  // scores of a row plus working set, the other roles need far fewer.
  if (warp < 8) {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;\n" ::"n"(kRegsSoftmax));
    softmax_loop<T, SOFTCAP, Geo<HD>::kRows>(p, bar, tmem, p_smem, warp >> 2, warp & 3, lane);
  } else if (warp < 12) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;\n" ::"n"(kRegsCorr));
    correction_loop<T, HD>(p, bar, tmem, warp & 3, lane);
  } else {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;\n" ::"n"(kRegsMma));
    // warp-uniform role code; one elected lane issues
    if (warp == kMmaWarp || warp == kMmaWarp + 1) mma_loop<AB_FMT, FIX, HD>(p, bar, q_smem, p_smem, kv_smem, tmem, warp - kMmaWarp);
    else if (warp == kTmaWarp) producer_loop<FIX, HD>(p, &tm_q, &tm_k, &tm_v, bar, q_smem, kv_smem);
    else if (FIX) tail_fix_loop<HD>(p, bar, kv_smem, lane);
  }

  tc_fence_before();
  __syncthreads();
  const int aborted = bar->abort_flag;
  if (aborted) {
    // give copies that may still be in flight time to land before the shared memory is released
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
    if (tid == 0) atomicExch(p.status, (aborted << 16) | (1 + blockIdx.x));
    __syncthreads();
  }
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ------------------------------------------------------------------------------------------------
// host
// ------------------------------------------------------------------------------------------------
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeFn get_encode() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(ptr);
  });
  return fn;
}

// (d, heads, rows, batch) view of a (batch, rows, heads, d)-strided 16-bit tensor; box = 64 x 1 x 128 x 1.
static bool encode_map(CUtensorMap* m, const void* ptr, int dtype, int d, int heads, int64_t rows, int64_t batch,
                       int64_t head_stride, int64_t row_stride, int64_t batch_stride, int box_rows = kBlockN) {
  EncodeFn enc = get_encode();
  if (!enc) return false;
  cuuint64_t dims[4] = {(cuuint64_t)d, (cuuint64_t)heads, (cuuint64_t)rows, (cuuint64_t)batch};
  cuuint64_t strides[3] = {(cuuint64_t)head_stride * 2, (cuuint64_t)row_stride * 2, (cuuint64_t)batch_stride * 2};
  if (batch == 1) strides[2] = (cuuint64_t)rows * row_stride * 2;
  cuuint32_t box[4] = {64, 1, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(m, dtype == FA_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                   const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// The status word of the bounded waits and index checks: one per device, part of the library image (no
// allocation; 0 when the module is loaded).  In host code the symbol is only a handle; its device address is
// looked up once per device, with that device current.
static __device__ int32_t g_status_word;

static int32_t* status_word() {
  static int32_t* words[64] = {nullptr};
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!words[dev]) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_status_word) != cudaSuccess) return nullptr;
    words[dev] = static_cast<int32_t*>(ptr);
  }
  return words[dev];
}

}  // namespace tc5

bool tc5_eligible(const fa_fwd_params& a, bool is_causal, bool is_local, int wl_on_device) {
  (void)is_causal;
  (void)is_local;
  // any head dim up to 256 that keeps rows 16-byte aligned: the tiles are 64, 128 or 256 columns wide and the TMA
  // unit fills the columns beyond the head dim with zeros
  if (a.d < 8 || a.d > 256 || a.d % 8 != 0 || a.seqlen_q < 128) return false;
  // varlen: both sides packed, and the number of k / v rows known (TMA bound)
  if ((a.cu_seqlens_q != nullptr) != (a.cu_seqlens_k != nullptr)) return false;
  if (a.cu_seqlens_k && a.total_k <= 0) return false;
  // KV cache without append: per-entry lengths, contiguous or paged with whole 128-key blocks per page
  if ((a.seqused_k || a.block_table) && (a.cu_seqlens_q || !a.seqused_k)) return false;
  if (a.block_table && (a.page_size <= 0 || a.page_size % tc5::kBlockN != 0)) return false;
  // new tokens (and rotary) are served by a prologue launch in front of the kernel; they need the cache lengths
  if ((a.k_new || a.rotary_cos) && (!a.seqused_k || !a.k_new || !a.v_new)) return false;
  if (a.alibi_slopes || (a.cache_batch_idx && !a.seqused_k)) return false;
  // A left window that may cover every key of the batch (the rule that turns it into "causal" needs the longest
  // cache length, known on the device only) is simply kept as a window here: the mask is the same either way.
  // With rotary tables the mode also decides where q is rotated (per token or all at the cache length), and the
  // other kernels decide that on the device: such calls are left to them so that every kernel gives one answer.
  if (wl_on_device && a.rotary_cos) return false;
  if (a.partial_out || a.kv_total > 0) return false;
  // TMA: 16-byte aligned bases and strides
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (!al(a.q) || !al(a.k) || !al(a.v) || !al(a.o)) return false;
  const int64_t st[] = {a.q_row_stride, a.q_head_stride, a.q_batch_stride, a.k_row_stride, a.k_head_stride,
                        a.k_batch_stride, a.v_row_stride, a.v_head_stride, a.v_batch_stride,
                        a.o_row_stride, a.o_head_stride, a.o_batch_stride};
  for (int64_t s : st)
    if (s % 8 != 0 || s < 0) return false;
  return true;
}

void tc5_fill_plan(const fa_fwd_params& a, fa_fwd_plan* pl) {
  const int tile_rows = a.d > 128 ? tc5::kBlockM : tc5::kTileM;  // Geo<HD>::kRows
  const int m_tiles = (a.seqlen_q + tile_rows - 1) / tile_rows;
  const long long total = (long long)m_tiles * a.b * a.h;
  int num_sm = a.num_sm;
  if (num_sm <= 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&num_sm, cudaDevAttrMultiProcessorCount, dev);
  }
  pl->kernel = FA_KERNEL_TCGEN05;
  pl->config = 0;
  pl->pack_gqa = 0;
  pl->block_m = tile_rows;
  pl->block_n = tc5::kBlockN;
  pl->m_blocks = m_tiles;
  pl->num_splits = 1;
  pl->blocks_per_split = 0;
  pl->grid = (int)std::min<long long>(total, num_sm > 0 ? num_sm : 148);
  pl->threads = tc5::kThreads;
  pl->smem_bytes = tc5::kSmemBytes;
  pl->launches = a.k_new ? 2 : 1;  // + the append / rotary prologue
  pl->workspace_bytes = a.rotary_cos ? (size_t)a.b * a.seqlen_q * a.h * a.d * 2 : 0;  // the rotated q
}

int tc5_launch(const fa_fwd_params& a, const fa_fwd_plan& pl, cudaStream_t st, std::string* err) {
  using namespace tc5;
  Tc5Params p;
  std::memset(&p, 0, sizeof(p));
  p.a = a;
  p.is_causal = pl.is_causal;
  p.is_local = pl.is_local;
  p.wl = pl.window_left;
  p.wr = pl.window_right;
  p.group = a.h / a.h_k;
  p.m_tiles = pl.m_blocks;
  p.total_tiles = pl.m_blocks * a.b * a.h;
  p.scale_log2 = a.softmax_scale * kLog2e;
  if (a.softcap > 0.f) {
    p.softcap_mul = a.softmax_scale / a.softcap;
    p.softcap_l2 = a.softcap * kLog2e;
  }
  p.fix_tail = (a.seqused_k || a.cu_seqlens_k) ? 1 : 0;
  {
    // L2 chunks of the tile order (tile_info).  A chunk is 2 * grid / gcd(2 * grid, m_tiles) pairs: a whole
    // even number of grid rounds.  Used when all K / V together would not stay in L2 but a chunk's does (packed
    // varlen input: judged by the longest sequence).
    const long long per_m = (long long)a.b * a.h;
    const long long kv_bytes_per_pair = 4LL * a.seqlen_k * a.d / std::max(1, a.h / a.h_k);  // K and V, shared by a group
    const long long l2_budget = 96LL << 20;
    auto gcd = [](long long x, long long y) { while (y) { const long long t = x % y; x = y; y = t; } return x; };
    long long chunk = 2LL * pl.grid / gcd(2LL * pl.grid, pl.m_blocks);
    if (const char* e = std::getenv("FA_B200_TC5_CHUNK")) chunk = std::atoll(e);  // tuning override (0: one chunk)
    else if (per_m * kv_bytes_per_pair <= l2_budget || chunk * kv_bytes_per_pair > l2_budget) chunk = per_m;
    if (chunk <= 0 || chunk > per_m) chunk = per_m;
    p.chunk_bh = (int)chunk;
  }
  p.status = status_word();
  if (!p.status) { *err = "cannot look up the device status word"; return FA_ERR_CUDA; }
  const bool varlen = a.cu_seqlens_q != nullptr;
  CUtensorMap tq, tk, tv;
  bool ok = true;
  if (varlen) {
    // Packed sequences: one row axis for the whole tensor.  A tile that runs past the end of its
    // sequence reads rows of the next one (masked by the key range, never stored), a tile that
    // runs past the end of the tensor reads the TMA fill value.
    ok = encode_map(&tq, a.q, a.dtype, a.d, a.h, a.total_q, 1, a.q_head_stride, a.q_row_stride, 0) &&
         encode_map(&tk, a.k, a.dtype, a.d, a.h_k, a.total_k, 1, a.k_head_stride, a.k_row_stride, 0) &&
         encode_map(&tv, a.v, a.dtype, a.d, a.h_k, a.total_k, 1, a.v_head_stride, a.v_row_stride, 0);
  } else if (a.block_table) {
    // (d, kv head, row in page, page): a block-table entry outside the pool reads zeros, not memory
    const int64_t n_pages = a.kv_outer;
    ok = encode_map(&tq, a.q, a.dtype, a.d, a.h, a.seqlen_q, a.b, a.q_head_stride, a.q_row_stride, a.q_batch_stride) &&
         encode_map(&tk, a.k, a.dtype, a.d, a.h_k, a.page_size, n_pages, a.k_head_stride, a.k_row_stride, a.k_batch_stride) &&
         encode_map(&tv, a.v, a.dtype, a.d, a.h_k, a.page_size, n_pages, a.v_head_stride, a.v_row_stride, a.v_batch_stride);
  } else {
    // with cache_batch_idx the cache may have more rows than the batch; an index outside it reads zeros
    const int64_t kv_batch = a.cache_batch_idx ? a.kv_outer : a.b;
    ok = encode_map(&tq, a.q, a.dtype, a.d, a.h, a.seqlen_q, a.b, a.q_head_stride, a.q_row_stride, a.q_batch_stride) &&
         encode_map(&tk, a.k, a.dtype, a.d, a.h_k, a.seqlen_k, kv_batch, a.k_head_stride, a.k_row_stride, a.k_batch_stride) &&
         encode_map(&tv, a.v, a.dtype, a.d, a.h_k, a.seqlen_k, kv_batch, a.v_head_stride, a.v_row_stride, a.v_batch_stride);
  }
  if (!ok) { *err = "cuTensorMapEncodeTiled failed"; return FA_ERR_CUDA; }
  cudaError_t e = cudaErrorInvalidValue;
  auto launch = [&](auto kern) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e == cudaSuccess) {
      kern<<<pl.grid, kThreads, kSmemBytes, st>>>(p, tq, tk, tv);
      e = cudaGetLastError();
    }
  };
  const bool bf = a.dtype == FA_BF16, cap = a.softcap > 0.f;
  auto pick = [&](auto fix_tag, auto cap_tag, auto hd_tag) {
    constexpr bool F = decltype(fix_tag)::value, C = decltype(cap_tag)::value;
    constexpr int HD = decltype(hd_tag)::value;
    if (bf) launch(fwd_tc5_kernel<__nv_bfloat16, 1, F, C, HD>);
    else launch(fwd_tc5_kernel<__half, 0, F, C, HD>);
  };
  auto pick_hd = [&](auto fix_tag, auto cap_tag) {
    if (a.d <= 64) pick(fix_tag, cap_tag, std::integral_constant<int, 64>{});
    else if (a.d <= 128) pick(fix_tag, cap_tag, std::integral_constant<int, 128>{});
    else pick(fix_tag, cap_tag, std::integral_constant<int, 256>{});
  };
  if (p.fix_tail) {
    if (cap) pick_hd(std::true_type{}, std::true_type{});
    else pick_hd(std::true_type{}, std::false_type{});
  } else {
    if (cap) pick_hd(std::false_type{}, std::true_type{});
    else pick_hd(std::false_type{}, std::false_type{});
  }
  if (e != cudaSuccess) { *err = std::string("tcgen05 kernel launch: ") + cudaGetErrorString(e); return FA_ERR_CUDA; }
  return FA_OK;
}

int32_t* device_status_word() { return tc5::status_word(); }

bool tma_encode_rows(CUtensorMap* m, const void* ptr, int dtype, int d, int heads, int64_t rows, int64_t outer,
                     int64_t head_stride, int64_t row_stride, int64_t outer_stride, int box_rows) {
  return tc5::encode_map(m, ptr, dtype, d, heads, rows, outer, head_stride, row_stride, outer_stride, box_rows);
}

int tc5_read_status(cudaStream_t st) {
  int32_t* w = tc5::status_word();
  if (!w) return 0;
  int32_t v = 0;
  if (cudaStreamSynchronize(st) != cudaSuccess) return -1;
  if (cudaMemcpy(&v, w, sizeof(v), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (v != 0) cudaMemset(w, 0, sizeof(v));
  return v;
}

}  // namespace fa
