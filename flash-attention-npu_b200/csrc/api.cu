// Host side of the C ABI: validation, window normalisation, tile / split planning and the
// kernel launches.  Replaces the host functions mha_fwd / mha_varlen_fwd / mha_fwd_kvcache of
// the reference (csrc/arch22/flash_attn_npu_v2/flash_api.cpp:356-1060) -- without their
// per-call device-to-host copy of the sequence lengths (:459), mask upload (:575-579) or
// tiling upload (:580): lengths are read on the device and masks are computed from indices.
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

#include "combine.cuh"
#include "exchange.cuh"
#include "decode_configs.cuh"
#include "mma_configs.cuh"
#include "tc5_api.cuh"
#include "kv_prologue.cuh"

namespace fa {

static thread_local std::string g_err;
static std::atomic<long long> g_launches{0};  // kernel launches issued so far (fa_b200_launch_count)

static int fail(int code, const std::string& msg);
int fail_bwd(int code, const std::string& msg) { return fail(code, msg); }  // for bwd.cu
void count_launches(int n) { g_launches += n; }
static int fail(int code, const std::string& msg) {
  g_err = msg;
  return code;
}

static int device_sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (dev < 0 || dev >= 64) return 0;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    cached[dev] = n;
  }
  return cached[dev];
}

static void normalize_window(int seqlen_q, int max_k, bool causal, int& wl, int& wr, bool& is_causal, bool& is_local) {
  // csrc/arch22/flash_attn_npu_v2/flash_api.cpp:483-494
  if (max_k > 0 && wl >= max_k - 1) wl = -1;
  if (seqlen_q > 0 && wr >= seqlen_q - 1) wr = -1;
  if (causal) wr = 0;
  is_causal = (wl < 0 && wr == 0);
  is_local = (wl >= 0 || wr >= 0) && !is_causal;
}

static bool s_new_too_long(const fa_fwd_params& a) { return a.seqlen_new > a.seqlen_k; }

struct Planned {
  fa_fwd_plan pl;
  KParams kp;
  int hd_pad;
};

// `forced`: a plan made earlier for the same problem (fa_b200_plan_encode): its kernel family, tile configuration
// and KV splits are taken over instead of being decided again; FA_ERR_UNSUPPORTED when they do not fit this call.
static int make_plan(const fa_fwd_params& a_in, Planned* out, const fa_fwd_plan* forced = nullptr) {
  std::memset(out, 0, sizeof(*out));
  fa_fwd_params a = a_in;
  if (forced) a.kernel = forced->kernel;
  if (a.b <= 0) return fail(FA_ERR_INVALID, "batch size must be positive");
  if (a.dtype != FA_FP16 && a.dtype != FA_BF16) return fail(FA_ERR_INVALID, "FlashAttention only supports FP16 and BF16 data types");
  if (a.d <= 0 || a.d > 256) return fail(FA_ERR_INVALID, "FlashAttention only supports head dimension at most 256");
  if (a.d % 8 != 0) return fail(FA_ERR_INVALID, "head dimension must be a multiple of 8 (pad it on the caller side)");
  if (a.h <= 0 || a.h_k <= 0 || a.h % a.h_k != 0)
    return fail(FA_ERR_INVALID, "Number of heads in key/value must divide number of heads in query");
  if (a.seqlen_q < 0 || a.seqlen_k < 0) return fail(FA_ERR_INVALID, "negative sequence length");
  if (a.softcap < 0.f) return fail(FA_ERR_INVALID, "softcap must be non-negative (0.0 disables softcap)");
  if (a.num_splits < 0) return fail(FA_ERR_INVALID, "num_splits must be >= 0");
  if (a.block_table && a.page_size <= 0) return fail(FA_ERR_INVALID, "paged KV cache needs page_size > 0");
  if (a.block_table && a.cu_seqlens_k) return fail(FA_ERR_INVALID, "block_table cannot be combined with cu_seqlens_k");
  if (a.block_table && !a.seqused_k) return fail(FA_ERR_INVALID, "paged KV cache needs the per-sequence key lengths");
  if ((a.k_new != nullptr) != (a.v_new != nullptr)) return fail(FA_ERR_INVALID, "k and v must be passed together");
  if (a.k_new && a.seqlen_new <= 0) return fail(FA_ERR_INVALID, "seqlen_new must be positive when k, v are given");
  if (!a.k_new && a.seqlen_new != 0) return fail(FA_ERR_INVALID, "seqlen_new given without k, v");
  if (a.k_new && !a.seqused_k) return fail(FA_ERR_INVALID, "appending k, v needs cache_seqlens");
  if ((a.rotary_cos != nullptr) != (a.rotary_sin != nullptr)) return fail(FA_ERR_INVALID, "rotary_cos and rotary_sin must be passed together");
  if (a.rotary_cos) {
    if (!a.k_new) return fail(FA_ERR_INVALID, "rotary embedding is only applied together with new k, v");
    if (a.rotary_dim <= 0 || a.rotary_dim % 16 != 0 || a.rotary_dim > a.d)
      return fail(FA_ERR_INVALID, "rotary_dim must be divisible by 16 and at most the head dimension");
  }
  if (a.kv_total < 0 || a.kv_pos_offset < 0) return fail(FA_ERR_INVALID, "negative kv shard position");
  if (a.kv_outer < 0) return fail(FA_ERR_INVALID, "negative kv_outer");
  if (a.block_table && a.kv_outer <= 0) return fail(FA_ERR_INVALID, "paged KV cache needs kv_outer = the number of pages");
  if (a.cache_batch_idx && !a.block_table && a.kv_outer <= 0)
    return fail(FA_ERR_INVALID, "cache_batch_idx needs kv_outer = the number of cache rows");
  if (a.seqused_k && s_new_too_long(a)) return fail(FA_ERR_INVALID, "the new tokens do not fit into the KV cache");

  const int s_new = a.seqlen_new;
  const int max_k_bound = a.seqlen_k + s_new;
  const int group = a.h / a.h_k;
  const int hd_pad = a.d <= 64 ? 64 : (a.d <= 128 ? 128 : 256);
  out->hd_pad = hd_pad;

  // ---- window normalisation ----
  int wl = a.window_left, wr = a.window_right;
  bool is_causal = false, is_local = false;
  int wl_on_device = 0;
  {
    int max_k = -1;
    if (!a.seqused_k) max_k = max_k_bound;  // dense: s_k; varlen: max_seqlen_k
    else if (a.max_seqlen_k_known >= 0) max_k = a.max_seqlen_k_known + s_new;
    if (a.kv_total > 0) max_k = a.kv_total;
    if (max_k < 0) {
      // Unknown on the host.  If the window already covers the largest possible length the rule
      // fires for certain; otherwise the kernel applies it from the device-side maximum.
      if (wl >= 0 && wl >= max_k_bound - 1) max_k = max_k_bound;
      else if (wl >= 0) wl_on_device = 1;
      if (max_k < 0) max_k = 0;  // leaves wl untouched below
    }
    normalize_window(a.seqlen_q, max_k, a.causal != 0, wl, wr, is_causal, is_local);
  }

  // ---- tile shape ----
  const bool pack = group > 1 && a.seqlen_q < 64;
  const int gp = pack ? group : 1;
  const int rows_max = a.seqlen_q * gp;
  int cfg = rows_max <= 16 ? 0 : (rows_max <= 32 ? 1 : (pack ? 2 : 3));
  if (const char* e = std::getenv("FA_B200_MMA_CONFIG")) {  // tuning override: tile configuration index
    const int forced = std::atoi(e);
    MmaConfigInfo t;
    if (mma_config_info(hd_pad, forced, &t) && t.block_m >= std::min(rows_max, 16)) cfg = forced;
  }
  if (forced && forced->kernel == FA_KERNEL_MMA) {
    MmaConfigInfo t;
    if (!mma_config_info(hd_pad, forced->config, &t) || t.block_m < std::min(rows_max, 16))
      return fail(FA_ERR_UNSUPPORTED, "the plan's tile configuration does not fit this problem");
    cfg = forced->config;
  }
  MmaConfigInfo ci;
  if (!mma_config_info(hd_pad, cfg, &ci)) return fail(FA_ERR_UNSUPPORTED, "no tile configuration");
  // ---- producer / consumer decode kernel: <= 32 packed rows, head dim <= 128 (> 64), rows that can
  //      be moved by 16-byte aligned bulk copies ----
  int kernel_id = FA_KERNEL_MMA;
  bool decode_one_segment_only = false;  // the chosen decode configuration keeps its merge slab over the ring
  {
    auto al16 = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; };
    const bool strides_ok = a.k_row_stride % 8 == 0 && a.k_head_stride % 8 == 0 && a.k_batch_stride % 8 == 0 &&
                            a.v_row_stride % 8 == 0 && a.v_head_stride % 8 == 0 && a.v_batch_stride % 8 == 0;
    // K / V stages are fetched by tiled TMA loads: exact head dim 128, 16-byte aligned strides, a
    // per-sequence length vector, and pages that hold whole key blocks
    const bool eligible = a.d == 128 && rows_max <= 32 && rows_max > 0 && !a.cu_seqlens_k && strides_ok &&
                          al16(a.k) && al16(a.v) && a.k_batch_stride > 0 && a.v_batch_stride > 0 &&
                          (!a.block_table || a.page_size % 128 == 0);
    if (a.kernel == FA_KERNEL_DECODE && !eligible)
      return fail(FA_ERR_UNSUPPORTED, "the decode kernel does not cover this problem");
    if (eligible && (a.kernel == FA_KERNEL_DECODE || a.kernel == FA_KERNEL_AUTO)) {
      // Measured best.  Up to 16 rows: two resident CTAs of 1x4 consumer warps.  17-32 rows: one CTA of 2x4
      // consumer warps for long key ranges and for launches that become persistent; for short ranges (a
      // sliding window, short caches) two resident CTAs of 2x2 warps, so that one CTA's Q load, slice
      // merge and store run under the other's streaming (paged window decode: 88 instead of 98 us).
      int dcfg = 3;
      if (rows_max > 16) {
        long long keys = max_k_bound;
        const bool windowed = is_local && wl >= 0 && (long long)wl + std::max(wr, 0) + 32 / gp + 2 < keys;
        if (windowed) keys = (long long)wl + std::max(wr, 0) + 32 / gp + 2;
        const bool may_persist = a.seqused_k && !windowed && a.num_splits == 0 && !a.cu_seqlens_q && a.kv_total == 0 &&
                                 !a.partial_out;
        dcfg = (!may_persist && keys <= 16384) ? 11 : 5;
      }
      if (const char* e = std::getenv("FA_B200_DECODE_CONFIG")) {  // tuning override: decode tile configuration
        const int forced = std::atoi(e);
        DecodeConfigInfo t;
        if (decode_config_info(hd_pad, forced, &t) && t.block_m >= rows_max) dcfg = forced;
      }
      if (forced && forced->kernel == FA_KERNEL_DECODE) {
        DecodeConfigInfo t;
        if (!decode_config_info(hd_pad, forced->config, &t) || t.block_m < rows_max)
          return fail(FA_ERR_UNSUPPORTED, "the plan's tile configuration does not fit this problem");
        dcfg = forced->config;
      }
      DecodeConfigInfo di;
      if (decode_config_info(hd_pad, dcfg, &di)) {
        kernel_id = FA_KERNEL_DECODE;
        cfg = dcfg;
        ci = MmaConfigInfo{di.block_m, di.block_n, di.threads, di.smem_bytes};
        decode_one_segment_only = di.slab_in_ring;
      }
    }
  }
  const int m_blocks = std::max(1, ceil_div(rows_max, ci.block_m));
  const int heads_eff = a.h / gp;

  // ---- KV range bound and splits ----
  int range = max_k_bound;
  if (is_local && wl >= 0) {
    const int i_span = ceil_div(ci.block_m, gp);
    const long long r = (long long)wl + std::max(wr, 0) + i_span + 1;
    if (r < range) range = (int)r;
  }
  int max_blocks = std::min(ceil_div(range, ci.block_n) + 1, std::max(1, ceil_div(max_k_bound, ci.block_n)));
  if (max_blocks < 1) max_blocks = 1;
  int num_sm = a.num_sm > 0 ? a.num_sm : device_sm_count();
  if (num_sm <= 0) return fail(FA_ERR_CUDA, "cannot query the SM count of the current device");
  const long long base = (long long)m_blocks * heads_eff * a.b;
  int ns = 1;
  if (a.num_splits >= 1) {
    ns = std::min(a.num_splits, max_blocks);
  } else if (kernel_id == FA_KERNEL_DECODE) {
    const bool window_bound = is_local && wl >= 0 && range < max_k_bound;
    if (a.seqused_k && a.kv_total == 0 && !window_bound) {
      // Ragged lengths (only their upper bound is known here): CTAs of about 3 K keys keep the tail
      // short without paying the per-CTA fixed cost too often (measured on lengths U[1024, 8191]).
      ns = std::max(1, std::min(max_blocks / 2, ceil_div(max_blocks * ci.block_n, 3072)));
    } else {
      // Uniform ranges: a CTA costs its KV blocks plus a fixed part worth about 512 keys (launch,
      // first TMA latency, epilogue); CTAs run in waves of num_sm * resident CTAs.
      const long long resident = std::max(1, (227 * 1024) / std::max(1, ci.smem_bytes));
      const long long slots = (long long)num_sm * resident;
      const double fixed = 512.0 / ci.block_n;
      double best = 1e30;
      for (int cand = 1; cand <= std::max(1, max_blocks / 2); ++cand) {
        const long long waves = (base * cand + slots - 1) / slots;
        const double cost = (double)waves * (ceil_div(max_blocks, cand) + fixed);
        if (cost < best * 0.97) { best = cost; ns = cand; }  // prefer fewer splits unless clearly better
      }
    }
  } else if (base < 8LL * num_sm && max_blocks >= 16) {
    long long per_sm = 16;
    if (const char* e = std::getenv("FA_B200_CTAS_PER_SM")) per_sm = std::max(1, std::atoi(e));  // tuning override
    long long want = (per_sm * num_sm + base - 1) / base;
    ns = (int)std::max(1LL, std::min<long long>(want, max_blocks / 8));
  }
  if (const char* e = std::getenv("FA_B200_NUM_SPLITS")) {  // tuning override of the split heuristic
    if (a.num_splits == 0) ns = std::max(1, std::min(std::atoi(e), max_blocks));
  }
  int bps = ceil_div(max_blocks, ns);
  ns = ceil_div(max_blocks, bps);

  // Persistent decode: ragged lengths leave a tail of unequal CTAs; CTAs that stay resident and take
  // equal shares of the KV blocks of the whole launch do not.  A unit cut by a CTA boundary is
  // finished by the merge kernel from up to kPersistSlots partials.  (Window-bound ranges are
  // nearly equal; there the merge launch costs what the balance gains -- measured.)
  constexpr int kPersistSlots = 4;
  bool persistent = false;
  long long persist_grid = 0;
  if (kernel_id == FA_KERNEL_DECODE && a.num_splits == 0 && !a.cu_seqlens_q && a.kv_total == 0 && !a.partial_out) {
    const bool window_bound = is_local && wl >= 0 && range < max_k_bound;
    const long long resident = std::max(1, (227 * 1024) / std::max(1, ci.smem_bytes));
    persist_grid = (long long)num_sm * resident;
    const bool can_persist = (a.seqused_k != nullptr || window_bound) && base * max_blocks >= 4 * persist_grid &&
                             base * (max_blocks + 1) < 0x3fffffffLL;
    persistent = can_persist && !window_bound && !decode_one_segment_only;
    if (const char* e = std::getenv("FA_B200_DECODE_PERSISTENT"))  // tuning override: 0 off, 1 default rule, 2 also window-bound
      persistent = can_persist && !decode_one_segment_only && (std::atoi(e) == 2 || (std::atoi(e) == 1 && !window_bound));
    if (const char* e = std::getenv("FA_B200_DECODE_PERSISTENT_GRID")) persist_grid = std::max(1, std::atoi(e));  // tuning override
    if (persistent) { ns = kPersistSlots; bps = 0; }
    if (forced && forced->kernel == FA_KERNEL_DECODE && forced->num_splits > 1 && forced->blocks_per_split == 0) {
      if (!can_persist || decode_one_segment_only || forced->grid <= 0 || forced->num_splits != kPersistSlots)
        return fail(FA_ERR_UNSUPPORTED, "the plan's persistent decode schedule does not fit this problem");
      persistent = true;
      persist_grid = forced->grid;
      ns = kPersistSlots;
      bps = 0;
    } else if (forced) {
      persistent = false;
    }
  }
  if (forced && forced->kernel != FA_KERNEL_TCGEN05 && !persistent) {
    if (forced->num_splits < 1 || forced->blocks_per_split < 1 ||
        (long long)forced->num_splits * forced->blocks_per_split < max_blocks)
      return fail(FA_ERR_UNSUPPORTED, "the plan's KV splits do not cover this problem's key range");
    ns = forced->num_splits;
    bps = forced->blocks_per_split;
  }

  const bool varlen_q = a.cu_seqlens_q != nullptr;
  const int64_t lse_elems = varlen_q ? (int64_t)a.h * a.total_q : (int64_t)a.b * a.h * a.seqlen_q;
  if (ns > 1) {
    const bool canonical = varlen_q ? (a.lse_head_stride == a.total_q)
                                    : (a.lse_batch_stride == (int64_t)a.h * a.seqlen_q && a.lse_head_stride == a.seqlen_q);
    if (!canonical) { ns = 1; bps = max_blocks; persistent = false; }
  }

  fa_fwd_plan& pl = out->pl;
  pl.kernel = kernel_id;
  pl.config = cfg;
  pl.pack_gqa = pack;
  pl.block_m = ci.block_m;
  pl.block_n = ci.block_n;
  pl.m_blocks = m_blocks;
  pl.num_splits = ns;
  pl.blocks_per_split = bps;
  pl.grid = persistent ? (int)persist_grid : (int)(base * ns);
  pl.threads = ci.threads;
  pl.smem_bytes = ci.smem_bytes;
  pl.is_causal = is_causal;
  pl.is_local = is_local;
  pl.window_left = wl;
  pl.window_right = wr;
  pl.launches = ns > 1 ? 2 : 1;
  pl.workspace_bytes = ns > 1 ? (((size_t)ns * lse_elems * sizeof(float) + 15) & ~(size_t)15) + (size_t)ns * lse_elems * a.d * sizeof(float) : 0;
  if (base * ns > 0x7fffffffLL) return fail(FA_ERR_UNSUPPORTED, "grid too large");

  KParams& kp = out->kp;
  kp.a = a;
  kp.causal_in = a.causal;
  kp.wl = wl;
  kp.wr = wr;
  kp.wl_on_device = wl_on_device;
  kp.group = group;
  kp.gp = gp;
  kp.heads_eff = heads_eff;
  kp.m_blocks = m_blocks;
  kp.num_splits = ns;
  kp.blocks_per_split = bps;
  kp.persistent = persistent ? 1 : 0;
  kp.scale_log2 = a.softmax_scale * kLog2e;
  kp.lse_elems = lse_elems;

  // ---- tcgen05 prefill kernel eligibility ----
  if (a.kernel != FA_KERNEL_MMA && a.kernel != FA_KERNEL_DECODE && tc5_eligible(a, is_causal, is_local, wl_on_device)) {
    tc5_fill_plan(a, &pl);
  } else if (a.kernel == FA_KERNEL_TCGEN05) {
    return fail(FA_ERR_UNSUPPORTED, "the tcgen05 kernel does not cover this problem");
  }
  return FA_OK;
}

// The merge kernel is launched with programmatic stream serialisation: the launch itself and the start of its CTAs
// overlap the tail of the kernel in front of it on the stream (the split-KV attention kernel, which signals
// griddepcontrol.launch_dependents when it starts); the kernel waits for that kernel's completion before it reads
// (combine.cuh).  This hides most of what a second launch costs behind a kernel of a few hundred microseconds.
template <typename OutT>
static cudaError_t launch_combine_t(const fa_combine_params& c, int grid, cudaStream_t st) {
  cudaLaunchConfig_t cfg;
  std::memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kCombineWarps * 32);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, combine_kernel<OutT>, c);
}

static int launch_combine(const fa_combine_params& c, cudaStream_t st) {
  const int64_t rows = (int64_t)c.b * c.s * c.h;
  if (rows == 0) return FA_OK;
  const int grid = (int)((rows + kCombineWarps - 1) / kCombineWarps);
  cudaError_t e;
  if (c.out_dtype == FA_BF16) e = launch_combine_t<__nv_bfloat16>(c, grid, st);
  else if (c.out_dtype == FA_FP16) e = launch_combine_t<__half>(c, grid, st);
  else if (c.out_dtype == 2) e = launch_combine_t<float>(c, grid, st);
  else return fail(FA_ERR_INVALID, "bad out_dtype");
  if (e != cudaSuccess) return fail(FA_ERR_CUDA, std::string("combine launch: ") + cudaGetErrorString(e));
  ++g_launches;
  return FA_OK;
}

// skip_merge: leave the split partials in the workspace (the caller merges them itself); *splits_out = their number.
static int run_fwd(const fa_fwd_params& a, void* workspace, size_t workspace_bytes, cudaStream_t st,
                   const fa_fwd_plan* forced = nullptr, bool skip_merge = false, int* splits_out = nullptr) {
  if (!a.q || !a.k || !a.v || !a.o || !a.lse) return fail(FA_ERR_INVALID, "q, k, v, o and lse must be non-null");
  Planned P;
  int rc = make_plan(a, &P, forced);
  if (rc != FA_OK) return rc;
  if (a.total_q == 0 || a.seqlen_q == 0) return FA_OK;
  if (P.pl.kernel == FA_KERNEL_TCGEN05) {
    fa_fwd_params a2 = a;
    if (a.k_new) {
      // New tokens: a prologue launch appends them to the cache (k rotated) and leaves the rotated q in
      // the workspace; the prefill kernel then sees a cache of cache_seqlens + s_new keys.
      void* q_rot = nullptr;
      if (a.rotary_cos) {
        if (!workspace || workspace_bytes < P.pl.workspace_bytes) return fail(FA_ERR_WORKSPACE, "workspace missing or too small");
        if ((reinterpret_cast<uintptr_t>(workspace) & 15) != 0) return fail(FA_ERR_WORKSPACE, "workspace must be 16-byte aligned");
        q_rot = workspace;
        a2.q = q_rot;
        a2.q_head_stride = a.d;
        a2.q_row_stride = (int64_t)a.h * a.d;
        a2.q_batch_stride = (int64_t)a.seqlen_q * a.h * a.d;
      }
      P.kp.status = device_status_word();
      cudaError_t e = launch_kv_prologue(P.kp, q_rot, P.pl.is_causal || P.pl.is_local, st);
      if (e != cudaSuccess) return fail(FA_ERR_CUDA, std::string("append prologue launch: ") + cudaGetErrorString(e));
      ++g_launches;
      a2.k_new = a2.v_new = nullptr;  // seqlen_new stays: the kernel adds it to the cache lengths
      a2.rotary_cos = a2.rotary_sin = nullptr;
    }
    rc = tc5_launch(a2, P.pl, st, &g_err);
    if (rc == FA_OK) ++g_launches;
    return rc;
  }

  KParams& kp = P.kp;
  kp.status = device_status_word();
  if (!kp.status) return fail(FA_ERR_CUDA, "cannot look up the device status word");
  if (P.pl.num_splits > 1) {
    if (!workspace || workspace_bytes < P.pl.workspace_bytes) return fail(FA_ERR_WORKSPACE, "workspace missing or too small");
    if ((reinterpret_cast<uintptr_t>(workspace) & 15) != 0) return fail(FA_ERR_WORKSPACE, "workspace must be 16-byte aligned");
    kp.lse_partial = reinterpret_cast<float*>(workspace);
    // O partials start at a 16-byte boundary after the LSE partials
    const size_t lse_bytes = ((size_t)P.pl.num_splits * kp.lse_elems * sizeof(float) + 15) & ~(size_t)15;
    kp.o_partial = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + lse_bytes);
  }
  cudaError_t e = cudaErrorInvalidValue;
  const bool bf = a.dtype == FA_BF16;
  if (P.pl.kernel == FA_KERNEL_DECODE) {
    CUtensorMap tm_k, tm_v;
    const bool paged = a.block_table != nullptr;
    // true outer extent (pages / cache rows): an index outside it makes the TMA return zeros, never a wild read
    const int64_t rows = paged ? a.page_size : a.seqlen_k, outer = a.kv_outer > 0 ? a.kv_outer : a.b;
    if (!tma_encode_rows(&tm_k, a.k, a.dtype, a.d, a.h_k, rows, outer, a.k_head_stride, a.k_row_stride, a.k_batch_stride, P.pl.block_n) ||
        !tma_encode_rows(&tm_v, a.v, a.dtype, a.d, a.h_k, rows, outer, a.v_head_stride, a.v_row_stride, a.v_batch_stride, P.pl.block_n))
      return fail(FA_ERR_CUDA, "cuTensorMapEncodeTiled failed for the KV cache");
    e = bf ? launch_decode_128_bf16(P.pl.config, kp, tm_k, tm_v, P.pl.grid, st)
           : launch_decode_128_fp16(P.pl.config, kp, tm_k, tm_v, P.pl.grid, st);
  } else
  switch (P.hd_pad) {
    case 64: e = bf ? launch_mma_64_bf16(P.pl.config, kp, P.pl.grid, st) : launch_mma_64_fp16(P.pl.config, kp, P.pl.grid, st); break;
    case 128: e = bf ? launch_mma_128_bf16(P.pl.config, kp, P.pl.grid, st) : launch_mma_128_fp16(P.pl.config, kp, P.pl.grid, st); break;
    case 256: e = bf ? launch_mma_256_bf16(P.pl.config, kp, P.pl.grid, st) : launch_mma_256_fp16(P.pl.config, kp, P.pl.grid, st); break;
  }
  if (e != cudaSuccess) return fail(FA_ERR_CUDA, std::string("attention kernel launch: ") + cudaGetErrorString(e));
  ++g_launches;
  if (splits_out) *splits_out = P.pl.num_splits;

  if (P.pl.num_splits > 1 && !skip_merge) {
    fa_combine_params c;
    std::memset(&c, 0, sizeof(c));
    const bool varlen_q = a.cu_seqlens_q != nullptr;
    c.o_partial = kp.o_partial;
    c.lse_partial = kp.lse_partial;
    c.o = a.o;
    c.lse = a.lse;
    c.num_splits = P.pl.num_splits;
    c.b = varlen_q ? 1 : a.b;
    c.s = varlen_q ? a.total_q : a.seqlen_q;
    c.h = a.h;
    c.d = a.d;
    c.lp_split_stride = kp.lse_elems;
    c.lp_batch_stride = a.lse_batch_stride;
    c.lp_row_stride = 1;
    c.lp_head_stride = a.lse_head_stride;
    c.op_split_stride = kp.lse_elems * a.d;
    c.op_batch_stride = a.lse_batch_stride * a.d;
    c.op_row_stride = a.d;
    c.op_head_stride = a.lse_head_stride * a.d;
    c.o_batch_stride = varlen_q ? 0 : a.o_batch_stride;
    c.o_row_stride = a.o_row_stride;
    c.o_head_stride = a.o_head_stride;
    c.lse_batch_stride = a.lse_batch_stride;
    c.lse_row_stride = 1;
    c.lse_head_stride = a.lse_head_stride;
    c.out_dtype = a.partial_out ? 2 : a.dtype;
    c.partial_out = a.partial_out;
    return launch_combine(c, st);
  }
  return FA_OK;
}

// ------------------------------------------------------------------------------------------------
// Allocation-free variant of the split-KV path.
//
// Some hosts may not allocate device memory once they are running: a serving process whose whole
// memory budget is carved up at start-up, a runtime that owns the GPU heap through its own arena,
// a latency-critical loop that forbids allocator calls.  For them the split partials live in this
// file-scope device array instead of a caller-supplied workspace.  Every GPU that loads the library
// holds kNoAllocScratchBytes of it until the process exits.
//
// In host code `g_noalloc_scratch` is only a stand-in for the symbol, not a device address; the
// address is obtained once per device, with that device current, through cudaGetSymbolAddress.
// ------------------------------------------------------------------------------------------------
constexpr size_t kNoAllocScratchBytes = 32u << 20;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

static int noalloc_scratch_ptr(void** out) {
  static void* ptrs[64] = {nullptr};
  static std::mutex mu;  // calls may come from several host threads
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return fail(FA_ERR_CUDA, "cannot query the current device");
  std::lock_guard<std::mutex> lock(mu);
  if (!ptrs[dev]) {
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (e != cudaSuccess || !ptr)
      return fail(FA_ERR_CUDA, std::string("cudaGetSymbolAddress(scratch): ") + cudaGetErrorString(e));
    ptrs[dev] = ptr;
  }
  *out = ptrs[dev];
  return FA_OK;
}

static int run_fwd_noalloc(const fa_fwd_params& a_in, cudaStream_t st) {
  fa_fwd_params a = a_in;
  a.kernel = FA_KERNEL_MMA;  // the register-accumulator kernel and the merge allocate nothing
  Planned P;
  int rc = make_plan(a, &P);
  if (rc != FA_OK) return rc;
  if (P.pl.workspace_bytes > kNoAllocScratchBytes)
    return fail(FA_ERR_WORKSPACE, "this problem needs " + std::to_string(P.pl.workspace_bytes) +
                                      " bytes of split-KV scratch but the built-in scratch array holds " +
                                      std::to_string(kNoAllocScratchBytes) + "; lower num_splits or use fa_b200_fwd");
  void* scratch = nullptr;
  rc = noalloc_scratch_ptr(&scratch);
  if (rc != FA_OK) return rc;
  return run_fwd(a, scratch, kNoAllocScratchBytes, st);
}

// ------------------------------------------------------------------------------------------------
// Sequence-sharded decode across GPUs over peer memory (exchange.cuh).
// ------------------------------------------------------------------------------------------------
static size_t exchange_bytes(int world, int64_t rows, int d) {
  return (size_t)kXchgHeaderBytes + (size_t)2 * world * rows * (d + 4) * sizeof(float);
}

static size_t exchange_workspace(const fa_fwd_params& a, int ns) {
  const size_t lse_elems = (size_t)a.b * a.h * a.seqlen_q;
  return (((size_t)ns * lse_elems * sizeof(float) + 15) & ~(size_t)15) + (size_t)ns * lse_elems * a.d * sizeof(float);
}

template <typename Kern>
static cudaError_t launch_dependent(Kern kern, const XchgParams& xp, int grid, cudaStream_t st) {
  cudaLaunchConfig_t cfg;
  std::memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kCombineWarps * 32);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, xp);
}

static int run_fwd_exchange(const fa_fwd_params& a_in, void* workspace, size_t workspace_bytes, const fa_exchange& x,
                            cudaStream_t st) {
  if (!a_in.q || !a_in.k || !a_in.v || !a_in.o || !a_in.lse) return fail(FA_ERR_INVALID, "q, k, v, o and lse must be non-null");
  if (x.world < 1 || x.world > FA_B200_MAX_RANKS || x.rank < 0 || x.rank >= x.world)
    return fail(FA_ERR_INVALID, "bad rank / world size of the exchange");
  for (int r = 0; r < x.world; ++r)
    if (!x.bufs[r]) return fail(FA_ERR_INVALID, "an exchange buffer is not mapped");
  if (a_in.cu_seqlens_q) return fail(FA_ERR_UNSUPPORTED, "the cross-GPU exchange takes dense (b, s_q, h, d) queries");
  if (a_in.d % 4 != 0) return fail(FA_ERR_INVALID, "head dimension must be a multiple of 4");
  const int64_t rows = (int64_t)a_in.b * a_in.seqlen_q * a_in.h;
  if (x.buf_bytes < exchange_bytes(x.world, rows, a_in.d))
    return fail(FA_ERR_WORKSPACE, "the exchange buffers are too small for this problem (fa_b200_exchange_bytes)");
  if (rows == 0) return FA_OK;

  // the attention over this rank's keys leaves fp32 partials [split][b, h, s_q] / [split][b, h, s_q][d] in the workspace
  fa_fwd_params a = a_in;
  a.partial_out = 1;
  a.lse_batch_stride = (int64_t)a.h * a.seqlen_q;
  a.lse_head_stride = a.seqlen_q;
  Planned P;
  int rc = make_plan(a, &P);
  if (rc != FA_OK) return rc;
  const int ns_plan = P.pl.kernel == FA_KERNEL_TCGEN05 ? 1 : P.pl.num_splits;
  if (ns_plan > 32) return fail(FA_ERR_UNSUPPORTED, "the cross-GPU exchange merges at most 32 local splits (set num_splits)");
  const size_t need = exchange_workspace(a, ns_plan);
  if (!workspace || workspace_bytes < need) return fail(FA_ERR_WORKSPACE, "workspace missing or too small (fa_b200_fwd_exchange_workspace)");
  if ((reinterpret_cast<uintptr_t>(workspace) & 15) != 0) return fail(FA_ERR_WORKSPACE, "workspace must be 16-byte aligned");
  const size_t lse_elems = (size_t)a.b * a.h * a.seqlen_q;
  float* lse_part = reinterpret_cast<float*>(workspace);
  float* o_part = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + (((size_t)ns_plan * lse_elems * sizeof(float) + 15) & ~(size_t)15));
  a.lse = lse_part;  // a single split writes its partial through o / lse, laid out like slot 0 of the split layout
  a.o = o_part;
  a.o_batch_stride = (int64_t)a.h * a.seqlen_q * a.d;
  a.o_head_stride = (int64_t)a.seqlen_q * a.d;
  a.o_row_stride = a.d;
  int ns = 1;
  rc = run_fwd(a, workspace, workspace_bytes, st, nullptr, true, &ns);
  if (rc != FA_OK) return rc;
  if (ns != ns_plan) return fail(FA_ERR_CUDA, "split plan changed between planning and launch");

  XchgParams xp;
  std::memset(&xp, 0, sizeof(xp));
  fa_combine_params& c = xp.c;
  c.o_partial = o_part;
  c.lse_partial = lse_part;
  c.o = a_in.o;
  c.lse = a_in.lse;
  c.num_splits = ns;
  c.b = a.b; c.s = a.seqlen_q; c.h = a.h; c.d = a.d;
  c.lp_split_stride = (int64_t)lse_elems;
  c.lp_batch_stride = a.lse_batch_stride;
  c.lp_row_stride = 1;
  c.lp_head_stride = a.lse_head_stride;
  c.op_split_stride = (int64_t)lse_elems * a.d;
  c.op_batch_stride = a.lse_batch_stride * a.d;
  c.op_row_stride = a.d;
  c.op_head_stride = a.lse_head_stride * a.d;
  c.o_batch_stride = a_in.o_batch_stride; c.o_row_stride = a_in.o_row_stride; c.o_head_stride = a_in.o_head_stride;
  c.lse_batch_stride = a_in.lse_batch_stride; c.lse_row_stride = 1; c.lse_head_stride = a_in.lse_head_stride;
  c.out_dtype = a_in.dtype;
  for (int r = 0; r < x.world; ++r) xp.bufs[r] = reinterpret_cast<char*>(x.bufs[r]);
  xp.world = x.world;
  xp.rank = x.rank;
  xp.timeout_cycles = x.timeout_cycles > 0 ? x.timeout_cycles : 4000000000LL;  // about two seconds of SM clock
  xp.status = device_status_word();
  const int grid = (int)((rows + kCombineWarps - 1) / kCombineWarps);
  cudaError_t e = launch_dependent(xchg_push_kernel, xp, grid, st);
  if (e != cudaSuccess) return fail(FA_ERR_CUDA, std::string("exchange push launch: ") + cudaGetErrorString(e));
  ++g_launches;
  e = a_in.dtype == FA_BF16 ? launch_dependent(xchg_merge_kernel<__nv_bfloat16>, xp, grid, st)
                            : launch_dependent(xchg_merge_kernel<__half>, xp, grid, st);
  if (e != cudaSuccess) return fail(FA_ERR_CUDA, std::string("exchange merge launch: ") + cudaGetErrorString(e));
  ++g_launches;
  return FA_OK;
}

// ------------------------------------------------------------------------------------------------
// Plans as bytes: what get_scheduler_metadata of the reference returns as an opaque tensor
// (csrc/arch22/flash_attn_npu_v3/flash_api.cpp:493-558: [causal mask | FAInferTilingData], filled by an AICPU
// kernel).  Here the bytes are a header that names the problem they were made for and the fa_fwd_plan itself; the
// forward that receives them checks the header against its own arguments and takes the plan over.
// ------------------------------------------------------------------------------------------------
constexpr uint32_t kPlanMagic = 0x0FA5B200u;
struct PlanBlob {
  uint32_t magic, abi, bytes, kind;
  int32_t b, seqlen_q, seqlen_k, h, h_k, d, dtype, causal, window_left, window_right, page_size, seqlen_new, num_splits;
  int32_t reserved[3];
  fa_fwd_plan plan;
};
static_assert(sizeof(PlanBlob) <= FA_B200_PLAN_BYTES, "FA_B200_PLAN_BYTES is too small");

// Which optional parts a call has: a plan only carries over between calls of the same kind.
static uint32_t plan_kind(const fa_fwd_params& a) {
  return (a.seqused_k ? 1u : 0u) | (a.block_table ? 2u : 0u) | (a.cu_seqlens_q ? 4u : 0u) | (a.cu_seqlens_k ? 8u : 0u) |
         (a.softcap > 0.f ? 16u : 0u) | (a.k_new ? 32u : 0u) | (a.alibi_slopes ? 64u : 0u) | (a.cache_batch_idx ? 128u : 0u) |
         (a.kv_total > 0 ? 256u : 0u) | (a.partial_out ? 512u : 0u);
}

static int plan_encode(const fa_fwd_params& a, void* buf, size_t n) {
  if (!buf || n < sizeof(PlanBlob)) return fail(FA_ERR_INVALID, "plan buffer too small (FA_B200_PLAN_BYTES)");
  Planned P;
  const int rc = make_plan(a, &P);
  if (rc != FA_OK) return rc;
  PlanBlob blob;
  std::memset(&blob, 0, sizeof(blob));
  blob.magic = kPlanMagic;
  blob.abi = FA_B200_ABI_VERSION;
  blob.bytes = sizeof(PlanBlob);
  blob.kind = plan_kind(a);
  blob.b = a.b; blob.seqlen_q = a.seqlen_q; blob.seqlen_k = a.seqlen_k; blob.h = a.h; blob.h_k = a.h_k; blob.d = a.d;
  blob.dtype = a.dtype; blob.causal = a.causal; blob.window_left = a.window_left; blob.window_right = a.window_right;
  blob.page_size = a.page_size; blob.seqlen_new = a.seqlen_new; blob.num_splits = a.num_splits;
  blob.plan = P.pl;
  std::memset(buf, 0, n);
  std::memcpy(buf, &blob, sizeof(blob));
  return FA_OK;
}

static int plan_decode(const void* buf, size_t n, PlanBlob* out) {
  if (!buf || n < sizeof(PlanBlob)) return fail(FA_ERR_INVALID, "scheduler metadata is too short to be a plan of this library");
  std::memcpy(out, buf, sizeof(PlanBlob));
  if (out->magic != kPlanMagic) return fail(FA_ERR_INVALID, "scheduler metadata was not made by get_scheduler_metadata of this library");
  if (out->abi != FA_B200_ABI_VERSION || out->bytes != sizeof(PlanBlob))
    return fail(FA_ERR_INVALID, "scheduler metadata was made by another version of this library");
  return FA_OK;
}

static int run_fwd_planned(const fa_fwd_params& a, const void* buf, size_t n, void* workspace, size_t workspace_bytes,
                           cudaStream_t st) {
  PlanBlob blob;
  int rc = plan_decode(buf, n, &blob);
  if (rc != FA_OK) return rc;
  // The problem the plan names must be the one at hand: a plan for other shapes is a caller's mistake.
  struct { const char* name; int32_t planned, given; } key[] = {
      {"batch size", blob.b, a.b}, {"max_seqlen_q", blob.seqlen_q, a.seqlen_q}, {"num_heads_q", blob.h, a.h},
      {"num_heads_kv", blob.h_k, a.h_k}, {"head dim", blob.d, a.d}, {"dtype", blob.dtype, a.dtype},
      {"causal", blob.causal, a.causal}, {"window_size_left", blob.window_left, a.window_left},
      {"window_size_right", blob.window_right, a.window_right}};
  for (const auto& f : key)
    if (f.planned != f.given)
      return fail(FA_ERR_INVALID, std::string("scheduler metadata was computed for a different problem: ") + f.name + " " +
                                      std::to_string(f.planned) + " there, " + std::to_string(f.given) + " here");
  const bool cache = a.seqused_k != nullptr;
  if (!cache && blob.seqlen_k != a.seqlen_k)
    return fail(FA_ERR_INVALID, "scheduler metadata was computed for a different problem: max_seqlen_k " +
                                    std::to_string(blob.seqlen_k) + " there, " + std::to_string(a.seqlen_k) + " here");
  // The tile configuration and KV splits only carry over to a call with the same optional parts; otherwise the
  // call is planned afresh (the reference's tests hand a plan made from cache lengths to the dense entry points).
  if (blob.kind == plan_kind(a) && blob.page_size == a.page_size && blob.seqlen_new == a.seqlen_new &&
      blob.num_splits == a.num_splits) {
    fa_fwd_params a2 = a;
    // A cache may be larger than the longest sequence the plan was made for.  The plan's splits cover
    // max_seqlen_k keys, so that becomes the bound: a longer cache_seqlens entry is clamped and reported through
    // the status word instead of being attended to in part.
    if (cache && blob.seqlen_k < a2.seqlen_k) {
      a2.seqlen_k = blob.seqlen_k;
      if (a2.block_table) a2.seqlen_k = ceil_div(a2.seqlen_k, a2.page_size) * a2.page_size;
      if (a2.max_seqlen_k_known > blob.seqlen_k) a2.max_seqlen_k_known = blob.seqlen_k;
    }
    rc = run_fwd(a2, workspace, workspace_bytes, st, &blob.plan);
    if (rc != FA_ERR_UNSUPPORTED) return rc;
  }
  return run_fwd(a, workspace, workspace_bytes, st);
}

}  // namespace fa

extern "C" {

int fa_b200_fwd_noalloc(const fa_fwd_params* p, void* stream) {
  if (!p) return fa::fail(FA_ERR_INVALID, "null params");
  fa::g_err.clear();
  return fa::run_fwd_noalloc(*p, reinterpret_cast<cudaStream_t>(stream));
}

int fa_b200_fwd(const fa_fwd_params* p, void* workspace, size_t workspace_bytes, void* stream) {
  if (!p) return fa::fail(FA_ERR_INVALID, "null params");
  fa::g_err.clear();
  return fa::run_fwd(*p, workspace, workspace_bytes, reinterpret_cast<cudaStream_t>(stream));
}

int fa_b200_fwd_planned(const fa_fwd_params* p, const void* plan, size_t plan_bytes, void* workspace, size_t workspace_bytes,
                        void* stream) {
  if (!p) return fa::fail(FA_ERR_INVALID, "null params");
  fa::g_err.clear();
  return fa::run_fwd_planned(*p, plan, plan_bytes, workspace, workspace_bytes, reinterpret_cast<cudaStream_t>(stream));
}

int fa_b200_plan_encode(const fa_fwd_params* p, void* buf, size_t buf_bytes) {
  if (!p) return fa::fail(FA_ERR_INVALID, "null params");
  fa::g_err.clear();
  return fa::plan_encode(*p, buf, buf_bytes);
}

int fa_b200_plan_decode(const void* buf, size_t buf_bytes, fa_fwd_plan* plan) {
  if (!plan) return fa::fail(FA_ERR_INVALID, "null argument");
  fa::g_err.clear();
  fa::PlanBlob blob;
  const int rc = fa::plan_decode(buf, buf_bytes, &blob);
  if (rc == FA_OK) *plan = blob.plan;
  return rc;
}

size_t fa_b200_exchange_bytes(int32_t world, int64_t rows, int32_t d) { return fa::exchange_bytes(world, rows, d); }

int fa_b200_exchange_alloc(size_t bytes, void** ptr, void* handle64) {
  fa::g_err.clear();
  if (!ptr || !handle64 || bytes < (size_t)fa::kXchgHeaderBytes) return fa::fail(FA_ERR_INVALID, "bad argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handles are 64 bytes");
  void* q = nullptr;
  cudaError_t e = cudaMalloc(&q, bytes);
  if (e == cudaSuccess) e = cudaMemset(q, 0, bytes);
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, q);
  if (e != cudaSuccess) {
    if (q) cudaFree(q);
    return fa::fail(FA_ERR_CUDA, std::string("exchange buffer: ") + cudaGetErrorString(e));
  }
  std::memcpy(handle64, &h, sizeof(h));
  *ptr = q;
  return FA_OK;
}

int fa_b200_exchange_open(const void* handle64, void** ptr) {
  fa::g_err.clear();
  if (!ptr || !handle64) return fa::fail(FA_ERR_INVALID, "bad argument");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle64, sizeof(h));
  void* q = nullptr;
  const cudaError_t e = cudaIpcOpenMemHandle(&q, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return fa::fail(FA_ERR_CUDA, std::string("mapping a peer's exchange buffer: ") + cudaGetErrorString(e));
  *ptr = q;
  return FA_OK;
}

int fa_b200_exchange_close(void* ptr) {
  fa::g_err.clear();
  const cudaError_t e = cudaIpcCloseMemHandle(ptr);
  return e == cudaSuccess ? FA_OK : fa::fail(FA_ERR_CUDA, std::string("unmapping a peer's exchange buffer: ") + cudaGetErrorString(e));
}

int fa_b200_exchange_free(void* ptr) {
  fa::g_err.clear();
  const cudaError_t e = cudaFree(ptr);
  return e == cudaSuccess ? FA_OK : fa::fail(FA_ERR_CUDA, std::string("freeing the exchange buffer: ") + cudaGetErrorString(e));
}

size_t fa_b200_fwd_exchange_workspace(const fa_fwd_params* p) {
  if (!p) return 0;
  fa::g_err.clear();
  fa_fwd_params a = *p;
  a.partial_out = 1;
  a.lse_batch_stride = (int64_t)a.h * a.seqlen_q;
  a.lse_head_stride = a.seqlen_q;
  fa::Planned P;
  if (fa::make_plan(a, &P) != FA_OK) return 0;
  return fa::exchange_workspace(a, P.pl.kernel == FA_KERNEL_TCGEN05 ? 1 : P.pl.num_splits);
}

int fa_b200_fwd_exchange(const fa_fwd_params* p, void* workspace, size_t workspace_bytes, const fa_exchange* x, void* stream) {
  if (!p || !x) return fa::fail(FA_ERR_INVALID, "null argument");
  fa::g_err.clear();
  return fa::run_fwd_exchange(*p, workspace, workspace_bytes, *x, reinterpret_cast<cudaStream_t>(stream));
}

int fa_b200_fwd_plan(const fa_fwd_params* p, fa_fwd_plan* plan) {
  if (!p || !plan) return fa::fail(FA_ERR_INVALID, "null argument");
  fa::g_err.clear();
  fa::Planned P;
  int rc = fa::make_plan(*p, &P);
  if (rc == FA_OK) *plan = P.pl;
  return rc;
}

int fa_b200_combine(const fa_combine_params* p, void* stream) {
  if (!p) return fa::fail(FA_ERR_INVALID, "null params");
  fa::g_err.clear();
  if (!p->o_partial || !p->lse_partial || !p->o) return fa::fail(FA_ERR_INVALID, "o_partial, lse_partial and o must be non-null");
  if (p->num_splits <= 0 || p->d <= 0 || p->d % 4 != 0) return fa::fail(FA_ERR_INVALID, "bad num_splits or head dimension");
  return fa::launch_combine(*p, reinterpret_cast<cudaStream_t>(stream));
}

int fa_b200_normalize_window(int32_t seqlen_q, int32_t max_seqlen_k, int32_t causal, int32_t* window_left,
                             int32_t* window_right, int32_t* is_causal, int32_t* is_local) {
  if (!window_left || !window_right || !is_causal || !is_local) return fa::fail(FA_ERR_INVALID, "null argument");
  int wl = *window_left, wr = *window_right;
  bool c = false, l = false;
  fa::normalize_window(seqlen_q, max_seqlen_k, causal != 0, wl, wr, c, l);
  *window_left = wl;
  *window_right = wr;
  *is_causal = c;
  *is_local = l;
  return FA_OK;
}

int fa_b200_check_status(void* stream) {
  const int v = fa::tc5_read_status(reinterpret_cast<cudaStream_t>(stream));
  if (v == 0) return FA_OK;
  if (v < 0) return fa::fail(FA_ERR_CUDA, "cannot read the device status word");
  if (v & fa::kStatusExchangeTimeout)
    return fa::fail(FA_ERR_CUDA, "a rank did not deliver its partial to the cross-GPU merge within the time limit "
                                 "(results of that call are invalid)");
  if (v & fa::kStatusBadIndex)
    return fa::fail(FA_ERR_INVALID, "a block_table / cache_batch_idx entry or a cache length was out of range "
                                    "(the kernels read zeros instead; results of that launch are invalid)");
  if (v & 0x40000000)
    return fa::fail(FA_ERR_CUDA, "a bounded device-side wait gave up in CTA " + std::to_string(v & 0xffffff) +
                                     " of the decode kernel (results of that launch are invalid)");
  if (v & 0x20000000)
    return fa::fail(FA_ERR_CUDA, "the tcgen05 kernel found its shared memory base not 1024-byte aligned (nothing was computed)");
  return fa::fail(FA_ERR_CUDA, "bounded device-side wait " + std::to_string((v >> 16) & 0xff) + " gave up in CTA " +
                                   std::to_string((v & 0xffff) - 1) +
                                   " of the tcgen05 kernel (results of that launch are invalid)");
}

const char* fa_b200_last_error(void) { return fa::g_err.c_str(); }

const char* fa_b200_status_string(int status) {
  switch (status) {
    case FA_OK: return "ok";
    case FA_ERR_INVALID: return "invalid argument";
    case FA_ERR_UNSUPPORTED: return "unsupported";
    case FA_ERR_CUDA: return "CUDA error";
    case FA_ERR_WORKSPACE: return "workspace missing or too small";
  }
  return "unknown status";
}

int fa_b200_abi_version(void) { return FA_B200_ABI_VERSION; }

long long fa_b200_launch_count(void) { return fa::g_launches.load(); }

}  // extern "C"
