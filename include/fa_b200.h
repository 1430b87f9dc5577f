/*
 * fa_b200.h -- C ABI of the B200 (sm_100a) attention-forward library, libfa_b200.so.
 *
 * Every entry point is extern "C", takes plain pointers / sizes / POD structs and a
 * CUDA stream passed as void* (cudaStream_t).  No torch types cross this boundary.
 * All tensor pointers are DEVICE pointers; strides are in ELEMENTS; the last
 * dimension of every tensor is contiguous.  Calls are asynchronous on `stream`.
 *
 * Which reference interface each entry point replaces (paths inside the reference
 * project Minghuas/flash-attention-npu):
 *
 *   fa_b200_fwd                 mha_fwd            csrc/arch22/flash_attn_npu_v2/flash_api.cpp:628-826
 *                               mha_varlen_fwd     csrc/arch22/flash_attn_npu_v2/flash_api.cpp:828-1060
 *                               mha_fwd_kvcache    csrc/arch22/flash_attn_npu_v2/flash_api.cpp:356-626
 *                               mha_fwd (unified)  csrc/arch22/flash_attn_npu_v3/flash_api.cpp:60-491
 *                               mha_fwd (arch35)   csrc/arch35/flash_attn_npu_v3/mha_fwd.cpp:38-358
 *                               (pybind names: fwd / varlen_fwd / fwd_kvcache,
 *                                csrc/arch22/flash_attn_npu_v2/flash_api.cpp:1301-1309,
 *                                csrc/arch22/flash_attn_npu_v3/flash_api.cpp:816-822)
 *   fa_b200_fwd_plan            the host tiling / flash-decode decision of the same functions
 *                               (flash_api.cpp:514-556) and the split planner
 *                               csrc/arch22/flash_attn_npu_v3/fa_split.h:483-510
 *   fa_b200_plan_encode /       get_scheduler_metadata, csrc/arch22/flash_attn_npu_v3/flash_api.cpp:493-558 (plan
 *   fa_b200_plan_decode /       computed ahead of the call, returned as opaque bytes) and the scheduler_metadata_
 *   fa_b200_fwd_planned         argument of mha_fwd, csrc/arch22/flash_attn_npu_v3/flash_api.cpp:92,322-380
 *   fa_b200_exchange_* /        (none: sequence-sharded decode across GPUs over peer memory)
 *   fa_b200_fwd_exchange
 *   fa_b200_combine             CombineScale, csrc/arch22/flash_attn_npu_v2/CombineScale.hpp:76-357
 *                               (and the Python-level flash_attn_combine,
 *                                flash_attn_npu_v3/interface_arch22.py:930-931)
 *   fa_b200_normalize_window    the window normalisation block, flash_api.cpp:483-494
 *   fa_b200_check_status        (none: device-side wait watchdog of this library)
 *   fa_b200_fwd_noalloc         (none: allocation-free variant of fa_b200_fwd)
 */
#ifndef FA_B200_H
#define FA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FA_B200_ABI_VERSION 2

enum fa_status {
  FA_OK = 0,
  FA_ERR_INVALID = -1,     /* bad argument (the reference raises through TORCH_CHECK) */
  FA_ERR_UNSUPPORTED = -2, /* valid but not implemented */
  FA_ERR_CUDA = -3,        /* a CUDA runtime call failed */
  FA_ERR_WORKSPACE = -4    /* workspace missing or too small */
};

enum fa_dtype { FA_FP16 = 0, FA_BF16 = 1 };

enum fa_kernel_id {
  FA_KERNEL_AUTO = 0,
  FA_KERNEL_MMA = 1,    /* register-accumulator kernel (decode, paged, ragged shapes) */
  FA_KERNEL_TCGEN05 = 2, /* tcgen05 / TMEM / TMA prefill kernel */
  FA_KERNEL_DECODE = 3   /* producer / consumer split-KV decode kernel (bulk-copy streaming) */
};

typedef struct fa_fwd_params {
  /* ---- device pointers ---- */
  const void* q;      /* (b, s_q, h, d), or (total_q, h, d) when cu_seqlens_q is set */
  const void* k;      /* dense (b, s_k, h_k, d) | varlen (total_k, h_k, d) | cache (b_c, s_cache, h_k, d)
                         | pages (n_blocks, page, h_k, d) when block_table is set */
  const void* v;
  void* o;            /* same layout as q; fp32 when partial_out != 0 */
  float* lse;         /* (b, h, s_q) or (h, total_q); natural log; required */
  const void* k_new;  /* (b, s_new, h_k, d) appended in place at [L_b, L_b + s_new); may be NULL */
  const void* v_new;
  const int32_t* cu_seqlens_q;    /* (b + 1) or NULL */
  const int32_t* cu_seqlens_k;    /* (b + 1) or NULL */
  const int32_t* seqused_k;       /* (b) keys already in the cache (cache_seqlens) or NULL */
  const int32_t* cache_batch_idx; /* (b) row of the cache used by sequence i, or NULL */
  const int32_t* block_table;     /* (b, max_blocks) physical page of logical page, or NULL */
  const void* rotary_cos;         /* (rotary_seqlen, rotary_dim / 2), dtype of q, or NULL */
  const void* rotary_sin;
  const float* alibi_slopes;      /* (h) or (b, h) fp32, or NULL */
  /* ---- element strides ---- */
  int64_t q_batch_stride, q_row_stride, q_head_stride;
  int64_t k_batch_stride, k_row_stride, k_head_stride; /* batch stride = page stride when paged */
  int64_t v_batch_stride, v_row_stride, v_head_stride;
  int64_t o_batch_stride, o_row_stride, o_head_stride;
  int64_t knew_batch_stride, knew_row_stride, knew_head_stride;
  int64_t vnew_batch_stride, vnew_row_stride, vnew_head_stride;
  int64_t lse_batch_stride, lse_head_stride; /* query index has stride 1 */
  int64_t block_table_batch_stride;
  int64_t alibi_batch_stride; /* 0 for (h) */
  /* ---- sizes ---- */
  int32_t b;
  int32_t seqlen_q;   /* s_q, or max_seqlen_q for varlen */
  int32_t seqlen_k;   /* s_k / max_seqlen_k / s_cache / max_blocks * page: an upper bound of every key length */
  int32_t h, h_k, d;
  int32_t total_q;    /* rows of q when cu_seqlens_q is set, else b * s_q */
  int32_t seqlen_new; /* s_new, 0 without append */
  int32_t page_size;  /* rows per page when block_table is set */
  int32_t rotary_dim, rotary_seqlen, rotary_interleaved;
  int32_t dtype;      /* enum fa_dtype */
  /* ---- masking (raw user values; normalised inside exactly like flash_api.cpp:483-494) ---- */
  int32_t causal, window_left, window_right;
  /* max over the batch of the key length, if the host knows it; -1 = take the maximum of
     seqused_k + seqlen_new on the device (only read when a window is requested) */
  int32_t max_seqlen_k_known;
  /* ---- sequence-sharded decode: this call sees keys [kv_pos_offset, kv_pos_offset + s_k) of a
     sequence of kv_total keys (0 = not sharded); only the mask / alibi positions change ---- */
  int32_t kv_pos_offset, kv_total;
  int32_t partial_out; /* 1: o is fp32 (normalised partial), lse = -inf for rows without keys */
  /* ---- tuning ---- */
  int32_t num_splits; /* 0 heuristic, 1 never split, > 1 requested number of KV splits */
  int32_t kernel;     /* enum fa_kernel_id */
  int32_t num_sm;     /* 0 = query the current device */
  int32_t total_k;    /* rows of k / v when cu_seqlens_k is set (0 = not given: the tcgen05 kernel, which needs
                         the bound for its TMA descriptors, is then not used for varlen input) */
  int32_t kv_outer;   /* extent of the outermost dimension of k / v: the number of pages when block_table is set,
                         the number of cache rows when cache_batch_idx is set (required in both cases), else 0 = b.
                         Entries of block_table / cache_batch_idx outside [0, kv_outer) are never dereferenced:
                         the kernels read zeros instead and raise the status word (fa_b200_check_status) */
  float softmax_scale;
  float softcap; /* 0 = off */
} fa_fwd_params;

typedef struct fa_fwd_plan {
  int32_t kernel;       /* enum fa_kernel_id actually chosen */
  int32_t config;       /* tile configuration index inside that kernel family */
  int32_t pack_gqa;     /* 1: the query heads of one kv head share a tile */
  int32_t block_m, block_n;
  int32_t m_blocks;
  int32_t num_splits;   /* KV splits launched (1 = none) */
  int32_t blocks_per_split;
  int32_t grid, threads, smem_bytes;
  int32_t is_causal, is_local, window_left, window_right; /* after host normalisation */
  int32_t launches;     /* kernel launches fa_b200_fwd will make */
  size_t workspace_bytes;
} fa_fwd_plan;

typedef struct fa_combine_params {
  const float* o_partial;   /* fp32 normalised partial outputs */
  const float* lse_partial; /* fp32 natural-log LSE; -inf marks an empty partial */
  void* o;                  /* out_dtype */
  float* lse;               /* may be NULL */
  int64_t op_split_stride, op_batch_stride, op_row_stride, op_head_stride;
  int64_t lp_split_stride, lp_batch_stride, lp_row_stride, lp_head_stride;
  int64_t o_batch_stride, o_row_stride, o_head_stride;
  int64_t lse_batch_stride, lse_row_stride, lse_head_stride;
  int32_t num_splits, b, s, h, d;
  int32_t out_dtype;   /* enum fa_dtype, or 2 = fp32 */
  int32_t partial_out; /* 1: rows without keys give lse = -inf (result is itself a partial) */
} fa_combine_params;

/* Attention forward: dense, varlen, KV-cache (contiguous / paged) with optional fused
 * in-place append + rotary, split-KV with its merge.  `workspace` (device memory, 256-byte
 * aligned) must hold fa_fwd_plan.workspace_bytes; it may be NULL when that is 0. */
int fa_b200_fwd(const fa_fwd_params* p, void* workspace, size_t workspace_bytes, void* stream);

/* fa_b200_fwd for callers that must not allocate device memory: same arguments and results,
 * but the split-KV partials go to a 32 MiB array that is part of the library image (every GPU
 * that loads the library holds it until the process exits) instead of a caller workspace, and the
 * call makes no cudaMalloc / cudaFree or any other allocating call.  It always uses the
 * register-accumulator kernel.  A problem whose plan needs more than 32 MiB of scratch is
 * refused with FA_ERR_WORKSPACE (pass a smaller num_splits, or use fa_b200_fwd).
 * The first call on a device makes the driver load the library's device image (which holds the
 * 32 MiB array) and looks up the array's device address: the free memory the driver reports drops
 * by about that much at that moment.  Make that first call once at start-up, outside any stream
 * capture, before the phase in which nothing may be allocated.  All calls share the one array,
 * which keeps the previous call's contents (nothing in it needs clearing: every slot that is read is written first), so two calls that
 * overlap on the GPU -- different streams or threads -- race on it.
 * This entry point has no counterpart in the reference. */
int fa_b200_fwd_noalloc(const fa_fwd_params* p, void* stream);

/* Host-only: validates `p` and reports what fa_b200_fwd would launch.  Needs no GPU when
 * p->num_sm > 0. */
int fa_b200_fwd_plan(const fa_fwd_params* p, fa_fwd_plan* plan);

/* Plans as opaque bytes (the scheduler metadata of the reference's FA3-style API).
 * fa_b200_plan_encode (host-only) plans `p` like fa_b200_fwd_plan -- only sizes, flags and NULL-ness of the
 * pointers matter, the pointers are never dereferenced -- and writes FA_B200_PLAN_BYTES bytes: a header naming the
 * problem (batch, max_seqlen_q, max_seqlen_k, heads, head dim, dtype, mask) and the plan.
 * fa_b200_fwd_planned is fa_b200_fwd with such bytes: it refuses them (FA_ERR_INVALID) when they were made by
 * another library version or for other shapes, dtype or mask; takes over kernel family, tile configuration and KV
 * splits when the call has the same optional parts (cache lengths, pages, new tokens, ...) as the planned one; and
 * plans afresh otherwise.  With a KV cache, max_seqlen_k of the plan bounds the keys of every sequence: a longer
 * cache_seqlens entry is clamped and reported by fa_b200_check_status.  The workspace must hold the larger of
 * fa_b200_plan_decode's and fa_b200_fwd_plan's workspace_bytes. */
#define FA_B200_PLAN_BYTES 192
int fa_b200_plan_encode(const fa_fwd_params* p, void* buf, size_t buf_bytes);
int fa_b200_plan_decode(const void* buf, size_t buf_bytes, fa_fwd_plan* plan);
int fa_b200_fwd_planned(const fa_fwd_params* p, const void* plan, size_t plan_bytes, void* workspace, size_t workspace_bytes,
                        void* stream);

/* ------------------------------------------------------------------------------------------------
 * Backward (dQ, dK, dV) of the dense / packed-varlen forward.  Replaces the reference's mha_bwd /
 * mha_varlen_bwd (pybind names bwd, varlen_bwd: csrc/arch22/flash_attn_npu_v2/flash_api.cpp:1301-1309;
 * called from flash_attn_npu_v2/interface_arch22.py:232-252); arithmetic of the reference's golden
  * tests/fa_small_op_golden.py:160-353.  No dropout or alibi (refused by the Python layer).
 * Head dims up to 256 (multiples of 8).  All tensors as in fa_fwd_params: device pointers, element
 * strides, last dimension contiguous; dq / dk / dv are written completely.
 * ------------------------------------------------------------------------------------------------ */
typedef struct fa_bwd_params {
  const void* q;     /* (b, s_q, h, d) or (total_q, h, d) */
  const void* k;     /* (b, s_k, h_k, d) or (total_k, h_k, d) */
  const void* v;
  const void* o;     /* forward output, layout of q */
  const void* dout;  /* gradient of o */
  const float* lse;  /* forward softmax_lse, contiguous (b, h, s_q) / (h, total_q) */
  void* dq;
  void* dk;
  void* dv;
  const int32_t* cu_seqlens_q; /* (b + 1) or NULL */
  const int32_t* cu_seqlens_k;
  int64_t q_batch_stride, q_row_stride, q_head_stride;
  int64_t k_batch_stride, k_row_stride, k_head_stride;
  int64_t v_batch_stride, v_row_stride, v_head_stride;
  int64_t o_batch_stride, o_row_stride, o_head_stride;
  int64_t do_batch_stride, do_row_stride, do_head_stride;
  int64_t dq_batch_stride, dq_row_stride, dq_head_stride;
  int64_t dk_batch_stride, dk_row_stride, dk_head_stride;
  int64_t dv_batch_stride, dv_row_stride, dv_head_stride;
  int64_t lse_batch_stride, lse_head_stride;
  int32_t b, seqlen_q, seqlen_k; /* max_seqlen_q / max_seqlen_k for varlen */
  int32_t h, h_k, d, total_q;
  int32_t dtype, causal, window_left, window_right;
  float softmax_scale;
  float softcap; /* 0 = off */
  int32_t total_k; /* rows of k / v for packed input (the tcgen05 kernels' TMA bounds); 0 = not given */
  int32_t kernel;  /* 0 automatic; 1 force the mma.sync kernel; 2 force the tcgen05 kernels (FA_ERR_UNSUPPORTED if they do not cover the problem) */
} fa_bwd_params;

/* Bytes of device scratch fa_b200_bwd needs: rowsum(dO o O), plus the fp32 dQ accumulator where the mma.sync kernel runs
 * (the tcgen05 kernels need 16 bytes instead). */
size_t fa_b200_bwd_workspace_bytes(const fa_bwd_params* p);
/* Three launches on `stream`.  Head dims up to 128: rowsum, then two tcgen05 kernels (dK / dV per key block,
 * dQ per query block; no atomics, so the results are bit-reproducible).  Otherwise: a memset of the fp32 dQ accumulator,
 * rowsum, the mma.sync kernel (dQ through atomic adds), dQ conversion. */
int fa_b200_bwd(const fa_bwd_params* p, void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Sequence-sharded decode across GPUs over peer memory (one process per GPU, NVLink / NVSwitch).  No counterpart in
 * the reference (it has no distributed code); the merge arithmetic is CombineScale's
 * (csrc/arch22/flash_attn_npu_v2/CombineScale.hpp:165-309).
 * Every rank owns one exchange buffer that all ranks map (CUDA IPC): fa_b200_exchange_alloc returns the buffer and a
 * 64-byte handle to hand to the other ranks (any host channel), fa_b200_exchange_open maps a peer's buffer.
 * fa_b200_fwd_exchange runs the attention over this rank's shard of the keys (p->kv_pos_offset / p->kv_total give its
 * place in the sequence), then one kernel that merges this rank's split partials and stores the result into every
 * rank's buffer with plain peer stores followed by a release flag, then one kernel that waits for every rank's flag
 * and merges the shards into p->o / p->lse.  The wait is bounded (timeout_cycles, default about two seconds): when
 * a rank does not deliver, the kernel gives up, fa_b200_check_status reports it, the call's results are invalid and
 * the context stays usable.  All ranks must make the same sequence of calls on one buffer set; a buffer is sized for
 * at most the rows x head dim it was allocated for.  q must be dense (b, s_q, h, d).
 * ------------------------------------------------------------------------------------------------ */
#define FA_B200_MAX_RANKS 16
typedef struct fa_exchange {
  void* bufs[FA_B200_MAX_RANKS]; /* exchange buffer of every rank as mapped into this process; [rank] is this rank's own */
  size_t buf_bytes;              /* size each of them was allocated with */
  int32_t world, rank;
  int64_t timeout_cycles;        /* SM clock cycles the merge waits for the slowest rank; 0 = default */
} fa_exchange;
size_t fa_b200_exchange_bytes(int32_t world, int64_t rows, int32_t d); /* rows = b * s_q * h */
int fa_b200_exchange_alloc(size_t bytes, void** ptr, void* handle64);  /* cudaMalloc + zero + IPC handle */
int fa_b200_exchange_open(const void* handle64, void** ptr);
int fa_b200_exchange_close(void* ptr);
int fa_b200_exchange_free(void* ptr);
size_t fa_b200_fwd_exchange_workspace(const fa_fwd_params* p);
int fa_b200_fwd_exchange(const fa_fwd_params* p, void* workspace, size_t workspace_bytes, const fa_exchange* x, void* stream);

/* Merge of split partials (also used across GPUs). */
int fa_b200_combine(const fa_combine_params* p, void* stream);

/* Host-only window normalisation; writes the normalised window and the two mode flags. */
int fa_b200_normalize_window(int32_t seqlen_q, int32_t max_seqlen_k, int32_t causal, int32_t* window_left,
                             int32_t* window_right, int32_t* is_causal, int32_t* is_local);

/* Synchronises `stream` and reports whether any bounded device-side wait of earlier launches gave
 * up (FA_ERR_CUDA) -- the kernels never spin forever; a protocol failure ends up here instead of
 * a hung GPU.  Clears the flag.  No counterpart in the reference (its kernels block in
 * CrossCoreWaitFlag, csrc/arch22/flash_attn_npu_v2/mha_fwd_kvcache.cpp:999-1001). */
int fa_b200_check_status(void* stream);

/* Message of the last error on the calling thread ("" if none). */
const char* fa_b200_last_error(void);
const char* fa_b200_status_string(int status);
int fa_b200_abi_version(void);

/* Kernel launches this library has issued in this process so far (all entry points, all threads).  No counterpart
 * in the reference; callers difference it around a region to count launches, e.g. to check that a path ran on the
 * GPU kernels of this library and how many of them it took. */
long long fa_b200_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* FA_B200_H */
