// Attention backward: C-ABI entry point and launch (kernels in bwd_kernel.cuh).
#include <cuda_runtime.h>

#include <algorithm>
#include <cstring>
#include <string>

#include "bwd_kernel.cuh"
#include "tc5_api.cuh"

namespace fa {

int fail_bwd(int code, const std::string& msg);  // api.cu: records the thread's last error
bool bwd_tc5_eligible(const fa_bwd_params& a);   // bwd_tc5.cu
int bwd_tc5_launch(const BwdParams& p, const fa_bwd_params& a, cudaStream_t st, std::string* err);
void count_launches(int n);                      // api.cu: fa_b200_launch_count

static size_t align16(size_t x) { return (x + 15) & ~(size_t)15; }

template <int HD, typename T>
static cudaError_t launch_bwd(const BwdParams& p, int n_kblocks, cudaStream_t st) {
  constexpr int smem = BwdSmem<HD>::BYTES;
  cudaError_t e = cudaFuncSetAttribute(bwd_kernel<HD, T>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  bwd_kernel<HD, T><<<dim3(n_kblocks, p.h_k, p.b), kBwdThreads, smem, st>>>(p);
  return cudaGetLastError();
}

}  // namespace fa

extern "C" {

// First part of the workspace: the fp32 dQ accumulator of the mma.sync kernel, or the two work-item counters of the
// tcgen05 kernels (which write dQ directly).
static size_t bwd_accum_bytes(const fa_bwd_params* a, int64_t rows) {
  if (a->kernel != 1 && fa::bwd_tc5_eligible(*a)) return 16;
  const int d_pad = a->d <= 64 ? 64 : (a->d <= 128 ? 128 : 256);
  return fa::align16((size_t)rows * a->h * d_pad * sizeof(float));
}

size_t fa_b200_bwd_workspace_bytes(const fa_bwd_params* a) {
  if (!a) return 0;
  const int64_t rows = a->cu_seqlens_q ? a->total_q : (int64_t)a->b * a->seqlen_q;
  return bwd_accum_bytes(a, rows) + fa::align16((size_t)rows * a->h * sizeof(float));
}

int fa_b200_bwd(const fa_bwd_params* a, void* workspace, size_t workspace_bytes, void* stream) {
  using namespace fa;
  if (!a) return fail_bwd(FA_ERR_INVALID, "null parameter block");
  if (!a->q || !a->k || !a->v || !a->o || !a->dout || !a->lse || !a->dq || !a->dk || !a->dv)
    return fail_bwd(FA_ERR_INVALID, "q, k, v, o, dout, lse, dq, dk and dv must be non-null");
  if (a->dtype != FA_FP16 && a->dtype != FA_BF16) return fail_bwd(FA_ERR_INVALID, "FlashAttention only supports FP16 and BF16 data types");
  if (a->b <= 0 || a->h <= 0 || a->h_k <= 0 || a->h % a->h_k != 0)
    return fail_bwd(FA_ERR_INVALID, "Number of heads in key/value must divide number of heads in query");
  if (a->d <= 0 || a->d % 8 != 0) return fail_bwd(FA_ERR_INVALID, "head dimension must be a multiple of 8 (pad it on the caller side)");
  if (a->d > 256) return fail_bwd(FA_ERR_INVALID, "FlashAttention only supports head dimension at most 256");
  if (a->softcap < 0.f) return fail_bwd(FA_ERR_INVALID, "softcap must be non-negative (0.0 disables softcap)");
  if ((a->cu_seqlens_q != nullptr) != (a->cu_seqlens_k != nullptr))
    return fail_bwd(FA_ERR_INVALID, "cu_seqlens_q and cu_seqlens_k must be passed together");
  const bool varlen = a->cu_seqlens_q != nullptr;
  const int64_t rows = varlen ? a->total_q : (int64_t)a->b * a->seqlen_q;
  if (rows == 0 || a->seqlen_k == 0) return FA_OK;
  const int64_t canon_head = varlen ? a->total_q : a->seqlen_q;
  if (a->lse_head_stride != canon_head || (!varlen && a->lse_batch_stride != (int64_t)a->h * a->seqlen_q))
    return fail_bwd(FA_ERR_INVALID, "softmax_lse must be contiguous (b, h, s_q) / (h, total_q)");
  const size_t need = fa_b200_bwd_workspace_bytes(a);
  if (!workspace || workspace_bytes < need) return fail_bwd(FA_ERR_WORKSPACE, "workspace missing or too small");
  if ((reinterpret_cast<uintptr_t>(workspace) & 15) != 0) return fail_bwd(FA_ERR_WORKSPACE, "workspace must be 16-byte aligned");
  const int64_t st[] = {a->q_row_stride, a->q_head_stride, a->k_row_stride, a->k_head_stride, a->v_row_stride, a->v_head_stride,
                        a->o_row_stride, a->o_head_stride, a->do_row_stride, a->do_head_stride, a->dq_row_stride,
                        a->dq_head_stride, a->dk_row_stride, a->dk_head_stride, a->dv_row_stride, a->dv_head_stride,
                        a->q_batch_stride, a->k_batch_stride, a->v_batch_stride, a->do_batch_stride, a->dq_batch_stride,
                        a->dk_batch_stride, a->dv_batch_stride, a->o_batch_stride};
  for (int64_t s : st)
    if (s % 8 != 0) return fail_bwd(FA_ERR_INVALID, "tensor strides must be multiples of 8 elements (16-byte rows)");
  const void* ptrs[] = {a->q, a->k, a->v, a->o, a->dout, a->dq, a->dk, a->dv};
  for (const void* ptr : ptrs)
    if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0) return fail_bwd(FA_ERR_INVALID, "tensors must be 16-byte aligned");

  cudaStream_t cs = reinterpret_cast<cudaStream_t>(stream);
  BwdParams p;
  std::memset(&p, 0, sizeof(p));
  p.q = a->q; p.k = a->k; p.v = a->v; p.o = a->o; p.dout = a->dout; p.lse = a->lse;
  p.dq = a->dq; p.dk = a->dk; p.dv = a->dv;
  p.cu_seqlens_q = a->cu_seqlens_q; p.cu_seqlens_k = a->cu_seqlens_k;
  p.q_batch_stride = a->q_batch_stride; p.q_row_stride = a->q_row_stride; p.q_head_stride = a->q_head_stride;
  p.k_batch_stride = a->k_batch_stride; p.k_row_stride = a->k_row_stride; p.k_head_stride = a->k_head_stride;
  p.v_batch_stride = a->v_batch_stride; p.v_row_stride = a->v_row_stride; p.v_head_stride = a->v_head_stride;
  p.o_batch_stride = a->o_batch_stride; p.o_row_stride = a->o_row_stride; p.o_head_stride = a->o_head_stride;
  p.do_batch_stride = a->do_batch_stride; p.do_row_stride = a->do_row_stride; p.do_head_stride = a->do_head_stride;
  p.dq_batch_stride = a->dq_batch_stride; p.dq_row_stride = a->dq_row_stride; p.dq_head_stride = a->dq_head_stride;
  p.dk_batch_stride = a->dk_batch_stride; p.dk_row_stride = a->dk_row_stride; p.dk_head_stride = a->dk_head_stride;
  p.dv_batch_stride = a->dv_batch_stride; p.dv_row_stride = a->dv_row_stride; p.dv_head_stride = a->dv_head_stride;
  p.lse_batch_stride = a->lse_batch_stride; p.lse_head_stride = a->lse_head_stride;
  p.b = a->b; p.seqlen_q = a->seqlen_q; p.seqlen_k = a->seqlen_k; p.h = a->h; p.h_k = a->h_k; p.d = a->d;
  p.d_pad = a->d <= 64 ? 64 : (a->d <= 128 ? 128 : 256);
  p.total_q = (int32_t)rows;
  // window normalisation of the golden (tests/fa_small_op_golden.py:21-33; the same rule as the forward's host code)
  int wl = a->window_left, wr = a->window_right;
  if (wl >= a->seqlen_k - 1) wl = -1;
  if (wr >= a->seqlen_q - 1) wr = -1;
  if (a->causal) wr = 0;
  p.is_causal = (wl < 0 && wr == 0) ? 1 : 0;
  p.is_local = ((wl >= 0 || wr >= 0) && !p.is_causal) ? 1 : 0;
  p.wl = wl; p.wr = wr;
  p.softmax_scale = a->softmax_scale;
  p.scale_log2 = a->softmax_scale * kLog2e;
  p.softcap = a->softcap;
  const size_t acc_bytes = bwd_accum_bytes(a, rows);
  p.dq_accum = reinterpret_cast<float*>(workspace);
  p.delta = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + acc_bytes);

  if (a->kernel < 0 || a->kernel > 2) return fail_bwd(FA_ERR_INVALID, "kernel must be 0 (automatic), 1 (mma.sync) or 2 (tcgen05)");
  const bool tc5 = a->kernel != 1 && bwd_tc5_eligible(*a);
  if (a->kernel == 2 && !tc5)
    return fail_bwd(FA_ERR_UNSUPPORTED, "the tcgen05 backward covers head dims up to 128 (packed input: total_k given)");
  cudaError_t e = cudaSuccess;
  if (!tc5) e = cudaMemsetAsync(p.dq_accum, 0, acc_bytes, cs);
  if (e != cudaSuccess) return fail_bwd(FA_ERR_CUDA, std::string("cudaMemsetAsync: ") + cudaGetErrorString(e));
  const bool bf = a->dtype == FA_BF16;
  const int delta_grid = (int)((rows * a->h + 7) / 8);  // 4 warps x 2 rows per block
  if (bf) bwd_delta_kernel<__nv_bfloat16><<<delta_grid, 128, 0, cs>>>(p);
  else bwd_delta_kernel<__half><<<delta_grid, 128, 0, cs>>>(p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail_bwd(FA_ERR_CUDA, std::string("backward (delta) launch: ") + cudaGetErrorString(e));
  if (tc5) {
    std::string err;
    const int rc = bwd_tc5_launch(p, *a, cs, &err);
    if (rc != FA_OK) return fail_bwd(rc, err);
    count_launches(3);
    return FA_OK;
  }
  const int n_kblocks = (a->seqlen_k + kBwdBN - 1) / kBwdBN;
  if (p.d_pad == 64) e = bf ? launch_bwd<64, __nv_bfloat16>(p, n_kblocks, cs) : launch_bwd<64, __half>(p, n_kblocks, cs);
  else if (p.d_pad == 128) e = bf ? launch_bwd<128, __nv_bfloat16>(p, n_kblocks, cs) : launch_bwd<128, __half>(p, n_kblocks, cs);
  else e = bf ? launch_bwd<256, __nv_bfloat16>(p, n_kblocks, cs) : launch_bwd<256, __half>(p, n_kblocks, cs);
  if (e != cudaSuccess) return fail_bwd(FA_ERR_CUDA, std::string("backward launch: ") + cudaGetErrorString(e));
  const int conv_grid = (int)std::min<int64_t>((rows * a->h * (p.d_pad / 4) + 255) / 256, 148 * 8);
  if (bf) bwd_convert_kernel<__nv_bfloat16><<<conv_grid, 256, 0, cs>>>(p);
  else bwd_convert_kernel<__half><<<conv_grid, 256, 0, cs>>>(p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail_bwd(FA_ERR_CUDA, std::string("backward (convert) launch: ") + cudaGetErrorString(e));
  count_launches(3);
  return FA_OK;
}

}  // extern "C"
