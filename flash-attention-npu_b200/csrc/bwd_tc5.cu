// tcgen05 backward kernels: TMA descriptors and launch (kernels in bwd_tc5_kernel.cuh).
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <string>
#include <type_traits>

#include "bwd_tc5_kernel.cuh"
#include "tc5_api.cuh"

namespace fa {

template <typename T>
struct TypeTag { using type = T; };

// Head dims up to 128 (tiles of 64 or 128 columns; the TMA unit zero-fills beyond the head dim); packed input needs the
// number of k / v rows for the TMA bounds.  Alignment and stride rules are those fa_b200_bwd has already checked.
bool bwd_tc5_eligible(const fa_bwd_params& a) {
  if (a.d > 128) return false;
  if (a.cu_seqlens_q && a.total_k <= 0) return false;
  return true;
}

int bwd_tc5_launch(const BwdParams& p, const fa_bwd_params& a, cudaStream_t st, std::string* err) {
  using namespace btc5;
  int32_t* status = device_status_word();
  if (!status) { *err = "cannot look up the device status word"; return FA_ERR_CUDA; }
  const bool varlen = a.cu_seqlens_q != nullptr;
  const int64_t q_rows = varlen ? a.total_q : a.seqlen_q, k_rows = varlen ? a.total_k : a.seqlen_k;
  const int64_t outer = varlen ? 1 : a.b;
  CUtensorMap tq, tdo, tk, tv, tq_u, tdo_u;  // _u: 64-row boxes (the units of the dK / dV kernel)
  // Packed sequences: one row axis for the whole tensor.  A tile that runs past the end of its sequence reads rows of
  // the next one (their P is 0 by the mask or by LSE = +inf), past the end of the tensor it reads zeros.
  const bool ok =
      tma_encode_rows(&tq, a.q, a.dtype, a.d, a.h, q_rows, outer, a.q_head_stride, a.q_row_stride, a.q_batch_stride, kBlk) &&
      tma_encode_rows(&tdo, a.dout, a.dtype, a.d, a.h, q_rows, outer, a.do_head_stride, a.do_row_stride, a.do_batch_stride, kBlk) &&
      tma_encode_rows(&tk, a.k, a.dtype, a.d, a.h_k, k_rows, outer, a.k_head_stride, a.k_row_stride, a.k_batch_stride, kBlk) &&
      tma_encode_rows(&tv, a.v, a.dtype, a.d, a.h_k, k_rows, outer, a.v_head_stride, a.v_row_stride, a.v_batch_stride, kBlk) &&
      tma_encode_rows(&tq_u, a.q, a.dtype, a.d, a.h, q_rows, outer, a.q_head_stride, a.q_row_stride, a.q_batch_stride, kUnit) &&
      tma_encode_rows(&tdo_u, a.dout, a.dtype, a.d, a.h, q_rows, outer, a.do_head_stride, a.do_row_stride, a.do_batch_stride, kUnit);
  if (!ok) { *err = "cuTensorMapEncodeTiled failed"; return FA_ERR_CUDA; }
  // persistent kernels: one CTA per SM (or per work item when there are fewer)
  int dev = 0, num_sm = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&num_sm, cudaDevAttrMultiProcessorCount, dev);
  const long long items_kv = (long long)((a.seqlen_k + kBlk - 1) / kBlk) * a.h_k * a.b;
  const long long items_q = (long long)((a.seqlen_q + kBlk - 1) / kBlk) * a.h * a.b;
  const dim3 grid_kv((unsigned)std::min<long long>(items_kv, num_sm)), grid_q((unsigned)std::min<long long>(items_q, num_sm));
  // the two work-item counters: the first 16 bytes of the workspace (where the mma.sync kernel has its fp32 dQ accumulator)
  int32_t* counters = reinterpret_cast<int32_t*>(p.dq_accum);
  cudaError_t e = cudaMemsetAsync(counters, 0, 2 * sizeof(int32_t), st);
  auto launch = [&](auto kern, dim3 grid, const CUtensorMap& mq, const CUtensorMap& mdo, int32_t* counter) {
    if (e != cudaSuccess) return;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e == cudaSuccess) {
      kern<<<grid, kThreads, kSmemBytes, st>>>(p, mq, mdo, tk, tv, status, counter);
      e = cudaGetLastError();
    }
  };
  auto both = [&](auto t_tag, auto fmt_tag, auto cap_tag, auto hd_tag) {  // tags: compile-time choices as types
    using T = typename decltype(t_tag)::type;
    constexpr uint32_t F = decltype(fmt_tag)::value;
    constexpr bool C = decltype(cap_tag)::value;
    constexpr int HD = decltype(hd_tag)::value;
    launch(bwd_dkv_kernel<T, F, C, HD>, grid_kv, tq_u, tdo_u, counters);
    launch(bwd_dq_kernel<T, F, C, HD>, grid_q, tq, tdo, counters + 1);
  };
  auto by_hd = [&](auto t_tag, auto fmt_tag, auto cap_tag) {
    if (a.d <= 64) both(t_tag, fmt_tag, cap_tag, std::integral_constant<int, 64>{});
    else both(t_tag, fmt_tag, cap_tag, std::integral_constant<int, 128>{});
  };
  auto by_cap = [&](auto t_tag, auto fmt_tag) {
    if (a.softcap > 0.f) by_hd(t_tag, fmt_tag, std::true_type{});
    else by_hd(t_tag, fmt_tag, std::false_type{});
  };
  if (a.dtype == FA_BF16) by_cap(TypeTag<__nv_bfloat16>{}, std::integral_constant<uint32_t, 1>{});
  else by_cap(TypeTag<__half>{}, std::integral_constant<uint32_t, 0>{});
  if (e != cudaSuccess) { *err = std::string("tcgen05 backward launch: ") + cudaGetErrorString(e); return FA_ERR_CUDA; }
  return FA_OK;
}

}  // namespace fa
