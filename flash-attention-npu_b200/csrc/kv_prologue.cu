// Prologue of the tcgen05 prefill kernel for flash_attn_with_kvcache calls that bring new tokens:
// k_new (rotated when rotary tables are given) and v_new go into the cache at positions
// cache_seqlens .. cache_seqlens + s_new - 1, and the rotated q goes to a workspace the prefill
// kernel reads instead of q.  Same arithmetic (append_to_cache, rotary_chunk) as the kernels that
// fuse the append, so the cache update is bit-identical whichever kernel serves the call
// (reference semantics: flash_attn_npu_v2/interface_arch22.py:1452-1537).
#include "fwd_mma.cuh"
#include "kv_prologue.cuh"

namespace fa {

template <typename T_>
struct PrologueTraits {
  using T = T_;
  static constexpr int NTHREADS = 256;
};

// grid (h_k [+ h], b): blocks x < h_k append kv head x of batch entry y; the others rotate q head x - h_k.
template <typename T>
__global__ void __launch_bounds__(256) kv_prologue_kernel(const __grid_constant__ KParams p, T* q_rot, int rot_per_token) {
  using Tr = PrologueTraits<T>;
  const int bi = blockIdx.y, unit = blockIdx.x, tid = threadIdx.x;
  const int l_cache = cache_len(p.a, bi, p.status);
  if (unit < p.a.h_k) {
    const int hk = unit;
    SeqView<T> sv;
    sv.q = nullptr;
    sv.q_len = p.a.seqlen_q;
    sv.q_row0 = 0;
    sv.l_cache = l_cache;
    sv.k_len = l_cache + p.a.seqlen_new;
    const T* kb = reinterpret_cast<const T*>(p.a.k) + (int64_t)hk * p.a.k_head_stride;
    const T* vb = reinterpret_cast<const T*>(p.a.v) + (int64_t)hk * p.a.v_head_stride;
    sv.pages = nullptr;
    if (p.a.block_table) {
      sv.pages = p.a.block_table + (int64_t)bi * p.a.block_table_batch_stride;
    } else {
      const int batch_row = p.a.cache_batch_idx ? outer_index(p.a, p.a.cache_batch_idx[bi], p.status) : bi;
      kb += (int64_t)batch_row * p.a.k_batch_stride;
      vb += (int64_t)batch_row * p.a.v_batch_stride;
    }
    sv.k = kb;
    sv.v = vb;
    sv.knew = reinterpret_cast<const T*>(p.a.k_new) + (int64_t)bi * p.a.knew_batch_stride + (int64_t)hk * p.a.knew_head_stride;
    sv.vnew = reinterpret_cast<const T*>(p.a.v_new) + (int64_t)bi * p.a.vnew_batch_stride + (int64_t)hk * p.a.vnew_head_stride;
    append_to_cache<Tr>(p, sv, tid, Tr::NTHREADS);
    return;
  }
  if (!q_rot) return;
  const int head = unit - p.a.h_k;
  const int chunks = p.a.d >> 3;
  const T* qb = reinterpret_cast<const T*>(p.a.q) + (int64_t)bi * p.a.q_batch_stride + (int64_t)head * p.a.q_head_stride;
  T* ob = q_rot + ((int64_t)bi * p.a.seqlen_q * p.a.h + head) * p.a.d;
  for (int c = tid; c < p.a.seqlen_q * chunks; c += Tr::NTHREADS) {
    const int i = c / chunks, ch = c - i * chunks;
    const T* qrow = qb + (int64_t)i * p.a.q_row_stride;
    uint4 q4 = *reinterpret_cast<const uint4*>(qrow + ch * 8);
    const int pos = l_cache + p.a.kv_pos_offset + (rot_per_token ? i : 0);
    const T* cosr = reinterpret_cast<const T*>(p.a.rotary_cos) + (int64_t)pos * (p.a.rotary_dim >> 1);
    const T* sinr = reinterpret_cast<const T*>(p.a.rotary_sin) + (int64_t)pos * (p.a.rotary_dim >> 1);
    q4 = rotary_chunk<T>(q4, qrow, ch * 8, cosr, sinr, p.a.rotary_dim, p.a.rotary_interleaved != 0);
    *reinterpret_cast<uint4*>(ob + (int64_t)i * p.a.h * p.a.d + ch * 8) = q4;
  }
}

cudaError_t launch_kv_prologue(const KParams& p, void* q_rot, bool rot_per_token, cudaStream_t st) {
  const dim3 grid(p.a.h_k + (q_rot ? p.a.h : 0), p.a.b);
  if (p.a.dtype == FA_BF16)
    kv_prologue_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(p, reinterpret_cast<__nv_bfloat16*>(q_rot), rot_per_token ? 1 : 0);
  else
    kv_prologue_kernel<__half><<<grid, 256, 0, st>>>(p, reinterpret_cast<__half*>(q_rot), rot_per_token ? 1 : 0);
  return cudaGetLastError();
}

}  // namespace fa
