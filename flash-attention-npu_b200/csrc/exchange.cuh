// Cross-GPU merge of sequence-sharded decode partials over peer memory (NVLink), one process per GPU.
//
// Every rank holds one exchange buffer that all ranks have mapped (CUDA IPC):
//   header | data[2 parities][world][rows][d + 4] fp32   (a row is O[d], LSE, 3 floats of padding: 16-byte aligned)
// Step e (a device-side epoch, so that a captured graph can be replayed):
//   push kernel    merges this rank's split partials row by row (the arithmetic of combine.cuh) and writes the
//                  row (O, LSE) into slot [e & 1][rank] of EVERY rank's buffer with plain stores; the CTA that
//                  finishes last publishes the epoch into flags[rank] of every rank (release, system scope);
//   merge kernel   waits until flags[r] >= e for every r (acquire, system scope, bounded by a cycle budget: on
//                  expiry it raises kStatusExchangeTimeout and goes on, the results of that call are invalid),
//                  then merges the world partials of slot [e & 1] into the output.
// A rank can be at most one step ahead of another (its merge of step e waits for the others' push of step e, which
// follows their merge of step e - 1 on their streams), so two parities are enough.  No multicast, no collective
// library: plain peer stores and loads.  The merged result equals what an all-gather followed by the merge kernel
// gives (same arithmetic, same order), which is how flash_b200.dist checks it.
#pragma once

#include "combine.cuh"

namespace fa {

constexpr int kStatusExchangeTimeout = 0x08000000;
constexpr int kXchgHeaderBytes = 256;

struct XchgHeader {
  unsigned int epoch;        // steps this rank has pushed
  unsigned int done_ctas;    // push kernel: CTAs finished in the current step
  unsigned int flags[FA_B200_MAX_RANKS];  // flags[r]: steps rank r has delivered into this buffer
};
static_assert(sizeof(XchgHeader) <= kXchgHeaderBytes, "exchange header too large");

struct XchgParams {
  fa_combine_params c;      // local partials (o_partial / lse_partial, strides, sizes); o / lse = final output
  char* bufs[FA_B200_MAX_RANKS];
  int32_t world, rank;
  long long timeout_cycles;
  int32_t* status;
};

__device__ __forceinline__ float* xchg_row(char* buf, int parity, int world, int src_rank, int64_t n_rows, int d, int64_t row) {
  const int64_t slot = ((int64_t)parity * world + src_rank) * n_rows + row;
  return reinterpret_cast<float*>(buf + kXchgHeaderBytes) + slot * (d + 4);
}

__global__ void __launch_bounds__(kCombineWarps * 32) xchg_push_kernel(const __grid_constant__ XchgParams p) {
  asm volatile("griddepcontrol.wait;\n" ::: "memory");  // the attention kernel in front has completed
  const fa_combine_params& c = p.c;
  XchgHeader* hdr = reinterpret_cast<XchgHeader*>(p.bufs[p.rank]);
  const unsigned int epoch = *reinterpret_cast<volatile unsigned int*>(&hdr->epoch) + 1u;  // this step
  const int parity = (int)(epoch & 1u);
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kCombineWarps + (threadIdx.x >> 5);
  const int64_t n_rows = (int64_t)c.b * c.s * c.h;
  if (row < n_rows) {
    const int hh = (int)(row % c.h);
    const int ss = (int)((row / c.h) % c.s);
    const int bb = (int)(row / ((int64_t)c.h * c.s));
    const float* lp = c.lse_partial + bb * c.lp_batch_stride + ss * c.lp_row_stride + hh * c.lp_head_stride;
    const float* op = c.o_partial + bb * c.op_batch_stride + ss * c.op_row_stride + hh * c.op_head_stride;
    // the arithmetic of combine_kernel; more than 32 local splits do not occur with a sharded key range
    float l_mine, w_mine, m, tot;
    bool dead;
    const int n = min(c.num_splits, 32);
    merge_weights(n, lane, [&](int i) { return lp[(int64_t)i * c.lp_split_stride]; }, l_mine, w_mine, m, tot, dead);
    const float lse_row = dead ? -INFINITY : m + logf(tot);
    for (int c0 = 0; c0 < c.d; c0 += 128) {
      const int col = c0 + lane * 4;
      const bool on = col < c.d;
      const float4 acc = merge_columns(n, l_mine, w_mine, [&](int i) {
        return on ? *reinterpret_cast<const float4*>(op + (int64_t)i * c.op_split_stride + col) : make_float4(0.f, 0.f, 0.f, 0.f);
      });
      if (on)
        for (int r = 0; r < p.world; ++r)  // the same row into every rank's buffer (peer stores over NVLink)
          *reinterpret_cast<float4*>(xchg_row(p.bufs[r], parity, p.world, p.rank, n_rows, c.d, row) + col) = acc;
    }
    if (lane == 0)
      for (int r = 0; r < p.world; ++r) xchg_row(p.bufs[r], parity, p.world, p.rank, n_rows, c.d, row)[c.d] = lse_row;
  }
  // The CTA that finishes last publishes the step to every rank: one thread per rank, so that the release stores
  // (each of which waits for its own round trip over NVLink) go out side by side instead of one after the other.
  __threadfence_system();
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) {
    const unsigned int before = atomicAdd(&hdr->done_ctas, 1u);
    s_last = (before + 1u == gridDim.x) ? 1 : 0;
    if (s_last) {
      hdr->done_ctas = 0u;
      *reinterpret_cast<volatile unsigned int*>(&hdr->epoch) = epoch;
      __threadfence_system();
    }
  }
  __syncthreads();
  if (s_last && (int)threadIdx.x < p.world) {
    unsigned int* flag = &reinterpret_cast<XchgHeader*>(p.bufs[threadIdx.x])->flags[p.rank];
    asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(flag), "r"(epoch) : "memory");
  }
}

template <typename OutT>
__global__ void __launch_bounds__(kCombineWarps * 32) xchg_merge_kernel(const __grid_constant__ XchgParams p) {
  asm volatile("griddepcontrol.wait;\n" ::: "memory");  // this rank's push kernel has completed (and set the epoch)
  const fa_combine_params& c = p.c;
  char* buf = p.bufs[p.rank];
  XchgHeader* hdr = reinterpret_cast<XchgHeader*>(buf);
  const unsigned int epoch = *reinterpret_cast<volatile unsigned int*>(&hdr->epoch);
  const int parity = (int)(epoch & 1u);
  // thread r waits for rank r's flag (all ranks side by side); every wait has the same cycle budget
  int ok = 1;
  if ((int)threadIdx.x < p.world) {
    const unsigned int* flag = &hdr->flags[threadIdx.x];
    const long long t0 = clock64();
    for (;;) {
      unsigned int v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(flag) : "memory");
      if ((int)(v - epoch) >= 0) break;
      if (clock64() - t0 > p.timeout_cycles) {  // a rank did not deliver: give up, say so, keep the context usable
        ok = 0;
        if (p.status) atomicOr(p.status, kStatusExchangeTimeout);
        break;
      }
      __nanosleep(100);
    }
  }
  if (!__syncthreads_and(ok)) return;
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kCombineWarps + (threadIdx.x >> 5);
  const int64_t n_rows = (int64_t)c.b * c.s * c.h;
  if (row >= n_rows) return;
  const int hh = (int)(row % c.h);
  const int ss = (int)((row / c.h) % c.s);
  const int bb = (int)(row / ((int64_t)c.h * c.s));
  float l_mine, w_mine, m, tot;
  bool dead;
  merge_weights(p.world, lane, [&](int r) { return __ldcg(xchg_row(buf, parity, p.world, r, n_rows, c.d, row) + c.d); }, l_mine,
                w_mine, m, tot, dead);
  OutT* out = reinterpret_cast<OutT*>(c.o) + bb * c.o_batch_stride + ss * c.o_row_stride + hh * c.o_head_stride;
  for (int c0 = 0; c0 < c.d; c0 += 128) {
    const int col = c0 + lane * 4;
    const bool on = col < c.d;
    const float4 acc = merge_columns(p.world, l_mine, w_mine, [&](int r) {
      return on ? __ldcg(reinterpret_cast<const float4*>(xchg_row(buf, parity, p.world, r, n_rows, c.d, row) + col))
                : make_float4(0.f, 0.f, 0.f, 0.f);
    });
    if (on) store4<OutT>(out + col, acc);
  }
  if (c.lse && lane == 0)
    c.lse[bb * c.lse_batch_stride + ss * c.lse_row_stride + hh * c.lse_head_stride] = dead ? INFINITY : m + logf(tot);
}

}  // namespace fa
