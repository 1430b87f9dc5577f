#!/usr/bin/env python
"""Benchmark of the attention-forward hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c3|c4|c5] [--impl reference]

Prints ONE JSON line (rank 0).  The headline (metric, value, ...) is the causal-prefill configuration the
metric's TFLOP/s half is quoted on (c2: bf16, batch 4, seqlen 4096, 32 heads, head dim 128); the decode half of
the metric (HBM GB/s on c3 contiguous decode, c4 paged windowed decode and c5 long-context sequence-sharded
decode) is measured in the same run and reported, entry by entry with the same keys, under "workloads", and so is
the backward at the headline shape (c2_bwd: dQ, dK, dV from the forward's out and lse).
--workload X measures X alone.  A "step" is one forward (c2_bwd: one backward) over one batch of seeded synthetic inputs.

* value        whole-job throughput with inputs resident in HBM, timed with CUDA events on the
               launching stream (barrier + synchronize on both sides, max over ranks).
* e2e          the same metric through the public API with HOST (pinned) buffers: host->device copy
               of q, k, v and device->host copy of O and LSE inside the timed region.
* roofline     achieved = algorithmic FLOPs (prefill) or bytes (decode) per launch / average kernel
               time; peak from MEASURED_PEAKS.json (driver-measured on this pool) or the fallback.
* cpu_baseline the CPU oracle (a port of the reference's PyTorch golden) timed on the host cores on
               a bounded sample of the same workload.
With N > 1 (torchrun) every rank runs the same per-GPU workload on its own independent
(batch x head) units -- no collective on the data path -- so scaling is "weak"; c5 is the one
workload with an exchange step (sequence-sharded KV, all-gather of the partials + merge).
"""
import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "flash-attention-npu_b200"))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

# dram__bytes_read.sum + dram__bytes_write.sum of the dominant kernel, from one ncu capture of a shrunk case of each
# workload (profiles/*.md), as (bytes, units of that case): traffic grows in proportion to the units a launch
# processes, so a full launch is  bytes * units / units_of_the_case.
NCU_TRAFFIC = {
    "c2": (586.76e6 + 129.76e6, 549755813888.0, "ncu, full size (profiles/fwd_tc5_kernel_c2_full_traffic.md), scaled by FLOPs"),
    "c2_bwd": (135.32e6 + 38.92e6, 343597383680.0, "ncu, dK / dV kernel at batch 1 of 4 (profiles/bwd_dkv_dq_kernels_c2_shrink4.md), scaled by FLOPs"),
    "c3": (255.98e6 + 4.84e6, 253687872.0, "ncu, batch 16 of 64 (profiles/fwd_decode_kernel_c3_shrink4.md), scaled by bytes"),
    "c4": (132.48e6 + 3.92e6, 130785280.0, "ncu, batch 8 of 32 (profiles/fwd_decode_kernel_c4_shrink4.md), scaled by bytes"),
    "c5": (537.13e6 + 3.56e6, 537135104.0, "ncu, key length / 8 (profiles/fwd_decode_kernel_c5_shrink8.md), scaled by bytes"),
}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        d["_source"] = "measured"
        return d
    d = dict(FALLBACK_PEAKS)
    d["_source"] = "fallback"
    return d


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons of one GPU while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.samples, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        mhz, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            parts = [x.strip() for x in s.split(",")]
            if len(parts) < 6:
                continue
            try:
                mhz.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        mhz.sort()
        # the busiest half of the samples is "under load"
        load = mhz[len(mhz) // 2:] if mhz else []
        med = load[len(load) // 2] if load else None
        return {"sm_mhz": med, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(mhz)}


# ------------------------------------------------------------------------------------------------
# workloads
# ------------------------------------------------------------------------------------------------
BF = torch.bfloat16


def _pin(t):
    return t.cpu().pin_memory()


class Workload:
    def release(self):
        """Drops what must not outlive the measurement (captured graphs and the tensors they own)."""
        for name in ("graph", "g_out", "host_pipe"):
            if getattr(self, name, None) is not None:
                setattr(self, name, None)


class Prefill(Workload):
    """c2: causal prefill, bf16, batch 4, seqlen 4096, 32 heads (MHA), head dim 128."""
    name, metric, unit, bound = "c2_causal_prefill_b4_s4096_h32_d128", "attn_fwd_causal_prefill_tflops", "TFLOP/s", "tensor"
    b, s, h, d = 4, 4096, 32, 128
    scale = 1e-12

    def setup(self, dev, rank, world):
        g = torch.Generator(device=dev).manual_seed(2 + 1000 * rank)
        shape = (self.b, self.s, self.h, self.d)
        self.q, self.k, self.v = [(torch.randn(shape, generator=g, device=dev) / math.sqrt(2)).to(BF) for _ in range(3)]
        self.units = 4.0 * self.b * self.h * self.s * self.s * self.d / 2  # FLOPs per step (causal convention)

    def setup_e2e(self):
        self.hq, self.hk, self.hv = _pin(self.q), _pin(self.k), _pin(self.v)
        self.ho = torch.empty(self.q.shape, dtype=BF).pin_memory()
        self.hl = torch.empty((self.b, self.h, self.s), dtype=torch.float32).pin_memory()
        self.h2d = sum(t.numel() * t.element_size() for t in (self.hq, self.hk, self.hv))
        self.d2h = self.ho.numel() * 2 + self.hl.numel() * 4

    def step(self):
        import flash_attn_npu_v2 as fa2
        return fa2.flash_attn_func(self.q, self.k, self.v, causal=True, return_attn_probs=True)

    def step_e2e(self):
        # host-buffer entry point of the package: copy in, kernel and copy out of different batch chunks overlap
        if getattr(self, "host_pipe", None) is None:
            from flash_b200.host import HostPrefill
            self.host_pipe = HostPrefill(self.q.shape, self.k.shape, BF, device=self.q.device, chunks=4)
        self.host_pipe(self.hq, self.hk, self.hv, self.ho, self.hl, after_current_stream=False, softmax_scale=self.d ** -0.5, causal=True)

    def cpu_sample(self, budget_s):
        """Oracle on (1 batch, 4 heads) slices until the time budget is used; returns (units, seconds, text)."""
        from oracle import api as OA
        g = torch.Generator().manual_seed(2)
        done, t_total, n = 0.0, 0.0, 0
        while t_total < budget_s and n < 256:
            q, k, v = [(torch.randn((1, self.s, 4, self.d), generator=g) / math.sqrt(2)).to(BF) for _ in range(3)]
            t0 = time.perf_counter()
            OA.flash_attn_func(q, k, v, causal=True)
            t_total += time.perf_counter() - t0
            done += 4.0 * 1 * 4 * self.s * self.s * self.d / 2
            n += 1
        return done, t_total, f"{n} slices of (batch 1, 4 heads, seqlen {self.s}, d {self.d}) causal, bf16"


class PrefillBackward(Prefill):
    """c2 shape, backward: dQ, dK, dV of the causal prefill from its out and lse (5 matmuls: 2.5 x the forward's FLOPs)."""
    name, metric = "c2_bwd_causal_b4_s4096_h32_d128", "attn_bwd_causal_tflops"

    def setup(self, dev, rank, world):
        Prefill.setup(self, dev, rank, world)
        import flash_attn_npu_v2 as fa2
        g = torch.Generator(device=dev).manual_seed(3 + 1000 * rank)
        self.out, self.lse, _ = fa2.flash_attn_func(self.q, self.k, self.v, causal=True, return_attn_probs=True)
        self.dout = (torch.randn(self.q.shape, generator=g, device=dev) / math.sqrt(2)).to(BF)
        self.dq, self.dk, self.dv = [torch.empty_like(self.q) for _ in range(3)]
        self.units *= 2.5

    def setup_e2e(self):
        self.host_in = [_pin(t) for t in (self.dout, self.q, self.k, self.v, self.out, self.lse)]
        self.host_out = [torch.empty(self.q.shape, dtype=BF).pin_memory() for _ in range(3)]
        self.h2d = sum(t.numel() * t.element_size() for t in self.host_in)
        self.d2h = sum(t.numel() * t.element_size() for t in self.host_out)

    def _bwd(self, dout, q, k, v, out, lse):
        from flash_b200 import ops
        return ops.attention_backward(dout, q, k, v, out, lse, dq=self.dq, dk=self.dk, dv=self.dv,
                                      softmax_scale=self.d ** -0.5, causal=True)

    def step(self):
        return self._bwd(self.dout, self.q, self.k, self.v, self.out, self.lse)

    def step_e2e(self):
        grads = self._bwd(*[t.to("cuda", non_blocking=True) for t in self.host_in])
        for h, g in zip(self.host_out, grads):
            h.copy_(g, non_blocking=True)

    def cpu_sample(self, budget_s):
        from oracle import api as OA
        from oracle import bwd as OB
        g = torch.Generator().manual_seed(3)
        done, t_total, n = 0.0, 0.0, 0
        while t_total < budget_s and n < 128:
            q, k, v, do = [(torch.randn((1, self.s, 4, self.d), generator=g) / math.sqrt(2)).to(BF) for _ in range(4)]
            _, lse = OA.flash_attn_func(q, k, v, causal=True)
            t0 = time.perf_counter()
            OB.attention_backward(q, k, v, do, lse, softmax_scale=self.d ** -0.5, causal=True)
            t_total += time.perf_counter() - t0
            done += 2.5 * 4.0 * 1 * 4 * self.s * self.s * self.d / 2
            n += 1
        return done, t_total, f"{n} slices of (batch 1, 4 heads, seqlen {self.s}, d {self.d}) causal backward, bf16"


class DecodeBase(Workload):
    metric, unit, bound = "kv_decode_hbm_gbs", "GB/s", "hbm"
    scale = 1e-9

    def setup_e2e(self):
        self.hq = _pin(self.q)
        self.ho = torch.empty(self.q.shape, dtype=BF).pin_memory()
        self.hl = torch.empty((self.q.shape[0], self.q.shape[2], self.q.shape[1]), dtype=torch.float32).pin_memory()
        self.h2d = self.hq.numel() * 2
        self.d2h = self.ho.numel() * 2 + self.hl.numel() * 4

    def step_e2e(self):
        if self.graph is not None:  # static input / output buffers of the captured call
            self.q.copy_(self.hq, non_blocking=True)
            out, lse = self.step()
        else:
            q = self.hq.to("cuda", non_blocking=True)
            out, lse = self.run(q)
        self.ho.copy_(out, non_blocking=True)
        self.hl.copy_(lse, non_blocking=True)

    # A step that is short against the host's launch work (c5 on 8 GPUs: ~0.1 ms of kernels behind five launches and
    # a collective) is replayed from a CUDA graph captured around the same public-API call.
    use_graph = False
    graph = None
    graph_launches = 0     # library launches inside one replay (counted during capture)
    replayed_launches = 0  # launches issued through replays so far
    _calls = 0

    def _capture(self):
        from flash_b200 import lib as _L
        try:
            g = torch.cuda.CUDAGraph()
            n0 = _L.load().fa_b200_launch_count()
            with torch.cuda.graph(g):
                self.g_out = self.run(self.q)
            self.graph_launches = int(_L.load().fa_b200_launch_count() - n0)
            self.graph = g
        except Exception as e:  # same code on every rank: a failure is symmetric
            print(f"[bench] CUDA graph capture failed ({e}); running eagerly", file=sys.stderr)
            self.use_graph = False

    def step(self):
        self._calls += 1
        if self.use_graph and self.graph is None and self._calls > 2:
            self._capture()
        if self.graph is not None:
            self.graph.replay()
            self.replayed_launches += self.graph_launches
            return self.g_out
        return self.run(self.q)


class DecodeContiguous(DecodeBase):
    """c3: contiguous KV-cache decode with in-place append + rotary, bf16, batch 64, GQA 32/8, d 128."""
    name = "c3_contiguous_decode_b64_h32_hk8_d128_cache8192_append_rotary"
    b, s_cache, h, hk, d = 64, 8192, 32, 8, 128

    def setup(self, dev, rank, world):
        g = torch.Generator(device=dev).manual_seed(3 + 1000 * rank)
        self.kc = torch.randn((self.b, self.s_cache, self.hk, self.d), generator=g, device=dev).to(BF)
        self.vc = torch.randn((self.b, self.s_cache, self.hk, self.d), generator=g, device=dev).to(BF)
        self.q = torch.randn((self.b, 1, self.h, self.d), generator=g, device=dev).to(BF)
        self.kn = torch.randn((self.b, 1, self.hk, self.d), generator=g, device=dev).to(BF)
        self.vn = torch.randn((self.b, 1, self.hk, self.d), generator=g, device=dev).to(BF)
        self.lens = torch.randint(1024, 8192, (self.b,), generator=g, device=dev, dtype=torch.int32)
        inv = 10000.0 ** (-torch.arange(0, 128, 2, dtype=torch.float32) / 128)
        ang = torch.arange(8192, dtype=torch.float32).view(-1, 1) * inv.view(1, -1)
        self.cos, self.sin = torch.cos(ang).to(BF).to(dev), torch.sin(ang).to(BF).to(dev)
        row = self.hk * self.d * 2 * 2
        self.units = float((self.lens.long() + 1).sum()) * row + 2 * self.b * self.h * self.d * 2 \
            + 2 * self.b * row + self.b * self.h * 4 + self.b * 4 + 2 * self.b * 64 * 2

    def setup_e2e(self):
        super().setup_e2e()
        self.hkn, self.hvn = _pin(self.kn), _pin(self.vn)
        self.h2d += self.hkn.numel() * 2 * 2

    def run(self, q, kn=None, vn=None):
        import flash_attn_npu_v2 as fa2
        return fa2.flash_attn_with_kvcache(q, self.kc, self.vc, self.kn if kn is None else kn,
                                           self.vn if vn is None else vn, rotary_cos=self.cos, rotary_sin=self.sin,
                                           cache_seqlens=self.lens, causal=True, rotary_interleaved=False,
                                           return_softmax_lse=True)

    def step_e2e(self):
        q, kn, vn = [t.to("cuda", non_blocking=True) for t in (self.hq, self.hkn, self.hvn)]
        out, lse = self.run(q, kn, vn)
        self.ho.copy_(out, non_blocking=True)
        self.hl.copy_(lse, non_blocking=True)

    def cpu_sample(self, budget_s):
        """Oracle on sequences of this configuration generated on the host (same shapes, distributions and length
        range as setup(); the device is not touched)."""
        from oracle import api as OA
        g = torch.Generator().manual_seed(3)
        inv = 10000.0 ** (-torch.arange(0, 128, 2, dtype=torch.float32) / 128)
        ang = torch.arange(8192, dtype=torch.float32).view(-1, 1) * inv.view(1, -1)
        cos, sin = torch.cos(ang).to(BF), torch.sin(ang).to(BF)
        done, t_total, n = 0.0, 0.0, 0
        while t_total < budget_s and n < self.b:
            kc = torch.randn((1, self.s_cache, self.hk, self.d), generator=g).to(BF)
            vc = torch.randn((1, self.s_cache, self.hk, self.d), generator=g).to(BF)
            q = torch.randn((1, 1, self.h, self.d), generator=g).to(BF)
            kn, vn = [torch.randn((1, 1, self.hk, self.d), generator=g).to(BF) for _ in range(2)]
            lens = torch.randint(1024, 8192, (1,), generator=g, dtype=torch.int32)
            t0 = time.perf_counter()
            OA.flash_attn_with_kvcache(q, kc, vc, kn, vn, rotary_cos=cos, rotary_sin=sin, cache_seqlens=lens,
                                       causal=True, rotary_interleaved=False)
            t_total += time.perf_counter() - t0
            done += (int(lens[0]) + 1) * self.hk * self.d * 4
            n += 1
        return done, t_total, f"{n} sequences of the configuration, one at a time (K/V bytes attended)"


class DecodePaged(DecodeBase):
    """c4: paged speculative decode, bf16, batch 32, s_q 4, GQA 64/8, d 128, page 256, window (4096, 0)."""
    name = "c4_paged_decode_b32_sq4_h64_hk8_d128_page256_window4096"
    b, s_q, h, hk, d, page, nblk = 32, 4, 64, 8, 128, 256, 4096

    def setup(self, dev, rank, world):
        g = torch.Generator(device=dev).manual_seed(4 + 1000 * rank)
        self.kp = torch.randn((self.nblk, self.page, self.hk, self.d), generator=g, device=dev).to(BF)
        self.vp = torch.randn((self.nblk, self.page, self.hk, self.d), generator=g, device=dev).to(BF)
        self.bt = torch.randperm(self.nblk, generator=g, device=dev).view(self.b, 128).to(torch.int32)
        self.lens = torch.randint(512, 32769, (self.b,), generator=g, device=dev, dtype=torch.int32)
        self.q = torch.randn((self.b, self.s_q, self.h, self.d), generator=g, device=dev).to(BF)
        n_b = torch.clamp(self.lens.long(), max=4096 + self.s_q)
        self.units = float(n_b.sum()) * self.hk * self.d * 4 + 2 * self.q.numel() * 2 + self.b * self.h * self.s_q * 4

    def run(self, q):
        import flash_attn_npu_v2 as fa2
        return fa2.flash_attn_with_kvcache(q, self.kp, self.vp, cache_seqlens=self.lens, block_table=self.bt,
                                           causal=True, window_size=(4096, 0), return_softmax_lse=True)

    def cpu_sample(self, budget_s):
        """Oracle on sequences of this configuration generated on the host: each with its own 128 pages in a
        permuted block table (the device is not touched)."""
        from oracle import api as OA
        g = torch.Generator().manual_seed(4)
        done, t_total, n = 0.0, 0.0, 0
        while t_total < budget_s and n < self.b:
            kp = torch.randn((128, self.page, self.hk, self.d), generator=g).to(BF)
            vp = torch.randn((128, self.page, self.hk, self.d), generator=g).to(BF)
            bt = torch.randperm(128, generator=g).view(1, 128).to(torch.int32)
            lens = torch.randint(512, 32769, (1,), generator=g, dtype=torch.int32)
            q = torch.randn((1, self.s_q, self.h, self.d), generator=g).to(BF)
            t0 = time.perf_counter()
            OA.flash_attn_with_kvcache(q, kp, vp, cache_seqlens=lens, block_table=bt, causal=True, window_size=(4096, 0))
            t_total += time.perf_counter() - t0
            done += min(int(lens[0]), 4096 + self.s_q) * self.hk * self.d * 4
            n += 1
        return done, t_total, f"{n} sequences of the configuration, one at a time (in-window K/V bytes; the golden reads whole sequences)"


class DecodeLongSharded(DecodeBase):
    """c5: long-context decode, bf16, batch 8, s_q 1, GQA 64/8, d 128, 131072 keys per sequence split
    evenly over the ranks; partial (O, LSE) all-gathered and merged on every rank."""
    name = "c5_long_decode_b8_h64_hk8_d128_L131072_seqsharded"
    b, L, h, hk, d = 8, 131072, 64, 8, 128
    strong = True
    use_graph = True

    exchange = "peer"  # "peer": partials over peer memory (flash_b200.dist.PeerExchange); "nccl": all-gather + merge
    px = None

    def setup(self, dev, rank, world):
        from flash_b200 import dist as D
        self.world = world
        if world > 1 and self.exchange == "peer":
            try:
                self.px = D.PeerExchange(self.b * self.h, self.d, dev)
            except Exception as e:  # every rank fails alike (the handles travel through a collective)
                print(f"[bench] peer exchange unavailable ({e}); using the NCCL all-gather", file=sys.stderr)
                self.px = None
        self.lo, self.hi = D.kv_shard_range(self.L, world, rank)
        g = torch.Generator(device=dev).manual_seed(5)
        self.q = torch.randn((self.b, 1, self.h, self.d), generator=g, device=dev).to(BF)
        g2 = torch.Generator(device=dev).manual_seed(50 + rank)
        n = self.hi - self.lo
        self.kc = torch.randn((self.b, n, self.hk, self.d), generator=g2, device=dev).to(BF)
        self.vc = torch.randn((self.b, n, self.hk, self.d), generator=g2, device=dev).to(BF)
        self.units = float(self.b) * n * self.hk * self.d * 4 + 264192

    def run(self, q):
        from flash_b200 import dist as D
        return D.sharded_decode(q, self.kc, self.vc, kv_pos_offset=self.lo, kv_total=self.L, causal=True, exchange=self.px)

    def local_only_ms(self, steps=50):
        """This rank's share of a step without the exchange (attention over its shard + merge of its own splits):
        what the cross-GPU step time is made of besides waiting for the slowest rank."""
        from flash_b200 import ops
        run = lambda: ops.attention_forward(self.q, self.kc, self.vc, softmax_scale=self.d ** -0.5, causal=True,
                                            kv_pos_offset=self.lo, kv_total=self.L, partial_out=True)
        for _ in range(10):
            run()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            run()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    def release(self):
        super().release()
        if self.px is not None:
            import torch.distributed as dist
            torch.cuda.synchronize()
            dist.barrier()  # every rank has finished its last merge before anybody unmaps
            self.px.close()
            self.px = None

    def cpu_sample(self, budget_s):
        """Oracle on the first 16384 keys of one sequence of this configuration, generated on the host."""
        from oracle import api as OA
        n_tok = 16384
        g = torch.Generator().manual_seed(5)
        kc = torch.randn((1, n_tok, self.hk, self.d), generator=g).to(BF)
        vc = torch.randn((1, n_tok, self.hk, self.d), generator=g).to(BF)
        q = torch.randn((1, 1, self.h, self.d), generator=g).to(BF)
        done, t_total, n = 0.0, 0.0, 0
        while t_total < budget_s and n < 8:
            t0 = time.perf_counter()
            OA.flash_attn_with_kvcache(q, kc, vc, cache_seqlens=n_tok, causal=True)
            t_total += time.perf_counter() - t0
            done += n_tok * self.hk * self.d * 4
            n += 1
        return done, t_total, f"{n} passes over {n_tok} keys of one sequence"


WORKLOADS = {"c2": Prefill, "c2_bwd": PrefillBackward, "c3": DecodeContiguous, "c4": DecodePaged, "c5": DecodeLongSharded}


# ------------------------------------------------------------------------------------------------
# driver
# ------------------------------------------------------------------------------------------------
HEADLINE = "c2"
DECODE_HALF = ("c3", "c4", "c5", "c2_bwd")  # entries of the default line's "workloads" object: the decode half of the metric, and the backward at the headline shape
DEFAULT_STEPS = {"c2": (20, 5), "c2_bwd": (10, 3)}  # (steps, warm-up); decode steps are 0.1-0.6 ms, so they run (200, 50)


def _cpu_entry(wl, budget, repeats=1, warm=False):
    """The CPU oracle (a port of the reference's PyTorch golden) on all host cores, on a bounded sample."""
    torch.set_num_threads(os.cpu_count() or 1)
    if warm:
        wl.cpu_sample(min(0.5, budget))
    done, secs, sample = 0.0, 0.0, ""
    for _ in range(repeats):
        d, t, sample = wl.cpu_sample(budget)
        done += d
        secs += t
    val = done / secs * wl.scale
    return {"value": val, "unit": wl.unit, "cores": torch.get_num_threads(), "kind": "port",
            "sample": sample + (f", x{repeats} steps" if repeats > 1 else ""), "seconds": secs}


def run_reference(args, rank, world):
    """--impl reference: the reference's CPU implementation of the path (its PyTorch golden, here the
    oracle port -- the reference's native code needs the Ascend toolchain) on the host cores, on the same
    workloads as the default arm: the prefill configuration as the headline, the decode configurations under
    "workloads".  Every step is a bounded sample of its workload; nothing here touches a GPU."""
    if rank != 0:
        return
    keys = [args.workload] if args.workload else [HEADLINE] + list(DECODE_HALF)
    entries = {}
    for key in keys:
        wl = WORKLOADS[key]()
        budget = 2.0 if key == keys[0] else max(1.0, 8.0 / max(args.steps, 1))
        cb = _cpu_entry(wl, budget, repeats=args.steps, warm=args.warmup > 0)
        entries[key] = {"impl": "reference", "metric": wl.metric, "value": cb["value"], "unit": wl.unit,
                        "steps": args.steps, "warmup": args.warmup, "ms_per_step": cb["seconds"] / args.steps * 1e3,
                        "config": {"workload": wl.name}, "cpu_baseline": cb,
                        "e2e": {"value": cb["value"], "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                        "gpu_launches": 0}
    first = entries[keys[0]]
    line = dict(first)
    line.update({"n_gpus": args.gpus, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
                 "data": "synthetic"})
    line["config"] = {"workload": first["config"]["workload"],
                      "note": "CPU golden (oracle port) on host cores; each step a bounded sample"}
    if len(keys) > 1:
        line["workloads"] = {k: entries[k] for k in keys[1:]}
    print(json.dumps(line))


def measure(key, args, steps, warmup, dev, rank, world, local_rank, peaks, barrier, cpu_budget):
    """Sets one workload up, times it (device-resident and end to end) and returns its result object (rank 0)
    or None (other ranks).  Every rank runs the same sequence of steps: c5 has a collective in each."""
    import torch.distributed as dist
    from flash_b200 import lib as _L
    wl = WORKLOADS[key]()
    if key == "c5":
        wl.exchange = args.c5_exchange
    if args.shrink > 1:
        if key == "c5":
            wl.L //= args.shrink
        else:
            wl.b = max(1, wl.b // args.shrink)
        if key == "c4":
            wl.nblk = wl.b * 128
        wl.name += f"_shrunk{args.shrink}"
    wl.setup(dev, rank, world)

    # ---- device-resident timing ----
    for _ in range(warmup):
        wl.step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    stream = torch.cuda.current_stream()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    barrier()
    # one more untimed step, so that the first timed one does not start on a GPU the barrier has just left idle (with
    # few timed steps a single slow first step on one rank is what the max over ranks reports)
    wl.step()
    launches0 = _L.load().fa_b200_launch_count() + getattr(wl, "replayed_launches", 0)
    ev[0].record(stream)
    for i in range(steps):
        wl.step()
        ev[i + 1].record(stream)
    # counted by the library (eager calls) or during the capture of the replayed graph, not assumed
    gpu_launches = int(_L.load().fa_b200_launch_count() + getattr(wl, "replayed_launches", 0) - launches0)
    barrier()
    total_ms = ev[0].elapsed_time(ev[-1])
    per = sorted(ev[i].elapsed_time(ev[i + 1]) for i in range(steps))
    # Keep the GPU busy a little longer so the clock sampler sees load even for short runs.  The
    # number of extra steps is derived from the rank-reduced time, so every rank runs the same count
    # (a workload with a collective would deadlock otherwise).
    t0 = torch.tensor([total_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t0, op=dist.ReduceOp.MAX)
    n_extra = int(min(2000, 600.0 / max(float(t0[0]) / steps, 1e-3))) if steps > 2 else 0
    for _ in range(n_extra):
        wl.step()
    barrier()
    clocks = sampler.stop() if rank == 0 else None

    # ---- end-to-end timing (host buffers) ----
    e2e_ms = float("nan")
    wl.h2d = wl.d2h = 0
    if not args.no_e2e:
        wl.setup_e2e()
        for _ in range(3):
            wl.step_e2e()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            wl.step_e2e()
        e1.record(stream)
        barrier()
        e2e_ms = e0.elapsed_time(e1)

    t = torch.tensor([total_ms, e2e_ms, wl.units], dtype=torch.float64, device=dev)
    if world > 1:
        tmax = t.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        tsum = t.clone()
        dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
        total_ms, e2e_ms, units_all = float(tmax[0]), float(tmax[1]), float(tsum[2])
    else:
        units_all = wl.units
    used_graph = getattr(wl, "graph", None) is not None
    local_ms = None
    if key == "c5" and world > 1:  # every rank's own work per step, gathered: the slowest one paces the lock-step
        mine = torch.tensor([wl.local_only_ms()], dtype=torch.float64, device=dev)
        every = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(every, mine)
        local_ms = sorted(float(x[0]) for x in every)
    entry = None
    if rank == 0:
        value = units_all * steps / (total_ms * 1e-3) * wl.scale
        e2e = units_all * steps / (e2e_ms * 1e-3) * wl.scale
        achieved = wl.units / (total_ms / steps * 1e-3) * wl.scale
        if wl.bound == "tensor":
            peak = peaks["bf16_tflops"] if total_ms < 1000 else peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])
            runit = "TFLOP/s"
        else:
            peak, runit = peaks["hbm_gbs"], "GB/s"
        traffic, traffic_src = None, None
        if key in NCU_TRAFFIC:
            t_bytes, t_units, traffic_src = NCU_TRAFFIC[key]
            traffic = t_bytes * wl.units / t_units
        entry = {
            "metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": total_ms / steps, "higher_is_better": True,
            "scaling": "strong" if getattr(wl, "strong", False) else "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": wl.name, "l2": "inputs larger than L2 (no flush needed)" if not key.startswith("c2")
                       else "q+k+v+o = 537 MB per step, larger than the 126 MB L2", "median_ms_per_step": per[len(per) // 2],
                       "per_gpu_units": wl.units, "cuda_graph": used_graph},
            "roofline": {"bound": wl.bound, "achieved": achieved, "peak": peak, "unit": runit,
                         "frac": achieved / peak, "traffic": traffic, "traffic_unit": "bytes per launch",
                         "traffic_source": traffic_src, "peak_source": peaks["_source"],
                         "per_launch": "one attention launch per step" + (" (+ merge)" if gpu_launches > steps else "")},
            "e2e": {"value": e2e, "unit": wl.unit, "h2d_bytes_per_step": wl.h2d, "d2h_bytes_per_step": wl.d2h,
                    # what the slowest rank's host link delivered: at N > 1 all ranks pull from one host's pinned memory
                    "h2d_gb_per_s_per_gpu": wl.h2d * steps / (e2e_ms * 1e-3) / 1e9, "ms_per_step": e2e_ms / steps},
            "gpu_launches": gpu_launches,
            "clocks": clocks,
        }
        if local_ms is not None:
            entry["config"]["local_ms_per_step_min_median_max"] = [local_ms[0], local_ms[len(local_ms) // 2], local_ms[-1]]
        if key == "c5":
            entry["config"]["exchange"] = ("peer memory (NVLink stores + flags)" if getattr(wl, "px", None) is not None
                                           else ("NCCL all-gather" if world > 1 else "none (one rank)"))
        if wl.bound == "hbm":  # the north star quotes the decode target against the nominal 8 TB/s too
            entry["roofline"]["frac_of_nominal_8tbs"] = achieved / 8000.0
        if not args.no_cpu_baseline and world == 1:
            entry["cpu_baseline"] = _cpu_entry(wl, cpu_budget)
    # A captured graph holds NCCL kernels, and the communicator cannot be torn down while such a graph is alive:
    # release it (and the tensors captured with it) here, with the stream idle.
    wl.release()
    del wl
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    return entry


def bind_to_gpu_numa_node(local_rank):
    """Multi-process runs: keep this process (and so the pinned host buffers it allocates, first touch) on the CPUs of
    the NUMA node its GPU hangs off, as a deployment would.  Without it all ranks' host buffers tend to land on one
    node and the end-to-end copies of all GPUs cross the same socket link.  Returns a short description, or None when
    the topology cannot be read (then nothing is changed)."""
    try:
        pr = torch.cuda.get_device_properties(local_rank)
        bdf = f"{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
        base = f"/sys/bus/pci/devices/{bdf}"
        node = int(open(base + "/numa_node").read().strip())
        cpus = set()
        for part in open(base + "/local_cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= os.sched_getaffinity(0)
        if node < 0 or not cpus:
            return None
        os.sched_setaffinity(0, cpus)
        return f"numa node {node}, {len(cpus)} cpus"
    except Exception:  # no sysfs, no permission, an unknown layout: run unbound
        return None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None, help="default: 20 (c2), 10 (c2_bwd), 200 (decode workloads)")
    ap.add_argument("--warmup", type=int, default=None, help="default: 5 (c2), 3 (c2_bwd), 50 (decode workloads)")
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS),
                    help="one workload only; default: c2 as the headline plus c3, c4, c5, c2_bwd under \"workloads\"")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-budget", type=float, default=12.0)
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--c5-exchange", default="peer", choices=["peer", "nccl"],
                    help="how the sequence shards of c5 are merged across GPUs")
    ap.add_argument("--shrink", type=int, default=1,
                    help="divide the batch (c2-c4) or the key length (c5) by this factor: small cases for ncu captures")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    head_key = args.workload or HEADLINE
    if args.impl == "reference":
        d_steps, d_warm = DEFAULT_STEPS.get(head_key, (20, 5))
        args.steps = min(d_steps, 20) if args.steps is None else args.steps
        args.warmup = d_warm if args.warmup is None else args.warmup
        run_reference(args, rank, world)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU implementation of the product path)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    import torch.distributed as dist
    host_binding = None
    if world > 1:
        host_binding = bind_to_gpu_numa_node(local_rank)  # (a single process keeps all cores: it also times the CPU baseline)
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    peaks = load_peaks()

    def counts(key, is_head):
        d_steps, d_warm = DEFAULT_STEPS.get(key, (200, 50))
        # --steps / --warmup are the headline's; a decode step is so short that fewer than its default count would
        # end before the clocks have risen, so the entries under "workloads" keep their own counts
        steps = args.steps if (is_head and args.steps is not None) else d_steps
        warm = args.warmup if (is_head and args.warmup is not None) else d_warm
        return steps, max(warm, 3)

    steps, warm = counts(head_key, True)
    line = measure(head_key, args, steps, warm, dev, rank, world, local_rank, peaks, barrier, args.cpu_budget)
    if args.workload is None:
        extra = {}
        for key in DECODE_HALF:
            steps, warm = counts(key, False)
            extra[key] = measure(key, args, steps, warm, dev, rank, world, local_rank, peaks, barrier,
                                 min(args.cpu_budget, 4.0))
        if rank == 0:
            line["workloads"] = extra
    if rank == 0:
        if world > 1:
            line["config"]["host_binding"] = host_binding or "none (topology not readable)"
        print(json.dumps(line))
        sys.stdout.flush()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
        # Every captured graph was released in measure(); should the teardown still not return (it once sat in
        # destroy_process_group until killed, with a graph of NCCL kernels alive), leave after a grace period:
        # everything is done, printed and synchronised.
        threading.Timer(30.0, lambda: os._exit(0)).start()
        dist.destroy_process_group()
        os._exit(0)


if __name__ == "__main__":
    main()
