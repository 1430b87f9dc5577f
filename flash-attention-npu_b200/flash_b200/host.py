"""Attention forward for callers whose tensors live in (pinned) host memory.

The reference's operators take device tensors; a host that feeds them from CPU memory pays
host->device copy, kernel and device->host copy one after the other.  ``HostPrefill`` cuts the
batch into chunks and runs the three phases of different chunks at the same time on three CUDA
streams (PCIe is full duplex and the copy engines are independent of the SMs), so a step costs
about its host->device copy alone.  The results are bit-identical to one call on the whole batch:
every (batch entry, head, query tile) is computed by the same code either way.

PyTorch is plumbing here (pinned memory, streams, events); the compute is ``ops.attention_forward``.
"""
import torch

from . import ops


class HostPrefill:
    """Device staging buffers, streams and events for one problem shape (allocate once, call per step).

    q (b, s_q, h, d), k / v (b, s_k, h_k, d), out like q, lse (b, h, s_q) fp32 -- all host tensors,
    pinned for the copies to be asynchronous.
    """

    def __init__(self, q_shape, k_shape, dtype, device=None, chunks=4):
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("flash_b200 runs on CUDA devices only (there is no CPU implementation)")
        b, s_q, h, d = q_shape
        if tuple(k_shape[:1]) != (b,) or k_shape[3] != d:
            raise RuntimeError("q and k must agree in batch size and head dim")
        self.n_chunks = max(1, min(int(chunks), b))
        self.bounds = [(b * i // self.n_chunks, b * (i + 1) // self.n_chunks) for i in range(self.n_chunks)]
        dev = self.device
        self.q = torch.empty(q_shape, dtype=dtype, device=dev)
        self.k = torch.empty(k_shape, dtype=dtype, device=dev)
        self.v = torch.empty(k_shape, dtype=dtype, device=dev)
        self.out = torch.empty(q_shape, dtype=dtype, device=dev)
        self.lse = torch.empty((b, h, s_q), dtype=torch.float32, device=dev)
        self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(dev) for _ in range(3))
        self.ev_in = [torch.cuda.Event() for _ in self.bounds]
        self.ev_run = [torch.cuda.Event() for _ in self.bounds]
        self.ev_out = [torch.cuda.Event() for _ in self.bounds]
        self.used = False

    def __call__(self, q, k, v, out, lse, after_current_stream=True, **kw):
        """Copies q, k, v in, runs the forward (keyword arguments of ``ops.attention_forward``) and
        copies O and LSE into ``out`` / ``lse``, chunk by chunk.  The current stream waits for the
        last copy out, so a synchronize (or an event) on it covers the whole step.

        ``after_current_stream`` (default) orders the step after the work already queued on the
        current stream, which includes the previous step's copies out.  A caller that streams
        independent steps passes False: the copies in of the next step then run under the copies
        out of this one (the staging buffers are still protected chunk by chunk), and it is the
        caller's business to have consumed ``out`` / ``lse`` before they are written again."""
        for name, t, ref in (("q", q, self.q), ("k", k, self.k), ("v", v, self.v), ("out", out, self.out), ("lse", lse, self.lse)):
            if t.is_cuda or t.shape != ref.shape or t.dtype != ref.dtype:
                raise RuntimeError(f"{name} must be a host tensor of shape {tuple(ref.shape)} and dtype {ref.dtype}")
        cur = torch.cuda.current_stream(self.device)
        if after_current_stream:
            self.s_in.wait_stream(cur)
            self.s_run.wait_stream(cur)
            self.s_out.wait_stream(cur)
        for i, (lo, hi) in enumerate(self.bounds):
            if self.used:  # staging buffers of this chunk: the previous step's kernel has read q, k, v; its copy out has read O
                self.s_in.wait_event(self.ev_run[i])
                self.s_run.wait_event(self.ev_out[i])
            with torch.cuda.stream(self.s_in):
                self.q[lo:hi].copy_(q[lo:hi], non_blocking=True)
                self.k[lo:hi].copy_(k[lo:hi], non_blocking=True)
                self.v[lo:hi].copy_(v[lo:hi], non_blocking=True)
                self.ev_in[i].record(self.s_in)
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(self.ev_in[i])
                ops.attention_forward(self.q[lo:hi], self.k[lo:hi], self.v[lo:hi], out=self.out[lo:hi], lse=self.lse[lo:hi], **kw)
                self.ev_run[i].record(self.s_run)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.ev_run[i])
                out[lo:hi].copy_(self.out[lo:hi], non_blocking=True)
                lse[lo:hi].copy_(self.lse[lo:hi], non_blocking=True)
                self.ev_out[i].record(self.s_out)
        self.used = True
        cur.wait_stream(self.s_out)
        return out, lse
