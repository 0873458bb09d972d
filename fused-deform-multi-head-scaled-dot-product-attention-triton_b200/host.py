"""Host-buffer front end: the operator for callers whose tensors live in (pinned) host memory.

The reference keeps everything on the device, and so does ``deform_sdpa_triton``.  A caller
that starts from host tensors pays a host->device copy of q, k, v, coords (and dout) and a
device->host copy of the results around the kernels.  Batch elements are independent
(reference ops/triton.py:47-51), so this front end cuts the batch into chunks and runs
three streams -- copy in, compute, copy out -- so that the PCIe traffic of one chunk hides
behind the kernels of another.  Results are identical to the one-shot call: the chunks
are whole batch elements.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .op import backward_raw, forward_raw


class HostPipeline:
    """Forward (+ backward) of the operator on pinned host tensors, chunked over the batch."""

    def __init__(self, device, W: int, H: int, sm_scale: float, chunk: int = 4, flags: Optional[int] = None):
        self.device = torch.device(device)
        self.W, self.H, self.sm_scale = int(W), int(H), float(sm_scale)
        self.chunk = max(1, int(chunk))
        self.flags = flags
        self.s_in = torch.cuda.Stream(self.device)
        self.s_comp = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)

    def _to_device(self, hosts: Sequence[Optional[torch.Tensor]], b0: int, b1: int):
        out = []
        for t in hosts:
            if t is None:
                out.append(None)
                continue
            d = t[b0:b1].to(self.device, non_blocking=True)
            d.record_stream(self.s_comp)
            out.append(d)
        return out

    def run(self, q, k, v, coords, dout=None, *, out, dq=None, dk=None, dv=None):
        """All arguments are host tensors (pinned for the copies to be asynchronous) with the
        operator's layouts; ``out`` (and ``dq, dk, dv`` when ``dout`` is given) receive the
        results.  Asynchronous with respect to the host; ordered after and before the work on
        the current stream of the device, like a kernel launch."""
        if q.is_cuda or out.is_cuda:
            raise ValueError("HostPipeline takes host tensors; use deform_sdpa_triton for device tensors")
        backward = dout is not None
        if backward and (dq is None or dk is None or dv is None):
            raise ValueError("dq, dk, dv host tensors are needed when dout is given")
        B = q.shape[0]
        cur = torch.cuda.current_stream(self.device)
        start = torch.cuda.Event()
        start.record(cur)
        for s in (self.s_in, self.s_comp, self.s_out):
            s.wait_event(start)
        for b0 in range(0, B, self.chunk):
            b1 = min(B, b0 + self.chunk)
            with torch.cuda.stream(self.s_in):
                dq_in, dk_in, dv_in, dc_in, ddo_in = self._to_device((q, k, v, coords, dout), b0, b1)
                ready = torch.cuda.Event()
                ready.record(self.s_in)
            self.s_comp.wait_event(ready)
            with torch.cuda.stream(self.s_comp):
                o, lse = forward_raw(dq_in, dk_in, dv_in, dc_in, self.W, self.H, self.sm_scale, flags=self.flags)
                results = [(out, o)]
                if backward:
                    gq, gk, gv, _ = backward_raw(dq_in, dk_in, dv_in, dc_in, o, lse, ddo_in, self.W, self.H,
                                                 self.sm_scale, flags=self.flags)
                    results += [(dq, gq), (dk, gk), (dv, gv)]
                done = torch.cuda.Event()
                done.record(self.s_comp)
            self.s_out.wait_event(done)
            with torch.cuda.stream(self.s_out):
                for host, dev_t in results:
                    dev_t.record_stream(self.s_out)
                    host[b0:b1].copy_(dev_t, non_blocking=True)
        end = torch.cuda.Event()
        end.record(self.s_out)
        cur.wait_event(end)
        return out
