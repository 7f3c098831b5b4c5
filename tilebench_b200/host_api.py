"""Host-buffer entry points: operators whose inputs and outputs live in (pinned) host memory.

The operator contract of the reference hands `run()` device tensors.  A caller whose weights sit in host
memory pays two PCIe transfers around the kernel; done back to back they add up (H2D, then the kernel, then
D2H).  PCIe is full duplex and the kernel is orders of magnitude faster than either copy, so the work is cut
into row chunks and pipelined over three streams — upload of chunk i+1, kernel of chunk i and download of
chunk i-1 overlap — which brings the end-to-end time down from H2D + D2H to about max(H2D, D2H).

Device staging buffers are allocated once per (shape, dtype, device) and reused; host tensors must be pinned
for the copies to be asynchronous (unpinned tensors still work, serialised by the runtime).
"""
from __future__ import annotations

import torch

from tilebench_b200 import native

_pipelines: dict = {}


class _Int8ChannelPipeline:
    def __init__(self, rows: int, cols: int, out_dtype: torch.dtype, device: torch.device, chunk_rows: int, depth: int):
        self.rows, self.cols, self.chunk_rows, self.depth = rows, cols, chunk_rows, depth
        self.w = [torch.empty((chunk_rows, cols), dtype=torch.int8, device=device) for _ in range(depth)]
        self.out = [torch.empty((chunk_rows, cols), dtype=out_dtype, device=device) for _ in range(depth)]
        self.scale = torch.empty(rows, dtype=torch.float32, device=device)
        self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(device=device) for _ in range(3))
        self.uploaded = [torch.cuda.Event() for _ in range(depth)]
        self.computed = [torch.cuda.Event() for _ in range(depth)]
        self.drained = [torch.cuda.Event() for _ in range(depth)]

    def run(self, ext, hw: torch.Tensor, hs: torch.Tensor, hout: torch.Tensor) -> None:
        cur = torch.cuda.current_stream(self.scale.device)
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_stream(cur)
        with torch.cuda.stream(self.s_in):
            self.scale.copy_(hs, non_blocking=True)
        n_chunks = -(-self.rows // self.chunk_rows)
        for i in range(n_chunks):
            slot = i % self.depth
            r0, r1 = i * self.chunk_rows, min(self.rows, (i + 1) * self.chunk_rows)
            n = r1 - r0
            with torch.cuda.stream(self.s_in):
                if i >= self.depth:
                    self.s_in.wait_event(self.computed[slot])       # the kernel has read the previous contents of this slot
                self.w[slot][:n].copy_(hw[r0:r1], non_blocking=True)
                self.uploaded[slot].record(self.s_in)
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(self.uploaded[slot])
                if i >= self.depth:
                    self.s_run.wait_event(self.drained[slot])       # the previous result of this slot has left the device
                ext.dequant_int8_rowwise(self.w[slot][:n], self.scale[r0:r1], self.out[slot][:n], False, 1.0)
                self.computed[slot].record(self.s_run)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.computed[slot])
                hout[r0:r1].copy_(self.out[slot][:n], non_blocking=True)
                self.drained[slot].record(self.s_out)
        cur.wait_stream(self.s_out)
        cur.wait_stream(self.s_run)
        cur.wait_stream(self.s_in)


def dequant_int8_channel_host(w: torch.Tensor, scale: torch.Tensor, out: torch.Tensor | None = None, *,
                              device: torch.device | str | None = None, chunk_rows: int = 4096, depth: int = 3) -> torch.Tensor:
    """out[r, c] = bf16(float(w[r, c]) * scale[r]) for HOST tensors w (int8 [rows, cols]) and scale (fp32 [rows]).

    The result is written to `out` (host, bf16 or fp16; allocated pinned if None) asynchronously with respect to
    the host: synchronise the current stream of `device` before reading it.  Same arithmetic and the same kernel
    as the device-tensor operator `dequant_int8_channel`."""
    ext = native.load()
    if w.is_cuda or scale.is_cuda:
        raise ValueError("dequant_int8_channel_host takes host tensors; call the operator's run() for device tensors")
    if w.dtype != torch.int8 or scale.dtype != torch.float32 or w.dim() != 2 or scale.shape != (w.shape[0],):
        raise ValueError("w must be int8 [rows, cols] and scale fp32 [rows]")
    dev = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
    rows, cols = w.shape
    if out is None:
        out = torch.empty((rows, cols), dtype=torch.bfloat16).pin_memory()
    if out.is_cuda or out.shape != w.shape or out.dtype not in (torch.bfloat16, torch.float16):
        raise ValueError("out must be a host bf16 / fp16 tensor of w's shape")
    chunk_rows = max(1, min(int(chunk_rows), rows))
    key = (rows, cols, out.dtype, dev, chunk_rows, depth)
    pipe = _pipelines.get(key)
    if pipe is None:
        _pipelines.clear()                                  # one staging set at a time: the buffers are large
        pipe = _pipelines[key] = _Int8ChannelPipeline(rows, cols, out.dtype, dev, chunk_rows, depth)
    pipe.run(ext, w, scale, out)
    return out
