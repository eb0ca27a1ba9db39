"""Row-wise ops on HOST tensors: chunks are copied in, processed and copied out in a pipeline.

The ops in popcorn_b200.ops take CUDA tensors.  When the data lives in host
memory, the PCIe link is the bottleneck, not the kernel; what matters then is
that the host-to-device copy of chunk i+1, the kernel of chunk i and the
device-to-host copy of chunk i-1 run at the same time (the link is full duplex).
`run_rows` does exactly that with three CUDA streams and a ring of device
buffers.  The arithmetic is the same sm_100a kernel as for device tensors.

popcorn itself has no host-tensor path: its harness moves inputs to the device
before a call (src/popcorn/bench/grid.py:707-711).
"""

from __future__ import annotations

from collections.abc import Callable, Sequence

import torch
from torch import Tensor

from popcorn_b200 import ops


def chunk_bounds(rows: int, chunk_rows: int) -> list[tuple[int, int]]:
    """[lo, hi) row ranges of the pipeline's chunks.  The first copy in and the last copy out have nothing to overlap
    with, so the chunks ramp up from chunk_rows / 8 at the start and back down at the end (each ramp costs four
    extra launches and shortens the exposed copy eightfold); short inputs are cut evenly."""
    if rows <= 0:
        return []
    ramp = [chunk_rows // 8, chunk_rows // 4, chunk_rows // 2] if chunk_rows >= 8 else []
    if rows < 4 * chunk_rows or not ramp:
        return [(lo, min(lo + chunk_rows, rows)) for lo in range(0, rows, chunk_rows)]
    sizes = list(ramp)
    middle = rows - 2 * sum(ramp)
    sizes += [chunk_rows] * (middle // chunk_rows)
    if middle % chunk_rows:
        sizes.append(middle % chunk_rows)
    sizes += ramp[::-1]
    bounds, lo = [], 0
    for size in sizes:
        bounds.append((lo, lo + size))
        lo += size
    return bounds


def run_rows(
    fn: Callable[..., Tensor | Sequence[Tensor]],
    inputs: Sequence[Tensor],
    outputs: Sequence[Tensor],
    device: torch.device | str = "cuda",
    chunk_rows: int = 1024,
    depth: int = 3,
) -> None:
    """outputs[j][rows] = fn(*[inp[rows] on the device for inp in inputs])[j], chunk by chunk.

    inputs / outputs: host tensors whose first dimension is the row dimension (pinned memory makes the
    copies asynchronous).  fn receives device chunks and returns one device tensor or a sequence of them.
    The call returns when every output chunk has landed in host memory."""
    device = torch.device(device)
    if not inputs or not outputs:
        raise ValueError("run_rows needs at least one input and one output")
    rows = inputs[0].shape[0]
    if any(t.shape[0] != rows for t in (*inputs, *outputs)):
        raise ValueError("all inputs and outputs must have the same number of rows")
    if rows == 0:
        return
    chunk_rows = max(1, min(chunk_rows, rows))
    bounds = chunk_bounds(rows, chunk_rows)
    with torch.cuda.device(device):
        copy_in, compute, copy_out = (torch.cuda.Stream(device) for _ in range(3))
        ring = [[torch.empty((chunk_rows, *t.shape[1:]), dtype=t.dtype, device=device) for t in inputs] for _ in range(depth)]
        drained = [None] * depth  # event: the kernel that last read ring[i] has finished
        start = torch.cuda.current_stream(device).record_event()
        copy_in.wait_event(start)
        last_out = None
        for index, (lo, hi) in enumerate(bounds):
            slot = ring[index % depth]
            with torch.cuda.stream(copy_in):
                if drained[index % depth] is not None:
                    copy_in.wait_event(drained[index % depth])
                for dst, src in zip(slot, inputs):
                    dst[: hi - lo].copy_(src[lo:hi], non_blocking=True)
                arrived = copy_in.record_event()
            with torch.cuda.stream(compute):
                compute.wait_event(arrived)
                result = fn(*[buf[: hi - lo] for buf in slot])
                result = (result,) if isinstance(result, Tensor) else tuple(result)
                done = compute.record_event()
                drained[index % depth] = done
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(done)
                for dst, src in zip(outputs, result):
                    dst[lo:hi].copy_(src, non_blocking=True)
                    src.record_stream(copy_out)  # allocated on `compute`, read on `copy_out`
                last_out = copy_out.record_event()
        torch.cuda.current_stream(device).wait_event(last_out)
        last_out.synchronize()


def add_rms_norm_host(
    x: Tensor, residual: Tensor, weight: Tensor, eps: float = 1e-6, offset: float = 0.0,
    *, y: Tensor | None = None, s: Tensor | None = None, device: torch.device | str = "cuda", chunk_rows: int = 1024,
) -> tuple[Tensor, Tensor]:
    """add_rms_norm over host tensors x, residual [rows, hidden]; returns host tensors (y, s).

    `weight` may live on either side.  Pass pinned `y` / `s` to reuse output buffers."""
    device = torch.device(device)
    if x.dim() != 2 or residual.shape != x.shape:
        raise ValueError("add_rms_norm_host: x and residual must be [rows, hidden] tensors of the same shape")
    pin = torch.cuda.is_available()
    y = torch.empty(x.shape, dtype=x.dtype, pin_memory=pin) if y is None else y
    s = torch.empty(x.shape, dtype=x.dtype, pin_memory=pin) if s is None else s
    weight_dev = weight.to(device)
    run_rows(lambda xc, rc: ops.add_rms_norm(xc, rc, weight_dev, eps, offset), [x, residual], [y, s], device, chunk_rows)
    return y, s
