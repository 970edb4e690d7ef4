"""Communication helpers around torch.distributed: side-stream collectives, NCCL communicator sizing,
gloo-free gather / scatter of large host objects, and the one-step-delayed logging all-reduce.

  async_all_gather / async_reduce_scatter / async_all_to_all
        run the collective on one lazily created communication stream after an optional event (or stream) wait and
        return ``(input, output, handle)``; ``handle.wait()`` makes the *current* stream wait for the result, so the
        caller decides where the dependency lands (reference: mindspeed/core/transformer/moe/comm_utils.py:8-138).
  NcclOptions / parse_buffer_spec / auto_buffer_sizes
        per-group communicator options: the user string ``"dp:200;tp:64"`` (MB) or sizes derived from the model
        shape; on NCCL the knobs are the per-communicator buffer size and CTA budget passed through
        ``ProcessGroupNCCL.Options.config`` (reference: mindspeed/core/hccl_buffer/adaptor.py:16-57 sizes HCCL buffers).
  gather_to_rank0_sliced / scatter_from_rank0_sliced
        optimizer-state movement without a gloo group: bounded device slices through device collectives
        (reference: mindspeed/core/megatron_basic/utils.py:608-685, --hccl-slice-size).
  AsyncLogAllReduce
        loss averaging issued asynchronously and consumed at the next step, so logging never stalls the step that
        produced the value (reference: mindspeed/core/data_parallel/async_log_allreduce.py:1-183).
"""
from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from . import mappings as M

_COMM_STREAM: Optional["torch.cuda.Stream"] = None


def get_comm_stream():
    """The process-wide communication side stream (None on CPU)."""
    global _COMM_STREAM
    if not torch.cuda.is_available():
        return None
    if _COMM_STREAM is None:
        _COMM_STREAM = torch.cuda.Stream()
    return _COMM_STREAM


class _Handle:
    """Completion handle: ``wait()`` orders the current stream after the side-stream collective."""

    def __init__(self, work, event):
        self.work, self.event = work, event

    def wait(self):
        if self.work is not None:
            self.work.wait()
        if self.event is not None:
            torch.cuda.current_stream().wait_event(self.event)

    def is_completed(self):
        return (self.work is None or self.work.is_completed()) and (self.event is None or self.event.query())


def _on_comm_stream(fn, tensor, event=None, stream=None):
    """Run ``fn()`` (which issues a collective, possibly async) on the comm stream after `event` / `stream`."""
    cs = get_comm_stream() if tensor.is_cuda else None
    if cs is None:
        out, work = fn()
        return out, _Handle(work, None)
    if event is not None:
        cs.wait_event(event)
    elif stream is not None:
        cs.wait_stream(stream)
    else:
        cs.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(cs):
        out, work = fn()
        if work is not None:
            work.wait()            # orders the comm stream, not the host
        done = torch.cuda.Event()
        done.record(cs)
    tensor.record_stream(cs)
    if isinstance(out, torch.Tensor):
        out.record_stream(torch.cuda.current_stream())
    return out, _Handle(None, done)


def async_all_gather(x: torch.Tensor, group, event=None, is_use_get_global_memory_buffer=False, last_dim=False, stream=None):
    if last_dim:
        def fn():
            return M.all_gather_last_dim(x, group), None
    else:
        def fn():
            return M.all_gather_first_dim(x, group, async_op=True)
    out, h = _on_comm_stream(fn, x, event, stream)
    return x, out, h


def async_reduce_scatter(x: torch.Tensor, group, event=None, stream=None, is_use_get_global_memory_buffer=False):
    out, h = _on_comm_stream(lambda: M.reduce_scatter_first_dim(x, group, async_op=True), x, event, stream)
    return x, out, h


def async_all_to_all(x: torch.Tensor, output_split_sizes, input_split_sizes, group, event=None, stream=None):
    out, h = _on_comm_stream(lambda: M.all_to_all_single(x, group, output_split_sizes, input_split_sizes, async_op=True),
                             x, event, stream)
    return x, out, h


# ---- communicator sizing ------------------------------------------------------------------------------------
@dataclasses.dataclass
class NcclOptions:
    """Per-group communicator tuning.  ``buffer_mb`` bounds NCCL's staging buffers (NCCL_BUFFSIZE equivalent per
    communicator); ``max_ctas`` / ``min_ctas`` bound the SMs a collective may occupy, which is what decides how
    much of the GPU stays free for a GEMM that overlaps it."""
    buffer_mb: Optional[int] = None
    max_ctas: Optional[int] = None
    min_ctas: Optional[int] = None
    high_priority_stream: bool = False

    def to_pg_options(self):
        """ProcessGroupNCCL.Options for dist.new_group(pg_options=...); None when NCCL is not available."""
        try:
            opts = dist.ProcessGroupNCCL.Options()
        except Exception:
            return None
        opts.is_high_priority_stream = self.high_priority_stream
        cfg = getattr(opts, "config", None)
        if cfg is not None:
            if self.max_ctas is not None and hasattr(cfg, "max_ctas"):
                cfg.max_ctas = int(self.max_ctas)
            if self.min_ctas is not None and hasattr(cfg, "min_ctas"):
                cfg.min_ctas = int(self.min_ctas)
        return opts


GROUP_KEYS = ("dp", "dp_cp", "cp", "mp", "tp", "pp", "embd", "tp_dp_cp", "tp_dp", "tp_cp", "tp_exp", "exp", "dp_modulo_exp",
              "pp_new_stream", "cp2", "cp_ulysses", "cp_ring", "cp_ring_intra", "cp_ring_intra_overlap", "nd1_dim1",
              "ag_x_sd_rcv_overlap", "nd1_dim2", "ag_y_sd_rcv_overlap", "nd2_dim1", "nd2_dim2")


def parse_buffer_spec(spec: Optional[str]) -> Dict[str, int]:
    """``"dp:200;tp:64"`` -> {"dp": 200, "tp": 64} (MB); unknown group names are rejected."""
    out: Dict[str, int] = {}
    if not spec:
        return out
    for item in spec.split(";"):
        item = item.strip()
        if not item:
            continue
        if ":" not in item:
            raise ValueError(f"bad communicator buffer entry '{item}', expected name:MB")
        k, v = item.split(":", 1)
        k = k.strip()
        if k not in GROUP_KEYS:
            raise ValueError(f"unknown parallel group '{k}' in communicator buffer spec")
        mb = int(v)
        if mb <= 0:
            raise ValueError("communicator buffer sizes must be positive")
        out[k] = mb
    return out


def _mb(nbytes: float) -> int:
    return max(1, int((nbytes + (1 << 20) - 1) // (1 << 20)))


def auto_buffer_sizes(args) -> Dict[str, int]:
    """Buffer sizes (MB) from the model shape: a group's buffer should hold the largest single message it carries,
    capped at 512 MB, so one collective is one staging pass.

      tp / tp-sp     one activation [s/cp, b, h] in bf16 (all-gather / reduce-scatter of the sequence shards)
      cp             one K+V block [2, s/cp, b, kv_heads*d / tp]
      pp             one boundary activation [s/(cp*tp if sp), b, h]
      ep             routed tokens: [s/cp * b * topk, h] (all-to-all)
      dp             one gradient bucket (default 40 M elements, fp32)
    """
    s = args.seq_length // max(1, getattr(args, "context_parallel_size", 1))
    b, h = args.micro_batch_size, args.hidden_size
    tp = max(1, args.tensor_model_parallel_size)
    e = 2  # bf16
    act = s * b * h * e
    nh = args.num_attention_heads
    kvh = getattr(args, "num_query_groups", None) or nh
    d = getattr(args, "kv_channels", None) or h // nh
    sizes = {"tp": _mb(act), "pp": _mb(act / (tp if getattr(args, "sequence_parallel", False) else 1)),
             "cp": _mb(2 * s * b * kvh * d * e / tp), "cp2": _mb(2 * s * b * kvh * d * e / tp)}
    if getattr(args, "num_experts", None):
        sizes["exp"] = _mb(s * b * getattr(args, "moe_router_topk", 2) * h * e)
        sizes["tp_exp"] = sizes["exp"]
    bucket = getattr(args, "ddp_bucket_size", None) or 40_000_000
    sizes["dp"] = _mb(bucket * 4)
    sizes["dp_cp"] = sizes["dp"]
    return {k: min(512, v) for k, v in sizes.items()}


def group_options(args) -> Dict[str, NcclOptions]:
    """Merge the user's spec over the automatic sizes (``--hccl-group-buffer`` / ``--hccl-group-buffer-adaptive``)."""
    sizes: Dict[str, int] = {}
    if getattr(args, "hccl_group_buffer_adaptive", False):
        sizes.update(auto_buffer_sizes(args))
    sizes.update(parse_buffer_spec(getattr(args, "hccl_group_buffer", None)))
    out = {}
    for k, mb in sizes.items():
        # collectives that are meant to overlap GEMMs get a CTA budget so that they leave SMs to the compute stream
        overlap = k in ("tp", "cp", "cp2", "exp", "tp_exp", "pp_new_stream")
        out[k] = NcclOptions(buffer_mb=mb, max_ctas=16 if overlap else None, high_priority_stream=overlap)
    return out


# ---- gloo-free host-object movement --------------------------------------------------------------------------
def default_slice_bytes() -> int:
    """--nccl-slice-size / --hccl-slice-size (bytes, one flag with two spellings) when arguments are set, else 10 MB."""
    try:
        from ..training.global_vars import get_args
        nbytes = getattr(get_args(), "hccl_slice_size", None)
        return int(nbytes) if nbytes else 10 * 1024 * 1024
    except RuntimeError:
        return 10 * 1024 * 1024


def gather_to_rank0_sliced(local: torch.Tensor, group, slice_bytes: Optional[int] = None,
                           device: Optional[torch.device] = None) -> Optional[List[torch.Tensor]]:
    """Gather equally shaped host tensors to group rank 0 through the device, ``slice_bytes`` at a time, so that no
    gloo group and no device buffer larger than ``world * slice_bytes`` is needed.  Returns the list on rank 0."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    flat = local.reshape(-1)
    slice_bytes = slice_bytes or default_slice_bytes()
    per = max(1, slice_bytes // max(1, flat.element_size()))
    dev = device or (torch.device("cuda", torch.cuda.current_device()) if dist.get_backend(group) == "nccl" else torch.device("cpu"))
    outs = [torch.empty_like(flat, device="cpu") for _ in range(world)] if rank == 0 else None
    for start in range(0, flat.numel(), per):
        n = min(per, flat.numel() - start)
        chunk = flat[start:start + n].to(dev)
        parts = [torch.empty_like(chunk) for _ in range(world)]
        dist.all_gather(parts, chunk, group=group)
        if rank == 0:
            for r in range(world):
                outs[r][start:start + n].copy_(parts[r])
    if rank == 0:
        return [o.view(local.shape) for o in outs]
    return None


def scatter_from_rank0_sliced(parts: Optional[List[torch.Tensor]], like: torch.Tensor, group,
                              slice_bytes: Optional[int] = None, device: Optional[torch.device] = None) -> torch.Tensor:
    """Inverse of ``gather_to_rank0_sliced``: rank 0 holds one host tensor per rank, every rank receives its own."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    out = torch.empty_like(like, device="cpu").reshape(-1)
    slice_bytes = slice_bytes or default_slice_bytes()
    per = max(1, slice_bytes // max(1, out.element_size()))
    dev = device or (torch.device("cuda", torch.cuda.current_device()) if dist.get_backend(group) == "nccl" else torch.device("cpu"))
    src = dist.get_global_rank(group, 0)
    for start in range(0, out.numel(), per):
        n = min(per, out.numel() - start)
        if rank == 0:
            stacked = torch.stack([p.reshape(-1)[start:start + n] for p in parts]).to(dev)
        else:
            stacked = torch.empty(world, n, dtype=out.dtype, device=dev)
        dist.broadcast(stacked, src=src, group=group)
        out[start:start + n].copy_(stacked[rank])
    return out.view(like.shape)


# ---- delayed logging all-reduce ------------------------------------------------------------------------------
class AsyncLogAllReduce:
    """Average logging scalars over a group without stalling: ``submit`` launches the all-reduce for step n and
    returns the finished averages of step n-1 (None at the first call); ``flush`` returns the last ones."""

    def __init__(self, group=None):
        self.group = group
        self._pending: Optional[Tuple[List[str], torch.Tensor, object, int]] = None

    def _world(self):
        if not dist.is_initialized():
            return 1
        return dist.get_world_size(self.group)

    def submit(self, values: Dict[str, torch.Tensor], step: int = 0) -> Optional[Tuple[int, Dict[str, float]]]:
        prev = self._collect()
        keys = sorted(values)
        if keys:
            buf = torch.stack([values[k].detach().float().reshape(()) for k in keys])
            work = None
            if self._world() > 1:
                work = dist.all_reduce(buf, group=self.group, async_op=True)
            self._pending = (keys, buf, work, step)
        return prev

    def _collect(self):
        if self._pending is None:
            return None
        keys, buf, work, step = self._pending
        self._pending = None
        if work is not None:
            work.wait()
        vals = (buf / self._world()).tolist()
        return step, dict(zip(keys, vals))

    def flush(self):
        return self._collect()
