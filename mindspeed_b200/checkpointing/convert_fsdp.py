"""Turn a checkpoint written by a fully sharded model (``--layerzero`` / ``--fsdp2-config-path``) into the regular layout.

  python -m mindspeed_b200.checkpointing.convert_fsdp --input_folder ckpt_fsdp --output_folder ckpt \\
      [--target_tp 2] [--target_pp 1] [--ema_model] [--for_release] [--prefix fsdp.]

A fully sharded run stores every parameter as a flat 1-D tensor (one key per parameter, per tensor-parallel rank and per
pipeline stage) plus the matching Adam moments; the regular layout stores named tensors with their shapes, per-layer tensors
stacked along a leading layer axis, which every data / tensor / pipeline layout of the distributed-data-parallel path can
read.  The conversion runs in one process without a GPU: the flat tensors are read whole, given back their shapes (kept in
the checkpoint's ``fsdp_layout`` record), tensor-parallel pieces are joined along their split axis, layers get their global
numbers, and the result is written with ``torch.distributed.checkpoint``.

``--target_tp``: a gated first MLP projection keeps its rows as ``[gate; up]`` per tensor-parallel rank; they are regrouped
from the source size to the target size, which the reader must then run with.  ``--target_pp`` is recorded only (the regular
layout is independent of the pipeline split).  The output holds weights only (``--for_release`` is accepted for
compatibility): continue from it with ``--finetune`` or ``--no-load-optim``.  ``--ema_model`` converts the optimizer's
``ema`` tensors instead of the live weights when the checkpoint has them.
reference: mindspeed/core/distributed/layerzero/state/scripts/convert_to_megatron.py:17-66 (same flags),
layerzero_checkpointer.py, mga_checkpoint.py (shard discovery and assembly).
"""
from __future__ import annotations

import argparse
import os
import sys
from typing import Dict, List, Optional

import torch


def regroup_gated(w: torch.Tensor, src_tp: int, dst_tp: int, dim: int = 0) -> torch.Tensor:
    """Rows laid out as [gate_0; up_0; gate_1; up_1; ...] over ``src_tp`` ranks -> the same for ``dst_tp`` ranks."""
    if src_tp == dst_tp:
        return w
    w = w.movedim(dim, 0)
    n = w.shape[0]
    if n % (2 * src_tp) or n % (2 * dst_tp):
        raise ValueError(f"gated projection with {n} rows cannot be regrouped from {src_tp} to {dst_tp} tensor-parallel ranks")
    parts = w.reshape(src_tp, 2, n // (2 * src_tp), *w.shape[1:])
    gate, up = parts[:, 0].reshape(n // 2, *w.shape[1:]), parts[:, 1].reshape(n // 2, *w.shape[1:])
    g, u = gate.reshape(dst_tp, 1, n // (2 * dst_tp), *w.shape[1:]), up.reshape(dst_tp, 1, n // (2 * dst_tp), *w.shape[1:])
    return torch.cat((g, u), dim=1).reshape(n, *w.shape[1:]).movedim(0, dim)


def _read_flat(path: str, keys_numel: Dict[str, int]) -> Dict[str, torch.Tensor]:
    from . import _load_sharded
    from .sharded import ShardedTensor
    sts = {k: ShardedTensor(k, torch.empty(n, dtype=torch.float32), (n,), (0,)) for k, n in keys_numel.items()}
    # dtype follows the file: read once into what the metadata says
    from torch.distributed.checkpoint import FileSystemReader
    md = FileSystemReader(path).read_metadata().state_dict_metadata
    for k, st in sts.items():
        if k not in md:
            raise KeyError(f"checkpoint has no tensor {k!r}")
        st.data = torch.empty(keys_numel[k], dtype=md[k].properties.dtype)
    missing = _load_sharded(sts, path, strict=True)
    if missing:
        raise KeyError(f"tensors missing from the checkpoint: {sorted(missing)[:5]}")
    return {k: st.data for k, st in sts.items()}


def assemble(layout: Dict[str, dict], flat: Dict[str, torch.Tensor], num_layers: int, target_tp: Optional[int] = None):
    """{regular key: full tensor} from the flat tensors; per-layer tensors stacked over ``num_layers``."""
    groups: Dict[tuple, List[tuple]] = {}
    for key, info in layout.items():
        if info.get("expert"):
            raise NotImplementedError("expert-parallel parameters of a fully sharded checkpoint are not converted")
        groups.setdefault((info["name"], info["layer"]), []).append((key, info))
    full: Dict[tuple, torch.Tensor] = {}
    src_tp = 1
    for (name, layer), items in groups.items():
        if items[0][1]["tp"] is None:
            key, info = items[0]                                    # replicated over tensor-parallel ranks: any copy
            full[(name, layer)] = flat[key].reshape(info["shape"])
            continue
        items.sort(key=lambda kv: kv[1]["tp"][0])
        _, world, dim, stride = items[0][1]["tp"]
        src_tp = world
        if [kv[1]["tp"][0] for kv in items] != list(range(world)):
            raise KeyError(f"{name}: pieces of tensor-parallel ranks {[kv[1]['tp'][0] for kv in items]} found, {world} expected")
        t = torch.cat([flat[k].reshape(i["shape"]) for k, i in items], dim=dim)
        if stride == 2 and target_tp is not None:
            t = regroup_gated(t, world, target_tp, dim)
        full[(name, layer)] = t
    out: Dict[str, torch.Tensor] = {}
    stacked: Dict[str, Dict[int, torch.Tensor]] = {}
    for (name, layer), t in full.items():
        if layer is None:
            out[name] = t
        else:
            stacked.setdefault(name, {})[layer] = t
    for name, rows in stacked.items():
        if sorted(rows) != list(range(num_layers)):
            raise KeyError(f"{name}: layers {sorted(rows)} found, 0..{num_layers - 1} expected")
        out[name] = torch.stack([rows[i] for i in range(num_layers)], dim=0)
    return out, src_tp


def convert(input_folder: str, output_folder: str, target_tp: Optional[int] = None, target_pp: Optional[int] = None,
            ema_model: bool = False, for_release: bool = True, prefix: str = "fsdp.", iteration: Optional[int] = None) -> str:
    from . import _save_sharded, get_checkpoint_name, read_latest_iteration
    from .sharded import ShardedTensor
    it = iteration if iteration is not None else read_latest_iteration(input_folder)
    if it is None:
        raise FileNotFoundError(f"no checkpoint under {input_folder!r}")
    src = get_checkpoint_name(input_folder, it)
    common = torch.load(os.path.join(src, "common.pt"), weights_only=False)
    layout = common.get("fsdp_layout")
    if not layout:
        raise ValueError(f"{src} was not written by a fully sharded model (no fsdp_layout record)")
    layout = {k: v for k, v in layout.items() if k.startswith(prefix)}
    num_layers = int(common.get("num_layers") or 0)
    numel = lambda shape: int(torch.Size(shape).numel())

    def load(kind: Optional[str]):
        """kind None: the weights; "exp_avg" / "exp_avg_sq" / "ema": the optimizer's per-parameter tensors of that name."""
        ren = (lambda k: k) if kind is None else (lambda k: "optimizer." + prefix + kind + "." + k[len(prefix):])
        flat = _read_flat(src, {ren(k): numel(v["shape"]) for k, v in layout.items()})
        return {k: flat[ren(k)] for k in layout}

    tensors, src_tp = assemble(layout, load("ema" if ema_model else None), num_layers, target_tp)
    tp_out = target_tp or src_tp
    sts = {k: ShardedTensor(k, t.contiguous(), tuple(t.shape), (0,) * t.dim()) for k, t in tensors.items()}
    dst = get_checkpoint_name(output_folder, it)
    _save_sharded(sts, dst)
    out_common = {k: v for k, v in common.items() if k not in ("fsdp_layout", "optimizer", "opt_param_scheduler")}
    args = dict(out_common.get("args") or {})
    args.update(tensor_model_parallel_size=tp_out, pipeline_model_parallel_size=target_pp or 1, layerzero=False, fsdp2_config_path=None)
    out_common["args"] = args
    out_common["converted_from"] = {"layout": "fully_sharded", "source_tp": src_tp, "weights": "ema" if ema_model else "model"}
    torch.save(out_common, os.path.join(dst, "common.pt"))
    with open(os.path.join(output_folder, "latest_checkpointed_iteration.txt"), "w") as f:
        f.write(str(it))
    return dst


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--input_folder", "--input-folder", dest="input_folder", required=True)
    ap.add_argument("--output_folder", "--output-folder", dest="output_folder", required=True)
    ap.add_argument("--target_tp", "--target-tp", dest="target_tp", type=int, default=None)
    ap.add_argument("--target_pp", "--target-pp", dest="target_pp", type=int, default=None)
    ap.add_argument("--ema_model", "--ema-model", dest="ema_model", action="store_true")
    ap.add_argument("--for_release", "--for-release", dest="for_release", action="store_true", default=True,
                    help="weights only (always the case: optimizer state is not converted)")
    ap.add_argument("--prefix", default="fsdp.")
    ap.add_argument("--iteration", type=int, default=None)
    a = ap.parse_args(argv)
    dst = convert(a.input_folder, a.output_folder, a.target_tp, a.target_pp, a.ema_model, a.for_release, a.prefix, a.iteration)
    print(dst)
    return 0


if __name__ == "__main__":
    sys.exit(main())
