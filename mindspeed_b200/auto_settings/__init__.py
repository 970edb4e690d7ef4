"""auto_settings: search tensor / context / pipeline / data / expert parallel sizes, micro-batch size and recompute for
a model on N GPUs (reference: mindspeed/auto_settings/auto_settings.py:30-164)."""
from __future__ import annotations

import json
import os

from .cost_model import Estimate, estimate, memory_gib, step_ms
from .hardware import Hardware, probe, probe_collectives
from .search_space import ModelDesc, SearchConfig, build_search_space
from .comm_predictors import CommPredictors
from .operator_db import OperatorDB
from .profiling_parse import ProfileSummary, parse_chrome_trace, summarize
from .searcher import black_search, mixed_search, white_search


class AutoSettings:
    def auto_setting_fun(self, args):
        """Entry used by ``pretrain`` under ``--auto-settings``: only local rank 0 of each node searches; the result is
        written to ``<work_dir>/auto_settings_result.json`` and returned."""
        if int(os.environ.get("LOCAL_RANK", "0")) != 0:
            return None
        model = ModelDesc.from_args(args)
        world = args.auto_settings_ranks
        hw = Hardware.load(getattr(args, "prof_file", None))
        try:
            hw = probe(hw)
        except Exception:
            pass
        kind = args.auto_settings_type
        os.makedirs(args.auto_settings_work_dir, exist_ok=True)
        # what profiled runs taught earlier searches in this work directory is reused: measured operator times and the
        # per-dimension communication lines
        from .comm_predictors import CommPredictors
        from .operator_db import OperatorDB
        db = OperatorDB(os.path.join(args.auto_settings_work_dir, "operator_db.sqlite"))
        comm = CommPredictors(hw)
        if kind == "white":
            best = white_search(model, world, hw, db=db if len(db) else None)
        else:
            from .executor import TorchrunExecutor
            base = self._base_flags(args)
            ex = TorchrunExecutor(base, world, master_port=args.master_port + 7,
                                  profile_dir=os.path.join(args.auto_settings_work_dir, "profiles") if kind == "mixed" else None)
            best = black_search(model, world, hw, ex) if kind == "black" else mixed_search(model, world, hw, ex, db=db, comm=comm)
        out = [{"rank": i, "config": e.config.as_dict(), "flags": e.config.to_flags(), "step_ms": e.step_ms, "memory_gib": e.memory_gib,
                "detail": e.detail} for i, e in enumerate(best)]
        with open(os.path.join(args.auto_settings_work_dir, "auto_settings_result.json"), "w") as f:
            json.dump(out, f, indent=1)
        for o in out:
            print(f"[auto_settings] #{o['rank']} step {o['step_ms']:.0f} ms, {o['memory_gib']:.0f} GiB: {' '.join(o['flags'])}", flush=True)
        return out

    @staticmethod
    def _base_flags(args):
        keep = ["num_layers", "hidden_size", "ffn_hidden_size", "num_attention_heads", "seq_length", "max_position_embeddings",
                "global_batch_size", "vocab_size", "lr", "num_query_groups", "num_experts", "moe_router_topk", "normalization",
                "position_embedding_type", "rotary_base"]
        flags = []
        for k in keep:
            v = getattr(args, k, None)
            if v is not None:
                flags += ["--" + k.replace("_", "-"), str(v)]
        for k in ("bf16", "swiglu", "group_query_attention", "untie_embeddings_and_output_weights", "use_flash_attn", "moe_grouped_gemm"):
            if getattr(args, k, False):
                flags.append("--" + k.replace("_", "-"))
        if not getattr(args, "add_bias_linear", True):
            flags.append("--disable-bias-linear")
        if getattr(args, "moe_token_dispatcher_type", None):
            flags += ["--moe-token-dispatcher-type", args.moe_token_dispatcher_type]
        return flags + ["--make-vocab-size-divisible-by", "1", "--mock-data", "--hidden-dropout", "0", "--attention-dropout", "0"]
