"""Distributed + model-parallel initialisation (Megatron ``initialize_megatron`` surface)."""
from __future__ import annotations

import datetime
import os
import random

import numpy as np
import torch
import torch.distributed as dist

from ..features import get_features_manager
from ..parallel import parallel_state as ps
from ..parallel.comm_ops import select_ops
from ..parallel.random import model_parallel_cuda_manual_seed
from . import global_vars
from .arguments import parse_args, validate_args


def _initialize_distributed(args):
    if dist.is_initialized():
        return
    backend = args.distributed_backend
    if backend == "nccl" and not torch.cuda.is_available():
        backend = "gloo"
    if torch.cuda.is_available() and backend == "nccl":
        torch.cuda.set_device(args.local_rank % max(1, torch.cuda.device_count()))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    dist.init_process_group(backend=backend, world_size=args.world_size, rank=args.rank,
                            timeout=datetime.timedelta(minutes=args.distributed_timeout_minutes))


def set_random_seed(seed, data_parallel_random_init=False):
    seed = seed + 100 * ps.get_pipeline_model_parallel_rank()
    if data_parallel_random_init:
        seed += 10 * ps.get_data_parallel_rank()
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    model_parallel_cuda_manual_seed(seed)


def initialize_megatron(extra_args_provider=None, args_defaults=None, ignore_unknown_args=False, args_list=None,
                        parsed_args=None):
    args = parsed_args if parsed_args is not None else parse_args(extra_args_provider, ignore_unknown_args, args_list)
    for k, v in (args_defaults or {}).items():
        if getattr(args, k, None) is None:
            setattr(args, k, v)
    validate_args(args)
    global_vars.set_args(args)
    fm = get_features_manager()
    fm.apply_features_pre_configure(args)
    _initialize_distributed(args)
    if not ps.model_parallel_is_initialized():
        ps.initialize_model_parallel(
            tensor_model_parallel_size=args.tensor_model_parallel_size,
            pipeline_model_parallel_size=args.pipeline_model_parallel_size,
            virtual_pipeline_model_parallel_size=args.virtual_pipeline_model_parallel_size,
            context_parallel_size=args.context_parallel_size,
            expert_model_parallel_size=args.expert_model_parallel_size,
            expert_tensor_parallel_size=args.expert_tensor_parallel_size,
            num_distributed_optimizer_instances=args.num_distributed_optimizer_instances,
            distributed_timeout_minutes=args.distributed_timeout_minutes,
            order="tp-cp-ep-dp-pp" if not args.use_tp_pp_dp_mapping else "tp-cp-ep-pp-dp",
            create_gloo_process_groups=not args.disable_gloo_group,
            use_cp_send_recv_overlap=args.use_cp_send_recv_overlap,
            ulysses_degree_in_cp=args.ulysses_degree_in_cp if args.context_parallel_algo.startswith("hybrid") else None,
            cp_window_size=args.cp_window_size,
            tp_2d=args.tp_2d, tp_x=args.tp_x, tp_y=args.tp_y,
            # the overlapped pipeline exchange needs one communicator per direction (executor.py)
            optimize_send_recv_comm=args.optimize_send_recv_comm or getattr(args, "overlap_p2p_comm", False),
        )
    if getattr(args, "overlap_p2p_comm", False) and args.pipeline_model_parallel_size > 1:
        from ..parallel.pipeline.p2p import warm_up_p2p
        warm_up_p2p()                    # pair communicators are created here, in one order on every rank
    set_random_seed(args.seed)
    fm.apply_features(args)
    kind = fm.resolve("tp_comm_ops", "default")
    select_ops(args.optimization_level, use_fused=(kind == "fused"), use_chunked=(kind == "chunked"),
               parallel_num=max(2, getattr(args, "coc_parallel_num", 2)))
    from ..parallel.pipeline.schedules import set_schedule
    set_schedule(fm.resolve("schedule", None))
    from ..ops.attention import set_backend as set_attention_backend
    want = getattr(args, "attention_backend", "auto")
    set_attention_backend("sm100" if (args.optimization_level >= 1 and want != "library" and torch.cuda.is_available()) else None)
    from ..parallel.context_parallel.ulysses import set_fused_all_to_all
    set_fused_all_to_all(args.optimization_level >= 2 and torch.cuda.is_available()
                         and not getattr(args, "no_fused_ulysses_a2a", False))
    return args
