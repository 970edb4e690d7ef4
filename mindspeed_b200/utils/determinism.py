"""Deterministic execution switch (reference: mindspeed/functional/npu_deterministic/npu_deterministic.py:9-31).
Sets the cuBLAS workspace config, NCCL algorithm pins and torch's deterministic mode; the hand-written
kernels in this package use fixed reduction orders; the one exception, k-block balancing of the weight-gradient
GEMM (partial tiles summed by reduce-adds in varying order), is switched off here."""
import os
import random

import numpy as np
import torch


def enable_determinism(seed=1234):
    os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":4096:8")
    os.environ.setdefault("NCCL_ALGO", "Ring")
    os.environ["MSB200_DETERMINISTIC"] = "1"
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    torch.use_deterministic_algorithms(True, warn_only=True)
    torch.backends.cudnn.deterministic = True
    torch.backends.cudnn.benchmark = False
    from ..ops import loader
    L = loader.lib()
    if L is not None:
        L.msb_gemm_set_stream_k(0)
