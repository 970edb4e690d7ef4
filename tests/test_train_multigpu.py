"""Two-GPU tensor+sequence-parallel training: fused comm kernels (level 2) follow the NCCL + cuBLAS path (level 0)."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CODE = r'''
import os, sys, json
import torch
import pretrain_gpt as pg
from mindspeed_b200.training import initialize_megatron, setup_model_and_optimizer, train_step
lvl = sys.argv[1]
mode = sys.argv[2] if len(sys.argv) > 2 else "tp"
al = ["--num-layers","2","--hidden-size","1024","--num-attention-heads","8","--group-query-attention","--num-query-groups","2",
 "--ffn-hidden-size","3072","--seq-length","1024","--max-position-embeddings","1024","--micro-batch-size","1","--global-batch-size","2",
 "--vocab-size","8192","--make-vocab-size-divisible-by","1","--bf16","--lr","1e-3","--lr-decay-style","constant","--hidden-dropout","0",
 "--attention-dropout","0","--swiglu","--normalization","RMSNorm","--position-embedding-type","rope","--disable-bias-linear",
 "--untie-embeddings-and-output-weights","--use-flash-attn","--use-distributed-optimizer","--train-iters","6","--optimization-level",lvl,
 ]
if mode == "tp":
    al += ["--tensor-model-parallel-size","2","--sequence-parallel"]
    if lvl == "2":
        al += ["--use-fused-tp-comm"]
else:   # data parallel 2: the distributed-optimizer step, library path or fused peer-memory kernel
    al += ["--clip-grad", "1.0"]
    if mode == "dp_fused":
        al += ["--use-fused-dist-opt"]
args = initialize_megatron(args_list=al)
model, opt, sched = setup_model_and_optimizer(pg.model_provider)
it = pg.train_valid_test_datasets_provider(args)
out = []
for _ in range(6):
    ld, *_ = train_step(pg.forward_step, it, model, opt, sched)
    out.append(float(ld["lm loss"]))
from mindspeed_b200.ops import gemm as G
torch.cuda.synchronize(); G.check_status()
from mindspeed_b200.parallel.comm_ops import get_ops
if int(os.environ["RANK"]) == 0:
    print("LOSSES", json.dumps({"ops": get_ops().name, "loss": out}))
torch.distributed.barrier()
from mindspeed_b200.parallel.symm_mem import destroy_heaps
destroy_heaps()
torch.distributed.destroy_process_group()
'''


def _run(level, port, mode="tp"):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), "-c", CODE, level]
    # torchrun cannot take -c; write the script next to the tests' temp dir instead
    import tempfile
    with tempfile.NamedTemporaryFile("w", suffix=".py", dir=ROOT, delete=False) as f:
        f.write(CODE)
        path = f.name
    try:
        cmd = cmd[:-3] + [path, level, mode]
        r = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=600)
    finally:
        os.remove(path)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-6000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("LOSSES")][0]
    return json.loads(line[len("LOSSES "):])


def test_level2_fused_comm_follows_level0():
    a = _run("0", 29701)
    b = _run("2", 29702)
    assert a["ops"] == "default" and b["ops"] == "fused"
    for x, y in zip(a["loss"], b["loss"]):
        assert abs(x - y) < 0.05 * max(1.0, abs(x)), (a, b)


def test_fused_distributed_optimizer_follows_nccl_path():
    a = _run("2", 29703, "dp")
    b = _run("2", 29704, "dp_fused")
    for x, y in zip(a["loss"], b["loss"]):
        assert abs(x - y) < 0.02 * max(1.0, abs(x)), (a, b)
    assert b["loss"][-1] < b["loss"][0]
