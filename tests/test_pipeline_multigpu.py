"""Pipeline schedules on GPUs (NCCL point-to-point, bf16, the package's kernels): the loss follows the same model on one GPU.

Every layout starts from weights that depend only on a parameter's global name and reads data keyed by (step, micro-batch),
so the only differences from the one-GPU run are the bf16 summation orders.
"""
import json
import os
import subprocess
import sys
import tempfile

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CODE = r'''
import os, sys, json
sys.path.insert(0, os.path.join(os.getcwd(), "tests"))
import torch
import pretrain_gpt as pg
from test_pipeline_cpu import _canonical_init
from mindspeed_b200.parallel import parallel_state as ps
from mindspeed_b200.parallel.pipeline.executor import current_microbatch
from mindspeed_b200.training import initialize_megatron, setup_model_and_optimizer, train_step
from mindspeed_b200.training.data import SyntheticGPTDataset
extra = json.loads(sys.argv[1])
al = ["--num-layers","4","--hidden-size","512","--num-attention-heads","4","--group-query-attention","--num-query-groups","2",
 "--ffn-hidden-size","1024","--seq-length","512","--max-position-embeddings","512","--micro-batch-size","1","--global-batch-size","8",
 "--vocab-size","2048","--make-vocab-size-divisible-by","1","--bf16","--lr","1e-3","--lr-decay-style","constant","--hidden-dropout","0",
 "--attention-dropout","0","--swiglu","--normalization","RMSNorm","--position-embedding-type","rope","--disable-bias-linear",
 "--untie-embeddings-and-output-weights","--use-flash-attn","--train-iters","4","--optimization-level","2","--seed","1234",
 "--weight-decay","0.0","--clip-grad","0.0"] + extra
args = initialize_megatron(args_list=al)
model, opt, sched = setup_model_and_optimizer(pg.model_provider)
_canonical_init(model)
opt.reload_model_params()
ds = SyntheticGPTDataset(args.padded_vocab_size, args.seq_length, 4096, seed=args.seed)
dp_r, dp_n = ps.get_data_parallel_rank(), ps.get_data_parallel_world_size()
nmb = args.global_batch_size // (args.micro_batch_size * dp_n)
state = {"step": 0, "i": 0}
dev = torch.device("cuda", torch.cuda.current_device())
piped = ps.get_pipeline_model_parallel_world_size() > 1

class It:
    def __iter__(self):
        return self
    def __next__(self):
        if piped:
            mb = current_microbatch()["mb"]
        else:
            mb = state["i"] % nmb
            state["i"] += 1
        item = ds[state["step"] * args.global_batch_size + dp_r * nmb + mb]
        return {k: v.unsqueeze(0).to(dev) for k, v in item.items()}

it = It()
out = []
for _ in range(4):
    ld, *_ = train_step(pg.forward_step, [it] * len(model) if len(model) > 1 else it, model, opt, sched)
    state["step"] += 1
    out.append(float(ld["lm loss"]) if "lm loss" in ld else None)
from mindspeed_b200.ops import gemm as G
torch.cuda.synchronize(); G.check_status()
res = [None] * torch.distributed.get_world_size()
torch.distributed.all_gather_object(res, out)
if int(os.environ["RANK"]) == 0:
    print("LOSSES", json.dumps([r for r in res if r[0] is not None][0]))
torch.distributed.barrier()
from mindspeed_b200.parallel.symm_mem import destroy_heaps
destroy_heaps()
torch.distributed.destroy_process_group()
'''


def _run(nproc, extra, port):
    with tempfile.NamedTemporaryFile("w", suffix=".py", dir=ROOT, delete=False) as f:
        f.write(CODE)
        path = f.name
    try:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc), "--master-addr",
               "127.0.0.1", "--master-port", str(port), path, json.dumps(extra)]
        r = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=240)
    finally:
        os.remove(path)
    log_dir = os.environ.get("MSB200_TEST_LOG_DIR")
    if r.returncode != 0 and log_dir:
        with open(os.path.join(log_dir, f"pipeline_multigpu_{port}_{nproc}.log"), "w") as f:
            f.write(" ".join(extra) + "\n" + r.stdout[-20000:] + "\n" + r.stderr[-60000:])
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-6000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("LOSSES")][0]
    return json.loads(line[len("LOSSES "):])


_REF = {}


def _reference(extra=()):
    key = tuple(extra)
    if key not in _REF:
        _REF[key] = _run(1, list(extra), 29720 + len(_REF))
    return _REF[key]


def _close(a, b, tol, decreasing=True):
    for x, y in zip(a, b):
        assert abs(x - y) < tol * max(1.0, abs(x)), (a, b)
    if decreasing:
        assert b[-1] < b[0]


@pytest.mark.parametrize("extra", [
    ["--pipeline-model-parallel-size", "2", "--overlap-p2p-communication"],
    ["--pipeline-model-parallel-size", "2", "--num-layers-per-virtual-pipeline-stage", "1", "--overlap-p2p-communication"],
    ["--pipeline-model-parallel-size", "2", "--schedules-method", "dualpipev", "--overlap-p2p-communication"],
    ["--pipeline-model-parallel-size", "2", "--schedules-method", "dualpipev"],
])
def test_two_stage_pipeline_follows_one_gpu(extra):
    _close(_reference(), _run(2, extra, 29730), 0.02)


MOE = ["--num-experts", "4", "--moe-router-topk", "2", "--moe-token-dispatcher-type", "alltoall", "--moe-grouped-gemm",
       "--moe-aux-loss-coeff", "0.0", "--global-batch-size", "16"]


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


@pytest.mark.skipif(_ngpu() < 4, reason="needs 4 GPUs (pipeline 2 x expert parallel 2) or 8 (x 4)")
@pytest.mark.parametrize("extra", [
    ["--pipeline-model-parallel-size", "2", "--overlap-p2p-communication"],
    ["--pipeline-model-parallel-size", "2", "--schedules-method", "dualpipev", "--overlap-p2p-communication", "--moe-alltoall-mc2"],
])
def test_pipeline_with_expert_parallel_follows_one_gpu(extra):
    n = 8 if _ngpu() >= 8 else 4
    _close(_reference(MOE), _run(n, MOE + ["--expert-model-parallel-size", str(n // 2)] + extra, 29740), 0.01, decreasing=False)


@pytest.mark.parametrize("overlap", [False, True])
def test_moe_forward_backward_overlap_follows_one_gpu(overlap):
    """Expert parallelism 2 with the fused dispatcher on two GPUs, plain and with ``--moe-fb-overlap`` (forward of one
    micro-batch interleaved with the backward of the previous one on two streams): the loss follows the one-GPU run."""
    extra = MOE + ["--expert-model-parallel-size", "2", "--moe-alltoall-mc2"] + (["--moe-fb-overlap"] if overlap else [])
    ref, got = _reference(MOE), _run(2, extra, 29750 + int(overlap))
    log_dir = os.environ.get("MSB200_TEST_LOG_DIR")
    if log_dir:
        with open(os.path.join(log_dir, f"moe_fb_overlap_{int(overlap)}.json"), "w") as f:
            json.dump({"ref": ref, "got": got}, f)
    _close(ref, got, 0.01, decreasing=False)      # four steps of a freshly initialised router do not lower the loss yet
