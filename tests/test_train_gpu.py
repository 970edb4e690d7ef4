"""End-to-end single-GPU training smoke tests through the public API."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_smoke_entry():
    r = subprocess.run([sys.executable, "-c", "import __graft_entry__ as g; g.smoke()"], cwd=ROOT, capture_output=True,
                       text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "smoke ok" in r.stdout


def test_loss_decreases_level1_vs_level0():
    code = r'''
import os, sys, json
os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT="29577", RANK="0", WORLD_SIZE="1")
import torch
import pretrain_gpt as pg
from mindspeed_b200.training import initialize_megatron, setup_model_and_optimizer, train_step
lvl = sys.argv[1]
al = ["--num-layers","2","--hidden-size","512","--num-attention-heads","4","--group-query-attention","--num-query-groups","2",
 "--ffn-hidden-size","1536","--seq-length","512","--max-position-embeddings","512","--micro-batch-size","2","--global-batch-size","4",
 "--vocab-size","4096","--make-vocab-size-divisible-by","1","--bf16","--lr","1e-3","--lr-decay-style","constant","--hidden-dropout","0",
 "--attention-dropout","0","--swiglu","--normalization","RMSNorm","--position-embedding-type","rope","--disable-bias-linear",
 "--untie-embeddings-and-output-weights","--use-flash-attn","--use-distributed-optimizer","--train-iters","8","--optimization-level",lvl]
args = initialize_megatron(args_list=al)
model, opt, sched = setup_model_and_optimizer(pg.model_provider)
it = pg.train_valid_test_datasets_provider(args)
out = []
for _ in range(8):
    ld, *_ = train_step(pg.forward_step, it, model, opt, sched)
    out.append(float(ld["lm loss"]))
print("LOSSES", json.dumps(out))
'''
    res = {}
    for lvl in ("0", "1"):
        r = subprocess.run([sys.executable, "-c", code, lvl], cwd=ROOT, capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
        import json
        line = [l for l in r.stdout.splitlines() if l.startswith("LOSSES")][0]
        res[lvl] = json.loads(line[len("LOSSES "):])
    # same data & seed: the fused-kernel path follows the library path within bf16 noise
    for a, b in zip(res["0"], res["1"]):
        assert abs(a - b) < 0.05 * max(1.0, abs(a)), res
    assert all(x == x and x < 12 for x in res["1"])
