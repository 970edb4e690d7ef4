"""Megatron-side training flags that launch scripts pass: each one acts (or is listed as having no effect)."""
import json
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def test_gpt2_bpe_tokenizer_round_trip_and_merge_order(tmp_path):
    from types import SimpleNamespace
    from mindspeed_b200.tokenizer.tokenizer import GPT2BPETokenizer, build_tokenizer
    # a tiny vocabulary: single mapped bytes, a few merges, the end-of-text token
    tok0 = GPT2BPETokenizer.__new__(GPT2BPETokenizer)
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAD)) + list(range(0xAE, 0x100))
    chars, n = {}, 0
    for b in range(256):
        if b in bs:
            chars[b] = chr(b)
        else:
            chars[b] = chr(256 + n)
            n += 1
    sp = chars[ord(" ")]
    merges = [("l", "o"), ("lo", "w"), (sp, "low"), ("e", "r"), ("low", "er")]
    vocab = {c: i for i, c in enumerate(sorted(set(chars.values())))}
    for a, b in merges:
        vocab[a + b] = len(vocab)
    vocab["<|endoftext|>"] = len(vocab)
    vf, mf = tmp_path / "vocab.json", tmp_path / "merges.txt"
    vf.write_text(json.dumps(vocab), encoding="utf-8")
    mf.write_text("#version: 0.2\n" + "\n".join(f"{a} {b}" for a, b in merges) + "\n", encoding="utf-8")
    tok = build_tokenizer(SimpleNamespace(tokenizer_type="GPT2BPETokenizer", vocab_file=str(vf), merge_file=str(mf),
                                          padded_vocab_size=None, make_vocab_size_divisible_by=128, tensor_model_parallel_size=1))
    ids = tok.tokenize("low lower slow")
    pieces = [tok.decoder[i] for i in ids]
    assert pieces == ["low", sp + "low", "er", sp, "s", "low"]          # merges applied by priority inside each word
    assert tok.detokenize(ids) == "low lower slow"
    text = "naïve café 你好 🙂\n\ttabs"
    assert tok.detokenize(tok.tokenize(text)) == text                   # any UTF-8 text survives (byte fallback)
    assert tok.eod == vocab["<|endoftext|>"] and tok.vocab_size == len(vocab)
    with pytest.raises(ValueError, match="vocab-file"):
        build_tokenizer(SimpleNamespace(tokenizer_type="GPT2BPETokenizer", vocab_file=None, merge_file=None))


def test_weight_decay_schedule_and_scheduler_state():
    from mindspeed_b200.training.training import OptimizerParamScheduler
    p = torch.nn.Parameter(torch.zeros(2))
    q = torch.nn.Parameter(torch.zeros(2))
    opt = torch.optim.AdamW([{"params": [p], "weight_decay": 0.1}, {"params": [q], "weight_decay": 0.0}], lr=1.0)
    s = OptimizerParamScheduler(opt, 1.0, 0.0, 0, 10, "constant", start_wd=0.1, end_wd=0.5, wd_incr_steps=4, wd_incr_style="linear")
    seen = []
    for _ in range(6):
        seen.append(round(opt.param_groups[0]["weight_decay"], 6))
        s.step(1)
    assert seen == [0.1, 0.2, 0.3, 0.4, 0.5, 0.5] and opt.param_groups[1]["weight_decay"] == 0.0
    c = OptimizerParamScheduler(opt, 1.0, 0.0, 0, 10, "constant", start_wd=0.0, end_wd=1.0, wd_incr_steps=2, wd_incr_style="cosine")
    c.step(1)
    assert abs(c.get_wd() - 0.5) < 1e-9
    sd = s.state_dict()
    assert sd["num_steps"] == 6 and sd["schedule"]["end_wd"] == 0.5 and sd["schedule"]["wd_style"] == "linear"
    k = OptimizerParamScheduler(opt, 1.0, 0.0, 0, 10, "constant", start_wd=0.3, end_wd=0.3)
    assert k.get_wd() == 0.3


def _run(rank, world, extra):
    import io
    from contextlib import redirect_stdout
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import pretrain_gpt as pg
    from test_pipeline_cpu import BASE
    from mindspeed_b200.training import pretrain
    base = [a for a in BASE]
    if "--train-samples" in extra:
        i = base.index("--train-iters")
        del base[i:i + 2]
    buf = io.StringIO()
    with redirect_stdout(buf):
        hist = pretrain(pg.train_valid_test_datasets_provider, pg.model_provider, forward_step_func=pg.forward_step,
                        args_list=base + list(extra))
    import gc
    enabled = gc.isenabled()
    gc.enable()
    return hist, buf.getvalue(), enabled


def test_training_flags_act(tmp_path):
    from dist_utils import run_distributed
    hist, out, gc_on = run_distributed(_run, 1, ["--train-samples", "16", "--log-num-zeros-in-grad", "--log-params-norm",
                                                 "--manual-gc", "--manual-gc-interval", "1"])[0]
    assert len(hist) == 2                                            # 16 samples / global batch 8
    assert all(h["num zeros"] >= 0 and h["params norm"] > 1.0 for h in hist) and "params norm" in out
    assert not gc_on                                                 # automatic collection was switched off
    # tensor-parallel ranks report the same parameter norm as one rank (duplicates counted once)
    tp = run_distributed(_run, 2, ["--train-samples", "8", "--log-params-norm", "--tensor-model-parallel-size", "2"])[0][0]
    one = run_distributed(_run, 1, ["--train-samples", "8", "--log-params-norm"])[0][0]
    assert tp[0]["params norm"] == pytest.approx(one[0]["params norm"], rel=0.2)      # same order (different random init per layout)
    # --skip-train: no steps, the evaluation still runs
    hist, out, _ = run_distributed(_run, 1, ["--skip-train", "--eval-iters", "1"])[0]
    assert len(hist) == 1 and "validation lm loss" in hist[0] and "validation loss (no training)" in out
    # --exit-on-missing-checkpoint
    hist, out, _ = run_distributed(_run, 1, ["--load", str(tmp_path / "nothing"), "--exit-on-missing-checkpoint"])[0]
    assert hist == [] and "exit-on-missing-checkpoint" in out


def test_spellings_and_mappings(monkeypatch):
    monkeypatch.setenv("WORLD_SIZE", "2")
    from mindspeed_b200.models.te_compat import DelayedScaling, recipe_from_args
    from mindspeed_b200.training.arguments import parse_args, validate_args
    base = ["--num-layers", "2", "--hidden-size", "64", "--num-attention-heads", "4", "--seq-length", "32",
            "--micro-batch-size", "1", "--vocab-size", "128"]
    a = validate_args(parse_args(args_list=base + ["--use-torch-fsdp2"]))
    assert a.layerzero
    a = validate_args(parse_args(args_list=base + ["--use-custom-fsdp", "--data-parallel-sharding-strategy", "optim_grads_params"]))
    assert a.layerzero
    a = validate_args(parse_args(args_list=base + ["--use-custom-fsdp", "--data-parallel-sharding-strategy", "optim"]))
    assert a.use_distributed_optimizer and not a.layerzero
    a = validate_args(parse_args(args_list=base + ["--multi-latent-attention", "--qk-head-dim", "32", "--qk-pos-emb-head-dim", "16",
                                                   "--rotary-scaling-factor", "4", "--beta-fast", "16", "--beta-slow", "2"]))
    assert (a.qk_nope_head_dim, a.qk_rope_head_dim, a.rope_scaling_factor, a.rope_scaling_beta_fast, a.rope_scaling_beta_slow) == (32, 16, 4, 16, 2)
    a = validate_args(parse_args(args_list=base + ["--no-position-embedding"]))
    assert a.position_embedding_type == "none"
    a = validate_args(parse_args(args_list=base + ["--fp8-format", "hybrid", "--fp8-recipe", "delayed", "--fp8-amax-history-len", "4",
                                                   "--fp8-amax-compute-algo", "most_recent"]))
    r = recipe_from_args(a)
    assert isinstance(r, DelayedScaling) and r.amax_history_len == 4 and r.amax_compute_algo == "most_recent"
    a = validate_args(parse_args(args_list=base + ["--start-weight-decay", "0.0", "--end-weight-decay", "0.1",
                                                   "--weight-decay-incr-style", "linear"]))
    assert a.weight_decay == 0.0 and a.end_weight_decay == 0.1
    with pytest.raises(AssertionError, match="end-weight-decay"):
        validate_args(parse_args(args_list=base + ["--start-weight-decay", "0.0"]))
    with pytest.raises(AssertionError, match="not both"):
        validate_args(parse_args(args_list=base + ["--train-iters", "3", "--train-samples", "16"]))


def test_router_dtype_and_seq_aux(monkeypatch):
    monkeypatch.setenv("WORLD_SIZE", "1")
    from mindspeed_b200.training.arguments import parse_args, validate_args
    base = ["--num-layers", "2", "--hidden-size", "64", "--num-attention-heads", "4", "--seq-length", "32",
            "--micro-batch-size", "1", "--vocab-size", "128", "--num-experts", "4"]
    a = validate_args(parse_args(args_list=base + ["--seq-aux", "--moe-router-dtype", "fp64"]))
    assert a.moe_router_load_balancing_type == "seq_aux_loss" and a.moe_router_dtype == "fp64"
    from mindspeed_b200.config import TransformerConfig
    from mindspeed_b200.parallel import parallel_state as ps
    from mindspeed_b200.parallel.moe.router import TopKRouter
    import torch.distributed as dist
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1"); os.environ.setdefault("MASTER_PORT", str(__import__("dist_utils")._free_port()))
    if not dist.is_initialized():
        dist.init_process_group("gloo", rank=0, world_size=1)
    ps.destroy_model_parallel()
    ps.initialize_model_parallel(1, 1)
    kw = dict(num_layers=1, hidden_size=32, num_attention_heads=4, use_cpu_initialization=True, optimization_level=0,
              num_moe_experts=4, moe_router_topk=2)
    cfg = TransformerConfig(**kw)
    r = TopKRouter(cfg, 1)
    x = torch.randn(6, 1, 32)
    assert r.gating(x).dtype == torch.float32
    cfg.moe_router_dtype = "fp64"
    assert r.gating(x).dtype == torch.float64
    probs, rmap = r(x)
    assert rmap.sum(-1).tolist() == [2] * 6 and torch.isfinite(probs).all()
    ps.destroy_model_parallel()


def test_yaml_file_with_megatron_sections_and_config_field_names(tmp_path, monkeypatch):
    """Sections ``language_model`` / ``model_parallel`` are flattened and configuration field names are translated to the
    arguments that carry them; nulls keep the defaults."""
    monkeypatch.setenv("WORLD_SIZE", "8")
    from mindspeed_b200.training.arguments import core_transformer_config_from_args, parse_args, validate_args
    y = tmp_path / "cfg.yaml"
    y.write_text("""
language_model:
  num_layers: 4
  hidden_size: 256
  num_attention_heads: 8
  num_query_groups: 4
  ffn_hidden_size: 512
  kv_channels: 32
  layernorm_epsilon: 0.00002
  layernorm_zero_centered_gamma: True
  add_bias_linear: False
  activation_func: swiglu
  num_moe_experts: null
  normalization: 'RMSNorm'
  window_size: null
  moe_router_topk: 2
  recompute_granularity: null
model_parallel:
  tensor_model_parallel_size: 2
  context_parallel_size: 4
  sequence_parallel: True
  bf16: True
  use_cpu_initialization: null
group_query_attention: True
seq_length: 64
micro_batch_size: 1
vocab_size: 128
adam_beta2: 0.95
ampipe_degree: 1
position_embedding_type: rope
""")
    a = validate_args(parse_args(args_list=["--yaml-cfg", str(y)]))
    assert (a.tensor_model_parallel_size, a.context_parallel_size, a.data_parallel_size) == (2, 4, 1)
    assert a.norm_epsilon == 0.00002 and a.apply_layernorm_1p and a.swiglu and a.num_experts is None and a.adam_beta2 == 0.95
    assert a.use_cpu_initialization is False                       # null: the default stays
    cfg = core_transformer_config_from_args(a)
    assert cfg.layernorm_epsilon == 0.00002 and cfg.layernorm_zero_centered_gamma and cfg.gated_linear_unit
    assert cfg.num_query_groups == 4 and cfg.sequence_parallel and not cfg.add_bias_linear and cfg.num_moe_experts is None


def test_launch_script_combinations_validate(monkeypatch):
    """Combinations the reference's own launch scripts use."""
    monkeypatch.setenv("WORLD_SIZE", "8")
    from mindspeed_b200.training.arguments import _layer_pattern, parse_args, validate_args
    base = ["--num-layers", "4", "--hidden-size", "64", "--num-attention-heads", "4", "--seq-length", "32",
            "--micro-batch-size", "1", "--vocab-size", "128"]
    assert _layer_pattern("([0]*1+[1]*3)") == [0, 1, 1, 1] and _layer_pattern("2") == 2
    with pytest.raises(AssertionError):
        _layer_pattern("__import__('os').getcwd()")
    a = validate_args(parse_args(args_list=base + ["--num-experts", "4", "--moe-layer-freq", "([0]*1+[1]*3)"]))
    assert a.moe_layer_freq == [0, 1, 1, 1]
    # data-parallel sharding of everything given together with the distributed optimizer
    a = validate_args(parse_args(args_list=base + ["--use-custom-fsdp", "--data-parallel-sharding-strategy", "optim_grads_params",
                                                   "--use-distributed-optimizer"]))
    assert a.layerzero and not a.use_distributed_optimizer
    # scheduler-placed recompute on top of full recompute flags: the scheduler takes over
    a = validate_args(parse_args(args_list=base + ["--pipeline-model-parallel-size", "2", "--recompute-in-advance",
                                                   "--recompute-granularity", "full", "--recompute-method", "block",
                                                   "--recompute-num-layers", "2"]))
    assert a.recompute_in_advance and a.recompute_granularity is None
    # forward/backward overlap of the DualPipeV schedule with a no-op layer
    a = validate_args(parse_args(args_list=base + ["--pipeline-model-parallel-size", "2", "--expert-model-parallel-size", "4",
                                                   "--num-experts", "8", "--moe-grouped-gemm", "--moe-token-dispatcher-type", "alltoall",
                                                   "--schedules-method", "dualpipev", "--moe-fb-overlap", "--noop-layers", "3",
                                                   "--global-batch-size", "16"]))
    assert a.moe_fb_overlap and a.noop_layers == [3]
