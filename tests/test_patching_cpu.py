"""Patch engine, deprecation helpers, adaptor entry and the patch CLI."""
import os
import subprocess
import sys
import types
import warnings

import pytest


def test_replace_wrap_alias_and_remove():
    from mindspeed_b200.patching import PatchesManager
    mod = types.ModuleType("zz_fake_pkg")
    mod.f = lambda x: x + 1
    sys.modules["zz_fake_pkg"] = mod
    user = types.ModuleType("zz_user")
    user.f = mod.f                                           # `from zz_fake_pkg import f`
    sys.modules["zz_user"] = user
    orig = mod.f

    def double_wrapper(fn):
        return lambda x: 2 * fn(x)

    def plus_ten_decorator(fn):
        return lambda x: fn(x) + 10

    PatchesManager.register_patch("zz_fake_pkg.f", double_wrapper)
    PatchesManager.register_patch("zz_fake_pkg.f", plus_ten_decorator)
    PatchesManager.register_patch("zz_missing_dep.sub.thing", lambda: "stub", create_dummy=True)
    PatchesManager.apply_patches()
    assert mod.f(1) == 14 and user.f(1) == 14               # wrappers stack in order; the alias was re-bound
    import zz_missing_dep.sub as s
    assert s.thing() == "stub" and getattr(sys.modules["zz_missing_dep"], "__dummy__", False)
    with pytest.raises(RuntimeError):
        PatchesManager.register_patch("zz_fake_pkg.g", lambda: 1)
        PatchesManager.register_patch("zz_fake_pkg.g", lambda: 2)
    PatchesManager.patches.pop("zz_fake_pkg.g")
    PatchesManager.remove_patches()
    assert mod.f is orig and user.f is orig
    for k in ("zz_fake_pkg", "zz_user", "zz_missing_dep", "zz_missing_dep.sub"):
        sys.modules.pop(k, None)


def test_deprecated_and_side_effect_switch():
    from mindspeed_b200.patching import AutoExecuteFunction, Deprecated, NoExecuteFunction

    @Deprecated("2099-01-01", ["old_api"], "use new_api instead.")
    def old(x):
        return x * 3

    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        assert old(2) == 6 and old(3) == 9
    assert len(w) == 1 and "2099-01-01" in str(w[0].message) and "new_api" in str(w[0].message)
    ran = []
    a = AutoExecuteFunction(ran.append, 1)
    with NoExecuteFunction():
        b = AutoExecuteFunction(ran.append, 2)
    assert ran == [1] and a.executed and not b.executed
    b.run()
    assert ran == [1, 2]


def test_adaptor_installs_megatron_names():
    code = ("from mindspeed_b200.patching import patch_features\n"
            "patch_features()\n"
            "import megatron.core.parallel_state as ps\n"
            "from megatron.core.tensor_parallel.layers import ColumnParallelLinear\n"
            "from megatron.training import pretrain\n"
            "import mindspeed_b200.parallel.parallel_state as mine\n"
            "assert ps is mine and callable(pretrain) and ColumnParallelLinear.__module__.startswith('mindspeed_b200')\n"
            "from apex.optimizers import FusedAdam\n"
            "import torch\n"
            "FusedAdam([torch.nn.Parameter(torch.zeros(2))], lr=0.1)\n"
            "print('OK')\n")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=root, timeout=300)
    assert r.returncode == 0 and "OK" in r.stdout, r.stderr[-2000:]


def test_optional_dependency_stand_ins_compute_what_the_packages_compute():
    import torch
    from mindspeed_b200.patching import compat as C
    g = torch.Generator().manual_seed(0)
    ts = [torch.randn(5, 3, generator=g), torch.randn(7, generator=g)]
    flag = torch.zeros(1, dtype=torch.int32)
    total, per = C.multi_tensor_applier(C.multi_tensor_l2norm, flag, [ts], True)
    assert torch.allclose(total, torch.cat([t.flatten() for t in ts]).norm().reshape(1))
    assert torch.allclose(per, torch.stack([t.norm() for t in ts]))
    out = [torch.empty_like(t) for t in ts]
    C.multi_tensor_applier(C.multi_tensor_scale, flag, [ts, out], 0.5)
    assert all(torch.allclose(o, t * 0.5) for o, t in zip(out, ts)) and int(flag) == 0
    C.multi_tensor_applier(C.multi_tensor_scale, flag, [[torch.tensor([1.0, float("inf")])], [torch.empty(2)]], 1.0)
    assert int(flag) == 1                                              # overflow seen: the caller skips the step
    flag.zero_()
    C.multi_tensor_applier(C.multi_tensor_axpby, flag, [ts, ts, out], 2.0, -1.0)
    assert all(torch.allclose(o, t) for o, t in zip(out, ts))
    # multi_tensor_adam against torch.optim.AdamW / Adam for three steps
    for mode, ref_cls in ((1, torch.optim.AdamW), (0, torch.optim.Adam)):
        p = torch.nn.Parameter(ts[0].clone())
        ref = ref_cls([p], lr=1e-2, betas=(0.9, 0.99), eps=1e-8, weight_decay=0.1)
        q, m, v = ts[0].clone(), torch.zeros_like(ts[0]), torch.zeros_like(ts[0])
        for step in range(1, 4):
            grad = torch.randn(ts[0].shape, generator=g)
            p.grad = grad.clone()
            ref.step()
            C.multi_tensor_applier(C.multi_tensor_adam, flag, [[grad], [q], [m], [v]], 1e-2, 0.9, 0.99, 1e-8, step, mode, True, 0.1)
        assert torch.allclose(q, p.detach(), atol=1e-6), mode
    # count of zero gradient entries (a shared parameter is counted once)
    a, b = torch.nn.Parameter(torch.zeros(4)), torch.nn.Parameter(torch.zeros(3))
    a.grad, b.main_grad = torch.tensor([0.0, 1.0, 0.0, 2.0]), torch.tensor([0.0, 0.0, 3.0])
    b.grad = None
    assert C.count_zeros_fp32([a, b]) == 4.0
    b.shared = True
    assert C.count_zeros_fp32([a, b]) == 2.0
    # flash-attn interface layouts on this framework's attention
    from mindspeed_b200.ops.attention import attention_ref
    q4, k4, v4 = (torch.randn(2, 9, 2, 8, generator=g) for _ in range(3))
    o = C.flash_attn_func(q4, k4, v4, causal=True)
    assert torch.allclose(o, attention_ref(q4.transpose(0, 1), k4.transpose(0, 1), v4.transpose(0, 1), causal=True).transpose(0, 1), atol=1e-5)
    qp, kp, vp = (torch.randn(9, 2, 8, generator=g) for _ in range(3))
    cu = torch.tensor([0, 4, 9])
    ov = C.flash_attn_varlen_func(qp, kp, vp, cu, cu, 5, 5, causal=True)
    first = attention_ref(qp[:4].unsqueeze(1), kp[:4].unsqueeze(1), vp[:4].unsqueeze(1), causal=True).squeeze(1)
    assert ov.shape == qp.shape and torch.allclose(ov[:4], first, atol=1e-5)
    # norm stand-ins
    paths = dict(C.optional_dependency_stubs())
    ln = paths["apex.normalization.FusedLayerNorm"](8)
    x = torch.randn(3, 8, generator=g)
    assert torch.allclose(ln(x), torch.nn.functional.layer_norm(x, (8,)), atol=1e-5)
    rn = paths["apex.normalization.MixedFusedRMSNorm"]((8,), eps=1e-6)
    assert torch.allclose(rn(x), x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6), atol=1e-5)
    assert {"transformer_engine.pytorch.Linear", "amp_C.multi_tensor_adam", "apex.optimizers.FusedSGD",
            "flash_attn.flash_attn_interface.flash_attn_unpadded_func"} <= set(paths)


def test_patch_cli_roundtrip(tmp_path):
    from mindspeed_b200.patching import cli
    repo = tmp_path / "repo"
    repo.mkdir()
    subprocess.run(["git", "init", "-q"], cwd=repo, check=True)
    (repo / "a.txt").write_text("one\ntwo\n")
    pd = tmp_path / "patches"
    pd.mkdir()
    (pd / "0001-change.patch").write_text("--- a/a.txt\n+++ b/a.txt\n@@ -1,2 +1,2 @@\n one\n-two\n+TWO\n")
    assert cli.main(["-P", "--target", str(repo), "--patch-dir", str(pd)]) == 0
    assert (repo / "a.txt").read_text() == "one\nTWO\n"
    assert cli.main(["-P", "--target", str(repo), "--patch-dir", str(pd)]) == 1     # already applied: refused, untouched
    assert cli.main(["-R", "--target", str(repo), "--patch-dir", str(pd)]) == 0
    assert (repo / "a.txt").read_text() == "one\ntwo\n"
