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
