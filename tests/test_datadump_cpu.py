import torch
import torch.nn as nn

from mindspeed_b200.utils.datadump import compare_dumps, install_data_dump


def test_dump_and_compare(tmp_path):
    torch.manual_seed(0)
    net = nn.Sequential(nn.Linear(8, 8), nn.Tanh(), nn.Linear(8, 2))
    x = torch.randn(4, 8)

    def run(d, perturb=0.0):
        dd = install_data_dump(net, str(d), steps=[1])
        for step in range(3):
            y = net(x + (perturb if step == 1 else 0.0))
            y.sum().backward()
            dd.end_step()
        dd.remove()
        return dd

    a = run(tmp_path / "a")
    assert {r["kind"] for r in a.index} == {"fwd", "bwd"} and all(r["module"] in ("0", "1", "2") for r in a.index)
    assert (tmp_path / "a" / "step1" / "rank0" / "0.fwd.0.pt").exists() and not (tmp_path / "a" / "step0").exists()
    run(tmp_path / "b")
    assert compare_dumps(str(tmp_path / "a"), str(tmp_path / "b")) == []
    run(tmp_path / "c", perturb=0.1)
    diff = compare_dumps(str(tmp_path / "a"), str(tmp_path / "c"))
    assert diff and any(p.endswith("0.fwd.0.pt") for p, _ in diff)
