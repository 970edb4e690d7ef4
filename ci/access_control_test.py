"""Gate used by CI: decide from the list of changed files whether the (slow) GPU suite has to run.
Usage: git diff --name-only origin/main... | python ci/access_control_test.py"""
import sys

GPU_RELEVANT = ("mindspeed_b200/csrc/", "mindspeed_b200/ops/", "mindspeed_b200/parallel/", "mindspeed_b200/models/", "bench.py",
                "__graft_entry__.py", "tests/test_")


def needs_gpu_suite(paths):
    return any(p.startswith(GPU_RELEVANT) for p in paths)


if __name__ == "__main__":
    changed = [l.strip() for l in sys.stdin if l.strip()]
    print("gpu" if needs_gpu_suite(changed) else "cpu-only")
