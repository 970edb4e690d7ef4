"""``python -m mindspeed_b200.patching.cli -P | -R [--target DIR]``: apply (or revert) every ``*.patch`` shipped under
``mindspeed_b200/patching/patches`` to a source checkout with ``git apply``, checking first that all of them apply.
reference: mindspeed/run/run.py:59-128 (``mindspeed -P / -R``)."""
from __future__ import annotations

import argparse
import glob
import os
import subprocess
import sys
from typing import List

PATCH_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "patches")


def find_patches(directory: str = PATCH_DIR) -> List[str]:
    return sorted(glob.glob(os.path.join(directory, "*.patch")))


def _git_apply(target: str, patch: str, reverse: bool, check: bool) -> subprocess.CompletedProcess:
    cmd = ["git", "apply"] + (["--check"] if check else []) + (["-R"] if reverse else []) + [patch]
    return subprocess.run(cmd, cwd=target, capture_output=True, text=True)


def apply_all(target: str, reverse: bool = False, directory: str = PATCH_DIR) -> int:
    patches = find_patches(directory)
    if reverse:
        patches = patches[::-1]
    if not patches:
        print(f"no patch files under {directory}")
        return 0
    for p in patches:                                  # all-or-nothing: verify everything before touching anything
        r = _git_apply(target, p, reverse, check=True)
        if r.returncode != 0:
            print(f"{os.path.basename(p)} does not {'revert' if reverse else 'apply'} cleanly:\n{r.stderr}", file=sys.stderr)
            return 1
    for p in patches:
        r = _git_apply(target, p, reverse, check=False)
        if r.returncode != 0:
            print(r.stderr, file=sys.stderr)
            return 1
        print(f"{'reverted' if reverse else 'applied'} {os.path.basename(p)}")
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="mindspeed_b200.patching.cli")
    g = ap.add_mutually_exclusive_group(required=True)
    g.add_argument("-P", "--patch", action="store_true", help="apply the shipped patches")
    g.add_argument("-R", "--reverse", action="store_true", help="revert them")
    ap.add_argument("--target", default=os.getcwd(), help="root of the git checkout to patch")
    ap.add_argument("--patch-dir", default=PATCH_DIR)
    a = ap.parse_args(argv)
    return apply_all(a.target, reverse=a.reverse, directory=a.patch_dir)


if __name__ == "__main__":
    sys.exit(main())
