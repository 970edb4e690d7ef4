"""Adaptor layer for code written against an external Megatron-LM checkout: symbol patching, dummy modules for missing
optional dependencies, deprecation helpers and the patch-file CLI.  The framework itself does not patch anything to
work - these tools exist so that user scripts and RL frameworks that import ``megatron.*`` can be pointed at it."""
from .patch_utils import Patch, PatchesManager
from .deprecate import AutoExecuteFunction, Deprecated, NoExecuteFunction
from .adaptor import patch_features, repatch

__all__ = ["Patch", "PatchesManager", "Deprecated", "AutoExecuteFunction", "NoExecuteFunction", "patch_features", "repatch"]
