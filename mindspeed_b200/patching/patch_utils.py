"""Replace or decorate any dotted symbol, creating dummy modules on the way when a dependency is not installed.

  PatchesManager.register_patch("pkg.mod.func", new_func)            replace
  PatchesManager.register_patch("pkg.mod.func", some_wrapper)        decorate: a patch whose name ends in "wrapper" or
                                                                     "decorator" is applied to the current value; several
                                                                     stack in registration order
  PatchesManager.register_patch("apex.optimizers.FusedAdam", cls, create_dummy=True)
                                                                     missing parents become empty modules in sys.modules
  PatchesManager.apply_patches()                                     applies everything once; every module that had
                                                                     imported the old object under any name is re-bound
  PatchesManager.remove_patches()                                    restores the originals
reference: mindspeed/patch_utils.py:43-210 (Patch, parse_path, MindSpeedPatchesManager).
"""
from __future__ import annotations

import importlib
import sys
import types
from typing import Callable, Dict, List, Optional


def _dummy_raiser(name):
    def fn(*a, **kw):
        raise RuntimeError(f"'{name}' is a placeholder created for a missing dependency and was called")
    fn.__name__ = name.rsplit(".", 1)[-1]
    return fn


class Patch:
    def __init__(self, orig_path: str, new_obj, create_dummy: bool = False):
        if "." not in orig_path:
            raise ValueError("patch target must be a dotted path module.attr")
        self.path = orig_path
        self.module_path, self.attr = orig_path.rsplit(".", 1)
        self.create_dummy = create_dummy
        self.replacement = None
        self.wrappers: List[Callable] = []
        self.applied = False
        self.had_orig = False
        self.orig = None
        self.module = None
        self.add(new_obj)

    @staticmethod
    def _is_wrapper(obj) -> bool:
        n = getattr(obj, "__name__", "")
        return n.endswith("wrapper") or n.endswith("decorator")

    def add(self, new_obj, force: bool = False):
        if new_obj is None:
            return
        if self._is_wrapper(new_obj):
            self.wrappers.append(new_obj)
        else:
            if self.replacement is not None and not force:
                raise RuntimeError(f"a replacement for {self.path} is already registered; pass force_patch=True to override")
            self.replacement = new_obj

    @staticmethod
    def parse_path(module_path: str, attr: Optional[str], create_dummy: bool):
        """Import ``module_path`` piece by piece; missing pieces become dummy modules when allowed.  Returns
        (module, current attribute value or None, attribute existed)."""
        parts = module_path.split(".")
        mod = None
        for i in range(1, len(parts) + 1):
            name = ".".join(parts[:i])
            if name in sys.modules:
                mod = sys.modules[name]
                continue
            try:
                mod = importlib.import_module(name)
            except ImportError:
                parent = sys.modules.get(".".join(parts[:i - 1])) if i > 1 else None
                if parent is not None and hasattr(parent, parts[i - 1]) and not isinstance(getattr(parent, parts[i - 1]), types.ModuleType):
                    # the "module" is really a class / namespace object: patch inside it
                    mod = getattr(parent, parts[i - 1])
                    continue
                if not create_dummy:
                    raise
                mod = types.ModuleType(name)
                mod.__dummy__ = True
                mod.__path__ = []           # lets `import a.b.c` treat the placeholder as a package
                sys.modules[name] = mod
                if parent is not None:
                    setattr(parent, parts[i - 1], mod)
        if attr is None:
            return mod, None, False
        if hasattr(mod, attr):
            return mod, getattr(mod, attr), True
        return mod, None, False

    def apply(self):
        if self.applied:
            return
        self.module, self.orig, self.had_orig = self.parse_path(self.module_path, self.attr, self.create_dummy)
        if not self.had_orig and not self.create_dummy and self.replacement is None:
            raise AttributeError(f"{self.path} does not exist and nothing replaces it")
        final = self.replacement if self.replacement is not None else (self.orig if self.had_orig else _dummy_raiser(self.path))
        for w in self.wrappers:
            final = w(final)
        setattr(self.module, self.attr, final)
        if isinstance(final, types.ModuleType):
            self._prev_sys_module = sys.modules.get(self.path)
            sys.modules[self.path] = final   # `import pkg.mod.name` must find the installed module too
        # re-bind aliases: `from pkg.mod import func` elsewhere holds the old object under the same name
        if self.had_orig and not isinstance(self.orig, (int, float, str, bool, type(None))):
            for m in list(sys.modules.values()):
                if m is None or m is self.module:
                    continue
                d = getattr(m, "__dict__", None)
                if d is None:
                    continue
                try:
                    if d.get(self.attr) is self.orig:
                        setattr(m, self.attr, final)
                except Exception:
                    continue
        self.final = final
        self.applied = True

    def remove(self):
        if not self.applied:
            return
        if isinstance(self.final, types.ModuleType) and sys.modules.get(self.path) is self.final:
            if getattr(self, "_prev_sys_module", None) is not None:
                sys.modules[self.path] = self._prev_sys_module
            else:
                sys.modules.pop(self.path, None)
        if self.had_orig:
            for m in list(sys.modules.values()):
                d = getattr(m, "__dict__", None)
                if d is not None and d.get(self.attr) is self.final:
                    try:
                        setattr(m, self.attr, self.orig)
                    except Exception:
                        pass
            setattr(self.module, self.attr, self.orig)
        else:
            try:
                delattr(self.module, self.attr)
            except AttributeError:
                pass
        self.applied = False


class PatchesManager:
    patches: Dict[str, Patch] = {}

    @classmethod
    def register_patch(cls, orig_path: str, new_obj=None, force_patch: bool = False, create_dummy: bool = False):
        p = cls.patches.get(orig_path)
        if p is None:
            cls.patches[orig_path] = Patch(orig_path, new_obj, create_dummy)
        else:
            p.create_dummy = p.create_dummy or create_dummy
            p.add(new_obj, force_patch)

    @classmethod
    def apply_patches(cls):
        for p in cls.patches.values():
            p.apply()

    @classmethod
    def remove_patches(cls):
        for p in reversed(list(cls.patches.values())):
            p.remove()
        cls.patches = {}
