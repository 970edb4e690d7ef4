"""Ordered application of features (reference: mindspeed/features_manager/features_manager.py:7-67).

Composition rule kept from the reference's patch manager (mindspeed/patch_utils.py:70-78,119-124):
one *replacement* per slot unless forced, any number of *wrappers* applied in registration order.
Here a "slot" is a named hook (e.g. ``"tp_comm_ops"``, ``"schedule"``) that model code reads.
"""
from __future__ import annotations

from typing import Callable, Dict, List


class FeaturesManager:
    def __init__(self, features: List):
        self.features = list(features)
        self.slots: Dict[str, object] = {}
        self.wrappers: Dict[str, List[Callable]] = {}
        self._owners: Dict[str, str] = {}

    # ---- args ----
    def register_features_args(self, parser):
        for f in self.features:
            f.register_args(parser)

    def pre_validate_features_args(self, args):
        for f in self.features:
            if f.is_need_apply(args):
                f.pre_validate_args(args)

    def post_validate_features_args(self, args):
        for f in self.features:
            if f.is_need_apply(args):
                f.post_validate_args(args)

    def validate_features_args(self, args):
        for f in self.features:
            if f.is_need_apply(args):
                f.validate_args(args)

    # ---- configuration ----
    def set_slot(self, name: str, value, owner: str = "", force: bool = False):
        if name in self.slots and not force and self._owners.get(name) != owner:
            raise RuntimeError(f"slot '{name}' already set by {self._owners.get(name)}; {owner} must use force=True")
        self.slots[name] = value
        self._owners[name] = owner

    def add_wrapper(self, name: str, wrapper: Callable):
        self.wrappers.setdefault(name, []).append(wrapper)

    def resolve(self, name: str, default=None):
        v = self.slots.get(name, default)
        for w in self.wrappers.get(name, []):
            v = w(v)
        return v

    def apply_features_pre_configure(self, args):
        for f in self.features:
            if f.is_need_apply(args):
                f.pre_configure(self, args)

    def apply_features(self, args):
        for f in self.features:
            if f.is_need_apply(args):
                f.configure(self, args)
        return self

    def active(self, args) -> List[str]:
        return [f.feature_name for f in self.features if f.is_need_apply(args)]
