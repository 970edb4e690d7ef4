"""Feature = (flags, validation, configuration).

Each capability is a ``Feature`` subclass that owns its command-line flags, validates them around
the core validation (pre -> core -> post -> validate) and, instead of monkey-patching another
framework, *configures* this one: it selects back ends, layer specs and schedules in ``configure``.
Life-cycle and gating follow the reference's ``MindSpeedFeature``
(mindspeed/features_manager/feature.py:9-76): a feature is active when its
``optimization_level`` is <= ``--optimization-level`` and its flag is truthy, or always when it is
a level-0 default feature.
"""
from __future__ import annotations

import argparse
from typing import List, Optional


class Feature:
    def __init__(self, feature_name: str, optimization_level: int = 2):
        self.feature_name = feature_name.strip().replace("-", "_")
        self.optimization_level = optimization_level
        self.default_patches = optimization_level == 0

    # ---- life-cycle hooks ----
    def register_args(self, parser: argparse.ArgumentParser):
        pass

    def pre_validate_args(self, args):
        pass

    def validate_args(self, args):
        pass

    def post_validate_args(self, args):
        pass

    def pre_configure(self, manager, args):
        """Runs before model construction for every active feature (the reference's pre_register_patches)."""

    def configure(self, manager, args):
        """Select back ends / specs / schedules (the reference's register_patches)."""

    # ---- helpers ----
    def is_need_apply(self, args) -> bool:
        lvl = getattr(args, "optimization_level", 2)
        return (self.optimization_level <= lvl and bool(getattr(args, self.feature_name, None))) or self.default_patches

    def incompatible_check(self, args, other: str):
        if getattr(args, self.feature_name, None) and getattr(args, other, None):
            raise AssertionError(f"{self.feature_name} and {other} are incompatible.")

    def dependency_check(self, args, other: str):
        if getattr(args, self.feature_name, None) and not getattr(args, other, None):
            raise AssertionError(f"{self.feature_name} requires {other}.")

    @staticmethod
    def add_parser_argument_choices_value(parser, argument_name: str, new_choice):
        for action in parser._actions:
            if isinstance(action, argparse._ArgumentGroup):
                continue
            if argument_name in action.option_strings and action.choices is not None and new_choice not in action.choices:
                action.choices.append(new_choice)


def add_arg(group, *names, **kw):
    """``add_argument`` that tolerates a flag registered by an earlier feature."""
    try:
        group.add_argument(*names, **kw)
    except argparse.ArgumentError:
        pass
