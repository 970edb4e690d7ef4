from .feature import Feature  # noqa: F401
from .manager import FeaturesManager  # noqa: F401
from .registry import create_features_list  # noqa: F401

_MANAGER = None


def get_features_manager() -> FeaturesManager:
    global _MANAGER
    if _MANAGER is None:
        _MANAGER = FeaturesManager(create_features_list())
    return _MANAGER


def set_features_manager(m):
    global _MANAGER
    _MANAGER = m
