"""YAML argument files (reference: mindspeed/yaml_arguments.py:6-25 wrapping Megatron's
``core_transformer_config_from_yaml``).  Keys may be nested one level (``model:``, ``training:`` ...);
dashes and underscores are interchangeable."""
import yaml


def load_yaml(path, args):
    with open(path) as f:
        doc = yaml.safe_load(f) or {}
    flat = {}
    for k, v in doc.items():
        if isinstance(v, dict):
            flat.update(v)
        else:
            flat[k] = v
    for k, v in flat.items():
        setattr(args, k.replace("-", "_"), v)
    return args


def core_transformer_config_from_yaml(args, transfomer_key="language_model"):
    from .arguments import core_transformer_config_from_args
    return core_transformer_config_from_args(args)
