"""YAML argument files (``--yaml-cfg``; reference: mindspeed/yaml_arguments.py:6-25 wrapping Megatron's
``core_transformer_config_from_yaml``).

A file is a mapping of argument names to values, optionally with the sections Megatron's YAML files use -
``language_model:`` (transformer configuration), ``model_parallel:`` (parallel sizes and options) - whose keys are the
configuration's field names.  Sections are flattened; dashes and underscores are interchangeable; a configuration field
whose command-line argument has another name is translated (``layernorm_epsilon`` -> ``norm_epsilon``,
``num_moe_experts`` -> ``num_experts``, ``activation_func: swiglu`` -> ``swiglu`` ...).  A ``null`` value leaves the
argument at what the command line (or its default) gave it; keys that name no argument are kept on the namespace, as
Megatron does, so later stages may read them.
"""
import yaml

# configuration field -> (argument, transform)
_RENAMES = {
    "layernorm_epsilon": ("norm_epsilon", None),
    "layernorm_zero_centered_gamma": ("apply_layernorm_1p", None),
    "num_moe_experts": ("num_experts", None),
    "virtual_pipeline_model_parallel_size": ("virtual_pipeline_model_parallel_size", None),
    "gradient_accumulation_fusion": ("gradient_accumulation_fusion", None),
    "fp8": ("fp8_format", None),
}


def _activation(args, name):
    name = (name or "gelu").lower()
    if name in ("swiglu", "silu"):
        args.swiglu = True
    elif name in ("squared_relu", "squaredrelu"):
        args.squared_relu = True
    elif name not in ("gelu",):
        raise ValueError(f"--yaml-cfg: unknown activation_func {name!r}")


def load_yaml(path, args):
    with open(path) as f:
        doc = yaml.safe_load(f) or {}
    flat = {}
    for k, v in doc.items():
        if isinstance(v, dict) and k in ("language_model", "model_parallel", "model", "training", "data", "optimizer"):
            flat.update(v)
        else:
            flat[k] = v
    for k, v in flat.items():
        k = k.replace("-", "_")
        if k == "activation_func":
            _activation(args, v)
            continue
        k, fn = _RENAMES.get(k, (k, None))
        if v is None and hasattr(args, k):
            continue                                   # null: keep the command line's / the default value
        setattr(args, k, fn(v) if fn else v)
    return args


def core_transformer_config_from_yaml(args, transfomer_key="language_model"):
    from .arguments import core_transformer_config_from_args
    return core_transformer_config_from_args(args)
