"""`wrap_with_flashdp_layers`: swap supported layers of a model for their DP twins.

Signature, selection rules, messages and errors follow flashdp/api/wrap_model.py:17-106:
* `target_modules` is mandatory and must be a non-empty subset of `dp_supported_modules`
  (ValueError otherwise, also when only `target_layers` is given -- :70-76);
* candidates are all module paths, or `target_layers` when given; `skip_layers` removes exact
  path matches only, so skipping a container does not skip its children (:169-182);
* a candidate is replaced when its type is one of `target_modules`; recursion stops there.
Beyond the reference: the twin also inherits the original layer's dtype, and subclasses of a
supported type are accepted (the reference's exact-type lookup raises KeyError for them, :198).
"""
from typing import List, Type

import torch.nn as nn

from ..layers.linear import DPLinear
from ..layers.layernorm import DPLayerNorm
from ..layers.transformers_conv1d import DPConv1D, Conv1D

dp_supported_modules = {
    nn.Linear: DPLinear,
    nn.LayerNorm: DPLayerNorm,
    Conv1D: DPConv1D,
}


def _module_paths(model):
    return [name for name, _ in model.named_modules() if name]


def _twin_class(module):
    for klass in type(module).__mro__:
        if klass in dp_supported_modules:
            return dp_supported_modules[klass]
    raise KeyError(type(module))


def _twin_kwargs(module):
    """Constructor arguments of the DP twin, read off the original layer (:109-137).  A Linear
    without bias passes bias=None, which the twin reads as "no bias"."""
    if isinstance(module, nn.Linear):
        return dict(in_features=module.in_features, out_features=module.out_features, bias=module.bias)
    if isinstance(module, nn.LayerNorm):
        return dict(normalized_shape=module.normalized_shape, eps=module.eps,
                    elementwise_affine=module.elementwise_affine)
    if isinstance(module, Conv1D):
        return dict(nf=module.nf, nx=module.weight.shape[0])
    raise NotImplementedError(f"Unsupported module type: {type(module)}")


def _replace(parent, prefix, chosen, kinds, hyper):
    for name, child in list(parent.named_children()):
        path = f"{prefix}.{name}" if prefix else name
        if path in chosen and isinstance(child, kinds) and not getattr(child, "dp", False):
            twin = _twin_class(child)(**_twin_kwargs(child), **hyper)
            first = next(child.parameters(), None)
            if first is not None:
                twin = twin.to(device=first.device, dtype=first.dtype)
            twin.load_state_dict(child.state_dict())
            twin.train(child.training)
            setattr(parent, name, twin)
        else:
            _replace(child, path, chosen, kinds, hyper)


def wrap_with_flashdp_layers(model, target_modules: List[Type[nn.Module]] = None,
                             target_layers: List[str] = None, skip_layers: List[str] = None,
                             priority_to_target: bool = False, feedback: bool = True, C=1.0,
                             noise_multiplier=1.0, clamp_value=1.0) -> nn.Module:
    """Replace the selected nn.Linear / nn.LayerNorm / transformers Conv1D layers of `model` by
    DPLinear / DPLayerNorm / DPConv1D carrying (C, noise_multiplier, clamp_value); returns `model`.

    Clip rule of every wrapped parameter tensor: g_b * min(C / (||g_b|| + 1e-10), clamp_value),
    averaged over the batch, plus N(0, (noise_multiplier/sqrt(B))^2).
    """
    print("Wrapping the model with FlashDP...")
    if target_modules is None and target_layers is None:
        raise ValueError("Either target_modules or target_layers must be specified.")
    if target_modules is None or len(target_modules) == 0:
        raise ValueError("target_modules cannot be empty and must be list of torch.nn.Module.")
    if not all(m in dp_supported_modules for m in target_modules):
        raise ValueError(f"target_modules must be among {dp_supported_modules.keys()}, got {target_modules}")
    target_layers = list(target_layers or [])
    skip_layers = list(skip_layers or [])

    paths = _module_paths(model)
    chosen = (set(target_layers) if target_layers else set(paths)) - set(skip_layers)

    used = {type(m) for m in model.modules()}
    for kind in target_modules:
        if not any(issubclass(u, kind) for u in used):
            print(f"Warning: Module type '{kind.__name__}' specified in target_modules is not used in the model.")
    for name in skip_layers:
        if name not in paths:
            print(f"Warning: '{name}' specified in skip_layers does not exist in the model.")

    _replace(model, "", chosen, tuple(target_modules),
             dict(C=C, clamp_value=clamp_value, noise_multiplier=noise_multiplier))

    if feedback:
        for label, names in (("Wrapped", sorted(chosen)), ("Skipped", skip_layers)):
            print(f"Layers {label}: {', '.join(names)}" if names else f"No layers {label}.")
    print("Model wrapped with FlashDP.")
    return model
