"""Leaf serializers for tensors and arrays.

A tensor is saved as a detached clone under its own key; on load the SHAPE must match the
template and dtype / device are taken from the template (a checkpoint written in fp32 on one
device restores into a bf16 template on another).  ``PerGroup`` and tree definitions are
template-restored: they describe structure, not run state.

Parity: packages/opaque-engine/src/opaque/api/engine/serialization/_structural.py:57-108.
"""
from __future__ import annotations

import numpy as np
import torch

from . import register_serializer, register_template_restored


def _save_tensor(t: torch.Tensor):
    return {"": t.detach().clone()}


def _load_tensor(template: torch.Tensor, sd):
    if "" not in sd:
        return template
    v = sd[""]
    v = torch.as_tensor(v)
    if tuple(v.shape) != tuple(template.shape):
        raise ValueError(f"shape mismatch: saved {tuple(v.shape)} vs template {tuple(template.shape)}")
    out = v.to(device=template.device, dtype=template.dtype)
    if isinstance(template, torch.nn.Parameter):
        return torch.nn.Parameter(out, requires_grad=template.requires_grad)
    return out


def _load_array(template: np.ndarray, sd):
    if "" not in sd:
        return template
    v = np.asarray(sd[""])
    if v.shape != template.shape:
        raise ValueError(f"shape mismatch: saved {v.shape} vs template {template.shape}")
    return v.astype(template.dtype)


register_serializer(torch.Tensor, _save_tensor, _load_tensor)
register_serializer(np.ndarray, lambda a: {"": a.copy()}, _load_array)


def _register_structural():
    from ..pytree import TreeDef
    from ..types import PerGroup
    register_template_restored(TreeDef)
    register_serializer(PerGroup, lambda p: {f"values.{k}": v for k, v in p.values.items()},
                        lambda t, sd: PerGroup(t.groups, {k: sd.get(f"values.{k}", v) for k, v in t.values.items()}))


_register_structural()
