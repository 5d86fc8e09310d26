"""Weights by tensor name: one check of a model folder against what the model's parts ask
for, and the copy to the device.

The reference binds tensors by name and validates every shape
(src/model.rs:759-905, :907-1088), reports a missing tensor by its name
(src/model.rs:1653-1657), fails closed on tensors it does not expect
(src/model.rs:829-842) and refuses a model without an output matrix unless the embeddings
are tied (src/model_source.rs:253-260). Here all findings come in one error.
"""
from __future__ import annotations

import torch

from ..errors import WeightsError

_FLOATS = (torch.float32, torch.bfloat16, torch.float16)


def check_tensors(specs: dict, names_shapes_dtypes: dict, *, tolerated: tuple = ()) -> None:
    """``specs``: name -> TensorSpec wanted. ``names_shapes_dtypes``: name -> (shape, dtype)
    found. Raises one ``WeightsError`` that lists missing and unexpected tensors and wrong
    shapes. ``tolerated`` names may be present without being wanted (a stored ``lm_head``
    of a model that ties its embeddings)."""
    missing = sorted(n for n in specs if n not in names_shapes_dtypes)
    unexpected = sorted(n for n in names_shapes_dtypes if n not in specs and n not in tolerated)
    wrong, other = [], []
    for n, spec in specs.items():
        if n in names_shapes_dtypes:
            shape, dtype = names_shapes_dtypes[n]
            if tuple(shape) != tuple(spec.shape):
                wrong.append((n, spec.shape, shape))
            if dtype not in _FLOATS:
                other.append(f"{n}: stored as {dtype}, expected a floating-point type")
    if missing or unexpected or wrong or other:
        raise WeightsError(missing, unexpected, wrong, other)


