"""Checks a checkpoint against a model's tensor list and loads it.

All problems are gathered and reported in one error: tensors the model needs and the file
lacks, tensors in the file the model does not know, and shapes that differ.  (The reference
stops at the first missing tensor, src/dense.rs:85.)

Kept dtypes: operands of matrix products and the embedding are held in the compute dtype
(bfloat16 or float32); norm weights, convolution taps, router rows and biases are held in
float32 (an exact widening of bfloat16, and a tensor stored in 32-bit stays so); integer
tensors become int32.
"""
from __future__ import annotations

import torch

from ..parts.base import FLOAT_ROLES, TensorSpec
from .safetensors_io import WeightsError, open_checkpoint


def kept_dtype(spec: TensorSpec, stored: torch.dtype, compute: torch.dtype) -> torch.dtype:
    if not stored.is_floating_point:
        return torch.int32
    if spec.role in FLOAT_ROLES:
        return torch.float32
    return compute


def check_names(specs: dict[str, TensorSpec], found: dict[str, tuple[int, ...]], where: str) -> None:
    """`found`: canonical name -> shape in the file.  Raises one WeightsError listing everything."""
    missing = [n for n, s in specs.items() if n not in found and not s.optional]
    unexpected = [n for n in found if n not in specs]
    wrong = [(n, specs[n].shape, found[n]) for n in specs if n in found and tuple(found[n]) != tuple(specs[n].shape)]
    if not (missing or unexpected or wrong):
        return
    lines = [f"{where}: the checkpoint does not fit the model"]
    if missing:
        lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(sorted(missing)))
    if unexpected:
        lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(sorted(unexpected)))
    if wrong:
        lines.append(f"  wrong shapes ({len(wrong)}): " + "; ".join(
            f"{n}: expected {list(e)}, found {list(f)}" for n, e, f in sorted(wrong)))
    raise WeightsError("\n".join(lines))


def load_model_dir(model, model_dir: str) -> None:
    """Loads DIR/model.safetensors (or its shards) into `model` on its device."""
    plan, env = model.plan, model.env
    ckpt = open_checkpoint(model_dir)
    alias = plan.tensor_aliases or (lambda n: n)
    by_canonical: dict[str, tuple] = {}
    for name, ref in ckpt.items():
        by_canonical[alias(name)] = ref
    specs = model.tensor_specs()
    check_names(specs, {n: f.shape(k) for n, (f, k) in by_canonical.items()
                        if n in specs or n not in plan.unused_tensors}, model_dir)
    tensors: dict[str, torch.Tensor] = {}
    for name, spec in specs.items():
        if name not in by_canonical:
            continue
        f, k = by_canonical[name]
        t = f.tensor(k)
        tensors[name] = t.to(device=env.device, dtype=kept_dtype(spec, t.dtype, env.dtype))
    model.load(tensors)


def load_random(model, seed: int, norm_init: str = "ones", round_to: torch.dtype | None = torch.bfloat16) -> None:
    """Random weights made on the model's device (no file).  `round_to` rounds the values as a
    folder of that dtype would, so a float32 engine and a bfloat16 engine see the same numbers."""
    from .random_init import random_tensor, std_for, storage_dtype

    plan, env = model.plan, model.env
    tensors = {}
    for name, spec in model.tensor_specs().items():
        if spec.optional:
            continue
        t = random_tensor(name, spec, seed, std_for(plan, name), norm_init, device=env.device)
        if round_to is not None:
            t = t.to(storage_dtype(spec, round_to))
        tensors[name] = t.to(kept_dtype(spec, t.dtype, env.dtype))
    model.load(tensors)
