"""Seeded random weights for a model plan, and the writing of a model folder.

Matrices, the embedding and the convolution taps are normal(0, std); norm weights are 1;
the router's expert bias is normal(0, 0.1); other biases are 0.  The std is the tensor's own
where its part names one, else the plan's entry for the tensor's name (`ModelPlan.init_stds`,
by suffix), else the plan's default.  Tensors a checkpoint may leave out are left out.  Each tensor has its own generator seeded from
(seed, tensor name), so the values do not depend on the order of creation.  The reference has
no such mode (it needs a GGUF file).
"""
from __future__ import annotations

import hashlib
import json
import os

import torch

from ..parts.base import BIAS, NORM, ModelPlan, TensorSpec
from .safetensors_io import save_file


def _seed_for(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


def random_tensor(name: str, spec: TensorSpec, seed: int, std: float, norm_init: str = "ones",
                  device="cpu") -> torch.Tensor:
    """Float32 values of one tensor."""
    dev = torch.device(device)
    g = torch.Generator(device=dev)
    g.manual_seed(_seed_for(seed, name))
    if spec.role == NORM:
        if norm_init == "ones":
            return torch.ones(spec.shape, dtype=torch.float32, device=dev)
        return 1.0 + 0.1 * torch.randn(spec.shape, generator=g, dtype=torch.float32, device=dev)
    s = spec.std if spec.std is not None else std
    if spec.role == BIAS and spec.std is None:
        return torch.zeros(spec.shape, dtype=torch.float32, device=dev)
    return s * torch.randn(spec.shape, generator=g, dtype=torch.float32, device=dev)


def std_for(plan: ModelPlan, name: str) -> float:
    for suffix, std in plan.init_stds.items():
        if name.endswith(suffix):
            return float(std)
    return plan.init_std


def storage_dtype(spec: TensorSpec, dtype: torch.dtype) -> torch.dtype:
    """Biases are stored in 32-bit; everything else in the folder's dtype."""
    return torch.float32 if spec.role == BIAS else dtype


def checkpoint_name(plan: ModelPlan, canonical: str) -> str:
    """Name under which a tensor is written: the architecture's checkpoint spelling."""
    head = plan.names.get("head", "head")
    return canonical if canonical.startswith(head + ".") else "model." + canonical


def write_model_dir(config: dict, out_dir: str, seed: int, dtype: str = "bfloat16",
                    norm_init: str = "ones") -> str:
    """Writes config.json and model.safetensors for `config` with random weights."""
    from ..engine.model import Model
    from ..parts.base import BuildEnv
    from ..registry import plan_from_config

    dt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    plan = plan_from_config(config)
    model = Model(plan, BuildEnv(device=torch.device("cpu"), dtype=dt))
    tensors = {}
    for name, spec in model.tensor_specs().items():
        if spec.optional:
            continue
        t = random_tensor(name, spec, seed, std_for(plan, name), norm_init)
        tensors[checkpoint_name(plan, name)] = t.to(storage_dtype(spec, dt))
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(config, f, indent=1)
    save_file(tensors, os.path.join(out_dir, "model.safetensors"),
              metadata={"format": "pt", "seed": str(seed)})
    return out_dir
