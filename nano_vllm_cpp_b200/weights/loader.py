"""Binding weights to a model by tensor name.

``check_tensors`` compares what a model needs with what a folder holds and raises one
``WeightsError`` that lists every missing tensor, every unexpected tensor and every wrong
shape.  (The reference checks element counts of a few tensors only, lets missing norm weights
default to one and ties the head silently when ``lm_head.weight`` is absent:
src/model.cpp:603-632; none of that is kept.)

Storage types on the device: in a float32 run everything is widened to float32.  In a
bfloat16 run a tensor stored as BF16 stays bfloat16, F16 is converted to bfloat16, and a
tensor stored in 32 bits stays float32 (the products then take the plain kernel for it);
integer tensors become int32.  Small vectors (norm weights, biases) are held in float32 in
both runs, which is exact for either storage type.
"""
from __future__ import annotations

import json
import os

import torch

from .random_values import host_values, tensor_key
from .safetensors_io import SafetensorsFolder, save_safetensors


class WeightsError(ValueError):
    pass


def check_tensors(specs: dict, found: dict) -> None:
    """``specs``: name -> TensorSpec; ``found``: name -> shape tuple."""
    missing = [n for n in specs if n not in found]
    unexpected = [n for n in found if n not in specs]
    wrong = [(n, tuple(specs[n].shape), tuple(found[n])) for n in specs
             if n in found and tuple(found[n]) != tuple(specs[n].shape)]
    if not (missing or unexpected or wrong):
        return
    lines = [f"the weights do not fit the model: {len(missing)} missing, {len(unexpected)} unexpected, "
             f"{len(wrong)} with a wrong shape"]

    def listing(title, items, fmt):
        if not items:
            return
        lines.append(f"{title} ({len(items)}):")
        for it in items[:50]:
            lines.append("  " + fmt(it))
        if len(items) > 50:
            lines.append(f"  ... and {len(items) - 50} more")

    listing("missing tensors", sorted(missing), str)
    listing("unexpected tensors", sorted(unexpected), str)
    listing("wrong shapes", sorted(wrong), lambda w: f"{w[0]}: expected {list(w[1])}, found {list(w[2])}")
    raise WeightsError("\n".join(lines))


def _device_dtype(stored: torch.dtype, kind: str, run_dtype: torch.dtype) -> torch.dtype:
    if not stored.is_floating_point:
        return torch.int32
    if run_dtype == torch.float32 or kind == "vector":
        return torch.float32
    if stored in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


class FolderSource:
    """Tensors of a model folder, moved to the device in the run's storage types."""

    def __init__(self, folder: SafetensorsFolder, specs: dict, device, run_dtype: torch.dtype):
        self.folder, self.specs, self.device, self.run_dtype = folder, specs, device, run_dtype

    def has(self, name: str) -> bool:
        return name in self.folder

    def get(self, name: str) -> torch.Tensor:
        t = self.folder.load(name)
        kind = self.specs[name].kind if name in self.specs else "matrix"
        return t.to(device=self.device, dtype=_device_dtype(t.dtype, kind, self.run_dtype))


class RandomSource:
    """Random tensors whose every value is a function of (seed, tensor name, element index): the order of
    requests, the presence of other tensors and the device that draws them do not matter, and a tensor drawn on
    the GPU has the bits of the one drawn on the CPU (see ``random_values``).  Matrices and biases are N(0, std);
    norm weights are 1 + N(0, norm_std).  Values are made in float32 and rounded once to ``store_dtype``."""

    def __init__(self, specs: dict, seed: int, std: float, norm_std: float, device, store_dtype: torch.dtype,
                 run_dtype: torch.dtype | None = None):
        self.specs, self.seed, self.std, self.norm_std = specs, seed, std, norm_std
        self.device, self.store_dtype = torch.device(device), store_dtype
        self.run_dtype = run_dtype or store_dtype

    def has(self, name: str) -> bool:
        return name in self.specs

    def _draw(self, name: str, shape, mean: float, std: float) -> torch.Tensor:
        n = 1
        for d in shape:
            n *= int(d)
        key = tensor_key(self.seed, name)
        if self.device.type == "cuda":
            from ..csrc import ops
            t = torch.empty(tuple(shape), dtype=self.store_dtype, device=self.device)
            ops.random_fill(t, key, mean, std)
            return t
        t = torch.from_numpy(host_values(key, n, mean, std)).reshape(tuple(shape))
        return t.to(self.store_dtype)

    def stored(self, name: str) -> torch.Tensor:
        spec = self.specs[name]
        if spec.init == "zeros":
            return torch.zeros(spec.shape, dtype=self.store_dtype, device=self.device)
        if spec.init == "ones":
            if self.norm_std > 0:
                return self._draw(name, spec.shape, 1.0, self.norm_std)
            return torch.ones(spec.shape, dtype=self.store_dtype, device=self.device)
        return self._draw(name, spec.shape, 0.0, self.std)

    def get(self, name: str) -> torch.Tensor:
        t = self.stored(name)
        return t.to(_device_dtype(t.dtype, self.specs[name].kind, self.run_dtype))


def write_model_folder(config: dict, out_dir: str, seed: int, *, std: float | None = None,
                       norm_std: float = 0.0, dtype: str = "bfloat16") -> str:
    """Random-weights mode: writes ``config.json`` and ``model.safetensors`` for the architecture
    that ``config`` names, drawn from ``seed``.  Returns ``out_dir``."""
    from ..config.registry import get_architecture
    from ..parts import Model
    arch = get_architecture(config["architectures"][0])
    cfg = arch.config_from_dict(config)
    spec = arch.build_model(cfg)
    model = Model(spec)
    specs = model.tensor_specs()
    store = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    src = RandomSource(specs, seed, spec.init_std if std is None else std, norm_std, "cpu", store)
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(config, f, indent=1)
    save_safetensors(os.path.join(out_dir, "model.safetensors"), {n: src.stored(n) for n in specs},
                     metadata={"format": "pt", "seed": seed})
    return out_dir


def load_model(model_dir: str, ctx, *, random_seed: int | None = None, norm_std: float = 0.0,
               std: float | None = None):
    """Builds the model that ``config.json`` names and binds its weights.

    With ``random_seed`` the weights are drawn on the device instead of read from files (the
    folder then needs only ``config.json``).  Returns ``(config, model)``."""
    from ..config.registry import load_model_config
    from ..parts import Model
    arch, cfg = load_model_config(model_dir)
    spec = arch.build_model(cfg)
    model = Model(spec)
    if random_seed is not None:
        specs = model.tensor_specs()
        src = RandomSource(specs, random_seed, spec.init_std if std is None else std, norm_std, ctx.device,
                           torch.bfloat16, ctx.act_dtype)
    else:
        folder = SafetensorsFolder(model_dir)
        specs = model.tensor_specs(lambda n: n in folder)
        check_tensors(specs, {n: i.shape for n, i in folder.tensors.items()})
        src = FolderSource(folder, specs, ctx.device, ctx.act_dtype)
    model.load(src, ctx)
    if random_seed is None:
        folder.close()
    return cfg, model
