"""Small Tirezen model folders for the tests, with weights that make every mechanism show.

The product's random-weights mode fills biases, decay logarithms and step biases with zeros and norm scales with
ones, under which a forgotten bias or a norm scale applied the wrong way would pass.  The folders made here draw
every tensor from a distribution wide enough to matter: decays between about 0.3 and 1, gates on both sides of
zero, attention scores that reach the soft cap.  Names and shapes come from the model's own list of expected
tensors; the values are this file's.
"""

import functools
import json
import os
import tempfile

import torch

from yalis_b200.config.presets import preset
from yalis_b200.config.registry import parse_config
from yalis_b200.engine.model import Model
from yalis_b200.weights.safetensors_io import write_safetensors

_ROOT = None


def _root():
    global _ROOT
    if _ROOT is None:
        _ROOT = tempfile.mkdtemp(prefix="yalis_b200_tirezen_")
    return _ROOT


def lively_tensor(name: str, shape, gen: torch.Generator, spread: float = 1.0) -> torch.Tensor:
    def normal(std):
        return torch.randn(shape, generator=gen) * std

    if name.endswith(".conv"):
        return normal(0.6)
    if name.endswith("A_log"):
        return torch.rand(shape, generator=gen) * 2.0 - 1.5
    if name.endswith("dt_bias"):
        return normal(1.0)
    if name.endswith(".b") and len(shape) == 1:          # biases of q, k, v
        return normal(0.5)
    if name.endswith(("norm1", "final.norm")):           # stored around zero
        return normal(0.2)
    if name.endswith("norm"):                            # plain scales
        return 1.0 + normal(0.2)
    if name == "loop.step":
        return normal(0.5)
    if name == "embed":
        return normal(1.0)
    fan_in = shape[-1]
    return normal(spread * 1.5 / fan_in ** 0.5)


def write_model(config: dict, out_dir: str, seed: int, spread: float = 1.0, overrides=None) -> str:
    """config.json and model.safetensors (bfloat16) for a Tirezen configuration; ``overrides`` name -> tensor."""
    arch, cfg = parse_config(config)
    expected = Model(arch.model_spec(cfg)).expected_tensors()
    gen = torch.Generator().manual_seed(seed)
    tensors = {}
    for name, ps in expected.items():
        t = lively_tensor(name, tuple(ps.shape), gen, spread)
        if overrides and name in overrides:
            t = overrides[name].reshape(ps.shape).float()
        tensors[name] = t.to(torch.bfloat16)
    os.makedirs(out_dir, exist_ok=True)
    write_safetensors(os.path.join(out_dir, "model.safetensors"), tensors)
    on_disk = {k: v for k, v in arch.config_to_dict(cfg).items()}
    for layer in on_disk["layers"]:                      # a folder gives the low-rank sizes by its tensors alone
        if layer["type"] == "parallel":
            layer["mixer"]["right"].pop("decay_rank", None)
            layer["mixer"]["right"].pop("gate_rank", None)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(on_disk, f)
    return out_dir


@functools.lru_cache(maxsize=None)
def tirezen_dir(which: str, seed: int = 0, spread: float = 1.0) -> str:
    return write_model(preset(f"tirezen-tiny-{which}"), os.path.join(_root(), f"{which}_{seed}_{spread}"), seed, spread)
