"""Dense feed-forward without a gate: down(act(up(x))), act a gelu (erf or tanh form) or silu."""

from __future__ import annotations

from typing import Dict, Optional

import torch

from yalis_b200.config.spec import PartSpec
from yalis_b200.ops.elementwise import ACTIVATIONS, activation
from .base import FeedForward, ParamSpec, Projected, register_part


class DenseFeedForward(FeedForward, Projected):
    """Parameters: ``hidden_size``, ``intermediate_size``, ``activation`` (``gelu_erf`` by default,
    ``gelu_tanh`` or ``silu``).  The activation is computed in float32."""

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        self.act = str(spec.params.get("activation", "gelu_erf"))
        if self.act not in ACTIVATIONS:
            raise ValueError(f"unknown activation {self.act!r} (one of {', '.join(ACTIVATIONS)})")
        self.hidden_width = self.inter
        self.w_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"up_proj": ParamSpec((self.inter, self.hidden)), "down_proj": ParamSpec((self.hidden, self.inter))}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.w_up = tensors["up_proj"].contiguous()
        self.w_down = tensors["down_proj"].contiguous()

    def in_weight(self) -> torch.Tensor:
        return self.w_up

    def out_weight(self) -> torch.Tensor:
        return self.w_down

    def release_projections(self) -> None:
        self.w_up = self.w_down = None

    def mix(self, z: torch.Tensor, ctx, cache, y: torch.Tensor) -> None:
        activation(z, self.act, out=y)

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        return self.project_and_mix(x, ctx, None)

    def capture_key(self, host):
        return None


register_part("feed_forward", "dense", DenseFeedForward)
