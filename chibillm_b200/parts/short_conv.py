"""A short causal convolution over time on each channel, added to its input:
y_t = x_t + sum_j w[:, j] * x_(t - taps + 1 + j).  Inputs before a sequence's
start count as zeros; inputs before a step's first token come from the
request's state, which holds its last ``taps`` - 1 inputs in the activations'
type (they are stored as they were read, so a prompt cut anywhere gives what
the whole prompt gives)."""
from __future__ import annotations

from typing import Dict, List

import torch

from .base import FixedStateNeed, Part, Runtime, TensorSpec


class ShortConv(Part):
    def __init__(self, spec, weight_name: str, runtime: Runtime):
        if spec.taps < 1:
            raise ValueError("a short convolution needs at least one tap")
        self.spec = spec
        self.weight_name = weight_name
        self.runtime = runtime
        self.weight: torch.Tensor = None
        self.weight_t: torch.Tensor = None          # [taps, size], for the kernel's wide loads

    def expected_tensors(self) -> List[TensorSpec]:
        return [TensorSpec(self.weight_name, (self.spec.size, self.spec.taps), init=("normal", 0.0, 0.1))]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name].float().contiguous()
        self.weight_t = self.weight.t().contiguous()

    def cache_need(self):
        return FixedStateNeed((("history", (max(self.spec.taps - 1, 1), self.spec.size), None),))

    def launch_key(self, ctx):
        return ()

    def forward(self, x: torch.Tensor, out: torch.Tensor, ctx, state) -> None:
        self.runtime.kernels.short_conv(x, self.weight, state.arrays["history"], out, ctx.q_start, ctx.positions,
                                        ctx.state_slots, ctx.max_q_len, weight_t=self.weight_t)
