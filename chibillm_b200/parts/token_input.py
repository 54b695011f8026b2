"""A per-layer input from the token's id, applied to the residual at the end of
a block (TokenInputSpec): with e the layer's slice of a table row of the token,

    g = act(G x) * e;   y = P g;   x += scale * y / rms(y) * w

The table is shared by all layers and owned by none (the model declares it).
For few tokens one kernel does all of it, together with the block's own update
of the residual and the next norm; for many tokens the two products run as
matrix products (x is cast to the activations' type for the first) and the
kernel takes y from them.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .base import Part, Runtime, TensorSpec

# up to so many tokens the kernel at a layer's end does the two small products itself, if the two
# matrices are small too (a block per token reads both of them)
FEW_TOKENS = 64
SMALL_MATRIX = 16384


class TokenInput(Part):
    def __init__(self, spec, names: Dict[str, str], runtime: Runtime):
        self.spec = spec
        self.names = names
        self.runtime = runtime
        self.table: torch.Tensor = None
        self.gate: torch.Tensor = None
        self.proj: torch.Tensor = None
        self.norm: torch.Tensor = None

    def expected_tensors(self) -> List[TensorSpec]:
        s = self.spec
        return [TensorSpec(self.names["token_gate"], (s.dim, s.hidden_size)),
                TensorSpec(self.names["token_proj"], (s.hidden_size, s.dim)),
                TensorSpec(self.names["token_norm"], (s.hidden_size,))]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        self.table = tensors[s.table_name]
        if tuple(self.table.shape) != (s.vocab_size, s.table_width) or s.offset + s.dim > s.table_width:
            raise ValueError(f"{s.table_name}: shape {tuple(self.table.shape)} does not hold this layer's columns")
        self.gate = tensors[self.names["token_gate"]].to(self.table.dtype).contiguous()
        self.proj = tensors[self.names["token_proj"]].to(self.table.dtype).contiguous()
        self.norm = tensors[self.names["token_norm"]].to(self.table.dtype).contiguous()

    def launch_key(self, ctx):
        return ()

    def kernel_arguments(self, ctx):
        s = self.spec
        return (ctx.tokens, self.table, s.offset, self.gate, self.proj, self.norm, s.activation, s.eps)

    def wants_products(self, tokens: int) -> bool:
        """Whether the two products run as matrix products of their own (many tokens)
        or inside the kernel at the layer's end."""
        large = tokens > FEW_TOKENS or self.spec.dim * self.spec.hidden_size > SMALL_MATRIX
        return large and getattr(self.runtime.kernels, "side_gate", None) is not None

    def products(self, x: torch.Tensor, ctx) -> torch.Tensor:
        """y [T, hidden] float32 = P (act(G x) * e) by matrix products; x is the residual in
        the activations' type."""
        rt, s = self.runtime, self.spec
        k = rt.kernels
        T = x.shape[0]
        g = ctx.workspace.get("token_input.g", (T, s.dim), rt.dtype)
        k.linear(x, self.gate, g)
        k.side_gate(g, ctx.tokens, self.table, s.offset, s.activation)
        y = ctx.workspace.get("token_input.y", (T, s.hidden_size), torch.float32)
        k.linear(g, self.proj, y)
        return y
