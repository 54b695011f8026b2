"""The generalised delta rule as a mixer: a linear recurrence with one state
matrix per head instead of a cache of keys.

One product gives r | k | v | gate | removal | low-rank decay input for all
heads.  The decay's logits W2 tanh(low) are made next (a small kernel for few
tokens, a matrix product for many).  The recurrence kernel turns all of it, per
token and head, into the decay w = exp(-decay_scale * sigmoid(logits + w0)), the removal rate
a = sigmoid(removal + bias) and the unit key u = k / sqrt(sum(k^2) + key_eps),
all in 32-bit, and runs

    S <- diag(w) S - (a * u) (u^T S) + k v^T,   o = S^T r

over the step's tokens of every sequence, from the state that the request's
slot holds to the state it leaves there (32-bit, [heads, key, value]).  A second
kernel divides each head's o by its root mean square, multiplies by the weight
and by sigmoid(gate); the output product adds into the residual.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .base import FixedStateNeed, Mixer, Runtime, TensorSpec, register_mixer

_PROJECTIONS = ("r_proj", "k_proj", "v_proj", "g_proj", "a_proj")


class DeltaRuleMixer(Mixer):
    def __init__(self, spec, names: Dict[str, str], runtime: Runtime):
        self.spec = spec
        self.names = names
        self.runtime = runtime
        self.stacked: torch.Tensor = None        # r | k | v | gate | removal | decay_in
        self.decay_out: torch.Tensor = None      # [rank, heads * d] 32-bit: transposed for the kernel
        self.decay_out_matrix: torch.Tensor = None
        self.decay_bias: torch.Tensor = None
        self.removal_bias: torch.Tensor = None
        self.norm_weight: torch.Tensor = None
        self.o_proj: torch.Tensor = None

    def expected_tensors(self) -> List[TensorSpec]:
        s = self.spec
        width = s.num_heads * s.head_dim
        out = [TensorSpec(self.names[r], (width, s.hidden_size)) for r in _PROJECTIONS]
        out += [TensorSpec(self.names["removal_bias"], (width,), init=("uniform", -2.0, 2.0)),
                TensorSpec(self.names["decay_in"], (s.decay_rank, s.hidden_size)),
                TensorSpec(self.names["decay_out"], (width, s.decay_rank), init=("normal", 0.0, 0.5)),
                TensorSpec(self.names["decay_bias"], (width,), init=("uniform", -6.0, 0.0)),
                TensorSpec(self.names["out_norm"], (width,)),
                TensorSpec(self.names["o_proj"], (s.hidden_size, width))]
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        mats = [tensors[self.names[r]] for r in _PROJECTIONS] + [tensors[self.names["decay_in"]]]
        self.stacked = torch.cat([m.to(mats[0].dtype) for m in mats], dim=0).contiguous()
        self.decay_out = tensors[self.names["decay_out"]].float().t().contiguous()
        self.decay_out_matrix = tensors[self.names["decay_out"]].contiguous()      # [heads * d, rank] for a product
        self.decay_bias = tensors[self.names["decay_bias"]].float().contiguous()
        self.removal_bias = tensors[self.names["removal_bias"]].float().contiguous()
        self.norm_weight = tensors[self.names["out_norm"]].float().contiguous()
        self.o_proj = tensors[self.names["o_proj"]].contiguous()

    accepts_scaled_rows = True       # x goes to the stacked product and nowhere else
    LOGITS_BY_PRODUCT_FROM = 32      # steps of more tokens make the decay's logits with a matrix product

    def cache_need(self):
        s = self.spec
        return FixedStateNeed((("state", (s.num_heads, s.head_dim, s.head_dim), torch.float32),))

    def launch_key(self, ctx):
        return ()

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, cache):
        s, rt = self.spec, self.runtime
        k = rt.kernels
        T = x.shape[0]
        width = s.num_heads * s.head_dim
        proj = ctx.workspace.get("delta.proj", (T, self.stacked.shape[0]), rt.dtype)
        k.linear(x, self.stacked, proj)
        o = ctx.workspace.get("delta.o", (T, width), torch.float32)
        logits = ctx.workspace.get("delta.decay_logits", (T, width), torch.float32)
        if T > self.LOGITS_BY_PRODUCT_FROM:
            # many tokens: tanh(low) W2^T is a matrix product on the tensor cores
            low = ctx.workspace.get("delta.low", (T, s.decay_rank), rt.dtype)
            k.cast_rows(proj[:, 5 * width:], low, activation="tanh")
            k.linear(low, self.decay_out_matrix, logits)
        else:
            k.decay_logits(proj[:, 5 * width:], self.decay_out, logits)
        k.delta_rule(proj, logits, self.decay_bias, self.removal_bias, cache.arrays["state"], o,
                     ctx.q_start, ctx.state_slots, s.num_heads, s.head_dim, s.decay_rank, s.decay_scale,
                     s.key_eps, ctx.max_q_len)
        gated = ctx.workspace.get("delta.gated", (T, width), rt.dtype)
        k.gated_group_norm(o, proj[:, 3 * width:4 * width], self.norm_weight, s.norm_eps, s.head_dim, gated)
        return k.linear(gated, self.o_proj, residual, residual=residual, defer=True)


register_mixer("delta_rule", DeltaRuleMixer, replace=True)
