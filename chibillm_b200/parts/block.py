"""Block arrangements.  "prenorm": residual += mixer(norm(residual)), then
residual += feed_forward(norm(residual)); the residual itself is never
normalised in place (src/qwen/qwen_layer.cc:124-146).  Two options of the
layer's spec: a short convolution over time between the first norm and the
mixer (it keeps its last inputs per request, so the block then has two cache
needs), and no feed-forward at all."""
from __future__ import annotations

from typing import Dict, List

import torch

from .base import (Block, Runtime, TensorSpec, make_feed_forward, make_mixer, make_norm,
                   register_block)
from .short_conv import ShortConv


class PreNormBlock(Block):
    def __init__(self, layer, runtime: Runtime):
        self.layer = layer
        self.runtime = runtime
        names = {role: layer.weight_prefix + name for role, name in layer.names().items()}
        self.mixer_norm = make_norm(layer.mixer_norm, names["mixer_norm"], runtime)
        self.mixer = make_mixer(layer.mixer, names, runtime)
        self.mixer_conv = None if layer.mixer_conv is None else ShortConv(layer.mixer_conv, names["mixer_conv"], runtime)
        self.feed_forward = self.feed_forward_norm = None
        if layer.feed_forward is not None:
            self.feed_forward_norm = make_norm(layer.feed_forward_norm, names["feed_forward_norm"], runtime)
            self.feed_forward = make_feed_forward(layer.feed_forward, names, runtime)
        self._parts = tuple(p for p in (self.mixer_norm, self.mixer_conv, self.mixer, self.feed_forward_norm,
                                        self.feed_forward) if p is not None)

    def expected_tensors(self) -> List[TensorSpec]:
        out: List[TensorSpec] = []
        for p in self._parts:
            out.extend(p.expected_tensors())
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for p in self._parts:
            p.bind(tensors)

    def cache_need(self):
        if self.mixer_conv is None:
            return self.mixer.cache_need()
        return (self.mixer.cache_need(), self.mixer_conv.cache_need())

    def launch_key(self, ctx):
        keys = [p.launch_key(ctx) for p in (self.mixer_conv, self.mixer, self.feed_forward) if p is not None]
        return None if any(k is None for k in keys) else tuple(keys)

    def forward(self, residual: torch.Tensor, ctx, cache, pending=None):
        x = ctx.workspace.get("block.normed", tuple(residual.shape), self.runtime.dtype)
        conv = self.mixer_conv
        normed = self.mixer_norm.forward_fused(residual, pending, x,
                                               conv is None and self.mixer.accepts_scaled_rows)
        normed = x if normed is None else normed
        if conv is not None:
            cache, conv_state = cache
            mixed = ctx.workspace.get("block.conv", tuple(residual.shape), self.runtime.dtype)
            conv.forward(normed, mixed, ctx, conv_state)
            normed = mixed
        pending = self.mixer.forward(normed, residual, ctx, cache)
        if self.feed_forward is None:
            return pending
        normed = self.feed_forward_norm.forward_fused(residual, pending, x, self.feed_forward.accepts_scaled_rows)
        return self.feed_forward.forward(x if normed is None else normed, residual, ctx)


register_block("prenorm", PreNormBlock, replace=True)
