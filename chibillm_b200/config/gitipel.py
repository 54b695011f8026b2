"""Gitipel: the typed configuration and its translation into parts.

A Gitipel config.json names the architecture under "architecture" and gives
every size and constant in nested objects:

* "vocab", "width"; "norm": {"eps"}; "embedding": {"scale"}; "logit_scale";
* "canon": {"taps"}: a short convolution over time after each layer's first norm;
* "layers": one object per layer with "type" ("attention" or "general_delta"),
  "mixer" (its sizes) and "mlp" ({"kind": "dense", "ff"} or null);
* "loop": {"start", "stop", "times"}: layers start .. stop - 1 run ``times``
  times in a row with the same weights; before each pass the residual is mixed
  with the embedding output and a vector of the pass is added.

Absent optional objects ("canon", "loop", "embedding", "logit_scale") switch
their mechanism off.  The rank of a delta-rule layer's decay input is not a key
of the file: it is the first size of the tensor "<layer>.mix.w1" (the loader of
a model folder adds the checkpoint's shapes to the object it hands to
:meth:`GitipelConfig.from_dict`), or the mixer's optional key "rank" (folders
written from a configuration alone).

Constants that the design fixes: the decay is exp(-exp(-1/2) * sigmoid(.)),
unit keys use 1e-6 inside the root.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple

from .base import ConfigError, KeyReader, finite_number as _number, object_at as _object
from .spec import (AdapterSpec, AttentionSpec, DeltaRuleSpec, DenseMLPSpec, LayerSpec, ModelSpec, NormSpec,
                   PositionSpec, RunStep, ShortConvSpec)

ARCHITECTURE = "Gitipel"
DECAY_SCALE = math.exp(-0.5)
KEY_EPS = 1e-6
SHAPES_KEY = "_tensor_shapes"          # filled in by the loader of a model folder


@dataclass(frozen=True)
class GitipelLayer:
    type: str                          # "attention" | "general_delta"
    heads: int
    dim: int
    kv_heads: int = 0                  # attention
    scale: float = 0.0                 # attention
    softcap: Optional[float] = None    # attention
    rank: int = 0                      # general_delta
    ff: Optional[int] = None           # None: no feed-forward


@dataclass(frozen=True)
class GitipelConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    logit_scale: float
    taps: Optional[int]
    layers: Tuple[GitipelLayer, ...]
    loop: Optional[Tuple[int, int, int]]          # (start, stop, times)

    @classmethod
    def from_dict(cls, obj: dict) -> "GitipelConfig":
        r = KeyReader(obj)
        vocab = r.positive_int("vocab")
        width = r.positive_int("width")
        eps = KeyReader(_object(r, "norm")).positive_float("eps")
        embedding_scale = _number(KeyReader(_object(r, "embedding")), "scale") if r.has("embedding") else 1.0
        logit_scale = _number(r, "logit_scale") if r.has("logit_scale") else 1.0
        taps = KeyReader(_object(r, "canon")).positive_int("taps") if r.has("canon") else None
        shapes = obj.get(SHAPES_KEY) or {}
        raw_layers = r.raw("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("invalid_field", "key 'layers' must be a non-empty list")
        layers = []
        for i, raw in enumerate(raw_layers):
            lr = KeyReader(raw)
            kind = lr.require_value("type", ("attention", "general_delta"))
            m = KeyReader(_object(lr, "mixer"))
            heads, dim = m.positive_int("heads"), m.positive_int("dim")
            ff = None
            if lr.has("mlp"):
                mlp = KeyReader(_object(lr, "mlp"))
                mlp.require_value("kind", ("dense",))
                ff = mlp.positive_int("ff")
            if kind == "attention":
                kv_heads = m.positive_int("kv_heads", heads)
                if heads % kv_heads != 0:
                    raise ConfigError("invalid_geometry", f"layer {i}: heads {heads} is not a multiple of "
                                                          f"kv_heads {kv_heads}")
                if m.has("vdim") and m.positive_int("vdim") != dim:
                    raise ConfigError("invalid_geometry", f"layer {i}: the values are the keys, so 'vdim' "
                                                          f"must equal 'dim' {dim}")
                layers.append(GitipelLayer(kind, heads, dim, kv_heads=kv_heads, scale=m.positive_float("scale"),
                                           softcap=m.positive_float("softcap") if m.has("softcap") else None,
                                           ff=ff))
            else:
                if m.has("rank"):
                    rank = m.positive_int("rank")
                elif f"l{i}.mix.w1" in shapes:
                    rank = int(shapes[f"l{i}.mix.w1"][0])
                else:
                    raise ConfigError("missing_field", f"layer {i}: the rank of the decay input is given neither by "
                                                       f"the mixer's key 'rank' nor by a tensor 'l{i}.mix.w1'")
                layers.append(GitipelLayer(kind, heads, dim, rank=rank, ff=ff))
        loop = None
        if r.has("loop"):
            lp = KeyReader(_object(r, "loop"))
            start = lp.raw("start")
            stop, times = lp.positive_int("stop"), lp.positive_int("times")
            if isinstance(start, bool) or not isinstance(start, int) or not (0 <= start < stop <= len(layers)):
                raise ConfigError("invalid_field", f"key 'loop': 0 <= start < stop <= {len(layers)} is required")
            loop = (start, stop, times)
        return cls(vocab, width, eps, embedding_scale, logit_scale, taps, tuple(layers), loop)

    def model_spec(self) -> ModelSpec:
        D = self.width
        norm = NormSpec("rmsnorm", D, self.eps, 0.0)
        conv = ShortConvSpec(D, self.taps) if self.taps is not None else None
        layers = []
        for i, l in enumerate(self.layers):
            names = [("mixer_norm", "norm1"), ("mixer_conv", "canon1"), ("o_proj", "mix.o")]
            if l.type == "attention":
                mixer = AttentionSpec(kind="attention", hidden_size=D, num_heads=l.heads, num_kv_heads=l.kv_heads,
                                      head_dim=l.dim, scale=l.scale, softcap=l.softcap, distance_bias="log",
                                      tied_values=True, position=PositionSpec(kind="none", head_dim=l.dim))
                names += [("q_proj", "mix.q"), ("k_proj", "mix.k"), ("distance_r1", "mix.r1"),
                          ("distance_r2", "mix.r2")]
            else:
                mixer = DeltaRuleSpec(kind="delta_rule", hidden_size=D, num_heads=l.heads, head_dim=l.dim,
                                      decay_rank=l.rank, decay_scale=DECAY_SCALE, key_eps=KEY_EPS, norm_eps=self.eps)
                names += [("r_proj", "mix.r"), ("k_proj", "mix.k"), ("v_proj", "mix.v"), ("g_proj", "mix.g"),
                          ("a_proj", "mix.a"), ("removal_bias", "mix.a.b"), ("decay_in", "mix.w1"),
                          ("decay_out", "mix.w2"), ("decay_bias", "mix.w0"), ("out_norm", "mix.norm")]
            ff = None
            if l.ff is not None:
                ff = DenseMLPSpec(kind="mlp", hidden_size=D, intermediate_size=l.ff, activation="gelu")
                names += [("feed_forward_norm", "norm2"), ("up_proj", "mlp.up"), ("down_proj", "mlp.down")]
            layers.append(LayerSpec(arrangement="prenorm", mixer=mixer, feed_forward=ff, mixer_norm=norm,
                                    feed_forward_norm=norm if ff is not None else None, weight_prefix=f"l{i}.",
                                    weight_names=tuple(names), mixer_conv=conv))
        n = len(layers)
        stream = ()
        if self.loop is None:
            order = [RunStep(layer=i) for i in range(n)]
        else:
            start, stop, times = self.loop
            stream = (AdapterSpec(kind="reentry_mix", weight_names=(("mix", "loop.in"), ("step", "loop.step")),
                                  params=(("hidden_size", D), ("turns", times))),)
            order = [RunStep(layer=i) for i in range(start)]
            for t in range(times):
                order += [RunStep(layer=i, enter=0 if i == start else None, turn=t) for i in range(start, stop)]
            order += [RunStep(layer=i) for i in range(stop, n)]
        return ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab, hidden_size=D, max_positions=0,
            layers=tuple(layers), run_order=tuple(order), final_norm=norm, embedding_name="embed",
            final_norm_name="final.norm", output_name="head", tie_output_to_embedding=False,
            input_adapters=(AdapterSpec(kind="scale", params=(("factor", self.embedding_scale),)),),
            logit_adapters=(AdapterSpec(kind="scale", params=(("factor", self.logit_scale),)),),
            stream_adapters=stream)
