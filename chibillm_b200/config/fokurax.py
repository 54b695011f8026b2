"""Fokurax: the typed configuration and its translation into parts.

A Fokurax config.json names the architecture under "architecture" and gives
every size and constant in nested objects:

* "vocab", "width"; "norm": {"eps"}; "embedding": {"scale"}; "residual_mult";
  "logit_softcap"; "token_side": {"dim"};
* "layers": one object per layer with "type" ("attention"), "mixer" and "mlp".
  A mixer gives "heads", "kv_heads", "dim" (a query's or key's size), "vdim" (a
  value's), "scale", "mask": {"size"} (attention inside blocks of that many
  positions), "rot": {"base", "dims", "scaling": {"factor", "original", "fast",
  "slow"}}, and optionally "kv_from": j (the layer has no key and value
  projections and reads layer j's cache).  "mlp" is null, {"kind": "dense", "ff"}
  or {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top"}}.

Absent optional objects ("embedding", "residual_mult", "logit_softcap",
"token_side", a mixer's "mask", "rot", "rot.scaling", "vdim", "kv_heads") switch
their mechanism off or fall back to the plain value.

What the design fixes: every layer is one norm (weight stored as a difference
from one) whose output both branches read; q and k are divided by their root
mean square after the rotation; the dense feed-forward is gated with the tanh
form of gelu and has biases, the experts are gated with silu and have none and
are chosen by a table from the token's id with equal weights; the amplitude of
a stretched rotation is 0.1 ln(factor) + 1.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .base import ConfigError, KeyReader, finite_number as _number, object_at as _object
from .spec import (AdapterSpec, AttentionSpec, GatedMLPSpec, LayerSpec, ModelSpec, NormSpec, PositionSpec, RunStep,
                   TableExpertsSpec, TokenInputSpec)

ARCHITECTURE = "Fokurax"
AMPLITUDE_SLOPE = 0.1
SIDE_TABLE = "side.embed"


@dataclass(frozen=True)
class FokuraxRotation:
    base: float
    dims: int
    factor: float = 0.0            # 0: frequencies as they are
    original: int = 0
    fast: float = 0.0
    slow: float = 0.0


@dataclass(frozen=True)
class FokuraxLayer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    chunk: Optional[int]
    rot: Optional[FokuraxRotation]
    kv_from: Optional[int]
    mlp: Optional[str]             # None | "dense" | "moe"
    ff: int = 0
    experts: int = 0
    top: int = 0


@dataclass(frozen=True)
class FokuraxConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    residual_mult: float
    logit_softcap: Optional[float]
    side_dim: Optional[int]
    layers: Tuple[FokuraxLayer, ...]

    @classmethod
    def from_dict(cls, obj: dict) -> "FokuraxConfig":
        r = KeyReader(obj)
        vocab, width = r.positive_int("vocab"), r.positive_int("width")
        eps = KeyReader(_object(r, "norm")).positive_float("eps")
        embedding_scale = _number(KeyReader(_object(r, "embedding")), "scale") if r.has("embedding") else 1.0
        residual_mult = _number(r, "residual_mult") if r.has("residual_mult") else 1.0
        softcap = r.positive_float("logit_softcap") if r.has("logit_softcap") else None
        side_dim = KeyReader(_object(r, "token_side")).positive_int("dim") if r.has("token_side") else None
        raw_layers = r.raw("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("invalid_field", "key 'layers' must be a non-empty list")
        layers = []
        for i, raw in enumerate(raw_layers):
            lr = KeyReader(raw)
            lr.require_value("type", ("attention",))
            m = KeyReader(_object(lr, "mixer"))
            heads, dim = m.positive_int("heads"), m.positive_int("dim")
            kv_heads = m.positive_int("kv_heads", heads)
            if heads % kv_heads != 0:
                raise ConfigError("invalid_geometry", f"layer {i}: heads {heads} is not a multiple of kv_heads {kv_heads}")
            vdim = m.positive_int("vdim", dim)
            chunk = KeyReader(_object(m, "mask")).positive_int("size") if m.has("mask") else None
            rot = None
            if m.has("rot"):
                rr = KeyReader(_object(m, "rot"))
                dims = rr.positive_int("dims")
                if dims % 2 or dims > dim:
                    raise ConfigError("invalid_geometry", f"layer {i}: rot.dims {dims} must be even and at most dim {dim}")
                rot = FokuraxRotation(rr.positive_float("base"), dims)
                if rr.has("scaling"):
                    sc = KeyReader(_object(rr, "scaling"))
                    rot = FokuraxRotation(rot.base, dims, sc.positive_float("factor"), sc.positive_int("original"),
                                          sc.positive_float("fast"), sc.positive_float("slow"))
            kv_from = None
            if m.has("kv_from"):
                kv_from = m.raw("kv_from")
                if isinstance(kv_from, bool) or not isinstance(kv_from, int) or not (0 <= kv_from < i):
                    raise ConfigError("invalid_field", f"layer {i}: 'kv_from' must name an earlier layer")
                src = layers[kv_from]
                if src.kv_from is not None:
                    raise ConfigError("invalid_field", f"layer {i}: 'kv_from' names layer {kv_from}, which has no "
                                                       f"keys and values of its own")
                if (src.kv_heads, src.dim, src.vdim) != (kv_heads, dim, vdim):
                    raise ConfigError("invalid_geometry", f"layer {i}: its kv_heads, dim and vdim must equal those "
                                                          f"of layer {kv_from}, whose cache it reads")
            kind, ff, experts, top = None, 0, 0, 0
            if lr.has("mlp"):
                mlp = KeyReader(_object(lr, "mlp"))
                kind = mlp.require_value("kind", ("dense", "moe"))
                if kind == "dense":
                    ff = mlp.positive_int("ff")
                else:
                    ff = KeyReader(_object(mlp, "expert")).positive_int("ff")
                    router = KeyReader(_object(mlp, "router"))
                    experts, top = router.positive_int("experts"), router.positive_int("top")
                    if top > experts:
                        raise ConfigError("invalid_geometry", f"layer {i}: top {top} exceeds experts {experts}")
            layers.append(FokuraxLayer(heads, kv_heads, dim, vdim, m.positive_float("scale"), chunk, rot, kv_from,
                                       kind, ff, experts, top))
        return cls(vocab, width, eps, embedding_scale, residual_mult, softcap, side_dim, tuple(layers))

    def model_spec(self) -> ModelSpec:
        D = self.width
        norm = NormSpec("rmsnorm", D, self.eps, 1.0)
        n = len(self.layers)
        layers, order = [], []
        for i, l in enumerate(self.layers):
            if l.rot is None:
                position = PositionSpec(kind="none", head_dim=l.dim)
            else:
                position = PositionSpec(kind="rope", head_dim=l.dim, rotary_dim=l.rot.dims, theta=l.rot.base,
                                        scaling_factor=l.rot.factor, original_positions=l.rot.original,
                                        fast_turns=l.rot.fast, slow_turns=l.rot.slow,
                                        amplitude_slope=AMPLITUDE_SLOPE if l.rot.factor else 0.0)
            mixer = AttentionSpec(kind="attention", hidden_size=D, num_heads=l.heads, num_kv_heads=l.kv_heads,
                                  head_dim=l.dim, scale=l.scale, position=position, value_dim=l.vdim, chunk=l.chunk,
                                  unit_norm_eps=self.eps, own_kv=l.kv_from is None)
            names = [("mixer_norm", "norm1"), ("q_proj", "mix.q"), ("k_proj", "mix.k"), ("v_proj", "mix.v"),
                     ("o_proj", "mix.o")]
            ff = None
            if l.mlp == "dense":
                ff = GatedMLPSpec(kind="gated_mlp", hidden_size=D, intermediate_size=l.ff, activation="gelu_tanh",
                                  biases=True)
                names += [("gate_proj", "mlp.gate"), ("up_proj", "mlp.up"), ("down_proj", "mlp.down"),
                          ("gate_bias", "mlp.gate.b"), ("up_bias", "mlp.up.b"), ("down_bias", "mlp.down.b")]
            elif l.mlp == "moe":
                ff = TableExpertsSpec(kind="table_experts", hidden_size=D, intermediate_size=l.ff,
                                      num_experts=l.experts, top=l.top, vocab_size=self.vocab, activation="silu")
                names += [("expert_table", "mlp.table"), ("expert_gate", "mlp.e{e}.gate"),
                          ("expert_up", "mlp.e{e}.up"), ("expert_down", "mlp.e{e}.down")]
            token_input = None
            if self.side_dim is not None:
                token_input = TokenInputSpec(hidden_size=D, dim=self.side_dim, offset=i * self.side_dim,
                                             table_name=SIDE_TABLE, table_width=n * self.side_dim,
                                             vocab_size=self.vocab, activation="gelu_tanh", eps=self.eps)
                names += [("token_gate", "side.gate"), ("token_proj", "side.proj"), ("token_norm", "side.norm")]
            layers.append(LayerSpec(arrangement="parallel", mixer=mixer, feed_forward=ff, mixer_norm=norm,
                                    feed_forward_norm=None, weight_prefix=f"l{i}.", weight_names=tuple(names),
                                    residual_scale=self.residual_mult, token_input=token_input))
            order.append(RunStep(layer=i, cache_of=l.kv_from))
        shared = ()
        if self.side_dim is not None:
            shared = ((SIDE_TABLE, (self.vocab, n * self.side_dim), "float"),)
        logit = ()
        if self.logit_softcap is not None:
            logit = (AdapterSpec(kind="softcap", params=(("cap", self.logit_softcap),)),)
        return ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab, hidden_size=D, max_positions=0,
            layers=tuple(layers), run_order=tuple(order), final_norm=norm, embedding_name="embed",
            final_norm_name="final.norm", output_name="head", tie_output_to_embedding=False,
            input_adapters=(AdapterSpec(kind="scale", params=(("factor", self.embedding_scale),)),),
            logit_adapters=logit, shared_tensors=shared)
