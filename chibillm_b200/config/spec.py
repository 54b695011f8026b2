"""Architecture-neutral description of a decoder: parts, layers and run order.

A configuration class (one per architecture) turns the keys of its own
``config.json`` into a :class:`ModelSpec`.  Everything below the configuration
(weights loader, parts, cache manager, step function) reads only the spec, so
no part knows which model it is in.

Every size and constant is a field of a spec; nothing here has a default that
stands for a model's value.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    """A normalisation over the last ``size`` features.

    ``kind`` names a registered norm part ("rmsnorm").  ``weight_offset`` is
    added to the stored weight before use (0 for plain RMSNorm, 1 for the
    zero-centred variant).
    """

    kind: str
    size: int
    eps: float
    weight_offset: float = 0.0


@dataclass(frozen=True)
class PositionSpec:
    """Position encoding applied inside a mixer.

    ``kind`` "rope": split-half rotation of the first ``rotary_dim`` features
    of every head with ``inv_freq[j] = theta ** (-2j / rotary_dim)``.
    ``kind`` "none": nothing is applied.
    """

    kind: str
    head_dim: int = 0
    rotary_dim: int = 0
    theta: float = 0.0


@dataclass(frozen=True)
class MixerSpec:
    """Base of all token mixers; ``kind`` names a registered mixer part."""

    kind: str


@dataclass(frozen=True)
class AttentionSpec(MixerSpec):
    """Causal grouped-query attention over a paged key/value cache.

    ``window`` None means every earlier key is visible; an integer W means the
    W most recent keys, the query's own included.  ``scale`` multiplies the
    scores after the dot product.  ``softcap`` c (None: off) then replaces a
    score s by c * tanh(s / c).  ``distance_bias`` "log" then takes
    r1[h] * ln(1 + r2[h] * (i - j)) off the score of query i and key j, with two
    learned numbers per query head (tensor roles "distance_r1", "distance_r2").
    ``tied_values``: the values are the keys as projected; there is no value
    projection and the cache holds keys only.
    """

    hidden_size: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    scale: float = 0.0
    window: Optional[int] = None
    qk_norm: Optional[NormSpec] = None
    position: PositionSpec = PositionSpec(kind="none")
    softcap: Optional[float] = None
    distance_bias: Optional[str] = None
    tied_values: bool = False


@dataclass(frozen=True)
class DeltaRuleSpec(MixerSpec):
    """Linear recurrence with a state matrix per head (``head_dim`` key rows by
    ``head_dim`` value columns, 32-bit, zero at a sequence's start).  With r, k, v
    projections of the input, a decay per key channel
    w = exp(-``decay_scale`` * sigmoid(W2 tanh(W1 x) + w0)) (W1 of low rank), a
    removal rate per key channel a = sigmoid(Wa x + ba) and the unit key
    u = k / sqrt(sum(k^2) + ``key_eps``):

        S <- diag(w) S - (a * u) (u^T S) + k v^T      (both products read the old S)
        o  = S^T r

    Each head's o is divided by its root mean square (``norm_eps`` inside the
    root), multiplied by a weight over all heads and by sigmoid(Wg x), and
    projected back to ``hidden_size``.
    """

    hidden_size: int = 0
    num_heads: int = 0
    head_dim: int = 0
    decay_rank: int = 0
    decay_scale: float = 0.0
    key_eps: float = 0.0
    norm_eps: float = 0.0


@dataclass(frozen=True)
class ShortConvSpec:
    """A causal convolution over time on each channel, added to its input:
    y_t = x_t + sum_j w[:, j] * x_(t - taps + 1 + j), zeros before the sequence's
    start.  The last ``taps`` - 1 inputs are part of a request's state."""

    size: int
    taps: int


@dataclass(frozen=True)
class FeedForwardSpec:
    """Base of all feed-forward parts; ``kind`` names a registered part."""

    kind: str


@dataclass(frozen=True)
class GatedMLPSpec(FeedForwardSpec):
    """Dense gated feed-forward: down(act(gate(x)) * up(x))."""

    hidden_size: int = 0
    intermediate_size: int = 0
    activation: str = "silu"


@dataclass(frozen=True)
class DenseMLPSpec(FeedForwardSpec):
    """Dense feed-forward without a gate: down(act(up(x))).  ``activation``:
    "gelu" (exact, with erf), "gelu_tanh", "silu" or "relu"."""

    hidden_size: int = 0
    intermediate_size: int = 0
    activation: str = "gelu"


@dataclass(frozen=True)
class LayerSpec:
    """One block: how mixer, feed-forward and norms are arranged.

    ``arrangement`` names a registered block ("prenorm": x + mixer(norm(x)),
    then x + ff(norm(x))).  ``weight_prefix`` is the checkpoint prefix of the
    block's tensors.  ``weight_names`` maps the part-local tensor roles to
    checkpoint names under that prefix.  ``feed_forward`` (with its norm) may be
    None: the block then ends after the mixer.  ``mixer_conv``: a short
    convolution between the mixer's norm and the mixer (tensor role
    "mixer_conv").
    """

    arrangement: str
    mixer: MixerSpec
    feed_forward: Optional[FeedForwardSpec]
    mixer_norm: NormSpec
    feed_forward_norm: Optional[NormSpec]
    weight_prefix: str
    weight_names: Tuple[Tuple[str, str], ...] = ()
    mixer_conv: Optional[ShortConvSpec] = None

    def names(self) -> dict:
        return dict(self.weight_names)


@dataclass(frozen=True)
class RunStep:
    """One entry of the run order.

    ``layer`` indexes ``ModelSpec.layers`` (a layer may be named twice: its
    weights are shared, every run has a cache of its own).  ``cache_of`` names
    an earlier run step whose cache this step reads instead of writing one.
    ``enter`` indexes ``ModelSpec.stream_adapters``: that adapter transforms the
    residual stream right before this step, with ``turn`` as its argument (the
    number of the pass that begins here, for a group of layers that runs
    several times).
    """

    layer: int
    cache_of: Optional[int] = None
    enter: Optional[int] = None
    turn: int = 0


@dataclass(frozen=True)
class AdapterSpec:
    """A part at one of the decoder's ends: after the token embedding (it
    changes the residual stream in place: a learned or absolute position table,
    a scale of the embeddings) or on the logits of the wanted rows (a soft cap,
    a bias).  ``kind`` names a registered adapter part; ``weight_names`` maps
    its tensor roles to checkpoint names; ``params`` are its constants."""

    kind: str
    weight_names: Tuple[Tuple[str, str], ...] = ()
    params: Tuple[Tuple[str, float], ...] = ()

    def names(self) -> dict:
        return dict(self.weight_names)

    def constants(self) -> dict:
        return dict(self.params)


@dataclass(frozen=True)
class ModelSpec:
    """A whole decoder: embedding, what follows it at once, layers, run order,
    final norm, output, what is done to the logits."""

    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int                                # 0: no limit of the model's own (the cache pool bounds a request)
    layers: Tuple[LayerSpec, ...]
    run_order: Tuple[RunStep, ...]
    final_norm: NormSpec
    embedding_name: str
    final_norm_name: str
    output_name: str
    tie_output_to_embedding: bool
    eos_token_id: Optional[int] = None
    bos_token_id: Optional[int] = None
    extra: dict = field(default_factory=dict, compare=False)
    input_adapters: Tuple[AdapterSpec, ...] = ()      # run on the residual right after the embedding
    logit_adapters: Tuple[AdapterSpec, ...] = ()      # run on the 32-bit logits of the wanted rows
    stream_adapters: Tuple[AdapterSpec, ...] = ()     # run on the residual where a run step's ``enter`` names them
