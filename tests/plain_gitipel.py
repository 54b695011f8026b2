"""A plain, slow implementation of the Gitipel design for whole sequences.

No cache, no batching, no paging: one sequence of token ids in, the logits of
every position out (and, if asked, the residual stream after every layer run).
One function per mechanism, written from the design's equations; it shares no
code with the package ``chibillm_b200``.  ``config`` is the content of a
config.json, ``weights`` a dict of tensors by checkpoint name, widened to the
type all arithmetic is done in (float64 for a yardstick, float32 otherwise).

Notation: T tokens, D the model's width, H heads, G key/value heads, d the
size of a head.  Linear weights are [out, in].
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    """y = x / sqrt(mean(x^2) + eps) (* weight) over the last dimension."""
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    return x @ w.t()


def short_convolution(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """h [T, D], w [D, taps]: y_t = h_t + sum_j w[:, j] * h_(t - taps + 1 + j), with
    zeros before the first token."""
    T, D = h.shape
    taps = w.shape[1]
    padded = torch.cat([h.new_zeros(taps - 1, D), h], dim=0)
    y = h.clone()
    for j in range(taps):
        y = y + w[:, j] * padded[j:j + T]
    return y


def capped_distance_attention(h, wq, wk, wo, r1, r2, heads, kv_heads, d, scale, softcap):
    """Causal softmax attention whose values are its keys.  score(i, j) =
    cap * tanh(scale * q_i . k_j / cap) - r1 * ln(1 + r2 * (i - j)) per head."""
    T = h.shape[0]
    q = linear(h, wq).view(T, heads, d)
    k = linear(h, wk).view(T, kv_heads, d)
    group = heads // kv_heads
    pos = torch.arange(T, dtype=h.dtype)
    dist = pos[:, None] - pos[None, :]
    visible = dist >= 0
    out = h.new_zeros(T, heads, d)
    for head in range(heads):
        kh = k[:, head // group]
        s = (q[:, head] @ kh.t()) * scale
        s = softcap * torch.tanh(s / softcap)
        s = s - r1[head] * torch.log1p(r2[head] * dist.clamp(min=0))
        s = s.masked_fill(~visible, float("-inf"))
        out[:, head] = torch.softmax(s, dim=-1) @ kh
    return linear(out.reshape(T, heads * d), wo)


def delta_rule_mixer(h, w, prefix, heads, d, eps):
    """The generalised delta rule.  Per head, with state S [d, d] (key rows, value
    columns) starting at zero:  S <- diag(decay) S - (a * u) (u^T S) + k v^T with
    both products reading the old S, u the key scaled to unit length; o = S^T r."""
    T = h.shape[0]
    r = linear(h, w[prefix + "r"]).view(T, heads, d)
    k = linear(h, w[prefix + "k"]).view(T, heads, d)
    v = linear(h, w[prefix + "v"]).view(T, heads, d)
    gate = torch.sigmoid(linear(h, w[prefix + "g"]))
    low = torch.tanh(linear(h, w[prefix + "w1"]))
    decay = torch.exp(-math.exp(-0.5) * torch.sigmoid(linear(low, w[prefix + "w2"]) + w[prefix + "w0"]))
    decay = decay.view(T, heads, d)
    a = torch.sigmoid(linear(h, w[prefix + "a"]) + w[prefix + "a.b"]).view(T, heads, d)
    u = k / torch.sqrt((k * k).sum(dim=-1, keepdim=True) + 1e-6)
    o = h.new_zeros(T, heads, d)
    for head in range(heads):
        S = h.new_zeros(d, d)
        for t in range(T):
            seen = u[t, head] @ S                                    # [d values]
            S = decay[t, head][:, None] * S - torch.outer(a[t, head] * u[t, head], seen) \
                + torch.outer(k[t, head], v[t, head])
            o[t, head] = S.t() @ r[t, head]
    o = rms_norm(o, None, eps).reshape(T, heads * d) * w[prefix + "norm"] * gate
    return linear(o, w[prefix + "o"])


def dense_feed_forward(h, up, down):
    """down(gelu(up(h))) with the exact (erf) gelu."""
    z = linear(h, up)
    return linear(0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0))), down)


def run_order(config: dict) -> List[tuple]:
    """(layer, pass number or None, first of its pass) for every layer run."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, None, False) for i in range(n)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, None, False) for i in range(start)]
    for t in range(times):
        order += [(i, t, i == start) for i in range(start, stop)]
    return order + [(i, None, False) for i in range(stop, n)]


def forward(config: dict, weights: Dict[str, torch.Tensor], token_ids: List[int],
            layer_outputs: Optional[list] = None) -> torch.Tensor:
    w = weights
    eps = config["norm"]["eps"]
    dtype = w["embed"].dtype
    x = w["embed"][torch.tensor(token_ids, dtype=torch.long)] * config["embedding"]["scale"]
    x0 = x
    for index, turn, first in run_order(config):
        layer = config["layers"][index]
        p = f"l{index}."
        if first:
            x = linear(torch.cat([x, x0], dim=-1), w["loop.in"]) + w["loop.step"][turn]
        h = rms_norm(x, w[p + "norm1"], eps)
        h = short_convolution(h, w[p + "canon1"])
        m = layer["mixer"]
        if layer["type"] == "attention":
            x = x + capped_distance_attention(h, w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.o"], w[p + "mix.r1"],
                                              w[p + "mix.r2"], m["heads"], m["kv_heads"], m["dim"], m["scale"],
                                              m["softcap"])
        elif layer["type"] == "general_delta":
            x = x + delta_rule_mixer(h, w, p + "mix.", m["heads"], m["dim"], eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            x = x + dense_feed_forward(rms_norm(x, w[p + "norm2"], eps), w[p + "mlp.up"], w[p + "mlp.down"])
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    x = rms_norm(x, w["final.norm"], eps)
    return linear(x, w["head"]) * config["logit_scale"]
