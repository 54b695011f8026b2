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


def capped_distance_scores(q, k, r1, r2, scale, softcap):
    """q [T, H, d], k [T, G, d] of one sequence -> the heads' outputs [T, H, d] of causal
    softmax attention whose values are its keys.  score(i, j) =
    cap * tanh(scale * q_i . k_j / cap) - r1 * ln(1 + r2 * (i - j)) per head (no cap
    when ``softcap`` is None)."""
    T, heads, d = q.shape
    group = heads // k.shape[1]
    pos = torch.arange(T, dtype=q.dtype)
    dist = pos[:, None] - pos[None, :]
    visible = dist >= 0
    out = q.new_zeros(T, heads, d)
    for head in range(heads):
        kh = k[:, head // group]
        s = (q[:, head] @ kh.t()) * scale
        if softcap is not None:
            s = softcap * torch.tanh(s / softcap)
        s = s - r1[head] * torch.log1p(r2[head] * dist.clamp(min=0))
        s = s.masked_fill(~visible, float("-inf"))
        out[:, head] = torch.softmax(s, dim=-1) @ kh
    return out


def capped_distance_attention(h, wq, wk, wo, r1, r2, heads, kv_heads, d, scale, softcap):
    T = h.shape[0]
    q = linear(h, wq).view(T, heads, d)
    k = linear(h, wk).view(T, kv_heads, d)
    return linear(capped_distance_scores(q, k, r1, r2, scale, softcap).reshape(T, heads * d), wo)


def delta_rule_inputs(low, removal, k, w2, w0, removal_bias, decay_scale, key_eps, heads, d):
    """Decay, removal rate and unit key per token, head and key channel, from the
    low-rank decay input, the removal projection and the keys (all [T, ...])."""
    T = k.shape[0]
    decay = torch.exp(-decay_scale * torch.sigmoid(linear(torch.tanh(low), w2) + w0)).view(T, heads, d)
    a = torch.sigmoid(removal + removal_bias).view(T, heads, d)
    k = k.view(T, heads, d)
    u = k / torch.sqrt((k * k).sum(dim=-1, keepdim=True) + key_eps)
    return decay, a, u


def delta_rule_recurrence(r, k, v, decay, a, u, state=None):
    """All [T, H, d].  Per head, with state S [d, d] (key rows, value columns) starting
    at zero (or at ``state`` [H, d, d]):  S <- diag(decay) S - (a * u) (u^T S) + k v^T
    with both products reading the old S; o = S^T r.  Returns o and the last state."""
    T, heads, d = r.shape
    o = r.new_zeros(T, heads, d)
    last = r.new_zeros(heads, d, d)
    for head in range(heads):
        S = r.new_zeros(d, d) if state is None else state[head].clone()
        for t in range(T):
            seen = u[t, head] @ S                                    # [d values]
            S = decay[t, head][:, None] * S - torch.outer(a[t, head] * u[t, head], seen) \
                + torch.outer(k[t, head], v[t, head])
            o[t, head] = S.t() @ r[t, head]
        last[head] = S
    return o, last


def gated_head_norm(o, gate, weight, eps):
    """o [T, H, d]: each head divided by its root mean square, then times the weight
    over all heads and sigmoid(gate) ([T, H * d])."""
    T, heads, d = o.shape
    return rms_norm(o, None, eps).reshape(T, heads * d) * weight * torch.sigmoid(gate)


def delta_rule_mixer(h, w, prefix, heads, d, eps):
    """The generalised delta rule as a mixer: projections, recurrence, gated norm, output."""
    T = h.shape[0]
    r = linear(h, w[prefix + "r"]).view(T, heads, d)
    k = linear(h, w[prefix + "k"])
    v = linear(h, w[prefix + "v"]).view(T, heads, d)
    decay, a, u = delta_rule_inputs(linear(h, w[prefix + "w1"]), linear(h, w[prefix + "a"]), k, w[prefix + "w2"],
                                    w[prefix + "w0"], w[prefix + "a.b"], math.exp(-0.5), 1e-6, heads, d)
    o, _ = delta_rule_recurrence(r, k.view(T, heads, d), v, decay, a, u)
    return linear(gated_head_norm(o, linear(h, w[prefix + "g"]), w[prefix + "norm"], eps), w[prefix + "o"])


def gelu(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def dense_feed_forward(h, up, down):
    """down(gelu(up(h))) with the exact (erf) gelu."""
    z = linear(h, up)
    return linear(gelu(z), down)


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
    x = w["embed"][torch.tensor(token_ids, dtype=torch.long)] * config.get("embedding", {}).get("scale", 1.0)
    x0 = x
    for index, turn, first in run_order(config):
        layer = config["layers"][index]
        p = f"l{index}."
        if first:
            x = linear(torch.cat([x, x0], dim=-1), w["loop.in"]) + w["loop.step"][turn]
        h = rms_norm(x, w[p + "norm1"], eps)
        if config.get("canon"):
            h = short_convolution(h, w[p + "canon1"])
        m = layer["mixer"]
        if layer["type"] == "attention":
            x = x + capped_distance_attention(h, w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.o"], w[p + "mix.r1"],
                                              w[p + "mix.r2"], m["heads"], m["kv_heads"], m["dim"], m["scale"],
                                              m.get("softcap"))
        elif layer["type"] == "general_delta":
            x = x + delta_rule_mixer(h, w, p + "mix.", m["heads"], m["dim"], eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            x = x + dense_feed_forward(rms_norm(x, w[p + "norm2"], eps), w[p + "mlp.up"], w[p + "mlp.down"])
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    x = rms_norm(x, w["final.norm"], eps)
    return linear(x, w["head"]) * config.get("logit_scale", 1.0)
