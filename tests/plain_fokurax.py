"""A plain, slow restatement of the Fokurax design: whole sequences, no cache,
one function per mechanism, on the CPU.  It shares no code with the package:
it takes the parsed config.json and a dict of tensors by their checkpoint
names and returns logits (and, if asked, the residual stream after every
layer).  ``dtype`` torch.float64 gives the yardstick for both engine types.

Notation: T tokens, D width, H query heads, G key/value heads, d the size of a
query or key head, e the size of a value head.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def centred_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The model's norm: its weight is stored as a difference from one."""
    return unit_rms(x, eps) * (1.0 + w)


def rotary_frequencies(rot: dict, dtype=torch.float64) -> (torch.Tensor, float):
    """One frequency per rotated pair, and the factor on cosines and sines."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    amplitude = 1.0
    sc = rot.get("scaling")
    if sc:
        factor, original = float(sc["factor"]), float(sc["original"])

        def turning_point(turns: float) -> float:
            return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

        lo = max(math.floor(turning_point(float(sc["fast"]))), 0)
        hi = min(math.ceil(turning_point(float(sc["slow"]))), dims - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        f = f / factor * ramp + f * (1.0 - ramp)
        amplitude = 0.1 * math.log(factor) + 1.0
    return f.to(dtype), amplitude


def rotate(x: torch.Tensor, positions: torch.Tensor, rot: Optional[dict]) -> torch.Tensor:
    """x [T, heads, d]; feature i of the first ``dims`` goes with feature i + dims / 2."""
    if not rot:
        return x
    dims = int(rot["dims"])
    f, amplitude = rotary_frequencies(rot, x.dtype)
    angle = positions.to(x.dtype)[:, None] * f[None, :]
    c, s = (torch.cos(angle) * amplitude)[:, None, :], (torch.sin(angle) * amplitude)[:, None, :]
    half = dims // 2
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def visible(T: int, mask: Optional[dict]) -> torch.Tensor:
    """[T, T] bool: may position i (row) see position j (column)?"""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if mask and mask.get("size"):
        size = int(mask["size"])
        ok = ok & (i // size == j // size)
    return ok


def keys_and_values(h: torch.Tensor, mixer: dict, w: Dict[str, torch.Tensor], prefix: str, eps: float):
    """What a layer with projections of its own puts into its cache: rotated, unit keys and values."""
    T = h.shape[0]
    G, d, e = int(mixer["kv_heads"]), int(mixer["dim"]), int(mixer["vdim"])
    pos = torch.arange(T)
    k = (h @ w[prefix + "k"].T).view(T, G, d)
    v = (h @ w[prefix + "v"].T).view(T, G, e)
    k = unit_rms(rotate(k, pos, mixer.get("rot")), eps)
    return k, v


def attention(h: torch.Tensor, mixer: dict, w: Dict[str, torch.Tensor], prefix: str, eps: float, k, v) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, e = int(mixer["heads"]), int(mixer["kv_heads"]), int(mixer["dim"]), int(mixer["vdim"])
    q = (h @ w[prefix + "q"].T).view(T, H, d)
    q = unit_rms(rotate(q, torch.arange(T), mixer.get("rot")), eps)
    ok = visible(T, mixer.get("mask"))
    out = torch.zeros(T, H, e, dtype=h.dtype)
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * float(mixer["scale"])
        s = s.masked_fill(~ok, float("-inf"))
        out[:, head] = torch.softmax(s, dim=-1) @ v[:, g]
    return out.reshape(T, H * e) @ w[prefix + "o"].T


def dense_feed_forward(h: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str) -> torch.Tensor:
    gate = h @ w[prefix + "gate"].T + w[prefix + "gate.b"]
    up = h @ w[prefix + "up"].T + w[prefix + "up.b"]
    return (gelu_tanh(gate) * up) @ w[prefix + "down"].T + w[prefix + "down.b"]


def routed_feed_forward(h: torch.Tensor, tokens: torch.Tensor, mlp: dict, w: Dict[str, torch.Tensor],
                        prefix: str) -> torch.Tensor:
    """Experts chosen by a table from the token id, each with weight 1 / top."""
    top = int(mlp["router"]["top"])
    table = w[prefix + "table"]
    out = torch.zeros(h.shape[0], w[prefix + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for slot in range(top):
            e = int(table[int(tokens[t]), slot])
            p = f"{prefix}e{e}."
            x = h[t]
            out[t] += ((silu(w[p + "gate"] @ x) * (w[p + "up"] @ x)) @ w[p + "down"].T) / top
    return out


def token_side_input(x: torch.Tensor, tokens: torch.Tensor, layer: int, side_dim: int, m: float, eps: float,
                     w: Dict[str, torch.Tensor]) -> torch.Tensor:
    p = f"l{layer}.side."
    e = w["side.embed"][tokens.long(), layer * side_dim:(layer + 1) * side_dim]
    g = gelu_tanh(x @ w[p + "gate"].T) * e
    y = g @ w[p + "proj"].T
    return x + m * unit_rms(y, eps) * w[p + "norm"]


def forward(config: dict, weights: Dict[str, torch.Tensor], tokens, dtype=torch.float64, layer_outputs: Optional[List] = None):
    """Logits [T, vocab] of one whole sequence."""
    w = {n: (t.to(dtype) if t.is_floating_point() else t) for n, t in weights.items()}
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    eps = float(config["norm"]["eps"])
    m = float(config.get("residual_mult", 1.0))
    x = w["embed"][tokens] * float((config.get("embedding") or {}).get("scale", 1.0))
    side = config.get("token_side")
    held = {}
    for i, layer in enumerate(config["layers"]):
        mixer = layer["mixer"]
        h = centred_norm(x, w[f"l{i}.norm1"], eps)
        src = mixer.get("kv_from")
        if src is None:
            held[i] = keys_and_values(h, mixer, w, f"l{i}.mix.", eps)
        k, v = held[i if src is None else int(src)]
        y = attention(h, mixer, w, f"l{i}.mix.", eps, k, v)
        mlp = layer.get("mlp")
        if mlp is not None:
            if mlp["kind"] == "dense":
                y = y + dense_feed_forward(h, w, f"l{i}.mlp.")
            else:
                y = y + routed_feed_forward(h, tokens, mlp, w, f"l{i}.mlp.")
        x = x + m * y
        if side:
            x = token_side_input(x, tokens, i, int(side["dim"]), m, eps, w)
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    h = centred_norm(x, w["final.norm"], eps)
    logits = h @ w["head"].T
    cap = config.get("logit_softcap")
    if cap:
        logits = float(cap) * torch.tanh(logits / float(cap))
    return logits
