"""Small Gitipel configurations and random weights for the tests.

The configurations differ from one another in every size and option: width,
vocabulary (also odd ones), head counts and groups, head sizes (16 to 128,
also 24, 40, 48, 80 and 96), the rank of the decay input (also odd ones), taps
(none, 2, 3, 5),
layers without a feed-forward, layers that run once, three times, or not in a
loop at all, a loop that starts after the first layer or covers all layers,
caps, scales (also a negative one) and eps.  The weights are made here, with torch's generator, and
written with the ``safetensors`` library; nothing of the package takes part.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List

import torch


def attention(heads, kv_heads, dim, scale=None, softcap=20.0, ff=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim,
         "scale": scale if scale is not None else 1.0 / math.sqrt(dim)}
    if softcap is not None:
        m["softcap"] = softcap
    return {"type": "attention", "mixer": m, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def delta(heads, dim, rank, ff=None):
    # "rank" is not a key of the design's file: the readers take it from the tensor's shape
    return {"type": "general_delta", "mixer": {"heads": heads, "dim": dim}, "_rank": rank,
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


CONFIGS: Dict[str, dict] = {
    # grouped heads (2 : 1 and 3 : 1), an odd rank and vocabulary, a layer without a feed-forward, a
    # loop of three passes that starts after the first layer
    "G1": {"architecture": "Gitipel", "vocab": 211, "width": 64, "norm": {"eps": 1e-6},
           "embedding": {"scale": 2.5}, "logit_scale": 0.25, "canon": {"taps": 3},
           "layers": [attention(4, 2, 32, scale=0.3, softcap=8.0, ff=96), delta(2, 32, 5, ff=80),
                      attention(3, 1, 48, softcap=30.0), delta(3, 16, 8, ff=72)],
           "loop": {"start": 1, "stop": 3, "times": 3}},
    # no loop, no short convolution, no scales; one head per group, head size 64, one delta head
    "G2": {"architecture": "Gitipel", "vocab": 128, "width": 96, "norm": {"eps": 1e-5},
           "layers": [delta(1, 64, 4, ff=128), attention(2, 2, 64, softcap=None, ff=128),
                      attention(1, 1, 16, softcap=5.0, ff=64)]},
    # a loop over all layers that runs once, five taps, head size 128 in the recurrence
    "G3": {"architecture": "Gitipel", "vocab": 300, "width": 80, "norm": {"eps": 3e-6},
           "embedding": {"scale": 1.0}, "logit_scale": 2.0, "canon": {"taps": 5},
           "layers": [attention(5, 5, 16, softcap=12.0, ff=160), delta(1, 128, 16, ff=96)],
           "loop": {"start": 0, "stop": 2, "times": 1}},
    # two taps, sizes that the tensor-core kernels take whole (multiples of 128), prompts of many rows
    "G4": {"architecture": "Gitipel", "vocab": 512, "width": 256, "norm": {"eps": 1e-5},
           "embedding": {"scale": 4.0}, "logit_scale": 0.5, "canon": {"taps": 2},
           "layers": [attention(4, 2, 64, softcap=25.0, ff=512), delta(4, 64, 8, ff=256),
                      attention(2, 1, 128, softcap=40.0, ff=384)],
           "loop": {"start": 0, "stop": 2, "times": 2}},
    # sizes that are no power of two anywhere: head sizes 80 and 40 (five query heads on one key
    # head), recurrent heads of 24 and 96 channels, ranks 6 and 7, five taps, a negative scale
    "G5": {"architecture": "Gitipel", "vocab": 257, "width": 160, "norm": {"eps": 1e-5},
           "embedding": {"scale": -1.5}, "logit_scale": 1.0, "canon": {"taps": 5},
           "layers": [attention(5, 1, 80, softcap=15.0, ff=200), delta(3, 24, 6, ff=120),
                      attention(2, 2, 40, softcap=None, ff=96), delta(1, 96, 7)],
           "loop": {"start": 2, "stop": 4, "times": 2}},
}


def get(name: str) -> dict:
    return json.loads(json.dumps(CONFIGS[name]))


def file_config(config: dict) -> dict:
    """The configuration as the design's file holds it (without this module's own keys)."""
    out = json.loads(json.dumps(config))
    for layer in out["layers"]:
        layer.pop("_rank", None)
    return out


def random_weights(config: dict, seed: int, dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    D, V = config["width"], config["vocab"]

    def normal(*shape, std):
        return (torch.randn(*shape, generator=g) * std).to(dtype)

    def uniform(n, lo, hi):
        return (lo + torch.rand(n, generator=g) * (hi - lo)).to(dtype)

    def matrix(out, inp):
        return normal(out, inp, std=1.0 / math.sqrt(inp))

    w = {"embed": normal(V, D, std=1.0), "final.norm": uniform(D, 0.7, 1.3), "head": matrix(V, D)}
    if config.get("loop"):
        w["loop.in"] = matrix(D, 2 * D)
        w["loop.step"] = normal(config["loop"]["times"], D, std=0.5)
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        w[p + "norm1"] = uniform(D, 0.7, 1.3)
        if config.get("canon"):
            w[p + "canon1"] = normal(D, config["canon"]["taps"], std=0.4)
        if layer["type"] == "attention":
            w[p + "mix.q"] = matrix(m["heads"] * m["dim"], D)
            w[p + "mix.k"] = matrix(m["kv_heads"] * m["dim"], D)
            w[p + "mix.o"] = matrix(D, m["heads"] * m["dim"])
            w[p + "mix.r1"] = uniform(m["heads"], 0.0, 2.0)
            w[p + "mix.r2"] = uniform(m["heads"], 0.1, 0.5)
        else:
            W, rank = m["heads"] * m["dim"], layer["_rank"]
            for name in ("r", "k", "v", "g", "a"):
                w[p + "mix." + name] = matrix(W, D)
            w[p + "mix.a.b"] = uniform(W, -2.0, 2.0)
            w[p + "mix.w1"] = matrix(rank, D)
            w[p + "mix.w2"] = normal(W, rank, std=1.0)
            w[p + "mix.w0"] = uniform(W, -6.0, 0.0)
            w[p + "mix.norm"] = uniform(W, 0.6, 1.4)
            w[p + "mix.o"] = matrix(D, W)
        if layer["mlp"] is not None:
            w[p + "norm2"] = uniform(D, 0.7, 1.3)
            w[p + "mlp.up"] = matrix(layer["mlp"]["ff"], D)
            w[p + "mlp.down"] = matrix(D, layer["mlp"]["ff"])
    return w


def write_model(config: dict, folder: str, seed: int, dtype=torch.bfloat16) -> str:
    from safetensors.torch import save_file

    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(file_config(config), f, indent=1)
    save_file({k: v.contiguous() for k, v in random_weights(config, seed, dtype).items()},
              os.path.join(folder, "model.safetensors"))
    return folder


def plain_logits(config: dict, seed: int, requests: Dict[str, List[int]], dtype=torch.float64,
                 stored=torch.bfloat16) -> Dict[str, torch.Tensor]:
    """The plain implementation on the weights that ``write_model`` stores."""
    import plain_gitipel

    w = {k: v.to(dtype) for k, v in random_weights(config, seed, stored).items()}
    cfg = file_config(config)
    return {rid: plain_gitipel.forward(cfg, w, ids).float() for rid, ids in requests.items()}
