"""Small Fokurax configurations and random weights for the tests.

The configurations differ from one another in every size and option: width and
vocabulary (also odd ones), head counts and groups, key sizes 16 to 128 (also
24, 40, 48, 80), value sizes equal to the key size and not, rotations over the
whole head and over a part of it, with and without stretched frequencies and
without any rotation, blocks of 5 to 128 positions and no blocks at all, layers
that read the cache of a layer right before them or further back, layers
without a feed-forward, dense ones, experts with one, two and three choices out
of 3 to 10, with and without the token input, the logit cap and the scales.
The token input has 11 features or more in these models: with 3 to 8 of them the direction
of y = P g hangs on so few rounded numbers that, after y is divided by its root mean square,
single positions of a bfloat16 run are 3 to 19 % of the largest logit away from the 32-bit
result -- in the arithmetic of the stand-in kernels just as on the device -- while the median
position stays at 0.3 %; the kernel's own test covers 3 and 5 features.
The weights are made here, with torch's generator, and written with the
``safetensors`` library; nothing of the package takes part.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional

import torch


def rot(dims, base=10000.0, factor=None, original=64, fast=12.0, slow=1.5):
    r = {"base": base, "dims": dims}
    if factor is not None:
        r["scaling"] = {"factor": factor, "original": original, "fast": fast, "slow": slow}
    return r


def layer(heads, kv_heads, dim, vdim=None, chunk=None, rotation=None, scale=None, kv_from=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim if vdim is None else vdim,
         "scale": scale if scale is not None else 2.0 / math.sqrt(dim)}
    if chunk is not None:
        m["mask"] = {"size": chunk}
    if rotation is not None:
        m["rot"] = rotation
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


CONFIGS: Dict[str, dict] = {
    # value heads smaller than key heads, two choices of five experts, blocks of 24 positions, a part of the
    # head rotated with stretched frequencies, the third layer reads the first one's cache
    "F1": {"architecture": "Fokurax", "vocab": 211, "width": 64, "norm": {"eps": 1e-6}, "embedding": {"scale": 3.0},
           "residual_mult": 0.7, "logit_softcap": 9.0, "token_side": {"dim": 13},
           "layers": [layer(4, 2, 32, vdim=16, chunk=24, rotation=rot(16, 5000.0, factor=4.0, original=32), mlp=dense(96)),
                      layer(4, 2, 32, vdim=16, chunk=24, rotation=rot(16, 5000.0, factor=4.0, original=32), mlp=moe(40, 5, 2)),
                      layer(4, 2, 32, vdim=16, chunk=24, rotation=rot(16, 5000.0, factor=4.0, original=32), kv_from=0,
                            mlp=moe(24, 3, 3))]},
    # no blocks, no stretching, the whole head rotated, no token input, no cap, no scales; a layer without a
    # feed-forward; one key head for three query heads; value heads larger than key heads
    "F2": {"architecture": "Fokurax", "vocab": 128, "width": 96, "norm": {"eps": 1e-5},
           "layers": [layer(3, 1, 48, vdim=64, rotation=rot(48, 100.0), mlp=moe(64, 4, 1)),
                      layer(3, 1, 48, vdim=64, rotation=rot(48, 100.0), kv_from=0),
                      layer(2, 2, 16, mlp=dense(80))]},
    # sizes that the tensor-core kernels take (head sizes 64 and 128, equal value size), blocks of 128 and of 50,
    # a reader right after its source and one two layers on, layers of different shapes
    "F3": {"architecture": "Fokurax", "vocab": 512, "width": 256, "norm": {"eps": 2e-5}, "embedding": {"scale": 8.0},
           "residual_mult": 0.6, "logit_softcap": 20.0, "token_side": {"dim": 16},
           "layers": [layer(4, 2, 64, chunk=128, rotation=rot(32, 30000.0, factor=6.0, original=128, fast=16.0, slow=2.0),
                            mlp=moe(128, 10, 2)),
                      layer(4, 2, 64, chunk=128, rotation=rot(32, 30000.0, factor=6.0, original=128, fast=16.0, slow=2.0),
                            kv_from=0, mlp=dense(384)),
                      layer(2, 1, 128, chunk=50, rotation=rot(128, 1000.0), mlp=moe(64, 6, 1)),
                      layer(2, 1, 128, chunk=50, rotation=rot(128, 1000.0), kv_from=2, mlp=moe(64, 6, 3))]},
    # sizes that are no power of two anywhere: five query heads on one key head of 80, values of 40, blocks of 5
    # positions (shorter than a page), an odd vocabulary, seven experts
    "F4": {"architecture": "Fokurax", "vocab": 257, "width": 160, "norm": {"eps": 3e-6}, "embedding": {"scale": -1.5},
           "residual_mult": 1.0, "logit_softcap": 30.0, "token_side": {"dim": 11},
           "layers": [layer(5, 1, 80, vdim=40, chunk=5, rotation=rot(40, 300.0, factor=2.0, original=16, fast=4.0), mlp=moe(56, 7, 2)),
                      layer(2, 2, 24, vdim=24, chunk=37, rotation=rot(24, 777.0), mlp=dense(200)),
                      layer(5, 1, 80, vdim=40, chunk=5, rotation=rot(40, 300.0, factor=2.0, original=16, fast=4.0), kv_from=0)]},
    # one layer, one head, no rotation
    "F5": {"architecture": "Fokurax", "vocab": 97, "width": 48, "norm": {"eps": 1e-5}, "residual_mult": 1.25,
           "token_side": {"dim": 16},
           "layers": [layer(1, 1, 40, vdim=8, chunk=64, mlp=moe(32, 3, 2))]},
}


def get(name: str) -> dict:
    return json.loads(json.dumps(CONFIGS[name]))


def random_weights(config: dict, seed: int, dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    D, V = config["width"], config["vocab"]

    def normal(*shape, std):
        return (torch.randn(*shape, generator=g) * std).to(dtype)

    def matrix(out, inp, gain=1.0):
        return normal(out, inp, std=gain / math.sqrt(inp))

    def around_zero(n):
        return ((torch.rand(n, generator=g) - 0.5) * 0.6).to(dtype)

    layers = config["layers"]
    w = {"embed": normal(V, D, std=1.0), "final.norm": around_zero(D), "head": matrix(V, D)}
    side = (config.get("token_side") or {}).get("dim")
    if side:
        w["side.embed"] = normal(V, len(layers) * side, std=1.0)
    for i, l in enumerate(layers):
        p = f"l{i}."
        m = l["mixer"]
        w[p + "norm1"] = around_zero(D)
        w[p + "mix.q"] = matrix(m["heads"] * m["dim"], D)
        if "kv_from" not in m:
            w[p + "mix.k"] = matrix(m["kv_heads"] * m["dim"], D)
            w[p + "mix.v"] = matrix(m["kv_heads"] * m["vdim"], D)
        w[p + "mix.o"] = matrix(D, m["heads"] * m["vdim"])
        mlp = l["mlp"]
        if mlp is not None and mlp["kind"] == "dense":
            for name, (o, n) in (("gate", (mlp["ff"], D)), ("up", (mlp["ff"], D)), ("down", (D, mlp["ff"]))):
                w[p + "mlp." + name] = matrix(o, n)
                w[p + "mlp." + name + ".b"] = normal(o, std=0.3)
        elif mlp is not None:
            E, top, ff = mlp["router"]["experts"], mlp["router"]["top"], mlp["expert"]["ff"]
            for e in range(E):
                w[f"{p}mlp.e{e}.gate"] = matrix(ff, D)
                w[f"{p}mlp.e{e}.up"] = matrix(ff, D)
                w[f"{p}mlp.e{e}.down"] = matrix(D, ff, gain=2.0)
            w[p + "mlp.table"] = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(V)]).to(torch.int32)
        if side:
            w[p + "side.gate"] = matrix(side, D)
            w[p + "side.proj"] = matrix(D, side)
            w[p + "side.norm"] = (0.5 + torch.rand(D, generator=g)).to(dtype)
    return w


def write_model(config: dict, folder: str, seed: int, dtype=torch.bfloat16, weights: Optional[dict] = None) -> str:
    from safetensors.torch import save_file

    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config, f, indent=1)
    weights = random_weights(config, seed, dtype) if weights is None else weights
    save_file({k: v.contiguous() for k, v in weights.items()}, os.path.join(folder, "model.safetensors"))
    return folder


def plain_logits(config: dict, seed: int, requests: Dict[str, List[int]], dtype=torch.float64, stored=torch.bfloat16,
                 weights: Optional[dict] = None) -> Dict[str, torch.Tensor]:
    """The plain implementation on the weights that ``write_model`` stores."""
    import plain_fokurax

    w = random_weights(config, seed, stored) if weights is None else weights
    return {rid: plain_fokurax.forward(config, w, ids, dtype).float() for rid, ids in requests.items()}
