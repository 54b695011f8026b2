"""Fokurax on the GPU against the plain implementation of the design
(tests/plain_fokurax.py): each mechanism's kernel alone, then whole models through
the step function -- whole prompts, the last tokens one by one, portions down to
two tokens, mixed batches with reused pages and slots, long decoding -- then greedy
generation through the package's entry point and the trace program."""
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import fokurax_models
import helpers
import plain_fokurax as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.fixture(scope="module")
def kernels():
    from chibillm_b200.kernels.ops import CudaKernels
    return CudaKernels(torch.device(DEV))


def close(got, ref, tol, what):
    got, ref = got.double().cpu(), ref.double().cpu()
    assert torch.isfinite(got).all(), f"{what}: not finite"
    worst = float((got - ref).abs().max())
    scale = float(ref.abs().max())
    assert worst <= tol * max(scale, 1e-30), f"{what}: max |diff| {worst:.3e} > {tol:.1e} * {scale:.3e}"


# ------------------------------------------------------------------ rotation, norm, append, attention in blocks
def run_attention(kernels, q_all, k_all, v_all, rot, eps, scale, chunk, dtype, page_size, portions, unit_norm=True):
    """Feeds one sequence's q | k | v in portions through the head kernel and the attention
    kernel (pages in a scrambled order, the sequence on row 1 of the table); returns the
    output [T, H, e] and the cached keys [T, G, d]."""
    dt = DTYPES[dtype]
    T, H, d = q_all.shape
    G, e = k_all.shape[1], v_all.shape[2]
    pages = (T + page_size - 1) // page_size + 3
    keys = torch.full((pages, G, page_size, d), float("nan"), dtype=dt, device=DEV)
    values = torch.full((pages, G, page_size, e), float("nan"), dtype=dt, device=DEV)
    order = torch.randperm(pages, generator=torch.Generator().manual_seed(5))
    table = torch.full((2, pages), -1, dtype=torch.int32, device=DEV)
    table[1, :pages] = order.to(torch.int32).to(DEV)
    rows = torch.tensor([1], dtype=torch.int32, device=DEV)
    qkv = torch.cat([q_all.reshape(T, H * d), k_all.reshape(T, G * d), v_all.reshape(T, G * e)], dim=1).to(dt)
    inv_freq, amplitude, dims = None, 1.0, 0
    if rot is not None:
        f, amplitude = plain.rotary_frequencies(rot)
        inv_freq, dims = f.float().to(DEV), rot["dims"]
    out_all = torch.zeros(T, H, e)
    for a, b in portions:
        n = b - a
        positions = torch.arange(a, b, dtype=torch.int32, device=DEV)
        seq_of = torch.zeros(n, dtype=torch.int32, device=DEV)
        q = torch.empty(n, H * d, dtype=dt, device=DEV)
        kernels.heads_rotate_append(qkv[a:b].to(DEV), q, keys, values, inv_freq, dims, amplitude, unit_norm, eps,
                                    positions, seq_of, table, H, G, d, e, page_size, rows)
        out = torch.empty(n, H * e, dtype=dt, device=DEV)
        kernels.attention(q, keys, values, out, table, torch.tensor([0, n], dtype=torch.int32, device=DEV),
                          torch.tensor([b], dtype=torch.int32, device=DEV), seq_of, positions, H, G, d, page_size,
                          scale, None, n, b, n, rows, chunk=chunk, value_dim=e if e != d else None)
        out_all[a:b] = out.float().cpu().view(n, H, e)
    idx = torch.arange(T)
    held = keys[order[idx // page_size].to(DEV), :, (idx % page_size).to(DEV), :].float().cpu()
    return out_all, held


def attention_reference(q, k, v, rot, eps, scale, chunk, unit_norm=True):
    T, H, d = q.shape
    G = k.shape[1]
    pos = torch.arange(T)
    q, k = plain.rotate(q.double(), pos, rot), plain.rotate(k.double(), pos, rot)
    if unit_norm:
        q, k = plain.unit_rms(q, eps), plain.unit_rms(k, eps)
    ok = plain.visible(T, {"size": chunk} if chunk else None)
    out = torch.zeros(T, H, v.shape[2], dtype=torch.float64)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T * scale).masked_fill(~ok, float("-inf"))
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, g].double()
    return out, k


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,d,e,chunk,dims,factor", [
    (4, 2, 16, 16, 7, 8, None), (3, 1, 48, 32, 40, 48, 4.0), (2, 2, 64, 64, 50, 32, 8.0), (6, 3, 80, 24, None, 40, 2.0),
    (2, 1, 128, 128, 128, 64, 8.0), (4, 1, 128, 128, 33, 128, None), (1, 1, 40, 72, 16, 0, None)])
def test_rotation_norm_and_attention_in_blocks(kernels, dtype, H, G, d, e, chunk, dims, factor):
    """The head kernel (rotation with amplitude, then the norm without a weight) and
    attention inside blocks of positions, with value heads of their own size, against the
    plain functions: whole, in portions that cut blocks and pages, and token by token."""
    g = torch.Generator().manual_seed(d + e)
    T, page_size = 300, 8
    dt = DTYPES[dtype]
    q = torch.randn(T, H, d, generator=g).to(dt)
    k = torch.randn(T, G, d, generator=g).to(dt)
    v = torch.randn(T, G, e, generator=g).to(dt)
    rot = None if not dims else fokurax_models.rot(dims, 500.0, factor, original=32, fast=8.0)
    scale, eps = 6.0 / math.sqrt(d), 1e-5
    ref, ref_keys = attention_reference(q, k, v, rot, eps, scale, chunk)
    tol = 2e-5 if dtype == "float32" else 2e-2
    for variant in ((1, 2) if dtype == "bfloat16" and d in (64, 128) and e == d else (0,)):
        kernels.tcgen05_attention_variant = variant
        try:
            whole, held = run_attention(kernels, q, k, v, rot, eps, scale, chunk, dtype, page_size, [(0, T)])
        finally:
            kernels.tcgen05_attention_variant = 0
        close(whole, ref, tol, f"attention whole, variant {variant}")
        close(held, ref_keys, 1e-5 if dtype == "float32" else 1e-2, "keys as the cache holds them")
    cuts = [(0, 61), (61, 63), (63, 64), (64, 199), (199, 201), (201, 260)] + [(i, i + 1) for i in range(260, T)]
    cut_up, _ = run_attention(kernels, q, k, v, rot, eps, scale, chunk, dtype, page_size, cuts)
    close(cut_up, ref, tol, "attention in portions and single tokens")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("d", [64, 80])
def test_attention_sees_its_block_and_nothing_before(kernels, dtype, d):
    """Keys are made to stand out: one far back but inside the query's block (next to a
    page border), one right before the block's first position.  The first must take the
    weight, the second must not be seen, in a prompt and for a token decoded alone."""
    H = G = 2
    T, page_size, chunk = 700, 16, 180
    g = torch.Generator().manual_seed(3)
    q = torch.randn(T, H, d, generator=g) * 0.3
    k = torch.randn(T, G, d, generator=g) * 0.3
    v = torch.randn(T, G, d, generator=g)
    direction = torch.randn(d, generator=g)
    direction /= direction.norm()
    inside, outside = 3 * chunk + 19, 3 * chunk - 1             # positions 559 (a page's last) and 539; queries at 699 and 660
    k[inside] = 8 * direction
    k[outside] = 8 * direction
    k[3 * chunk] = 8 * direction                                  # the block's first position
    for t in (T - 1, T - 40, 3 * chunk):
        q[t] = 8 * direction
    dt = DTYPES[dtype]
    q, k, v = q.to(dt), k.to(dt), v.to(dt)
    scale = 0.5                                                   # a marked pair scores 32, any other about 0
    ref, _ = attention_reference(q, k, v, None, 1e-6, scale, chunk, unit_norm=False)
    # the block's first query sees only itself; the later ones share the weight between the two marked keys inside
    assert float((ref[3 * chunk, 0] - v[3 * chunk, 0].double()).abs().max()) < 1e-9
    both = (v[inside, 0].double() + v[3 * chunk, 0].double()) / 2
    assert float((ref[T - 1, 0] - both).abs().max()) < 0.05 * float(both.abs().max())
    got, _ = run_attention(kernels, q, k, v, None, 1e-6, scale, chunk, dtype, page_size, [(0, T - 1), (T - 1, T)],
                           unit_norm=False)
    tol = 2e-5 if dtype == "float32" else 2e-2
    for t, what in ((T - 1, "decoded token"), (T - 40, "inside a prompt"), (3 * chunk, "a block's first position"),
                    (3 * chunk - 1, "a block's last position")):
        close(got[t], ref[t], tol, f"marked keys, {what}")
    close(got, ref, tol, "marked keys, all rows")
    # the same without blocks: the key right before the block is seen again
    free, _ = attention_reference(q, k, v, None, 1e-6, scale, None, unit_norm=False)
    got, _ = run_attention(kernels, q, k, v, None, 1e-6, scale, None, dtype, page_size, [(0, T - 1), (T - 1, T)],
                           unit_norm=False)
    close(got, free, tol, "marked keys, no blocks")
    assert float((free[T - 1] - ref[T - 1]).abs().max()) > 0.1


@pytest.mark.parametrize("chunk", [1024, 300, 4096])
@pytest.mark.parametrize("d", [64, 128])
def test_a_short_portion_after_a_long_context(kernels, d, chunk):
    """A portion of 110 tokens after 1,990: the tcgen05 prompt kernel cuts the keys of its few
    rows into ranges for several CTAs and merges them.  With blocks of 1,024 the rows' keys
    begin inside the context, with blocks of 300 most ranges are empty, with blocks of 4,096
    nothing is cut off; then single tokens (the split-key decode kernel) from 2,100 on."""
    H, G, T, page_size = 4, 1, 2110, 16
    g = torch.Generator().manual_seed(chunk + d)
    q = torch.randn(T, H, d, generator=g).bfloat16()
    k = torch.randn(T, G, d, generator=g).bfloat16()
    v = torch.randn(T, G, d, generator=g).bfloat16()
    rot = fokurax_models.rot(d // 2, 10000.0, 8.0, original=256)
    scale, eps = 4.0 / math.sqrt(d), 1e-5
    ref, _ = attention_reference(q, k, v, rot, eps, scale, chunk)
    cuts = [(0, 1990), (1990, 2100)] + [(i, i + 1) for i in range(2100, T)]
    got, _ = run_attention(kernels, q, k, v, rot, eps, scale, chunk, "bfloat16", page_size, cuts)
    close(got[1990:], ref[1990:], 2e-2, "a short portion and single tokens after a long context")
    close(got, ref, 2e-2, "all rows")


# ------------------------------------------------------------------ feed-forwards
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["gelu_tanh", "silu"])
def test_gated_activation_with_biases(kernels, dtype, kind):
    g = torch.Generator().manual_seed(1)
    dt = DTYPES[dtype]
    T = 37
    act = plain.gelu_tanh if kind == "gelu_tanh" else plain.silu
    for n in (50, 56):                       # 56 columns: bfloat16 rows take the kernel with 16-byte accesses
        gate_up = (torch.randn(T, 2 * n, generator=g) * 2).to(dt)
        bias = torch.randn(2 * n, generator=g).to(dt)
        for b in (bias, None):
            gu = gate_up.double() + (b.double() if b is not None else 0.0)
            ref = act(gu[:, :n]) * gu[:, n:]
            out = torch.empty(T, n, dtype=dt, device=DEV)
            kernels.gated_activation(gate_up.to(DEV), b.to(DEV) if b is not None else None, out, kind)
            close(out, ref, 1e-6 if dtype == "float32" else 1e-2, f"gated activation {kind}, {n} columns")
    # blocks of 16 gate columns, each followed by its 16 up columns
    n = 48
    gate_up = (torch.randn(T, 2 * n, generator=g) * 2).to(dt)
    blocks = gate_up.double().view(T, n // 16, 2, 16)
    ref = act(blocks[:, :, 0].reshape(T, n)) * blocks[:, :, 1].reshape(T, n)
    out = torch.empty(T, n, dtype=dt, device=DEV)
    kernels.gated_activation(gate_up.to(DEV), None, out, kind, interleaved=True)
    close(out, ref, 1e-6 if dtype == "float32" else 1e-2, f"gated activation {kind}, interleaved")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,D,F,E,top", [(1, 64, 40, 5, 2), (9, 96, 24, 3, 3), (300, 80, 100, 7, 1), (700, 128, 64, 4, 2),
                                         (33, 72, 130, 12, 5), (3, 96, 32, 6, 2), (1000, 160, 96, 5, 3),
                                         (130, 256, 224, 3, 1), (70, 192, 128, 4, 2), (5, 256, 320, 9, 3),
                                         (300, 192, 128, 5, 3), (2048, 256, 192, 8, 2), (1, 128, 64, 4, 2)])
def test_experts_chosen_by_a_table(kernels, dtype, T, D, F, E, top):
    """Few tokens (every tile holds a row or two), many (several tiles an expert), sizes
    that end inside a tile, tokens that repeat, experts that nobody uses.  With sizes that
    are multiples of 32 the bfloat16 runs take the tensor-core kernels (multiples of 64 and 256
    pairs or more: tcgen05, and once more with that switched off: mma.sync), else the plain one."""
    g = torch.Generator().manual_seed(T + E)
    dt = DTYPES[dtype]
    V = 50
    table = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(V)]).to(torch.int32)
    if E > 3:
        table[table == E - 1] = 0 if top == 1 else table[table == E - 1]       # with one choice: the last expert idle
    tokens = torch.randint(0, V, (T,), generator=g, dtype=torch.int32)
    x = torch.randn(T, D, generator=g).to(dt)
    w = {"m.table": table}
    for e in range(E):
        w[f"m.e{e}.gate"] = (torch.randn(F, D, generator=g) / math.sqrt(D)).to(dt)
        w[f"m.e{e}.up"] = (torch.randn(F, D, generator=g) / math.sqrt(D)).to(dt)
        w[f"m.e{e}.down"] = (torch.randn(D, F, generator=g) / math.sqrt(F)).to(dt)
    ref = plain.routed_feed_forward(x.double(), tokens, {"router": {"top": top}},
                                    {n: (t.double() if t.is_floating_point() else t) for n, t in w.items()}, "m.")
    fast = kernels.expert_tensor_cores(dt, D, F)
    if fast:        # blocks of 16 gate rows and their 16 up rows, as the tensor-core kernel wants them
        gate_up = torch.stack([kernels.interleave_expert_gate_up(w[f"m.e{e}.gate"], w[f"m.e{e}.up"])
                               for e in range(E)]).to(DEV)
    else:
        gate_up = torch.stack([torch.cat([w[f"m.e{e}.gate"], w[f"m.e{e}.up"]]) for e in range(E)]).to(DEV)
    down = torch.stack([w[f"m.e{e}.down"] for e in range(E)]).to(DEV)
    start = torch.randn(T, D, generator=g)
    route = torch.empty(kernels.route_words(T * top, E), dtype=torch.int32, device=DEV)
    act = torch.empty(T * top, F, dtype=dt, device=DEV)
    y = torch.empty(T * top, D, dtype=torch.float32, device=DEV)
    sorted_x = torch.empty(T * top, D, dtype=dt, device=DEV) if fast else None
    for tcgen05 in ((True, False) if fast else (True,)):
        kernels.use_tcgen05_experts = tcgen05
        try:
            acc = start.clone().to(DEV)
            act.fill_(float("nan"))
            y.fill_(float("nan"))
            kernels.routed_experts(x.to(DEV), tokens.to(DEV), table.to(DEV), gate_up, down, acc, route, act, y, "silu",
                                   1.0 / top, interleaved=fast, sorted_x=sorted_x)
            kernels.check_error_word()
        finally:
            kernels.use_tcgen05_experts = True
        close(acc.cpu() - start, ref, 2e-5 if dtype == "float32" else 2e-2, f"experts (tcgen05 {tcgen05})")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,D,side", [(3, 64, 5), (70, 96, 16), (200, 256, 24), (5, 1000, 3)])
def test_layer_end(kernels, dtype, T, D, side):
    """residual += m * delta, the token input, the next norm: in one kernel, and with the
    two small products taken from outside (``y_in``)."""
    g = torch.Generator().manual_seed(T)
    wt = DTYPES[dtype]
    V, layers, layer, m, eps = 40, 3, 1, 0.6, 1e-5
    w = {"side.embed": torch.randn(V, layers * side, generator=g).to(wt),
         "l1.side.gate": (torch.randn(side, D, generator=g) / math.sqrt(D)).to(wt),
         "l1.side.proj": (torch.randn(D, side, generator=g) / math.sqrt(side)).to(wt),
         "l1.side.norm": (0.5 + torch.rand(D, generator=g)).to(wt)}
    norm_w = ((torch.rand(D, generator=g) - 0.5) * 0.5).to(wt)
    tokens = torch.randint(0, V, (T,), generator=g, dtype=torch.int32)
    x0 = torch.randn(T, D, generator=g)
    delta = torch.randn(T, D, generator=g)
    x1 = x0.double() + m * delta.double()
    ref = plain.token_side_input(x1, tokens, layer, side, m, eps, {n: t.double() for n, t in w.items()})
    ref_norm = plain.centred_norm(ref, norm_w.double(), eps)
    args = (tokens.to(DEV), w["side.embed"].to(DEV), layer * side, w["l1.side.gate"].to(DEV), w["l1.side.proj"].to(DEV),
            w["l1.side.norm"].to(DEV), "gelu_tanh", eps)
    tol = 2e-6
    # all in one
    res = x0.clone().to(DEV)
    out = torch.empty(T, D, dtype=wt, device=DEV)
    kernels.layer_end(res, delta.to(DEV), m, side=args, norm=(norm_w.to(DEV), eps, 1.0, out))
    close(res, ref, tol, "layer end, residual")
    close(out, ref_norm, tol if dtype == "float32" else 1e-2, "layer end, next norm")
    # the update alone, then the token input from y computed outside
    res = x0.clone().to(DEV)
    copy = torch.empty(T, D, dtype=wt, device=DEV)
    kernels.layer_end(res, delta.to(DEV), m, copy_out=copy)
    close(res, x1, 1e-7, "layer end, update only")
    assert torch.equal(copy, res.to(wt))
    e = w["side.embed"][tokens.long(), layer * side:(layer + 1) * side].double()
    y = ((plain.gelu_tanh(x1 @ w["l1.side.gate"].double().T) * e) @ w["l1.side.proj"].double().T).float()
    kernels.layer_end(res, None, m, side=args, y_in=y.to(DEV))
    close(res, ref, tol, "layer end, y from outside")
    # no token input at all, with the norm
    res = x0.clone().to(DEV)
    kernels.layer_end(res, delta.to(DEV), m, norm=(norm_w.to(DEV), eps, 1.0, out))
    close(out, plain.centred_norm(x1, norm_w.double(), eps), tol if dtype == "float32" else 1e-2, "layer end, norm only")
    gate = (x1 @ w["l1.side.gate"].double().T).to(wt)
    gd = gate.clone().to(DEV)
    kernels.side_gate(gd, tokens.to(DEV), w["side.embed"].to(DEV), layer * side, "gelu_tanh")
    close(gd, plain.gelu_tanh(gate.double()) * e, 1e-6 if dtype == "float32" else 1e-2, "side gate")


def test_softcap_and_zero(kernels):
    x = torch.randn(7, 33) * 30
    d = x.clone().to(DEV)
    kernels.softcap(d, 12.5)
    close(d, 12.5 * torch.tanh(x.double() / 12.5), 1e-6, "softcap")
    kernels.zero(d)
    assert float(d.abs().max()) == 0.0


# ------------------------------------------------------------------ whole models
CASES = {
    # name: (page size, request lengths, lengths of the mixed run)
    "F1": (4, [1, 33, 130, 260], [50, 100, 30, 128, 64, 90, 17]),
    "F2": (16, [2, 70, 131, 300], [1, 200, 33, 250, 64, 129, 7]),
    "F3": (16, [5, 129, 260, 400], [400, 31, 129, 64, 350, 3, 222]),
    "F4": (8, [3, 64, 129, 190], [150, 20, 65, 2, 180, 99, 40]),
    "F5": (16, [4, 66, 140, 300], [300, 20, 131, 64, 150, 2, 90]),
}
SEED = 21


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("fokurax")
    return {name: fokurax_models.write_model(fokurax_models.get(name), str(root / name), seed=SEED) for name in CASES}


@pytest.fixture(scope="module")
def expected():
    out = {}
    for name, (_, lengths, mixed_lengths) in CASES.items():
        cfg = fokurax_models.get(name)
        reqs = helpers.random_requests(cfg["vocab"], lengths, seed=100)
        mixed = helpers.random_requests(cfg["vocab"], mixed_lengths, seed=200)
        out[name] = (reqs, fokurax_models.plain_logits(cfg, SEED, reqs, torch.float32),
                     mixed, fokurax_models.plain_logits(cfg, SEED, mixed, torch.float32))
    return out


def make_runner(folder, dtype, page_size, pool_tokens, max_requests=4):
    from chibillm_b200.engine.runner import ModelRunner
    runner = ModelRunner.from_folder(folder, dtype=dtype, device=DEV, page_size=page_size,
                                     pool_tokens=pool_tokens, max_requests=max_requests)
    runner.storage.poison()
    return runner


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", list(CASES))
def test_cutting_and_batching(folders, expected, case, dtype):
    page_size, lengths, _ = CASES[case]
    reqs, ref, mixed_reqs, mixed_ref = expected[case]
    tol = helpers.TOL[dtype]
    runner = make_runner(folders[case], dtype, page_size, pool_tokens=helpers.round64(max(lengths)))
    for trace, what in ((helpers.trace_whole(reqs), "whole"),
                        (helpers.trace_last_decoded(reqs, 32), "last 32 decoded"),
                        (helpers.trace_portions(reqs, seed=2), "portions")):
        got = helpers.run_trace(runner, trace)
        helpers.assert_logits_close(got, ref, tol, f"fokurax {case} {dtype} {what}")
        runner.cache.check_invariants()
        assert not runner.cache.requests
    runner.runtime.kernels.check_error_word()
    pool = 640 if sum(helpers.round64(len(v)) for v in mixed_reqs.values()) > 640 else 384
    trace = helpers.trace_mixed(mixed_reqs, pool, seed=6)
    assert sum(helpers.round64(len(v)) for v in mixed_reqs.values()) > pool       # pages and slots are used again
    runner2 = make_runner(folders[case], dtype, page_size, pool)
    got = helpers.run_trace(runner2, trace)
    helpers.assert_logits_close(got, mixed_ref, tol, f"fokurax {case} {dtype} mixed")
    runner2.cache.check_invariants()
    assert not runner2.cache.requests


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_experts_sorted_on_the_host(folders, expected, dtype, monkeypatch):
    """Prompt steps whose experts are sorted on the host and run one after the other
    through the ordinary products (what large experts of sizes that the tcgen05 kernel of
    the routed rows does not take do), on a small model with that kernel switched off."""
    from chibillm_b200.parts.mlp import TableExperts
    monkeypatch.setattr(TableExperts, "MANY_PAIRS", 4)
    monkeypatch.setattr(TableExperts, "MUCH_WORK", 0)
    reqs, ref, mixed_reqs, mixed_ref = expected["F3"]
    runner = make_runner(folders["F3"], dtype, 16, 448)
    runner.runtime.kernels.use_tcgen05_experts = False
    got = helpers.run_trace(runner, helpers.trace_portions(reqs, seed=4))
    helpers.assert_logits_close(got, ref, helpers.TOL[dtype], f"fokurax F3 {dtype} experts sorted on the host")
    runner = make_runner(folders["F3"], dtype, 16, 640)
    runner.runtime.kernels.use_tcgen05_experts = False
    got = helpers.run_trace(runner, helpers.trace_mixed(mixed_reqs, 640, seed=6))
    helpers.assert_logits_close(got, mixed_ref, helpers.TOL[dtype], f"fokurax F3 {dtype} experts sorted on the host, mixed")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(folders, dtype):
    """Three tokens of prompt, then 300 tokens one by one (captured steps replayed):
    blocks of 24 positions begin and end a dozen times under single tokens."""
    cfg = fokurax_models.get("F1")
    reqs = helpers.random_requests(cfg["vocab"], [303], seed=9)
    ref = fokurax_models.plain_logits(cfg, SEED, reqs, torch.float32)
    runner = make_runner(folders["F1"], dtype, 4, 320)
    got = helpers.run_trace(runner, helpers.trace_last_decoded(reqs, 300))
    helpers.assert_logits_close(got, ref, helpers.TOL[dtype], f"fokurax F1 {dtype} long decoding")
    assert runner.graph_replays > 200


def test_greedy_generation_through_the_entry_point(folders):
    """``LLM.generate`` (scheduler, sampler, portions of 16 tokens, three requests at a
    time): every generated token is the plain implementation's best one, wherever that
    leads by more than the rounding of a 32-bit run."""
    from chibillm_b200 import LLM
    cfg = fokurax_models.get("F3")
    prompts = list(helpers.random_requests(cfg["vocab"], [5, 40, 23, 61], seed=12).values())
    llm = LLM(folders["F3"], dtype="float32", context_length=128, max_sequences=3, max_batch_tokens=48,
              prefill_chunk_tokens=16, page_size=16)
    outs = llm.generate(prompts, max_tokens=12, ignore_eos=True)
    for prompt, new in zip(prompts, outs):
        assert len(new) == 12
        ref = fokurax_models.plain_logits(cfg, SEED, {"a": prompt + new})["a"]
        for i, tok in enumerate(new):
            row = ref[len(prompt) + i - 1]
            top = torch.topk(row, 2).values
            if float(top[0] - top[1]) > 1e-4 * float(row.abs().max()):
                assert int(torch.argmax(row)) == tok, f"token {i} of a prompt of {len(prompt)}"


def test_trace_program(folders, tmp_path):
    """bin/trace_run on a Fokurax folder: portions, single tokens, two live requests."""
    cfg = fokurax_models.get("F4")
    reqs = helpers.random_requests(cfg["vocab"], [40, 21], seed=5)
    ref = fokurax_models.plain_logits(cfg, SEED, reqs, torch.float32)
    a, b = reqs["r0"], reqs["r1"]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[30:31], "want": [0]},
                                     {"id": "b", "tokens": b[:19], "want": [18]}], "end": []},
             {"step": 2, "entries": [{"id": "b", "tokens": b[19:], "want": [0, 1]},
                                     {"id": "a", "tokens": a[31:], "want": [8]}], "end": ["a", "b"]}]
    want = [[ref["r0"][0], ref["r0"][29]], [ref["r0"][30], ref["r1"][18]], [ref["r1"][19], ref["r1"][20], ref["r0"][39]]]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for dtype in ("float32", "bfloat16"):
        out_dir = str(tmp_path / dtype)
        proc = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folders["F4"],
                               "--dtype", dtype, "--out", out_dir, "--max-tokens", "128"],
                              input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True,
                              timeout=600)
        assert proc.returncode == 0, proc.stderr[-2000:]
        assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
        for i, rows in enumerate(want):
            got = torch.from_numpy(np.fromfile(os.path.join(out_dir, f"{i}.f32"), dtype="<f4").reshape(len(rows), -1))
            scale = float(torch.stack(rows).abs().max())
            assert float((got - torch.stack(rows)).abs().max()) <= helpers.TOL[dtype] * scale


def test_random_weights_made_on_the_device(tmp_path):
    """``ModelRunner.from_random`` makes on the device the values that ``write_random_model``
    stores (the expert tables included): both give the same logits."""
    from chibillm_b200.engine.batch import StepEntry
    from chibillm_b200.engine.runner import ModelRunner
    from chibillm_b200.weights import write_random_model
    cfg = fokurax_models.get("F4")
    folder = write_random_model(cfg, str(tmp_path / "random"), seed=6)
    ids = helpers.random_requests(cfg["vocab"], [50], seed=2)["r0"]
    a = ModelRunner.from_folder(folder, dtype="float32", device=DEV, page_size=8, pool_tokens=64)
    b = ModelRunner.from_random(cfg, seed=6, dtype="float32", device=DEV, page_size=8, pool_tokens=64)
    la = a.step([StepEntry("x", ids, list(range(50)))]).clone()
    lb = b.step([StepEntry("x", ids, list(range(50)))]).clone()
    assert torch.equal(la, lb)
