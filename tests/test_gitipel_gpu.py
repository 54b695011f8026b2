"""Gitipel on the GPU against the plain implementation of the design
(tests/plain_gitipel.py): each mechanism's kernel alone, then whole models
through the step function -- whole prompts, the last tokens one by one,
portions down to two tokens, mixed batches with reused pages and state slots,
long decoding -- then greedy generation through the package's entry point and
the trace program."""
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import gitipel_models
import helpers
import plain_gitipel as plain

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


def cut(length, sizes, rng):
    """Portions of a sequence: sizes drawn from ``sizes`` until ``length`` is used up."""
    out, pos = [], 0
    while pos < length:
        n = min(sizes[int(rng.integers(len(sizes)))], length - pos)
        out.append((pos, pos + n))
        pos += n
    return out


def batches_of(lengths, sizes, seed):
    """Steps of a batch in which every sequence brings its next portion (a sequence that
    has ended drops out): [(sequence index, begin, end), ...] per step."""
    rng = np.random.default_rng(seed)
    cuts = [cut(n, sizes, rng) for n in lengths]
    steps = []
    for i in range(max(len(c) for c in cuts)):
        steps.append([(s, *c[i]) for s, c in enumerate(cuts) if i < len(c)])
    return steps


# ------------------------------------------------------------------ short convolution
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("taps", [1, 2, 4, 7])
def test_short_conv_kernel(kernels, dtype, taps):
    """Whole sequences against portions of 1, 2, 3 and 20 tokens (shorter than the
    history too), several sequences a step, slots in another order than the batch."""
    g = torch.Generator().manual_seed(taps)
    # 70 channels take the kernel with one channel per thread, 72 (with the transposed weight) the wide one
    D, lengths, slots = (70 if taps % 2 else 72), [1, 2, 9, 45, 30], [3, 0, 4, 1, 2]
    dt = DTYPES[dtype]
    w = (torch.randn(D, taps, generator=g) * 0.5)
    xs = [torch.randn(n, D, generator=g).to(dt) for n in lengths]
    ref = [plain.short_convolution(x.double(), w.double()) for x in xs]
    history = torch.full((5, max(taps - 1, 1), D), float("nan"), dtype=dt, device=DEV)
    for rounds in range(2):                         # the second round meets slots that were used before
        history[:] = float("nan")
        history[slots] = 0                          # what admitting a request does
        got = [torch.zeros(n, D, dtype=dt) for n in lengths]
        for step in batches_of(lengths, [1, 2, 3, 20], seed=taps + rounds):
            x = torch.cat([xs[s][a:b] for s, a, b in step]).to(DEV)
            q_start = torch.tensor(np.cumsum([0] + [b - a for _, a, b in step]), dtype=torch.int32, device=DEV)
            slot_t = torch.tensor([slots[s] for s, _, _ in step], dtype=torch.int32, device=DEV)
            out = torch.empty_like(x)
            kernels.short_conv(x, w.to(DEV), history, out, q_start, None, slot_t, max(b - a for _, a, b in step),
                               weight_t=w.t().contiguous().to(DEV))
            at = 0
            for s, a, b in step:
                got[s][a:b] = out[at:at + b - a].cpu()
                at += b - a
        for s in range(len(lengths)):
            close(got[s], ref[s], 1e-6 if dtype == "float32" else 1e-2, f"short_conv taps {taps} seq {s}")


# ------------------------------------------------------------------ delta rule
def delta_reference(proj, w2, w0, ab, heads, d, rank, decay_scale, key_eps, state=None):
    W = heads * d
    p = proj.double()
    T = p.shape[0]
    r, k, v = p[:, :W], p[:, W:2 * W], p[:, 2 * W:3 * W]
    decay, a, u = plain.delta_rule_inputs(p[:, 5 * W:], p[:, 4 * W:5 * W], k, w2.double(), w0.double(), ab.double(),
                                          decay_scale, key_eps, heads, d)
    return plain.delta_rule_recurrence(r.view(T, heads, d), k.reshape(T, heads, d), v.reshape(T, heads, d), decay, a, u,
                                       state)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,d,rank", [(2, 16, 5), (1, 32, 8), (3, 48, 3), (2, 64, 16), (1, 128, 4), (1, 200, 6)])
def test_delta_rule_kernel(kernels, dtype, heads, d, rank):
    """The recurrence over whole sequences and over portions (single tokens too) with
    the state carried in its slot, against the plain loop; then a slot used again."""
    g = torch.Generator().manual_seed(d)
    dt = DTYPES[dtype]
    W = heads * d
    lengths, slots = [1, 37, 20], [2, 0, 1]
    w2 = torch.randn(W, rank, generator=g)
    w0 = -6.0 * torch.rand(W, generator=g)
    ab = 4.0 * torch.rand(W, generator=g) - 2.0
    projs = [torch.randn(n, 5 * W + rank, generator=g).to(dt) for n in lengths]
    scale, eps = math.exp(-0.5), 1e-6
    refs = [delta_reference(p, w2, w0, ab, heads, d, rank, scale, eps) for p in projs]
    state = torch.full((3, heads, d, d), float("nan"), dtype=torch.float32, device=DEV)
    # the decay's logits come from the small kernel, in the third round ready made (as a step of many tokens has them)
    for sizes, ready in (([64], False), ([1, 2, 5, 17], False), ([64], True)):
        state[:] = 0
        got = [torch.zeros(n, W) for n in lengths]
        for step in batches_of(lengths, sizes, seed=rank):
            proj = torch.cat([projs[s][a:b] for s, a, b in step]).to(DEV)
            q_start = torch.tensor(np.cumsum([0] + [b - a for _, a, b in step]), dtype=torch.int32, device=DEV)
            slot_t = torch.tensor([slots[s] for s, _, _ in step], dtype=torch.int32, device=DEV)
            o = torch.empty(proj.shape[0], W, dtype=torch.float32, device=DEV)
            logits = torch.empty(proj.shape[0], W, dtype=torch.float32, device=DEV)
            if ready:
                logits.copy_((torch.tanh(proj[:, 5 * W:].double().cpu()) @ w2.double().t()).float())
            else:
                kernels.decay_logits(proj[:, 5 * W:], w2.t().contiguous().to(DEV), logits)
            kernels.delta_rule(proj, logits, w0.to(DEV), ab.to(DEV), state, o, q_start, slot_t, heads, d, rank,
                               scale, eps, max(b - a for _, a, b in step))
            at = 0
            for s, a, b in step:
                got[s][a:b] = o[at:at + b - a].cpu()
                at += b - a
        for s, n in enumerate(lengths):
            close(got[s], refs[s][0].reshape(n, W), 2e-5, f"delta rule d {d} portions {sizes} seq {s}")
            # the slot holds the last state, value index before key index
            close(state[slots[s]].transpose(1, 2), refs[s][1], 2e-5, f"delta rule d {d} state of seq {s}")


def test_delta_rule_forgets_and_removes(kernels):
    """Inputs made so that a fault shows: with decay near 1 and no removal a value
    written at the first token is read back 300 tokens later; when the last token
    removes fully along the same key, it is gone."""
    d, T = 32, 300
    W = d
    for removal, expect in ((-30.0, 1.0), (30.0, 0.0)):
        proj = torch.zeros(T, 5 * W + 1)
        key = torch.zeros(d)
        key[3] = 2.0
        proj[0, W:2 * W] = key                       # k of the first token
        proj[0, 2 * W:3 * W] = torch.arange(d).float()        # its value
        proj[1:, W:2 * W] = torch.eye(d)[5] * 1e-3   # later keys point elsewhere (and are tiny)
        proj[T - 1, W:2 * W] = key                   # the last token's key is the first one again (its value is 0)
        proj[T - 1, :W] = key                        # and it asks along that key
        proj[:, 4 * W:5 * W] = removal
        w2, w0, ab = torch.zeros(W, 1), torch.full((W,), -40.0), torch.zeros(W)      # decay = exp(-c * sigmoid(-40)) ~ 1
        state = torch.zeros(1, 1, d, d, device=DEV)
        o = torch.empty(T, W, device=DEV)
        q_start = torch.tensor([0, T], dtype=torch.int32, device=DEV)
        kernels.delta_rule(proj.to(DEV), torch.zeros(T, W, device=DEV), w0.to(DEV), ab.to(DEV), state, o, q_start,
                           torch.zeros(1, dtype=torch.int32, device=DEV), 1, d, 1, math.exp(-0.5), 1e-6, T)
        ref, _ = delta_reference(proj, w2, w0, ab, 1, d, 1, math.exp(-0.5), 1e-6)
        close(o[:T - 1], ref[:T - 1, 0], 1e-5, "delta rule, the tokens before the last")
        if expect:
            close(o[T - 1], ref[T - 1, 0], 1e-5, "delta rule far value")
        want = 4.0 * torch.arange(d).float() * expect       # (k . r) v = 4 v, if it is still there
        if expect:
            close(o[T - 1], want, 1e-3, "delta rule keeps a value")
        else:
            assert float(o[T - 1].abs().max()) < 1e-3


# ------------------------------------------------------------------ gated norm, activations
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gated_group_norm_kernel(kernels, dtype):
    g = torch.Generator().manual_seed(0)
    dt = DTYPES[dtype]
    for heads, d in ((3, 16), (2, 48), (1, 200), (3, 32), (2, 64), (1, 128)):
        T, W = 11, heads * d
        x = torch.randn(T, W, generator=g) * 3
        wide = torch.randn(T, 3 * W + 5, generator=g).to(dt)       # the gate is a column range of a wider array
        weight = 1 + 0.3 * torch.randn(W, generator=g)
        out = torch.empty(T, W, dtype=dt, device=DEV)
        wide_dev = wide.to(DEV)
        kernels.gated_group_norm(x.to(DEV), wide_dev[:, W:2 * W], weight.to(DEV), 1e-5, d, out)
        ref = plain.gated_head_norm(x.double().view(T, heads, d), wide[:, W:2 * W].double(), weight.double(), 1e-5)
        close(out, ref, 1e-6 if dtype == "float32" else 8e-3, f"gated norm {heads} x {d}")


def plain_activation(z, kind):
    if kind == "gelu":
        return plain.gelu(z)
    if kind == "gelu_tanh":
        return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))
    return z * torch.sigmoid(z) if kind == "silu" else z.clamp(min=0)


@pytest.mark.parametrize("kind", ["gelu", "gelu_tanh", "silu", "relu"])
def test_activation_kernels(kernels, kind):
    g = torch.Generator().manual_seed(1)
    z = torch.randn(7, 33, generator=g) * 3
    for dtype, tol in (("float32", 1e-6), ("bfloat16", 8e-3)):
        x = z.to(DTYPES[dtype]).to(DEV)
        kernels.activation(x, kind)
        close(x, plain_activation(z.to(DTYPES[dtype]).double(), kind), tol, f"activation {kind} {dtype}")
    # the product with the activation on its 32-bit sums: few rows (split product) and many rows (epilogue)
    for M, K, N in ((4, 256, 512), (300, 256, 512), (130, 192, 384)):
        a = torch.randn(M, K, generator=g).bfloat16()
        w = (torch.randn(N, K, generator=g) / math.sqrt(K)).bfloat16()
        out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
        if not kernels.linear_activation(a.to(DEV), w.to(DEV), out, kind):
            kernels.linear(a.to(DEV), w.to(DEV), out)
            kernels.activation(out, kind)
        close(out, plain_activation(a.double() @ w.double().t(), kind), 8e-3, f"linear + {kind}, {M} rows")


def test_scale_cast_rows_add_vector(kernels):
    g = torch.Generator().manual_seed(2)
    x = torch.randn(9, 20, generator=g)
    d = x.to(DEV)
    kernels.scale(d, 1.75)
    close(d, x * 1.75, 1e-7, "scale")
    wide = torch.zeros(9, 50, dtype=torch.bfloat16, device=DEV)
    kernels.cast_rows(x.to(DEV), wide[:, 20:40])
    close(wide[:, 20:40], x.bfloat16(), 0.0, "cast_rows")
    assert float(wide[:, :20].abs().max()) == 0 and float(wide[:, 40:].abs().max()) == 0
    vec = torch.randn(20, generator=g)
    d = x.to(DEV)
    kernels.add_row_vector(d, vec.to(DEV))
    close(d, x + vec, 1e-7, "add_row_vector")


# ------------------------------------------------------------------ attention with a cap, a bias and tied values
def run_attention(kernels, q_all, k_all, r1, r2, scale, softcap, dtype, page_size, portions):
    """Feeds one sequence's q | k in portions through the append and attention kernels
    (keys only in the cache, pages in a scrambled order); returns [T, H, d]."""
    dt = DTYPES[dtype]
    T, H, d = q_all.shape
    G = k_all.shape[1]
    pages = (T + page_size - 1) // page_size + 3
    cache = torch.full((pages, G, page_size, d), float("nan"), dtype=dt, device=DEV)
    order = torch.randperm(pages, generator=torch.Generator().manual_seed(5))
    table = torch.full((2, pages), -1, dtype=torch.int32, device=DEV)
    table[1, :pages] = order.to(torch.int32).to(DEV)
    rows = torch.tensor([1], dtype=torch.int32, device=DEV)
    out_all = torch.zeros(T, H, d)
    qk = torch.cat([q_all.reshape(T, H * d), k_all.reshape(T, G * d)], dim=1).to(dt)
    bias = None if r1 is None else (r1.float().to(DEV), r2.float().to(DEV))
    for a, b in portions:
        n = b - a
        positions = torch.arange(a, b, dtype=torch.int32, device=DEV)
        seq_of = torch.zeros(n, dtype=torch.int32, device=DEV)
        q = torch.empty(n, H * d, dtype=dt, device=DEV)
        kernels.qk_norm_rope_append(qk[a:b].to(DEV), q, cache, None, None, None, None, 0, 0.0, 0.0, positions, seq_of,
                                    table, H, G, d, page_size, rows)
        out = torch.empty(n, H * d, dtype=dt, device=DEV)
        kernels.attention(q, cache, cache, out, table, torch.tensor([0, n], dtype=torch.int32, device=DEV),
                          torch.tensor([b], dtype=torch.int32, device=DEV), seq_of, positions, H, G, d, page_size,
                          scale, None, n, b, n, rows, softcap=softcap, distance_bias=bias)
        out_all[a:b] = out.float().cpu().view(n, H, d)
    return out_all


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,d", [(4, 2, 16), (3, 1, 48), (2, 2, 64), (6, 3, 80), (2, 1, 128), (1, 1, 40)])
def test_attention_with_cap_bias_and_tied_values(kernels, dtype, H, G, d):
    g = torch.Generator().manual_seed(d)
    T, page_size = 150, 8
    dt = DTYPES[dtype]
    q = torch.randn(T, H, d, generator=g).to(dt)
    k = torch.randn(T, G, d, generator=g).to(dt)
    r1, r2 = 2 * torch.rand(H, generator=g), 0.1 + 0.4 * torch.rand(H, generator=g)
    scale = 3.0 / math.sqrt(d)                       # scores of a few units: the cap of 4 bends them
    for softcap, bias in ((4.0, True), (None, True), (4.0, False)):
        ref = plain.capped_distance_scores(q.double(), k.double(), r1.double() if bias else torch.zeros(H).double(),
                                           r2.double(), scale, softcap)
        tol = 2e-5 if dtype == "float32" else 2e-2
        # head sizes 64 and 128 in bfloat16 run prompts on tcgen05: both of its kernels (one and two
        # query tiles per CTA) are asked for in turn; 0 leaves the choice to the kernels
        for variant in ((1, 2) if dtype == "bfloat16" and d in (64, 128) else (0,)):
            kernels.tcgen05_attention_variant = variant
            try:
                whole = run_attention(kernels, q, k, r1 if bias else None, r2 if bias else None, scale, softcap, dtype,
                                      page_size, [(0, T)])
            finally:
                kernels.tcgen05_attention_variant = 0
            close(whole, ref, tol, f"attention whole cap {softcap} bias {bias} variant {variant}")
        cut_up = run_attention(kernels, q, k, r1 if bias else None, r2 if bias else None, scale, softcap, dtype,
                               page_size, [(0, 61), (61, 63), (63, 64), (64, 130)] + [(i, i + 1) for i in range(130, T)])
        close(cut_up, ref, tol, f"attention portions and single tokens cap {softcap} bias {bias}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_finds_a_far_key(kernels, dtype):
    """One key, hundreds of positions back and next to a page border, is made to stand
    out (its score reaches the cap, the bias by distance is small): the output must be
    that key, in a prompt and for a token decoded alone."""
    H = G = 2
    d, T, page_size, far = 80, 700, 16, 15
    g = torch.Generator().manual_seed(3)
    q = torch.randn(T, H, d, generator=g) * 0.05
    k = torch.randn(T, G, d, generator=g) * 0.05
    direction = torch.randn(d, generator=g)
    direction /= direction.norm()
    k[far] = 6 * direction
    q[T - 1] = 6 * direction
    q[T - 40] = 6 * direction
    r1, r2 = torch.full((H,), 0.05), torch.full((H,), 0.2)
    dt = DTYPES[dtype]
    q, k = q.to(dt), k.to(dt)
    ref = plain.capped_distance_scores(q.double(), k.double(), r1.double(), r2.double(), 1.0, 30.0)
    assert float((ref[T - 1, 0] - k[far, 0].double()).abs().max()) < 0.05 * 6      # the far key takes the weight
    got = run_attention(kernels, q, k, r1, r2, 1.0, 30.0, dtype, page_size, [(0, T - 1), (T - 1, T)])
    tol = 2e-5 if dtype == "float32" else 2e-2
    close(got[T - 1], ref[T - 1], tol, "far key, decoded token")
    close(got[T - 40], ref[T - 40], tol, "far key, inside a prompt")
    close(got, ref, tol, "far key, all rows")


# ------------------------------------------------------------------ whole models
CASES = {
    # name: (page size, request lengths, lengths of the mixed run)
    "G1": (4, [1, 33, 130, 260], [50, 100, 30, 128, 64, 90, 17]),
    "G2": (16, [2, 70, 131, 300], [1, 200, 33, 250, 64, 129, 7]),
    "G3": (8, [3, 64, 129, 190], [150, 20, 65, 2, 180, 99, 40]),
    "G4": (16, [5, 129, 260, 400], [400, 31, 129, 64, 350, 3, 222]),
    "G5": (16, [4, 66, 140, 300], [300, 20, 131, 64, 150, 2, 90]),
}
SEED = 21


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("gitipel")
    return {name: gitipel_models.write_model(gitipel_models.get(name), str(root / name), seed=SEED) for name in CASES}


@pytest.fixture(scope="module")
def expected():
    out = {}
    for name, (_, lengths, mixed_lengths) in CASES.items():
        cfg = gitipel_models.get(name)
        reqs = helpers.random_requests(cfg["vocab"], lengths, seed=100)
        mixed = helpers.random_requests(cfg["vocab"], mixed_lengths, seed=200)
        out[name] = (reqs, gitipel_models.plain_logits(cfg, SEED, reqs, torch.float32),
                     mixed, gitipel_models.plain_logits(cfg, SEED, mixed, torch.float32))
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
        helpers.assert_logits_close(got, ref, tol, f"gitipel {case} {dtype} {what}")
        runner.cache.check_invariants()
        assert not runner.cache.requests
    if dtype == "bfloat16":
        assert runner.runtime.kernels.tensor_core_calls > 0

    pool = 640 if sum(helpers.round64(len(v)) for v in mixed_reqs.values()) > 640 else 384
    trace = helpers.trace_mixed(mixed_reqs, pool, seed=6)
    assert sum(helpers.round64(len(v)) for v in mixed_reqs.values()) > pool       # pages and slots are used again
    runner2 = make_runner(folders[case], dtype, page_size, pool)
    got = helpers.run_trace(runner2, trace)
    helpers.assert_logits_close(got, mixed_ref, tol, f"gitipel {case} {dtype} mixed")
    runner2.cache.check_invariants()
    assert not runner2.cache.requests


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(folders, dtype):
    """Three tokens of prompt, then 300 tokens one by one (captured steps replayed):
    the state and the history are carried hundreds of times, pages fill up and follow."""
    cfg = gitipel_models.get("G1")
    reqs = helpers.random_requests(cfg["vocab"], [303], seed=9)
    ref = gitipel_models.plain_logits(cfg, SEED, reqs, torch.float32)
    runner = make_runner(folders["G1"], dtype, 4, 320)
    got = helpers.run_trace(runner, helpers.trace_last_decoded(reqs, 300))
    helpers.assert_logits_close(got, ref, helpers.TOL[dtype], f"gitipel G1 {dtype} long decoding")
    assert runner.graph_replays > 200


def test_greedy_generation_through_the_entry_point(folders):
    """``LLM.generate`` (scheduler, sampler, portions of 16 tokens, three requests at a
    time): every generated token is the plain implementation's best one, wherever that
    leads by more than the rounding of a 32-bit run."""
    from chibillm_b200 import LLM
    cfg = gitipel_models.get("G1")
    prompts = list(helpers.random_requests(cfg["vocab"], [5, 40, 23, 61], seed=12).values())
    llm = LLM(folders["G1"], dtype="float32", context_length=128, max_sequences=3, max_batch_tokens=48,
              prefill_chunk_tokens=16, page_size=16)
    outs = llm.generate(prompts, max_tokens=12, ignore_eos=True)
    for prompt, new in zip(prompts, outs):
        assert len(new) == 12
        ref = gitipel_models.plain_logits(cfg, SEED, {"a": prompt + new})["a"]
        for i, tok in enumerate(new):
            row = ref[len(prompt) + i - 1]
            top = torch.topk(row, 2).values
            if float(top[0] - top[1]) > 1e-4 * float(row.abs().max()):
                assert int(torch.argmax(row)) == tok, f"token {i} of a prompt of {len(prompt)}"


def test_trace_program(folders, tmp_path):
    """bin/trace_run on a Gitipel folder: portions, single tokens, two live requests."""
    cfg = gitipel_models.get("G3")
    reqs = helpers.random_requests(cfg["vocab"], [40, 21], seed=5)
    ref = gitipel_models.plain_logits(cfg, SEED, reqs, torch.float32)
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
        proc = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folders["G3"],
                               "--dtype", dtype, "--out", out_dir, "--max-tokens", "128"],
                              input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True,
                              timeout=600)
        assert proc.returncode == 0, proc.stderr[-2000:]
        assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
        for i, rows in enumerate(want):
            got = torch.from_numpy(np.fromfile(os.path.join(out_dir, f"{i}.f32"), dtype="<f4").reshape(len(rows), -1))
            scale = float(torch.stack(rows).abs().max())
            assert float((got - torch.stack(rows)).abs().max()) <= helpers.TOL[dtype] * scale


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_recurrent_layers_only(tmp_path, dtype):
    """A model without any attention layer: no page group, state slots only."""
    cfg = {"architecture": "Gitipel", "vocab": 97, "width": 64, "norm": {"eps": 1e-5}, "canon": {"taps": 2},
           "layers": [gitipel_models.delta(2, 32, 4, ff=64), gitipel_models.delta(1, 64, 8)],
           "loop": {"start": 1, "stop": 2, "times": 2}}
    folder = gitipel_models.write_model(cfg, str(tmp_path / "m"), seed=3)
    reqs = helpers.random_requests(97, [5, 70, 133], seed=1)
    ref = gitipel_models.plain_logits(cfg, 3, reqs, torch.float32)
    runner = make_runner(folder, dtype, 16, 192)
    assert runner.plan.groups == ()
    for trace, what in ((helpers.trace_whole(reqs), "whole"), (helpers.trace_last_decoded(reqs, 20), "decoded"),
                        (helpers.trace_mixed(reqs, 256, seed=1, decode_tail=6), "mixed")):
        got = helpers.run_trace(runner, trace)
        # bfloat16: twice the usual limit.  At a sequence's first positions the state holds one or two
        # outer products and the per-head norm divides o by its own small size, so the rounding of r, k
        # and v shows in full (32-bit: 1.4e-6 in every trace; bfloat16: 2.5e-2 whole, 3.4e-2 mixed).
        tol = helpers.TOL[dtype] * (2 if dtype == "bfloat16" else 1)
        helpers.assert_logits_close(got, ref, tol, f"gitipel recurrent only {dtype} {what}")
    assert not runner.cache.requests
