"""Fokurax without a GPU: the configuration reader, the plain implementation's own
consistency on cases checked by hand, and the engine's logic (batching, paging,
shared caches, routed experts, the token input) on the plain PyTorch stand-ins of
the kernels, against the plain implementation of the design."""
import io
import json
import math
import os

import pytest
import torch

import fokurax_models
import helpers
import plain_fokurax as plain
from reference_ops import ReferenceKernels


def cpu_runner(folder, page_size, pool_tokens, max_requests=4):
    from chibillm_b200.engine.runner import ModelRunner
    runner = ModelRunner.from_folder(folder, dtype="float32", device="cpu", page_size=page_size,
                                     pool_tokens=pool_tokens, max_requests=max_requests,
                                     kernels=ReferenceKernels())
    runner.storage.poison()
    return runner


# ------------------------------------------------------------------ configuration
def test_parts_follow_the_file(tmp_path):
    from chibillm_b200.config import load_config
    folder = fokurax_models.write_model(fokurax_models.get("F1"), str(tmp_path / "f1"), seed=1)
    arch, config, spec = load_config(folder)
    assert arch.name == "Fokurax" and spec.max_positions == 0
    assert [(s.layer, s.cache_of) for s in spec.run_order] == [(0, None), (1, None), (2, 0)]
    assert [l.arrangement for l in spec.layers] == ["parallel"] * 3
    att = spec.layers[2].mixer
    assert (att.num_heads, att.num_kv_heads, att.head_dim, att.value_dim, att.chunk, att.own_kv, att.unit_norm_eps) == \
        (4, 2, 32, 16, 24, False, 1e-6)
    assert (att.position.rotary_dim, att.position.theta, att.position.scaling_factor, att.position.original_positions) \
        == (16, 5000.0, 4.0, 32)
    assert spec.layers[0].mixer.own_kv and spec.layers[0].residual_scale == 0.7
    assert [l.feed_forward.kind for l in spec.layers] == ["gated_mlp", "table_experts", "table_experts"]
    assert spec.layers[0].feed_forward.biases and spec.layers[0].feed_forward.activation == "gelu_tanh"
    assert (spec.layers[2].feed_forward.num_experts, spec.layers[2].feed_forward.top) == (3, 3)
    assert [l.token_input.offset for l in spec.layers] == [0, 13, 26] and spec.shared_tensors[0][1] == (211, 39)
    assert spec.final_norm.weight_offset == 1.0
    assert [a.kind for a in spec.input_adapters + spec.logit_adapters] == ["scale", "softcap"]

    _, _, bare = load_config(fokurax_models.write_model(fokurax_models.get("F2"), str(tmp_path / "f2"), seed=1))
    assert bare.logit_adapters == () and bare.shared_tensors == () and bare.layers[0].token_input is None
    assert bare.layers[1].feed_forward is None and bare.layers[0].residual_scale == 1.0
    assert bare.layers[0].mixer.chunk is None and bare.layers[0].mixer.position.scaling_factor == 0.0
    assert bare.layers[2].mixer.position.kind == "none" and bare.layers[0].mixer.value_dim == 64


def test_config_errors_name_the_key():
    from chibillm_b200.config import ConfigError, FokuraxConfig
    good = fokurax_models.get("F1")

    def read(change):
        obj = json.loads(json.dumps(good))
        change(obj)
        return FokuraxConfig.from_dict(obj)

    read(lambda o: None)
    for change, word in [
            (lambda o: o.pop("vocab"), "vocab"),
            (lambda o: o["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
            (lambda o: o["layers"][0]["mixer"]["rot"].update(dims=15), "rot.dims"),
            (lambda o: o["layers"][0]["mixer"]["rot"].update(dims=34), "rot.dims"),
            (lambda o: o["layers"][2]["mixer"].update(kv_from=2), "kv_from"),
            (lambda o: o["layers"][2]["mixer"].update(kv_from=1, vdim=8), "vdim"),
            (lambda o: o["layers"][1]["mixer"].update(kv_from=0) or o["layers"][2]["mixer"].update(kv_from=1), "kv_from"),
            (lambda o: o["layers"][1]["mlp"]["router"].update(top=6), "top"),
            (lambda o: o["layers"][1]["mlp"].update(kind="sparse"), "kind"),
            (lambda o: o["layers"][0].update(type="recurrent"), "type"),
            (lambda o: o["layers"][0]["mixer"]["mask"].update(size=0), "size"),
            (lambda o: o.update(logit_softcap=-1.0), "logit_softcap")]:
        with pytest.raises(ConfigError) as e:
            read(change)
        assert word in str(e.value), str(e.value)


def test_a_reader_must_name_a_layer_with_the_same_cache(tmp_path):
    """The cache plan refuses a reader whose key or value size differs from its source's."""
    from chibillm_b200.cache.manager import CacheError
    from chibillm_b200.cache.storage import plan_cache
    from chibillm_b200.parts.base import PagedKVNeed
    a = PagedKVNeed(2, 32, None, False, 16)
    plan = plan_cache([a, a, PagedKVNeed(2, 32)], [None, 0, None], 8, 64)
    assert [s[1:] for s in plan.steps] == [("kv2x32v16", 0, True), ("kv2x32v16", 0, False), ("kv2x32", 0, True)]
    assert dict(plan.value_dims) == {"kv2x32v16": 16}
    with pytest.raises(CacheError):
        plan_cache([a, PagedKVNeed(2, 32, None, False, 8)], [None, 0], 8, 64)


# ------------------------------------------------------------------ the plain implementation itself
def test_plain_rotation_by_hand():
    r = {"base": 100.0, "dims": 4}
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 5.0]]], dtype=torch.float64).repeat(3, 1, 1)
    y = plain.rotate(x, torch.tensor([0, 1, 2]), r)
    assert torch.equal(y[0], x[0])                                       # position 0: nothing turns
    f = [1.0, 100.0 ** -0.5]
    for p in (1, 2):
        for i in range(2):
            a = p * f[i]
            assert abs(float(y[p, 0, i]) - (x[p, 0, i] * math.cos(a) - x[p, 0, i + 2] * math.sin(a))) < 1e-12
            assert abs(float(y[p, 0, i + 2]) - (x[p, 0, i + 2] * math.cos(a) + x[p, 0, i] * math.sin(a))) < 1e-12
        assert float(y[p, 0, 4]) == 5.0                                  # beyond dims: unchanged
    # stretched: fast pairs keep their frequency, slow ones are divided by the factor, amplitude 0.1 ln f + 1
    r = {"base": 10000.0, "dims": 32, "scaling": {"factor": 8.0, "original": 64, "fast": 8.0, "slow": 1.0}}
    f, amp = plain.rotary_frequencies(r)
    plain_f = 10000.0 ** (-2.0 * torch.arange(16, dtype=torch.float64) / 32)
    assert abs(amp - (0.1 * math.log(8.0) + 1.0)) < 1e-15
    assert float(f[0]) == float(plain_f[0]) and abs(float(f[15]) - float(plain_f[15]) / 8.0) < 1e-18
    assert all(float(plain_f[i]) / 8.0 - 1e-18 <= float(f[i]) <= float(plain_f[i]) for i in range(16))
    assert any(float(plain_f[i]) / 8.0 + 1e-12 < float(f[i]) < float(plain_f[i]) - 1e-12 for i in range(16))


def test_plain_blocks_of_positions():
    ok = plain.visible(7, {"size": 3})
    assert ok.int().tolist() == [[1, 0, 0, 0, 0, 0, 0], [1, 1, 0, 0, 0, 0, 0], [1, 1, 1, 0, 0, 0, 0],
                                 [0, 0, 0, 1, 0, 0, 0], [0, 0, 0, 1, 1, 0, 0], [0, 0, 0, 1, 1, 1, 0],
                                 [0, 0, 0, 0, 0, 0, 1]]
    assert plain.visible(4, None).int().tolist() == [[1, 0, 0, 0], [1, 1, 0, 0], [1, 1, 1, 0], [1, 1, 1, 1]]


def test_plain_logits_depend_on_the_own_block_only():
    """With every layer in blocks of the same size, a position's logits depend on the tokens
    of its own block up to itself and on nothing before it, and they do depend on the
    block's first token."""
    cfg = fokurax_models.get("F1")
    w = fokurax_models.random_weights(cfg, 3)
    ids = helpers.random_requests(cfg["vocab"], [60], seed=1)["r0"]
    base = plain.forward(cfg, w, ids)
    other = list(ids)
    other[23] = (other[23] + 1) % cfg["vocab"]                            # the last token of block 0
    changed = plain.forward(cfg, w, other)
    assert float((changed[24:] - base[24:]).abs().max()) < 1e-12
    assert float((changed[23] - base[23]).abs().max()) > 1e-3
    other = list(ids)
    other[24] = (other[24] + 1) % cfg["vocab"]                            # the first token of block 1
    changed = plain.forward(cfg, w, other)
    assert float((changed[47] - base[47]).abs().max()) > 1e-4
    assert float((changed[48:] - base[48:]).abs().max()) < 1e-12
    assert float((changed[:24] - base[:24]).abs().max()) == 0.0


def test_plain_experts_by_hand():
    h = torch.tensor([[1.0, -2.0], [0.5, 3.0]], dtype=torch.float64)
    w = {"m.table": torch.tensor([[1, 0], [0, 1], [1, 0]], dtype=torch.int32)}
    for e in range(2):
        w[f"m.e{e}.gate"] = torch.tensor([[1.0 + e, 0.0]], dtype=torch.float64)
        w[f"m.e{e}.up"] = torch.tensor([[0.0, 1.0]], dtype=torch.float64)
        w[f"m.e{e}.down"] = torch.tensor([[1.0], [float(e)]], dtype=torch.float64)
    out = plain.routed_feed_forward(h, torch.tensor([2, 1]), {"router": {"top": 2}}, w, "m.")
    def expert(e, x):
        g = (1.0 + e) * x[0]
        a = g / (1.0 + math.exp(-g)) * x[1]
        return [a, a * e]
    for t, x in enumerate(h.tolist()):
        want = [(expert(0, x)[c] + expert(1, x)[c]) / 2 for c in range(2)]
        assert all(abs(float(out[t, c]) - want[c]) < 1e-12 for c in range(2))


# ------------------------------------------------------------------ the engine on the stand-in kernels
@pytest.mark.parametrize("name,page_size,lengths", [("F1", 4, [1, 30, 75]), ("F2", 16, [2, 40, 70]),
                                                    ("F4", 8, [3, 23, 66]), ("F5", 16, [5, 70])])
def test_cutting_and_batching_on_cpu(tmp_path, name, page_size, lengths):
    cfg = fokurax_models.get(name)
    folder = fokurax_models.write_model(cfg, str(tmp_path / name), seed=11)
    reqs = helpers.random_requests(cfg["vocab"], lengths, seed=4)
    ref = fokurax_models.plain_logits(cfg, 11, reqs)
    runner = cpu_runner(folder, page_size, helpers.round64(max(lengths)))
    for trace, what in ((helpers.trace_whole(reqs), "whole"), (helpers.trace_last_decoded(reqs, 12), "decoded"),
                        (helpers.trace_portions(reqs, seed=2), "portions")):
        got = helpers.run_trace(runner, trace)
        helpers.assert_logits_close(got, ref, helpers.TOL["float32"], f"fokurax {name} cpu {what}")
        runner.cache.check_invariants()
        assert not runner.cache.requests
    mixed_reqs = helpers.random_requests(cfg["vocab"], [20, 64, 9, 50, 33, 2], seed=8)
    mixed_ref = fokurax_models.plain_logits(cfg, 11, mixed_reqs)
    pool = 192
    trace = helpers.trace_mixed(mixed_reqs, pool, seed=6, decode_tail=5)
    assert sum(helpers.round64(len(v)) for v in mixed_reqs.values()) > pool       # pages and slots are reused
    runner2 = cpu_runner(folder, page_size, pool)
    got = helpers.run_trace(runner2, trace)
    helpers.assert_logits_close(got, mixed_ref, helpers.TOL["float32"], f"fokurax {name} cpu mixed")
    runner2.cache.check_invariants()
    assert not runner2.cache.requests


def test_a_reader_layer_holds_no_pages_of_its_own(tmp_path):
    cfg = fokurax_models.get("F3")
    folder = fokurax_models.write_model(cfg, str(tmp_path / "f3"), seed=2)
    runner = cpu_runner(folder, 16, 128)
    # four layers, two caches: layers 1 and 3 read those of 0 and 2
    assert sorted(g.name for g in runner.plan.groups) == ["kv1x128", "kv2x64"]
    assert [g.num_entries for g in runner.plan.groups] == [1, 1]
    assert [v.writes for v in runner.storage.views] == [True, False, True, False]
    assert runner.storage.views[1].keys.data_ptr() == runner.storage.views[0].keys.data_ptr()


def test_random_model_folder_of_the_package(tmp_path):
    """``write_random_model`` takes a Fokurax configuration: the expert tables it makes
    name different experts in a row, and the folder runs and agrees with the plain
    implementation on the stored weights."""
    from chibillm_b200.weights import write_random_model
    from safetensors import safe_open
    cfg = fokurax_models.get("F1")
    folder = write_random_model(cfg, str(tmp_path / "random"), seed=2)
    weights = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            weights[name] = f.get_tensor(name)
    table = weights["l2.mlp.table"]
    assert table.dtype == torch.int32 and tuple(table.shape) == (211, 3)
    assert all(sorted(row) == [0, 1, 2] for row in table.tolist())
    two = weights["l1.mlp.table"]
    assert all(a != b and 0 <= a < 5 and 0 <= b < 5 for a, b in two.tolist()) and len(set(map(tuple, two.tolist()))) > 5
    reqs = helpers.random_requests(cfg["vocab"], [30], seed=1)
    ref = fokurax_models.plain_logits(cfg, 0, reqs, weights=weights)
    got = helpers.run_trace(cpu_runner(folder, 4, 64), helpers.trace_portions(reqs, seed=1))
    helpers.assert_logits_close(got, ref, helpers.TOL["float32"], "fokurax random folder")


def test_command_line_and_scheduler_on_cpu(tmp_path):
    """Four prompts through the package's command line with room for three at a time and
    portions of 8 tokens: every greedy token is the plain implementation's best one
    (wherever that leads by more than rounding)."""
    from chibillm_b200 import cli
    cfg = fokurax_models.get("F1")
    folder = fokurax_models.write_model(cfg, str(tmp_path / "f1"), seed=4)
    prompts = list(helpers.random_requests(cfg["vocab"], [1, 7, 23, 30], seed=1).values())
    argv = ["--context-length", "64", "--max-tokens", "5", "--max-seqs", "3", "--max-batch-tokens", "16",
            "--prefill-chunk", "8", "--dtype", "float32", "--ignore-eos", "--no-stream"]
    for p in prompts:
        argv += ["--prompt-ids", ",".join(map(str, p))]
    out, err = io.StringIO(), io.StringIO()
    assert cli.run(cli.parse_cli_options(argv + [folder]), io.StringIO(""), out, err,
                   kernels=ReferenceKernels(), device="cpu") == 0, err.getvalue()
    replies = [[int(t) for t in line.split()] for line in out.getvalue().splitlines()]
    assert len(replies) == 4 and all(len(r) == 5 for r in replies)
    for prompt, new in zip(prompts, replies):
        ref = fokurax_models.plain_logits(cfg, 4, {"a": prompt + new})["a"]
        for i, tok in enumerate(new):
            row = ref[len(prompt) + i - 1]
            top = torch.topk(row, 2).values
            if float(top[0] - top[1]) > 1e-4 * float(row.abs().max()):
                assert int(torch.argmax(row)) == tok


def test_experts_sorted_on_the_host_agree_with_the_device_plan(tmp_path, monkeypatch):
    """Prompt steps of many (token, choice) pairs are sorted by expert on the host and go
    expert by expert through the ordinary products: same logits as the plan made on the
    device, in whole prompts and in portions (a portion of one token takes the other way)."""
    from chibillm_b200.parts.mlp import TableExperts
    cfg = fokurax_models.get("F1")
    folder = fokurax_models.write_model(cfg, str(tmp_path / "f1"), seed=7)
    reqs = helpers.random_requests(cfg["vocab"], [40, 9], seed=3)
    ref = fokurax_models.plain_logits(cfg, 7, reqs)
    monkeypatch.setattr(TableExperts, "MANY_PAIRS", 4)
    monkeypatch.setattr(TableExperts, "MUCH_WORK", 0)
    runner = cpu_runner(folder, 4, 64)
    for trace, what in ((helpers.trace_whole(reqs), "whole"), (helpers.trace_portions(reqs, seed=1), "portions"),
                        (helpers.trace_last_decoded(reqs, 5), "decoded")):
        got = helpers.run_trace(runner, trace)
        helpers.assert_logits_close(got, ref, helpers.TOL["float32"], f"fokurax experts sorted on the host, {what}")
    calls = runner.runtime.kernels.calls
    assert calls.get("combine_experts", 0) > 0 and calls.get("routed_experts", 0) > 0
