"""Gitipel without a GPU: the configuration reader, the cache plan of blocks with
several needs, and the engine's logic (batching, paging, state slots, layers that
run several times) on the plain PyTorch stand-ins of the kernels, against the
plain implementation of the design."""
import json
import os

import pytest
import torch

import gitipel_models
import helpers
import plain_gitipel
from reference_ops import ReferenceKernels


def cpu_runner(folder, page_size, pool_tokens, max_requests=4):
    from chibillm_b200.engine.runner import ModelRunner
    runner = ModelRunner.from_folder(folder, dtype="float32", device="cpu", page_size=page_size,
                                     pool_tokens=pool_tokens, max_requests=max_requests,
                                     kernels=ReferenceKernels())
    runner.storage.poison()
    return runner


# ------------------------------------------------------------------ configuration
def test_run_order_and_parts_follow_the_file(tmp_path):
    from chibillm_b200.config import load_config
    folder = gitipel_models.write_model(gitipel_models.get("G1"), str(tmp_path / "g1"), seed=1)
    arch, config, spec = load_config(folder)
    assert arch.name == "Gitipel" and spec.max_positions == 0
    # layer 0 once, layers 1 and 2 three times with the re-entry before layer 1, then layer 3
    assert [(s.layer, s.enter, s.turn) for s in spec.run_order] == [
        (0, None, 0), (1, 0, 0), (2, None, 0), (1, 0, 1), (2, None, 1), (1, 0, 2), (2, None, 2), (3, None, 0)]
    assert [l.mixer.kind for l in spec.layers] == ["attention", "delta_rule", "attention", "delta_rule"]
    assert spec.layers[1].mixer.decay_rank == 5 and spec.layers[3].mixer.decay_rank == 8      # from the tensors
    assert spec.layers[2].feed_forward is None and spec.layers[2].feed_forward_norm is None
    att = spec.layers[0].mixer
    assert (att.num_heads, att.num_kv_heads, att.head_dim, att.softcap, att.tied_values, att.distance_bias) == \
        (4, 2, 32, 8.0, True, "log")
    assert spec.layers[0].mixer_conv.taps == 3
    assert [a.kind for a in spec.input_adapters + spec.logit_adapters + spec.stream_adapters] == \
        ["scale", "scale", "reentry_mix"]

    _, _, plain = load_config(gitipel_models.write_model(gitipel_models.get("G2"), str(tmp_path / "g2"), seed=1))
    assert [(s.layer, s.enter) for s in plain.run_order] == [(0, None), (1, None), (2, None)]
    assert plain.stream_adapters == () and plain.layers[0].mixer_conv is None
    assert plain.layers[1].mixer.softcap is None


def test_config_errors_name_the_key():
    from chibillm_b200.config import ConfigError, GitipelConfig
    good = gitipel_models.file_config(gitipel_models.get("G1"))
    shapes = {"l1.mix.w1": (5, 64), "l3.mix.w1": (8, 64)}

    def read(change):
        obj = json.loads(json.dumps(good))
        change(obj)
        obj["_tensor_shapes"] = shapes
        return GitipelConfig.from_dict(obj)

    read(lambda o: None)
    with pytest.raises(ConfigError, match="vdim"):
        read(lambda o: o["layers"][0]["mixer"].update(vdim=16))
    with pytest.raises(ConfigError, match="kv_heads"):
        read(lambda o: o["layers"][0]["mixer"].update(kv_heads=3))
    with pytest.raises(ConfigError, match="loop"):
        read(lambda o: o["loop"].update(stop=9))
    with pytest.raises(ConfigError, match="type"):
        read(lambda o: o["layers"][1].update(type="other"))
    with pytest.raises(ConfigError, match="rank"):
        GitipelConfig.from_dict(good)                   # no tensor shapes and no key
    with pytest.raises(ConfigError, match="eps"):
        read(lambda o: o["norm"].pop("eps"))


def test_cache_plan_of_blocks_with_several_needs():
    from chibillm_b200.cache.storage import plan_cache
    from chibillm_b200.parts.base import FixedStateNeed, PagedKVNeed
    conv = FixedStateNeed((("history", (2, 8), None),))
    state = FixedStateNeed((("state", (2, 4, 4), torch.float32),))
    needs = [(PagedKVNeed(2, 16, None, tied_values=True), conv), (state, conv),
             (PagedKVNeed(2, 16, None, tied_values=True), conv), PagedKVNeed(2, 16, None)]
    plan = plan_cache(needs, [None] * 4, page_size=4, pool_tokens=64)
    assert [g.name for g in plan.groups] == ["k2x16", "kv2x16"] and plan.tied == ("k2x16",)
    assert plan.groups[0].num_entries == 2 and plan.groups[1].num_entries == 1
    assert plan.steps[0][0] == "several" and plan.steps[0][1][0][:3] == ("paged", "k2x16", 0)
    assert plan.steps[2][1][0][:3] == ("paged", "k2x16", 1)
    assert plan.steps[1][1][0][0] == "state" and plan.steps[3][0] == "paged"


# ------------------------------------------------------------------ the plain implementation
def test_plain_implementation_is_consistent():
    for name in ("G1", "G2", "G3"):
        cfg = gitipel_models.get(name)
        ids = helpers.random_requests(cfg["vocab"], [40], seed=7)["r0"]
        l64 = gitipel_models.plain_logits(cfg, 3, {"a": ids}, torch.float64)["a"]
        l32 = gitipel_models.plain_logits(cfg, 3, {"a": ids}, torch.float32)["a"]
        assert float((l32 - l64).abs().max()) < 5e-5 * float(l64.abs().max())
        prefix = gitipel_models.plain_logits(cfg, 3, {"a": ids[:17]}, torch.float64)["a"]
        assert float((prefix - l64[:17]).abs().max()) < 1e-5 * float(l64.abs().max())


def test_plain_mechanisms_on_small_cases():
    # short convolution: y_t = x_t + sum_j w_j x_(t - taps + 1 + j)
    x = torch.tensor([[1.0], [2.0], [4.0]])
    y = plain_gitipel.short_convolution(x, torch.tensor([[10.0, 100.0, 1000.0]]))
    assert y.flatten().tolist() == [1.0 + 1000.0, 2.0 + 100.0 + 2000.0, 4.0 + 10.0 + 200.0 + 4000.0]
    # delta rule, one head of size 1: S <- w S - a u u S + k v with u = k / |k|; o = S r
    w = {"p.r": torch.tensor([[1.0]]), "p.k": torch.tensor([[2.0]]), "p.v": torch.tensor([[3.0]]),
         "p.g": torch.tensor([[0.0]]), "p.a": torch.tensor([[0.0]]), "p.a.b": torch.tensor([0.0]),
         "p.w1": torch.tensor([[0.0]]), "p.w2": torch.tensor([[0.0]]), "p.w0": torch.tensor([0.0]),
         "p.norm": torch.tensor([1.0]), "p.o": torch.tensor([[1.0]])}
    out = plain_gitipel.delta_rule_mixer(torch.tensor([[1.0], [1.0]], dtype=torch.float64),
                                         {k: v.double() for k, v in w.items()}, "p.", 1, 1, 0.0)
    # o is divided by its own magnitude (one channel): +-1, times sigmoid(0) = 0.5
    assert torch.allclose(out.flatten(), torch.tensor([0.5, 0.5], dtype=torch.float64))
    # attention: with r1 = 0 and no cap in reach, a far key with a large score takes all the weight
    h = torch.zeros(6, 2, dtype=torch.float64)
    h[0] = torch.tensor([0.0, 9.0])
    h[5] = torch.tensor([0.0, 9.0])
    eye = torch.eye(2, dtype=torch.float64)
    o = plain_gitipel.capped_distance_attention(h, eye, eye, eye, torch.zeros(1), torch.ones(1), 1, 1, 2, 1.0, 1e6)
    assert torch.allclose(o[5], torch.tensor([0.0, 9.0], dtype=torch.float64), atol=1e-6)
    # ... and a strong bias by distance gives it back to the query's own key
    h[5] = torch.tensor([1.0, 9.0])
    o = plain_gitipel.capped_distance_attention(h, eye, eye, eye, torch.full((1,), 50.0), torch.ones(1), 1, 1, 2,
                                                1.0, 1e6)
    assert torch.allclose(o[5], h[5], atol=1e-6)


# ------------------------------------------------------------------ the engine on the stand-ins
@pytest.mark.parametrize("name,page_size,lengths", [("G1", 4, [1, 9, 30]), ("G2", 8, [2, 21, 37]),
                                                    ("G3", 16, [3, 18, 33]), ("G5", 8, [2, 11, 34])])
def test_cutting_and_batching_on_cpu(tmp_path, name, page_size, lengths):
    cfg = gitipel_models.get(name)
    folder = gitipel_models.write_model(cfg, str(tmp_path / name), seed=11)
    reqs = helpers.random_requests(cfg["vocab"], lengths, seed=1)
    ref = gitipel_models.plain_logits(cfg, 11, reqs)
    runner = cpu_runner(folder, page_size, helpers.round64(max(lengths)))
    for trace, what in ((helpers.trace_whole(reqs), "whole"),
                        (helpers.trace_last_decoded(reqs, 8), "last 8 decoded"),
                        (helpers.trace_portions(reqs, seed=2), "portions")):
        got = helpers.run_trace(runner, trace)
        helpers.assert_logits_close(got, ref, helpers.TOL["float32"], f"gitipel {name} cpu {what}")
        runner.cache.check_invariants()
        assert not runner.cache.requests

    mixed_reqs = helpers.random_requests(cfg["vocab"], [20, 33, 7, 28, 12, 30], seed=4)
    mixed_ref = gitipel_models.plain_logits(cfg, 11, mixed_reqs)
    pool = 128
    trace = helpers.trace_mixed(mixed_reqs, pool, seed=6, decode_tail=5)
    assert sum(helpers.round64(len(v)) for v in mixed_reqs.values()) > pool       # pages and slots are reused
    runner2 = cpu_runner(folder, page_size, pool)
    got = helpers.run_trace(runner2, trace)
    helpers.assert_logits_close(got, mixed_ref, helpers.TOL["float32"], f"gitipel {name} cpu mixed")
    runner2.cache.check_invariants()
    assert not runner2.cache.requests


def test_a_step_taken_back_leaves_the_state_as_it_was(tmp_path):
    """A provisional step that is rolled back restores the recurrent state and the
    convolution's history, so the same entries give the same logits again."""
    from chibillm_b200.engine.batch import StepEntry
    cfg = gitipel_models.get("G1")
    folder = gitipel_models.write_model(cfg, str(tmp_path / "g"), seed=5)
    ids = helpers.random_requests(cfg["vocab"], [14], seed=3)["r0"]
    runner = cpu_runner(folder, 4, 64)
    runner.step([StepEntry("a", ids[:9], [])])
    first = runner.step([StepEntry("a", ids[9:12], [0, 1, 2])], provisional=True).clone()
    runner.rollback_step()
    again = runner.step([StepEntry("a", ids[9:12], [0, 1, 2])], provisional=True).clone()
    runner.settle_step()
    assert torch.equal(first, again)
    ref = gitipel_models.plain_logits(cfg, 5, {"a": ids[:12]})["a"]
    assert float((again - ref[9:12]).abs().max()) < helpers.TOL["float32"] * float(ref.abs().max())


def test_random_model_folder_of_the_package(tmp_path):
    """``write_random_model`` takes a Gitipel configuration (with the rank as the
    mixer's optional key), and the folder runs."""
    from chibillm_b200.weights import write_random_model
    from chibillm_b200.engine.batch import StepEntry
    cfg = gitipel_models.file_config(gitipel_models.get("G1"))
    cfg["layers"][1]["mixer"]["rank"] = 6
    cfg["layers"][3]["mixer"]["rank"] = 4
    folder = write_random_model(cfg, str(tmp_path / "random"), seed=2)
    runner = cpu_runner(folder, 4, 64)
    logits = runner.step([StepEntry("a", [1, 2, 3, 4, 5], [4])])
    assert logits.shape == (1, cfg["vocab"]) and torch.isfinite(logits).all()
    from safetensors import safe_open
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        assert (f.get_tensor("l0.mix.r2") > 0).all()          # the logarithm's argument stays positive
        assert tuple(f.get_tensor("l1.mix.w1").shape) == (6, cfg["width"])


def test_command_line_and_scheduler_on_cpu(tmp_path):
    """Four prompts through the package's command line with room for three at a
    time and portions of 8 tokens: the scheduler mixes portions with decoded
    tokens, a request waits for a slot, and every greedy token is the plain
    implementation's best one (wherever that leads by more than rounding)."""
    import io
    from chibillm_b200 import cli
    cfg = gitipel_models.get("G1")
    folder = gitipel_models.write_model(cfg, str(tmp_path / "g1"), seed=4)
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
    assert err.getvalue().count("[stop] len_limit") == 4
    for prompt, new in zip(prompts, replies):
        ref = gitipel_models.plain_logits(cfg, 4, {"a": prompt + new})["a"]
        for i, tok in enumerate(new):
            row = ref[len(prompt) + i - 1]
            top = torch.topk(row, 2).values
            if float(top[0] - top[1]) > 1e-4 * float(row.abs().max()):
                assert int(torch.argmax(row)) == tok


def test_a_model_of_recurrent_layers_only_runs_without_a_paged_cache(tmp_path):
    """No attention layer at all: the cache plan has no page group, requests hold
    state slots only; a looped layer has a state of its own per pass."""
    cfg = {"architecture": "Gitipel", "vocab": 97, "width": 48, "norm": {"eps": 1e-5}, "canon": {"taps": 2},
           "layers": [gitipel_models.delta(2, 16, 4, ff=64), gitipel_models.delta(1, 32, 3)],
           "loop": {"start": 1, "stop": 2, "times": 2}}
    folder = gitipel_models.write_model(cfg, str(tmp_path / "m"), seed=3)
    reqs = helpers.random_requests(97, [5, 19, 33], seed=1)
    ref = gitipel_models.plain_logits(cfg, 3, reqs)
    runner = cpu_runner(folder, 16, 64)
    assert runner.plan.groups == () and len(runner.storage.state_views()) == 6      # 3 layer runs x (state, history)
    for trace, what in ((helpers.trace_whole(reqs), "whole"), (helpers.trace_portions(reqs, seed=2), "portions"),
                        (helpers.trace_mixed(reqs, 128, seed=1, decode_tail=4), "mixed")):
        got = helpers.run_trace(runner, trace)
        helpers.assert_logits_close(got, ref, helpers.TOL["float32"], f"gitipel recurrent only {what}")
    assert not runner.cache.requests
