"""Zozezen without a GPU: its configuration, what it declares, the plain implementation's own consistency, and the host-side
logic (parts, block, caches, state slots, step function) on the CPU with plain PyTorch functions standing in for the kernels,
in every cutting, against the plain implementation."""

from __future__ import annotations

import copy

import pytest
import torch

import helpers
import plain_ops
import plain_zozezen as plain
import zozezen_helpers as zh


def test_configuration_reads_every_size_and_round_trips():
    import miniserve_b200  # noqa: F401
    from miniserve_b200.config import ZozezenConfig, resolve_architecture
    from miniserve_b200.parts import DecoderModel, PagedKVNeed, StateNeed

    for name, raw in zh.CONFIGS.items():
        architecture = resolve_architecture(raw)
        config = architecture.config_class.from_dict(raw)
        assert isinstance(config, ZozezenConfig) and config.to_dict() == raw
        spec = architecture.build_spec(config)
        assert spec.output_name == "head" and spec.vocab_size == raw["vocab"] and spec.embedding_scale == 1.0
        assert all(layer.block.kind == "sandwich" and layer.mixer_post_norm is not None for layer in spec.layers)
        model = DecoderModel(spec, torch.float32, "cpu")
        for index, (entry, run, plan) in enumerate(zip(raw["layers"], spec.order, model.run_caches)):
            mixer = model.blocks[index].mixer
            if entry["type"] == "mamba2":
                m = entry["mixer"]
                channels = m["heads"] * m["vdim"] + 2 * m["groups"] * m["state"]
                assert mixer.cache_need() == StateNeed(((m["conv"] - 1) * channels + m["heads"] * m["vdim"] * m["state"],), torch.float32)
                assert plan.writable
            else:
                m = entry["mixer"]
                assert mixer.cache_need() == PagedKVNeed(m["kv_heads"], m["dim"], None, None if m["vdim"] == m["dim"] else m["vdim"])
                assert run.cache_of == m.get("kv_from") and plan.writable == ("kv_from" not in m)
                if "kv_from" in m:
                    lender = model.run_caches[m["kv_from"]]
                    assert (plan.group, plan.slot) == (lender.group, lender.slot)
        names = {s.name: s for s in model.param_specs()}
        for index, entry in enumerate(raw["layers"]):
            borrowed = "kv_from" in entry["mixer"]
            assert (f"l{index}.mix.k" in names) == (entry["type"] == "attention" and not borrowed)
            assert (f"l{index}.mix.k.norm" in names) == (entry["type"] == "attention" and not borrowed)
            assert (f"l{index}.norm2" in names) == (entry["mlp"] is not None) == (f"l{index}.norm2b" in names)
            if entry["mlp"]:
                router = entry["mlp"]["router"]
                assert names[f"l{index}.mlp.router"].shape == (router["experts"] + router["identity"], raw["width"])
                assert f"l{index}.mlp.e{router['experts'] - 1}.gate" in names and f"l{index}.mlp.e{router['experts']}.gate" not in names
                assert (f"l{index}.mlp.shared.sg" in names) == (entry["mlp"]["shared"] is not None)


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].__setitem__("type", "hyena"), "not implemented"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_from", 2), "earlier attention layer"),
    (lambda c: c["layers"][3]["mixer"].__setitem__("kv_from", 1), "keys and values of its own"),
    (lambda c: c["layers"][3]["mixer"].__setitem__("vdim", 16), "differ from this layer's"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("heads", 7), "multiple of kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 26), "exceeds the head size"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("groups", 4), "multiple of groups"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("norm_groups", 5), "does not divide"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].__setitem__("count", 2), "router outputs"),
    (lambda c: c["layers"][2]["mlp"]["router"].__setitem__("top", 5), "exceeds"),
    (lambda c: c["layers"][0]["mlp"]["expert"].__delitem__("limit"), "limit"),
    (lambda c: c["norm"].__setitem__("eps", 0.0), "positive"),
])
def test_configuration_refuses_what_it_cannot_run(change, message):
    import miniserve_b200  # noqa: F401
    from miniserve_b200.config import resolve_architecture

    raw = copy.deepcopy(zh.ZOZEZEN_A)
    change(raw)
    with pytest.raises(ValueError, match=message):
        resolve_architecture(raw).config_class.from_dict(raw)


def test_plain_recurrence_is_the_same_in_one_pass_and_in_two():
    """The oracle against itself: a sequence's state-space output does not change when the sequence is walked as one, and
    an attention row sees exactly the keys up to its own position (a key behind it changes nothing)."""
    torch.manual_seed(0)
    m = dict(heads=4, vdim=6, state=5, groups=2, conv=3, norm_groups=2)
    inner, width = 24, 16
    w = {"x.mix.in": torch.randn(2 * inner + 20 + 4, width, dtype=plain.F64) * 0.3, "x.mix.conv": torch.randn(inner + 20, 3, dtype=plain.F64) * 0.5,
         "x.mix.conv.b": torch.randn(inner + 20, dtype=plain.F64) * 0.1, "x.mix.dt_bias": torch.randn(4, dtype=plain.F64),
         "x.mix.A_log": torch.randn(4, dtype=plain.F64) - 1, "x.mix.D": torch.randn(4, dtype=plain.F64),
         "x.mix.norm": torch.ones(inner, dtype=plain.F64), "x.mix.o": torch.randn(width, inner, dtype=plain.F64) * 0.3}
    h = torch.randn(30, width, dtype=plain.F64)
    whole = plain.state_space(h, w, "x.", m, 1e-5)
    assert torch.allclose(plain.state_space(h[:17], w, "x.", m, 1e-5), whole[:17], atol=1e-12)
    changed = h.clone()
    changed[20] += 1.0
    assert torch.allclose(plain.state_space(changed, w, "x.", m, 1e-5)[:20], whole[:20], atol=1e-12)
    assert not torch.allclose(plain.state_space(changed, w, "x.", m, 1e-5)[25], whole[25], atol=1e-6)       # the state remembers


def test_plain_router_groups_identities_and_negative_choice_scores():
    w = {"f.mlp.router": torch.eye(6, dtype=plain.F64) * 4, "f.mlp.correction": torch.tensor([-1.0, -1.01, -1.02, -1.2, -1.21, -1.22], dtype=plain.F64)}
    mlp = dict(router=dict(experts=4, identity=2, top=2, groups=dict(count=2, keep=1)))
    h = torch.zeros(2, 6, dtype=plain.F64)
    h[0, 4] = 1.0        # output 4 stands out: its group (3, 4, 5) is kept although all choice scores are negative
    h[1, 0] = 1.0
    ids, weights, gap = plain.route(h, w, "f.", mlp)
    assert sorted(ids[0].tolist()) == [3, 4] and sorted(ids[1].tolist()) == [0, 1] and gap > 0
    scores = torch.softmax(h @ w["f.mlp.router"].T, dim=-1)
    assert torch.allclose(weights[0], scores[0, ids[0]]) and float(weights[0].sum()) < 1.0      # the scores as they are


@pytest.fixture
def cpu_runtime(monkeypatch, tmp_path):
    import miniserve_b200  # noqa: F401
    from miniserve_b200.config import EngineConfig
    from miniserve_b200.engine import runtime as runtime_module

    plain_ops.install(monkeypatch)
    monkeypatch.setattr(runtime_module, "require_device", lambda device: torch.device("cpu"))
    monkeypatch.setattr(runtime_module.kernels, "library", lambda: None)
    monkeypatch.setattr(torch.cuda, "set_device", lambda device: None)

    def build(name, num_pages, page_size, max_seqs=4):
        folder = zh.make_folder(tmp_path, name, seed=2)
        runtime = runtime_module.build_runtime(folder, EngineConfig(
            dtype="float32", kv_block_size=page_size, num_kv_blocks=num_pages, max_num_seqs=max_seqs,
            enable_prefix_cache=True, device="cpu", decode_execution="eager"))
        return folder, runtime
    return build


@pytest.mark.parametrize("name,page_size", [("a", 8), ("b", 4)])
@pytest.mark.parametrize("cutting", ["whole", "tail", "portions", "mixed"])
def test_cuttings_match_plain_on_cpu(cpu_runtime, name, page_size, cutting):
    from miniserve_b200.trace import TraceSession

    vocab = zh.CONFIGS[name]["vocab"]
    requests = {f"r{i}": helpers.random_tokens(vocab, n, seed=20 + i) for i, n in enumerate((1, 6, 17, 30, 41))}
    steps = {"whole": helpers.cut_whole, "tail": lambda r: helpers.cut_decode_tail(r, 9),
             "portions": helpers.cut_portions, "mixed": helpers.cut_mixed}[cutting](requests)
    pages = (helpers.max_live_tokens(steps, granule=page_size * 2) + page_size - 1) // page_size
    folder, runtime = cpu_runtime(name, pages, page_size)
    assert runtime.max_model_len == pages * page_size            # no position limit of the design's own: the pool's size
    assert runtime.manager.prefix is None                        # a model with per-request state shares no pages
    session, outputs = TraceSession(runtime), {}
    for record in steps:
        outputs[record["step"]] = session.run(record).double()
        runtime.manager.check_invariants()
    got = helpers.collect(steps, outputs)
    config, weights = plain.load_folder(folder)
    for index, entry in enumerate(config["layers"]):
        if entry["mlp"]:
            h = plain.norm_one_plus(weights["embed"], weights[f"l{index}.norm2"], config["norm"]["eps"])
            assert plain.route(h, weights, f"l{index}.", entry["mlp"])[2] > 0.0015      # (the marks decide, then the correction's steps)
    for rid, tokens in requests.items():
        expected = plain.forward(tokens, weights, config)
        assert sorted(got[rid]) == list(range(len(tokens)))
        for position, row in got[rid].items():
            assert torch.allclose(row, expected[position], atol=2e-4, rtol=2e-4), (rid, position)
    assert not runtime.manager.requests
    assert all(a.free_count == a.num_pages for a in runtime.manager.allocators)


def test_odd_heads_no_rotation_and_norms_that_nothing_reads(cpu_runtime, monkeypatch, tmp_path):
    """An odd head size without any rotation, and a checkpoint that carries feed-forward norms for a layer that has no
    feed-forward: the loader lets them be, and the engine computes what the plain implementation computes."""
    import json

    from safetensors.torch import save_file

    from miniserve_b200.config import EngineConfig
    from miniserve_b200.engine import runtime as runtime_module
    from miniserve_b200.trace import TraceSession
    from miniserve_b200.weights import random_tensors

    config = dict(architecture="Zozezen", vocab=61, width=40, norm=dict(eps=1e-5), layers=[
        zh.layer(zh.attn(3, 1, 7, 5, 0.3, 0), None),
        zh.layer(zh.ssm(2, 9, 5, 2, 3, 3), zh.moe(2, 2, 2, 6, 0.9, 2, 2, 10, 1.1)),
        zh.layer(zh.attn(2, 1, 7, 5, 0.6, 0, kv_from=0), zh.moe(3, 0, 2, 6, 0.9, 1, 1, None)),
    ])
    tensors = random_tensors(config, 5, "float32", 0.1)
    zh.steer_routers(tensors, config)
    tensors["l0.norm2"], tensors["l0.norm2b"] = torch.zeros(40), torch.zeros(40)
    folder = tmp_path / "odd"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(config))
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"))
    runtime = runtime_module.build_runtime(folder, EngineConfig(dtype="float32", kv_block_size=4, num_kv_blocks=16, max_num_seqs=2,
                                                               enable_prefix_cache=False, device="cpu", decode_execution="eager"))
    tokens = helpers.random_tokens(61, 19, seed=3)
    steps = helpers.cut_portions({"r": tokens})
    session, outputs = TraceSession(runtime), {}
    for record in steps:
        outputs[record["step"]] = session.run(record).double()
    got = helpers.collect(steps, outputs)["r"]
    loaded_config, weights = plain.load_folder(folder)
    expected = plain.forward(tokens, weights, loaded_config)
    for position, row in got.items():
        assert torch.allclose(row, expected[position], atol=2e-4, rtol=2e-4), position
