"""Vesidra without a GPU: its configuration, what it declares, and its host-side logic (parts, block, cache of latent
vectors, step function) run on the CPU with plain PyTorch functions standing in for the kernels, in every cutting,
against the plain implementation."""

from __future__ import annotations

import copy

import pytest
import torch

import helpers
import plain_ops
import plain_vesidra as plain
import vesidra_helpers as vh


def test_configuration_reads_every_size_and_round_trips():
    import miniserve_b200  # noqa: F401
    from miniserve_b200.config import VesidraConfig, resolve_architecture
    from miniserve_b200.parts import DecoderModel, PagedLatentNeed

    for name, raw in vh.CONFIGS.items():
        architecture = resolve_architecture(raw)
        config = architecture.config_class.from_dict(raw)
        assert isinstance(config, VesidraConfig) and config.to_dict() == raw
        spec = architecture.build_spec(config)
        assert spec.output_name is None and spec.embedding_scale == raw["embedding"]["scale"] and spec.vocab_size == raw["vocab"]
        assert all(layer.block.kind == "parallel" and layer.feed_forward_norm is None for layer in spec.layers)
        model = DecoderModel(spec, torch.float32, "cpu")
        needs = [g.need for g in model.cache_groups]
        assert all(isinstance(need, PagedLatentNeed) for need in needs)
        assert sorted({(m["mixer"]["kv_rank"], m["mixer"]["rot_dim"]) for m in raw["layers"]}) == sorted((n.rank, n.rot) for n in needs)
        names = {s.name: s.shape for s in model.param_specs()}
        first = raw["layers"][0]["mixer"]
        assert names["l0.mix.q"] == (first["heads"] * (first["dim"] + first["rot_dim"]), raw["width"])
        assert names["l0.mix.dkv"] == (first["kv_rank"] + first["rot_dim"], raw["width"])
        assert names["l0.mix.uk"] == (first["heads"] * first["dim"], first["kv_rank"])
        assert names["l0.mix.uv"] == (first["heads"] * first["vdim"], first["kv_rank"])
        assert names["l0.mix.g"] == (first["heads"], raw["width"]) and names["final.norm"] == (raw["width"],)
        for index, entry in enumerate(raw["layers"]):
            has = {n.split(".", 2)[2] for n in names if n.startswith(f"l{index}.mlp.")}
            if entry["mlp"] is None:
                assert not has
            elif entry["mlp"]["kind"] == "dense":
                assert has == {"gate", "up", "down"}
            else:
                wanted = {"router", "router.b"} | {f"e{e}.{p}" for e in range(entry["mlp"]["router"]["experts"]) for p in ("up", "down")}
                if entry["mlp"]["shared"]:
                    wanted |= {"shared.up", "shared.down"}
                assert has == wanted


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="ring_attention"), "not implemented"),
    (lambda c: c["layers"][0]["mlp"].update(kind="bilinear"), "not implemented"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "odd"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=64), "exceeds"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "exceeds"),
    (lambda c: c["norm"].update(eps=0.0), "positive"),
    (lambda c: c.update(layers=[]), "non-empty"),
    (lambda c: c.update(width=2.5), "integer"),
])
def test_configuration_refuses_what_it_cannot_run(change, message):
    import miniserve_b200  # noqa: F401
    from miniserve_b200.config import VesidraConfig

    raw = copy.deepcopy(vh.VESIDRA_A)
    change(raw)
    with pytest.raises(ValueError, match=message):
        VesidraConfig.from_dict(raw)


def test_scaled_frequencies_against_the_plain_statement():
    import miniserve_b200  # noqa: F401
    from miniserve_b200.parts.position import RotaryPosition

    for dims, base, scaling in [(8, 5000.0, vh.YARN_A), (16, 5000.0, vh.YARN_B), (32, 10000.0, dict(factor=4.0, original=1000, fast=30.0, slow=1.5)),
                                (6, 100.0, None), (64, 1e6, dict(factor=1.0, original=4096, fast=32.0, slow=1.0))]:
        part = RotaryPosition(head_dim=dims, theta=base, rotary_dim=dims, scaling=scaling)
        expected, magnitude = plain.rotary_frequencies(dict(base=base, dims=dims, scaling=scaling))
        got = part.inv_freq("cpu").double()
        assert torch.allclose(got, expected, rtol=2e-7, atol=0) and abs(part.magnitude - magnitude) < 1e-12
        if scaling and scaling["factor"] > 1:
            assert float(got[-1]) < float(base ** (-2.0 * (dims // 2 - 1) / dims)) or dims <= 8     # the slow pairs are stretched


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
        folder = vh.make_folder(tmp_path, name, seed=2)
        runtime = runtime_module.build_runtime(folder, EngineConfig(
            dtype="float32", kv_block_size=page_size, num_kv_blocks=num_pages, max_num_seqs=max_seqs,
            enable_prefix_cache=False, device="cpu", decode_execution="eager"))
        return folder, runtime
    return build


@pytest.mark.parametrize("name,page_size", [("a", 8), ("b", 4)])
@pytest.mark.parametrize("cutting", ["whole", "tail", "portions", "mixed"])
def test_cuttings_match_plain_on_cpu(cpu_runtime, name, page_size, cutting):
    from miniserve_b200.trace import TraceSession

    vocab = vh.CONFIGS[name]["vocab"]
    requests = {f"r{i}": helpers.random_tokens(vocab, n, seed=20 + i) for i, n in enumerate((1, 6, 17, 30, 41))}
    steps = {"whole": helpers.cut_whole, "tail": lambda r: helpers.cut_decode_tail(r, 9),
             "portions": helpers.cut_portions, "mixed": helpers.cut_mixed}[cutting](requests)
    pages = (helpers.max_live_tokens(steps, granule=page_size * 2) + page_size - 1) // page_size
    folder, runtime = cpu_runtime(name, pages, page_size)
    assert runtime.max_model_len == pages * page_size            # no position limit of the design's own: the pool's size
    session, outputs = TraceSession(runtime), {}
    for record in steps:
        outputs[record["step"]] = session.run(record).double()
        runtime.manager.check_invariants()
    got = helpers.collect(steps, outputs)
    config, weights = plain.load_folder(folder)
    for rid, tokens in requests.items():
        expected, _, gap = plain.forward(tokens, weights, config, return_layers=True)
        assert gap > 0.2, "the routing is too close to a tie for this test to mean anything"
        assert sorted(got[rid]) == list(range(len(tokens)))
        for position, row in got[rid].items():
            assert torch.allclose(row, expected[position], atol=2e-4, rtol=2e-4), (rid, position)
    assert not runtime.manager.requests
    assert all(a.free_count == a.num_pages for a in runtime.manager.allocators)
