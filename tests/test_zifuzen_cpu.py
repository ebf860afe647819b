"""Zifuzen without a GPU: configuration, the spec that is built from it, the state its delta layers ask the cache
manager for, and the engine's host side (batch layout, cache and state manager, step function, scheduler, replay,
generation) driven through the stand-in kernels against the plain implementation."""

import pytest
import torch

import replay_util as ru
import zifuzen_util as zu
from plain import zifuzen_plain as plain

LENGTHS = (1, 2, 19, 47, 130)


def test_configuration_reads_every_size_and_names_what_is_wrong():
    from ampere_kv_engine_b200.config.model_config import ConfigError
    from ampere_kv_engine_b200.models.registry import config_from_dict
    arch, cfg = config_from_dict(zu.config("Z1"))
    assert arch.name == "Zifuzen" and cfg.vocab_size == 211 and cfg.width == 72 and len(cfg.layers) == 4
    assert cfg.max_position_embeddings == 300 and cfg.embedding_scale == 3.0 and cfg.logit_softcap == 7.0
    assert config_from_dict(cfg.to_dict())[1] == cfg
    assert config_from_dict(zu.config("Z2"))[1].logit_softcap is None
    for path, value, word in ((("layers", 1, "type"), "conv", "type"), (("layers", 1, "mixer", "conv"), 0, "conv"),
                              (("layers", 0, "mixer", "kv_heads"), 3, "kv_heads"), (("norm", "eps"), 0, "eps"),
                              (("layers", 1, "mlp", "kind"), "routed", "kind"), (("vocab",), -1, "vocab"),
                              (("layers", 2, "mixer", "kv_from"), 1, "kv_from"),       # a delta layer has no keys
                              (("layers", 2, "mixer", "kv_from"), 2, "kv_from"),       # not an earlier layer
                              (("layers", 2, "mixer", "vdim"), 16, "kv_from"),         # another shape than the source's
                              (("layers", 1, "mlp", "router", "groups", "count"), 4, "count"),
                              (("layers", 1, "mlp", "router", "top"), 5, "top"),
                              (("layers", 1, "mlp", "expert", "limit"), 0, "limit"),
                              (("logit_softcap",), -2.0, "logit_softcap"), (("max_positions",), 0, "max_positions")):
        raw = zu.config("Z1")
        node = raw
        for key in path[:-1]:
            node = node[key]
        node[path[-1]] = value
        with pytest.raises(ConfigError, match=word):
            config_from_dict(raw)


def test_spec_gives_layers_their_parts_and_borrowers_their_source():
    from ampere_kv_engine_b200.models.decoder import DecoderModel
    from ampere_kv_engine_b200.models.registry import config_from_dict
    arch, cfg = config_from_dict(zu.config("Z2"))
    spec = arch.build_spec(cfg)
    assert [l.mixer.kind for l in spec.layers] == ["gated_delta", "scored_attention", "gated_delta", "scored_attention",
                                                   "scored_attention"]
    assert [l.block for l in spec.layers] == ["postnorm"] * 5
    assert [e.cache_of for e in spec.schedule] == [None, None, None, 1, 1]
    assert [None if l.feed_forward is None else l.feed_forward.kind for l in spec.layers] == \
        [None, "routed_experts", "gated_mlp", "gated_mlp", None]
    assert spec.layers[1].feed_forward.params["groups"] == 2 and spec.layers[1].feed_forward.params["keep_groups"] == 1
    model = DecoderModel(spec, dtype=torch.float32, device="cpu")
    specs = model.param_specs()
    wanted = {name for name, ps in specs.items() if not ps.optional}
    assert {"embed", "pos", "final.norm", "head", "l0.mix.q.conv", "l0.mix.A_log", "l0.mix.dt_bias", "l1.mix.k.norm",
            "l1.mlp.e7.down", "l1.mlp.correction", "l1.mlp.shared.up", "l2.mlp.gate.b", "l3.mix.q.norm",
            "l3.mix.o"} <= wanted
    # a layer that reads another's pages has no key or value tensors; a layer without a feed-forward no second norm
    assert not ({"l3.mix.k", "l3.mix.v", "l3.mix.k.norm", "l4.mix.k", "l0.mlp.gate"} & set(specs))
    assert specs["l0.norm2"].optional and specs["l4.norm2"].optional and "l0.norm2" not in wanted
    assert specs["l0.mix.q.conv"].shape == (24, 1) and specs["l2.mix.v.conv"].shape == (96, 3)
    # one state per delta layer (its memory and its convolutions' inputs), one cache group for the attention layers
    from ampere_kv_engine_b200.kernels import ops
    states = [s.state_shape for s in model.cache_specs()]
    assert states == [(ops.delta_state_floats(2, 1, 24, 8, 1)[1],), (), (ops.delta_state_floats(6, 2, 8, 16, 3)[1],), (), ()]
    assert states[0][0] >= 2 * 24 * 8 and states[2][0] >= 6 * 8 * 16 + 2 * (2 * 16 + 96) and states[2][0] % 4 == 0
    assert len({s.group_key() for s in model.cache_specs() if s.kind != "none"}) == 1


def test_state_slots_are_zeroed_when_a_request_opens_and_a_captured_step_would_not_touch_padding():
    from ampere_kv_engine_b200.cache.manager import CacheManager
    from ampere_kv_engine_b200.engine.batch import BatchLayout, SeqStep, fill_host
    from ampere_kv_engine_b200.parts.base import CacheSpec
    import numpy as np
    m = CacheManager([CacheSpec(kind="none", state_shape=(5,)), CacheSpec(kind="full", num_kv_heads=1, head_dim=8)],
                     [None, None], page_size=4, num_pages=8, max_seqs=3)
    a = m.open("a")
    m.state[0][a.state_slot] = 7.0
    m.close(a)
    b = m.open("b")
    assert b.state_slot == a.state_slot and float(m.state[0][b.state_slot].abs().sum()) == 0.0
    m.reserve(b, 1)
    layout = BatchLayout(4, 4, 4, 4, (1,))
    host = np.empty(layout.total, dtype=np.int32)
    fill_host(m, [SeqStep(b, [3], [0])], layout, host, 1)
    slots = host[layout.offsets[4]:layout.offsets[4] + 4].tolist()
    assert slots == [b.state_slot, -1, -1, -1]


@pytest.mark.parametrize("name", ["Z1", "Z2"])
@pytest.mark.parametrize("mode", ["whole", "last32", "portions", "mixed"])
def test_replay_matches_plain(fake_ext, name, mode):
    raw, page = zu.CONFIGS[name]
    folder = zu.model_folder(name)
    requests = ru.make_requests(raw["vocab"], LENGTHS + ((70, 45) if mode == "mixed" else ()), seed=11)
    expected = zu.plain_logits(folder, raw, requests)
    max_tokens = 64 * 6
    trace = {"whole": ru.trace_whole, "last32": ru.trace_last_decoded, "portions": ru.trace_portions,
             "mixed": lambda r: ru.trace_mixed(r, max_tokens, seed=5)}[mode](requests)
    outputs = ru.run_inprocess(folder, "float32", trace, max_tokens, page_size=page)
    ru.compare(trace, outputs, expected, "float32")


def test_greedy_generation_through_the_scheduler(fake_ext):
    from ampere_kv_engine_b200.engine.engine import Engine
    raw, page = zu.CONFIGS["Z1"]
    folder = zu.model_folder("Z1")
    engine = Engine.from_pretrained(folder, dtype="float32", device="cpu", page_size=page, num_pages=12,
                                    max_batch_tokens=24, max_seqs=4)
    prompts = [torch.randint(0, raw["vocab"], (n,), generator=torch.Generator().manual_seed(n)).tolist()
               for n in (3, 30, 61)]
    got = engine.generate(prompts, max_new_tokens=6, ignore_eos=True)
    w = zu.plain_weights(folder)
    assert got == [plain.greedy_generate(raw, w, p, 6) for p in prompts]
    assert engine.manager.free_pages() == [12] * len(engine.manager.groups)
    engine.manager.check_invariants()
    # the same prompts again land in state slots that were used before and give the same tokens
    assert engine.generate(prompts, max_new_tokens=6, ignore_eos=True) == got


def test_a_model_of_delta_layers_alone_has_no_pages_and_still_runs(fake_ext, tmp_path):
    from ampere_kv_engine_b200.engine.engine import Engine
    from ampere_kv_engine_b200.models.registry import config_from_dict
    from ampere_kv_engine_b200.weights.random_init import write_random_model
    raw = zu.config("Z1")
    raw["layers"] = [raw["layers"][1], raw["layers"][3]]
    _, cfg = config_from_dict(raw)
    folder = write_random_model(cfg, 4, str(tmp_path / "deltas"), torch.float32)
    engine = Engine.from_pretrained(folder, dtype="float32", device="cpu", page_size=16, num_pages=4, max_seqs=2)
    assert engine.manager.groups == []
    prompt = [5, 7, 11, 13, 17, 19, 23, 29, 31]
    got = engine.generate([prompt], max_new_tokens=5, ignore_eos=True)
    assert got == [plain.greedy_generate(raw, zu.plain_weights(folder), prompt, 5)]


def test_a_borrowing_mixer_must_be_scheduled_behind_its_source(fake_ext):
    """A mixer without keys and values of its own that the schedule gives a cache of its own fails loudly."""
    from ampere_kv_engine_b200.config.spec import ScheduleEntry
    from ampere_kv_engine_b200.engine.batch import SeqStep
    from ampere_kv_engine_b200.engine.step import ModelRunner
    from ampere_kv_engine_b200.models.decoder import DecoderModel
    from ampere_kv_engine_b200.models.registry import config_from_dict
    from ampere_kv_engine_b200.weights.random_init import init_random
    import dataclasses
    arch, cfg = config_from_dict(zu.config("Z1"))
    spec = arch.build_spec(cfg)
    spec = dataclasses.replace(spec, schedule=tuple(ScheduleEntry(i) for i in range(len(spec.layers))))
    model = DecoderModel(spec, dtype=torch.float32, device="cpu")
    init_random(model, 0)
    runner = ModelRunner(model, page_size=4, num_pages=8, max_seqs=2, cuda_graphs=False)
    with pytest.raises(ValueError, match="cache_of"):
        runner.step([SeqStep(runner.open("a"), [1, 2, 3], [2])])


@pytest.mark.parametrize("seed", [1, 2, 3, 4])
def test_random_configurations_replay(fake_ext, seed):
    """Seeded random configurations (layer order, sizes, groups, shared experts, borrowed pages drawn anew) through
    the engine's host side in a mixed trace."""
    folder = zu.random_model_folder(seed)
    raw = zu.CONFIGS[f"random{seed}"][0]
    requests = ru.make_requests(raw["vocab"], (1, 2, 23, 61, 37), seed=seed)
    expected = zu.plain_logits(folder, raw, requests)
    trace = ru.trace_mixed(requests, 64 * 4, seed=seed)
    outputs = ru.run_inprocess(folder, "float32", trace, 64 * 4, page_size=16)
    ru.compare(trace, outputs, expected, "float32")
