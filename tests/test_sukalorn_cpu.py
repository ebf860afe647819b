"""Sukalorn without a GPU: configuration, the spec that is built from it, the cache kind its block attention asks
for, and the engine's host side (batch layout, cache manager, step function, scheduler, replay, generation) driven
through the stand-in kernels against the plain implementation."""

import copy

import pytest
import torch

import replay_util as ru
import sukalorn_util as su
from plain import sukalorn_plain as plain

LENGTHS = (1, 2, 19, 47, 130)


def test_configuration_reads_every_size_and_names_what_is_wrong():
    from ampere_kv_engine_b200.config.model_config import ConfigError
    from ampere_kv_engine_b200.models.registry import config_from_dict
    arch, cfg = config_from_dict(su.config("S1"))
    assert arch.name == "Sukalorn" and cfg.vocab_size == 211 and cfg.width == 72 and len(cfg.layers) == 5
    assert config_from_dict(cfg.to_dict())[1] == cfg
    for path, value, word in ((("layers", 1, "type"), "conv", "type"), (("layers", 0, "mixer", "rot", "dims"), 3, "dims"),
                              (("layers", 1, "mixer", "kv_heads"), 3, "kv_heads"), (("norm", "eps"), 0, "eps"),
                              (("layers", 1, "mlp", "kind"), "routed", "kind"), (("vocab",), -1, "vocab")):
        raw = su.config("S1")
        node = raw
        for key in path[:-1]:
            node = node[key]
        node[path[-1]] = value
        with pytest.raises(ConfigError, match=word):
            config_from_dict(raw)


def test_spec_gives_blending_layers_their_roles_and_layers_their_parts():
    from ampere_kv_engine_b200.models.registry import config_from_dict
    arch, cfg = config_from_dict(su.config("S1"))
    spec = arch.build_spec(cfg)
    kinds = [l.mixer.kind for l in spec.layers]
    assert kinds == ["latent_attention", "scored_attention", "scored_attention", "scored_attention", "latent_attention"]
    assert [l.mixer.params.get("value_blend") for l in spec.layers[1:4]] == ["source", "reader", None]
    assert [l.feed_forward is None for l in spec.layers] == [False, False, True, False, True]
    assert spec.layers[1].mixer.params["chunk"] == 20 and spec.layers[1].mixer.params["softcap"] == 2.0
    from ampere_kv_engine_b200.models.decoder import DecoderModel
    specs = DecoderModel(spec, dtype=torch.float32, device="cpu").param_specs()
    wanted = {name for name, ps in specs.items() if not ps.optional}
    assert {"embed", "embed.norm", "final.norm", "head", "l0.mix.dq.norm", "l1.mix.vmix", "l1.mix.g", "l3.mlp.down",
            "l0.norm2", "l2.norm1"} <= wanted
    # a layer without a feed-forward wants no second norm, a layer that does not blend no blend scalar; a checkpoint
    # may still carry them
    assert "l2.mlp.up" not in specs and not ({"l2.norm2", "l3.mix.vmix"} & wanted)
    assert specs["l2.norm2"].optional and specs["l3.mix.vmix"].optional


def test_block_cache_gives_pages_back_once_a_sequence_has_left_the_block():
    from ampere_kv_engine_b200.cache.manager import CacheManager
    from ampere_kv_engine_b200.parts.base import CacheSpec
    spec = CacheSpec(kind="chunk", num_kv_heads=1, head_dim=8, chunk=20)
    full = CacheSpec(kind="full", num_kv_heads=1, head_dim=8)
    m = CacheManager([spec, full], [None, None], page_size=4, num_pages=40, max_seqs=2, allocate_storage=False)
    assert len(m.groups) == 2
    seq = m.open("a")
    for step, (tokens, held) in enumerate(((19, 5), (1, 0), (1, 1), (18, 5), (3, 1), (45, 2))):
        m.reserve(seq, tokens)
        m.commit(seq, tokens)
        # the block of position `length` starts at length // 20 * 20: pages wholly before it are back in the pool
        assert len(seq.held_pages(0)) == held, (step, seq.length, seq.held_pages(0))
        assert len(seq.held_pages(1)) == (seq.length + 3) // 4
        m.check_invariants()
    first = seq.length // 20 * 20
    assert m.slot_of(seq, 0, first) >= 0
    with pytest.raises(ValueError):
        m.slot_of(seq, 0, first - 1 - (first - 1) % 4)
    m.close(seq)
    assert m.free_pages() == [40, 40]


@pytest.mark.parametrize("name", ["S1", "S2"])
@pytest.mark.parametrize("mode", ["whole", "last32", "portions", "mixed"])
def test_replay_matches_plain(fake_ext, name, mode):
    raw, page = su.CONFIGS[name]
    folder = su.model_folder(name)
    requests = ru.make_requests(raw["vocab"], LENGTHS + ((70, 45) if mode == "mixed" else ()), seed=11)
    expected = su.plain_logits(folder, raw, requests)
    max_tokens = 64 * 6
    trace = {"whole": ru.trace_whole, "last32": ru.trace_last_decoded, "portions": ru.trace_portions,
             "mixed": lambda r: ru.trace_mixed(r, max_tokens, seed=5)}[mode](requests)
    outputs = ru.run_inprocess(folder, "float32", trace, max_tokens, page_size=page)
    ru.compare(trace, outputs, expected, "float32")


def test_greedy_generation_through_the_scheduler(fake_ext):
    from ampere_kv_engine_b200.engine.engine import Engine
    raw, page = su.CONFIGS["S2"]
    folder = su.model_folder("S2")
    engine = Engine.from_pretrained(folder, dtype="float32", device="cpu", page_size=page, num_pages=12,
                                    max_batch_tokens=24, max_seqs=4)
    prompts = [torch.randint(0, raw["vocab"], (n,), generator=torch.Generator().manual_seed(n)).tolist()
               for n in (3, 30, 61)]
    got = engine.generate(prompts, max_new_tokens=6, ignore_eos=True)
    w = su.plain_weights(folder)
    assert got == [plain.greedy_generate(w, raw, p, 6) for p in prompts]
    assert engine.manager.free_pages() == [12] * len(engine.manager.groups)
    engine.manager.check_invariants()


def test_a_reader_without_a_source_is_refused(fake_ext):
    """A blending layer needs the source's values of the same step; a spec that names no source fails loudly."""
    from ampere_kv_engine_b200.config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    from ampere_kv_engine_b200.engine.batch import SeqStep
    from ampere_kv_engine_b200.engine.step import ModelRunner
    from ampere_kv_engine_b200.models.decoder import DecoderModel
    from ampere_kv_engine_b200.weights.random_init import init_random
    norm = lambda name: PartSpec("rmsnorm", {"eps": 1e-6}, name)
    mixer = PartSpec("scored_attention", {"num_heads": 2, "num_kv_heads": 1, "head_dim": 8, "v_dim": 8, "scale": 0.3,
                                          "value_blend": "reader"}, "l0.attn")
    spec = ModelSpec(hidden_size=16, vocab_size=31, embedding=PartSpec("token_embedding", {"vocab_size": 31}, "emb"),
                     layers=(LayerSpec("prenorm", mixer, None, norm("l0.n1")),), schedule=(ScheduleEntry(0),),
                     final_norm=norm("final"), head=PartSpec("linear_head", {"vocab_size": 31}, "head"),
                     max_position=64)
    model = DecoderModel(spec, dtype=torch.float32, device="cpu")
    init_random(model, 0)
    runner = ModelRunner(model, page_size=4, num_pages=8, max_seqs=2, cuda_graphs=False)
    with pytest.raises(ValueError, match="no layer before"):
        runner.step([SeqStep(runner.open("a"), [1, 2, 3], [2])])
    assert runner.manager.free_pages() == [8]


def test_a_checkpoint_may_carry_tensors_of_parts_a_layer_does_not_have(fake_ext, tmp_path):
    """The second norm of a layer without a feed-forward and the blend scalar of a layer that does not blend are
    accepted when a checkpoint has them, and change nothing."""
    import os
    import shutil
    from safetensors.torch import load_file, save_file
    from ampere_kv_engine_b200.engine.engine import Engine
    raw, page = su.CONFIGS["S1"]
    folder = su.model_folder("S1")
    copy_dir = str(tmp_path / "with_extras")
    shutil.copytree(folder, copy_dir)
    tensors = load_file(os.path.join(copy_dir, "model.safetensors"))
    assert "l2.norm2" not in tensors and "l3.mix.vmix" not in tensors
    tensors["l2.norm2"] = torch.full((raw["width"],), 0.5)
    tensors["l3.mix.vmix"] = torch.tensor(0.9)
    save_file(tensors, os.path.join(copy_dir, "model.safetensors"), metadata={"format": "pt"})
    prompts = [[5, 7, 11, 13, 17, 19, 23]]
    a = Engine.from_pretrained(folder, dtype="float32", device="cpu", page_size=page, num_pages=8, max_seqs=2)
    b = Engine.from_pretrained(copy_dir, dtype="float32", device="cpu", page_size=page, num_pages=8, max_seqs=2)
    assert a.generate(prompts, max_new_tokens=4, ignore_eos=True) == b.generate(prompts, max_new_tokens=4, ignore_eos=True)
