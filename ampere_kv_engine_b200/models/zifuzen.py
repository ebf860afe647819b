"""The ``Zifuzen`` decoder as a model spec.

A scaled token embedding plus a learned position row; layers whose branches are normed on the way *out*
(``x += LN(mixer(x))``, ``x += LN(ff(x))``, the branches read the stream itself); a mixer chosen layer by layer
(``scored_attention`` with a weighted RMS norm on queries and keys and nothing else done to the scores, possibly
reading the pages of an earlier attention layer; or ``gated_delta``); a feed-forward chosen layer by layer (a gated
dense one with biases and tanh GELU, ``routed_experts``, or none); a final LayerNorm, an untied head and a soft cap on
the logits.  Tensor names: ``embed``, ``pos``, ``l<i>.norm1|norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``,
``head``.

A layer with ``kv_from: j`` becomes a schedule position that reads the cache of position ``j``.
"""

from __future__ import annotations

from ..config.model_config import ZifuzenConfig
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .registry import register_architecture

#: constants the design fixes
UNIT_EPS = 1e-6             # inside the root when queries and keys of the delta rule are made unit vectors
SWISH_SLOPE = 1.702         # g * sigmoid(SWISH_SLOPE * g) in an expert
GROUP_TOP = 2               # a group of experts is scored by the sum of this many of its best choice scores
WEIGHT_EPS = 1e-20          # added to the sum the chosen experts' scores are divided by


def _norm(config: ZifuzenConfig, prefix: str, tensor: str) -> PartSpec:
    return PartSpec("layernorm", {"eps": config.norm_eps, "tensor": tensor}, prefix)


def _feed_forward(mlp: dict, prefix: str) -> PartSpec:
    if mlp.get("kind", "dense") == "dense":
        return PartSpec("gated_mlp", {
            "intermediate_size": mlp["ff"], "activation": "gelu_tanh", "bias": True,
            "names": {"gate": "gate", "up": "up", "down": "down", "gate_bias": "gate.b", "up_bias": "up.b",
                      "down_bias": "down.b"}}, prefix)
    router, groups = mlp["router"], mlp["router"].get("groups") or {"count": 1, "keep": 1}
    shared = mlp.get("shared")
    return PartSpec("routed_experts", {
        "experts": router["experts"], "top": router["top"], "groups": groups["count"], "keep_groups": groups["keep"],
        "group_top": GROUP_TOP, "route_scale": router["scale"], "weight_eps": WEIGHT_EPS, "score": "sigmoid",
        "intermediate_size": mlp["expert"]["ff"], "limit": mlp["expert"]["limit"], "swish_slope": SWISH_SLOPE,
        "shared": None if shared is None else {"intermediate_size": shared["ff"], "limit": shared["limit"]},
        "names": {"expert": "e{}", "gate": "gate", "up": "up", "down": "down", "router": "router",
                  "correction": "correction", "shared": "shared"}}, prefix)


def build_spec(config: ZifuzenConfig) -> ModelSpec:
    layers, schedule, unused = [], [], []
    for i, layer in enumerate(config.layers):
        prefix, m = f"l{i}", layer.mixer
        cache_of = None
        if layer.type == "attention":
            cache_of = m.get("kv_from")
            mixer = PartSpec("scored_attention", {
                "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"], "v_dim": m["vdim"],
                "scale": m["scale"], "unit_norm": True, "norm_weights": True, "norm_eps": config.norm_eps,
                "own_kv": cache_of is None,
                "names": {"q": "q", "k": "k", "v": "v", "out": "o", "q_norm": "q.norm", "k_norm": "k.norm"},
            }, f"{prefix}.mix")
        else:
            mixer = PartSpec("gated_delta", {
                "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"], "v_dim": m["vdim"],
                "taps": m["conv"], "unit_eps": UNIT_EPS, "norm_eps": config.norm_eps,
                "names": {"q": "q", "k": "k", "v": "v", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv",
                          "beta": "b", "step": "a", "rate_log": "A_log", "step_bias": "dt_bias", "gate": "g",
                          "norm": "norm", "out": "o"},
            }, f"{prefix}.mix")
        ff = ff_norm = None
        if layer.mlp is not None:
            ff = _feed_forward(layer.mlp, f"{prefix}.mlp")
            ff_norm = _norm(config, prefix, "norm2")
        else:
            unused.append((f"{prefix}.norm2", (config.width,)))     # a layer without a feed-forward may still carry it
        layers.append(LayerSpec(block="postnorm", mixer=mixer, feed_forward=ff, mixer_norm=_norm(config, prefix, "norm1"),
                                feed_forward_norm=ff_norm))
        schedule.append(ScheduleEntry(i, cache_of=cache_of))
    return ModelSpec(
        hidden_size=config.width,
        vocab_size=config.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": config.vocab, "tensor": "embed",
                                               "scale": config.embedding_scale, "position_tensor": "pos",
                                               "max_positions": config.max_positions}, ""),
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=_norm(config, "final", "norm"),
        head=PartSpec("linear_head", {"vocab_size": config.vocab, "tied": False, "tensor": "head",
                                      "softcap": config.logit_softcap}, ""),
        max_position=config.max_positions,
        eos_token_ids=config.eos_token_id,
        unused_tensors=tuple(unused),
    )


register_architecture("Zifuzen", ZifuzenConfig, build_spec)
