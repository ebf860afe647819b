"""The ``Sukalorn`` decoder as a model spec.

A normed token embedding, then pre-norm layers whose mixer is chosen layer by layer (``scored_attention`` with the
design's constants, or ``latent_attention``), each followed by a dense relu-squared feed-forward or by none, a final
norm and an untied head.  All norms keep their weight around zero (``1 + w``).  Tensor names: ``embed``,
``embed.norm``, ``l<i>.norm1|norm2``, ``l<i>.mix.*``, ``l<i>.mlp.up|down``, ``final.norm``, ``head``.

The first layer whose mixer blends values publishes its own values to the step; every later blending layer mixes
them into its own before they are cached.
"""

from __future__ import annotations

from ..config.model_config import SukalornConfig
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .registry import register_architecture

#: the distance bias of head h is 2 ** (-SLOPE_SPAN (h + 1) / heads) per position
SLOPE_SPAN = 8.0


def _norm(config: SukalornConfig, prefix: str, tensor: str) -> PartSpec:
    return PartSpec("rmsnorm", {"eps": config.norm_eps, "tensor": tensor, "unit_offset": True}, prefix)


def build_spec(config: SukalornConfig) -> ModelSpec:
    layers, unused = [], []
    blending_seen = False
    for i, layer in enumerate(config.layers):
        prefix, m = f"l{i}", layer.mixer
        if layer.type == "attention":
            blend = None
            if m.get("v_mix"):
                blend = "reader" if blending_seen else "source"
                blending_seen = True
            mask = m.get("mask") or {}
            mixer = PartSpec("scored_attention", {
                "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"], "v_dim": m["vdim"],
                "scale": m["scale"], "unit_norm": True, "norm_eps": config.norm_eps, "softcap": m.get("softcap"),
                "slope_span": SLOPE_SPAN, "chunk": mask.get("size"), "gated": True, "value_blend": blend,
                "names": {"q": "q", "k": "k", "v": "v", "gate": "g", "out": "o", "blend": "vmix"},
            }, f"{prefix}.mix")
        else:
            mixer = PartSpec("latent_attention", {
                "num_heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"], "v_dim": m["vdim"],
                "q_rank": m["q_rank"], "kv_rank": m["kv_rank"], "scale": m["scale"], "norm_eps": config.norm_eps,
                "rotary_base": m["rot"]["base"], "rotary_dims": m["rot"]["dims"],
                "names": {"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm",
                          "uk": "uk", "uv": "uv", "out": "o"},
            }, f"{prefix}.mix")
        ff = ff_norm = None
        if layer.mlp is not None:
            ff = PartSpec("dense_mlp", {"intermediate_size": layer.mlp["ff"], "activation": "relu2", "up": "up",
                                        "down": "down"}, f"{prefix}.mlp")
            ff_norm = _norm(config, prefix, "norm2")
        else:
            unused.append((f"{prefix}.norm2", (config.width,)))     # a layer without a feed-forward may still carry it
        layers.append(LayerSpec(block="prenorm", mixer=mixer, feed_forward=ff, mixer_norm=_norm(config, prefix, "norm1"),
                                feed_forward_norm=ff_norm))
    return ModelSpec(
        hidden_size=config.width,
        vocab_size=config.vocab,
        embedding=PartSpec("normed_token_embedding", {"vocab_size": config.vocab, "tensor": "embed",
                                                      "norm": _norm(config, "embed", "norm")}, ""),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=_norm(config, "final", "norm"),
        head=PartSpec("linear_head", {"vocab_size": config.vocab, "tied": False, "tensor": "head"}, ""),
        max_position=config.max_position_embeddings,
        eos_token_ids=config.eos_token_id,
        unused_tensors=tuple(unused),
    )


register_architecture("Sukalorn", SukalornConfig, build_spec)
