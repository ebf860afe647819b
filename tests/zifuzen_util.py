"""Small Zifuzen configurations of the tests, model folders with random weights for them (made in a temporary
folder, never committed), requests whose routing is decisive, and the plain implementation's logits.

The configurations differ from one another in every size, in the order of their layers and in what is present:

* ``Z1``: attention first, with values wider than keys (the kernel for keys and values of different widths), two
  query heads per key/value head; a delta layer with two value heads per q/k head and four taps under routed experts
  in three groups of which two are kept, with a shared expert; an attention layer without a feed-forward that reads
  the first layer's pages; a ``delta_2`` layer with as many q/k heads as value heads and two taps under routed experts
  without groups, without a shared expert and with a top of one; a soft cap on the logits; widths that are no
  multiple of 16.
* ``Z2``: a delta layer first, with a convolution of one tap (no convolution memory) and no feed-forward; attention
  whose keys and values share a width the plain kernels take, one key/value head per query head; a top of four
  among eight experts in two groups of which one is kept; a dense feed-forward on a delta layer; two attention layers
  that read a third one's pages; no cap on the logits.
* ``Z3``: sizes at which the tensor-core attention kernels, the small-batch product kernel and the 16-byte paths
  run: attention heads of 128 and of 64 dims, delta heads of 128 x 128 and 64 x 32.

Random matrices of N(0, 0.02) would leave every expert choice to the correction alone and every decay near one half;
the folders' routers are scaled up, their decay rates spread over one to two orders of magnitude, and the embedding
is brought to the size of the normed branches.
"""

from __future__ import annotations

import copy
import functools
import os
import tempfile

import torch
from safetensors.torch import load_file, save_file

from plain import zifuzen_plain as plain


def _attention(heads, kv_heads, dim, vdim, scale, kv_from=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return mixer


def _delta(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def _moe(experts, top, ff, limit, scale, groups=None, shared=None):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    mlp = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": router}
    if shared is not None:
        mlp["shared"] = {"ff": shared[0], "limit": shared[1]}
    return mlp


def _layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": mlp} if isinstance(mlp, int) else mlp}


Z1 = {
    "architecture": "Zifuzen", "vocab": 211, "width": 72, "max_positions": 300, "embedding": {"scale": 3.0},
    "norm": {"eps": 1e-5}, "logit_softcap": 7.0,
    "layers": [
        _layer("attention", _attention(4, 2, 8, 24, 0.5), 96),
        _layer("delta", _delta(4, 2, 12, 8, 4), _moe(6, 2, 40, 1.5, 1.5, groups=(3, 2), shared=(24, 0.7))),
        _layer("attention", _attention(4, 2, 8, 24, 0.4, kv_from=0), None),
        _layer("delta_2", _delta(3, 3, 16, 20, 2), _moe(5, 1, 24, 2.5, 0.8)),
    ],
}
Z2 = {
    "architecture": "Zifuzen", "vocab": 97, "width": 48, "max_positions": 260, "embedding": {"scale": 1.0},
    "norm": {"eps": 1e-6}, "logit_softcap": None,
    "layers": [
        _layer("delta_2", _delta(2, 1, 24, 8, 1), None),
        _layer("attention", _attention(3, 3, 16, 16, 0.3), _moe(8, 4, 16, 3.0, 2.5, groups=(2, 1), shared=(32, 3.0))),
        _layer("delta", _delta(6, 2, 8, 16, 3), 64),
        _layer("attention", _attention(6, 3, 16, 16, 0.25, kv_from=1), 40),
        _layer("attention", _attention(3, 3, 16, 16, 0.35, kv_from=1), None),
    ],
}
Z3 = {
    "architecture": "Zifuzen", "vocab": 320, "width": 256, "max_positions": 400, "embedding": {"scale": 8.0},
    "norm": {"eps": 1e-6}, "logit_softcap": 20.0,
    "layers": [
        _layer("delta", _delta(4, 2, 128, 128, 4), _moe(8, 2, 128, 2.0, 1.0, groups=(4, 2), shared=(192, 2.0))),
        _layer("attention", _attention(4, 2, 128, 128, 0.09), 512),
        _layer("delta_2", _delta(8, 8, 64, 32, 3), None),
        _layer("attention", _attention(8, 2, 128, 128, 0.09, kv_from=1), _moe(6, 2, 64, 1.0, 2.0)),
        _layer("attention", _attention(8, 1, 64, 64, 0.12), 384),
    ],
}
CONFIGS = {"Z1": (Z1, 16), "Z2": (Z2, 32), "Z3": (Z3, 16)}


def config(name: str) -> dict:
    return copy.deepcopy(CONFIGS[name][0])


@functools.lru_cache(maxsize=None)
def model_folder(name: str, seed: int = 3) -> str:
    from ampere_kv_engine_b200.models.registry import config_from_dict
    from ampere_kv_engine_b200.weights.random_init import write_random_model
    _, cfg = config_from_dict(config(name))
    out = tempfile.mkdtemp(prefix=f"zifuzen_{name}_")
    write_random_model(cfg, seed, out, torch.float32)
    path = os.path.join(out, "model.safetensors")
    tensors = load_file(path)
    g = torch.Generator().manual_seed(seed + 100)
    tensors["embed"] = tensors["embed"] * (25.0 / cfg.embedding_scale)
    tensors["pos"] = tensors["pos"] * 25.0
    for i, layer in enumerate(cfg.layers):
        if layer.type != "attention":
            heads = layer.mixer["heads"]
            # decays between about 0.995 and 0.6 a token: what is written is still there a hundred tokens on
            tensors[f"l{i}.mix.A_log"] = torch.empty(heads).uniform_(-4.5, -0.5, generator=g)
            tensors[f"l{i}.mix.a"] = tensors[f"l{i}.mix.a"] * 20.0
            tensors[f"l{i}.mix.b"] = tensors[f"l{i}.mix.b"] * 20.0
            for name_ in ("q", "k", "v"):
                tensors[f"l{i}.mix.{name_}.conv"] = tensors[f"l{i}.mix.{name_}.conv"] - 0.3     # taps of both signs
        if layer.mlp is not None and layer.mlp.get("kind") == "moe":
            # router logits of about the same spread at every width
            tensors[f"l{i}.mlp.router"] = tensors[f"l{i}.mlp.router"] * (12.0 * (72.0 / cfg.width) ** 0.5)
            # expert outputs large enough for the clamps to bite
            for e in range(layer.mlp["router"]["experts"]):
                tensors[f"l{i}.mlp.e{e}.gate"] = tensors[f"l{i}.mlp.e{e}.gate"] * 15.0
                tensors[f"l{i}.mlp.e{e}.up"] = tensors[f"l{i}.mlp.e{e}.up"] * 15.0
    # bfloat16-representable values: both precisions then run on the same weights
    save_file({k: v.to(torch.bfloat16).to(torch.float32).contiguous() for k, v in tensors.items()}, path,
              metadata={"format": "pt"})
    return out


def plain_weights(folder: str) -> dict:
    return {k: v.double() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}


def plain_logits(folder: str, raw: dict, requests: dict[str, list[int]]) -> dict[str, torch.Tensor]:
    """float64 logits of every request as a whole sequence, as float32."""
    w = plain_weights(folder)
    return {rid: plain.forward(raw, w, toks).float() for rid, toks in requests.items()}


def decisive_requests(folder: str, raw: dict, lengths, seed: int, margin: float = 0.03, tries: int = 400
                      ) -> dict[str, list[int]]:
    """Random requests of the given lengths in which no expert choice is a close call: for every token and routed
    layer the chosen experts (and kept groups) lead the others by at least ``margin`` in the plain implementation, so
    that a rounding of the router's input cannot change the choice.  Found by trying seeds; a request that cannot be
    had whole is put together token by token."""
    w = plain_weights(folder)
    g = torch.Generator().manual_seed(seed)
    routed = any((l.get("mlp") or {}).get("kind") == "moe" for l in raw["layers"])
    out = {}
    for i, n in enumerate(lengths):
        toks: list[int] = []
        while len(toks) < n:
            for _ in range(tries):
                cand = toks + torch.randint(0, raw["vocab"], (min(4, n - len(toks)),), generator=g).tolist()
                margins: list = []
                if routed:
                    plain.forward(raw, w, cand, margins=margins)
                if all(float(m[len(toks):].min()) >= margin for m in margins):
                    toks = cand
                    break
            else:
                raise AssertionError("no decisive continuation found; lower the margin")
        out[f"r{i}"] = toks
    return out


def random_config(seed: int) -> dict:
    """A seeded random configuration of the design: 3 to 6 layers in any order, every size drawn anew (widths and
    head sizes that are no multiples of 16 among them), optional groups, shared expert, feed-forward and logit cap, and
    attention layers that read the pages of a random earlier attention layer of the same shape."""
    import random
    rng = random.Random(seed)
    width = rng.choice((40, 48, 64, 72, 96, 104, 128))
    layers, owners = [], []          # owners: (layer index, kv_heads, dim, vdim) of attention layers with their own k/v
    for i in range(rng.randint(3, 6)):
        if rng.random() < 0.5:
            kv = rng.choice((1, 2, 3))
            heads = kv * rng.choice((1, 2, 4))
            dim = rng.choice((8, 12, 16, 24, 32, 48, 64))
            vdim = dim if rng.random() < 0.5 else rng.choice((8, 16, 20, 32, 40))
            source = None
            same = [o for o in owners if rng.random() < 0.6]
            if same:
                j, kv, dim, vdim = rng.choice(same)
                heads = kv * rng.choice((1, 2, 4))
                source = j
            else:
                owners.append((i, kv, dim, vdim))
            mixer = _attention(heads, kv, dim, vdim, round(rng.uniform(0.5, 2.0) * dim ** -0.5, 4), kv_from=source)
            kind = "attention"
        else:
            kv = rng.choice((1, 2, 3))
            mixer = _delta(kv * rng.choice((1, 2, 3)), kv, rng.choice((8, 12, 16, 24, 32, 64)),
                           rng.choice((4, 8, 12, 16, 32)), rng.choice((1, 2, 3, 4, 5)))
            kind = rng.choice(("delta", "delta_2"))
        choice = rng.random()
        if choice < 0.2:
            mlp = None
        elif choice < 0.45:
            mlp = rng.choice((24, 40, 64, 96))
        else:
            count = rng.choice((1, 2, 3, 4))
            per = rng.choice((1, 2, 3, 4))
            keep = rng.randint(1, count)
            experts = count * per
            top = rng.randint(1, min(4, keep * per))
            mlp = _moe(experts, top, rng.choice((8, 16, 24, 40)), rng.choice((0.5, 1.0, 2.0, 7.0)),
                       round(rng.uniform(0.5, 3.0), 3), groups=(count, keep) if rng.random() < 0.7 or count > 1 else None,
                       shared=(rng.choice((8, 16, 48)), rng.choice((0.5, 2.0))) if rng.random() < 0.6 else None)
        layers.append(_layer(kind, mixer, mlp))
    return {"architecture": "Zifuzen", "vocab": rng.choice((61, 128, 257)), "width": width,
            "max_positions": 200, "embedding": {"scale": round(rng.uniform(0.5, 20.0), 3)},
            "norm": {"eps": rng.choice((1e-5, 1e-6))}, "logit_softcap": rng.choice((None, 5.0, 30.0)), "layers": layers}


@functools.lru_cache(maxsize=None)
def random_model_folder(seed: int) -> str:
    """A model folder for :func:`random_config` with the same scalings as :func:`model_folder`."""
    CONFIGS[f"random{seed}"] = (random_config(seed), 16)
    return model_folder(f"random{seed}", seed=seed)
