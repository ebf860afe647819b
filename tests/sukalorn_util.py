"""Small Sukalorn configurations of the tests, model folders with random weights for them (made in a temporary
folder, never committed) and the plain implementation's logits.

The configurations differ from one another in every size and in the order of their layers:

* ``S1``: a latent layer first; three attention layers of which the first two blend values (the first of them is the
  source) and the third does not; groups of two query heads; value width larger than the key width; a layer without a
  feed-forward; blocks of 20 positions (no multiple of the page size); widths that are no multiple of 16.
* ``S2``: attention first; as many key/value heads as query heads; one key/value head in another layer; blocks of 7
  and of 64 positions in different layers (two cache groups); a layer without blocks or cap; a rotation over fewer
  dims than the rotated part has.
* ``S3``: head and latent widths at which 16-byte key loads, the small-batch product kernel and the tensor-core
  attention kernels' scored forms run (keys and values of 128 dims: prompt and decode; of 64 dims: decode).

Random matrices of N(0, 0.02) would leave every softmax nearly flat; the folders' query/key matrices of the latent
mixers are scaled up so that attention weights differ by orders of magnitude.
"""

from __future__ import annotations

import copy
import functools
import os
import tempfile

import torch
from safetensors.torch import load_file, save_file

from plain import sukalorn_plain as plain


def _attention(heads, kv_heads, dim, vdim, scale, size=None, softcap=None, v_mix=False):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "v_mix": v_mix}
    if size is not None:
        mixer["mask"] = {"size": size}
    if softcap is not None:
        mixer["softcap"] = softcap
    return mixer


def _latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base, dims=None):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
            "scale": scale, "rot": {"base": base, "dims": rot_dim if dims is None else dims}}


def _layer(kind, mixer, ff):
    return {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


S1 = {
    "architecture": "Sukalorn", "vocab": 211, "width": 72, "norm": {"eps": 1e-5},
    "layers": [
        _layer("latent_attention", _latent(3, 8, 8, 12, 40, 24, 0.25, 100.0), 96),
        _layer("attention", _attention(4, 2, 8, 24, 0.5, size=20, softcap=2.0, v_mix=True), 96),
        _layer("attention", _attention(4, 2, 8, 24, 0.5, size=20, softcap=2.0, v_mix=True), None),
        _layer("attention", _attention(4, 2, 8, 24, 0.5, size=20, softcap=2.0, v_mix=False), 80),
        _layer("latent_attention", _latent(3, 8, 8, 12, 40, 24, 0.25, 100.0), None),
    ],
}
S2 = {
    "architecture": "Sukalorn", "vocab": 97, "width": 48, "norm": {"eps": 1e-6},
    "layers": [
        _layer("attention", _attention(3, 3, 16, 8, 0.3, size=7, softcap=30.0, v_mix=True), 64),
        _layer("attention", _attention(6, 1, 12, 24, 0.4, size=64, softcap=4.0, v_mix=False), 64),
        _layer("latent_attention", _latent(2, 12, 12, 20, 16, 36, 0.2, 5000.0, dims=4), 32),
        _layer("attention", _attention(3, 3, 16, 8, 0.3, size=7, softcap=30.0, v_mix=True), 64),
        _layer("attention", _attention(2, 2, 8, 8, 0.35), 64),
    ],
}
S3 = {
    "architecture": "Sukalorn", "vocab": 320, "width": 256, "norm": {"eps": 1e-6},
    "layers": [
        _layer("attention", _attention(4, 2, 128, 128, 0.09, size=96, softcap=10.0, v_mix=True), 512),
        _layer("latent_attention", _latent(20, 48, 16, 40, 96, 256, 0.1, 10000.0), 512),
        _layer("attention", _attention(4, 2, 128, 128, 0.09, size=96, softcap=10.0, v_mix=True), 512),
        _layer("attention", _attention(8, 1, 64, 64, 0.12, size=40, softcap=3.0, v_mix=False), None),
    ],
}
CONFIGS = {"S1": (S1, 16), "S2": (S2, 32), "S3": (S3, 16)}


def config(name: str) -> dict:
    return copy.deepcopy(CONFIGS[name][0])


@functools.lru_cache(maxsize=None)
def model_folder(name: str, seed: int = 3) -> str:
    from ampere_kv_engine_b200.models.registry import config_from_dict
    from ampere_kv_engine_b200.weights.random_init import write_random_model
    _, cfg = config_from_dict(config(name))
    out = tempfile.mkdtemp(prefix=f"sukalorn_{name}_")
    write_random_model(cfg, seed, out, torch.float32)
    path = os.path.join(out, "model.safetensors")
    tensors = load_file(path)
    for i, layer in enumerate(cfg.layers):
        if layer.type == "latent_attention":
            rank = layer.mixer["kv_rank"]
            tensors[f"l{i}.mix.uq"] = tensors[f"l{i}.mix.uq"] * 12.0
            tensors[f"l{i}.mix.uk"] = tensors[f"l{i}.mix.uk"] * 12.0
            down = tensors[f"l{i}.mix.dkv"].clone()
            down[rank:] *= 12.0
            tensors[f"l{i}.mix.dkv"] = down
    # bfloat16-representable values: both precisions then run on the same weights
    save_file({k: v.to(torch.bfloat16).to(torch.float32).contiguous() for k, v in tensors.items()}, path,
              metadata={"format": "pt"})
    return out


def plain_weights(folder: str) -> dict:
    return {k: v.double() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}


def plain_logits(folder: str, raw: dict, requests: dict[str, list[int]]) -> dict[str, torch.Tensor]:
    """float64 logits of every request as a whole sequence, as float32."""
    w = plain_weights(folder)
    return {rid: plain.forward(w, raw, toks).float() for rid, toks in requests.items()}
