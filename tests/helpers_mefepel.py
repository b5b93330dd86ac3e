"""Small Mefepel configurations for the tests, none with the sizes of any published model: they differ from one another
in every size, in the order of their layers' feed-forwards and in the routers' `top`."""
from __future__ import annotations

import json
import tempfile
from pathlib import Path

import torch

from tests import plain_mefepel as plain


def mixer(heads, dim, vdim, kv_rank, q_rank, scale=None):
    return dict(heads=heads, dim=dim, vdim=vdim, kv_rank=kv_rank, q_rank=q_rank, scale=scale if scale is not None else dim ** -0.5)


def dense(ff, limit):
    return dict(kind="dense", ff=ff, limit=limit)


def moe(ff, experts, top):
    return dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top))


def layer(mix, mlp):
    return dict(type="latent_attention", mixer=mix, mlp=mlp)


def config(vocab, width, max_positions, eps, layers):
    return dict(architecture="Mefepel", vocab=vocab, width=width, max_positions=max_positions, norm=dict(eps=eps), layers=layers)


# odd sizes everywhere: nothing is a multiple of 8, value heads wider than query heads, two experts per token
MEF_ODD = config(211, 52, 300, 1e-5, [
    layer(mixer(3, 10, 14, 36, 20, 0.4), moe(22, 5, 2)),
    layer(mixer(3, 10, 14, 36, 20, 0.4), None),
    layer(mixer(2, 12, 6, 44, 28, 0.25), dense(70, 0.9)),
])
# sizes the tensor-core kernels take (latent of 64), layers of different shapes, a router that takes three of six
MEF_FAST = config(384, 128, 1200, 1e-6, [
    layer(mixer(4, 16, 16, 64, 48), dense(192, 2.0)),
    layer(mixer(8, 32, 16, 64, 40, 0.2), moe(64, 6, 3)),
    layer(mixer(4, 16, 24, 64, 48), moe(48, 4, 1)),
])
# a latent of 128 under many heads (more than one tile of 16 query heads), one layer only
MEF_WIDE = config(300, 96, 700, 1e-5, [
    layer(mixer(20, 8, 8, 128, 32, 0.5), moe(40, 3, 2)),
])

CONFIGS = {"odd": MEF_ODD, "fast": MEF_FAST, "wide": MEF_WIDE}


def make_model_dir(cfg: dict, seed: int, folder=None, store_dtype=torch.float32, spread: float = 1.0):
    """config.json + model.safetensors with the tests' own random weights; returns the folder and the float32 weights."""
    from qwenforge_b200.weights import save_safetensors

    folder = Path(folder or tempfile.mkdtemp(prefix="mef_model_"))
    folder.mkdir(parents=True, exist_ok=True)
    weights = plain.random_weights(cfg, seed, spread)
    (folder / "config.json").write_text(json.dumps(cfg))
    save_safetensors(folder / "model.safetensors", {k: v.to(store_dtype) for k, v in weights.items()})
    return folder, weights
