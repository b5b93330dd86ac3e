"""Small Zebovik configurations for the tests, none with the sizes of any published model: they differ from one another in
every size and in the order of their layers."""
from __future__ import annotations

import json
import tempfile
from pathlib import Path

import torch

from tests import plain_zebovik as plain


def attention(heads, kv_heads, dim, vdim, mask, rot_dims, base=10000.0, scale=None, softcap=20.0, kv_from=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, mask=dict(size=mask), rot=dict(dims=rot_dims, base=base),
             scale=scale if scale is not None else dim ** -0.5, softcap=softcap)
    if kv_from is not None:
        m["kv_from"] = kv_from
    return "attention", m


def mlstm(heads, dim, vdim, gate_cap=10.0):
    return "mlstm", dict(heads=heads, dim=dim, vdim=vdim, gate_cap=gate_cap)


def mamba2(heads, vdim, state, groups, conv, norm_groups):
    return "mamba2", dict(heads=heads, vdim=vdim, state=state, groups=groups, conv=conv, norm_groups=norm_groups)


def layer(mix, ff):
    return dict(type=mix[0], mixer=mix[1], mlp=None if ff is None else dict(kind="dense", ff=ff))


def config(vocab, width, eps, logit_softcap, layers):
    return dict(architecture="Zebovik", vocab=vocab, width=width, norm=dict(eps=eps), logit_softcap=logit_softcap, layers=layers)


# odd sizes everywhere; values wider than keys; a reader whose blocks differ from its source's; layers without a feed-forward
ZEB_ODD = config(211, 52, 1e-5, 9.0, [
    layer(attention(4, 2, 10, 14, 37, 6, 5000.0, 0.9, 7.0), 70),
    layer(attention(4, 2, 10, 14, 23, 6, 5000.0, 1.3, 4.0, kv_from=0), None),
    layer(mlstm(3, 12, 9, 6.0), 44),
    layer(mamba2(4, 6, 10, 2, 3, 3), None),
    layer(mamba2(2, 40, 20, 1, 5, 1), 36),
])
# sizes the vector and tensor-core kernels take; a recurrent layer first, blocks of two pages
ZEB_FAST = config(384, 128, 1e-6, 30.0, [
    layer(mlstm(2, 32, 64), 192),
    layer(attention(4, 1, 64, 64, 128, 64, 100000.0, 1.5), 256),
    layer(mamba2(4, 32, 64, 1, 4, 1), None),
    layer(attention(4, 1, 64, 64, 128, 64, 100000.0, 2.5, kv_from=1), 128),
])
# what other configurations make larger than 1 or unequal: one query head per key head, one head per group, a part of the
# norm per head, blocks of one position, no rotation, keys wider than values, a convolution of two taps
ZEB_ONES = config(97, 40, 1e-6, 50.0, [
    layer(attention(3, 3, 16, 8, 1, 0, 10000.0, 2.0, 50.0), 24),
    layer(mamba2(5, 8, 12, 5, 2, 5), 60),
    layer(attention(2, 2, 8, 8, 5, 8, 300.0, 2.0, 3.0), None),
    layer(mlstm(1, 20, 28, 2.0), None),
])

# wide states: more rows than one pass of the scan's smallest form holds, a state-space layer of 144 rows under seven
# taps, values wider than keys at a size the tensor-core kernels take (keys padded with zeros), blocks of one page
ZEB_WIDE = config(150, 72, 1e-5, 25.0, [
    layer(attention(2, 2, 96, 128, 64, 48, 20000.0, 0.2, 40.0), 80),
    layer(mlstm(1, 160, 33, 5.0), None),
    layer(mamba2(4, 16, 144, 2, 7, 4), 56),
    layer(attention(2, 2, 96, 128, 100, 48, 20000.0, 0.1, 12.0, kv_from=0), None),
])

CONFIGS = {"odd": ZEB_ODD, "fast": ZEB_FAST, "ones": ZEB_ONES, "wide": ZEB_WIDE}


def make_model_dir(cfg: dict, seed: int, folder=None, store_dtype=torch.float32, weights=None):
    """config.json + model.safetensors with the tests' own random weights; returns the folder and the float32 weights."""
    from qwenforge_b200.weights import save_safetensors

    folder = Path(folder or tempfile.mkdtemp(prefix="zeb_model_"))
    folder.mkdir(parents=True, exist_ok=True)
    weights = plain.random_weights(cfg, seed) if weights is None else weights
    (folder / "config.json").write_text(json.dumps(cfg))
    save_safetensors(folder / "model.safetensors", {k: v.to(store_dtype) for k, v in weights.items()})
    return folder, weights
