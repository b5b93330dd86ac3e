"""The Mefepel design through the package's own configuration, loader, cache and step function on the CPU, with every
CUDA kernel replaced by its plain reference (the `reference_kernels` fixture), against the plain implementation of
tests/plain_mefepel.py. This checks the host side: names and shapes, the order of the parts, the one-plane latent cache,
positions of continued sequences, slot and page reuse. The kernels themselves are checked on a GPU."""
import pytest
import torch

from tests import plain_mefepel as plain
from tests.helpers import max_err, random_tokens
from tests.helpers_mefepel import CONFIGS, MEF_ODD, make_model_dir


def build(cfg, tmp_path, seed=0):
    from qwenforge_b200.engine import Model
    folder, weights = make_model_dir(cfg, seed, tmp_path)
    return Model.from_dir(folder, "float32", "cpu"), weights, folder


def test_configuration_names_every_tensor(tmp_path):
    from qwenforge_b200.config import MefepelConfig, config_from_dict
    from qwenforge_b200.engine import Model
    for cfg in CONFIGS.values():
        config = config_from_dict(cfg)
        assert isinstance(config, MefepelConfig)
        wanted = {t.name: tuple(t.shape) for t in Model.tensor_specs_of(config.model_spec())}
        assert wanted == plain.tensor_shapes(cfg)
        assert config_from_dict(config.to_dict()).model_spec() == config.model_spec()
    with pytest.raises(ValueError, match="top"):
        bad = dict(MEF_ODD, layers=[dict(MEF_ODD["layers"][0], mlp=dict(kind="moe", expert=dict(ff=8), router=dict(experts=2, top=3)))])
        config_from_dict(bad)
    with pytest.raises(ValueError, match="kind"):
        config_from_dict(dict(MEF_ODD, layers=[dict(MEF_ODD["layers"][0], mlp=dict(kind="other"))]))


def test_a_layer_without_feed_forward_may_carry_its_norms(reference_kernels, tmp_path):
    """Files that hold norm2 / norm2b for a layer without a feed-forward still load; nothing reads them."""
    import json
    from qwenforge_b200.engine import Model
    from qwenforge_b200.weights import save_safetensors
    folder, weights = make_model_dir(MEF_ODD, 3, tmp_path)
    extra = dict(weights)
    extra["l1.norm2"] = torch.ones(MEF_ODD["width"])
    extra["l1.norm2b"] = torch.ones(MEF_ODD["width"])
    save_safetensors(folder / "model.safetensors", extra)
    model = Model.from_dir(folder, "float32", "cpu")
    cache = model.new_cache(128, 2)
    tokens = random_tokens(MEF_ODD["vocab"], 9, 1)
    got = model.step(cache, [(cache.open(), tokens)], want=[list(range(9))])
    assert max_err(got, plain.forward_logits(MEF_ODD, weights, tokens)) < 2e-5


@pytest.mark.parametrize("name", list(CONFIGS))
def test_every_cut_gives_the_plain_logits(reference_kernels, name, tmp_path):
    cfg = CONFIGS[name]
    model, weights, _ = build(cfg, tmp_path)
    cache = model.new_cache(64 * 8, 3)
    seqs = [random_tokens(cfg["vocab"], n, 10 + n) for n in (70, 5, 33, 101, 64)]
    refs = [plain.forward_logits(cfg, weights, s) for s in seqs]
    for round_ in range(2):                               # the second round runs in slots and pages used before
        for begin in range(0, len(seqs), 3):
            batch = list(range(begin, min(begin + 3, len(seqs))))
            slots = {i: cache.open() for i in batch}
            heads = {i: max(1, len(seqs[i]) - 4 - i) for i in batch}
            logits = model.step(cache, [(slots[i], seqs[i][:heads[i]]) for i in batch],
                                want=[list(range(heads[i])) for i in batch])
            got = {i: [] for i in batch}
            o = 0
            for i in batch:
                got[i].append(logits[o:o + heads[i]])
                o += heads[i]
            fed = dict(heads)
            live = [i for i in batch if fed[i] < len(seqs[i])]
            while live:
                logits = model.step(cache, [(slots[i], [seqs[i][fed[i]]]) for i in live])
                for row, i in enumerate(live):
                    got[i].append(logits[row:row + 1])
                    fed[i] += 1
                for i in [i for i in live if fed[i] == len(seqs[i])]:
                    cache.close(slots.pop(i))
                live = [i for i in live if fed[i] < len(seqs[i])]
            for i in list(slots):
                cache.close(slots.pop(i))
            for i in batch:
                assert max_err(torch.cat(got[i]), refs[i]) < 5e-5, (name, round_, i)
    assert cache.slots.n_free == cache.max_seqs and all(g.pages.n_free == g.pages.n_pages for g in cache.kv_groups)


def test_the_plain_implementation_decodes_as_it_prefills():
    cfg = MEF_ODD
    weights = plain.random_weights(cfg, 5)
    tokens = random_tokens(cfg["vocab"], 40, 2)
    assert max_err(plain.decode_logits(cfg, weights, tokens, 17), plain.forward_logits(cfg, weights, tokens)) < 1e-9


def test_the_latent_cache_holds_one_plane(reference_kernels, tmp_path):
    model, _, _ = build(MEF_ODD, tmp_path)
    cache = model.new_cache(256, 2)
    ranks = sorted({g.need.head_dim for g in cache.kv_groups})
    assert ranks == [36, 44] and all(g.need.planes == 1 and g.need.kv_heads == 1 for g in cache.kv_groups)
    assert all(g.storage.shape[2] == 1 for g in cache.kv_groups)
    # what a decode step reads: rank numbers per position and layer, not heads * (dim + vdim)
    assert cache.read_bytes([100]) == 100 * (36 * 2 + 44) * 4


@pytest.mark.parametrize("order", ["none_last", "none_first", "only_none"])
def test_layers_without_a_feed_forward_at_either_end(reference_kernels, order, tmp_path):
    from tests.helpers_mefepel import config, dense, layer, mixer, moe
    with_ff = [layer(mixer(2, 6, 10, 20, 12, 0.3), moe(14, 3, 3)), layer(mixer(3, 4, 4, 12, 8, 0.5), dense(30, 1.1))]
    bare = layer(mixer(2, 8, 6, 16, 10, 0.35), None)
    layers = {"none_last": with_ff + [bare], "none_first": [bare] + with_ff, "only_none": [bare, bare]}[order]
    cfg = config(90, 28, 80, 2e-5, layers)
    model, weights, _ = build(cfg, tmp_path, seed=9)
    cache = model.new_cache(128, 2)
    tokens = random_tokens(cfg["vocab"], 30, 3)
    slot = cache.open()
    first = model.step(cache, [(slot, tokens[:19])], want=[list(range(19))])
    rest = [model.step(cache, [(slot, [t])]) for t in tokens[19:]]
    assert max_err(torch.cat([first] + rest), plain.forward_logits(cfg, weights, tokens)) < 5e-5
