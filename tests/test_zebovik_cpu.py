"""The Zebovik design through the package's own configuration, loader, cache, state and step function on the CPU, with
every CUDA kernel replaced by its plain reference (the `reference_kernels` fixture), against the plain implementation of
tests/plain_zebovik.py. This checks the host side: names and shapes, the order of the parts, padded heads, the layer that
reads another's cache, recurrent state in reused slots, pages given back as blocks of the mask pass. The kernels
themselves are checked on a GPU."""
import pytest
import torch

from tests import plain_zebovik as plain
from tests.helpers import max_err, random_tokens
from tests.helpers_zebovik import CONFIGS, ZEB_FAST, ZEB_ODD, ZEB_ONES, attention, config, layer, make_model_dir, mlstm


def build(cfg, tmp_path, seed=0):
    from qwenforge_b200.engine import Model
    folder, weights = make_model_dir(cfg, seed, tmp_path)
    return Model.from_dir(folder, "float32", "cpu"), weights, folder


def test_configuration_names_every_tensor():
    from qwenforge_b200.config import ZebovikConfig, config_from_dict
    from qwenforge_b200.engine import Model
    for cfg in CONFIGS.values():
        cfg_obj = config_from_dict(cfg)
        assert isinstance(cfg_obj, ZebovikConfig)
        wanted = {t.name: tuple(t.shape) for t in Model.tensor_specs_of(cfg_obj.model_spec())}
        assert wanted == plain.tensor_shapes(cfg)
        assert config_from_dict(cfg_obj.to_dict()).model_spec() == cfg_obj.model_spec()
    with pytest.raises(ValueError, match="kv_from"):
        config_from_dict(config(50, 16, 1e-6, 5.0, [layer(attention(2, 1, 8, 8, 16, 8, kv_from=0), None)]))
    with pytest.raises(ValueError, match="kv_from"):
        config_from_dict(config(50, 16, 1e-6, 5.0, [layer(mlstm(1, 8, 8), None), layer(attention(2, 1, 8, 8, 16, 8, kv_from=0), None)]))
    with pytest.raises(ValueError, match="dim differs"):
        config_from_dict(config(50, 16, 1e-6, 5.0, [layer(attention(2, 1, 8, 8, 16, 8), None),
                                                    layer(attention(2, 1, 4, 8, 16, 4, kv_from=0), None)]))
    with pytest.raises(ValueError, match="not supported"):
        config_from_dict(config(50, 16, 1e-6, 5.0, [dict(type="other", mixer={}, mlp=None)]))


def test_the_plain_implementation_decodes_as_it_prefills():
    for cfg in CONFIGS.values():
        weights = plain.random_weights(cfg, 5)
        tokens = random_tokens(cfg["vocab"], 90, 2)
        assert max_err(plain.decode_logits(cfg, weights, tokens, 41), plain.forward_logits(cfg, weights, tokens)) < 1e-9


def test_cache_needs_of_readers_and_recurrent_layers(reference_kernels, tmp_path):
    from qwenforge_b200.cache import KvNeed, StateNeed
    model, _, _ = build(ZEB_ODD, tmp_path)
    needs = model.cache_needs()
    # the reader's blocks differ from its source's: the source keeps every position; heads are padded to the wider size
    assert needs[0] == KvNeed(2, 14, 0, 2, 0) and needs[1] is None
    assert needs[2] == StateNeed((3 * 12 * 9 + 3 * 12 + 3,)) and needs[3] == StateNeed((4 * 10 * 6 + 2 * (24 + 40),))
    model, _, _ = build(ZEB_FAST, tmp_path / "fast")
    assert model.cache_needs()[1] == KvNeed(1, 64, 0, 2, 128)


def test_pages_leave_as_blocks_pass(reference_kernels, tmp_path):
    model, weights, _ = build(ZEB_FAST, tmp_path)
    cache = model.new_cache(64 * 8, 2)
    tokens = random_tokens(ZEB_FAST["vocab"], 300, 4)
    slot = cache.open()
    got = [model.step(cache, [(slot, tokens[:250])], want=[list(range(250))])]
    group = cache.kv_groups[0]
    assert group.pages_held(slot) == 2            # block 1 (positions 128..255) is the current one
    for t in tokens[250:]:
        got.append(model.step(cache, [(slot, [t])]))
    assert group.pages_held(slot) == 1            # positions 256..299: one page of block 2
    assert max_err(torch.cat(got), plain.forward_logits(ZEB_FAST, weights, tokens)) < 5e-5
    cache.close(slot)
    assert group.pages.n_free == group.pages.n_pages


@pytest.mark.parametrize("name", list(CONFIGS))
def test_every_cut_gives_the_plain_logits(reference_kernels, name, tmp_path):
    cfg = CONFIGS[name]
    model, weights, _ = build(cfg, tmp_path)
    cache = model.new_cache(64 * 8, 3)
    seqs = [random_tokens(cfg["vocab"], n, 10 + n) for n in (70, 5, 33, 101, 64)]
    refs = [plain.forward_logits(cfg, weights, s) for s in seqs]
    for round_ in range(2):                               # the second round runs in slots, pages and state rows used before
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


def test_portions_down_to_two_tokens(reference_kernels, tmp_path):
    model, weights, _ = build(ZEB_ONES, tmp_path, seed=3)
    cache = model.new_cache(256, 2)
    tokens = random_tokens(ZEB_ONES["vocab"], 61, 8)
    slot, at, got = cache.open(), 0, []
    for size in (2, 7, 2, 1, 30, 3, 16):
        got.append(model.step(cache, [(slot, tokens[at:at + size])], want=[list(range(size))]))
        at += size
    assert at == len(tokens)
    assert max_err(torch.cat(got), plain.forward_logits(ZEB_ONES, weights, tokens)) < 5e-5


def test_presets_are_valid_configurations():
    from qwenforge_b200.config import preset_config, preset_names
    from qwenforge_b200.engine import Model
    names = [n for n in preset_names() if n.startswith("zebovik")]
    assert {"zebovik-tiny", "zebovik-0.5b", "zebovik-3b"} <= set(names)
    for name in names:
        spec = preset_config(name).model_spec()
        assert len(Model.tensor_specs_of(spec)) > 0 and any(e.cache_from is not None for e in spec.schedule)
