"""The Zebovik design on a GPU: each new kernel and kernel option against its plain reference, the model against the plain
implementation (tests/plain_zebovik.py) whole, decoded, cut into portions, in unequal batches, in slots, pages and state
rows used before, and through the engine's own entry point with greedy generation. The tests make their own small
configurations (tests/helpers_zebovik.py) and weights; where random weights would hide a fault (a key far back, the edge
of a block of the mask, the sink), weights or inputs are made so that it shows."""
import copy
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from tests import kernel_refs as refs
from tests import plain_zebovik as plain
from tests.helpers import max_err, random_tokens
from tests.helpers_zebovik import CONFIGS, ZEB_FAST, ZEB_ODD, ZEB_ONES, attention, config, layer, make_model_dir, mamba2, mlstm

pytestmark = pytest.mark.gpu
DEV = "cuda"
BOTH = [torch.float32, torch.bfloat16]


def close(got, want, dtype, what="", f32=3e-5, bf16=3e-2):
    got, want = got.double().cpu(), want.double().cpu()
    scale = float(want.abs().max()) + 1e-9
    bound = (f32 if dtype == torch.float32 else bf16) * scale
    err = float((got - want).abs().max())
    assert err <= bound, f"{what}: max |diff| {err:.3e} exceeds {bound:.3e}"


def logits_close(got, want, dtype, what=""):
    """The difference with its mean taken off, root mean square over the vocabulary, against the spread of the logits."""
    got, want = got.double().cpu(), want.double().cpu()
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    err = d.square().mean(-1).sqrt() / want.std(-1)
    if dtype == torch.float32:
        assert float(err.max()) <= 1e-4, f"{what}: worst row {float(err.max()):.3e} exceeds 1e-4"
    else:   # the typical row within rounding, and no row lost: a wrong key, a mask one position off or a lost state moves
        # every later row by about its whole spread, which the median sees; a single row whose sharp softmax magnifies
        # the rounding of its scores may stand out
        far = float((err > 0.4).double().mean())
        assert float(err.median()) <= 0.05 and far <= 0.02 and float(err.max()) <= 1.0, \
            f"{what}: median {float(err.median()):.3e}, {far:.1%} of the rows over 0.4, worst {float(err.max()):.3e}"


def rand(g, *shape, dtype=torch.float32, spread=1.0):
    return (spread * torch.randn(*shape, generator=g)).to(dtype).to(DEV)


def ints(values):
    return torch.tensor(values, dtype=torch.int32, device=DEV)


class Batch:
    """The integers of a step of sequences with the given slots and (start, length) spans."""

    def __init__(self, slots, spans):
        self.slots, self.n_seqs = ints(slots), len(slots)
        cu, seq, pos = [0], [], []
        for s, (start, length) in enumerate(spans):
            cu.append(cu[-1] + length)
            seq += [s] * length
            pos += list(range(start, start + length))
        self.cu_q, self.tok_seq, self.tok_pos, self.n_tokens = ints(cu), ints(seq), ints(pos), cu[-1]
        self.max_q_len = max(length for _, length in spans)
        self.max_kv_len = max(start + length for start, length in spans)


# ------------------------------------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("kind", ["relu2", "gelu_tanh", "silu", "relu"])
@pytest.mark.parametrize("width", [45, 384])
def test_bias_act(dtype, kind, width):
    from qwenforge_b200 import ops
    g = torch.Generator().manual_seed(width)
    x, b = rand(g, 9, width, dtype=dtype, spread=2.0), rand(g, width, dtype=dtype)
    for bias in (b, None):
        out, want = torch.empty_like(x), torch.empty_like(x)
        ops.bias_act(x, bias, kind, out)
        refs.bias_act(x, bias, kind, want)
        close(out, want, dtype, kind, bf16=1e-2)


def test_softcap_in_place():
    from qwenforge_b200 import ops
    x = torch.linspace(-90, 90, 1001, device=DEV).view(7, 143).contiguous()
    want = x.clone()
    refs.softcap_(want, 15.0)
    ops.softcap_(x, 15.0)
    assert max_err(x, want) < 1e-5 and float(x.abs().max()) < 15.0


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("heads,kv_heads,dim,norm_dim,rot", [(4, 2, 14, 10, 6), (3, 3, 64, 64, 64), (2, 1, 40, 40, 0), (5, 1, 96, 96, 48)])
def test_rotation_unit_norm_and_cache_write(dtype, heads, kv_heads, dim, norm_dim, rot):
    """Bias, partial rotation, the unit norm over a head's own components (the rest are padding and stay zero), queries out
    and keys and values into the pages; also rows that hold queries only."""
    from qwenforge_b200 import ops
    from qwenforge_b200.cache import KvNeed, SequenceCache
    g = torch.Generator().manual_seed(dim)
    batch = Batch([1, -1, 0], [(60, 9), (0, 3), (5, 70)])
    caches = [SequenceCache([KvNeed(kv_heads, dim)], 512, 3, 512, dtype, DEV) for _ in range(2)]
    for cache in caches:
        for slot, total in ((cache.open(), 75), (cache.open(), 69)):
            cache.reserve([(slot, total)])
        cache.flush()
    inv_freq = (1.0 / (300.0 ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))).to(DEV) if rot else None
    for has_kv in (True, False):
        width = (heads + (2 * kv_heads if has_kv else 0)) * dim
        qkv, bias = rand(g, batch.n_tokens, width, dtype=dtype), rand(g, width, dtype=dtype)
        view = qkv.view(batch.n_tokens, -1, dim)
        view[:, :, norm_dim:] = 0          # padded heads carry zeros beyond their own size
        bias.view(-1, dim)[:, norm_dim:] = 0
        outs = []
        for fn, cache in ((ops.rope_cache_write, caches[0]), (refs.rope_cache_write, caches[1])):
            site = cache.site(0)
            q = torch.empty(batch.n_tokens, heads * dim, dtype=dtype, device=DEV)
            err = torch.zeros(1, dtype=torch.int32, device=DEV)
            args = ops.KvSiteArgs(site.storage, site.table, kv_heads, dim) if fn is ops.rope_cache_write else site
            fn(qkv, batch.tok_seq, batch.tok_pos, batch.slots, inv_freq, rot, heads, q, args, has_kv, err, bias=bias,
               unit_norm_eps=1e-5, norm_dim=norm_dim, has_kv=has_kv)
            assert int(err) == 0
            outs.append(q)
        close(outs[0], outs[1], dtype, "queries", bf16=1e-2)
        close(caches[0].site(0).storage, caches[1].site(0).storage, dtype, "pages", bf16=1e-2)
    assert float(caches[0].site(0).storage.abs().max()) > 0


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("heads,kv_heads,dim,chunk,cap", [(4, 2, 14, 37, 5.0), (4, 1, 64, 128, 20.0), (3, 3, 24, 1, 0.0), (2, 2, 96, 190, 2.0)])
def test_attention_in_blocks_with_capped_scores_and_a_unit_sink(dtype, heads, kv_heads, dim, chunk, cap):
    """Prompts, continuations across a block's edge and single tokens over more than one chunk of keys, each against the
    reference; scores are wide enough that the cap bends most of them."""
    from qwenforge_b200 import ops
    from qwenforge_b200.cache import KvNeed, SequenceCache
    g = torch.Generator().manual_seed(chunk)
    cache = SequenceCache([KvNeed(kv_heads, dim)], 2048, 4, 1024, dtype, DEV)
    slots = [cache.open() for _ in range(3)]
    cache.reserve([(slots[0], 700), (slots[1], 420), (slots[2], 420)])
    cache.flush()
    site = cache.site(0)
    site.storage.copy_(rand(g, *site.storage.shape, dtype=dtype))
    args = ops.KvSiteArgs(site.storage, site.table, kv_heads, dim)
    sinks = torch.zeros(heads, dtype=torch.float32, device=DEV)
    scratch = ops.DecodeScratch(DEV)
    spans = [[(0, 700), (0, 300), (0, 90)], [(chunk * 2 - 3 if chunk > 3 else 5, 9), (290, 10), (0, 1)],
             [(699, 1), (299, 1), (chunk, 1)], [(2 * chunk - 1, 1), (2 * chunk, 1), (89, 1)], [(300, 1), (419, 1), (chunk - 1, 1)]]
    for span in spans:
        batch = Batch(slots, span)
        q = rand(g, batch.n_tokens, heads * dim, dtype=dtype, spread=1.5)
        out, want = torch.empty_like(q), torch.empty_like(q)
        err = torch.zeros(1, dtype=torch.int32, device=DEV)
        ops.attention_generic(q, out, batch.cu_q, batch.tok_pos, batch.slots, args, heads, 3, batch.max_q_len, 0.7, 0, err,
                              scratch=scratch, max_kv_len=batch.max_kv_len, sinks=sinks, chunk=chunk, softcap=cap)
        refs.attention_generic(q, want, batch.cu_q, batch.tok_pos, batch.slots, site, heads, 3, batch.max_q_len, 0.7, 0, err,
                               sinks=sinks, chunk=chunk, softcap=cap)
        assert int(err) == 0
        close(out, want, dtype, f"spans {span}", f32=2e-5, bf16=2e-2)


@pytest.mark.parametrize("heads,kv_heads,dim,chunk,cap", [(4, 1, 64, 128, 20.0), (6, 3, 96, 190, 12.0), (2, 2, 32, 70, 0.0), (6, 2, 128, 64, 4.0)])
def test_tensor_core_attention_takes_the_block_mask_the_cap_and_the_sink(heads, kv_heads, dim, chunk, cap):
    """The bfloat16 kernels of prompts and of single tokens with the same options, against the reference: prompts,
    continuations across a block's edge, single tokens just inside and just outside a block, long and short together."""
    from qwenforge_b200 import ops
    from qwenforge_b200.cache import KvNeed, SequenceCache
    g = torch.Generator().manual_seed(chunk)
    dtype = torch.bfloat16
    cache = SequenceCache([KvNeed(kv_heads, dim)], 4096, 4, 2048, dtype, DEV)
    slots = [cache.open() for _ in range(3)]
    cache.reserve([(slots[0], 1500), (slots[1], 420), (slots[2], 420)])
    cache.flush()
    site = cache.site(0)
    site.storage.copy_(rand(g, *site.storage.shape, dtype=dtype))
    args = ops.KvSiteArgs(site.storage, site.table, kv_heads, dim)
    sinks = torch.zeros(heads, dtype=torch.float32, device=DEV)
    scratch = ops.DecodeScratch(DEV)
    spans = [[(0, 1100), (0, 300), (0, 90)], [(chunk * 2 - 3, 9), (290, 70), (0, 2)],
             [(1499, 1), (299, 1), (chunk, 1)], [(2 * chunk - 1, 1), (2 * chunk, 1), (89, 1)], [(5 * chunk + 1, 1), (419, 1), (chunk - 1, 1)]]
    for span in spans:
        batch = Batch(slots, span)
        q = rand(g, batch.n_tokens, heads * dim, dtype=dtype, spread=1.5)
        out, want = torch.empty_like(q), torch.empty_like(q)
        err = torch.zeros(1, dtype=torch.int32, device=DEV)
        if batch.max_q_len == 1:
            ops.attention_decode(q, out, batch.cu_q, batch.tok_pos, batch.slots, args, heads, 3, 0.3, 0, 4, scratch, err,
                                 sinks=sinks, chunk=chunk, softcap=cap)
        else:
            ops.attention_prefill(q, out, batch.cu_q, batch.tok_pos, batch.slots, args, heads, 3, batch.max_q_len, 0.3, 0, err,
                                  max_kv_len=batch.max_kv_len, sinks=sinks, chunk=chunk, softcap=cap)
        refs.attention_generic(q, want, batch.cu_q, batch.tok_pos, batch.slots, site, heads, 3, batch.max_q_len, 0.3, 0, err,
                               sinks=sinks, chunk=chunk, softcap=cap)
        assert int(err) == 0
        close(out, want, dtype, f"spans {span}", bf16=2e-2)


def test_stabilized_gates_carry_their_maximum():
    from qwenforge_b200 import ops
    g = torch.Generator().manual_seed(3)
    heads = 5
    bias = rand(g, 2 * heads)
    bias[heads:] += 2.0
    states = [torch.zeros(4, 40, device=DEV) for _ in range(2)]
    for spans in ([(0, 70), (0, 1), (0, 33)], [(70, 1), (1, 45), (33, 2)]):
        batch = Batch([2, -1, 0], spans)
        pre = rand(g, batch.n_tokens, 2 * heads + 3, spread=4.0)[:, :2 * heads]   # strided rows
        outs = []
        for fn, state in ((ops.stabilized_gates, states[0]), (refs.stabilized_gates, states[1])):
            trio = [torch.empty(batch.n_tokens, heads, device=DEV) for _ in range(3)]
            fn(pre, bias, 6.0, batch.cu_q, batch.slots, state, 7, heads, *trio)
            outs.append(trio)
        for got, want in zip(*outs):
            assert max_err(got, want) < 1e-5 * (1 + float(want.abs().max()))
        assert max_err(states[0], states[1]) < 1e-5 and float(states[0][1].abs().max()) == 0.0


def test_decay_gates():
    from qwenforge_b200 import ops
    g = torch.Generator().manual_seed(4)
    pre = rand(g, 19, 9, spread=30.0)[:, :6]
    dt_bias, rate_log = rand(g, 6), rand(g, 6)
    got, want = [torch.empty(19, 6, device=DEV) for _ in range(2)], [torch.empty(19, 6, device=DEV) for _ in range(2)]
    ops.decay_gates(pre, dt_bias, rate_log, *got)
    refs.decay_gates(pre, dt_bias, rate_log, *want)
    assert max_err(got[0], want[0]) < 1e-6 and max_err(got[1], want[1]) < 1e-4 and bool(torch.isfinite(got[1]).all())


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("heads,groups,dim,vdim,with_n", [(3, 3, 12, 9, True), (4, 2, 10, 6, False), (2, 1, 64, 70, False),
                                                         (1, 1, 20, 32, True), (2, 2, 130, 40, True)])
def test_outer_state_scan_carries_its_state(dtype, heads, groups, dim, vdim, with_n):
    from qwenforge_b200 import ops
    g = torch.Generator().manual_seed(dim)
    s_off, n_off = 3, 3 + heads * dim * vdim + 5
    floats = n_off + heads * dim + 2
    states = [torch.zeros(4, floats, device=DEV) for _ in range(2)]
    for spans in ([(0, 40), (0, 1), (0, 17)], [(40, 1), (1, 1), (17, 1)], [(41, 23), (2, 50), (18, 2)]):
        batch = Batch([3, -1, 1], spans)
        n = batch.n_tokens
        wide = rand(g, n, 2 * groups * dim + heads * vdim + 1, dtype=dtype)
        q, k, v = wide[:, :groups * dim], wide[:, groups * dim:2 * groups * dim], wide[:, 2 * groups * dim:-1]
        decay, take = torch.rand(n, heads, generator=g).to(DEV), torch.rand(n, heads, generator=g).to(DEV) * 2
        outs = []
        for fn, state in ((ops.outer_state_scan, states[0]), (refs.outer_state_scan, states[1])):
            y = torch.empty(n, heads * vdim, device=DEV)
            nq = torch.empty(n, heads, device=DEV) if with_n else None
            fn(q, k, v, decay, take, batch.cu_q, batch.slots, state, s_off, n_off if with_n else -1, heads, groups, dim, vdim,
               0.3, y, nq)
            outs.append((y, nq))
        close(outs[0][0], outs[1][0], torch.float32, "y")
        if with_n:
            close(outs[0][1], outs[1][1], torch.float32, "n . q")
        close(states[0], states[1], torch.float32, "state")
        assert float(states[0][0].abs().max()) == 0.0 and float(states[0][:, :s_off].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("heads,vdim,parts,gate,first,extras", [(3, 9, 3, "sigmoid", False, "denominator"), (4, 6, 3, "silu", True, "skip"),
                                                                (2, 200, 1, "silu", True, "skip"), (6, 64, 6, "sigmoid", False, "denominator")])
def test_gated_group_norm(dtype, heads, vdim, parts, gate, first, extras):
    from qwenforge_b200 import ops
    g = torch.Generator().manual_seed(vdim)
    n, c = 11, heads * vdim
    y, wide = rand(g, n, c, spread=3.0), rand(g, n, 2 * c + 8, dtype=dtype)
    gate_in, skip_x, weight = wide[:, :c], wide[:, c + 8:], (1 + 0.2 * torch.randn(c, generator=g)).to(dtype).to(DEV)
    more = {}
    if extras == "denominator":
        more = dict(nq=rand(g, n, heads, spread=2.0), floor=torch.rand(n, heads, generator=g).to(DEV) * 3, floor_add=1e-6)
    else:
        more = dict(skip=rand(g, heads), skip_x=skip_x)
    out, want = torch.empty(n, c, dtype=dtype, device=DEV), torch.empty(n, c, dtype=dtype, device=DEV)
    ops.gated_group_norm(y, gate_in, weight, 1e-5, out, parts, heads, gate, first, **more)
    refs.gated_group_norm(y, gate_in, weight, 1e-5, want, parts, heads, gate, first, **more)
    close(out, want, dtype, bf16=1e-2)


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("taps,channels", [(4, 70), (2, 33), (1, 20), (7, 512)])
def test_causal_conv_keeps_its_last_inputs(dtype, taps, channels):
    """Steps shorter than the taps, so that the kept inputs are partly old and partly new."""
    from qwenforge_b200 import ops
    g = torch.Generator().manual_seed(taps)
    weight, bias = rand(g, channels, taps, spread=0.5), rand(g, channels)
    floats = 5 + (taps - 1) * channels
    states = [torch.zeros(3, floats, device=DEV) for _ in range(2)]
    for spans in ([(0, 9), (0, 2), (0, 1)], [(9, 1), (2, 1), (1, 1)], [(10, 2), (3, 30), (2, 1)], [(12, 1), (33, 1), (3, 1)]):
        batch = Batch([2, -1, 0], spans)
        x = rand(g, batch.n_tokens, channels + 3, dtype=dtype)[:, 3:]
        out, want = (torch.empty(batch.n_tokens, channels, dtype=dtype, device=DEV) for _ in range(2))
        ops.causal_conv_silu(x, weight, bias, batch.cu_q, batch.tok_seq, batch.slots, states[0], 5, out)
        refs.causal_conv_silu(x, weight, bias, batch.cu_q, batch.tok_seq, batch.slots, states[1], 5, want)
        close(out, want, dtype, f"spans {spans}", bf16=1e-2)
        assert max_err(states[0], states[1]) < 1e-6 and float(states[0][1].abs().max()) == 0.0


# ------------------------------------------------------------------------------------------------ the model
def build(cfg, folder, dtype, seed=0, weights=None):
    """The model on the GPU and the weights it holds: in bfloat16 the plain implementation gets the rounded weights, so
    that the comparison sees the arithmetic and not the rounding of the file."""
    from qwenforge_b200.engine import Model
    weights = plain.random_weights(cfg, seed) if weights is None else weights
    if dtype == torch.bfloat16:
        weights = {k: v.to(torch.bfloat16).float() for k, v in weights.items()}
    folder, weights = make_model_dir(cfg, seed, folder, weights=weights)
    return Model.from_dir(folder, dtype, DEV), weights, folder


def run(model, cache, tokens, cuts):
    """One sequence fed in portions of the given sizes (the rest one by one); the logits of every position."""
    slot, at, got = cache.open(), 0, []
    for size in list(cuts) + [1] * (len(tokens) - sum(cuts)):
        got.append(model.step(cache, [(slot, tokens[at:at + size])], want=[list(range(size))]))
        at += size
    cache.close(slot)
    model.raise_on_kernel_error()
    return torch.cat(got)


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompts_decoding_and_portions_agree_with_the_plain_implementation(dtype, name, tmp_path):
    cfg = CONFIGS[name]
    model, weights, _ = build(cfg, tmp_path, dtype)
    cache = model.new_cache(64 * 12, 3)
    tokens = random_tokens(cfg["vocab"], 300, 7)
    want = plain.forward_logits(cfg, weights, tokens)
    for cuts in ([300], [260], [2, 61, 2, 130, 65, 3, 2], [129, 128]):
        logits_close(run(model, cache, tokens, cuts), want, dtype, f"{name} cuts {cuts[:3]}")
    assert all(g.pages.n_free == g.pages.n_pages for g in cache.kv_groups)


def test_the_residual_stream_after_every_layer(tmp_path):
    model, weights, _ = build(ZEB_ODD, tmp_path, torch.float32)
    cache = model.new_cache(256, 2)
    tokens = random_tokens(ZEB_ODD["vocab"], 50, 1)
    seen = {}
    model.observer = lambda i, hidden, delta: seen.__setitem__(i, (hidden if delta is None else hidden + delta.float()).clone())
    run(model, cache, tokens, [50])
    model.observer = None
    seq = plain.Sequence(ZEB_ODD, weights)
    seq.feed(tokens)
    for i in range(len(ZEB_ODD["layers"])):
        assert max_err(seen[i + 1], seq.streams[i]) < 2e-4 * (1 + float(seq.streams[i].abs().max())), f"after layer {i}"


@pytest.mark.parametrize("dtype", BOTH)
def test_unequal_batches_in_slots_used_before(dtype, tmp_path):
    """Requests of unequal lengths start together, are decoded together and end one by one; the second round runs in slots,
    pages and state rows that the first has used. Each request's logits equal those of the plain implementation alone."""
    cfg = ZEB_ODD
    model, weights, _ = build(cfg, tmp_path, dtype, seed=2)
    cache = model.new_cache(64 * 10, 3)
    seqs = [random_tokens(cfg["vocab"], n, 30 + n) for n in (150, 3, 66, 1, 91)]
    want = [plain.forward_logits(cfg, weights, s) for s in seqs]
    for round_ in range(2):
        for batch in ([0, 1, 2], [3, 4]):
            slots = {i: cache.open() for i in batch}
            heads = {i: max(1, len(seqs[i]) - 20) for i in batch}
            logits = model.step(cache, [(slots[i], seqs[i][:heads[i]]) for i in batch], want=[list(range(heads[i])) for i in batch])
            got, o = {i: [] for i in batch}, 0
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
                live = [i for i in live if fed[i] < len(seqs[i])]
            for i in batch:
                cache.close(slots[i])
                logits_close(torch.cat(got[i]), want[i], dtype, f"round {round_} request {i}")
    model.raise_on_kernel_error()


def peaked(cfg, weights, seed):
    """Weights under which one score stands out: attention's q and k projections and biases grown so that scores reach the
    cap's bend and single keys dominate, the sink then matters only where every score is low."""
    w = {k: v.clone() for k, v in weights.items()}
    for i, lay in enumerate(cfg["layers"]):
        if lay["type"] == "attention":
            w[f"l{i}.mix.q"] *= 4.0
            if f"l{i}.mix.k" in w:
                w[f"l{i}.mix.k"] *= 4.0
    return w


@pytest.mark.parametrize("dtype", BOTH)
def test_keys_far_back_and_at_the_edges_of_blocks_and_pages(dtype, tmp_path):
    """Blocks of 150 positions over pages of 64: a prompt that ends just inside and just outside a block, decoding across the
    edge, with sharpened scores, against the plain implementation; then the same model with the masks' blocks made one
    position longer must differ at the edge (the test sees a block that is one token off)."""
    cfg = config(120, 48, 1e-6, 20.0, [
        layer(attention(4, 2, 16, 16, 150, 8, 40000.0, 1.0, 25.0), 64),
        layer(attention(4, 2, 16, 16, 150, 8, 40000.0, 1.0, 25.0, kv_from=0), None),
        layer(mlstm(2, 8, 12), 32)])
    weights = peaked(cfg, plain.random_weights(cfg, 11), 11)
    model, _, _ = build(cfg, tmp_path, dtype, weights=weights)
    cache = model.new_cache(64 * 16, 2)
    tokens = random_tokens(cfg["vocab"], 460, 5)
    want = plain.forward_logits(cfg, weights, tokens)
    for cuts in ([460], [149], [150, 1, 1, 140, 9], [298]):
        logits_close(run(model, cache, tokens, cuts), want, dtype, f"cuts {cuts}")
    off = copy.deepcopy(cfg)
    for lay in off["layers"][:2]:
        lay["mixer"]["mask"]["size"] = 151
    other = plain.forward_logits(off, weights, tokens)
    d = (other - want).abs().max(-1).values
    assert float(d[:150].max()) < 1e-9 and float(d[150]) > 1e-3      # position 150 is where the two masks part


@pytest.mark.parametrize("dtype", BOTH)
def test_long_decoding_keeps_the_recurrent_state_exact(dtype, tmp_path):
    cfg = config(90, 32, 1e-6, 12.0, [layer(mlstm(2, 16, 16, 4.0), 48), layer(mamba2(4, 8, 16, 2, 4, 2), None),
                                      layer(attention(2, 1, 16, 16, 64, 16), 40)])
    model, weights, _ = build(cfg, tmp_path, dtype, seed=4)
    cache = model.new_cache(64 * 12, 2)
    tokens = random_tokens(cfg["vocab"], 420, 9)
    logits_close(run(model, cache, tokens, [3]), plain.forward_logits(cfg, weights, tokens), dtype)


def test_greedy_generation_through_the_engine(tmp_path):
    """StudentEngine.generate_ids (the scheduler's batches, CUDA-graph decoding with padding rows, prompt graphs) against
    greedy decoding of the plain implementation, in float32 where ties are the only way to differ."""
    from qwenforge_b200.engine import StudentEngine
    for name, cfg in (("odd", ZEB_ODD), ("ones", ZEB_ONES)):
        folder, weights = make_model_dir(cfg, 6, tmp_path / name)
        prompts = [random_tokens(cfg["vocab"], n, n) for n in (5, 70, 1, 33, 12)]
        want = [plain.greedy_generate(cfg, weights, p, 12) for p in prompts]
        for graphs in (True, False):
            engine = StudentEngine(str(folder), device=DEV, dtype="float32", cuda_graphs=graphs)
            got = engine.generate_ids(prompts, max_new_tokens=12, batch_size=3, ignore_eos=True)
            assert got == want, (name, graphs)
    engine = StudentEngine(str(folder), device=DEV, dtype="bfloat16")
    assert all(len(t) == 12 for t in engine.generate_ids(prompts, max_new_tokens=12, batch_size=5, ignore_eos=True))


def test_trace_replay_as_a_subprocess(tmp_path):
    import json
    import numpy as np
    cfg = ZEB_ODD
    folder, weights = make_model_dir(cfg, 8, tmp_path / "m", store_dtype=torch.bfloat16)
    weights = {k: v.to(torch.bfloat16).float() for k, v in weights.items()}
    a, b = random_tokens(cfg["vocab"], 80, 1), random_tokens(cfg["vocab"], 9, 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:70], "want": [0, 69]}, {"id": "b", "tokens": b[:8], "want": [7]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[70:71], "want": [0]}, {"id": "b", "tokens": b[8:], "want": [0]}], "end": ["b"]}]
    steps += [{"step": 2 + i, "entries": [{"id": "a", "tokens": [a[71 + i]], "want": [0]}], "end": ["a"] if i == 8 else []} for i in range(9)]
    root = Path(__file__).resolve().parent.parent
    out = tmp_path / "out"
    done = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(out),
                           "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
                          timeout=900)
    assert done.returncode == 0, done.stderr[-2000:]
    assert [l for l in done.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(11)]
    wa, wb = plain.forward_logits(cfg, weights, a), plain.forward_logits(cfg, weights, b)
    first = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(3, cfg["vocab"]))
    logits_close(first, torch.stack((wa[0], wa[69], wb[7])), torch.float32)
    second = torch.from_numpy(np.fromfile(out / "1.f32", dtype="<f4").reshape(2, cfg["vocab"]))
    logits_close(second, torch.stack((wa[70], wb[8])), torch.float32)
    last = torch.from_numpy(np.fromfile(out / "10.f32", dtype="<f4").reshape(1, cfg["vocab"]))
    logits_close(last, wa[79:80], torch.float32)
