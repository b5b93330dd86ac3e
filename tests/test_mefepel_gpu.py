"""The Mefepel design on a GPU: each new kernel against its plain reference, the model against the plain implementation
(tests/plain_mefepel.py) whole, decoded, cut into portions, in unequal batches, in slots and pages used before, and
through the engine's own entry point with greedy generation. The tests make their own small configurations
(tests/helpers_mefepel.py) and weights; where random weights would hide a fault, inputs are made so that it shows."""
import math

import pytest
import torch

from tests import kernel_refs as refs
from tests import plain_mefepel as plain
from tests.helpers import max_err, random_tokens
from tests.helpers_mefepel import CONFIGS, MEF_FAST, MEF_ODD, MEF_WIDE, config, dense, layer, make_model_dir, mixer, moe

pytestmark = pytest.mark.gpu
DEV = "cuda"


def close(got, want, dtype, what=""):
    """float32: rounding of sums only. bfloat16: 8 bits of mantissa in every activation."""
    got, want = got.double().cpu(), want.double().cpu()
    scale = float(want.abs().max()) + 1e-9
    bound = (3e-5 if dtype == torch.float32 else 3e-2) * scale
    err = float((got - want).abs().max())
    assert err <= bound, f"{what}: max |diff| {err:.3e} exceeds {bound:.3e}"


def logits_close(got, want, dtype, what="", margins=None):
    """Like the design's own measure: the difference with its mean taken off, root mean square over the vocabulary,
    against the spread of the logits. `margins` (plain.router_margins): in bfloat16 a token whose router has two
    candidates closer than the rounding of its input may rightly go to the other expert, which moves its logits by far
    more than rounding; such rows are left out there (float32 checks every row)."""
    got, want = got.double().cpu(), want.double().cpu()
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    err = d.square().mean(-1).sqrt() / want.std(-1)
    if dtype == torch.float32:
        assert float(err.max()) <= 1e-4, f"{what}: worst row {float(err.max()):.3e} exceeds 1e-4"
        return
    # (A row routed otherwise also moves the few later rows whose attention hangs on it, in the layers above: so even among
    # the clearly routed rows a few in a hundred may be far off, while the typical row is well within rounding.)
    assert bool(torch.isfinite(err).all())
    if err.numel() < 30:     # too few rows for a statement about most of them
        assert float(err.median()) <= 0.05, f"{what}: median {float(err.median()):.3e}"
        return
    clear = err if margins is None else err[margins > 0.03]
    assert clear.numel() >= 0.6 * err.numel()
    far_off = float((clear > 0.15).double().mean())
    limit = 0.0 if margins is None or not bool(torch.isfinite(margins).any()) else 0.03
    assert far_off <= limit and float(clear.median()) <= 0.035, \
        f"{what}: {far_off:.1%} of the clearly routed rows over 0.15 (worst {float(clear.max()):.3e}), median {float(clear.median()):.3e}"


# ------------------------------------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed_positions(dtype):
    from qwenforge_b200 import ops
    g = torch.Generator().manual_seed(1)
    table, pos = torch.randn(50, 37, generator=g).to(dtype).to(DEV), torch.randn(90, 37, generator=g).to(dtype).to(DEV)
    ids = torch.randint(0, 50, (23,), generator=g).int().to(DEV)
    places = torch.randint(0, 90, (23,), generator=g).int().to(DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.empty(23, 37, dtype=torch.float32, device=DEV)
    ops.embed_positions(ids, places, table, pos, out, err)
    want = torch.empty_like(out)
    refs.embed_positions(ids, places, table, pos, want, err)
    assert max_err(out, want) < 1e-6 and int(err) == 0
    places[3] = 90
    ops.embed_positions(ids, places, table, pos, out, err)
    assert int(err) == ops.ERR_POSITION_RANGE


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [52, 328, 1500, 5000])
def test_sandwich_norm(dtype, width):
    from qwenforge_b200 import ops
    g = torch.Generator().manual_seed(width)
    hidden = torch.randn(7, width, generator=g).to(DEV)
    y = (3 * torch.randn(7, width, generator=g)).to(dtype).to(DEV)
    w1, w2 = (1 + 0.2 * torch.randn(width, generator=g)).to(dtype).to(DEV), (1 + 0.2 * torch.randn(width, generator=g)).to(dtype).to(DEV)
    want_h, want_out = hidden.clone(), torch.empty(7, width, dtype=dtype, device=DEV)
    refs.sandwich_norm(want_h, y, w1, 1e-5, w2, 2e-5, want_out)
    out = torch.empty_like(want_out)
    ops.sandwich_norm(hidden, y, w1, 1e-5, w2, 2e-5, out)
    assert max_err(hidden, want_h) < 2e-5
    close(out, want_out, dtype, "normed stream")
    only_add = want_h.clone()
    refs.sandwich_norm(only_add, y, w1, 1e-5)
    ops.sandwich_norm(hidden, y, w1, 1e-5)
    assert max_err(hidden, only_add) < 2e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("weighted", [False, True])
@pytest.mark.parametrize("top,width", [(3, 200), (2, 1100), (6, 72), (1, 2500)])
def test_sandwich_norm_sums_a_tokens_rows_on_the_way_in(dtype, weighted, top, width):
    from qwenforge_b200 import ops
    g = torch.Generator().manual_seed(5)
    tokens = 9
    hidden = torch.randn(tokens, width, generator=g).to(DEV)
    rows = torch.randn(tokens * top, width, generator=g).to(dtype).to(DEV)
    dest = torch.randperm(tokens * top, generator=g).int().to(DEV)
    row_weight = torch.rand(tokens * top, generator=g).to(DEV) if weighted else None
    w1, w2 = (1 + 0.2 * torch.randn(width, generator=g)).to(dtype).to(DEV), (1 + 0.2 * torch.randn(width, generator=g)).to(dtype).to(DEV)
    want_h, want_out = hidden.clone(), torch.empty(tokens, width, dtype=dtype, device=DEV)
    refs.sandwich_norm(want_h, rows, w1, 1e-5, w2, 1e-5, want_out, dest=dest, top=top, row_weight=row_weight)
    out = torch.empty_like(want_out)
    ops.sandwich_norm(hidden, rows, w1, 1e-5, w2, 1e-5, out, dest=dest, top=top, row_weight=row_weight)
    assert max_err(hidden, want_h) < 2e-5
    close(out, want_out, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_clamped_glu_clamps_both_halves(dtype):
    from qwenforge_b200 import ops
    g = torch.Generator().manual_seed(2)
    gate_up = (4 * torch.randn(9, 2 * 45, generator=g)).to(dtype).to(DEV)   # many values beyond the limit on both sides
    out, want = torch.empty(9, 45, dtype=dtype, device=DEV), torch.empty(9, 45, dtype=dtype, device=DEV)
    ops.clamped_glu(gate_up, 1.25, 1.702, out)
    refs.clamped_glu(gate_up, 1.25, 1.702, want)
    close(out, want, dtype)
    gate = gate_up[:, :45].float()
    assert bool((gate > 1.25).any()) and bool((gate < -1.25).any())   # the gate is clamped from above only


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(3, 10, 36, 5), (4, 16, 64, 70), (20, 8, 128, 200), (2, 24, 50, 33), (4, 16, 64, 700), (3, 40, 72, 513)])
def test_head_linear(dtype, shape):
    from qwenforge_b200 import ops
    heads, k, n, rows = shape
    g = torch.Generator().manual_seed(sum(shape))
    x = torch.randn(rows, heads * k, generator=g).to(dtype).to(DEV)
    w = torch.randn(heads, n, k, generator=g).to(dtype).to(DEV)
    out, want = torch.empty(rows, heads * n, dtype=dtype, device=DEV), torch.empty(rows, heads * n, dtype=dtype, device=DEV)
    ops.head_linear(x, w, out)
    refs.head_linear(x, w, want)
    close(out, want, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(37, 5, 2, 52, 22), (300, 6, 3, 128, 64), (1, 4, 1, 96, 40), (130, 3, 3, 40, 24),
                                   (1500, 4, 2, 128, 72), (900, 3, 1, 200, 136), (1024, 70, 4, 64, 24)])
def test_routing_and_expert_products(dtype, shape):
    """Routing, sorting by expert, the gathered rows, both grouped products and the combination, against the references;
    with an expert that nobody chooses and one that nearly everybody does."""
    from qwenforge_b200 import ops
    tokens, experts, top, width, ff = shape
    g = torch.Generator().manual_seed(sum(shape))
    logits = torch.randn(tokens, experts, generator=g)
    logits[:, 0] -= 30.0          # never among the chosen (unless top == experts)
    logits[:, 1] += 3.0           # nearly always
    logits = logits.to(DEV)
    x = torch.randn(tokens, width, generator=g).to(dtype).to(DEV)
    w1 = (torch.randn(experts, 2 * ff, width, generator=g) / math.sqrt(width)).to(dtype).to(DEV)
    w2 = (torch.randn(experts, width, ff, generator=g) / math.sqrt(ff)).to(dtype).to(DEV)
    tile_rows = ops.moe_tile_rows(tokens, experts, top, w1)   # 128 for the two largest shapes in bfloat16
    assert tile_rows == (128 if dtype == torch.bfloat16 and tokens >= 900 and experts < 10 else 64)
    plan, want_plan = ops.moe_plan(logits, top, tile_rows=tile_rows), refs.moe_plan(logits.cpu(), top)
    offsets = plan.offsets.cpu().tolist()
    counts = torch.bincount(want_plan.row_expert, minlength=experts).tolist()
    assert [offsets[e + 1] - offsets[e] for e in range(experts)] == counts
    dest, sorted_token, sorted_weight = plan.dest.cpu().long(), plan.sorted_token.cpu().long(), plan.sorted_weight.cpu()
    scores = torch.sigmoid(logits.cpu())
    chosen = torch.topk(scores, top).indices
    for t in range(tokens):
        for j in range(top):
            row = int(dest[t * top + j])
            e = int(chosen[t, j])
            assert offsets[e] <= row < offsets[e + 1] and int(sorted_token[row]) == t
            assert abs(float(sorted_weight[row]) - float(scores[t, e])) < 1e-6
    n_tiles = int(plan.n_tiles)
    assert n_tiles == sum(-(-c // tile_rows) for c in counts) <= plan.max_tiles
    # the whole feed-forward, with the weight on the input
    rows = torch.empty(plan.pairs, width, dtype=dtype, device=DEV)
    ops.moe_gather(x, plan, rows, True)
    want_rows = (x.double()[sorted_token.to(DEV)] * sorted_weight.to(DEV).double()[:, None])
    close(rows, want_rows, dtype, "gathered rows")
    gate_up = torch.empty(plan.pairs, 2 * ff, dtype=dtype, device=DEV)
    ops.expert_linear(rows, w1, plan, gate_up)
    row_expert = torch.empty(plan.pairs, dtype=torch.long)
    for e in range(experts):
        row_expert[offsets[e]:offsets[e + 1]] = e
    want_gu = torch.einsum("rk,rnk->rn", rows.double(), w1.double()[row_expert.to(DEV)])
    close(gate_up, want_gu, dtype, "gate/up of the experts")
    # the same rows read through the plan's row map, the weight moved behind the product
    unscaled = torch.empty_like(gate_up)
    ops.expert_linear(x, w1, plan, unscaled, gather=True)
    close(unscaled, torch.einsum("rk,rnk->rn", x.double()[sorted_token.to(DEV)], w1.double()[row_expert.to(DEV)]), dtype, "gathered product")
    act_scaled, want_act = torch.empty(plan.pairs, ff, dtype=dtype, device=DEV), torch.empty(plan.pairs, ff, dtype=dtype, device=DEV)
    ops.scaled_swiglu(unscaled, plan.sorted_weight, act_scaled)
    refs.scaled_swiglu(unscaled, plan.sorted_weight, want_act)
    close(act_scaled, want_act, dtype, "gate of scaled rows")
    act = torch.empty(plan.pairs, ff, dtype=dtype, device=DEV)
    ops.swiglu(gate_up, act)
    close(act_scaled, act, torch.bfloat16, "the weight before and behind the product")
    if ops.expert_gate_takes(x, w1, plan):   # bfloat16, tiles of 64 rows: the gate in the product's epilogue
        fused = torch.full((plan.pairs, ff), 7.0, dtype=dtype, device=DEV)
        ops.expert_gate_up(x, w1, plan, fused, plan.sorted_weight, gather=True)
        gu = torch.einsum("rk,rnk->rn", x.double()[sorted_token.to(DEV)], w1.double()[row_expert.to(DEV)]) * plan.sorted_weight.double()[:, None]
        close(fused, gu[:, :ff] * torch.sigmoid(gu[:, :ff]) * gu[:, ff:], dtype, "gate in the small tile's epilogue")
    else:
        assert dtype == torch.float32 or tile_rows == 128 or width % 8
    y = torch.empty(plan.pairs, width, dtype=dtype, device=DEV)
    ops.expert_linear(act, w2, plan, y)
    close(y, torch.einsum("rk,rnk->rn", act.double(), w2.double()[row_expert.to(DEV)]), dtype, "down of the experts")
    out = torch.empty(tokens, width, dtype=dtype, device=DEV)
    ops.moe_combine(y, plan, out, False)
    close(out, y.double()[dest.to(DEV)].view(tokens, top, width).sum(1), dtype, "combined")


@pytest.mark.parametrize("shape", [(1500, 4, 2, 128, 72), (900, 3, 1, 200, 136), (2100, 5, 3, 320, 64)])
def test_expert_products_on_tcgen05(shape):
    """The grouped form of the tcgen05 product: tiles that start at any row and end with their expert, experts whose size is
    no multiple of a tile's columns, the gate (with the rows' scale) in the first product's epilogue."""
    from qwenforge_b200 import ops
    tokens, experts, top, width, ff = shape
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(sum(shape))
    logits = torch.randn(tokens, experts, generator=g)
    logits[:, 0] -= 30.0
    logits = logits.to(DEV)
    x = torch.randn(tokens, width, generator=g).to(dtype).to(DEV)
    w1 = (torch.randn(experts, 2 * ff, width, generator=g) / math.sqrt(width)).to(dtype).to(DEV)
    w2 = (torch.randn(experts, width, ff, generator=g) / math.sqrt(ff)).to(dtype).to(DEV)
    plan = ops.moe_plan(logits, top, tile_rows=128)
    want_plan = refs.moe_plan(logits.cpu(), top)
    offsets = plan.offsets.cpu().tolist()
    row_expert = torch.empty(plan.pairs, dtype=torch.long)
    for e in range(experts):
        row_expert[offsets[e]:offsets[e + 1]] = e
    rows = torch.empty(plan.pairs, width, dtype=dtype, device=DEV)
    ops.moe_gather(x, plan, rows, False)
    assert ops.tc_gemm_grouped_takes(rows, w1, plan, ops.TC_SWIGLU)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    act = torch.full((plan.pairs, ff), 7.0, dtype=dtype, device=DEV)
    ops.tc_gemm_grouped(ops.TC_SWIGLU, rows, w1, plan, act, plan.sorted_weight, err)
    gu = torch.einsum("rk,rnk->rn", rows.double(), w1.double()[row_expert.to(DEV)]) * plan.sorted_weight.double()[:, None]
    want_act = gu[:, :ff] * torch.sigmoid(gu[:, :ff]) * gu[:, ff:]
    close(act, want_act, dtype, "gate in the epilogue")
    y = torch.full((plan.pairs, width), 7.0, dtype=dtype, device=DEV)
    ops.tc_gemm_grouped(ops.TC_PLAIN, act, w2, plan, y, None, err)
    close(y, torch.einsum("rk,rnk->rn", act.double(), w2.double()[row_expert.to(DEV)]), dtype, "down product")
    assert int(err) == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_plan_makes_the_routers_logits_itself_for_few_tokens(dtype):
    from qwenforge_b200 import ops
    g = torch.Generator().manual_seed(17)
    x = torch.randn(11, 200, generator=g).to(dtype).to(DEV)
    router = torch.randn(7, 200, generator=g).to(dtype).to(DEV)
    logits = (x.double() @ router.double().T).float()
    a, b = ops.moe_plan(None, 3, x=x, router=router), ops.moe_plan(logits, 3)
    assert torch.equal(a.offsets, b.offsets) and torch.equal(a.n_tiles, b.n_tiles)
    assert torch.equal(a.sorted_token[a.dest.long()], b.sorted_token[b.dest.long()])
    for plan in (a, b):   # pair (t, j) sits in a row of the expert chosen j-th for t, with that expert's score
        experts = torch.bucketize(plan.dest.long(), plan.offsets.long()[1:], right=True).view(11, 3).cpu()
        assert torch.equal(experts, torch.topk(logits.cpu(), 3).indices)
    assert max_err(a.sorted_weight[a.dest.long()], b.sorted_weight[b.dest.long()]) < 1e-5


def _latent_case(dtype, rank, heads, lengths, new, seed, sink_value=None):
    """A one-plane cache filled with random latents for sequences of `lengths`, queries for their last `new` positions."""
    from qwenforge_b200 import ops
    from qwenforge_b200.cache import KvNeed, SequenceCache
    g = torch.Generator().manual_seed(seed)
    cache = SequenceCache([KvNeed(1, rank, 0, planes=1)], 64 * 40, 8, 2048, dtype, DEV)
    slots = [cache.open() for _ in lengths]
    cache.reserve(list(zip(slots, lengths)))
    cache.flush()
    site = cache.site(0)
    latents = []
    for slot, n in zip(slots, lengths):
        c = torch.randn(n, rank, generator=g).to(dtype)
        latents.append(c)
        pages = site.table[slot, torch.arange(n, device=DEV) // 64].long()
        site.storage[pages, 0, 0, torch.arange(n, device=DEV) % 64] = c.to(DEV)
    q = torch.randn(sum(new), heads * rank, generator=g).to(dtype).to(DEV)
    sinks = (torch.randn(heads, generator=g) * 2 if sink_value is None else torch.full((heads,), sink_value)).float().to(DEV)
    cu = [0]
    for n in new:
        cu.append(cu[-1] + n)
    tok_pos = torch.cat([torch.arange(L - n, L) for L, n in zip(lengths, new)]).int().to(DEV)
    ctx = dict(cu_q=torch.tensor(cu, dtype=torch.int32, device=DEV), tok_pos=tok_pos, slots=torch.tensor(slots, dtype=torch.int32, device=DEV))
    return cache, site, ops.KvSiteArgs(site.storage, site.table, 1, rank), latents, q, sinks, ctx


def _latent_reference(latents, q, sinks, lengths, new, heads, rank, scale):
    rows, o = [], 0
    for c, L, n in zip(latents, lengths, new):
        c = c.double()
        for i in range(n):
            p = L - n + i
            qt = q[o + i].double().cpu().view(heads, rank)
            s = scale * qt @ c[:p + 1].T
            w = plain.sink_softmax(s, sinks.double().cpu()[:, None])
            rows.append((w @ c[:p + 1]).reshape(-1))
        o += n
    return torch.stack(rows)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rank,heads", [(36, 3), (64, 4), (128, 20), (300, 2)])
def test_generic_attention_with_sinks_over_a_shared_plane(dtype, rank, heads):
    from qwenforge_b200 import ops
    lengths, new = [130, 64, 7], [130, 3, 7]
    cache, site, args, latents, q, sinks, ctx = _latent_case(dtype, rank, heads, lengths, new, 5)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.empty_like(q)
    scale = 0.7 / math.sqrt(rank)
    ops.attention_generic(q, out, ctx["cu_q"], ctx["tok_pos"], ctx["slots"], args, heads, 3, max(new), scale, 0, err,
                          sinks=sinks, shared_values=True)
    close(out, _latent_reference(latents, q, sinks, lengths, new, heads, rank, scale), dtype)
    assert int(err) == 0


@pytest.mark.parametrize("rank,heads", [(32, 5), (64, 4), (96, 3), (128, 20)])
def test_tensor_core_attention_with_sinks_over_a_shared_plane(rank, heads):
    """The mma.sync prefill kernel and the split-K decode kernel read the latent plane as keys and as values and count the
    sink once, also when a sequence's runs are folded by the block with the last ticket."""
    from qwenforge_b200 import ops
    dtype = torch.bfloat16
    scale = 0.7 / math.sqrt(rank)
    lengths, new = [700, 65, 129], [200, 65, 2]
    cache, site, args, latents, q, sinks, ctx = _latent_case(dtype, rank, heads, lengths, new, 6)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.empty_like(q)
    ops.attention_prefill(q, out, ctx["cu_q"], ctx["tok_pos"], ctx["slots"], args, heads, 3, max(new), scale, 0, err,
                          max_kv_len=max(lengths), sinks=sinks, shared_values=True)
    close(out, _latent_reference(latents, q, sinks, lengths, new, heads, rank, scale), dtype, "prefill")
    if rank in (64, 128):   # the tcgen05 kernel: blocks of 128 rows, also as pairs of blocks that share a tile
        for lengths, new in (([700, 300, 129], [700, 130, 2]), ([1400], [1400])):
            cache, site, args, latents, q, sinks, ctx = _latent_case(dtype, rank, heads, lengths, new, 16)
            out = torch.empty_like(q)
            ops.attention_prefill_tc(q, out, ctx["cu_q"], ctx["tok_pos"], ctx["slots"], args, heads, len(lengths), max(new), scale, 0,
                                     err, max_kv_len=max(lengths), sinks=sinks, shared_values=True)
            close(out, _latent_reference(latents, q, sinks, lengths, new, heads, rank, scale), dtype, f"tcgen05 prefill {new}")
    for n_splits in (1, 4):
        lengths, new = [1500, 64, 65, 1], [1, 1, 1, 1]
        cache, site, args, latents, q, sinks, ctx = _latent_case(dtype, rank, heads, lengths, new, 7 + n_splits)
        scratch = ops.DecodeScratch(torch.device(DEV))
        out = torch.empty_like(q)
        ops.attention_decode(q, out, ctx["cu_q"], ctx["tok_pos"], ctx["slots"], args, heads, 4, scale, 0, n_splits, scratch, err,
                             sinks=sinks, shared_values=True)
        close(out, _latent_reference(latents, q, sinks, lengths, new, heads, rank, scale), dtype, f"decode, {n_splits} splits")
    assert int(err) == 0


@pytest.mark.parametrize("kernel", ["generic", "prefill", "prefill_tc", "decode"])
def test_a_large_sink_takes_the_weight_and_a_small_one_none(kernel):
    """With a sink far above every score the output vanishes; far below, the result is the plain softmax's."""
    from qwenforge_b200 import ops
    dtype, rank, heads, scale = torch.bfloat16, 64, 4, 0.1
    lengths, new = ([300], [1]) if kernel == "decode" else ([300], [300]) if kernel == "prefill_tc" else ([300], [100])
    for sink_value, what in ((60.0, "large"), (-60.0, "small")):
        cache, site, args, latents, q, sinks, ctx = _latent_case(dtype, rank, heads, lengths, new, 9, sink_value)
        err = torch.zeros(1, dtype=torch.int32, device=DEV)
        out = torch.empty_like(q)
        if kernel == "generic":
            ops.attention_generic(q, out, ctx["cu_q"], ctx["tok_pos"], ctx["slots"], args, heads, 1, max(new), scale, 0, err,
                                  sinks=sinks, shared_values=True)
        elif kernel in ("prefill", "prefill_tc"):
            run = ops.attention_prefill if kernel == "prefill" else ops.attention_prefill_tc
            run(q, out, ctx["cu_q"], ctx["tok_pos"], ctx["slots"], args, heads, 1, max(new), scale, 0, err, sinks=sinks, shared_values=True)
        else:
            ops.attention_decode(q, out, ctx["cu_q"], ctx["tok_pos"], ctx["slots"], args, heads, 1, scale, 0, 2,
                                 ops.DecodeScratch(torch.device(DEV)), err, sinks=sinks, shared_values=True)
        want = _latent_reference(latents, q, sinks, lengths, new, heads, rank, scale)
        close(out, want, dtype, f"{kernel}, {what} sink")
        assert (float(want.abs().max()) < 1e-6) == (what == "large")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_norm_cache_writes_each_token_to_its_own_place(dtype):
    from qwenforge_b200 import ops
    from qwenforge_b200.cache import KvNeed, SequenceCache
    q_rank, rank = 20, 36
    cache = SequenceCache([KvNeed(1, rank, 0, planes=1)], 64 * 8, 4, 512, dtype, DEV)
    a, b = cache.open(), cache.open()
    cache.reserve([(a, 70), (b, 3)])
    cache.flush()
    site = cache.site(0)
    args = ops.KvSiteArgs(site.storage, site.table, 1, rank)
    g = torch.Generator().manual_seed(3)
    down = torch.randn(9, q_rank + rank, generator=g).to(DEV)
    wq, wkv = (1 + 0.2 * torch.randn(q_rank, generator=g)).to(dtype).to(DEV), (1 + 0.2 * torch.randn(rank, generator=g)).to(dtype).to(DEV)
    tok_seq = torch.tensor([0] * 6 + [1] * 3, dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor([62, 63, 64, 65, 66, 67, 0, 1, 2], dtype=torch.int32, device=DEV)   # across a page border
    slots = torch.tensor([a, b], dtype=torch.int32, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    q_latent = torch.empty(9, q_rank, dtype=dtype, device=DEV)
    plain_out = torch.empty(9, rank, dtype=dtype, device=DEV)
    ops.latent_norm_cache(down, q_rank, wq, wkv, 1e-5, tok_seq, tok_pos, slots, q_latent, args, True, err, latent_out=plain_out)
    close(q_latent, refs._rms(down[:, :q_rank], wq, 1e-5), dtype, "query latent")
    want = refs._rms(down[:, q_rank:], wkv, 1e-5)
    close(plain_out, want, dtype, "latent")
    for t in range(9):
        slot, pos = int(slots[int(tok_seq[t])]), int(tok_pos[t])
        page = int(site.table[slot, pos // 64])
        assert torch.equal(site.storage[page, 0, 0, pos % 64], plain_out[t])
    assert int(err) == 0


# ------------------------------------------------------------------------------------------------ the model
def build(cfg, tmp_path, dtype, seed=0, spread=1.0):
    from qwenforge_b200.engine import Model
    folder, weights = make_model_dir(cfg, seed, tmp_path, spread=spread)
    return Model.from_dir(folder, dtype, DEV), weights, folder


def run_cuts(model, cache, tokens, cuts, want_all=True):
    """Feed `tokens` in steps of the given sizes through one slot; returns the logits of every position."""
    slot = cache.open()
    rows, at = [], 0
    for n in cuts:
        rows.append(model.step(cache, [(slot, tokens[at:at + n])], want=[list(range(n))]))
        at += n
    assert at == len(tokens)
    cache.close(slot)
    model.raise_on_kernel_error()
    return torch.cat(rows)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompts_decoding_and_portions(name, dtype, tmp_path):
    cfg = CONFIGS[name]
    model, weights, _ = build(cfg, tmp_path, dtype)
    torch_dtype = torch.float32 if dtype == "float32" else torch.bfloat16
    cache = model.new_cache(64 * 12, 4)
    tokens = random_tokens(cfg["vocab"], 200, 4)
    want, margins = plain.forward_logits(cfg, weights, tokens), plain.router_margins(cfg, weights, tokens)
    for cuts in ([200], [150] + [1] * 50, [64, 64, 64, 8], [63, 2, 65, 2, 2, 66], [1] * 3 + [197], [2] * 100):
        got = run_cuts(model, cache, tokens, cuts)
        logits_close(got, want, torch_dtype, f"{name} cut {cuts[:4]}", margins)
    # the first token of a sequence, alone
    if dtype == "float32" or float(margins[0]) > 0.03:
        logits_close(run_cuts(model, cache, tokens[:1], [1]), want[:1], torch_dtype, "one token")
    assert all(g.pages.n_free == g.pages.n_pages for g in cache.kv_groups)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cuts_agree_with_one_another_to_rounding(dtype, tmp_path):
    """float32: what a position's logits are must not depend on the cut beyond the rounding of sums."""
    cfg = MEF_FAST
    model, weights, _ = build(cfg, tmp_path, dtype, seed=8)
    cache = model.new_cache(64 * 12, 4)
    tokens = random_tokens(cfg["vocab"], 150, 6)
    whole, margins = run_cuts(model, cache, tokens, [150]), plain.router_margins(cfg, weights, tokens)
    for cuts in ([100] + [1] * 50, [7, 64, 79], [2] * 75):
        got = run_cuts(model, cache, tokens, cuts)
        logits_close(got, whole, torch.float32 if dtype == "float32" else torch.bfloat16, str(cuts[:3]), margins)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["odd", "fast"])
def test_unequal_batches_against_each_alone_in_reused_slots(name, dtype, tmp_path):
    cfg = CONFIGS[name]
    model, weights, _ = build(cfg, tmp_path, dtype, seed=1)
    torch_dtype = torch.float32 if dtype == "float32" else torch.bfloat16
    cache = model.new_cache(64 * 10, 3)       # three slots for five requests: slots and pages come back
    seqs = [random_tokens(cfg["vocab"], n, 20 + n) for n in (1, 130, 65, 64, 3)]
    refs_ = [plain.forward_logits(cfg, weights, s) for s in seqs]
    margins = [plain.router_margins(cfg, weights, s) for s in seqs]
    tail = 6
    for round_ in range(2):
        for batch in ([0, 1, 2], [3, 4]):
            slots = {i: cache.open() for i in batch}
            heads = {i: max(1, len(seqs[i]) - tail) for i in batch}
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
                for i in [i for i in live if fed[i] == len(seqs[i])]:
                    cache.close(slots.pop(i))       # ends earlier than the others: its slot is free for the next batch
                live = [i for i in live if fed[i] < len(seqs[i])]
            for i in list(slots):
                cache.close(slots.pop(i))
            for i in batch:
                if len(seqs[i]) > 8:    # (the shortest ones have too few rows for a statement about most rows)
                    logits_close(torch.cat(got[i]), refs_[i], torch_dtype, f"{name} round {round_} request {i}", margins[i])
                elif dtype == "float32":
                    logits_close(torch.cat(got[i]), refs_[i], torch_dtype, f"{name} round {round_} request {i}")
    model.raise_on_kernel_error()
    assert cache.slots.n_free == cache.max_seqs


def test_a_long_prompt_takes_the_tensor_core_experts(tmp_path):
    """1,600 tokens over four experts: tiles of 128 rows, both expert products on tcgen05, against the plain implementation."""
    cfg = config(300, 128, 1700, 1e-5, [layer(mixer(4, 16, 16, 64, 48), moe(64, 4, 2)), layer(mixer(4, 16, 16, 64, 48), dense(160, 2.0))])
    model, weights, _ = build(cfg, tmp_path, "bfloat16", seed=4)
    tokens = random_tokens(cfg["vocab"], 1600, 8)
    cache = model.new_cache(64 * 30, 2)
    got = run_cuts(model, cache, tokens, [1600])
    want = plain.forward_logits(cfg, weights, tokens)
    logits_close(got[::7], want[::7], torch.bfloat16, "long prompt", plain.router_margins(cfg, weights, tokens)[::7])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("order", ["none_last", "none_first", "only_none"])
def test_layers_without_a_feed_forward_at_either_end(order, dtype, tmp_path):
    """The last post-norm of the model has no next layer to ride on, and a layer without a feed-forward hands its mixer's
    output straight to the next layer's first norm."""
    with_ff = [layer(mixer(2, 16, 24, 32, 40, 0.3), moe(24, 3, 3)), layer(mixer(3, 8, 8, 96, 16, 0.5), dense(56, 1.1))]
    bare = layer(mixer(5, 8, 6, 64, 24, 0.35), None)
    layers = {"none_last": with_ff + [bare], "none_first": [bare] + with_ff, "only_none": [bare, bare]}[order]
    cfg = config(190, 40, 400, 2e-5, layers)
    model, weights, _ = build(cfg, tmp_path, dtype, seed=9)
    cache = model.new_cache(64 * 8, 2)
    tokens = random_tokens(cfg["vocab"], 150, 3)
    got = run_cuts(model, cache, tokens, [120] + [1] * 30)
    logits_close(got, plain.forward_logits(cfg, weights, tokens), torch.float32 if dtype == "float32" else torch.bfloat16, order,
                 plain.router_margins(cfg, weights, tokens))


def _far_key_model(kind):
    """One layer whose attention is made to hang on ONE far position: queries and keys are scaled up, so that a key that is
    lost, shifted by one or read from the wrong page changes the logits by far more than rounding."""
    return config(200, 64, 1500, 1e-5, [layer(mixer(2, 16, 16, 64 if kind == "fast" else 40, 24, 1.0), dense(96, 3.0))])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["fast", "generic"])
def test_far_keys_and_page_borders_show_in_the_logits(kind, dtype, tmp_path):
    cfg = _far_key_model(kind)
    # wide matrices: a peaked attention (less so in bfloat16, where scores of several tens carry their rounding into the weights)
    model, weights, folder = build(cfg, tmp_path, dtype, seed=12, spread=3.0 if dtype == "float32" else 1.5)
    torch_dtype = torch.float32 if dtype == "float32" else torch.bfloat16
    tokens = random_tokens(cfg["vocab"], 1100, 9)
    want = plain.forward_logits(cfg, weights, tokens)
    # the attention is peaked: dropping the most-attended far key would move the logits
    cache = model.new_cache(64 * 20, 2)
    places = [0, 1, 62, 63, 64, 65, 127, 128, 129, 511, 512, 1023, 1024, 1025, 1099]
    for cuts in ([1100], [1024, 76], [1000] + [1] * 100, [63, 1, 1, 1035]):
        got = run_cuts(model, cache, tokens, cuts)
        logits_close(got[places], want[places], torch_dtype, f"{kind} {cuts[:3]}")
        logits_close(got[-40:], want[-40:], torch_dtype, f"{kind} {cuts[:3]} tail")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_graphs_and_the_entry_point(dtype, tmp_path):
    """Greedy generation through StudentEngine (its scheduler, decode graphs, sampler) against greedy decoding with the
    plain implementation: float32 token by token; bfloat16 wherever the plain logits' margin allows a difference."""
    from qwenforge_b200.engine import StudentEngine
    cfg = MEF_FAST
    folder, weights = make_model_dir(cfg, 21, tmp_path)
    engine = StudentEngine(str(folder), device=DEV, dtype=dtype)
    assert engine.cuda_graphs      # every part of the design is graph safe
    prompts = [random_tokens(cfg["vocab"], n, 30 + n) for n in (5, 70, 33)]
    n_new = 40
    got = engine.generate_ids(prompts, max_new_tokens=n_new, batch_size=3, ignore_eos=True)
    for prompt, tokens in zip(prompts, got):
        assert len(tokens) == n_new
        seq = list(prompt)
        for step, token in enumerate(tokens):
            row = plain.forward_logits(cfg, weights, seq)[-1]
            best = torch.topk(row, 2)
            if dtype == "float32" or float(best.values[0] - best.values[1]) > 0.15 * float(row.std()):
                assert token == int(best.indices[0]), (dtype, step)
            seq.append(token)   # follow the engine's own choice
    # a second call runs in the slots and pages of the first
    again = engine.generate_ids(prompts, max_new_tokens=n_new, batch_size=2, ignore_eos=True)
    assert again == got


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_as_a_user_runs_it(dtype, tmp_path):
    """bin/trace_run in a process of its own: whole prompts, a prompt and then its last tokens one by one, and a batch of
    unequal requests decoded together whose shorter members end earlier; requests that end give their slots back."""
    import json
    import subprocess
    import sys
    from pathlib import Path

    import numpy as np
    root = Path(__file__).resolve().parent.parent
    cfg = MEF_ODD
    folder, weights = make_model_dir(cfg, 31, tmp_path / "model")
    vocab = cfg["vocab"]
    torch_dtype = torch.float32 if dtype == "float32" else torch.bfloat16
    requests = {f"q{i}": random_tokens(vocab, n, 70 + i) for i, n in enumerate((90, 1, 40, 130))}
    want = {k: plain.forward_logits(cfg, weights, v) for k, v in requests.items()}
    margins = {k: plain.router_margins(cfg, weights, v) for k, v in requests.items()}

    def run(steps, out_dir, max_tokens):
        text = "".join(json.dumps(s) + "\n" for s in steps)
        done = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
                               "--out", str(out_dir), "--max-tokens", str(max_tokens)], input=text, capture_output=True, text=True, timeout=900)
        assert done.returncode == 0, done.stderr[-2000:]
        assert [line for line in done.stdout.splitlines() if line.startswith("done ")] == [f"done {s['step']}" for s in steps]

    def read(out_dir, step):
        return torch.from_numpy(np.fromfile(Path(out_dir) / f"{step}.f32", dtype="<f4").reshape(-1, vocab).copy())

    # whole, one after the other in one process: at most 130 tokens are live at any time
    steps = [dict(step=i, entries=[dict(id=k, tokens=v, want=list(range(len(v))))], end=[k]) for i, (k, v) in enumerate(requests.items())]
    run(steps, tmp_path / "whole", 130)
    for i, k in enumerate(requests):
        if len(requests[k]) > 8:
            logits_close(read(tmp_path / "whole", i), want[k], torch_dtype, f"whole {k}", margins[k])
    # a prompt, then its last 20 tokens one by one; the step that wants nothing writes no file
    k, v = "q3", requests["q3"]
    head = len(v) - 20
    steps = [dict(step=0, entries=[dict(id=k, tokens=v[:head], want=[])], end=[])]
    steps += [dict(step=1 + t, entries=[dict(id=k, tokens=[v[head + t]], want=[0])], end=[k] if t == 19 else []) for t in range(20)]
    run(steps, tmp_path / "tail", 130)
    assert not (tmp_path / "tail" / "0.f32").exists()
    tail = torch.cat([read(tmp_path / "tail", 1 + t) for t in range(20)])
    logits_close(tail, want[k][head:], torch_dtype, "last tokens one by one", margins[k][head:])
    # three requests start together (the lengths differ), are decoded together, and the shorter ones end earlier
    cut = {"q0": 85, "q1": 1, "q2": 33}
    steps = [dict(step=0, entries=[dict(id=k, tokens=requests[k][:n], want=[n - 1]) for k, n in cut.items()], end=["q1"])]
    fed, live, n = dict(cut), ["q0", "q2"], 1
    got = {k: [] for k in cut}
    order = {0: list(cut)}
    while live:
        steps.append(dict(step=n, entries=[dict(id=k, tokens=[requests[k][fed[k]]], want=[0]) for k in live],
                          end=[k for k in live if fed[k] + 1 == len(requests[k])]))
        order[n] = list(live)
        for k in live:
            fed[k] += 1
        live = [k for k in live if fed[k] < len(requests[k])]
        n += 1
    run(steps, tmp_path / "batch", 85 + 1 + 33 + 12)
    for step, names in order.items():
        rows = read(tmp_path / "batch", step)
        for row, k in zip(rows, names):
            got[k].append(row)
    for k in ("q0", "q2"):
        logits_close(torch.stack(got[k]), want[k][cut[k] - 1:], torch_dtype, f"batch {k}", margins[k][cut[k] - 1:])
