"""Plain PyTorch references of every CUDA kernel, with the kernels' own signatures.

Each function states in tensor operations what its kernel computes; the `-m gpu` tests compare the
two on the same inputs. The functions work on any device, so the CPU tests can also put them in
the kernels' place (`conftest.reference_kernels`) to exercise the step function, the cache and the
generation loop without a GPU. They are test code: the package never imports them.
"""
from __future__ import annotations

import torch

from tests import plain_qwen2 as plain

PAGE = 64


def _f(t):
    return t.to(torch.float64)


def embed_gather(ids, table, out, err):
    out.copy_(table[ids.long()].to(torch.float32))


def gather_rows(hidden, delta, rows, out, err):
    picked = hidden[rows.long()]
    if delta is not None:
        picked = picked + delta[rows.long()].to(torch.float32)
    out.copy_(picked)


def gather_rows_norm(hidden, delta, rows, weight, eps, out, err):
    picked = hidden[rows.long()]
    if delta is not None:
        picked = picked + delta[rows.long()].to(torch.float32)
    x = _f(picked)
    out.copy_((x * torch.rsqrt(x.square().mean(-1, keepdim=True) + eps) * _f(weight)).to(out.dtype))


def add_rms_norm(hidden, delta, weight, eps, out):
    if delta is not None:
        hidden += delta.to(torch.float32)
    x = _f(hidden)
    normed = x * torch.rsqrt(x.square().mean(-1, keepdim=True) + eps) * _f(weight)
    out.copy_(normed.to(out.dtype))


def gemm_f32(x, weight, bias, out):
    y = _f(x) @ _f(weight).T
    if bias is not None:
        y = y + _f(bias)
    out.copy_(y.to(out.dtype))


def linear(x, weight, bias=None, out=None, out_dtype=None):
    y = _f(x) @ _f(weight).T
    if bias is not None:
        y = y + _f(bias)
    y = y.to(out_dtype or x.dtype)
    if out is not None:
        out.copy_(y)
        return out
    return y


def _kv_rows(site, slot, positions, head, which):
    """storage rows of `positions` (list) for one head: returns (page ids, offsets)."""
    pages = site.table[slot, torch.as_tensor(positions, device=site.table.device) // PAGE].long()
    offs = torch.as_tensor(positions, device=site.table.device) % PAGE
    return pages, offs


def rope_cache_write(qkv, tok_seq, tok_pos, slots, inv_freq, rot_dim, n_heads, q_out, site, write_cache, err, bias=None):
    n = qkv.shape[0]
    d, kvh = site.head_dim, site.kv_heads
    x = _f(qkv)
    if bias is not None:
        x = x + _f(bias)
    q = x[:, :n_heads * d].reshape(n, n_heads, d).clone()
    k = x[:, n_heads * d:(n_heads + kvh) * d].reshape(n, kvh, d).clone()
    v = x[:, (n_heads + kvh) * d:].reshape(n, kvh, d)
    if inv_freq is not None and rot_dim > 0:
        angle = (tok_pos.to(torch.float32).unsqueeze(-1) * inv_freq.to(torch.float32)).to(torch.float64)
        cos, sin = angle.cos().unsqueeze(1), angle.sin().unsqueeze(1)
        half = rot_dim // 2
        for t in (q, k):
            x1, x2 = t[..., :half].clone(), t[..., half:rot_dim].clone()
            t[..., :half] = x1 * cos - x2 * sin
            t[..., half:rot_dim] = x2 * cos + x1 * sin
    q_out.copy_(q.reshape(n, n_heads * d).to(q_out.dtype))
    if not write_cache:
        return
    for t in range(n):
        slot = int(slots[int(tok_seq[t])])
        if slot < 0:
            continue
        pos = int(tok_pos[t])
        page = int(site.table[slot, pos // PAGE])
        assert page >= 0, "reference: write to a page that is not held"
        site.storage[page, 0, :, pos % PAGE, :] = k[t].to(site.storage.dtype)
        site.storage[page, 1, :, pos % PAGE, :] = v[t].to(site.storage.dtype)


def gather_kv(site, slot, lo, hi):
    """Keys and values of positions lo..hi-1 of `slot`: two [kv_heads, hi-lo, head_dim] float64 tensors."""
    pos = torch.arange(lo, hi, device=site.table.device)
    pages = site.table[slot, pos // PAGE].long()
    assert bool((pages >= 0).all()), "reference: read of a page that is not held"
    k = site.storage[pages, 0, :, pos % PAGE, :]  # [n, kvh, d]
    v = site.storage[pages, 1, :, pos % PAGE, :]
    return _f(k).transpose(0, 1), _f(v).transpose(0, 1)


def gather_keys(site, slot, lo, hi):
    """Rows lo..hi-1 of a one-plane cache: [kv_heads, hi-lo, head_dim] float64."""
    pos = torch.arange(lo, hi, device=site.table.device)
    pages = site.table[slot, pos // PAGE].long()
    assert bool((pages >= 0).all()), "reference: read of a page that is not held"
    return _f(site.storage[pages, 0, :, pos % PAGE, :]).transpose(0, 1)


def attention_generic(q, out, cu_q, tok_pos, slots, site, n_heads, n_seqs, max_q_len, scale, window, err, scratch=None, max_kv_len=None,
                      sinks=None, shared_values=False):
    d, kvh = site.head_dim, site.kv_heads
    groups = n_heads // kvh
    for s in range(n_seqs):
        b, e = int(cu_q[s]), int(cu_q[s + 1])
        slot = int(slots[s])
        if slot < 0:
            out[b:e] = 0
            continue
        for t in range(b, e):
            p = int(tok_pos[t])
            lo = max(0, p - window + 1) if window > 0 else 0
            if shared_values:
                k = v = gather_keys(site, slot, lo, p + 1)
            else:
                k, v = gather_kv(site, slot, lo, p + 1)
            qt = _f(q[t]).view(n_heads, d)
            k = k.repeat_interleave(groups, dim=0)
            v = v.repeat_interleave(groups, dim=0)
            scores = torch.einsum("hd,hjd->hj", qt, k) * scale
            if sinks is not None:   # one more term in the denominator, with no value
                weights = torch.softmax(torch.cat((scores, _f(sinks)[:, None]), dim=-1), -1)[:, :-1]
            else:
                weights = torch.softmax(scores, -1)
            ctx = torch.einsum("hj,hjd->hd", weights, v)
            out[t] = ctx.reshape(-1).to(out.dtype)


def swiglu(gate_up, out):
    inter = gate_up.shape[1] // 2
    g, u = _f(gate_up[:, :inter]), _f(gate_up[:, inter:])
    out.copy_((g * torch.sigmoid(g) * u).to(out.dtype))


def sample(logits, temperature, seed, seq_ids, steps, out, scratch=None):
    for r in range(logits.shape[0]):
        token, _ = plain.sample_token(logits[r].cpu(), temperature, seed,
                                      int(seq_ids[r]) if seq_ids is not None else 0,
                                      int(steps[r]) if steps is not None else 0)
        out[r] = token


def _rms(x, weight, eps):
    x = _f(x)
    return x * torch.rsqrt(x.square().mean(-1, keepdim=True) + eps) * _f(weight)


def embed_positions(ids, tok_pos, table, positions, out, err):
    out.copy_((_f(table[ids.long()]) + _f(positions[tok_pos.long()])).to(torch.float32))


def sandwich_norm(hidden, y, post_weight, post_eps, next_weight=None, next_eps=0.0, out=None, dest=None, top=1, row_weight=None):
    if dest is not None:
        y = _f(y) if row_weight is None else _f(y) * _f(row_weight)[:, None]
        y = y[dest.long()].view(-1, top, y.shape[1]).sum(1)
    hidden += _rms(y, post_weight, post_eps).to(torch.float32)
    if next_weight is not None:
        out.copy_(_rms(hidden, next_weight, next_eps).to(out.dtype))


def clamped_glu(gate_up, limit, alpha, out):
    inter = gate_up.shape[1] // 2
    g = _f(gate_up[:, :inter]).clamp(max=limit)
    u = _f(gate_up[:, inter:]).clamp(min=-limit, max=limit)
    out.copy_((g * torch.sigmoid(alpha * g) * (u + 1)).to(out.dtype))


def latent_norm_cache(down, q_rank, q_norm, kv_norm, eps, tok_seq, tok_pos, slots, q_latent, site, write_cache, err, latent_out=None):
    if q_rank:
        q_latent.copy_(_rms(down[:, :q_rank], q_norm, eps).to(q_latent.dtype))
    c = _rms(down[:, q_rank:], kv_norm, eps)
    if latent_out is not None:
        latent_out.copy_(c.to(latent_out.dtype))
    if not write_cache:
        return
    for t in range(down.shape[0]):
        slot = int(slots[int(tok_seq[t])])
        if slot < 0:
            continue
        pos = int(tok_pos[t])
        page = int(site.table[slot, pos // PAGE])
        assert page >= 0, "reference: write to a page that is not held"
        site.storage[page, 0, 0, pos % PAGE, :] = c[t].to(site.storage.dtype)


def head_linear(x, weight, out):
    groups, n, k = weight.shape
    y = torch.einsum("tgk,gnk->tgn", _f(x).view(x.shape[0], groups, k), _f(weight))
    out.copy_(y.reshape(x.shape[0], groups * n).to(out.dtype))


class _Routing:
    pass


def linear_rows(x, weight, out_dtype=None):
    return linear(x, weight, None, out_dtype=out_dtype)


def moe_tile_rows(n_tokens, n_experts, top, weight):
    return 64


def expert_gate_takes(x, weight, plan):
    return False


def tc_gemm_grouped(epilogue, x, weight, plan, out, row_scale=None, err=None):
    y = torch.einsum("rk,rnk->rn", _f(x), _f(weight)[plan.row_expert])
    if epilogue == 1:   # gate rows then up rows, a scale on both before the gate
        inter = y.shape[1] // 2
        s = _f(row_scale)[:, None] if row_scale is not None else 1.0
        g, u = y[:, :inter] * s, y[:, inter:] * s
        y = g * torch.sigmoid(g) * u
    out.copy_(y.to(out.dtype))


def scaled_swiglu(gate_up, row_scale, out):
    inter = gate_up.shape[1] // 2
    g, u = _f(gate_up[:, :inter]) * _f(row_scale)[:, None], _f(gate_up[:, inter:]) * _f(row_scale)[:, None]
    out.copy_((g * torch.sigmoid(g) * u).to(out.dtype))


def moe_plan(logits, top, softmax_scores=False, renormalize=False, tile_rows=64, x=None, router=None):
    if logits is None:
        logits = (_f(x) @ _f(router).T)
    z = logits.to(torch.float32)
    scores = torch.softmax(z, -1) if softmax_scores else torch.sigmoid(z)
    chosen = torch.topk(scores, top, dim=-1)
    weights = chosen.values / chosen.values.sum(-1, keepdim=True) if renormalize else chosen.values
    plan = _Routing()
    plan.n_tokens, plan.n_experts, plan.top, plan.pairs = z.shape[0], z.shape[1], top, z.shape[0] * top
    experts = chosen.indices.reshape(-1)
    order = torch.sort(experts, stable=True).indices                    # rows: pairs sorted by expert
    plan.sorted_token = (order // top).to(torch.int32)
    plan.sorted_weight = weights.reshape(-1)[order].to(torch.float32)
    plan.row_expert = experts[order]
    plan.dest = torch.empty(plan.pairs, dtype=torch.int32)
    plan.dest[order] = torch.arange(plan.pairs, dtype=torch.int32)
    return plan


def moe_gather(x, plan, out, scale_input):
    rows = _f(x)[plan.sorted_token.long()]
    if scale_input:
        rows = rows * _f(plan.sorted_weight)[:, None]
    out.copy_(rows.to(out.dtype))


def moe_combine(y, plan, out, scale_output):
    rows = _f(y)
    if scale_output:
        rows = rows * _f(plan.sorted_weight)[:, None]
    out.copy_(rows[plan.dest.long()].view(plan.n_tokens, plan.top, -1).sum(1).to(out.dtype))


def expert_linear(x, weight, plan, out, gather=False):
    rows = _f(x)[plan.sorted_token.long()] if gather else _f(x)
    out.copy_(torch.einsum("rk,rnk->rn", rows, _f(weight)[plan.row_expert]).to(out.dtype))


ALL = dict(expert_gate_takes=expert_gate_takes, linear_rows=linear_rows, moe_tile_rows=moe_tile_rows, scaled_swiglu=scaled_swiglu, embed_positions=embed_positions, sandwich_norm=sandwich_norm, clamped_glu=clamped_glu, latent_norm_cache=latent_norm_cache,
           head_linear=head_linear, moe_plan=moe_plan, moe_gather=moe_gather, moe_combine=moe_combine, expert_linear=expert_linear,
           embed_gather=embed_gather, gather_rows=gather_rows, gather_rows_norm=gather_rows_norm, add_rms_norm=add_rms_norm, gemm_f32=gemm_f32,
           linear=linear, rope_cache_write=rope_cache_write, attention_generic=attention_generic, swiglu=swiglu,
           sample=sample)
