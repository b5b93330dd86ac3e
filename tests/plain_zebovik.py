"""A plain, slow implementation of the Zebovik decoder, one function per mechanism, in float64 on the CPU.

It shares no code with the package: the tests compare the package's kernels, cache, state and step function with it.

The design, in this file's notation (t: a token of a sequence at position p_t, counted from 0; h: a sublayer's input):

  stream      x_t = E[token_t]
  layer       x += rms(mixer(rms(x; w1)); w1b),  then, if the layer has a feed-forward,  x += rms(ff(rms(x; w2)); w2b)
  rms(v; w)   v / sqrt(mean(v^2) + eps) * w;   unit(v) = v / sqrt(mean(v^2) + eps)
  attention   q = Wq h + bq, k = Wk h + bk, v = Wv h + bv, in heads; the first `rot.dims` components of q and k are
              rotated by p_t (component i with i + dims/2, angle p * base^(-2i/dims)); then q <- unit(q), k <- unit(k)
              per head; s_ij = cap * tanh(scale * q_i . k_j / cap) for j <= i in the same block of `mask.size` positions;
              w_ij = exp(s_ij) / (1 + sum_j' exp(s_ij'));  out = Wo concat_heads(sum_j w_ij v_j).
              A layer with `kv_from: j` has no k and v of its own: it reads what layer j keeps.
  mlstm       q = Wq h / sqrt(dim), k = Wk h, v = Wv h in heads;  a = cap tanh((Wi h + bi) / cap),
              f = logsigmoid(cap tanh((Wf h + bf) / cap)) per head;  with m_-1 = 0, S_-1 = 0, n_-1 = 0:
              m_t = max(f_t + m_t-1, a_t);  S_t = exp(f_t + m_t-1 - m_t) S_t-1 + exp(a_t - m_t) k_t v_t^T;  n_t likewise with k_t;
              o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6);  out = Wo (concat_heads(unit(o_t)) * wn * sigmoid(Wg h))
  mamba2      [z | x | B | C | dt] = W_in h;  (x, B, C) <- silu(causal_conv(x, B, C) + b);  dt <- softplus(dt + dt_bias);
              per head (its group's B and C):  S_t = exp(-exp(A_log) dt_t) S_t-1 + dt_t B_t x_t^T;  y_t = S_t^T C_t + D x_t;
              out = Wo (rms_in_parts(y * silu(z)) * wn)
  dense ff    Wd relu(Wu h + bu)^2 + bd
  logits      c tanh(H rms(x; wf) / c)
"""
from __future__ import annotations

import math

import torch

F = torch.float64
MLSTM_FLOOR = 1e-6   # added to the mLSTM's denominator


def rms(v: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return v / torch.sqrt((v * v).mean(dim=-1, keepdim=True) + eps) * w


def unit(v: torch.Tensor, eps: float) -> torch.Tensor:
    return v / torch.sqrt((v * v).mean(dim=-1, keepdim=True) + eps)


def softcap(z: torch.Tensor, cap: float) -> torch.Tensor:
    return cap * torch.tanh(z / cap)


def rotate(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, heads, dim]; the first `dims` components of every head turn by the token's position."""
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    angle = positions.to(F)[:, None, None] * freq
    u, w = x[..., :half], x[..., half:dims]
    return torch.cat((u * angle.cos() - w * angle.sin(), w * angle.cos() + u * angle.sin(), x[..., dims:]), dim=-1)


def sink_softmax(scores: torch.Tensor) -> torch.Tensor:
    """Rows of scores (hidden entries -inf) with one more term of score 0 in the denominator."""
    top = torch.clamp(scores.max(dim=-1, keepdim=True).values, min=0.0)
    e = torch.exp(scores - top)
    return e / (e.sum(dim=-1, keepdim=True) + torch.exp(-top))


# ------------------------------------------------------------------ attention
def attention_keys_values(weights, prefix, mixer, h, first_position, eps):
    """What an attention layer keeps for T consecutive positions: rotated unit keys [T, G, dim], values [T, G, vdim]."""
    t, g = h.shape[0], mixer["kv_heads"]
    positions = torch.arange(first_position, first_position + t)
    k = (h @ weights[prefix + "k"].to(F).T + weights[prefix + "k.b"].to(F)).view(t, g, mixer["dim"])
    v = (h @ weights[prefix + "v"].to(F).T + weights[prefix + "v.b"].to(F)).view(t, g, mixer["vdim"])
    k = unit(rotate(k, positions, mixer["rot"]["dims"], float(mixer["rot"]["base"])), eps)
    return k, v


def attention(weights, prefix, mixer, h, first_position, eps, keys, values):
    """h [T, W] at positions first_position..; keys/values hold ALL positions 0..first_position+T-1."""
    t, heads, g = h.shape[0], mixer["heads"], mixer["kv_heads"]
    positions = torch.arange(first_position, first_position + t)
    q = (h @ weights[prefix + "q"].to(F).T + weights[prefix + "q.b"].to(F)).view(t, heads, mixer["dim"])
    q = unit(rotate(q, positions, mixer["rot"]["dims"], float(mixer["rot"]["base"])), eps)
    block = int(mixer["mask"]["size"])
    j = torch.arange(keys.shape[0])
    hidden = (j[None, :] > positions[:, None]) | (j[None, :] // block != positions[:, None] // block)
    out = torch.zeros(t, heads, mixer["vdim"], dtype=F)
    for head in range(heads):
        kv = head // (heads // g)
        s = softcap(float(mixer["scale"]) * (q[:, head] @ keys[:, kv].T), float(mixer["softcap"]))
        out[:, head] = sink_softmax(s.masked_fill(hidden, -math.inf)) @ values[:, kv]
    return out.reshape(t, -1) @ weights[prefix + "o"].to(F).T


# ------------------------------------------------------------------ mLSTM
def mlstm_gates(weights, prefix, mixer, h):
    """Log input gate and log forget gate, [T, heads] each."""
    cap = float(mixer["gate_cap"])
    a = softcap(h @ weights[prefix + "i"].to(F).T + weights[prefix + "i.b"].to(F), cap)
    f = torch.nn.functional.logsigmoid(softcap(h @ weights[prefix + "f"].to(F).T + weights[prefix + "f.b"].to(F), cap))
    return a, f


def mlstm(weights, prefix, mixer, h, eps, state=None):
    """state: (S [heads, dim, vdim], n [heads, dim], m [heads]) or None for a sequence's start."""
    t, heads, dim, vdim = h.shape[0], mixer["heads"], mixer["dim"], mixer["vdim"]
    q = (h @ weights[prefix + "q"].to(F).T).view(t, heads, dim) * dim ** -0.5
    k = (h @ weights[prefix + "k"].to(F).T).view(t, heads, dim)
    v = (h @ weights[prefix + "v"].to(F).T).view(t, heads, vdim)
    a, f = mlstm_gates(weights, prefix, mixer, h)
    if state is None:
        state = (torch.zeros(heads, dim, vdim, dtype=F), torch.zeros(heads, dim, dtype=F), torch.zeros(heads, dtype=F))
    S, n, m = (x.clone() for x in state)
    out = torch.zeros(t, heads, vdim, dtype=F)
    for i in range(t):
        m_new = torch.maximum(f[i] + m, a[i])
        keep, take = torch.exp(f[i] + m - m_new), torch.exp(a[i] - m_new)
        S = keep[:, None, None] * S + take[:, None, None] * k[i][:, :, None] * v[i][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[i]
        m = m_new
        below = torch.maximum((n * q[i]).sum(-1).abs(), torch.exp(-m)) + MLSTM_FLOOR
        out[i] = torch.einsum("hdv,hd->hv", S, q[i]) / below[:, None]
    y = unit(out, eps).reshape(t, heads * vdim) * weights[prefix + "norm"].to(F)
    y = y * torch.sigmoid(h @ weights[prefix + "g"].to(F).T)
    return y @ weights[prefix + "o"].to(F).T, (S, n, m)


# ------------------------------------------------------------------ Mamba-2
def causal_conv(u, taps_weight, bias, before):
    """u [T, C]; taps_weight [C, taps] (last column weighs the current token); before [taps - 1, C]: the inputs of the
    positions just before (zeros at a sequence's start). Returns the convolution [T, C] and the new `before`."""
    taps = taps_weight.shape[1]
    padded = torch.cat((before, u))
    out = torch.zeros_like(u)
    for j in range(taps):
        out += padded[j:j + u.shape[0]] * taps_weight[:, j]
    return out + bias, padded[padded.shape[0] - (taps - 1):]


def mamba2(weights, prefix, mixer, h, eps, state=None):
    """state: (S [heads, N, vdim], before [taps - 1, channels]) or None."""
    t, heads, vdim, N, G = h.shape[0], mixer["heads"], mixer["vdim"], mixer["state"], mixer["groups"]
    inner, taps = heads * vdim, mixer["conv"]
    proj = h @ weights[prefix + "in"].to(F).T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    if state is None:
        state = (torch.zeros(heads, N, vdim, dtype=F), torch.zeros(taps - 1, xbc.shape[1], dtype=F))
    S, before = state[0].clone(), state[1]
    xbc, before = causal_conv(xbc, weights[prefix + "conv"].to(F), weights[prefix + "conv.b"].to(F), before)
    xbc = torch.nn.functional.silu(xbc)
    x = xbc[:, :inner].view(t, heads, vdim)
    B = xbc[:, inner:inner + G * N].view(t, G, N)
    C = xbc[:, inner + G * N:].view(t, G, N)
    dt = torch.nn.functional.softplus(dt + weights[prefix + "dt_bias"].to(F))
    rate = torch.exp(weights[prefix + "A_log"].to(F))
    skip = weights[prefix + "D"].to(F)
    group_of = torch.arange(heads) // (heads // G)
    y = torch.zeros(t, heads, vdim, dtype=F)
    for i in range(t):
        keep = torch.exp(-rate * dt[i])
        S = keep[:, None, None] * S + dt[i][:, None, None] * B[i][group_of][:, :, None] * x[i][:, None, :]
        y[i] = torch.einsum("hnv,hn->hv", S, C[i][group_of]) + skip[:, None] * x[i]
    y = y.reshape(t, inner) * torch.nn.functional.silu(z)
    parts = mixer["norm_groups"]
    y = unit(y.view(t, parts, inner // parts), eps).reshape(t, inner) * weights[prefix + "norm"].to(F)
    return y @ weights[prefix + "o"].to(F).T, (S, before)


# ------------------------------------------------------------------ feed-forward, head
def dense_ff(weights, prefix, h):
    up = torch.relu(h @ weights[prefix + "up"].to(F).T + weights[prefix + "up.b"].to(F))
    return (up * up) @ weights[prefix + "down"].to(F).T + weights[prefix + "down.b"].to(F)


def logits_of(cfg, weights, x):
    z = rms(x, weights["final.norm"].to(F), float(cfg["norm"]["eps"])) @ weights["head"].to(F).T
    return softcap(z, float(cfg["logit_softcap"]))


# ------------------------------------------------------------------ a sequence
class Sequence:
    """One sequence: `feed(tokens)` runs the next tokens from what earlier calls left and returns their logits."""

    def __init__(self, cfg, weights):
        self.cfg, self.weights, self.length = cfg, weights, 0
        self.kept = [None] * len(cfg["layers"])
        self.streams = None   # after every layer, of the last call: [layers, T, width]

    def feed(self, tokens):
        cfg, w, eps = self.cfg, self.weights, float(self.cfg["norm"]["eps"])
        x = w["embed"].to(F)[torch.as_tensor(tokens, dtype=torch.long)]
        streams = []
        for i, layer in enumerate(cfg["layers"]):
            p, mixer, kind = f"l{i}.", layer["mixer"], layer["type"]
            h = rms(x, w[p + "norm1"].to(F), eps)
            if kind == "attention":
                source = mixer.get("kv_from")
                if source is None:
                    k, v = attention_keys_values(w, p + "mix.", mixer, h, self.length, eps)
                    if self.kept[i] is not None:
                        k, v = torch.cat((self.kept[i][0], k)), torch.cat((self.kept[i][1], v))
                    self.kept[i] = (k, v)
                else:
                    k, v = self.kept[int(source)]
                y = attention(w, p + "mix.", mixer, h, self.length, eps, k, v)
            elif kind == "mlstm":
                y, self.kept[i] = mlstm(w, p + "mix.", mixer, h, eps, self.kept[i])
            elif kind == "mamba2":
                y, self.kept[i] = mamba2(w, p + "mix.", mixer, h, eps, self.kept[i])
            else:
                raise ValueError(f"unknown mixer {kind!r}")
            x = x + rms(y, w[p + "norm1b"].to(F), eps)
            if layer.get("mlp") is not None:
                h = rms(x, w[p + "norm2"].to(F), eps)
                x = x + rms(dense_ff(w, p + "mlp.", h), w[p + "norm2b"].to(F), eps)
            streams.append(x)
        self.length += len(tokens)
        self.streams = torch.stack(streams)
        return logits_of(cfg, w, x)


def forward_logits(cfg, weights, tokens):
    return Sequence(cfg, weights).feed(tokens)


def decode_logits(cfg, weights, tokens, first: int):
    """The first `first` tokens in one call, the rest one by one."""
    seq = Sequence(cfg, weights)
    return torch.cat([seq.feed(tokens[:first])] + [seq.feed([t]) for t in tokens[first:]])


def greedy_generate(cfg, weights, prompt, n_new: int):
    seq = Sequence(cfg, weights)
    out = [int(seq.feed(prompt)[-1].argmax())]
    while len(out) < n_new:
        out.append(int(seq.feed([out[-1]])[-1].argmax()))
    return out


# ------------------------------------------------------------------ names, shapes, random weights
def tensor_shapes(cfg) -> dict:
    W, shapes = cfg["width"], {"embed": (cfg["vocab"], cfg["width"]), "final.norm": (cfg["width"],),
                               "head": (cfg["vocab"], cfg["width"])}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        shapes[p + "norm1"] = shapes[p + "norm1b"] = (W,)
        if layer["type"] == "attention":
            shapes[p + "mix.q"], shapes[p + "mix.q.b"] = (m["heads"] * m["dim"], W), (m["heads"] * m["dim"],)
            shapes[p + "mix.o"] = (W, m["heads"] * m["vdim"])
            if m.get("kv_from") is None:
                shapes[p + "mix.k"], shapes[p + "mix.k.b"] = (m["kv_heads"] * m["dim"], W), (m["kv_heads"] * m["dim"],)
                shapes[p + "mix.v"], shapes[p + "mix.v.b"] = (m["kv_heads"] * m["vdim"], W), (m["kv_heads"] * m["vdim"],)
        elif layer["type"] == "mlstm":
            hd, hv = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            shapes.update({p + "mix.q": (hd, W), p + "mix.k": (hd, W), p + "mix.v": (hv, W), p + "mix.g": (hv, W),
                           p + "mix.o": (W, hv), p + "mix.norm": (hv,), p + "mix.i": (m["heads"], W),
                           p + "mix.i.b": (m["heads"],), p + "mix.f": (m["heads"], W), p + "mix.f.b": (m["heads"],)})
        else:
            inner, gn = m["heads"] * m["vdim"], m["groups"] * m["state"]
            shapes.update({p + "mix.in": (2 * inner + 2 * gn + m["heads"], W), p + "mix.conv": (inner + 2 * gn, m["conv"]),
                           p + "mix.conv.b": (inner + 2 * gn,), p + "mix.dt_bias": (m["heads"],), p + "mix.A_log": (m["heads"],),
                           p + "mix.D": (m["heads"],), p + "mix.norm": (inner,), p + "mix.o": (W, inner)})
        if layer.get("mlp") is not None:
            ff = layer["mlp"]["ff"]
            shapes[p + "norm2"] = shapes[p + "norm2b"] = (W,)
            shapes.update({p + "mlp.up": (ff, W), p + "mlp.up.b": (ff,), p + "mlp.down": (W, ff), p + "mlp.down.b": (W,)})
    return shapes


def random_weights(cfg, seed: int, spread: float = 1.0) -> dict:
    """Float32 weights that exercise every term: matrices N(0, spread / sqrt(in)), norms near 1, biases and gates wide
    enough that caps, sinks and decays all matter."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".", 1)[-1] if name.startswith("l") else name
        if len(shape) == 2 and not leaf.endswith("conv"):
            t = torch.randn(shape, generator=g) * spread / math.sqrt(shape[1])
            if leaf in ("mix.i", "mix.f"):
                t = t * 2.0
        elif leaf.endswith("conv"):
            t = torch.randn(shape, generator=g) * 0.5
        elif "norm" in leaf:
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif leaf == "mix.A_log":
            t = torch.randn(shape, generator=g) * 0.5 - 0.5
        elif leaf == "mix.dt_bias":
            t = torch.randn(shape, generator=g) * 0.5 - 1.0
        elif leaf == "mix.D":
            t = 1.0 + 0.3 * torch.randn(shape, generator=g)
        elif leaf == "mix.f.b":
            t = 2.0 + torch.randn(shape, generator=g)
        else:
            t = 0.3 * torch.randn(shape, generator=g)
        out[name] = t.to(torch.float32)
    return out
