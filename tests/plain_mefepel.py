"""A plain, slow implementation of the Mefepel decoder, one function per mechanism, in float64 on the CPU.

It shares no code with the package: the tests compare the package's kernels, cache and step function with it.

The design, in this file's notation (t: a token of a sequence at position p_t, counted from 0):

  stream     x_t = E[token_t] + P[p_t]
  layer      x += rms(mixer(rms(x; w1)); w1b)   then, if the layer has a feed-forward,
             x += rms(ff(rms(x; w2)); w2b)
  rms(v; w)  v / sqrt(mean(v^2) + eps) * w
  mixer      latent attention: a = rms(Dq h; nq), q = Uq a  (heads of `dim`);  c = rms(Dkv h; nkv)  (the cached latent)
             k_j = Uk c_j, v_j = Uv c_j per head;  s_ij = scale * q_i . k_j for j <= i
             w_ij = exp(s_ij) / (exp(sink_head) + sum_{j' <= i} exp(s_ij'))   (the sink has no key and no value)
             out = O concat_heads(sum_j w_ij v_j)
  dense ff   g = min(G h, limit), u = clamp(U h, -limit, limit), y = g * sigmoid(1.702 g) * (u + 1), out = D y
  moe ff     s = sigmoid(R h); the `top` experts with the largest s; out = sum over them of expert_e(s_e * h),
             expert(v) = D_e (silu(G_e v) * (U_e v))
  logits     H rms(x; wf)
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def rms(v: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return v / torch.sqrt((v * v).mean(dim=-1, keepdim=True) + eps) * w


def embed(weights, tokens, first_position: int = 0) -> torch.Tensor:
    ids = torch.as_tensor(tokens, dtype=torch.long)
    places = torch.arange(first_position, first_position + len(ids))
    return weights["embed"].to(F)[ids] + weights["pos"].to(F)[places]


def latent_of(weights, prefix: str, h: torch.Tensor, eps: float) -> torch.Tensor:
    """What the mixer keeps per position: the normalised key/value latent."""
    return rms(h @ weights[prefix + "dkv"].to(F).T, weights[prefix + "dkv.norm"].to(F), eps)


def queries_of(weights, prefix: str, h: torch.Tensor, eps: float) -> torch.Tensor:
    a = rms(h @ weights[prefix + "dq"].to(F).T, weights[prefix + "dq.norm"].to(F), eps)
    return a @ weights[prefix + "uq"].to(F).T


def sink_softmax(scores: torch.Tensor, sink: torch.Tensor) -> torch.Tensor:
    """Rows of `scores` [..., keys] (masked entries -inf) against one extra term exp(sink) in the denominator."""
    top = torch.maximum(scores.max(dim=-1, keepdim=True).values, sink)
    e = torch.exp(scores - top)
    return e / (e.sum(dim=-1, keepdim=True) + torch.exp(sink - top))


def latent_attention(weights, prefix: str, mixer: dict, h: torch.Tensor, eps: float, latents_before=None):
    """h [T, width]: the normed input of T consecutive positions that follow `latents_before` [T0, kv_rank] (or nothing).
    Returns the mixer's output [T, width] and all latents [T0 + T, kv_rank]."""
    heads, dim, vdim, scale = mixer["heads"], mixer["dim"], mixer["vdim"], float(mixer["scale"])
    c_new = latent_of(weights, prefix, h, eps)
    c = c_new if latents_before is None else torch.cat((latents_before, c_new))
    t0, t = c.shape[0] - h.shape[0], h.shape[0]
    q = queries_of(weights, prefix, h, eps).view(t, heads, dim)
    k = (c @ weights[prefix + "uk"].to(F).T).view(-1, heads, dim)
    v = (c @ weights[prefix + "uv"].to(F).T).view(-1, heads, vdim)
    sinks = weights[prefix + "sink"].to(F)
    out = torch.zeros(t, heads, vdim, dtype=F)
    key_index = torch.arange(c.shape[0])
    for head in range(heads):
        s = scale * (q[:, head] @ k[:, head].T)                               # [t, t0 + t]
        hidden = key_index[None, :] > (t0 + torch.arange(t))[:, None]
        s = s.masked_fill(hidden, -math.inf)
        out[:, head] = sink_softmax(s, sinks[head]) @ v[:, head]
    return out.reshape(t, heads * vdim) @ weights[prefix + "o"].to(F).T, c


def dense_ff(weights, prefix: str, mlp: dict, h: torch.Tensor) -> torch.Tensor:
    limit = float(mlp["limit"])
    g = torch.clamp(h @ weights[prefix + "gate"].to(F).T, max=limit)
    u = torch.clamp(h @ weights[prefix + "up"].to(F).T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ weights[prefix + "down"].to(F).T


def expert_ff(weights, prefix: str, v: torch.Tensor) -> torch.Tensor:
    g = v @ weights[prefix + "gate"].to(F).T
    return (g * torch.sigmoid(g) * (v @ weights[prefix + "up"].to(F).T)) @ weights[prefix + "down"].to(F).T


def route(weights, prefix: str, mlp: dict, h: torch.Tensor):
    """Per token the chosen experts and their weights (the sigmoid scores themselves)."""
    s = torch.sigmoid(h @ weights[prefix + "router"].to(F).T)
    chosen = torch.topk(s, int(mlp["router"]["top"]), dim=-1)
    return chosen.indices, chosen.values


def moe_ff(weights, prefix: str, mlp: dict, h: torch.Tensor) -> torch.Tensor:
    experts, scores = route(weights, prefix, mlp, h)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, s in zip(experts[t].tolist(), scores[t]):
            out[t] += expert_ff(weights, f"{prefix}e{e}.", (s * h[t])[None])[0]
    return out


def feed_forward(weights, prefix: str, mlp: dict, h: torch.Tensor) -> torch.Tensor:
    return dense_ff(weights, prefix, mlp, h) if mlp["kind"] == "dense" else moe_ff(weights, prefix, mlp, h)


def layer(weights, config: dict, index: int, x: torch.Tensor, latents_before=None):
    spec, eps, p = config["layers"][index], float(config["norm"]["eps"]), f"l{index}."
    mixed, latents = latent_attention(weights, p + "mix.", spec["mixer"], rms(x, weights[p + "norm1"].to(F), eps), eps,
                                      latents_before)
    x = x + rms(mixed, weights[p + "norm1b"].to(F), eps)
    if spec.get("mlp") is not None:
        y = feed_forward(weights, p + "mlp.", spec["mlp"], rms(x, weights[p + "norm2"].to(F), eps))
        x = x + rms(y, weights[p + "norm2b"].to(F), eps)
    return x, latents


def router_margins(config: dict, weights, tokens) -> torch.Tensor:
    """Per token, the smallest gap over all routed layers between the last chosen expert's logit and the first one left
    out, relative to the token's largest logit there (inf without routed layers). A token whose margin is below the
    rounding of a 16-bit path may rightly be routed otherwise there."""
    x = embed(weights, tokens)
    eps = float(config["norm"]["eps"])
    margins = torch.full((len(tokens),), math.inf, dtype=F)
    for i, spec in enumerate(config["layers"]):
        mlp, p = spec.get("mlp"), f"l{i}."
        if mlp is not None and mlp["kind"] == "moe" and mlp["router"]["top"] < mlp["router"]["experts"]:
            mixed, _ = latent_attention(weights, p + "mix.", spec["mixer"], rms(x, weights[p + "norm1"].to(F), eps), eps)
            h = rms(x + rms(mixed, weights[p + "norm1b"].to(F), eps), weights[p + "norm2"].to(F), eps)
            z = torch.sort(h @ weights[p + "mlp.router"].to(F).T, dim=-1, descending=True).values
            top = mlp["router"]["top"]
            margins = torch.minimum(margins, (z[:, top - 1] - z[:, top]) / z.abs().max(-1).values)
        x, _ = layer(weights, config, i, x)
    return margins


def logits_of(weights, config: dict, x: torch.Tensor) -> torch.Tensor:
    return rms(x, weights["final.norm"].to(F), float(config["norm"]["eps"])) @ weights["head"].to(F).T


def forward_logits(config: dict, weights, tokens, streams: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of a whole sequence in one go. `streams`, if given, receives x after every layer."""
    x = embed(weights, tokens)
    for i in range(len(config["layers"])):
        x, _ = layer(weights, config, i, x)
        if streams is not None:
            streams.append(x.clone())
    return logits_of(weights, config, x)


def decode_logits(config: dict, weights, tokens, first: int) -> torch.Tensor:
    """The same logits computed as a prompt of `first` tokens and then one token at a time over kept latents."""
    kept = [None] * len(config["layers"])
    rows = []
    cuts = [(0, first)] + [(i, i + 1) for i in range(first, len(tokens))]
    for lo, hi in cuts:
        x = embed(weights, tokens[lo:hi], lo)
        for i in range(len(config["layers"])):
            x, kept[i] = layer(weights, config, i, x, kept[i])
        rows.append(logits_of(weights, config, x))
    return torch.cat(rows)


# ------------------------------------------------------------------------------------------------ test models
def tensor_shapes(config: dict) -> dict:
    width, shapes = config["width"], {}
    shapes["embed"] = (config["vocab"], width)
    shapes["pos"] = (config["max_positions"], width)
    for i, spec in enumerate(config["layers"]):
        p, m = f"l{i}.", spec["mixer"]
        shapes[p + "norm1"] = shapes[p + "norm1b"] = (width,)
        shapes[p + "mix.dq"] = (m["q_rank"], width)
        shapes[p + "mix.dq.norm"] = (m["q_rank"],)
        shapes[p + "mix.uq"] = (m["heads"] * m["dim"], m["q_rank"])
        shapes[p + "mix.dkv"] = (m["kv_rank"], width)
        shapes[p + "mix.dkv.norm"] = (m["kv_rank"],)
        shapes[p + "mix.uk"] = (m["heads"] * m["dim"], m["kv_rank"])
        shapes[p + "mix.uv"] = (m["heads"] * m["vdim"], m["kv_rank"])
        shapes[p + "mix.sink"] = (m["heads"],)
        shapes[p + "mix.o"] = (width, m["heads"] * m["vdim"])
        mlp = spec.get("mlp")
        if mlp is None:
            continue
        shapes[p + "norm2"] = shapes[p + "norm2b"] = (width,)
        if mlp["kind"] == "dense":
            shapes[p + "mlp.gate"] = shapes[p + "mlp.up"] = (mlp["ff"], width)
            shapes[p + "mlp.down"] = (width, mlp["ff"])
        else:
            shapes[p + "mlp.router"] = (mlp["router"]["experts"], width)
            for e in range(mlp["router"]["experts"]):
                shapes[f"{p}mlp.e{e}.gate"] = shapes[f"{p}mlp.e{e}.up"] = (mlp["expert"]["ff"], width)
                shapes[f"{p}mlp.e{e}.down"] = (width, mlp["expert"]["ff"])
    shapes["final.norm"] = (width,)
    shapes["head"] = (config["vocab"], width)
    return shapes


def random_weights(config: dict, seed: int, spread: float = 1.0) -> dict:
    """float32 weights whose values bfloat16 holds exactly (so that both precisions load the same model). Matrices are
    drawn wide enough that attention and the routers are far from uniform."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        if name.endswith("sink"):
            value = torch.randn(shape, generator=g) * 1.5
        elif len(shape) == 1:
            value = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif name in ("embed", "pos"):
            value = torch.randn(shape, generator=g)
        else:
            value = torch.randn(shape, generator=g) * spread * (2.0 / math.sqrt(shape[1]))
        out[name] = value.to(torch.bfloat16).to(torch.float32)
    return out
