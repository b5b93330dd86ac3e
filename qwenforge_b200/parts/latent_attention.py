"""Latent attention without positions: queries and keys/values both go through a low-rank latent, and the key/value
latent is all that is kept per position.

  a = rmsnorm(Dq h) * nq,   q = Uq a            queries, `heads` heads of `dim`
  c = rmsnorm(Dkv h) * nkv                      the cached latent, `kv_rank` numbers per position
  k_j = Uk c_j,  v_j = Uv c_j  (per head)       never formed:
      score_ij = scale * q_i . (Uk c_j) = scale * (Uk^T q_i) . c_j      the query goes into the latent space,
      out_i    = Uv (sum_j w_ij c_j)                                     the weighted latents come back out,
  so every head attends to the one latent "head" as key and as value (`shared_values`), and a step over a long cache
  reads kv_rank numbers per position instead of heads * (dim + vdim).
  w_ij = exp(score_ij) / (exp(sink_head) + sum_{j' <= i} exp(score_ij'))  a learned sink per head joins the denominator
  result = O concat_heads(out_i)

Dq and Dkv run as one product (float32 out: both norms read 32-bit sums); the two norms and the cache write are one
kernel (`ops.latent_norm_cache`); the per-head maps into and out of the latent space are one grouped launch each
(`ops.head_linear`). Nothing here knows a model: ranks, head sizes, scale and eps come from the spec, `q_rank` 0 means
queries straight from h, `sinks` false means a plain softmax, `window` limits the keys like any attention's.
"""
from __future__ import annotations

import torch

from .. import ops
from ..cache import PAGE_TOKENS, KvNeed
from .attention import TC_PREFILL_MIN_TOKENS
from .base import Mixer, TensorSpec
from .registry import register_part


class LatentAttention(Mixer):
    """params: hidden_size, num_heads, head_dim, value_dim, kv_rank, q_rank, scale, eps, sinks (bool), window.
    tensors: q_down [q_rank, W], q_norm [q_rank], q_up [H*dim, q_rank] (q_rank 0: q_up [H*dim, W] alone), kv_down [kv_rank, W],
    kv_norm [kv_rank], k_up [H*dim, kv_rank], v_up [H*vdim, kv_rank], sink [H], o_weight [W, H*vdim]."""

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.n_heads = int(p["num_heads"])
        self.head_dim = int(p["head_dim"])
        self.value_dim = int(p.get("value_dim") or self.head_dim)
        self.kv_rank = int(p["kv_rank"])
        self.q_rank = int(p.get("q_rank") or 0)
        self.scale = float(p.get("scale") or self.head_dim ** -0.5)
        self.eps = float(p["eps"])
        self.has_sinks = bool(p.get("sinks", False))
        self.window = int(p.get("window") or 0)
        if self.kv_rank > ops.GENERIC_MAX_HEAD_DIM:
            raise ValueError(f"latent_attention: kv_rank {self.kv_rank} > {ops.GENERIC_MAX_HEAD_DIM} is not supported by the attention kernels")
        self.down_weight = self.q_norm = self.kv_norm = self.q_up = self.k_absorb = self.v_up = self.sinks = self.o_weight = None

    def tensor_specs(self):
        h, d, v, r, q, w = self.n_heads, self.head_dim, self.value_dim, self.kv_rank, self.q_rank, self.hidden
        specs = [TensorSpec(self.file_name("kv_down"), (r, w)), TensorSpec(self.file_name("kv_norm"), (r,), init="norm"),
                 TensorSpec(self.file_name("k_up"), (h * d, r)), TensorSpec(self.file_name("v_up"), (h * v, r)),
                 TensorSpec(self.file_name("o_weight"), (w, h * v))]
        if q:
            specs += [TensorSpec(self.file_name("q_down"), (q, w)), TensorSpec(self.file_name("q_norm"), (q,), init="norm"),
                      TensorSpec(self.file_name("q_up"), (h * d, q))]
        else:
            specs.append(TensorSpec(self.file_name("q_up"), (h * d, w)))
        if self.has_sinks:
            specs.append(TensorSpec(self.file_name("sink"), (h,), init="logit", keep="float32"))
        return specs

    def kernel_libraries(self, dtype):
        libs = {"latent_cache", "attention_generic", "grouped_gemm"}
        if dtype == torch.float32:
            libs.add("gemm_f32")
        elif self.kv_rank in ops.FAST_ATTENTION_HEAD_DIMS:
            libs |= {"attention_decode", "attention_prefill", "skinny_gemm"}
            if self.kv_rank in ops.TC_ATTENTION_HEAD_DIMS:
                libs.add("attention_prefill_tc")
        return libs

    def cache_need(self):
        return KvNeed(1, self.kv_rank, self.window, planes=1)

    def bind(self, tensors, dtype, device):
        t = lambda logical: tensors[self.file_name(logical)]
        h, d, v, r = self.n_heads, self.head_dim, self.value_dim, self.kv_rank
        if self.q_rank:
            self.down_weight = torch.cat((t("q_down"), t("kv_down")), dim=0).contiguous()
            self.q_norm = t("q_norm")
        else:
            self.down_weight = t("kv_down")
        self.kv_norm = t("kv_norm")
        self.q_up = t("q_up")
        self.k_absorb = t("k_up").view(h, d, r).transpose(1, 2).contiguous()   # [H, kv_rank, dim]: q_h -> Uk_h^T q_h
        self.v_up = t("v_up").view(h, v, r)                                    # [H, vdim, kv_rank]
        self.o_weight = t("o_weight")
        self.sinks = t("sink").to(torch.float32).contiguous() if self.has_sinks else None

    def step_weights(self):
        return [x for x in (self.down_weight, self.q_norm, self.kv_norm, self.q_up, self.k_absorb, self.v_up, self.sinks,
                            self.o_weight) if x is not None]

    # ------------------------------------------------------------------ the step
    def _latents(self, x, ctx, args, writes_cache):
        """The queries of the step's tokens, [T, H * dim], after the key/value latents went into the cache."""
        n = x.shape[0]
        down = ops.linear_rows(x, self.down_weight, out_dtype=torch.float32)
        if not self.q_rank:
            ops.latent_norm_cache(down, 0, None, self.kv_norm, self.eps, ctx.tok_seq, ctx.tok_pos, ctx.slots, None, args,
                                  writes_cache, ctx.err)
            return ops.linear_rows(x, self.q_up)
        q_latent = torch.empty((n, self.q_rank), dtype=x.dtype, device=x.device)
        ops.latent_norm_cache(down, self.q_rank, self.q_norm, self.kv_norm, self.eps, ctx.tok_seq, ctx.tok_pos, ctx.slots,
                              q_latent, args, writes_cache, ctx.err)
        return ops.linear_rows(q_latent, self.q_up)

    def forward(self, x, ctx, site, writes_cache):
        n, h, r = x.shape[0], self.n_heads, self.kv_rank
        args = ops.KvSiteArgs(site.storage, site.table, 1, r)
        q = self._latents(x, ctx, args, writes_cache)
        q_in_latent = torch.empty((n, h * r), dtype=x.dtype, device=x.device)
        ops.head_linear(q, self.k_absorb, q_in_latent)
        attended = torch.empty_like(q_in_latent)
        fast = ctx.attention == "auto" and x.dtype == torch.bfloat16 and r in ops.FAST_ATTENTION_HEAD_DIMS
        if fast and ctx.is_decode and n == ctx.n_seqs:
            n_splits = self.decode_splits(ctx)
            ops.attention_decode(q_in_latent, attended, ctx.cu_q, ctx.tok_pos, ctx.slots, args, h, ctx.n_seqs, self.scale,
                                 self.window, n_splits, ctx.decode_scratch, ctx.err, self.decode_plan(ctx, n_splits),
                                 sinks=self.sinks, shared_values=True)
        elif fast:
            # long steps on the tcgen05 kernel (blocks of 128 query rows), from the same sizes as any attention's
            least = TC_PREFILL_MIN_TOKENS.get(r)
            prefill = (ops.attention_prefill_tc if least is not None and n >= least and ctx.max_q_len >= 128
                       else ops.attention_prefill)
            prefill(q_in_latent, attended, ctx.cu_q, ctx.tok_pos, ctx.slots, args, h, ctx.n_seqs, ctx.max_q_len,
                                  self.scale, self.window, ctx.err, max_kv_len=ctx.max_kv_len, sinks=self.sinks,
                                  shared_values=True)
        else:
            ops.attention_generic(q_in_latent, attended, ctx.cu_q, ctx.tok_pos, ctx.slots, args, h, ctx.n_seqs, ctx.max_q_len,
                                  self.scale, self.window, ctx.err, scratch=ctx.decode_scratch, max_kv_len=ctx.max_kv_len,
                                  sinks=self.sinks, shared_values=True)
        values = torch.empty((n, h * self.value_dim), dtype=x.dtype, device=x.device)
        ops.head_linear(attended, self.v_up, values)
        return ops.linear_rows(values, self.o_weight)

    def decode_plan(self, ctx, n_splits: int) -> torch.Tensor:
        """The decode attention's plan of this step, shared through the step's memo by every layer of this shape."""
        key = ("latent_attention.decode_plan", self.n_heads, self.kv_rank, self.window, n_splits)
        memo = ctx.step_memo if ctx.step_memo is not None else {}
        plan = memo.get(key)
        if plan is None:
            plan = memo[key] = ops.attention_decode_plan(ctx.cu_q, ctx.tok_pos, ctx.slots, 1, self.kv_rank, self.n_heads,
                                                         ctx.n_seqs, self.window, n_splits, ctx.decode_scratch)
        return plan

    def decode_splits(self, ctx) -> int:
        """The most blocks that may share one sequence's latents (see `GqaAttention.decode_splits`)."""
        span = ctx.max_kv_len if self.window <= 0 else min(ctx.max_kv_len, self.window + PAGE_TOKENS)
        pages = max(1, -(-span // PAGE_TOKENS))
        warps = ops.attention_decode_warps(self.kv_rank)
        return max(1, min(-(-pages // warps), 64))


register_part("mixer", "latent_attention", LatentAttention)
