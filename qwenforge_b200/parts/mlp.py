"""The two-product feed-forward without a gate: out = Wd act(Wu h + bu) + bd. The activation is a parameter (the square
of relu, tanh-GELU, silu, relu), as are the biases; the first bias and the activation are one kernel."""
from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, TensorSpec
from .registry import register_part


class ActivatedMlp(FeedForward):
    """params: hidden_size, intermediate_size, activation, bias (bool). tensors: up_weight [I, W], down_weight [W, I]
    (+ up_bias [I], down_bias [W])."""

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(self.params["hidden_size"])
        self.inter = int(self.params["intermediate_size"])
        self.activation = str(self.params["activation"])
        self.bias = bool(self.params.get("bias", False))
        if self.activation not in ops.ACTIVATIONS:
            raise ValueError(f"activated_mlp: unknown activation {self.activation!r}; known: {', '.join(ops.ACTIVATIONS)}")
        self.up_weight = self.down_weight = self.up_bias = self.down_bias = None

    def tensor_specs(self):
        specs = [TensorSpec(self.file_name("up_weight"), (self.inter, self.hidden)),
                 TensorSpec(self.file_name("down_weight"), (self.hidden, self.inter))]
        if self.bias:
            specs += [TensorSpec(self.file_name("up_bias"), (self.inter,), init="bias"),
                      TensorSpec(self.file_name("down_bias"), (self.hidden,), init="bias")]
        return specs

    def kernel_libraries(self, dtype):
        return {"activation"} | ({"gemm_f32"} if dtype == torch.float32 else {"skinny_gemm"})

    def bind(self, tensors, dtype, device):
        self.up_weight = tensors[self.file_name("up_weight")]
        self.down_weight = tensors[self.file_name("down_weight")]
        if self.bias:
            self.up_bias = tensors[self.file_name("up_bias")]
            self.down_bias = tensors[self.file_name("down_bias")]

    def step_weights(self):
        return [t for t in (self.up_weight, self.up_bias, self.down_weight, self.down_bias) if t is not None]

    def forward(self, x, ctx):
        up = ops.linear_rows(x, self.up_weight)
        act = torch.empty_like(up)
        ops.bias_act(up, self.up_bias, self.activation, act)
        if self.down_bias is None:
            return ops.linear_rows(act, self.down_weight)
        return ops.linear(act, self.down_weight, self.down_bias)


register_part("feed_forward", "activated_mlp", ActivatedMlp)
