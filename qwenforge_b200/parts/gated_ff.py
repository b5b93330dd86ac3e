"""Feed-forwards with other gates than SwiGLU's.

`clamped_glu`: both halves of the gate/up product are clamped before they meet, the gate is x * sigmoid(alpha x) and
the linear half is shifted by one:
    g = min(G h, limit),  u = clamp(U h, -limit, limit),  out = D (g * sigmoid(alpha * g) * (u + 1))
Gate and up weights are concatenated by rows so that one product yields both halves; no biases."""
from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, TensorSpec
from .registry import register_part


class ClampedGlu(FeedForward):
    """params: hidden_size, intermediate_size, limit, alpha. tensors: gate_weight [I, W], up_weight [I, W], down_weight [W, I]."""

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(self.params["hidden_size"])
        self.inter = int(self.params["intermediate_size"])
        self.limit = float(self.params["limit"])
        self.alpha = float(self.params["alpha"])
        self.gate_up_weight = self.down_weight = None

    def tensor_specs(self):
        return [
            TensorSpec(self.file_name("gate_weight"), (self.inter, self.hidden)),
            TensorSpec(self.file_name("up_weight"), (self.inter, self.hidden)),
            TensorSpec(self.file_name("down_weight"), (self.hidden, self.inter)),
        ]

    def kernel_libraries(self, dtype):
        return {"activation"} | ({"gemm_f32"} if dtype == torch.float32 else {"skinny_gemm"})

    def bind(self, tensors, dtype, device):
        self.gate_up_weight = torch.cat((tensors[self.file_name("gate_weight")], tensors[self.file_name("up_weight")]),
                                        dim=0).contiguous()
        self.down_weight = tensors[self.file_name("down_weight")]

    def step_weights(self):
        return [self.gate_up_weight, self.down_weight]

    def forward(self, x, ctx):
        act = torch.empty((x.shape[0], self.inter), dtype=x.dtype, device=x.device)
        ops.clamped_glu(ops.linear_rows(x, self.gate_up_weight), self.limit, self.alpha, act)
        return ops.linear_rows(act, self.down_weight)


register_part("feed_forward", "clamped_glu", ClampedGlu)
