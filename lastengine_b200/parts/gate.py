"""Gates on a sublayer's result.

sigmoid_gate: s = sigmoid(R h + b), one factor per channel, computed from the same input h the
sublayer reads; the block arrangement multiplies the sublayer's result by it before the sum into
the residual stream.  The product runs in the activation type with a float result; bias, sigmoid,
product and sum are float.
"""
from __future__ import annotations

import torch

from ..ops import kernels
from ..registry import GATES
from .base import BIAS, MATRIX, BuildEnv, Part, TensorSpec


@GATES.register("sigmoid_gate")
class SigmoidGate(Part):
    def __init__(self, hidden_size: int, bias: bool = True, tensor: str = "weight", bias_tensor: str = "bias"):
        self.D = int(hidden_size)
        self.bias = bool(bias)
        self.tensor, self.bias_tensor = str(tensor), str(bias_tensor)
        self.w = self.b = None

    def tensors(self) -> dict[str, TensorSpec]:
        t = {self.tensor: TensorSpec((self.D, self.D), MATRIX)}
        if self.bias:
            t[self.bias_tensor] = TensorSpec((self.D,), BIAS, std=0.5)
        return t

    def load(self, tensors, env: BuildEnv) -> None:
        self.w = tensors[self.tensor].contiguous()
        self.b = tensors[self.bias_tensor].to(torch.float32).contiguous() if self.bias else None

    def add_gated(self, x: torch.Tensor, y: torch.Tensor, h: torch.Tensor, env: BuildEnv, z: torch.Tensor | None = None,
                  next_norm=None, h_out: torch.Tensor | None = None) -> None:
        """x += y * sigmoid(R h + b); x the float residual, y the sublayer's float result, h its input.
        `z`: R h where another product has already formed it (a sublayer that took this gate's rows
        into its own first product).  `next_norm` and `h_out`: the same launch also leaves the norm
        of the new x there, for the sublayer that reads the stream next."""
        if z is None:
            M = h.shape[0]
            z = env.workspace.get("gate.z", (M, self.D), torch.float32)
            kernels.linear(z, h, self.w)
        if next_norm is not None:
            kernels.gated_residual(x, y, z, self.b, h_out, next_norm.weight, next_norm.eps)
        else:
            kernels.gated_residual(x, y, z, self.b)

    def give_rows_to(self, part) -> bool:
        """Lets `part` form R h in its own first product (one launch fewer); the gate then holds no matrix."""
        take = getattr(part, "absorb_input_rows", None)
        if self.w is None or take is None or not take(self.w):
            return False
        self.w = None
        return True
