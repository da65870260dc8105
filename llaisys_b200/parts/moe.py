from __future__ import annotations

import torch

from .. import kernels
from .base import FeedForward, TensorDecl, register_part


@register_part("ffn", "routed_experts")
class RoutedExperts(FeedForward):
    """A mixture of small feed-forward experts of which every token uses `top`, plus (optionally) a shared expert
    that every token uses.

      gates     g = sigmoid(Wr h), computed in float32
      choice    the `top` experts with the largest g + bias (`bias`: a per-expert correction that steers the choice
                only); ties go to the lower index
      weights   g of the chosen experts times route_scale, not renormalised
      expert    Wd act(Wu h), no biases; act = max(., 0)^2 ("relu_squared")
      output    sum over the chosen experts of weight * expert(h), plus shared(h)

    The experts' matrices are kept stacked ([E, ff, H] and [E, H, ff]).  A step's (token, choice) pairs are grouped by
    expert on the device (kernels.moe_plan) and the two products run over those groups: in bfloat16 on tcgen05, the
    second one ending in the weighted add into the float32 residual stream (float32 atomics, arrival order); in float32
    (and for widths the tensor-core kernel does not take) on the CUDA cores with the weighted sum added in a fixed
    order.  Nothing is read back to the host, so a step can be captured.

    params: hidden_size, experts, top, expert_ff, route_scale, act, shared_ff (None: no shared expert), use_bias, names
    (local tensor names: router, bias, expert_up, expert_down with {e} for the expert's index, shared_up, shared_down).
    """
    capturable = True
    NAMES = {"router": "router", "bias": "correction", "expert_up": "e{e}.up", "expert_down": "e{e}.down",
             "shared_up": "shared.up", "shared_down": "shared.down"}

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden, self.n_experts, self.top = int(p["hidden_size"]), int(p["experts"]), int(p["top"])
        self.ff = int(p["expert_ff"])
        self.route_scale = float(p.get("route_scale", 1.0))
        self.act = str(p.get("act", "relu_squared"))
        if self.act != "relu_squared":
            raise ValueError(f"expert activation {self.act!r} is not built (relu_squared)")
        if not (1 <= self.top <= self.n_experts):
            raise ValueError(f"a token cannot use {self.top} of {self.n_experts} experts")
        self.shared_ff = int(p["shared_ff"]) if p.get("shared_ff") else None
        self.use_bias = bool(p.get("use_bias", True))
        self.names = dict(self.NAMES, **(p.get("names") or {}))
        self.router = self.bias = self.up = self.down = self.shared_up = self.shared_down = None

    def tensors(self):
        n = self.names
        t = {n["router"]: TensorDecl((self.n_experts, self.hidden))}
        if self.use_bias:
            t[n["bias"]] = TensorDecl((self.n_experts,), use="vector")
        for e in range(self.n_experts):
            t[n["expert_up"].format(e=e)] = TensorDecl((self.ff, self.hidden))
            t[n["expert_down"].format(e=e)] = TensorDecl((self.hidden, self.ff))
        if self.shared_ff:
            t[n["shared_up"]] = TensorDecl((self.shared_ff, self.hidden))
            t[n["shared_down"]] = TensorDecl((self.hidden, self.shared_ff))
        return t

    def load(self, tensors):
        n = self.names
        self.router = tensors[n["router"]].contiguous()
        self.bias = tensors[n["bias"]].to(torch.float32).contiguous() if self.use_bias else None
        self.up = torch.stack([tensors[n["expert_up"].format(e=e)] for e in range(self.n_experts)]).contiguous()
        self.down = torch.stack([tensors[n["expert_down"].format(e=e)] for e in range(self.n_experts)]).contiguous()
        if self.shared_ff:
            self.shared_up, self.shared_down = tensors[n["shared_up"]].contiguous(), tensors[n["shared_down"]].contiguous()

    def forward(self, x, ctx):
        out = torch.zeros((x.shape[0], self.hidden), dtype=torch.float32, device=x.device)
        self.forward_into(x, ctx, out)
        return out

    def forward_into(self, x, ctx, residual):
        idx, wgt = kernels.moe_route(x, self.router, self.bias, self.top, self.route_scale)
        tc = kernels.moe_tc_ok(x, self.up, self.down) and residual.stride(1) == 1
        plan = kernels.moe_plan(idx, self.n_experts, kernels.moe_tc_tile_rows(idx.numel(), self.n_experts) if tc else None)
        if tc:
            # tensor cores: the tokens' rows in slot order, the up projection with its activation, and the down
            # projection that ends in the weighted add into the stream
            act = kernels.moe_gemm_tc(kernels.moe_gather_rows(x, plan), self.up, plan, self.act, out_dtype=x.dtype)
            kernels.moe_gemm_tc(act, self.down, plan, "weighted_add", out=residual, wgt=wgt)
        else:
            act = kernels.moe_gemm(x, self.up, plan, gather=True, act=self.act, out_dtype=x.dtype)
            y = kernels.moe_gemm(act, self.down, plan, gather=False, act=None, out_dtype=torch.float32)
            kernels.moe_combine(residual, y, plan, wgt)
        if self.shared_ff:
            a = kernels.relu_squared_(kernels.linear(x, self.shared_up))
            if kernels.linear_into_ok(a, self.shared_down, None, residual):
                kernels.linear_into(a, self.shared_down, None, residual)
            else:
                kernels.residual_add(residual, kernels.linear(a, self.shared_down))
        return True
