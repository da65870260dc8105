from __future__ import annotations

import torch

from .. import kernels
from .base import Mixer, TensorDecl, register_part


@register_part("mixer", "gated_linear_attention")
class GatedLinearAttention(Mixer):
    """A recurrent mixer with a matrix of memory per head, S [key_dim, value_dim] in float32, kept in the cache's
    fixed-size state of the sequence (zero when the sequence starts) and carried from token to token:

        q = Wq h * query_scale, k = Wk h, v = Wv h                     (heads x key_dim, heads x value_dim)
        a = sigmoid(Wa2 (Wa1 h) + b)^(1 / decay_root)                  per key channel, through a low-rank bottleneck
        S <- diag(a) S + k v^T,      o = S^T q
        out = Wo (rms_norm(o over value_dim; weight shared by heads) * silu(Wg h))

    q, k and v are one matrix product whose output stays float32 in both precisions (o is a sum with cancellation that
    a norm then scales to unit size, so rounding q, k, v to 16 bits would be magnified wherever o happens to be small);
    the output gate and the bottleneck are a second one; the decay logits leave their product in float32, and everything
    from there to o (the decay, the state, the sums) is float32.  One kernel runs the recurrence for
    whole prompts, portions and single tokens.  The bottleneck's size is the shape of `a1`.

    params: hidden_size, num_heads, key_dim, value_dim, decay_root, query_scale, eps, decay_rank (random weights only),
    names (local tensor names of q, k, v, g, o, norm, a1, a2, a2_bias).
    """
    capturable = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden, self.nh, self.dk, self.dv = int(p["hidden_size"]), int(p["num_heads"]), int(p["key_dim"]), int(p["value_dim"])
        self.root, self.q_scale, self.eps = float(p["decay_root"]), float(p.get("query_scale", 1.0)), float(p["eps"])
        if self.root <= 0:
            raise ValueError(f"the decay's root must be positive, got {self.root}")
        if self.dk > kernels.mixers.GLA_MAX_KEY_DIM:
            raise kernels.KernelError(f"gated linear attention: {self.dk} key channels a head; the kernel takes up to "
                                      f"{kernels.mixers.GLA_MAX_KEY_DIM}")
        self.rank = int(p.get("decay_rank", 16))
        self.names = dict({"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm", "a1": "a1", "a2": "a2",
                           "a2_bias": "a2.b"}, **(p.get("names") or {}))
        self.w_in = self.w_gate = self.w_a2 = self.b_a2 = self.w_norm = self.w_o = None

    def state_size(self):
        return self.nh * self.dk * self.dv

    def tensors(self):
        n, D, K, V = self.names, self.hidden, self.nh * self.dk, self.nh * self.dv
        return {n["q"]: TensorDecl((K, D)), n["k"]: TensorDecl((K, D)), n["v"]: TensorDecl((V, D)), n["g"]: TensorDecl((V, D)),
                n["o"]: TensorDecl((D, V)), n["norm"]: TensorDecl((self.dv,), init="one_plus_normal", use="vector"),
                n["a1"]: TensorDecl((self.rank, D), free=(0,)), n["a2"]: TensorDecl((K, self.rank), free=(1,)),
                n["a2_bias"]: TensorDecl((K,), use="vector")}

    def load(self, tensors):
        n = self.names
        self.rank = int(tensors[n["a1"]].shape[0])
        if tensors[n["a2"]].shape[1] != self.rank:
            raise ValueError(f"the decay's two matrices do not fit: {tuple(tensors[n['a1']].shape)} and {tuple(tensors[n['a2']].shape)}")
        def fuse(keys):
            ts = [tensors[n[k]] for k in keys]
            dt = ts[0].dtype
            for t in ts[1:]:
                dt = torch.promote_types(dt, t.dtype)
            return torch.cat([t.to(dt) for t in ts], dim=0).contiguous()

        self.w_in = fuse(("q", "k", "v"))
        self.w_gate = fuse(("g", "a1"))
        self.w_a2 = tensors[n["a2"]].contiguous()
        self.b_a2 = tensors[n["a2_bias"]].float().contiguous()
        self.w_norm = tensors[n["norm"]].contiguous()
        self.w_o = tensors[n["o"]].contiguous()

    def forward(self, x, ctx, call):
        from .mlp import delta_dtype
        V = self.nh * self.dv
        qkv = kernels.linear(x, self.w_in, out_dtype=torch.float32)                  # [T, q | k | v]
        gate = kernels.linear(x, self.w_gate)                                        # [T, g | bottleneck]
        z = kernels.linear(gate[:, V:], self.w_a2, self.b_a2, out_dtype=torch.float32)
        o = kernels.gla_scan(qkv, self.nh, self.dk, self.dv, z, ctx.state(call), ctx.seq_start, ctx.seq_slot, ctx.n_seqs,
                             self.q_scale, self.root)
        y = kernels.gla_out(o, gate[:, :V], self.w_norm, self.nh, self.dv, self.eps, x.dtype)
        return kernels.linear(y, self.w_o, out_dtype=delta_dtype(y))
