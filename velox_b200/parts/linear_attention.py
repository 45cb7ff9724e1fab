"""Linear attention with a fixed decay per head, as a recurrence: per head a state S [dim, vdim] with
S_p = decay * S_(p-1) + k_p v_p^T and o_p = S_p^T q_p, where q, k = act(W_q h), act(W_k h) and v = act(W_v h).
The heads' outputs are joined, RMS-normed over their whole width with a weight, multiplied by sigmoid(W_g h)
and projected by W_o.  There is no other scale and no position encoding.

The state is float32, starts at zero and lives in the request's state slot (`FixedState`), so a step runs
only the tokens it brings.  The four input projections are one matrix here ([W_q; W_k; W_v; W_g]).  Three
kernels share the work (`ops.linear_attention`, `csrc/linear_attention.cu`): the recurrence token by token
(decode steps, short portions, float32), chunks of 64 tokens on the tensor cores one after the other, and, for
portions of 256 tokens or more, all chunks side by side with a scan between them.  The activation of q, k, v
is taken in float32 (rounded to bfloat16 in a bfloat16 engine, the same way by every kernel).  Decays, state,
outputs, the norm and the gate are float32.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from ..csrc import ops
from .base import FixedState, Mixer, Runtime, TensorSpec
from .linear import Linear


class DecayedLinearAttention(Mixer):
    cuda_graph_safe = True  # reads nothing of a step but device tensors and sizes fixed per graph

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, head_dim: int, v_head_dim: int,
                 decay: Sequence[float], eps: float = 1e-6, activation: str = "silu",
                 names: Sequence[str] = ("q", "k", "v", "g", "o", "norm")):
        super().__init__(prefix)
        self.hidden_size, self.num_heads = int(hidden_size), int(num_heads)
        self.head_dim, self.v_head_dim, self.eps = int(head_dim), int(v_head_dim), float(eps)
        self.decay_values = [float(d) for d in decay]
        if len(self.decay_values) != self.num_heads:
            raise ValueError("%s%d decays for %d heads" % (prefix, len(self.decay_values), self.num_heads))
        if activation not in ("silu", "none"):
            raise ValueError("%sthe recurrence kernel applies silu or nothing to q, k, v; got %r" % (prefix, activation))
        if not 0 < self.head_dim <= ops.LINEAR_ATTENTION_MAX_DIM:
            raise ValueError("%shead_dim %d: the recurrence kernel takes up to %d" % (prefix, head_dim, ops.LINEAR_ATTENTION_MAX_DIM))
        self.activation = activation
        self.names = dict(zip(("q", "k", "v", "g", "o", "norm"), (prefix + n for n in names)))
        self.proj: Optional[Linear] = None
        self.out: Optional[Linear] = None
        self.norm_weight = self.decay = None

    def tensor_specs(self) -> List[TensorSpec]:
        e, qk, vv = self.hidden_size, self.num_heads * self.head_dim, self.num_heads * self.v_head_dim
        n = self.names
        return [TensorSpec(n["q"], (qk, e), "matrix"), TensorSpec(n["k"], (qk, e), "matrix"),
                TensorSpec(n["v"], (vv, e), "matrix"), TensorSpec(n["g"], (vv, e), "matrix"),
                TensorSpec(n["o"], (e, vv), "matrix"), TensorSpec(n["norm"], (vv,), "norm")]

    def bind(self, tensors: Dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(tensors, runtime)
        n = self.names
        self.proj = Linear(torch.cat([tensors[n[x]] for x in ("q", "k", "v", "g")], dim=0).contiguous())
        self.out = Linear(tensors[n["o"]])
        self.norm_weight = tensors[n["norm"]]
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=runtime.device)

    def cache_spec(self):
        return FixedState((self.num_heads, self.head_dim, self.v_head_dim), "float32")

    def forward(self, h: torch.Tensor, ctx, cache) -> torch.Tensor:
        H, D, Dv = self.num_heads, self.head_dim, self.v_head_dim
        x = self.proj(h)   # [tokens, q | k | v | g]
        o = ops.linear_attention(x, 0, H * D, 2 * H * D, self.decay, cache.state, ctx.cu_seqlens, ctx.state_slots,
                                 ctx.n_seqs, ctx.max_new, H, D, Dv, silu=self.activation == "silu")
        y = ops.gated_rmsnorm(o, x[:, 2 * H * D + H * Dv:], self.norm_weight, self.eps)
        return self.out(y)
