"""A routed feed-forward (mixture of experts): every token is sent to the `top` experts whose router logits
z = W_r h + b are largest and gets sum_e softmax(z over the chosen)_e * expert_e(h); an optional shared
feed-forward (any registered kind) runs for every token and is added.  An expert is a gated feed-forward
down(act(gate(h)) * up(h)) without biases.

A second way of routing, `scores="softmax_all"`: s = softmax(z) over ALL the router's outputs; the choice is made by
s + correction (a stored vector that moves the choice and not the weights), restricted to the outputs of the
`keep_groups` best of `groups` equal groups of neighbouring outputs (a group's score is its largest choice score);
the weights are the chosen s times `route_scale`, not renormalised.  The router's last `identity` outputs are
identity experts: they have no matrices and return the token itself (times the weight).  With `shared_gate_name`
the shared feed-forward's output is multiplied by sigmoid(w . h), one number per token; w is a stored [1, hidden]
matrix that rides as one more row of the router's matrix.

Nothing of a step comes back to the host: the router kernel leaves the assignments on the device, a plan
kernel orders them by expert, and two grouped matrix products (gate and up with the activation on their
accumulators, then down) walk the row tiles of that order; see `csrc/moe.cu`.  The router's matrix is held and
applied in float32 whatever the engine's element type.  The experts' matrices are stacked at bind time:
[experts, 2 * inner, hidden] with gate and up rows in tiles of 8 (as `GatedMLP` does for one matrix), and
[experts, hidden, inner].
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from ..csrc import ops
from .base import FeedForward, Runtime, TensorSpec
from .mlp import GATE_TILE
from .plan import PartSpec
from .registry import build_part


class RoutedExperts(FeedForward):
    @property
    def cuda_graph_safe(self) -> bool:
        return self.shared is None or bool(self.shared.cuda_graph_safe)

    def __init__(self, prefix: str, hidden_size: int, experts: int, top: int, intermediate_size: int,
                 activation: str = "silu", router_bias: bool = True, shared: Optional[PartSpec] = None,
                 router_names: Sequence[str] = ("router", "router.b"), expert_prefix: str = "e%d.",
                 names: Sequence[str] = ("gate", "up", "down"), scores: str = "softmax_chosen",
                 correction_name: Optional[str] = None, groups: int = 1, keep_groups: int = 1, route_scale: float = 1.0,
                 identity: int = 0, shared_gate_name: Optional[str] = None):
        super().__init__(prefix)
        self.hidden_size, self.experts, self.top = int(hidden_size), int(experts), int(top)
        self.intermediate_size = int(intermediate_size)
        self.identity, self.groups, self.keep_groups = int(identity), int(groups), int(keep_groups)
        self.outputs = self.experts + self.identity   # what the router chooses among
        self.scores, self.route_scale = scores, float(route_scale)
        if scores not in ("softmax_chosen", "softmax_all"):
            raise ValueError("%sscores %r is not one of softmax_chosen, softmax_all" % (prefix, scores))
        if scores == "softmax_chosen" and (correction_name or self.groups != 1 or self.route_scale != 1.0):
            raise ValueError("%sa correction, groups and a multiplier of the weights go with scores='softmax_all'" % prefix)
        if self.experts <= 0 or self.identity < 0 or not 0 < self.top <= self.outputs:
            raise ValueError("%stop %d of %d experts and %d identity experts" % (prefix, self.top, self.experts, self.identity))
        if self.groups < 1 or self.outputs % self.groups or not 1 <= self.keep_groups <= self.groups \
                or self.top > self.keep_groups * (self.outputs // self.groups):
            raise ValueError("%s%d outputs in %d groups of which %d are kept cannot give %d choices"
                             % (prefix, self.outputs, self.groups, self.keep_groups, self.top))
        if shared_gate_name and shared is None:
            raise ValueError("%sa shared gate needs a shared feed-forward" % prefix)
        self.correction_name = prefix + correction_name if correction_name else None
        self.shared_gate_name = prefix + shared_gate_name if shared_gate_name else None
        self.correction = None
        if activation not in ops.ACTIVATIONS:
            raise ValueError("activation %r is not one of %s" % (activation, sorted(ops.ACTIVATIONS)))
        self.activation, self.router_bias = activation, bool(router_bias)
        self.router_name, self.bias_name = prefix + router_names[0], prefix + router_names[1]
        self.expert_names = [tuple(prefix + expert_prefix % e + n for n in names) for e in range(self.experts)]
        self.shared = build_part("feed_forward", shared) if shared is not None else None
        self.router = self.bias = self.gate_up = self.down = None

    def tensor_specs(self) -> List[TensorSpec]:
        e, i = self.hidden_size, self.intermediate_size
        specs = [TensorSpec(self.router_name, (self.outputs, e), "matrix_f32")]
        if self.router_bias:
            specs.append(TensorSpec(self.bias_name, (self.outputs,), "bias"))
        if self.correction_name:
            specs.append(TensorSpec(self.correction_name, (self.outputs,), "bias"))
        if self.shared_gate_name:
            specs.append(TensorSpec(self.shared_gate_name, (1, e), "matrix_f32"))
        for gate, up, down in self.expert_names:
            specs += [TensorSpec(gate, (i, e), "matrix"), TensorSpec(up, (i, e), "matrix"), TensorSpec(down, (e, i), "matrix")]
        return specs + (self.shared.tensor_specs() if self.shared is not None else [])

    def ignored_tensors(self) -> List[str]:
        return self.shared.ignored_tensors() if self.shared is not None else []

    def bind(self, tensors: Dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(tensors, runtime)
        e, i = self.hidden_size, self.intermediate_size
        self.router = tensors[self.router_name]
        if self.shared_gate_name:   # (the shared gate's vector: one more row for the router kernel)
            self.router = torch.cat([self.router, tensors[self.shared_gate_name].to(torch.float32).view(1, e)], 0).contiguous()
        self.bias = tensors[self.bias_name] if self.router_bias else None
        self.correction = tensors[self.correction_name].to(torch.float32).contiguous() if self.correction_name else None
        self.tile = GATE_TILE if i % GATE_TILE == 0 else 0
        self.gate_up = torch.empty((self.experts, 2 * i, e), dtype=runtime.dtype, device=runtime.device)
        self.down = torch.empty((self.experts, e, i), dtype=runtime.dtype, device=runtime.device)
        for x, (gate, up, down) in enumerate(self.expert_names):
            g, u = tensors[gate], tensors[up]
            if self.tile:
                self.gate_up[x] = torch.stack([g.view(i // GATE_TILE, GATE_TILE, e), u.view(i // GATE_TILE, GATE_TILE, e)],
                                              1).reshape(2 * i, e)
            else:
                self.gate_up[x, :i], self.gate_up[x, i:] = g, u
            self.down[x] = tensors[down]
        if self.shared is not None:
            self.shared.bind(tensors, runtime)

    def _route(self, h: torch.Tensor, tile_rows: int):
        return ops.moe_route(h, self.router, self.bias, self.outputs, self.top, tile_rows, scores=self.scores,
                             correction=self.correction, groups=self.groups, keep_groups=self.keep_groups,
                             route_scale=self.route_scale, identity=self.identity,
                             shared_gate=self.shared_gate_name is not None)

    def forward(self, h: torch.Tensor, ctx=None) -> torch.Tensor:
        i, e = self.intermediate_size, self.hidden_size
        if self.tile and ops.moe_tcgen05_supported(h, h.shape[0] * self.top, 2 * i, e) and i % 8 == 0 and e % 16 == 0:
            # a prompt portion: the tokens' rows are copied into expert order once, and both grouped products run on
            # the tcgen05 tensor cores over row tiles of 128 (operands by TMA, the activation on the accumulators)
            plan = self._route(h, ops.MOE_TCGEN05_TILE_ROWS)
            a = ops.moe_gemm_tcgen05(ops.moe_gather_rows(h, plan), self.gate_up, plan, gated_activation=self.activation)
            y = ops.moe_gemm_tcgen05(a, self.down, plan)
            shared = self.shared.forward(h, ctx) if self.shared is not None else None
            return ops.moe_combine(y, plan, shared, h.dtype, h=h)
        # (a decode step's few rows per expert: row tiles of 16; the second product reads rows of `inner` elements)
        rows = ops.moe_tile_rows(h, h.shape[0] * self.top) if i % 8 == 0 else ops.MOE_TILE_ROWS
        plan = self._route(h, rows)
        if self.tile:
            a = ops.moe_gemm(h, self.gate_up, plan, True, h.dtype, gated_activation=self.activation)
        else:
            # an inner size that is no multiple of 8: all gates, then all ups; the activation by a kernel of its own
            a = ops.gated_act(ops.moe_gemm(h, self.gate_up, plan, True, torch.float32), self.activation, 0, out_dtype=h.dtype)
        y = ops.moe_gemm(a, self.down, plan, False, torch.float32)
        shared = self.shared.forward(h, ctx) if self.shared is not None else None
        return ops.moe_combine(y, plan, shared, h.dtype, h=h)
