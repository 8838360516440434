"""Mixture-of-experts feed-forward: a float32 router picks, per token, the ``top`` experts with the largest
softmax scores; their outputs are weighted by those scores over their sum; optionally a shared expert runs for
every token. An expert is down(act(up h)), act(v) = max(v, 0)^2, no biases.

The spec may change each of these: ``activation`` 'clamped_glu' (an expert has a gate and an up matrix:
g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit), down(g * sigmoid(alpha g) * (u + 1))), ``identity_experts``
(the router's last outputs stand for experts whose output is their input; they have no tensors), ``score_correction``
(a learned number per router output steers the choice, the weights stay the plain scores), ``renormalize`` False (the
weights are the chosen scores themselves) and ``router_input`` 'input' (the router reads the sublayer's normed input
instead of the float32 stream), ``activation`` 'silu_glu' (down(silu(W_gate h) * (W_up h))), ``scoring`` 'sigmoid' (an
expert's score is the sigmoid of its own router logit) and ``weight_input`` (a chosen expert runs on its weight times
the token's row, expert(w h), and the outputs are summed as they are: the up product is linear, W (w h) = w (W h), so
the weight multiplies both halves of the stored product inside the activation kernel and costs no pass of its own).

A step's (token, choice) pairs are put in expert order on the device and the experts run as two grouped
products over row tiles; nothing is read back to the host and no token is ever dropped, so a token's result
does not depend on what else is in the batch. The part sits in blocks whose norm follows the sublayer
(``forward_stream``): the weighted sum, the shared expert's term, the norm and the float32 residual sum are
one kernel.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, TensorSpec, register_feed_forward


class Experts(FeedForward):
    graph_safe = True

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        if spec.activation not in ("relu_squared", "clamped_glu", "silu_glu"):
            raise ValueError(f"activation {spec.activation!r} is not supported (relu_squared, clamped_glu, silu_glu)")
        if spec.scoring not in ("softmax", "sigmoid"):
            raise ValueError(f"scoring {spec.scoring!r} is not supported (softmax, sigmoid)")
        if spec.weight_input and (spec.activation != "silu_glu" or spec.identity_experts or spec.shared_size):
            raise ValueError("experts weighted at their input are silu-gated ones, without identity or shared experts")
        if spec.activation == "clamped_glu" and not spec.glu_limit > 0:
            raise ValueError("clamped_glu needs a positive limit")
        if spec.identity_experts < 0 or spec.top > spec.num_experts + spec.identity_experts:
            raise ValueError("top exceeds the number of router outputs")
        if spec.shared_size and spec.activation != "relu_squared":
            raise ValueError("a shared expert is built with the relu_squared activation only")
        self.glu = spec.activation in ("clamped_glu", "silu_glu")
        self.w_router = self.w_up = self.w_down = self.w_shared_up = self.w_shared_down = self.correction = None

    def tensors(self):
        s = self.spec
        t = {}
        for e in range(s.num_experts):
            if self.glu:
                t[f"e{e}.gate"] = TensorSpec((s.expert_size, s.hidden_size))
            t[f"e{e}.up"] = TensorSpec((s.expert_size, s.hidden_size))
            t[f"e{e}.down"] = TensorSpec((s.hidden_size, s.expert_size))
        t["router"] = TensorSpec((s.num_experts + s.identity_experts, s.hidden_size))
        if s.score_correction:
            t["correction"] = TensorSpec((s.num_experts + s.identity_experts,), role="vector32")
        if s.shared_size:
            t["shared.up"] = TensorSpec((s.shared_size, s.hidden_size))
            t["shared.down"] = TensorSpec((s.hidden_size, s.shared_size))
        return t

    def load(self, tensors):
        s = self.spec
        if self.glu:       # an expert's rows: [gate | up], one grouped product for both
            self.w_up = torch.stack([torch.cat([tensors[f"e{e}.gate"], tensors[f"e{e}.up"]], dim=0)
                                     for e in range(s.num_experts)]).contiguous()
        else:
            self.w_up = torch.stack([tensors[f"e{e}.up"] for e in range(s.num_experts)]).contiguous()
        if s.score_correction:
            self.correction = tensors["correction"].contiguous()
        self.w_down = torch.stack([tensors[f"e{e}.down"] for e in range(s.num_experts)]).contiguous()
        self.w_router = tensors["router"].contiguous()
        if s.shared_size:
            self.w_shared_up = tensors["shared.up"].contiguous()
            self.w_shared_down = tensors["shared.down"].contiguous()

    def _experts(self, x32, x):
        """(routing, float32 sorted rows of the experts' outputs, the shared expert's output or None)."""
        s = self.spec
        # the more rows an expert gets, the taller the row tiles its grouped products are planned with
        routing = ops.route_experts(x32, self.w_router, s.top, s.weight_eps,
                                    tile_rows=ops.expert_tile_rows(x, s.num_experts, s.top, s.expert_size),
                                    correction=self.correction, renormalize=s.renormalize, real_experts=s.num_experts,
                                    scoring=s.scoring)
        if self.glu:
            gate_up = ops.expert_linear(x, self.w_up, routing, up=True, activation=False)
            hidden = (ops.silu_glu(gate_up, routing.slot_weight if s.weight_input else None) if s.activation == "silu_glu"
                      else ops.clamped_glu(gate_up, s.glu_limit, s.glu_alpha))
        else:
            hidden = ops.expert_linear(x, self.w_up, routing, up=True)
        down = ops.expert_linear(hidden, self.w_down, routing, up=False)
        shared = None
        if s.shared_size:
            shared = ops.linear(ops.relu_squared(ops.linear(x, self.w_shared_up)), self.w_shared_down)
        return routing, down, shared

    def forward_stream(self, x32, x, norm, step):
        """x32 += norm(feed_forward(x)) for a float32 stream ``x32`` with its copy ``x`` in the compute dtype;
        returns the new (x32, copy). The router reads the float32 rows."""
        rms = norm.as_rms()
        if rms is None:
            raise ValueError("the experts' fused output needs an RMSNorm behind them")
        if self.spec.identity_experts or self.spec.weight_input:
            raise ValueError("identity experts and experts weighted at their input are not built into the fused output "
                             "of this arrangement")
        routing, down, shared = self._experts(x if self.spec.router_input == "input" else x32, x)
        return ops.experts_combine_norm_add(x32, down, shared, routing, rms[0], rms[1], self.dtype)

    def forward(self, x, step=None):
        """The plain weighted sum in the compute dtype, for arrangements whose residual work is not the experts'
        business. The router reads ``x`` (its logits are float32 all the same)."""
        s = self.spec
        if s.identity_experts and s.router_input != "input":
            raise ValueError("identity experts pass the sublayer's input on, which is also what the router must read")
        routing, down, shared = self._experts(x if s.router_input == "input" or x.dtype == torch.float32 else x.float(), x)
        out = ops.experts_combine(down, x, routing, s.num_experts, weighted=not s.weight_input)
        if shared is not None:
            out = ops.add(out, shared)
        return out


register_feed_forward("experts", Experts)
