"""The gated delta rule with a decay per head and key channel ("Gated Delta Networks: Improving Mamba2 with Delta
Rule", Yang, Kautz and Hatamizadeh, 2024, with the scalar decay made channel-wise). q and k (kv heads of key_dim) and
v (heads of value_dim) pass a short causal convolution per channel and silu; q and k become unit vectors per head, q
also times key_dim^-1/2; beta = sigmoid(W_b h) per head; g = exp(-exp(A_log) softplus(W_a2 (W_a1 h) + dt_bias)) per
head and key channel. Per head, for every token in order:
    S <- diag(g) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
so the read-out sees the token's own write. Every head's o is divided by its root mean square, weighted by one
weight shared by the heads, gated by sigmoid(W_g2 (W_g1 h)) and projected.

Float32: the convolution's arithmetic, the unit vectors, beta, the decay's logits (their product leaves its kernel
unrounded), softplus and exponentials, the state, the recurrence, its outputs and their norm. The state slot of a
request holds S (transposed, [heads, value_dim, key_dim]) and behind it the convolution's last taps - 1 inputs.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import Mixer, StateNeed, TensorSpec, register_mixer, state_slices


class ChannelDelta(Mixer):
    graph_safe = True

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError("channel_delta: heads must be a multiple of kv_heads")
        if spec.conv_taps < 1:
            raise ValueError("channel_delta: the convolution has at least one tap")
        self.w_qkv = self.w_low = self.w_a2 = self.w_g2 = self.w_b = self.w_o = None
        self.conv_w = self.a_log = self.dt_bias = self.norm_w = None

    # convolved channels: [q | k | v]
    @property
    def _sizes(self):
        s = self.spec
        return s.num_kv_heads * s.key_dim, s.num_kv_heads * s.key_dim, s.num_heads * s.value_dim

    def _state_shapes(self):
        s = self.spec
        shapes = [(s.num_heads, s.value_dim, s.key_dim)]
        return shapes + [(s.conv_taps - 1, sum(self._sizes))] if s.conv_taps > 1 else shapes

    def state_need(self):
        s = self.spec
        return StateNeed((s.num_heads * s.value_dim * s.key_dim + (s.conv_taps - 1) * sum(self._sizes),), torch.float32)

    def tensors(self):
        s = self.spec
        nq, nk, nv = self._sizes
        rank = s.gate_rank if s.gate_rank > 0 else -1
        return {"q": TensorSpec((nq, s.hidden_size)), "q.conv": TensorSpec((nq, s.conv_taps), role="vector32", init="ones_noise"),
                "k": TensorSpec((nk, s.hidden_size)), "k.conv": TensorSpec((nk, s.conv_taps), role="vector32", init="ones_noise"),
                "v": TensorSpec((nv, s.hidden_size)), "v.conv": TensorSpec((nv, s.conv_taps), role="vector32", init="ones_noise"),
                "b": TensorSpec((s.num_heads, s.hidden_size)),
                "A_log": TensorSpec((s.num_heads,), role="vector32"),
                "norm": TensorSpec((s.value_dim,), role="vector32", init="ones_noise"),
                "a1": TensorSpec((rank, s.hidden_size)), "a2": TensorSpec((s.num_heads * s.key_dim, rank)),
                "dt_bias": TensorSpec((s.num_heads * s.key_dim,), role="vector32"),
                "g1": TensorSpec((rank, s.hidden_size)), "g2": TensorSpec((nv, rank)),
                "o": TensorSpec((s.hidden_size, nv))}

    def load(self, tensors):
        if tensors["a1"].shape[0] != tensors["a2"].shape[1] or tensors["g1"].shape[0] != tensors["g2"].shape[1]:
            raise ValueError("the two projections of the decay, or of the gate, do not fit each other")
        self.w_qkv = torch.cat([tensors["q"], tensors["k"], tensors["v"]], dim=0).contiguous()
        self.w_a1, self.w_a2 = tensors["a1"].contiguous(), tensors["a2"].contiguous()
        self.w_g1, self.w_g2 = tensors["g1"].contiguous(), tensors["g2"].contiguous()
        self.w_b = tensors["b"].contiguous()
        # tap by tap, [taps, channels]: neighbouring channels are neighbours in memory, as the kernel reads them
        self.conv_w = torch.cat([tensors["q.conv"], tensors["k.conv"], tensors["v.conv"]], dim=0).t().contiguous()
        self.a_log, self.dt_bias, self.norm_w = tensors["A_log"], tensors["dt_bias"], tensors["norm"]
        self.w_o = tensors["o"].contiguous()

    def _features(self, x, step, cache):
        s = self.spec
        nq, nk, nv = self._sizes
        width = nq + nk + nv
        qkv = ops.linear(x, self.w_qkv)                                               # [T, q | k | v] before the convolution
        decay = ops.linear(ops.linear(x, self.w_a1), self.w_a2, out_float32=True)     # float32 [T, heads * key_dim]
        beta = ops.linear(x, self.w_b, out_float32=True)                              # float32 [T, heads]
        gate = ops.linear(ops.linear(x, self.w_g1), self.w_g2)                        # [T, heads * value_dim]
        state, history = (state_slices(cache.state, self._state_shapes()) + [None])[:2]
        single = step.num_tokens == step.num_seqs          # every request brings one token: the kernel keeps the history itself
        conv = ops.short_conv(qkv, offset=0, width=width, history=history, weight=self.conv_w, bias=None, silu=True,
                              token_seq=step.token_seq, cu_seqlens=step.cu_seqlens, state_slots=step.state_slots,
                              shift_history=single)
        if not single:
            ops.conv_state_update(history, qkv, offset=0, width=width, taps=s.conv_taps, cu_seqlens=step.cu_seqlens,
                                  state_slots=step.state_slots, num_seqs=step.num_seqs)
        o = ops.delta_scan(conv, conv, conv, decay, beta, a_log=self.a_log, dt_bias=self.dt_bias, state=state,
                           heads=s.num_heads, groups=s.num_kv_heads, key_dim=s.key_dim, value_dim=s.value_dim,
                           q_offset=0, k_offset=nq, v_offset=nq + nk, q_scale=s.key_dim ** -0.5, unit_eps=s.unit_eps,
                           cu_seqlens=step.cu_seqlens, state_slots=step.state_slots, num_seqs=step.num_seqs)
        return ops.gated_group_norm(o, gate, self.norm_w, group=s.value_dim, eps=s.norm_eps, gate_first=False,
                                    out_dtype=self.dtype, gate_activation="sigmoid")

    def forward(self, x, step, cache):
        return ops.linear(self._features(x, step, cache), self.w_o)

    def forward_residual(self, x, residual, step, cache):
        return ops.linear(self._features(x, step, cache), self.w_o, residual=residual)


register_mixer("channel_delta", ChannelDelta)
