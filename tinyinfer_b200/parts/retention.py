"""Retention ("Retentive Network: A Successor to Transformer for Large Language Models", Sun et al., 2023): linear
attention with a fixed decay per head and neither softmax nor denominator. Per head a matrix state S
(key_dim x value_dim): S <- decay_h S + k v^T, o = S^T q, with q and k rotated by their positions and k scaled by
key_dim^-1/2 after the rotation. Every head's o is divided by its root mean square (no weight), the heads side by
side are multiplied by silu(W_g h) and projected.

One packed product gives [q | k | v | g]; the rotation leaves [q | k | v] as float32 rows (what enters the
recurrence is not rounded again after it); the scan is the matrix-state scan of the other linear-attention mixers
with one constant row of decays; the state is float32 and lives in the request's state slot (zero at the start).
"""
from __future__ import annotations

import torch

from .. import ops
from .base import Mixer, StateNeed, TensorSpec, build_position, register_mixer


class Retention(Mixer):
    graph_safe = True

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        if len(spec.decays) != spec.num_heads:
            raise ValueError("retention: one decay per head")
        self.position = build_position(spec.position, dtype, device)
        self._rotation = self.position.rotation()
        self.decays = torch.tensor([list(spec.decays)], dtype=torch.float32, device=device)      # [1, H]: every token's row
        self.ones = torch.ones(spec.value_dim, dtype=torch.float32, device=device)               # the norm has no weight
        self.w_in = self.w_o = None

    def state_need(self):
        s = self.spec
        return StateNeed((s.num_heads * s.key_dim * s.value_dim,), torch.float32)

    def tensors(self):
        s = self.spec
        nk, nv = s.num_heads * s.key_dim, s.num_heads * s.value_dim
        return {"q": TensorSpec((nk, s.hidden_size)), "k": TensorSpec((nk, s.hidden_size)),
                "v": TensorSpec((nv, s.hidden_size)), "g": TensorSpec((nv, s.hidden_size)),
                "o": TensorSpec((s.hidden_size, nv))}

    def load(self, tensors):
        self.w_in = torch.cat([tensors["q"], tensors["k"], tensors["v"], tensors["g"]], dim=0).contiguous()
        self.w_o = tensors["o"].contiguous()

    def _features(self, x, step, cache):
        s = self.spec
        nk, nv = s.num_heads * s.key_dim, s.num_heads * s.value_dim
        packed = ops.linear(x, self.w_in)                                            # [T, q | k | v | g]
        qkv = ops.head_rotation(packed, num_heads=s.num_heads, num_kv_heads=s.num_heads, head_dim=s.key_dim,
                                v_dim=s.value_dim, has_kv=True, positions=step.positions, token_seq=step.token_seq,
                                rotation=self._rotation, k_scale=s.key_dim ** -0.5, out_float32=True)
        state = cache.state.unflatten(1, (s.num_heads, s.value_dim, s.key_dim))
        o = ops.linear_scan(qkv, qkv, qkv, ops.ScanGate("constant", self.decays, per_channel=False), state=state,
                            heads=s.num_heads, groups=s.num_heads, key_dim=s.key_dim, value_dim=s.value_dim,
                            q_offset=0, k_offset=nk, v_offset=2 * nk, cu_seqlens=step.cu_seqlens,
                            state_slots=step.state_slots, num_seqs=step.num_seqs, max_q_len=step.max_q_len)
        return ops.gated_group_norm(o, packed, self.ones, group=s.value_dim, eps=s.norm_eps, gate_first=False,
                                    out_dtype=self.dtype, gate_offset=2 * nk + nv)

    def forward(self, x, step, cache):
        return ops.linear(self._features(x, step, cache), self.w_o)

    def forward_residual(self, x, residual, step, cache):
        return ops.linear(self._features(x, step, cache), self.w_o, residual=residual)


register_mixer("retention", Retention)
