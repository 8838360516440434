"""Grouped-query attention mixer over the paged cache.

Order of operations as in the reference (tinyinfer/models/qwen3.py:106-132): packed q/k/v
projection, per-head RMSNorm of q and k, rotation, append of k and v to the cache, attention of
every token over its own request's keys, output projection. The q, k and v matrices are packed
row-wise as [q; k; v] like the reference's loader does (tinyinfer/utils/loader.py:52-96).

Beyond the reference's layer the spec may ask for: values of another size than the keys (``v_dim``), a rotation of
only the first features of a head, a learned sink per query head in the softmax denominator (``head_sinks``), an
output gate sigmoid(W_g x)_h per (token, head) (``head_gate``: W_g's rows ride in the packed projection), and a
layer without key/value tensors that reads what another layer cached (``shares_cache``), biases on q, k and v alone
(``qkv_bias``), scores capped smoothly by a tanh (``softcap``) and q and k divided by their root mean square after the
rotation (``qk_unit_norm``); these may be combined with a window. Such a layer runs
``_attend_general``: packed product [q | k | v | g], per-head norm + rotation + append (``ops.head_rotation``),
attention with the sinks and the gate in its epilogue.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import CacheNeed, Mixer, TensorSpec, build_position, register_mixer


class Attention(Mixer):
    graph_safe = True

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        self.position = build_position(spec.position, dtype, device)
        self._rotation = self.position.rotation()      # opaque here: the kernel reads it
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = None
        self.q_norm = self.k_norm = self.sinks = None
        self._general = bool(spec.value_dim != spec.head_dim or spec.head_sinks or spec.head_gate or spec.shares_cache
                             or spec.qkv_bias or spec.softcap or spec.qk_unit_norm is not None
                             or getattr(spec.position, "interleaved", False) or getattr(spec.position, "blend", None))
        if self._general and spec.bias:
            raise ValueError("biases on all four projections are not combined with value sizes, sinks, gates or shared caches")
        if spec.qk_unit_norm is not None and spec.qk_norm is not None:
            raise ValueError("q and k are normed before the rotation or after it, not both")
        if spec.qkv_bias and (spec.bias or spec.shares_cache or not spec.short_names):
            raise ValueError("biases on q, k and v alone come with short tensor names and key/value tensors of the layer's own")
        short = spec.short_names
        self._n = {"q": "q" if short else "q_proj.weight", "k": "k" if short else "k_proj.weight",
                   "v": "v" if short else "v_proj.weight", "o": "o" if short else "o_proj.weight",
                   "q_norm": "q.norm" if short else "q_norm.weight", "k_norm": "k.norm" if short else "k_norm.weight",
                   "sink": "sink" if short else "sinks", "g": "g" if short else "g_proj.weight"}

    def cache_need(self):
        s = self.spec
        if s.value_dim != s.head_dim:       # keys and values of different sizes lie side by side in one row a token
            return CacheNeed(s.num_kv_heads, s.head_dim + s.value_dim, s.window, planes=1)
        return CacheNeed(s.num_kv_heads, s.head_dim, s.window)

    def tensors(self):
        s, n = self.spec, self._n
        t = {n["q"]: TensorSpec((s.q_size, s.hidden_size))}
        if not s.shares_cache:
            t[n["k"]] = TensorSpec((s.kv_size, s.hidden_size))
            t[n["v"]] = TensorSpec((s.num_kv_heads * s.value_dim, s.hidden_size))
        t[n["o"]] = TensorSpec((s.hidden_size, s.num_heads * s.value_dim))
        if s.qk_norm is not None:
            t[n["q_norm"]] = TensorSpec((s.head_dim,), role="vector32", init="ones_noise")
            if not s.shares_cache:
                t[n["k_norm"]] = TensorSpec((s.head_dim,), role="vector32", init="ones_noise")
        if s.head_sinks:
            t[n["sink"]] = TensorSpec((s.num_heads,), role="vector32")
        if s.head_gate:
            t[n["g"]] = TensorSpec((s.num_heads, s.hidden_size))
        if s.qkv_bias:
            t[n["q"] + ".b"] = TensorSpec((s.q_size,), role="vector32")
            t[n["k"] + ".b"] = TensorSpec((s.kv_size,), role="vector32")
            t[n["v"] + ".b"] = TensorSpec((s.num_kv_heads * s.value_dim,), role="vector32")
        if s.bias:
            t["q_proj.bias"] = TensorSpec((s.q_size,), role="vector32")
            t["k_proj.bias"] = TensorSpec((s.kv_size,), role="vector32")
            t["v_proj.bias"] = TensorSpec((s.kv_size,), role="vector32")
            t["o_proj.bias"] = TensorSpec((s.hidden_size,), role="vector32")
        return t

    def load(self, tensors):
        s, n = self.spec, self._n
        rows = [tensors[n["q"]]] + ([] if s.shares_cache else [tensors[n["k"]], tensors[n["v"]]])
        if s.head_gate:
            rows.append(tensors[n["g"]])                 # the gate's rows follow q, k and v
        if self._general:
            # zero rows fill the packed matrix up to a multiple of eight rows, which the tensor-core product wants
            # of its output's row length
            fill = (-sum(r.shape[0] for r in rows)) % 8
            if fill:
                rows.append(rows[0].new_zeros((fill, rows[0].shape[1])))
        self.w_qkv = torch.cat(rows, dim=0).contiguous()
        self.w_o = tensors[n["o"]].contiguous()
        if s.qk_norm is not None:
            self.q_norm = tensors[n["q_norm"]]
            self.k_norm = None if s.shares_cache else tensors[n["k_norm"]]
        if s.head_sinks:
            self.sinks = tensors[n["sink"]].contiguous()
        if s.qkv_bias:              # zeros under the gate's and the filling rows
            bias = torch.cat([tensors[n["q"] + ".b"], tensors[n["k"] + ".b"], tensors[n["v"] + ".b"]])
            self.b_qkv = torch.cat([bias, bias.new_zeros(self.w_qkv.shape[0] - bias.shape[0])]).contiguous()
        if s.bias:
            self.b_qkv = torch.cat([tensors["q_proj.bias"], tensors["k_proj.bias"],
                                    tensors["v_proj.bias"]]).contiguous()
            self.b_o = tensors["o_proj.bias"]

    def _attend_general(self, x, step, cache):
        s = self.spec
        own = not s.shares_cache
        if own != bool(cache.writes):
            raise ValueError("a layer with key/value tensors writes its cache entry; one without them only reads")
        packed = ops.linear(x, self.w_qkv, bias=self.b_qkv)  # [T, q | (k | v) | (g) | fill]
        gate_at = s.q_size + ((s.kv_size + s.num_kv_heads * s.value_dim) if own else 0)
        q = ops.head_rotation(packed, num_heads=s.num_heads, num_kv_heads=s.num_kv_heads, head_dim=s.head_dim,
                              v_dim=s.value_dim, has_kv=own, positions=step.positions, token_seq=step.token_seq,
                              q_norm_weight=self.q_norm, k_norm_weight=self.k_norm,
                              eps=(s.qk_norm.eps if s.qk_norm is not None else s.qk_unit_norm or 0.0),
                              rotation=self._rotation, norm_after=s.qk_unit_norm is not None,
                              cache=cache.kv if own else None, block_table=cache.block_table, status=step.status)
        extras = dict(head_sinks=self.sinks, gate=packed if s.head_gate else None, gate_offset=gate_at,
                      window=s.window, softcap=s.softcap or 0.0)
        if cache.kv.shape[0] == 2:          # keys and values of one size: the paged attention, tensor cores where the sizes allow
            return ops.paged_attention(q, cache.kv, positions=step.positions, token_seq=step.token_seq,
                                       block_table=cache.block_table, scale=s.scale, step=step, status=step.status,
                                       **extras)
        return ops.attention_rows(q, cache.kv, v_dim=s.value_dim, positions=step.positions, token_seq=step.token_seq,
                                  block_table=cache.block_table, scale=s.scale, step=step, status=step.status, **extras)

    def _attend(self, x, step, cache, link=None, link_eps=0.0):
        s = self.spec
        if self._general:
            if link is not None:
                raise ValueError("this attention layer takes its input normed")
            return self._attend_general(x, step, cache)
        qkv = (ops.linear(x, self.w_qkv, bias=self.b_qkv) if link is None
               else ops.linear(x, self.w_qkv, bias=self.b_qkv, link=link, link_eps=link_eps))
        q = ops.qk_norm_rope_append(
            qkv, num_heads=s.num_heads, num_kv_heads=s.num_kv_heads, head_dim=s.head_dim,
            q_norm_weight=self.q_norm, k_norm_weight=self.k_norm,
            eps=s.qk_norm.eps if s.qk_norm is not None else 0.0,
            rotation=self._rotation, positions=step.positions, token_seq=step.token_seq,
            kv_cache=cache.kv if cache.writes else None, block_table=cache.block_table,
            status=step.status)
        return ops.paged_attention(q, cache.kv, positions=step.positions, token_seq=step.token_seq,
                                   block_table=cache.block_table, scale=s.scale, window=s.window,
                                   step=step, status=step.status)

    def forward(self, x, step, cache):
        return ops.linear(self._attend(x, step, cache), self.w_o, bias=None if self._general else self.b_o)

    def forward_residual(self, x, residual, step, cache):
        return ops.linear(self._attend(x, step, cache), self.w_o, bias=self.b_o, residual=residual)

    def forward_prenorm(self, x, norm, link, next_norm, step, cache):
        rms = norm.as_rms()
        if rms is None or self._general or not ops.norm_link_ok(x):
            return super().forward_prenorm(x, norm, link, next_norm, step, cache)
        # few tokens: the packed projection takes the norm's second half (if the product before left the
        # first), and the output projection leaves the first half of the norm that follows
        if link is not None and link.weight is rms[0]:
            attended = self._attend(link.scaled, step, cache, link=link, link_eps=rms[1])
        else:
            attended = self._attend(norm.forward(x), step, cache)
        after = next_norm.as_rms() if next_norm is not None else None
        if after is None:
            return ops.linear(attended, self.w_o, bias=self.b_o, residual=x), None
        return ops.linear(attended, self.w_o, bias=self.b_o, residual=x, next_norm_weight=after[0])


register_mixer("attention", Attention)
