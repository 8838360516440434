"""Attention over a cached latent: a token leaves one row [c | k_rot] in the cache, c a normed low-rank latent
from which every head's keys and values are linear maps (W_uk, W_uv), k_rot a rotated key part that all heads
share. The queries pass through a latent of their own.

Keys and values are never raised from the cache. A head's unrotated query is carried through its key map first,
q_c = W_uk[h]^T q_plain, so that the score is (q_c . c + q_rot . k_rot) * scale and the head's output is
W_uv[h] (sum_j p_j c_j): every head reads the same cached rows, once. Order of kernels: the packed down
projections [W_dq; W_dkv] (float32 out), the norms of both latents with the rotation of k_rot and the write into
the pages, the query up projection, its rotated parts and the batched product with the key maps, the attention,
the batched product with the value maps, the output projection.

``q_rank`` 0: the queries have no latent; q = W_q h (tensor 'q') rides in the packed product's place of the query
latent's up projection. ``output_gate``: the heads' values side by side are multiplied by sigmoid(W_g h) (tensor 'g'),
in the epilogue of the product with the value maps.

A layer that ``shares_cache`` has no W_dkv: it runs on the cache entry another layer writes (the run order
names it with ``writes_cache=False``) with queries, key and value maps of its own.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import CacheNeed, Mixer, TensorSpec, build_position, register_mixer


class LatentAttention(Mixer):
    graph_safe = True

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        self.position = build_position(spec.position, dtype, device)
        self._rotation = self.position.rotation()
        self.w_down = self.w_uq = self.w_uk_t = self.w_uv = self.w_o = None
        self.q_norm = self.kv_norm = self.sink = self.w_q = self.w_g = None
        if spec.q_rank < 0:
            raise ValueError("q_rank must not be negative")

    def cache_need(self):
        s = self.spec
        return CacheNeed(1, s.kv_rank + s.rot_dim, s.window, planes=1)

    def tensors(self):
        s = self.spec
        if s.q_rank:
            t = {
                "dq": TensorSpec((s.q_rank, s.hidden_size)),
                "dq.norm": TensorSpec((s.q_rank,), role="vector32", init="ones_noise"),
                "uq": TensorSpec((s.num_heads * (s.head_dim + s.rot_dim), s.q_rank)),
            }
        else:
            t = {"q": TensorSpec((s.num_heads * (s.head_dim + s.rot_dim), s.hidden_size))}
        if not s.shares_cache:
            t["dkv"] = TensorSpec((s.kv_rank + s.rot_dim, s.hidden_size))
            t["dkv.norm"] = TensorSpec((s.kv_rank,), role="vector32", init="ones_noise")
        t["uk"] = TensorSpec((s.num_heads * s.head_dim, s.kv_rank))
        t["uv"] = TensorSpec((s.num_heads * s.v_dim, s.kv_rank))
        if s.sink:
            t["sink"] = TensorSpec((s.num_heads,), role="vector32")
        if s.output_gate:
            t["g"] = TensorSpec((s.num_heads * s.v_dim, s.hidden_size))
        t["o"] = TensorSpec((s.hidden_size, s.num_heads * s.v_dim))
        return t

    def load(self, tensors):
        s = self.spec
        down = ([tensors["dq"]] if s.q_rank else []) + ([] if s.shares_cache else [tensors["dkv"]])
        self.w_down = torch.cat(down, dim=0).contiguous() if down else None
        if not s.shares_cache:
            self.kv_norm = tensors["dkv.norm"]
        if s.q_rank:
            self.q_norm = tensors["dq.norm"]
            self.w_uq = tensors["uq"].contiguous()
        else:               # one product for the queries and, behind them, the gate's logits
            self.w_q = torch.cat([tensors["q"]] + ([tensors["g"]] if s.output_gate else []), dim=0).contiguous()
        if s.output_gate and s.q_rank:
            self.w_g = tensors["g"].contiguous()
        # per head [rank, head_dim]: the key map transposed, so that q_c = w_uk_t[h] q_plain
        self.w_uk_t = tensors["uk"].view(s.num_heads, s.head_dim, s.kv_rank).transpose(1, 2).contiguous()
        self.w_uv = tensors["uv"].view(s.num_heads, s.v_dim, s.kv_rank).contiguous()
        self.w_o = tensors["o"].contiguous()
        self.sink = tensors["sink"] if s.sink else None

    def forward(self, x, step, cache):
        s = self.spec
        writes = cache.writes and not s.shares_cache
        if s.shares_cache and cache.writes:
            raise RuntimeError("a latent-attention layer without a key/value down projection cannot write a cache")
        q_latent = None
        if self.w_down is not None:
            down = ops.linear(x, self.w_down, out_float32=True)
            q_latent = ops.latent_prepare(
                down, q_rank=s.q_rank, rank=s.kv_rank, rot=s.rot_dim, q_norm_weight=self.q_norm,
                kv_norm_weight=self.kv_norm, eps=s.norm_eps, rotation=self._rotation, positions=step.positions,
                token_seq=step.token_seq, cache=cache.kv if writes else None, block_table=cache.block_table,
                dtype=self.dtype, status=step.status)
        q_width = s.num_heads * (s.head_dim + s.rot_dim)
        gate, gate_at = None, 0
        if s.q_rank:
            q = ops.linear(q_latent, self.w_uq)                   # [T, H * (head_dim + rot_dim)]
            if s.output_gate:
                gate = ops.linear(x, self.w_g)
        else:
            q = ops.linear(x, self.w_q)                           # [T, H * (head_dim + rot_dim) (+ H * v_dim gate logits)]
            if s.output_gate:
                gate, gate_at = q, q_width
        rows = torch.empty((q.shape[0], s.num_heads * (s.kv_rank + s.rot_dim)), dtype=torch.float32, device=q.device)
        ops.batched_linear(q, self.w_uk_t, x_batch_stride=s.head_dim + s.rot_dim, k=s.head_dim, out=rows,
                           out_batch_stride=s.kv_rank + s.rot_dim)
        ops.latent_query_rotate(rows, q, heads=s.num_heads, plain=s.head_dim, rot=s.rot_dim, rank=s.kv_rank,
                                rotation=self._rotation, positions=step.positions)
        mixed = ops.latent_attention(
            rows, cache.kv, heads=s.num_heads, rank=s.kv_rank, rot=s.rot_dim, scale=s.scale, sink=self.sink,
            positions=step.positions, token_seq=step.token_seq, block_table=cache.block_table,
            max_context=step.max_context, window=s.window, step=step, status=step.status)
        values = ops.batched_linear(mixed, self.w_uv, x_batch_stride=s.kv_rank, k=s.kv_rank,     # [T, H * v_dim]
                                    gate=gate, gate_offset=gate_at)
        return ops.linear(values, self.w_o)


register_mixer("latent_attention", LatentAttention)
