"""Block arrangements. 'pre_norm' is the reference's decoder layer
(tinyinfer/models/qwen3.py:192-221): x += mixer(norm(x)); x += feed_forward(norm(x)).
The residual sums are left to the parts' last kernels where they can fuse them."""
from __future__ import annotations

from .base import Block, register_block


class PreNormBlock(Block):
    def forward(self, x, step, cache):
        return self.forward_linked(x, None, None, step, cache)[0]

    def forward_linked(self, x, link, next_norm, step, cache):
        # each part gets its input before the norm, with the norm and with the norm that comes after it:
        # parts whose products can share a norm between them do so (a decode step saves the norm kernels)
        x, link = self.mixer.forward_prenorm(x, self.mixer_norm, link, self.feed_forward_norm, step, cache)
        x, link = self.feed_forward.forward_prenorm(x, self.feed_forward_norm, link, next_norm, step)
        return x, link


class OutputNormBlock(Block):
    """x <- x + norm1(mixer(x)); x <- x + norm2(feed_forward(x)): both sublayers read x itself and the norm sits on
    a sublayer's OUTPUT. The stream is a pair (x32, copy): the residual sums are float32, ``copy`` is their
    rounding in the compute dtype, which the matrix products read (the same tensor in a float32 model).
    A block may have no feed-forward."""

    def forward(self, x, step, cache):
        return self.forward_linked(x, None, None, step, cache)[0]

    def forward_linked(self, x, link, next_norm, step, cache):
        from .. import ops
        x32, copy = x
        rms = self.mixer_norm.as_rms()
        if rms is None:
            raise ValueError("the output-norm arrangement needs RMSNorms")
        mixed = self.mixer.forward(copy, step, cache)
        x32, copy = ops.norm_add(x32, mixed, rms[0], rms[1], self.mixer.dtype)
        if self.feed_forward is not None:
            if hasattr(self.feed_forward, "forward_stream"):
                x32, copy = self.feed_forward.forward_stream(x32, copy, self.feed_forward_norm, step)
            else:
                rms = self.feed_forward_norm.as_rms()
                x32, copy = ops.norm_add(x32, self.feed_forward.forward(copy, step), rms[0], rms[1], self.mixer.dtype)
        return (x32, copy), None


class MultiStreamBlock(Block):
    """The residual is ``streams`` float32 copies X [S, T, W] (hyper-connections). Sublayer q (1: the mixer,
    2: the feed-forward) reads u = sum_s in_q[s] X[s] through its norm and leaves
    X[t] <- sum_s mix_q[s, t] X[s] + out_q[t] * y for all streams at once. What travels between blocks is the pair
    (X, update still to be applied): one kernel applies the update a sublayer left and makes the next sublayer's
    input, so a sublayer costs one kernel for all of its residual work. With ``learned_mixing`` the block owns
    ``hc1.{in,out,mix}`` (and ``hc2.*`` if it has a feed-forward); without, all coefficients are 1, which with one
    stream is the pre-norm residual kept in float32. A block may have no feed-forward.
    ``mixer_out_norm`` / ``feed_forward_out_norm`` of the spec: the sublayer's output passes an RMS norm of its own
    (a tensor of the block, named from the layer's prefix) before it is added; the same kernel applies it."""

    def _coefficients(self):
        return [f"hc{q}" for q in ((1, 2) if self.feed_forward is not None else (1,))]

    def tensors(self):
        from .base import TensorSpec
        out = {}
        for norm in self._out_norms().values():
            out[norm.tensor] = TensorSpec((norm.size,), role="vector32", init="ones_noise")
        if not self.spec.learned_mixing:
            return out
        n = self.spec.streams
        for name in self._coefficients():
            out[f"{name}.in"] = TensorSpec((n,), role="vector32", init="ones_noise")
            out[f"{name}.out"] = TensorSpec((n,), role="vector32", init="ones_noise")
            out[f"{name}.mix"] = TensorSpec((n, n), role="vector32", init="eye_noise")
        return out

    def _out_norms(self):
        """sublayer -> the NormSpec of the norm on its output, for those that have one."""
        found = {"hc1": getattr(self.spec, "mixer_out_norm", None)}
        if self.feed_forward is not None:
            found["hc2"] = getattr(self.spec, "feed_forward_out_norm", None)
        for norm in found.values():
            if norm is not None and (norm.kind != "rmsnorm" or norm.offset):
                raise ValueError("the norm on a sublayer's output is a plain RMS norm")
        return {k: v for k, v in found.items() if v is not None}

    def load(self, tensors):
        out_names = {norm.tensor for norm in self._out_norms().values()}
        self.coefficients = {name: tensors[name].contiguous() for name in self.tensors() if name not in out_names}
        self.out_norm_weights = {name: tensors[norm.tensor].contiguous() for name, norm in self._out_norms().items()}

    def _coef(self, name: str, device):
        table = getattr(self, "coefficients", None)
        if table is None:
            table = self.coefficients = {}
        if name not in table:              # not learned: all ones
            import torch
            n = self.spec.streams
            table[name] = torch.ones((n, n) if name.endswith(".mix") else (n,), dtype=torch.float32, device=device)
        return table[name]

    def forward(self, x, step, cache):
        return self.forward_linked(x, None, None, step, cache)[0]

    def forward_linked(self, x, link, next_norm, step, cache):
        from .. import ops
        streams, pending = x
        dev, dtype = streams.device, self.mixer.dtype
        sublayers = [("hc1", self.mixer_norm, lambda h: self.mixer.forward(h, step, cache))]
        if self.feed_forward is not None:
            sublayers.append(("hc2", self.feed_forward_norm, lambda h: self.feed_forward.forward(h, step)))
        out_norms = self._out_norms()
        for name, norm, run in sublayers:
            rms = norm.as_rms()
            if rms is None:
                raise ValueError("the multi-stream arrangement needs RMSNorms")
            h = ops.streams_step(streams, pending, self._coef(f"{name}.in", dev), rms[0], rms[1], dtype)
            after = out_norms.get(name)
            pending = ops.StreamUpdate(run(h), self._coef(f"{name}.mix", dev), self._coef(f"{name}.out", dev),
                                       norm_weight=self.out_norm_weights[name] if after is not None else None,
                                       norm_eps=after.eps if after is not None else 0.0)
        return (streams, pending), None


register_block("pre_norm", PreNormBlock)
register_block("multi_stream", MultiStreamBlock)
register_block("output_norm", OutputNormBlock)
