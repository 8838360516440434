"""Fezozen: a decoder whose layers are listed one by one and mix three kinds of softmax attention (grouped-query with
biases, a partial interleaved rotation stretched for long contexts and tanh-capped scores; grouped-query with q and k
divided by their root mean square after the rotation, behind a sliding window; attention over a cached latent with a
window and an output gate), each with a mixture of sigmoid-scored experts that are weighted at their input. Every
sublayer is normed before and after, x += norm_b(sublayer(norm(x))), around a float32 residual, and a layer may run
another layer's tensors on a cache of its own. The blocks, cache and step function are the generic decoder's; the
frame (scaled embedding into the float32 stream, final norm on the wanted rows, untied head) is the stream decoder's."""
from __future__ import annotations

from ..config.fezozen import NAME, FezozenConfig
from ..config.registry import register_architecture
from .decoder import StreamDecoderModel


class FezozenForCausalLM(StreamDecoderModel):
    def __init__(self, config: FezozenConfig, dtype, device):
        super().__init__(config.model_spec(), dtype, device, embedding_scale=config.embedding_scale)
        self.config = config


def _scaling(original: int):
    return dict(factor=4.0, original=original, fast=32.0, slow=1.0)


def _layers(pattern: str, full: dict, latent: dict, windowed: dict, moe: dict):
    """config.json layers from a pattern of letters: 'a' attention over all keys, 'l' latent attention, 'w' the
    windowed attention with unit q and k; a capital letter runs the tensors of the last layer of its kind written
    small, on a cache of its own."""
    kinds = {"a": ("attention", full), "l": ("latent_attention", latent), "w": ("attention_2", windowed)}
    out = []
    for letter in pattern:
        kind, mixer = kinds[letter.lower()]
        entry = dict(type=kind, mixer=dict(mixer), mlp=dict(moe))
        if letter.isupper():
            entry["weights_of"] = max(i for i, l in enumerate(out) if l["type"] == kind and "weights_of" not in l)
        out.append(entry)
    return out


# Sizes worth running with random weights (config.json keys): a toy, and two with the layer sizes of models of about
# one and of a few billion parameters, six layers each (a benchmark runs as many layers as it lists).
PRESETS = {
    "fezozen-tiny": dict(
        vocab=256, width=64, norm=dict(eps=1e-5), embedding=dict(scale=4.0),
        layers=_layers("alwAL",
                       dict(heads=4, kv_heads=2, dim=16, vdim=8, scale=0.25, softcap=10.0,
                            rot=dict(base=10000.0, dims=8, scaling=_scaling(32))),
                       dict(heads=2, dim=16, rot_dim=8, vdim=24, kv_rank=16, scale=0.2, mask=dict(size=12),
                            rot=dict(base=10000.0, dims=8, scaling=_scaling(64))),
                       dict(heads=4, kv_heads=1, dim=16, vdim=16, scale=0.25, mask=dict(size=7), rot=dict(base=10000.0, dims=16)),
                       dict(kind="moe", expert=dict(ff=32), router=dict(experts=6, top=2)))),
    "fezozen-1b": dict(
        vocab=102400, width=1024, norm=dict(eps=1e-6), embedding=dict(scale=32.0),
        layers=_layers("alwALW",
                       dict(heads=8, kv_heads=4, dim=128, vdim=128, scale=128 ** -0.5, softcap=30.0,
                            rot=dict(base=1000000.0, dims=64, scaling=_scaling(4096))),
                       dict(heads=8, dim=128, rot_dim=64, vdim=128, kv_rank=256, scale=192 ** -0.5, mask=dict(size=1024),
                            rot=dict(base=10000.0, dims=64, scaling=_scaling(4096))),
                       dict(heads=8, kv_heads=4, dim=128, vdim=128, scale=1.0, mask=dict(size=512),
                            rot=dict(base=1000000.0, dims=128)),
                       dict(kind="moe", expert=dict(ff=704), router=dict(experts=32, top=4)))),
    "fezozen-2b": dict(
        vocab=102400, width=2048, norm=dict(eps=1e-6), embedding=dict(scale=45.0),
        layers=_layers("alwALW",
                       dict(heads=16, kv_heads=8, dim=128, vdim=128, scale=128 ** -0.5, softcap=30.0,
                            rot=dict(base=1000000.0, dims=64, scaling=_scaling(4096))),
                       dict(heads=16, dim=128, rot_dim=64, vdim=128, kv_rank=512, scale=192 ** -0.5, mask=dict(size=1024),
                            rot=dict(base=10000.0, dims=64, scaling=_scaling(4096))),
                       dict(heads=16, kv_heads=8, dim=128, vdim=128, scale=1.0, mask=dict(size=512),
                            rot=dict(base=1000000.0, dims=128)),
                       dict(kind="moe", expert=dict(ff=1408), router=dict(experts=64, top=6)))),
}

register_architecture(NAME, FezozenConfig, FezozenForCausalLM, presets=PRESETS)
