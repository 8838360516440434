"""Sinulix: a pre-norm decoder whose layers mix softmax attention (per-head norm and rotation of q and k, a learned
sink per head in the denominator, a per-head output gate, some layers reading an earlier layer's keys and values),
retention (linear attention with a fixed decay per head) and the gated delta rule with a decay per key channel, each
with a dense gated feed-forward, a mixture of experts or none, around a float32 residual. The blocks, cache and step
function are the generic decoder's; this class only has the frame: an embedding that is scaled into the float32
stream, and at the end the final norm on the wanted rows, an untied head and a smooth cap on the logits."""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.sinulix import NAME, SinulixConfig
from .decoder import StreamDecoderModel


class SinulixForCausalLM(StreamDecoderModel):
    def __init__(self, config: SinulixConfig, dtype, device):
        super().__init__(config.model_spec(), dtype, device, embedding_scale=config.embedding_scale,
                         logit_softcap=config.logit_softcap)
        self.config = config


def _layers(pattern: str, attention: dict, retention: dict, delta: dict, dense: dict, moe: dict):
    """config.json layers from a pattern of letters: 'a' attention, 'k' attention reading the keys and values of the
    last 'a' before it, 'r' retention, 'd' the delta rule; a capital letter gives the layer the mixture of experts,
    a small one the dense feed-forward."""
    out = []
    for letter in pattern:
        kind = letter.lower()
        mlp = dict(moe) if letter.isupper() else dict(dense)
        if kind == "a":
            out.append(dict(type="attention", mixer=dict(attention), mlp=mlp))
        elif kind == "k":
            src = max(i for i, l in enumerate(out) if l["type"] == "attention" and "kv_from" not in l["mixer"])
            out.append(dict(type="attention", mixer=dict(attention, kv_from=src), mlp=mlp))
        elif kind == "r":
            out.append(dict(type="retention", mixer=dict(retention), mlp=mlp))
        else:
            out.append(dict(type="channel_delta", mixer=dict(delta), mlp=mlp))
    return out


def _decays(heads: int):
    """1 - 2^-(5 + 3 h / heads): slow and fast heads side by side."""
    return [1.0 - 2.0 ** -(5.0 + 3.0 * h / heads) for h in range(heads)]


# Sizes worth running with random weights (config.json keys): a toy, and two with the layer sizes of models of about
# one and of a few billion parameters, eight layers each (a benchmark runs as many layers as it lists).
PRESETS = {
    "sinulix-tiny": dict(
        vocab=256, width=64, norm=dict(eps=1e-5), embedding=dict(scale=4.0), logit_softcap=20.0,
        layers=_layers("rDaKd",
                       dict(heads=4, kv_heads=2, dim=16, vdim=16, scale=0.25, rot=dict(base=10000.0, dims=8)),
                       dict(heads=2, dim=16, vdim=24, decay=_decays(2), rot=dict(base=10000.0, dims=16)),
                       dict(heads=4, kv_heads=2, dim=16, vdim=8, conv=3, gate_rank=8),
                       dict(kind="dense", ff=96),
                       dict(kind="moe", expert=dict(ff=32, limit=2.0), router=dict(experts=6, top=2, identity=1)))),
    "sinulix-1b": dict(
        vocab=102400, width=1024, norm=dict(eps=1e-6), embedding=dict(scale=32.0), logit_softcap=30.0,
        layers=_layers("rDaK" * 2,
                       dict(heads=8, kv_heads=4, dim=128, vdim=128, scale=128 ** -0.5, rot=dict(base=1000000.0, dims=128)),
                       dict(heads=8, dim=128, vdim=128, decay=_decays(8), rot=dict(base=10000.0, dims=128)),
                       dict(heads=8, kv_heads=8, dim=128, vdim=128, conv=4, gate_rank=32),
                       dict(kind="dense", ff=3072),
                       dict(kind="moe", expert=dict(ff=704, limit=7.0), router=dict(experts=32, top=4, identity=2)))),
    "sinulix-2b": dict(
        vocab=102400, width=2048, norm=dict(eps=1e-6), embedding=dict(scale=45.0), logit_softcap=30.0,
        layers=_layers("rDaK" * 2,
                       dict(heads=16, kv_heads=8, dim=128, vdim=128, scale=128 ** -0.5, rot=dict(base=1000000.0, dims=128)),
                       dict(heads=16, dim=128, vdim=128, decay=_decays(16), rot=dict(base=10000.0, dims=128)),
                       dict(heads=16, kv_heads=16, dim=128, vdim=128, conv=4, gate_rank=64),
                       dict(kind="dense", ff=6144),
                       dict(kind="moe", expert=dict(ff=1408, limit=7.0), router=dict(experts=64, top=6, identity=2)))),
}

register_architecture(NAME, SinulixConfig, SinulixForCausalLM, presets=PRESETS)
