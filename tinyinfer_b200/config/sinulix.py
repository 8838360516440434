"""Typed configuration of the Sinulix decoder, read from the keys of its own config.json.

config.json: ``architecture`` (the name), ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``, ``logit_softcap``
and ``layers``, a list whose entries give ``type`` (which mixer), ``mixer`` (its sizes) and ``mlp`` (its
feed-forward, or null). Mixer types:
``attention``: ``heads, kv_heads, dim, vdim, scale, rot.{base, dims}`` and optionally ``kv_from`` (the layer has no
key/value tensors and reads the keys and values that layer caches);
``retention``: ``heads, dim, vdim, decay`` (one number per head), ``rot.{base, dims}``;
``channel_delta``: ``heads, kv_heads, dim, vdim, conv`` (the inner size of its two-step projections is the
checkpoint's, or ``gate_rank`` for random weights).
Feed-forward: ``kind`` "dense" with ``ff``, or "moe" with ``expert.{ff, limit}`` and ``router.{experts, top,
identity}``. Every size and constant comes from there; tensors are named ``embed``, ``head``, ``final.norm`` and
``l<i>.{norm1, norm2, mix.*, mlp.*}``. A key that is absent switches its mechanism off where that means something
(``embedding.scale``: 1; ``logit_softcap``: none; ``rot``: no rotation; ``router.identity``: 0).
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import List, Optional

from .specs import (AttentionSpec, ChannelDeltaSpec, ExecStep, ExpertsSpec, GatedMLPSpec, LayerSpec, ModelSpec, NormSpec,
                    PositionSpec, RetentionSpec, TensorNames)

NAME = "Sinulix"
MAX_POSITIONS = 1 << 20         # the design sets no limit; the engine's tables need one
NORM_OFFSET = 1.0               # the layers' norms store their weight around zero: x / rms(x) * (1 + w)
GLU_ALPHA = 1.702               # an expert's gate is g * sigmoid(1.702 g)
UNIT_EPS = 1e-6                 # q and k of the delta rule: x / sqrt(sum x^2 + 1e-6)
_REQUIRED = {
    "attention": ("heads", "kv_heads", "dim", "vdim", "scale"),
    "retention": ("heads", "dim", "vdim", "decay"),
    "channel_delta": ("heads", "kv_heads", "dim", "vdim", "conv"),
}


def _position(m: dict) -> PositionSpec:
    rot = m.get("rot")
    if not rot or not int(rot.get("dims", 0)):
        return PositionSpec(kind="none")
    return PositionSpec(kind="rope", theta=float(rot["base"]), rotary_dim=int(rot["dims"]), exact_frequencies=True)


@dataclass
class SinulixConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: List[dict]
    embedding_scale: float = 1.0
    logit_softcap: Optional[float] = None
    eos_token_id: Optional[int] = None
    torch_dtype: Optional[str] = None
    architectures: List[str] = field(default_factory=lambda: [NAME])

    # ------------------------------------------------------------------ parsing
    @classmethod
    def from_dict(cls, data: dict) -> "SinulixConfig":
        missing = [k for k in ("vocab", "width", "layers", "norm") if k not in data]
        if missing:
            raise ValueError(f"config.json lacks required keys: {missing}")
        cap = data.get("logit_softcap")
        cfg = cls(vocab=int(data["vocab"]), width=int(data["width"]), norm_eps=float(data["norm"]["eps"]),
                  layers=copy.deepcopy(list(data["layers"])),
                  embedding_scale=float((data.get("embedding") or {}).get("scale", 1.0)),
                  logit_softcap=float(cap) if cap else None, eos_token_id=data.get("eos_token_id"),
                  torch_dtype=data.get("torch_dtype", data.get("dtype")))
        cfg.validate()
        return cfg

    def to_dict(self) -> dict:
        d = {"architecture": NAME, "embedding": {"scale": self.embedding_scale}, "layers": copy.deepcopy(self.layers),
             "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d

    # ------------------------------------------------------------------ checks
    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or not self.layers:
            raise ValueError("vocab, width and the number of layers must be positive")
        if not self.norm_eps > 0:
            raise ValueError("norm.eps must be positive")
        if self.logit_softcap is not None and not self.logit_softcap > 0:
            raise ValueError("logit_softcap must be positive")
        for i, layer in enumerate(self.layers):
            kind, m = layer.get("type"), layer.get("mixer")
            if not isinstance(m, dict):
                raise ValueError(f"layer {i} has no mixer sizes")
            if kind not in _REQUIRED:
                raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
            for key in _REQUIRED[kind]:
                if key not in m:
                    raise ValueError(f"layer {i} ({kind}) lacks mixer.{key}")
            rot = m.get("rot")
            if rot and int(rot.get("dims", 0)):
                if "base" not in rot or int(rot["dims"]) % 2 or int(rot["dims"]) > int(m["dim"]):
                    raise ValueError(f"layer {i}: rot needs a base, and dims even and at most dim")
            if kind != "retention" and int(m["heads"]) % int(m["kv_heads"]):
                raise ValueError(f"layer {i}: heads must be a multiple of kv_heads")
            if kind == "retention" and len(m["decay"]) != int(m["heads"]):
                raise ValueError(f"layer {i}: decay lists one number per head")
            if kind == "channel_delta" and int(m["conv"]) < 1:
                raise ValueError(f"layer {i}: conv must be at least 1")
            src = m.get("kv_from")
            if src is not None:
                if kind != "attention":
                    raise ValueError(f"layer {i}: only an attention layer reads another layer's keys and values")
                other = self.layers[int(src)] if 0 <= int(src) < i else None
                if other is None or other.get("type") != "attention" or other["mixer"].get("kv_from") is not None:
                    raise ValueError(f"layer {i}: kv_from must name an earlier attention layer with key/value "
                                     "projections of its own")
                o = other["mixer"]
                if any(o.get(k) != m.get(k) for k in ("heads", "kv_heads", "dim", "vdim", "rot")):
                    raise ValueError(f"layer {i}: head counts, sizes and rot must equal those of layer {src}")
            f = layer.get("mlp")
            if f is None:
                continue
            if f.get("kind") == "dense":
                if "ff" not in f:
                    raise ValueError(f"layer {i}: a dense feed-forward needs ff")
            elif f.get("kind") == "moe":
                router, expert = f.get("router") or {}, f.get("expert") or {}
                if any(k not in router for k in ("experts", "top")) or any(k not in expert for k in ("ff", "limit")):
                    raise ValueError(f"layer {i}: a mixture of experts needs router.experts, router.top, expert.ff "
                                     "and expert.limit")
                if int(router["top"]) > int(router["experts"]) + int(router.get("identity", 0)):
                    raise ValueError(f"layer {i}: top exceeds the number of router outputs")
            else:
                raise ValueError(f"layer {i}: unknown feed-forward kind {f.get('kind')!r}")

    # ------------------------------------------------------------------ layers
    def model_spec(self) -> ModelSpec:
        eps, width = float(self.norm_eps), self.width
        norm = NormSpec(width, eps, tensor="", offset=NORM_OFFSET)
        layers, execution, entry_of = [], [], {}
        for i, layer in enumerate(self.layers):
            kind, m, f = layer["type"], layer["mixer"], layer.get("mlp")
            src = m.get("kv_from")
            if kind == "attention":
                mixer = AttentionSpec(
                    hidden_size=width, num_heads=int(m["heads"]), num_kv_heads=int(m["kv_heads"]), head_dim=int(m["dim"]),
                    scale=float(m["scale"]), position=_position(m),
                    qk_norm=NormSpec(int(m["dim"]), eps, tensor=""), v_dim=int(m["vdim"]), head_sinks=True,
                    head_gate=True, shares_cache=src is not None, short_names=True)
            elif kind == "retention":
                mixer = RetentionSpec(hidden_size=width, num_heads=int(m["heads"]), key_dim=int(m["dim"]),
                                      value_dim=int(m["vdim"]), decays=tuple(float(d) for d in m["decay"]),
                                      position=_position(m), norm_eps=eps)
            else:
                mixer = ChannelDeltaSpec(hidden_size=width, num_heads=int(m["heads"]), num_kv_heads=int(m["kv_heads"]),
                                         key_dim=int(m["dim"]), value_dim=int(m["vdim"]), conv_taps=int(m["conv"]),
                                         norm_eps=eps, unit_eps=UNIT_EPS, gate_rank=int(m.get("gate_rank", 0)))
            # every layer with keys, values or a state of its own has a cache entry; a reader works on its writer's
            if src is None:
                entry_of[i] = len(entry_of)
                execution.append(ExecStep(layer=i, cache=entry_of[i], writes_cache=True))
            else:
                execution.append(ExecStep(layer=i, cache=entry_of[int(src)], writes_cache=False))
            ffn = None
            if f is not None and f["kind"] == "dense":
                ffn = GatedMLPSpec(hidden_size=width, intermediate_size=int(f["ff"]), names=("gate", "up", "down"))
            elif f is not None:
                router, expert = f["router"], f["expert"]
                ffn = ExpertsSpec(hidden_size=width, num_experts=int(router["experts"]), top=int(router["top"]),
                                  expert_size=int(expert["ff"]), activation="clamped_glu", glu_limit=float(expert["limit"]),
                                  glu_alpha=GLU_ALPHA, identity_experts=int(router.get("identity", 0)),
                                  score_correction=True, renormalize=False, router_input="input")
            layers.append(LayerSpec(mixer=mixer, feed_forward=ffn, mixer_norm=norm,
                                    feed_forward_norm=norm if ffn is not None else None, arrangement="multi_stream",
                                    streams=1, learned_mixing=False))
        names = TensorNames(embedding="embed", layer="l{i}.", mixer="mix.", feed_forward="mlp.", mixer_norm="norm1",
                            feed_forward_norm="norm2", final_norm="final.norm", head="head")
        return ModelSpec(architecture=NAME, vocab_size=self.vocab, hidden_size=width, layers=tuple(layers),
                         execution=tuple(execution), final_norm=norm, tie_embeddings=False,
                         max_positions=MAX_POSITIONS, names=names)
