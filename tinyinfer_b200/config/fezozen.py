"""Typed configuration of the Fezozen decoder, read from the keys of its own config.json.

config.json: ``architecture`` (the name), ``vocab``, ``width``, ``norm.eps``, ``embedding.scale`` and ``layers``, a list
whose entries give ``type`` (which mixer), ``mixer`` (its sizes), ``mlp`` (its feed-forward, or null) and optionally
``weights_of: j``: the layer has no tensors of its own and runs layer j's mixer, feed-forward and norms on a cache of
its own. Mixer types:
``attention``: ``heads, kv_heads, dim, vdim, scale``, optionally ``softcap`` (scores pass softcap * tanh(s / softcap)),
``rot.{base, dims, scaling}`` and ``mask.size`` (a sliding window); q, k and v have biases;
``attention_2``: the same keys, no biases; q and k are divided by their root mean square per head after the rotation;
``latent_attention``: ``heads, dim, rot_dim, vdim, kv_rank, scale``, ``rot.{base, scaling}``, optionally ``mask.size``;
the queries are a plain projection, the heads' outputs pass a sigmoid gate feature by feature.
``rot.scaling`` = ``{factor, original, fast, slow}`` slows the rotation's slow pairs down for contexts longer than
``original`` (see ``specs.FrequencyBlend``); pairs are neighbouring features (2j, 2j + 1).
Feed-forward: ``kind`` "moe" with ``expert.ff`` and ``router.{experts, top}``: sigmoid scores, the ``top`` largest
chosen, an expert reads its score times the token's row. Every layer is x += norm1b(mixer(norm1(x))),
x += norm2b(ff(norm2(x))) around a float32 residual. Tensors are named ``embed``, ``head``, ``final.norm`` and
``l<i>.{norm1, norm1b, norm2, norm2b, mix.*, mlp.*}``.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import List, Optional

from .specs import (AttentionSpec, ExecStep, ExpertsSpec, FrequencyBlend, LatentAttentionSpec, LayerSpec, ModelSpec, NormSpec,
                    PositionSpec, TensorNames)

NAME = "Fezozen"
MAX_POSITIONS = 1 << 20         # the design sets no limit; the engine's tables need one
_REQUIRED = {
    "attention": ("heads", "kv_heads", "dim", "vdim", "scale"),
    "attention_2": ("heads", "kv_heads", "dim", "vdim", "scale"),
    "latent_attention": ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale"),
}


def _position(rot: Optional[dict], dims: int) -> PositionSpec:
    if not rot or not dims:
        return PositionSpec(kind="none")
    blend = None
    s = rot.get("scaling")
    if s:
        blend = FrequencyBlend(factor=float(s["factor"]), original=int(s["original"]), fast=float(s["fast"]),
                               slow=float(s["slow"]))
    return PositionSpec(kind="rope", theta=float(rot["base"]), rotary_dim=dims, exact_frequencies=True, interleaved=True,
                        blend=blend)


def _window(m: dict) -> Optional[int]:
    size = (m.get("mask") or {}).get("size")
    return int(size) if size else None


@dataclass
class FezozenConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: List[dict]
    embedding_scale: float = 1.0
    eos_token_id: Optional[int] = None
    torch_dtype: Optional[str] = None
    architectures: List[str] = field(default_factory=lambda: [NAME])

    # ------------------------------------------------------------------ parsing
    @classmethod
    def from_dict(cls, data: dict) -> "FezozenConfig":
        missing = [k for k in ("vocab", "width", "layers", "norm") if k not in data]
        if missing:
            raise ValueError(f"config.json lacks required keys: {missing}")
        cfg = cls(vocab=int(data["vocab"]), width=int(data["width"]), norm_eps=float(data["norm"]["eps"]),
                  layers=copy.deepcopy(list(data["layers"])),
                  embedding_scale=float((data.get("embedding") or {}).get("scale", 1.0)),
                  eos_token_id=data.get("eos_token_id"), torch_dtype=data.get("torch_dtype", data.get("dtype")))
        cfg.validate()
        return cfg

    def to_dict(self) -> dict:
        d = {"architecture": NAME, "embedding": {"scale": self.embedding_scale}, "layers": copy.deepcopy(self.layers),
             "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d

    # ------------------------------------------------------------------ checks
    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or not self.layers:
            raise ValueError("vocab, width and the number of layers must be positive")
        if not self.norm_eps > 0:
            raise ValueError("norm.eps must be positive")
        for i, layer in enumerate(self.layers):
            kind, m = layer.get("type"), layer.get("mixer")
            if not isinstance(m, dict):
                raise ValueError(f"layer {i} has no mixer sizes")
            if kind not in _REQUIRED:
                raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
            for key in _REQUIRED[kind]:
                if key not in m:
                    raise ValueError(f"layer {i} ({kind}) lacks mixer.{key}")
            latent = kind == "latent_attention"
            if not latent and int(m["heads"]) % int(m["kv_heads"]):
                raise ValueError(f"layer {i}: heads must be a multiple of kv_heads")
            rot = m.get("rot")
            dims = int(m["rot_dim"]) if latent else int((rot or {}).get("dims", 0))
            if latent and rot and int(rot.get("dims", dims)) != dims:
                raise ValueError(f"layer {i}: rot.dims of a latent attention is its rot_dim")
            if dims:
                if not rot or "base" not in rot or dims % 2 or dims > (dims if latent else int(m["dim"])):
                    raise ValueError(f"layer {i}: rot needs a base, and dims even and at most dim")
                s = rot.get("scaling")
                if s and any(k not in s for k in ("factor", "original", "fast", "slow")):
                    raise ValueError(f"layer {i}: rot.scaling needs factor, original, fast and slow")
            if latent and m.get("softcap"):
                raise ValueError(f"layer {i}: a latent attention's scores are not capped")
            size = (m.get("mask") or {}).get("size")
            if size is not None and int(size) < 1:
                raise ValueError(f"layer {i}: mask.size must be at least 1")
            src = layer.get("weights_of")
            if src is not None:
                other = self.layers[int(src)] if 0 <= int(src) < len(self.layers) and int(src) != i else None
                if other is None or other.get("weights_of") is not None:
                    raise ValueError(f"layer {i}: weights_of must name another layer with tensors of its own")
                if any(other.get(k) != layer.get(k) for k in ("type", "mixer", "mlp")):
                    raise ValueError(f"layer {i}: apart from weights_of its entry must equal layer {src}'s")
            f = layer.get("mlp")
            if f is None:
                continue
            if f.get("kind") != "moe":
                raise ValueError(f"layer {i}: unknown feed-forward kind {f.get('kind')!r}")
            router, expert = f.get("router") or {}, f.get("expert") or {}
            if any(k not in router for k in ("experts", "top")) or "ff" not in expert:
                raise ValueError(f"layer {i}: a mixture of experts needs router.experts, router.top and expert.ff")
            if not 1 <= int(router["top"]) <= int(router["experts"]):
                raise ValueError(f"layer {i}: top must lie between 1 and the number of experts")

    # ------------------------------------------------------------------ layers
    def _layer_spec(self, i: int, layer: dict) -> LayerSpec:
        eps, width = float(self.norm_eps), self.width
        kind, m, f = layer["type"], layer["mixer"], layer.get("mlp")
        if kind == "latent_attention":
            mixer = LatentAttentionSpec(
                hidden_size=width, num_heads=int(m["heads"]), head_dim=int(m["dim"]), rot_dim=int(m["rot_dim"]),
                v_dim=int(m["vdim"]), q_rank=0, kv_rank=int(m["kv_rank"]), scale=float(m["scale"]),
                position=_position(m.get("rot"), int(m["rot_dim"])), norm_eps=eps, window=_window(m), output_gate=True)
        else:
            second = kind == "attention_2"
            softcap = m.get("softcap")
            mixer = AttentionSpec(
                hidden_size=width, num_heads=int(m["heads"]), num_kv_heads=int(m["kv_heads"]), head_dim=int(m["dim"]),
                scale=float(m["scale"]), position=_position(m.get("rot"), int((m.get("rot") or {}).get("dims", 0))),
                window=_window(m), v_dim=int(m["vdim"]), short_names=True, qkv_bias=not second,
                softcap=float(softcap) if softcap else None, qk_unit_norm=eps if second else None)
        ffn = None
        if f is not None:
            router, expert = f["router"], f["expert"]
            ffn = ExpertsSpec(hidden_size=width, num_experts=int(router["experts"]), top=int(router["top"]),
                              expert_size=int(expert["ff"]), activation="silu_glu", renormalize=False, router_input="input",
                              scoring="sigmoid", weight_input=True)
        has_ffn = ffn is not None
        return LayerSpec(mixer=mixer, feed_forward=ffn, mixer_norm=NormSpec(width, eps, tensor=""),
                         feed_forward_norm=NormSpec(width, eps, tensor="") if has_ffn else None,
                         arrangement="multi_stream", streams=1, learned_mixing=False,
                         mixer_out_norm=NormSpec(width, eps, tensor="norm1b"),
                         feed_forward_out_norm=NormSpec(width, eps, tensor="norm2b") if has_ffn else None, index=i)

    def model_spec(self) -> ModelSpec:
        # only layers with tensors of their own become layers of the model; a layer that runs another's tensors is
        # one more entry of the run order on that layer, with a cache entry of its own
        place, layers, execution = {}, [], []
        for i, layer in enumerate(self.layers):
            if layer.get("weights_of") is None:
                place[i] = len(layers)
                layers.append(self._layer_spec(i, layer))
        for i, layer in enumerate(self.layers):
            src = layer.get("weights_of")
            execution.append(ExecStep(layer=place[i if src is None else int(src)], cache=i, writes_cache=True))
        names = TensorNames(embedding="embed", layer="l{i}.", mixer="mix.", feed_forward="mlp.", mixer_norm="norm1",
                            feed_forward_norm="norm2", final_norm="final.norm", head="head")
        return ModelSpec(architecture=NAME, vocab_size=self.vocab, hidden_size=self.width, layers=tuple(layers),
                         execution=tuple(execution), final_norm=NormSpec(self.width, float(self.norm_eps), tensor=""),
                         tie_embeddings=False, max_positions=MAX_POSITIONS, names=names)
