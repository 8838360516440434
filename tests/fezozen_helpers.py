"""Small Fezozen configurations and model folders for the tests. Tensor names and shapes are derived here from the
configuration, independently of the engine, so a folder written here also checks what the engine's loader expects.
Weights are drawn so that every mechanism carries weight in the logits: matrices of unit gain, norm weights and
biases of order one, router rows large enough that the sigmoid scores spread between nought and one."""
from __future__ import annotations

import json
import random
from pathlib import Path
from typing import Dict, List, Sequence

import numpy as np
import torch
from safetensors.torch import save_file

import plain_fezozen as plain


def scaling(factor, original, fast=8.0, slow=1.0):
    return dict(factor=factor, original=original, fast=fast, slow=slow)


def rot(base, dims, scaled=None):
    r = dict(base=base, dims=dims)
    if scaled is not None:
        r["scaling"] = scaled
    return r


def attention(heads, kv_heads, dim, vdim, scale=None, rot_=None, softcap=None, window=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=dim ** -0.5 if scale is None else scale)
    if rot_ is not None:
        m["rot"] = rot_
    if softcap is not None:
        m["softcap"] = softcap
    if window is not None:
        m["mask"] = dict(size=window)
    return m


def latent(heads, dim, rot_dim, vdim, kv_rank, scale=None, base=10000.0, scaled=None, window=None):
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank,
             scale=(dim + rot_dim) ** -0.5 if scale is None else scale, rot=rot(base, rot_dim, scaled))
    if window is not None:
        m["mask"] = dict(size=window)
    return m


def moe(experts, top, ff):
    return dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top))


def layer(kind, mixer, mlp=None, weights_of=None):
    entry = dict(type=kind, mixer=mixer, mlp=mlp)
    if weights_of is not None:
        entry["weights_of"] = weights_of
    return entry


def shared(layers, j):
    """One more layer that runs layer j's tensors."""
    return layer(layers[j]["type"], dict(layers[j]["mixer"]), None if layers[j]["mlp"] is None else dict(layers[j]["mlp"]), weights_of=j)


def config(layers, vocab=300, width=72, eps=1e-5, scale=3.0):
    return dict(architecture="Fezozen", vocab=vocab, width=width, norm=dict(eps=eps), embedding=dict(scale=scale), layers=layers)


def _mix():
    layers = [
        layer("attention", attention(6, 2, 20, 12, scale=0.3, rot_=rot(10000.0, 12, scaling(3.0, 24)), softcap=5.0), moe(5, 2, 24)),
        layer("latent_attention", latent(3, 12, 8, 20, 24, scale=0.25, scaled=scaling(2.0, 16, fast=4.0), window=19), moe(3, 3, 40)),
        layer("attention_2", attention(4, 4, 16, 16, scale=0.3, rot_=rot(500.0, 8), window=11), moe(7, 1, 16)),
    ]
    layers.append(shared(layers, 0))
    layers.append(layer("attention_2", attention(6, 3, 12, 20, scale=0.4, rot_=rot(10000.0, 12), window=5), None))
    layers.append(shared(layers, 1))
    return config(layers)


def _wide():
    """Sizes that reach the tensor-core products and attention kernels: heads of 64 and of 128 features with values of
    the same size, a latent whose rows are a multiple of eight features."""
    layers = [
        layer("attention", attention(4, 2, 64, 64, scale=0.2, rot_=rot(1e6, 32, scaling(4.0, 64, fast=16.0)), softcap=8.0), moe(8, 2, 64)),
        layer("attention_2", attention(4, 2, 128, 128, scale=0.08, rot_=rot(1e4, 128), window=70), moe(8, 3, 64)),
        layer("latent_attention", latent(4, 32, 16, 32, 64, scaled=scaling(4.0, 128, fast=16.0), window=50), moe(4, 1, 128)),
    ]
    layers.append(shared(layers, 1))
    layers.append(shared(layers, 0))
    return config(layers, vocab=515, width=128, eps=1e-6, scale=8.0)


def _one():
    """One head of everything, one expert, windows of one and two keys, no rotation in one layer, a layer listed BEFORE
    the one whose tensors it runs, no cap."""
    first = layer("latent_attention", latent(1, 8, 4, 40, 12, window=2), moe(1, 1, 16))
    layers = [
        layer("attention_2", attention(3, 1, 8, 8, window=1), moe(2, 2, 8), weights_of=2),
        first,
        layer("attention_2", attention(3, 1, 8, 8, window=1), moe(2, 2, 8)),
        layer("attention", attention(1, 1, 40, 8, rot_=rot(100.0, 40)), None),
        layer("attention", attention(2, 2, 8, 8, scale=0.5, window=3), moe(3, 1, 8)),
    ]
    return config(layers, width=40, scale=1.0)


MIX, WIDE, ONE = _mix(), _wide(), _one()


def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    W = cfg["width"]
    shapes = {"embed": (cfg["vocab"], W), "head": (cfg["vocab"], W), "final.norm": (W,)}
    for i, entry in enumerate(cfg["layers"]):
        if entry.get("weights_of") is not None:
            continue
        p, m, kind = f"l{i}.", entry["mixer"], entry["type"]
        shapes[p + "norm1"] = shapes[p + "norm1b"] = (W,)
        if kind == "latent_attention":
            H, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            shapes.update({p + "mix.q": (H * (d + r), W), p + "mix.dkv": (rank + r, W), p + "mix.dkv.norm": (rank,),
                           p + "mix.uk": (H * d, rank), p + "mix.uv": (H * dv, rank), p + "mix.g": (H * dv, W),
                           p + "mix.o": (W, H * dv)})
        else:
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            shapes.update({p + "mix.q": (H * d, W), p + "mix.k": (G * d, W), p + "mix.v": (G * dv, W), p + "mix.o": (W, H * dv)})
            if kind == "attention":
                shapes.update({p + "mix.q.b": (H * d,), p + "mix.k.b": (G * d,), p + "mix.v.b": (G * dv,)})
        f = entry.get("mlp")
        if f is None:
            continue
        shapes[p + "norm2"] = shapes[p + "norm2b"] = (W,)
        for e in range(f["router"]["experts"]):
            shapes.update({p + f"mlp.e{e}.gate": (f["expert"]["ff"], W), p + f"mlp.e{e}.up": (f["expert"]["ff"], W),
                           p + f"mlp.e{e}.down": (W, f["expert"]["ff"])})
        shapes[p + "mlp.router"] = (f["router"]["experts"], W)
    return shapes


def draw_tensors(cfg: dict, seed: int, dtype=torch.float32) -> Dict[str, torch.Tensor]:
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        t = torch.randn(shape, generator=gen, dtype=torch.float32)
        leaf = name.split(".", 1)[1] if name.startswith("l") else name
        if leaf in ("norm1", "norm2", "norm1b", "norm2b", "mix.dkv.norm") or name == "final.norm":
            t = 1.0 + 0.2 * t
        elif leaf.endswith(".b"):
            t = 0.5 * t
        elif leaf == "mlp.router":
            t = 2.0 * t / shape[-1] ** 0.5
        elif name == "embed":
            t = 0.5 * t
        else:
            t = t / shape[-1] ** 0.5                     # unit gain
        out[name] = t.to(dtype).contiguous()
    return out


def write_folder(folder, cfg: dict, seed: int, dtype: str = "float32", edit=None) -> Path:
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    tensors = draw_tensors(cfg, seed, torch.float32 if dtype == "float32" else torch.bfloat16)
    if edit is not None:
        edit(tensors)
    (folder / "config.json").write_text(json.dumps(cfg))
    save_file(tensors, str(folder / "model.safetensors"))
    return folder


def read_folder(folder):
    from safetensors.torch import load_file
    cfg = json.loads((Path(folder) / "config.json").read_text())
    return cfg, {k: (v.to(torch.float64) if v.is_floating_point() else v)
                 for k, v in load_file(str(Path(folder) / "model.safetensors")).items()}


def random_requests(cfg: dict, lengths: Sequence[int], seed: int) -> Dict[str, List[int]]:
    rng = random.Random(seed)
    return {f"r{i}": [rng.randrange(cfg["vocab"]) for _ in range(n)] for i, n in enumerate(lengths)}


def forward(cfg, w, tokens, residuals=None) -> np.ndarray:
    return plain.Model(cfg, w, torch.float64).run(tokens, residuals=residuals).numpy()


def plain_logits(folder, requests) -> Dict[str, np.ndarray]:
    cfg, w = read_folder(folder)
    return {rid: forward(cfg, w, toks) for rid, toks in requests.items()}
