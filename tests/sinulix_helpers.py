"""Small Sinulix configurations and model folders for the tests. Tensor names and shapes are derived here from the
configuration, independently of the engine, so a folder written here also checks what the engine's loader expects.
Weights are drawn so that every mechanism carries weight in the logits: matrices of unit gain, norm weights, sinks,
corrections and convolution taps of order one, decays near one so that a state remembers far tokens."""
from __future__ import annotations

import json
import random
from pathlib import Path
from typing import Dict, List, Sequence

import numpy as np
import torch
from safetensors.torch import save_file

import plain_sinulix as plain


def attention(heads, kv_heads, dim, vdim, scale=None, rot=None, base=10000.0, kv_from=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=dim ** -0.5 if scale is None else scale,
             rot=dict(base=base, dims=dim if rot is None else rot))
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def retention(heads, dim, vdim, decay=None, rot=None, base=10000.0):
    decay = [1.0 - 2.0 ** -(3 + h) for h in range(heads)] if decay is None else list(decay)
    return dict(heads=heads, dim=dim, vdim=vdim, decay=decay, rot=dict(base=base, dims=dim if rot is None else rot))


def delta(heads, kv_heads, dim, vdim, conv=4, gate_rank=6):
    return dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv, gate_rank=gate_rank)


def layer(kind, mixer, mlp=None):
    return dict(type=kind, mixer=mixer, mlp=mlp)


def dense(ff):
    return dict(kind="dense", ff=ff)


def moe(experts, top, ff, identity=0, limit=1.5):
    return dict(kind="moe", expert=dict(ff=ff, limit=limit), router=dict(experts=experts, top=top, identity=identity))


def config(layers, vocab=300, width=72, eps=1e-5, scale=3.0, softcap=12.0):
    cfg = dict(architecture="Sinulix", vocab=vocab, width=width, norm=dict(eps=eps), embedding=dict(scale=scale),
               layers=layers)
    if softcap is not None:
        cfg["logit_softcap"] = softcap
    return cfg


# nothing a power of two; key and value sizes differ; grouped heads; a partial rotation; a reader two layers behind
# its writer; a layer without feed-forward; experts with and without identity experts
MIX = config([
    layer("retention", retention(3, 20, 12, rot=8), dense(88)),
    layer("attention", attention(6, 2, 20, 12, scale=0.3, rot=12), moe(5, 2, 24, identity=2)),
    layer("channel_delta", delta(6, 3, 12, 20, conv=3), moe(7, 3, 40, identity=0, limit=0.8)),
    layer("attention", attention(6, 2, 20, 12, scale=0.3, rot=12, kv_from=1), None),
    layer("channel_delta", delta(2, 2, 28, 12, conv=5, gate_rank=3), dense(40)),
])
# sizes that reach the tensor-core products and attention kernels (keys and values of 64 features, two planes)
WIDE = config([
    layer("attention", attention(4, 2, 64, 64, scale=0.2), dense(256)),
    layer("channel_delta", delta(4, 4, 32, 32, conv=4, gate_rank=16), moe(8, 2, 64, identity=1, limit=2.0)),
    layer("attention", attention(4, 2, 64, 64, scale=0.2, kv_from=0), moe(8, 3, 64, identity=3, limit=1.0)),
    layer("retention", retention(4, 32, 64, rot=16), dense(128)),
], vocab=515, width=128, eps=1e-6, scale=8.0, softcap=None)
# one head of everything, one expert of which one is chosen, one tap, heads sharing one key head, no rotation at all
ONE = config([
    layer("channel_delta", delta(1, 1, 40, 8, conv=1, gate_rank=2), moe(1, 1, 16, identity=1)),
    layer("attention", attention(3, 1, 8, 8, rot=0), dense(24)),
    layer("retention", retention(1, 8, 40, decay=[0.97], rot=0), None),
    layer("channel_delta", delta(4, 1, 8, 12, conv=2), moe(3, 3, 8, identity=0)),
], width=40, scale=1.0)


def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    W = cfg["width"]
    shapes = {"embed": (cfg["vocab"], W), "head": (cfg["vocab"], W), "final.norm": (W,)}
    for i, entry in enumerate(cfg["layers"]):
        p, m, kind = f"l{i}.", entry["mixer"], entry["type"]
        shapes[p + "norm1"] = (W,)
        if kind == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            shapes.update({p + "mix.q": (H * d, W), p + "mix.q.norm": (d,), p + "mix.sink": (H,), p + "mix.g": (H, W),
                           p + "mix.o": (W, H * dv)})
            if m.get("kv_from") is None:
                shapes.update({p + "mix.k": (G * d, W), p + "mix.v": (G * dv, W), p + "mix.k.norm": (d,)})
        elif kind == "retention":
            H, d, dv = m["heads"], m["dim"], m["vdim"]
            shapes.update({p + "mix.q": (H * d, W), p + "mix.k": (H * d, W), p + "mix.v": (H * dv, W),
                           p + "mix.g": (H * dv, W), p + "mix.o": (W, H * dv)})
        else:
            H, G, d, dv, r = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["gate_rank"]
            for name, n in (("q", G * d), ("k", G * d), ("v", H * dv)):
                shapes[p + f"mix.{name}"] = (n, W)
                shapes[p + f"mix.{name}.conv"] = (n, m["conv"])
            shapes.update({p + "mix.b": (H, W), p + "mix.A_log": (H,), p + "mix.norm": (dv,), p + "mix.a1": (r, W),
                           p + "mix.a2": (H * d, r), p + "mix.dt_bias": (H * d,), p + "mix.g1": (r, W),
                           p + "mix.g2": (H * dv, r), p + "mix.o": (W, H * dv)})
        f = entry.get("mlp")
        if f is None:
            continue
        shapes[p + "norm2"] = (W,)
        if f["kind"] == "dense":
            shapes.update({p + "mlp.gate": (f["ff"], W), p + "mlp.up": (f["ff"], W), p + "mlp.down": (W, f["ff"])})
        else:
            outputs = f["router"]["experts"] + f["router"].get("identity", 0)
            for e in range(f["router"]["experts"]):
                shapes.update({p + f"mlp.e{e}.gate": (f["expert"]["ff"], W), p + f"mlp.e{e}.up": (f["expert"]["ff"], W),
                               p + f"mlp.e{e}.down": (W, f["expert"]["ff"])})
            shapes.update({p + "mlp.router": (outputs, W), p + "mlp.correction": (outputs,)})
    return shapes


def draw_tensors(cfg: dict, seed: int, dtype=torch.float32) -> Dict[str, torch.Tensor]:
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        t = torch.randn(shape, generator=gen, dtype=torch.float32)
        leaf = name.split(".", 1)[1] if name.startswith("l") else name
        if leaf in ("norm1", "norm2") or name == "final.norm":
            t = 0.2 * t                                  # stored around zero
        elif leaf in ("mix.norm", "mix.q.norm", "mix.k.norm"):
            t = 1.0 + 0.2 * t
        elif leaf.endswith(".conv"):
            t = 0.6 * t
        elif leaf == "mix.sink":
            t = 1.0 + t                                  # a sink that takes a good share of the denominator
        elif leaf == "mix.A_log":
            t = -2.0 + 0.7 * t                           # decays near one: the state remembers far tokens
        elif leaf == "mix.dt_bias":
            t = 0.5 * t
        elif leaf == "mlp.correction":
            t = 0.3 * t                                  # large against scores of 1 / outputs: the choice follows it
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
    stored = {k: v for k, v in cfg.items()}
    stored["layers"] = [dict(l, mixer={k: v for k, v in l["mixer"].items() if k != "gate_rank"}) for l in cfg["layers"]]
    (folder / "config.json").write_text(json.dumps(stored))      # the inner sizes are the checkpoint's alone
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


def forward(cfg, w, tokens) -> np.ndarray:
    model = plain.PlainSinulix(cfg, w, torch.float64)
    return model.feed(model.new_request(), tokens).numpy()


def plain_logits(folder, requests, edit=None) -> Dict[str, np.ndarray]:
    cfg, w = read_folder(folder)
    if edit is not None:
        edit(cfg, w)
    return {rid: forward(cfg, w, toks) for rid, toks in requests.items()}
