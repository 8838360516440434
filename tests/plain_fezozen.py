"""A plain, slow statement of the Fezozen decoder on the CPU, one function per mechanism, written from the design's
equations. It shares no code with the engine: tensors come in as a dict name -> torch tensor, the configuration as
the dict of config.json. Everything runs token by token in one precision (float64 by default), so it is the
yardstick for prompts, decoding, portions and batches alike.

Notation: h is a sublayer's input (the normed residual), W_x the tensor '<layer>.mix.x' or '<layer>.mlp.x', stored
[out, in] and applied as W h. A layer with ``weights_of: j`` runs layer j's tensors on a cache of its own.
"""
from __future__ import annotations

import math

import torch


def rms_norm(x, eps, weight=None):
    """x / sqrt(mean(x^2) + eps) over the last axis, times the weight if there is one."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def frequencies(rot: dict, dtype=torch.float64):
    """(frequency per pair, factor on cosines and sines). Without ``scaling`` the frequencies are base^(-2i/dims) and
    the factor is one. With it (factor F, original length L, fast and slow turn counts) the pairs that turn fewer
    than ``slow`` times in L positions are slowed down F times, those that turn more than ``fast`` times stay, and
    the pairs between are blended linearly in the pair index; cosines and sines grow by 0.1 ln F + 1."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=dtype)
    f = base ** (-2.0 * i / dims)
    s = rot.get("scaling")
    if not s:
        return f, 1.0

    def pair_of(turns):       # the (fractional) pair index that makes ``turns`` full turns over the original length
        return dims * math.log(s["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(s["fast"])), 0)
    hi = min(math.ceil(pair_of(s["slow"])), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / s["factor"] * ramp + f * (1.0 - ramp), 0.1 * math.log(s["factor"]) + 1.0


def rotate(x, position, rot):
    """x [heads, dim]: the first rot.dims features of every head turn in neighbouring pairs (2i, 2i + 1) by the angle
    position * frequency_i; the rest pass."""
    if not rot or not int(rot.get("dims", 0)):
        return x
    dims = int(rot["dims"])
    f, factor = frequencies(rot, x.dtype)
    angle = position * f
    c, s = torch.cos(angle) * factor, torch.sin(angle) * factor
    u, v = x[:, 0:dims:2], x[:, 1:dims:2]
    turned = torch.stack([u * c - v * s, v * c + u * s], dim=-1).reshape(x.shape[0], dims)
    return torch.cat([turned, x[:, dims:]], dim=-1)


def silu(x):
    return x * torch.sigmoid(x)


def visible(position, window):
    """First key a query at ``position`` sees: all of them without a window, else the last ``window`` (itself included)."""
    return 0 if not window else max(0, position - window + 1)


def softmax_mix(scores, values):
    p = torch.softmax(scores, dim=0)
    return (p[:, None] * values).sum(0)


def attention(w, m, eps, h, position, cache):
    """Grouped-query attention with biases on q, k and v, a partial rotation and tanh-capped scores; all keys seen."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rotate((w["q"] @ h + w["q.b"]).view(H, d), position, m.get("rot"))
    cache["k"].append(rotate((w["k"] @ h + w["k.b"]).view(G, d), position, m.get("rot")))
    cache["v"].append((w["v"] @ h + w["v.b"]).view(G, dv))
    first = visible(position, (m.get("mask") or {}).get("size"))
    keys, values = torch.stack(cache["k"][first:position + 1]), torch.stack(cache["v"][first:position + 1])
    out = []
    for head in range(H):
        g = head // (H // G)
        score = (keys[:, g] @ q[head]) * m["scale"]
        cap = m.get("softcap")
        if cap:
            score = cap * torch.tanh(score / cap)
        out.append(softmax_mix(score, values[:, g]))
    return w["o"] @ torch.cat(out)


def attention_2(w, m, eps, h, position, cache):
    """Grouped-query attention without biases whose q and k are divided by their root mean square per head AFTER
    the rotation; a sliding window."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_norm(rotate((w["q"] @ h).view(H, d), position, m.get("rot")), eps)
    cache["k"].append(rms_norm(rotate((w["k"] @ h).view(G, d), position, m.get("rot")), eps))
    cache["v"].append((w["v"] @ h).view(G, dv))
    first = visible(position, (m.get("mask") or {}).get("size"))
    keys, values = torch.stack(cache["k"][first:position + 1]), torch.stack(cache["v"][first:position + 1])
    out = []
    for head in range(H):
        g = head // (H // G)
        out.append(softmax_mix((keys[:, g] @ q[head]) * m["scale"], values[:, g]))
    return w["o"] @ torch.cat(out)


def latent_attention(w, m, eps, h, position, cache):
    """Attention over a cached latent: a token leaves c (normed, kv_rank features) and one rotated key part of
    rot_dim features that all heads share. A head's key is [W_uk c | rotated part], its value W_uv c. Sliding
    window; the heads side by side are multiplied by sigmoid(W_g h)."""
    H, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rot = dict(m["rot"], dims=r)
    q = (w["q"] @ h).view(H, d + r)
    q_plain, q_rot = q[:, :d], rotate(q[:, d:], position, rot)
    down = w["dkv"] @ h
    cache["c"].append(rms_norm(down[:rank], eps, w["dkv.norm"]))
    cache["r"].append(rotate(down[rank:][None], position, rot)[0])
    first = visible(position, (m.get("mask") or {}).get("size"))
    c, kr = torch.stack(cache["c"][first:position + 1]), torch.stack(cache["r"][first:position + 1])
    uk, uv = w["uk"].view(H, d, rank), w["uv"].view(H, dv, rank)
    out = []
    for head in range(H):
        keys, values = c @ uk[head].t(), c @ uv[head].t()
        out.append(softmax_mix((keys @ q_plain[head] + kr @ q_rot[head]) * m["scale"], values))
    return w["o"] @ (torch.cat(out) * torch.sigmoid(w["g"] @ h))


def experts(w, f, h):
    """Router scores sigmoid(W_router h); the ``top`` largest are chosen (first index on ties); a chosen expert runs
    on ITS SCORE TIMES h: sum_e W_down (silu(W_gate (s_e h)) * (W_up (s_e h)))."""
    score = torch.sigmoid(w["router"] @ h)
    out = torch.zeros_like(h)
    for e in torch.topk(score, int(f["router"]["top"])).indices.tolist():
        x = score[e] * h
        out = out + w[f"e{e}.down"] @ (silu(w[f"e{e}.gate"] @ x) * (w[f"e{e}.up"] @ x))
    return out


MIXERS = {"attention": attention, "attention_2": attention_2, "latent_attention": latent_attention}


def new_cache(kind):
    return {"c": [], "r": []} if kind == "latent_attention" else {"k": [], "v": []}


def sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


class Model:
    def __init__(self, cfg: dict, tensors: dict, dtype=torch.float64):
        self.cfg = cfg
        self.t = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
        self.dtype = dtype

    def new_request(self):
        return [new_cache(layer["type"]) for layer in self.cfg["layers"]]

    def token(self, caches, token_id, position, residuals=None):
        """Logits of one token at ``position`` of a request whose caches hold the positions before it."""
        cfg, t, eps = self.cfg, self.t, self.cfg["norm"]["eps"]
        x = t["embed"][token_id] * cfg["embedding"]["scale"]
        for i, layer in enumerate(cfg["layers"]):
            p = f"l{layer.get('weights_of', i)}."
            h = rms_norm(x, eps, t[p + "norm1"])
            y = MIXERS[layer["type"]](sub(t, p + "mix."), layer["mixer"], eps, h, position, caches[i])
            x = x + rms_norm(y, eps, t[p + "norm1b"])
            if layer.get("mlp") is not None:
                h = rms_norm(x, eps, t[p + "norm2"])
                x = x + rms_norm(experts(sub(t, p + "mlp."), layer["mlp"], h), eps, t[p + "norm2b"])
            if residuals is not None:
                residuals.append(x.clone())
        return t["head"] @ rms_norm(x, eps, t["final.norm"])

    def run(self, tokens, want=None, residuals=None):
        """Logits [len(want), vocab] of a whole request fed token by token (``want``: positions, default all)."""
        caches, out = self.new_request(), []
        for pos, tok in enumerate(tokens):
            per_layer = [] if residuals is not None else None
            logits = self.token(caches, tok, pos, per_layer)
            if residuals is not None:
                residuals.append(torch.stack(per_layer))
            if want is None or pos in want:
                out.append(logits)
        return torch.stack(out)
