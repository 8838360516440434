"""A plain, slow statement of the Sinulix decoder on the CPU, one function per mechanism, written from the
design's equations. It shares no code with the engine: tensors come in as a dict name -> torch tensor, the
configuration as the dict of config.json. Everything runs token by token in one precision (float64 by default),
so it is the yardstick for prompts, decoding, portions and batches alike.

Notation: h is a sublayer's input (the normed residual), W_x the tensor '<layer>.mix.x' or '<layer>.mlp.x',
stored [out, in] and applied as W h.
"""
from __future__ import annotations

import math

import torch


def rms_norm(x, eps, weight=None, one_plus=False):
    """x / sqrt(mean(x^2) + eps) over the last axis, times the weight (or 1 + weight)."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    if weight is None:
        return y
    return y * (1.0 + weight if one_plus else weight)


def rotate(x, position, dims, base):
    """x [heads, dim]: the first ``dims`` features of every head turn in pairs (i, i + dims / 2) by the angle
    position * base^(-2i / dims); the rest pass."""
    if not dims:
        return x
    half = dims // 2
    i = torch.arange(half, dtype=x.dtype)
    angle = position * base ** (-2.0 * i / dims)
    c, s = torch.cos(angle), torch.sin(angle)
    u, v = x[:, :half], x[:, half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[:, dims:]], dim=-1)


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30))))


def silu(x):
    return x * torch.sigmoid(x)


def short_conv(history, x, weight):
    """history [taps - 1, channels] (oldest first, zeros at the start), x [channels] the current input,
    weight [channels, taps] whose last column meets the current token. Returns (output, new history)."""
    window = torch.cat([history, x[None]], dim=0)                 # [taps, channels]
    out = (window * weight.t()).sum(0)
    return out, window[1:]


class Attention:
    """Grouped-query softmax attention with per-head norm of q and k, rotation, a learned sink in the denominator
    and a per-head output gate. ``cache`` is a dict with lists 'k' and 'v'; a layer with kv_from reads another's."""

    @staticmethod
    def step(w, m, eps, h, position, cache, writes):
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        rot = m.get("rot") or {}
        q = (w["q"] @ h).view(H, d)
        q = rotate(rms_norm(q, eps, w["q.norm"]), position, rot.get("dims", 0), rot.get("base", 1.0))
        if writes:
            k = (w["k"] @ h).view(G, d)
            k = rotate(rms_norm(k, eps, w["k.norm"]), position, rot.get("dims", 0), rot.get("base", 1.0))
            cache["k"].append(k)
            cache["v"].append((w["v"] @ h).view(G, dv))
        keys = torch.stack(cache["k"][:position + 1])             # [n, G, d]
        values = torch.stack(cache["v"][:position + 1])           # [n, G, dv]
        gate = torch.sigmoid(w["g"] @ h)                          # [H]
        out = []
        for head in range(H):
            g = head // (H // G)
            score = (keys[:, g] @ q[head]) * m["scale"]
            top = torch.maximum(score.max(), w["sink"][head])
            e = torch.exp(score - top)
            p = e / (e.sum() + torch.exp(w["sink"][head] - top))
            out.append((p[:, None] * values[:, g]).sum(0) * gate[head])
        return w["o"] @ torch.cat(out)


class Retention:
    """Linear attention with a fixed decay per head: S <- decay S + k v^T, o = S^T q; q and k rotated, k scaled by
    dim^-1/2; each head's o divided by its root mean square, gated by silu(W_g h)."""

    @staticmethod
    def new_state(m, dtype):
        return {"S": torch.zeros(m["heads"], m["dim"], m["vdim"], dtype=dtype)}

    @staticmethod
    def step(w, m, eps, h, position, state):
        H, d, dv = m["heads"], m["dim"], m["vdim"]
        rot = m.get("rot") or {}
        q = rotate((w["q"] @ h).view(H, d), position, rot.get("dims", 0), rot.get("base", 1.0))
        k = rotate((w["k"] @ h).view(H, d), position, rot.get("dims", 0), rot.get("base", 1.0)) * d ** -0.5
        v = (w["v"] @ h).view(H, dv)
        decay = torch.tensor(m["decay"], dtype=h.dtype)
        state["S"] = decay[:, None, None] * state["S"] + k[:, :, None] * v[:, None, :]
        o = torch.einsum("hkv,hk->hv", state["S"], q)
        o = rms_norm(o, eps)
        return w["o"] @ (o.reshape(-1) * silu(w["g"] @ h))


class ChannelDelta:
    """Gated delta rule with a decay per head and key channel; q, k, v pass a short causal convolution and silu; q and
    k are unit vectors per head."""

    @staticmethod
    def new_state(m, dtype):
        H, G, d, dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
        return {"S": torch.zeros(H, d, dv, dtype=dtype),
                "q": torch.zeros(taps - 1, G * d, dtype=dtype), "k": torch.zeros(taps - 1, G * d, dtype=dtype),
                "v": torch.zeros(taps - 1, H * dv, dtype=dtype)}

    @staticmethod
    def step(w, m, eps, h, position, state):
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        parts = {}
        for name in ("q", "k", "v"):
            out, state[name] = short_conv(state[name], w[name] @ h, w[name + ".conv"])
            parts[name] = silu(out)
        q, k, v = parts["q"].view(G, d), parts["k"].view(G, d), parts["v"].view(H, dv)
        q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
        k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
        beta = torch.sigmoid(w["b"] @ h)                                          # [H]
        dt = softplus(w["a2"] @ (w["a1"] @ h) + w["dt_bias"]).view(H, d)
        g = torch.exp(-torch.exp(w["A_log"])[:, None] * dt)                       # [H, d]
        out = []
        for head in range(H):
            kh, qh = k[head // (H // G)], q[head // (H // G)]
            S = g[head][:, None] * state["S"][head]
            u = beta[head] * (v[head] - S.t() @ kh)
            S = S + kh[:, None] * u[None, :]
            state["S"][head] = S
            out.append(S.t() @ qh)
        o = rms_norm(torch.stack(out), eps, w["norm"])                            # [H, dv]
        gate = torch.sigmoid(w["g2"] @ (w["g1"] @ h))
        return w["o"] @ (o.reshape(-1) * gate)


def dense_mlp(w, h):
    return w["down"] @ (silu(w["gate"] @ h) * (w["up"] @ h))


def experts_mlp(w, f, h):
    """Mixture of experts: softmax over all router outputs (the last ``identity`` of them stand for experts whose
    output is h itself); the ``top`` largest of score + correction are chosen; weights are the plain scores."""
    r, e = f["router"], f["expert"]
    scores = torch.softmax(w["router"] @ h, dim=-1)
    chosen = torch.topk(scores + w["correction"], r["top"]).indices
    real = r["experts"]
    limit = e["limit"]
    out = torch.zeros_like(h)
    for idx in chosen.tolist():
        if idx >= real:
            out = out + scores[idx] * h
            continue
        g = torch.clamp(w[f"e{idx}.gate"] @ h, max=limit)
        u = torch.clamp(w[f"e{idx}.up"] @ h, min=-limit, max=limit)
        out = out + scores[idx] * (w[f"e{idx}.down"] @ (g * torch.sigmoid(1.702 * g) * (u + 1.0)))
    return out


MIXERS = {"attention": Attention, "retention": Retention, "channel_delta": ChannelDelta}


class PlainSinulix:
    def __init__(self, config: dict, tensors: dict, dtype=torch.float64):
        self.cfg, self.dtype = config, dtype
        self.t = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
        self.eps = config["norm"]["eps"]

    def _sub(self, prefix):
        n = len(prefix)
        return {k[n:]: v for k, v in self.t.items() if k.startswith(prefix)}

    def new_request(self):
        states = []
        for layer in self.cfg["layers"]:
            kind, m = layer["type"], layer["mixer"]
            states.append({"k": [], "v": []} if kind == "attention" else MIXERS[kind].new_state(m, self.dtype))
        return {"length": 0, "layers": states}

    def feed(self, request, tokens, keep_layers=False):
        """Runs the tokens one by one; returns logits [len(tokens), vocab] (and, if asked, the residual after every
        layer, [layers, tokens, width])."""
        cfg, eps = self.cfg, self.eps
        logits, residuals = [], []
        for token in tokens:
            p = request["length"]
            x = self.t["embed"][token] * cfg["embedding"]["scale"]
            per_layer = []
            for i, layer in enumerate(cfg["layers"]):
                kind, m, f = layer["type"], layer["mixer"], layer.get("mlp")
                w = self._sub(f"l{i}.mix.")
                h = rms_norm(x, eps, self.t[f"l{i}.norm1"], one_plus=True)
                if kind == "attention":
                    src = m.get("kv_from")
                    cache = request["layers"][i if src is None else src]
                    y = Attention.step(w, m, eps, h, p, cache, writes=src is None)
                else:
                    y = MIXERS[kind].step(w, m, eps, h, p, request["layers"][i])
                x = x + y
                if f is not None:
                    h = rms_norm(x, eps, self.t[f"l{i}.norm2"], one_plus=True)
                    wf = self._sub(f"l{i}.mlp.")
                    x = x + (dense_mlp(wf, h) if f["kind"] == "dense" else experts_mlp(wf, f, h))
                per_layer.append(x)
            request["length"] = p + 1
            z = self.t["head"] @ rms_norm(x, eps, self.t["final.norm"], one_plus=True)
            cap = cfg.get("logit_softcap")
            if cap:
                z = cap * torch.tanh(z / cap)
            logits.append(z)
            residuals.append(torch.stack(per_layer))
        out = torch.stack(logits)
        if keep_layers:
            return out, torch.stack(residuals, dim=1)
        return out


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))
