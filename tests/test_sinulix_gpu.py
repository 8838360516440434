"""The Sinulix design in the engine against its plain statement (tests/plain_sinulix.py): the new kernels alone, each
mechanism alone in a model, then whole models in every way of cutting the work (whole prompts, a decoded tail,
portions down to two tokens, mixed batches with pages and state slots used again), tokens far back that carry the
result, long decoding through captured graphs, and greedy generation through the entry point and its scheduler.
Cache pages are poisoned with NaN so that a read outside a request's own rows shows."""
import copy
import random

import numpy as np
import pytest
import torch

import helpers
import plain_sinulix as plain
import sinulix_helpers as sh

pytestmark = pytest.mark.gpu

TOL = {"float32": 5e-5, "bfloat16": 4e-2}     # relative to the largest |logit| of the plain statement
LENGTHS = [1, 7, 33, 90, 61, 47, 2, 70, 18, 120, 64, 65, 3]


def row_errors(got, want):
    scale = max(float(np.abs(w).max()) for w in want.values())
    return np.array([float(np.abs(got[r][p].astype(np.float64) - want[r][p]).max()) / scale
                     for r in sorted(got) for p in sorted(got[r])])


def agrees(got, want, dtype):
    """float32: every row within the tolerance; this is what judges the cache, the state and the batching.
    bfloat16: activations rounded to 8 bits through several layers (and now and then an expert chosen otherwise on a
    close call) leave a few rows further off than the typical row, so nearly all rows must be within the tolerance,
    the typical row well within it, and none far outside."""
    err = row_errors(got, want)
    if not np.isfinite(err).all():
        return False
    if dtype == "float32":
        return bool(err.max() <= TOL[dtype])
    return bool((err > TOL[dtype]).mean() <= 0.03 and np.median(err) <= TOL[dtype] / 3 and err.max() <= 4 * TOL[dtype])


def run(folder, dtype, steps, page, **kw):
    from tinyinfer_b200.engine.replay import TraceSession
    session = TraceSession(folder, dtype, helpers.peak_tokens(steps, max(64, page)), page_size=page, poison_cache=True, **kw)
    got = helpers.collect(session, steps)
    session.runner.check_status()
    session.runner.manager.check_consistency()
    return got, session


# ------------------------------------------------------------------ the kernels alone
def delta_plain(q, k, v, g, beta, S):
    """S [H, dk, dv]; q, k, g [T, H, dk]; v [T, H, dv]; beta [T, H]. Returns o [T, H, dv] and the last S."""
    out = []
    for t in range(q.shape[0]):
        S = g[t][:, :, None] * S
        u = beta[t][:, None] * (v[t] - torch.einsum("hkv,hk->hv", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        out.append(torch.einsum("hkv,hk->hv", S, q[t]))
    return torch.stack(out), S


@pytest.mark.parametrize("heads,groups,dk,dv", [(3, 3, 24, 20), (6, 2, 20, 12), (2, 1, 130, 9), (1, 1, 8, 70),
                                                (4, 4, 64, 64), (2, 2, 128, 128), (4, 1, 12, 36)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_delta_scan_against_plain(heads, groups, dk, dv, dtype):
    """Two requests of unequal length in three calls (a prompt's portion, then a portion beside one decoded token, then
    a portion of many of the kernel's chunks beside a short one): the state goes through slots that lie inside a
    larger state, with someone else's floats in front."""
    from tinyinfer_b200 import ops
    gen = torch.Generator().manual_seed(heads * dk + dv)
    pad = 5
    a_log, dt_bias = torch.randn(heads, generator=gen) - 2, 0.5 * torch.randn(heads * dk, generator=gen)
    state_d = torch.zeros(3, 11 + heads * dk * dv).cuda()
    view = state_d[:, 11:].unflatten(1, (heads, dv, dk))
    S = [torch.zeros(heads, dk, dv, dtype=torch.float64) for _ in range(2)]
    per = heads // groups
    for lens in ([37, 5], [1, 22], [3, 141]):
        T = sum(lens)
        row = torch.randn(T, pad + 2 * groups * dk + heads * dv, generator=gen).to(dtype)
        a = torch.randn(T, 3 + heads * dk, generator=gen)
        b = torch.randn(T, 2 + heads, generator=gen)
        cu = torch.tensor([0, lens[0], T], dtype=torch.int32)
        slots = torch.tensor([2, 0], dtype=torch.int32)
        rd = row.cuda()
        got = ops.delta_scan(rd, rd, rd, a.cuda(), b.cuda(), a_log=a_log.cuda(), dt_bias=dt_bias.cuda(), state=view,
                             heads=heads, groups=groups, key_dim=dk, value_dim=dv, q_offset=pad, k_offset=pad + groups * dk,
                             v_offset=pad + 2 * groups * dk, decay_offset=3, beta_offset=2, q_scale=dk ** -0.5,
                             unit_eps=1e-6, cu_seqlens=cu.cuda(), state_slots=slots.cuda(), num_seqs=2).cpu()
        r = row.double()
        q = r[:, pad:pad + groups * dk].reshape(T, groups, dk)
        k = r[:, pad + groups * dk:pad + 2 * groups * dk].reshape(T, groups, dk)
        q = (q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5).repeat_interleave(per, dim=1)
        k = (k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)).repeat_interleave(per, dim=1)
        v = r[:, pad + 2 * groups * dk:].reshape(T, heads, dv)
        dt = plain.softplus(a[:, 3:].double() + dt_bias.double()).reshape(T, heads, dk)
        g = torch.exp(-torch.exp(a_log.double())[None, :, None] * dt)
        beta = torch.sigmoid(b[:, 2:].double())
        at = 0
        for i, n in enumerate(lens):
            want, S[i] = delta_plain(q[at:at + n], k[at:at + n], v[at:at + n], g[at:at + n], beta[at:at + n], S[i])
            assert (got[at:at + n].double().reshape(n, heads, dv) - want).abs().max() <= 2e-5 * max(1.0, want.abs().max()), (i, lens)
            at += n
    kept = state_d.cpu()
    assert (kept[:, :11] == 0).all() and (kept[1] == 0).all()
    for i, slot in enumerate((2, 0)):
        assert (kept[slot, 11:].reshape(heads, dv, dk).transpose(1, 2).double() - S[i]).abs().max() <= 2e-5 * max(1.0, S[i].abs().max())


def test_delta_rule_overwrites_a_key():
    """With beta = 1, no decay and the same unit key twice, the second value replaces the first: what a query along
    that key reads is the second value alone, and a key at right angles keeps its own value."""
    from tinyinfer_b200 import ops
    dk, dv = 16, 8
    row = torch.zeros(3, 2 * dk + dv)
    row[0, 0], row[0, dk + 0], row[0, 2 * dk:] = 1.0, 1.0, torch.arange(dv) + 1.0          # write v0 under key e0
    row[1, 1], row[1, dk + 1], row[1, 2 * dk:] = 1.0, 1.0, -2.0                            # v1 under e1
    row[2, 0], row[2, dk + 0], row[2, 2 * dk:] = 1.0, 1.0, 7.0                             # v2 under e0 again
    a = torch.full((3, dk), -80.0)                                                          # softplus -> 0: g = 1
    b = torch.full((3, 1), 80.0)                                                            # beta = 1
    state = torch.zeros(1, 1, dv, dk).cuda()
    got = ops.delta_scan(row.cuda(), row.cuda(), row.cuda(), a.cuda(), b.cuda(), a_log=torch.zeros(1).cuda(), dt_bias=None,
                         state=state, heads=1, groups=1, key_dim=dk, value_dim=dv, q_offset=0, k_offset=dk, v_offset=2 * dk,
                         q_scale=1.0, unit_eps=0.0, cu_seqlens=torch.tensor([0, 3], dtype=torch.int32).cuda(),
                         state_slots=torch.zeros(1, dtype=torch.int32).cuda(), num_seqs=1).cpu()
    assert torch.allclose(got[0], torch.arange(dv) + 1.0) and torch.allclose(got[1], torch.full((dv,), -2.0))
    assert torch.allclose(got[2], torch.full((dv,), 7.0), atol=1e-5)
    S = state.cpu()[0, 0]                                                                   # [dv, dk]
    assert torch.allclose(S[:, 0], torch.full((dv,), 7.0), atol=1e-5) and torch.allclose(S[:, 1], torch.full((dv,), -2.0))


@pytest.mark.parametrize("hq,hkv,d,dv,rot,normed", [(6, 2, 20, 12, 12, True), (3, 3, 16, 16, 16, False), (4, 1, 8, 24, 0, True),
                                                    (8, 8, 128, 128, 64, False)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_head_rotation_rows_against_plain(hq, hkv, d, dv, rot, normed, dtype):
    """The row form (for a recurrent mixer): norm, a rotation of the first features only, factors; values pass."""
    from tinyinfer_b200 import ops
    from tinyinfer_b200.config import PositionSpec
    from tinyinfer_b200.parts.base import build_position
    gen = torch.Generator().manual_seed(hq * d + rot)
    T, off = 11, 3
    rows = torch.randn(T, off + hq * d + hkv * (d + dv) + 2, generator=gen).to(dtype)
    pos = torch.tensor([0, 1, 2, 500, 501, 7, 100000, 3, 64, 65, 4095], dtype=torch.int32)
    wq, wk = 1 + 0.3 * torch.randn(d, generator=gen), 1 + 0.3 * torch.randn(d, generator=gen)
    spec = PositionSpec(kind="rope", theta=777.0, rotary_dim=rot, exact_frequencies=True) if rot else PositionSpec(kind="none")
    rotation = build_position(spec, dtype, "cuda").rotation()
    got = ops.head_rotation(rows.cuda(), num_heads=hq, num_kv_heads=hkv, head_dim=d, v_dim=dv, has_kv=True,
                            positions=pos.cuda(), token_seq=torch.zeros(T, dtype=torch.int32).cuda(), offset=off,
                            q_norm_weight=wq.cuda() if normed else None, k_norm_weight=wk.cuda() if normed else None,
                            eps=1e-5, rotation=rotation, q_scale=1.0, k_scale=d ** -0.5, out_float32=True).cpu().double()
    r = rows.double()
    for t in range(T):
        q = r[t, off:off + hq * d].view(hq, d)
        k = r[t, off + hq * d:off + (hq + hkv) * d].view(hkv, d)
        if normed:
            q, k = plain.rms_norm(q, 1e-5, wq.double()), plain.rms_norm(k, 1e-5, wk.double())
        q = plain.rotate(q, int(pos[t]), rot, 777.0)
        k = plain.rotate(k, int(pos[t]), rot, 777.0) * d ** -0.5
        want = torch.cat([q.reshape(-1), k.reshape(-1), r[t, off + (hq + hkv) * d:off + (hq + hkv) * d + hkv * dv]])
        # a float32 angle p * f carries a rounding of about 1e-7 of its size: 4e-4 radians at position 4,095
        tol = 2e-5 + 3e-7 * int(pos[t])
        assert (got[t] - want).abs().max() <= tol * max(1.0, want.abs().max()), t


def attention_plain(q, keys, values, scale, sinks, gate):
    """q [Hq, d]; keys [n, Hkv, d]; values [n, Hkv, dv]; sinks, gate [Hq] (gate: logits). Returns [Hq * dv]."""
    hq, per = q.shape[0], q.shape[0] // keys.shape[1]
    out = []
    for h in range(hq):
        s = (keys[:, h // per] @ q[h]) * scale
        top = torch.maximum(s.max(), sinks[h])
        e = torch.exp(s - top)
        p = e / (e.sum() + torch.exp(sinks[h] - top))
        out.append((p[:, None] * values[:, h // per]).sum(0) * torch.sigmoid(gate[h]))
    return torch.cat(out)


ATTENTION_SHAPES = [
    # hq, hkv, d, dv, page, [(context, q_len)]
    (6, 2, 20, 12, 8, [(37, 37), (50, 1), (9, 2)]),                       # rows of [k | v]: the float32-arithmetic kernel
    (3, 1, 8, 40, 4, [(130, 1), (17, 17)]),
    (8, 2, 64, 64, 16, [(130, 130), (129, 1), (200, 2)]),                 # two planes: the tensor-core kernels
    (8, 4, 128, 128, 64, [(1500, 1), (1, 1), (256, 1), (257, 1), (700, 513)]),
    (4, 4, 128, 128, 64, [(1300, 897), (64, 64), (65, 1)]),
    (6, 2, 64, 64, 16, [(150, 150), (131, 1), (90, 3)]),                   # odd numbers of query heads a key head
    (5, 1, 128, 128, 32, [(300, 1), (70, 70), (33, 2)]),
    (14, 2, 64, 64, 64, [(200, 1), (129, 129)]),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("pairs", [False, True])
@pytest.mark.parametrize("hq,hkv,d,dv,page,work", ATTENTION_SHAPES)
def test_attention_with_head_sinks_and_gates(monkeypatch, dtype, pairs, hq, hkv, d, dv, page, work):
    """A sink per head in the denominator and a gate per (token, head) on the output, in every attention kernel that
    a layer of this kind can reach; with sinks from tiny to dominant so that each head differs."""
    from tinyinfer_b200 import ops
    if pairs and (d != dv or d < 128 or dtype == torch.float32):
        pytest.skip("one CTA pair form")
    monkeypatch.setattr(ops, "PAIR_MIN_CTAS", 0 if pairs else 1 << 30)
    gen = torch.Generator().manual_seed(hq * d)
    lens = [c for c, _ in work]
    pages_of = [(n + page - 1) // page for n in lens]
    total = sum(pages_of) + 3
    perm = torch.randperm(total, generator=gen).tolist()
    width = max(pages_of)
    tables, nxt = [], 0
    for nb in pages_of:
        tables.append(perm[nxt:nxt + nb] + [-1] * (width - nb))
        nxt += nb
    bt = torch.tensor(tables, dtype=torch.int32)
    planes = d == dv
    cache = torch.full((2, total, hkv, page, d) if planes else (1, total, hkv, page, d + dv), float("nan"), dtype=dtype)
    ks = [torch.randn(n, hkv, d, generator=gen).to(dtype) for n in lens]
    vs = [torch.randn(n, hkv, dv, generator=gen).to(dtype) for n in lens]
    for i, n in enumerate(lens):
        for p in range(n):
            pg = tables[i][p // page]
            if planes:
                cache[0, pg, :, p % page], cache[1, pg, :, p % page] = ks[i][p], vs[i][p]
            else:
                cache[0, pg, :, p % page] = torch.cat([ks[i][p], vs[i][p]], dim=-1)
    pos = torch.tensor([p for c, n in work for p in range(c - n, c)], dtype=torch.int32)
    seq = torch.tensor([i for i, (c, n) in enumerate(work) for _ in range(n)], dtype=torch.int32)
    T = pos.shape[0]
    q = (2.0 * torch.randn(T, hq, d, generator=gen)).to(dtype)
    sinks = torch.linspace(-20.0, 6.0, hq)
    gate = torch.randn(T, 5 + hq, generator=gen).to(dtype)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    args = dict(positions=pos.cuda(), token_seq=seq.cuda(), block_table=bt.cuda(), scale=d ** -0.5, status=status,
                head_sinks=sinks.cuda(), gate=gate.cuda(), gate_offset=5)
    if planes:
        out = ops.paged_attention(q.cuda(), cache.cuda(), **args)
    else:
        out = ops.attention_rows(q.cuda(), cache.cuda(), v_dim=dv, **args)
    assert int(status.item()) == 0
    out = out.cpu().double()
    worst = 0.0
    for t in range(T):
        i, p = int(seq[t]), int(pos[t])
        want = attention_plain(q[t].double(), ks[i][:p + 1].double(), vs[i][:p + 1].double(), d ** -0.5, sinks.double(),
                               gate[t, 5:].double())
        worst = max(worst, float((out[t] - want).abs().max()))
    assert worst <= (2e-5 if dtype == torch.float32 else 2e-2), worst


@pytest.mark.parametrize("experts,identity,top,ff,width,tokens", [(5, 2, 2, 24, 72, 37), (1, 1, 1, 16, 40, 9), (3, 0, 3, 8, 40, 5),
                                                                  (16, 3, 4, 64, 128, 600)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_experts_with_corrections_and_identity_experts(experts, identity, top, ff, width, tokens, dtype):
    """The router's choice by score + correction with plain scores as weights, the clamped gate, identity experts and
    the weighted sum, op by op as the experts' part strings them together. Router logits are drawn apart (no close
    calls), limits are small enough that the clamps bite."""
    from tinyinfer_b200 import ops
    gen = torch.Generator().manual_seed(experts * 7 + top)
    outputs = experts + identity
    x = torch.randn(tokens, width, generator=gen).to(dtype)
    router = (3.0 * torch.randn(outputs, width, generator=gen) / width ** 0.5).to(dtype)
    correction = 0.4 * torch.randn(outputs, generator=gen)
    up = (torch.randn(experts, 2 * ff, width, generator=gen) / width ** 0.5).to(dtype)
    down = (torch.randn(experts, width, ff, generator=gen) / ff ** 0.5).to(dtype)
    limit = 0.7
    xd = x.cuda()
    routing = ops.route_experts(xd, router.cuda(), top, 0.0, tile_rows=ops.expert_tile_rows(xd, experts, top, ff),
                                correction=correction.cuda(), renormalize=False, real_experts=experts)
    scores = torch.softmax(x.double() @ router.double().t(), dim=-1)
    choice = scores + correction.double()
    want_chosen = torch.topk(choice, top).indices
    ranked = torch.sort(choice, dim=-1, descending=True).values
    clear = (ranked[:, top - 1] - ranked[:, top]) > 1e-3 if top < outputs else torch.ones(tokens, dtype=torch.bool)
    got_chosen = routing.chosen.cpu().long()
    assert clear.float().mean() > 0.9
    assert torch.equal(torch.sort(got_chosen[clear], dim=-1).values, torch.sort(want_chosen[clear], dim=-1).values)
    assert (routing.weight.cpu().double() - torch.gather(scores, 1, got_chosen)).abs().max() < 1e-5
    # the weights are not renormalized: they sum to less than one wherever something was not chosen
    if top < outputs:
        assert float(routing.weight.sum(-1).max()) < 1.0
    hidden = ops.clamped_glu(ops.expert_linear(xd, up.cuda(), routing, up=True, activation=False), limit, 1.702)
    rows = ops.expert_linear(hidden, down.cuda(), routing, up=False)
    got = ops.experts_combine(rows, xd, routing, experts).cpu().double()
    want = torch.zeros(tokens, width, dtype=torch.float64)
    clamped = 0
    for t in range(tokens):
        h = x[t].double()
        for c in range(top):
            e, wgt = int(got_chosen[t, c]), scores[t, got_chosen[t, c]]
            if e >= experts:
                want[t] += wgt * h
                continue
            gu = up[e].double() @ h
            if dtype == torch.bfloat16:
                gu = gu.to(dtype).double()
            g, u = torch.clamp(gu[:ff], max=limit), torch.clamp(gu[ff:], -limit, limit)
            clamped += int((gu[:ff] > limit).sum() + (gu[ff:].abs() > limit).sum())
            y = g * torch.sigmoid(1.702 * g) * (u + 1.0)
            if dtype == torch.bfloat16:
                y = y.to(dtype).double()
            want[t] += wgt * (down[e].double() @ y)
    assert clamped > 0 or experts == 1
    assert (got - want).abs().max() <= (2e-5 if dtype == torch.float32 else 3e-2) * max(1.0, want.abs().max())


def test_soft_cap_scaled_embedding_and_sigmoid_gate():
    from tinyinfer_b200 import ops
    z = torch.linspace(-90, 90, 1001)
    assert (ops.soft_cap_(z.clone().cuda(), 13.0).cpu().double() - 13.0 * torch.tanh(z.double() / 13.0)).abs().max() < 1e-5
    table = torch.randn(50, 24)
    ids = torch.tensor([3, 49, 0, 3], dtype=torch.int32)
    for dtype in (torch.float32, torch.bfloat16):
        got = ops.streams_embed(ids.cuda(), table.to(dtype).cuda(), 1, 6.5)
        assert got.dtype == torch.float32 and torch.equal(got.cpu()[0], table.to(dtype).float()[ids.long()] * 6.5)
    gen = torch.Generator().manual_seed(5)
    y, gate, w = torch.randn(7, 60, generator=gen), torch.randn(7, 60, generator=gen), 1 + 0.3 * torch.randn(12, generator=gen)
    got = ops.gated_group_norm(y.cuda(), gate.cuda(), w.cuda(), group=12, eps=1e-5, gate_first=False, out_dtype=torch.float32,
                               gate_activation="sigmoid").cpu().double()
    want = plain.rms_norm(y.double().reshape(7, 5, 12), 1e-5, w.double()).reshape(7, 60) * torch.sigmoid(gate.double())
    assert (got - want).abs().max() < 1e-5


# ------------------------------------------------------------------ each mechanism alone
def single(kind, mlp=None, **kw):
    if kind == "attention":
        layers = [sh.layer("attention", sh.attention(6, 2, 20, 12, scale=0.35, rot=12), mlp)]
    elif kind == "attention_planes":
        layers = [sh.layer("attention", sh.attention(4, 2, 64, 64, scale=0.2, rot=32), mlp)]
    elif kind == "shared":
        layers = [sh.layer("attention", sh.attention(4, 4, 12, 20, rot=4), mlp),
                  sh.layer("attention", sh.attention(4, 4, 12, 20, rot=4, kv_from=0), mlp),
                  sh.layer("attention", sh.attention(4, 4, 12, 20, rot=4, kv_from=0), None)]
    elif kind == "retention":
        layers = [sh.layer("retention", sh.retention(3, 20, 12, rot=8), mlp)]
    elif kind == "delta":
        layers = [sh.layer("channel_delta", sh.delta(6, 3, 12, 20, conv=4), mlp)]
    else:
        raise ValueError(kind)
    return sh.config(layers, **kw)


@pytest.mark.parametrize("kind,mlp", [("attention", None), ("attention_planes", None), ("shared", None), ("retention", None),
                                      ("delta", None), ("retention", sh.dense(56)), ("delta", sh.moe(6, 2, 24, identity=2)),
                                      ("attention", sh.moe(4, 4, 16, identity=0, limit=0.5))])
def test_one_mechanism_alone(tmp_path, kind, mlp):
    cfg = single(kind, mlp)
    folder = sh.write_folder(tmp_path / "m", cfg, seed=11)
    requests = sh.random_requests(cfg, [75, 1, 2, 19], seed=4)
    want = sh.plain_logits(folder, requests)
    for steps in (helpers.trace_whole(requests), helpers.trace_chunked(requests, seed=3), helpers.trace_decode_tail(requests, tail=80)):
        got, _ = run(folder, "float32", steps, page=8)
        assert helpers.first_bad(got, want, TOL["float32"]) is None


def test_residual_after_every_layer(tmp_path):
    """The float32 stream after every layer of a prompt, not only the logits at its end."""
    from tinyinfer_b200.engine.replay import TraceSession
    cfg = sh.MIX
    folder = sh.write_folder(tmp_path / "m", cfg, seed=2)
    tokens = sh.random_requests(cfg, [23], seed=1)["r0"]
    c, w = sh.read_folder(folder)
    model = plain.PlainSinulix(c, w, torch.float64)
    _, want = model.feed(model.new_request(), tokens, keep_layers=True)            # [layers, tokens, width]
    session = TraceSession(folder, "float32", 64, page_size=8, cuda_graphs=False)
    got = []
    for block in session.model.blocks:          # a block returns the stream and the update that the next norm applies
        inner = block.forward_linked

        def watched(x, link, next_norm, step, cache, _inner=inner):
            out = _inner(x, link, next_norm, step, cache)
            (stream, pending), _ = out
            got.append((stream[0] + pending.y.float()).detach().cpu().double())
            return out
        block.forward_linked = watched
    session.run_step({"step": 0, "entries": [{"id": "a", "tokens": tokens, "want": [len(tokens) - 1]}], "end": ["a"]})
    assert len(got) == len(cfg["layers"])
    for i, rows in enumerate(got):
        assert (rows.reshape(len(tokens), -1) - want[i]).abs().max() <= 2e-5 * want[i].abs().max(), i


# ------------------------------------------------------------------ whole models, every cut
def traces_for(requests, max_live=4):
    return {"whole": helpers.trace_whole(requests), "tail": helpers.trace_decode_tail(requests, tail=32),
            "chunked": helpers.trace_chunked(requests, seed=1), "mixed": helpers.trace_mixed(requests, seed=2, max_live=max_live)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,page", [("MIX", 8), ("WIDE", 16), ("ONE", 4)])
def test_every_cut_matches_plain(tmp_path, name, page, dtype):
    cfg = getattr(sh, name)
    folder = sh.write_folder(tmp_path / name, cfg, seed=3, dtype=dtype)
    requests = sh.random_requests(cfg, LENGTHS, seed=5)
    want = sh.plain_logits(folder, requests)
    results = {}
    for tag, steps in traces_for(requests).items():
        got, session = run(folder, dtype, steps, page, max_live=4)
        assert {r: len(v) for r, v in got.items()} == {r: len(t) for r, t in requests.items()}, tag
        assert agrees(got, want, dtype), (tag, helpers.first_bad(got, want, TOL[dtype]), np.sort(row_errors(got, want))[-8:])
        if tag == "mixed":
            stats = session.runner.manager.stats()
            assert all(g["pages_taken"] > g["pages"] for g in stats["groups"]), "pages were not used again"
        results[tag] = got
    for tag in ("tail", "chunked", "mixed"):        # the cuts against each other: rounding only
        assert agrees(results[tag], {r: np.stack([results["whole"][r][p] for p in range(len(t))]) for r, t in requests.items()},
                      dtype), tag


def test_two_state_slots_serve_many_requests(tmp_path):
    """Slots (convolution histories and matrix states) and pages are handed from finished requests to new ones; a
    slot that is taken again starts from zero, not from what its last owner left."""
    cfg = sh.MIX
    folder = sh.write_folder(tmp_path / "m", cfg, seed=8)
    requests = sh.random_requests(cfg, [30, 9, 41, 2, 17, 55, 5, 26], seed=9)
    want = sh.plain_logits(folder, requests)
    steps = helpers.trace_mixed(requests, seed=4, max_live=2, decode_tail=6)
    got, session = run(folder, "float32", steps, page=4, max_live=2)
    assert helpers.first_bad(got, want, TOL["float32"]) is None
    assert session.runner.manager.stats()["free_state_slots"] == 2


def test_batch_of_unequal_requests_equals_each_alone(tmp_path):
    cfg = sh.WIDE
    folder = sh.write_folder(tmp_path / "m", cfg, seed=5)
    requests = sh.random_requests(cfg, [50, 3, 128, 17], seed=2)
    together = [{"step": 0, "entries": [{"id": r, "tokens": t, "want": list(range(len(t)))} for r, t in requests.items()],
                 "end": list(requests)}]
    got, _ = run(folder, "float32", together, page=16)
    alone, _ = run(folder, "float32", helpers.trace_whole(requests), page=16)
    want = sh.plain_logits(folder, requests)
    assert helpers.first_bad(got, want, TOL["float32"]) is None
    scale = max(float(np.abs(w).max()) for w in want.values())
    assert max(float(np.abs(got[r][p] - alone[r][p]).max()) for r in requests for p in got[r]) / scale <= 1e-5


def test_a_request_left_out_of_steps_goes_on(tmp_path):
    """A request pauses for some steps while others run and end (their slots and pages change hands meanwhile)."""
    cfg = sh.MIX
    folder = sh.write_folder(tmp_path / "m", cfg, seed=4)
    requests = sh.random_requests(cfg, [40, 21, 33], seed=7)
    a, b, c = (requests[f"r{i}"] for i in range(3))
    want = sh.plain_logits(folder, requests)
    every = lambda toks, lo, hi: {"tokens": toks[lo:hi], "want": list(range(hi - lo))}
    steps = [
        {"step": 0, "entries": [dict(id="r0", **every(a, 0, 13)), dict(id="r1", **every(b, 0, 21))], "end": ["r1"]},
        {"step": 1, "entries": [dict(id="r2", **every(c, 0, 2))], "end": []},
        {"step": 2, "entries": [dict(id="r2", **every(c, 2, 33))], "end": ["r2"]},
        {"step": 3, "entries": [dict(id="r0", **every(a, 13, 14))], "end": []},
        {"step": 4, "entries": [dict(id="r0", **every(a, 14, 40))], "end": ["r0"]},
    ]
    got, _ = run(folder, "float32", steps, page=8, max_live=2)
    assert helpers.first_bad(got, want, TOL["float32"]) is None


# ------------------------------------------------------------------ tokens far back, page borders, the first tokens
def sharp_config():
    """Softmax scores sharp enough that one key anywhere in the context takes nearly all the weight of a head (or
    the sink does); decays so close to one that the first tokens are still in every matrix state at the end."""
    a = sh.attention(4, 2, 16, 24, scale=3.0, rot=8)
    return sh.config([
        sh.layer("attention", a, sh.dense(48)),
        sh.layer("retention", sh.retention(2, 16, 16, decay=[0.999, 0.9995], rot=16), None),
        sh.layer("attention", dict(a, kv_from=0), None),
        sh.layer("channel_delta", sh.delta(2, 1, 16, 16, conv=2), sh.dense(48)),
    ], width=64)


def slow_decay(t):
    t["l3.mix.A_log"] = torch.full_like(t["l3.mix.A_log"], -7.0)
    t["l0.mix.sink"] = torch.tensor([-30.0, 0.0, 4.0, 9.0])


def test_far_tokens_carry_the_result(tmp_path):
    """Positions around the borders of pages and of the kernels' key tiles are decoded one by one; cutting the first 64
    tokens off moves the last logits by far more than the tolerance, so a missing or misplaced row, or a state lost
    on the way, shows."""
    cfg = sharp_config()
    folder = sh.write_folder(tmp_path / "m", cfg, seed=21, edit=slow_decay)
    requests = sh.random_requests(cfg, [700], seed=13)
    tokens = requests["r0"]
    want = sh.plain_logits(folder, requests)
    c, w = sh.read_folder(folder)
    cut = sh.forward(c, w, tokens[64:])
    assert np.abs(cut[-40:] - want["r0"][-40:]).max() > 100 * TOL["float32"] * np.abs(want["r0"]).max()
    for steps in (helpers.trace_whole(requests), helpers.trace_decode_tail(requests, tail=140),
                  helpers.trace_chunked(requests, seed=7)):
        got, _ = run(folder, "float32", steps, page=16)
        assert helpers.first_bad(got, want, TOL["float32"]) is None
    folder16 = sh.write_folder(tmp_path / "m16", cfg, seed=21, dtype="bfloat16", edit=slow_decay)
    want16 = sh.plain_logits(folder16, requests)
    for steps in (helpers.trace_whole(requests), helpers.trace_decode_tail(requests, tail=140),
                  helpers.trace_chunked(requests, seed=7)):
        got, _ = run(folder16, "bfloat16", steps, page=16)
        err = row_errors(got, want16)
        assert np.isfinite(err).all() and np.median(err) <= 3e-2 and (err > 0.2).mean() <= 0.02, np.sort(err)[-5:]


def test_one_far_key_among_hundreds(tmp_path):
    """One query head is scaled so that the key of one early token outscores all others by a wide margin: the logits
    at the end then hang on that token's value. The same prompt with that token replaced differs at the end; the
    engine agrees with the plain statement on both, decoded through the cache, at several page sizes."""
    cfg = sh.config([sh.layer("attention", sh.attention(2, 1, 16, 16, scale=1.0, rot=0), None),
                     sh.layer("attention", sh.attention(2, 1, 16, 16, scale=1.0, rot=0, kv_from=0), sh.dense(32))], width=32)

    def loud(t):
        t["l0.mix.q"] *= 6.0
        t["l0.mix.sink"] = torch.tensor([-5.0, -5.0])
    folder = sh.write_folder(tmp_path / "m", cfg, seed=5, edit=loud)
    base = sh.random_requests(cfg, [300], seed=3)["r0"]
    c, w = sh.read_folder(folder)
    full = sh.forward(c, w, base)
    # which early token the last position looks at most is found from the plain statement itself: replace each of a
    # few candidates and keep the one that moves the last logits most
    moves = {}
    for p in (3, 15, 16, 17, 31, 32, 63, 64, 65):
        other = list(base)
        other[p] = (other[p] + 1) % cfg["vocab"]
        moves[p] = float(np.abs(sh.forward(c, w, other)[-1] - full[-1]).max())
    far = max(moves, key=moves.get)
    assert moves[far] > 1e-3 * np.abs(full).max()
    changed = list(base)
    changed[far] = (changed[far] + 1) % cfg["vocab"]
    requests = {"r0": base, "r1": changed}
    want = sh.plain_logits(folder, requests)
    for page in (4, 16, 64):
        got, _ = run(folder, "float32", helpers.trace_decode_tail(requests, tail=40), page=page)
        assert helpers.first_bad(got, want, TOL["float32"]) is None, page


def test_the_first_tokens(tmp_path):
    """Position zero (no rotation angle, an empty state, a convolution that sees only zeros behind it, a softmax of
    one key and the sink), then the next few, as prompts of one to six tokens and decoded one by one from the start."""
    cfg = sh.MIX
    folder = sh.write_folder(tmp_path / "m", cfg, seed=12)
    requests = sh.random_requests(cfg, [1, 2, 3, 4, 5, 6], seed=8)
    want = sh.plain_logits(folder, requests)
    got, _ = run(folder, "float32", helpers.trace_whole(requests), page=4)
    assert helpers.first_bad(got, want, TOL["float32"]) is None
    got, _ = run(folder, "float32", helpers.trace_decode_tail(requests, tail=6), page=4)
    assert helpers.first_bad(got, want, TOL["float32"]) is None


# ------------------------------------------------------------------ long decoding through graphs
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_replays_graphs(tmp_path, dtype):
    cfg = sh.MIX
    folder = sh.write_folder(tmp_path / "m", cfg, seed=6, dtype=dtype)
    requests = sh.random_requests(cfg, [160, 150], seed=1)
    want = sh.plain_logits(folder, requests)
    steps = [{"step": 0, "entries": [{"id": r, "tokens": t[:4], "want": [0, 1, 2, 3]} for r, t in requests.items()], "end": []}]
    for p in range(4, 150):
        steps.append({"step": p, "entries": [{"id": r, "tokens": [t[p]], "want": [0]} for r, t in requests.items()],
                      "end": list(requests) if p == 149 else []})
    got, session = run(folder, dtype, steps, page=8)
    assert session.runner.graph_replays > 100
    assert agrees(got, {r: w[:150] for r, w in want.items()}, dtype)


# ------------------------------------------------------------------ generation through the entry point
@pytest.mark.parametrize("dtype,tol", [("float32", 1e-4), ("bfloat16", 6e-2)])
def test_greedy_generation_through_the_scheduler(tmp_path, dtype, tol):
    from tinyinfer_b200 import LLM
    from tinyinfer_b200.sampling import SamplingParams
    cfg = sh.MIX
    folder = sh.write_folder(tmp_path / "m", cfg, seed=3, dtype=dtype)
    llm = LLM(folder, dtype=dtype, max_num_batched_tokens=24, max_num_seqs=3, kvcache_block_size=8,
              num_kvcache_blocks=40, prefill_chunk=9, max_model_len=128)
    assert llm.config.enable_prefix_caching is False          # a state cannot be rebuilt from pages
    prompts = list(sh.random_requests(cfg, [1, 7, 16, 33, 50], seed=6).values())
    outs = llm.generate(prompts, SamplingParams(greedy=True, max_tokens=10))
    c, w = sh.read_folder(folder)
    for p, o in zip(prompts, outs):
        assert o["all_token_ids"] == p + o["token_ids"] and len(o["token_ids"]) == 10
        logits = sh.forward(c, w, p + o["token_ids"])
        for i, tok in enumerate(o["token_ids"]):          # teacher forcing: the token has (nearly) the largest plain logit
            row = logits[len(p) - 1 + i]
            assert row.max() - row[tok] <= tol * np.abs(logits).max()
    assert not llm.runner.manager.live_requests
    llm.runner.manager.check_consistency()
    llm.close()


def test_command_line_generates_with_a_folder_and_with_a_preset(tmp_path):
    import json
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    folder = sh.write_folder(tmp_path / "m", sh.ONE, seed=3)
    common = ["--dtype", "fp32", "--prompt-ids", "5,17,3,200", "--prompt-len", "9", "--greedy", "--max-tokens", "6",
              "--max-num-seqs", "2", "--max-num-batched-tokens", "16", "--block-size", "4", "--num-kvcache-blocks", "32",
              "--max-model-len", "64"]
    res = subprocess.run([sys.executable, str(root / "examples" / "generate.py"), "--model", str(folder)] + common,
                         capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    rows = [json.loads(l) for l in res.stdout.splitlines() if l.startswith("{")]
    assert len(rows) == 2 and all(len(r["token_ids"]) == 6 for r in rows)
    c, w = sh.read_folder(folder)
    logits = sh.forward(c, w, [5, 17, 3, 200] + rows[0]["token_ids"])
    for i, tok in enumerate(rows[0]["token_ids"]):
        assert logits[3 + i].max() - logits[3 + i][tok] <= 1e-4 * np.abs(logits).max()
    res = subprocess.run([sys.executable, str(root / "examples" / "generate.py"), "--random-config", "sinulix-tiny"] + common,
                         capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]


def test_trace_runner_program(tmp_path):
    """The replay program itself: steps on standard input, a file of logits per step that wants some, 'done' lines."""
    import json
    import subprocess
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    cfg = sh.ONE
    folder = sh.write_folder(tmp_path / "m", cfg, seed=9, dtype="bfloat16")
    requests = sh.random_requests(cfg, [20, 70, 9], seed=2)
    steps = helpers.trace_mixed(requests, seed=1, max_live=3, decode_tail=5)
    out = tmp_path / "out"
    out.mkdir()
    res = subprocess.run([str(root / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(out),
                          "--max-tokens", str(helpers.peak_tokens(steps))], input="".join(json.dumps(s) + "\n" for s in steps),
                         capture_output=True, text=True, timeout=1200)
    assert res.returncode == 0, res.stderr[-2000:]
    assert [l for l in res.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
    want = sh.plain_logits(folder, requests)
    upto = {}
    for s in steps:
        wanted = [(e["id"], upto.get(e["id"], 0) + p) for e in s["entries"] for p in e["want"]]
        for e in s["entries"]:
            upto[e["id"]] = upto.get(e["id"], 0) + len(e["tokens"])
        rows = np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(len(wanted), cfg["vocab"])
        for row, (rid, p) in zip(rows, wanted):
            assert np.abs(row - want[rid][p]).max() <= TOL["float32"] * np.abs(want[rid]).max()


def random_config(seed):
    """A model of random sizes and layer order: odd head counts and sizes, one to five taps, partial and no rotation,
    readers of earlier layers' keys, with and without feed-forward, experts with and without identity experts."""
    rng = random.Random(seed)
    width = rng.choice([40, 72, 100, 136])
    layers, writers = [], {}
    for i in range(rng.randint(2, 6)):
        roll = rng.random()
        mlp = None if roll < 0.2 else sh.dense(rng.choice([24, 56, 136])) if roll < 0.6 else \
            sh.moe(rng.randint(1, 9), 1, rng.choice([8, 24, 40]), identity=rng.randint(0, 3), limit=rng.uniform(0.5, 3.0))
        if mlp is not None and mlp["kind"] == "moe":
            mlp["router"]["top"] = rng.randint(1, min(4, mlp["router"]["experts"] + mlp["router"]["identity"]))
        kind = rng.choice(["attention", "attention", "retention", "channel_delta"])
        if kind == "attention":
            if writers and rng.random() < 0.4:
                src = rng.choice(sorted(writers))
                layers.append(sh.layer("attention", dict(writers[src], kv_from=src), mlp))
                continue
            kv = rng.randint(1, 3)
            d = rng.choice([8, 12, 20, 40, 64])
            same = rng.random() < 0.4
            m = sh.attention(kv * rng.randint(1, 3), kv, d, d if same else rng.choice([4, 8, 24, 36]), scale=rng.uniform(0.1, 0.5),
                             rot=rng.choice([0, 4, d // 2 // 2 * 2, d]), base=rng.choice([100.0, 10000.0, 1e6]))
            writers[i] = m
            layers.append(sh.layer("attention", m, mlp))
        elif kind == "retention":
            h, d = rng.randint(1, 5), rng.choice([8, 12, 36, 72])
            layers.append(sh.layer("retention", sh.retention(h, d, rng.choice([4, 12, 20, 40]), decay=[rng.uniform(0.8, 0.999) for _ in range(h)],
                                                            rot=rng.choice([0, 4, d])), mlp))
        else:
            g = rng.randint(1, 3)
            layers.append(sh.layer("channel_delta", sh.delta(g * rng.randint(1, 3), g, rng.choice([8, 12, 36, 72]), rng.choice([4, 12, 20, 40]),
                                                             conv=rng.randint(1, 5), gate_rank=rng.choice([3, 8, 16])), mlp))
    return sh.config(layers, vocab=rng.choice([97, 256, 300]), width=width, eps=rng.choice([1e-5, 1e-6]),
                     scale=rng.choice([1.0, 3.0, 7.5]), softcap=rng.choice([None, 8.0, 30.0]))


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6])
def test_models_of_random_sizes_and_orders(tmp_path, seed):
    cfg = random_config(seed)
    page = [4, 8, 16, 32, 64, 16][seed - 1]
    requests = sh.random_requests(cfg, [70, 1, 37, 150, 2, 64], seed=seed)
    folder = sh.write_folder(tmp_path / "m", cfg, seed=seed)
    want = sh.plain_logits(folder, requests)
    for steps in (helpers.trace_whole(requests), helpers.trace_mixed(requests, seed=seed, max_live=3, decode_tail=20)):
        got, _ = run(folder, "float32", steps, page, max_live=3)
        assert helpers.first_bad(got, want, TOL["float32"]) is None, cfg
    folder16 = sh.write_folder(tmp_path / "m16", cfg, seed=seed, dtype="bfloat16")
    got, _ = run(folder16, "bfloat16", helpers.trace_mixed(requests, seed=seed, max_live=3, decode_tail=20), page, max_live=3)
    err = row_errors(got, sh.plain_logits(folder16, requests))
    assert np.isfinite(err).all() and np.median(err) <= TOL["bfloat16"] / 2, (np.median(err), cfg)
