"""The Sinulix design on the CPU: configuration, tensor names and shapes, run order and cache entries, refused
configurations, loader errors, the random-weights folder, and the plain statement against itself (the premises of the
GPU tests: what a lost sink, a lost state or a forgotten correction does to the logits)."""
import copy
import json

import numpy as np
import pytest
import torch

import plain_sinulix as plain
import sinulix_helpers as sh
from tinyinfer_b200 import models  # noqa: F401
from tinyinfer_b200.config import SinulixConfig, load_config, lookup_architecture, preset_config
from tinyinfer_b200.weights import write_random_model


def build(cfg):
    return lookup_architecture("Sinulix").model_factory(SinulixConfig.from_dict(cfg), torch.float32, "cpu")


@pytest.mark.parametrize("name", ["MIX", "WIDE", "ONE"])
def test_names_and_shapes_follow_the_configuration(name):
    cfg = getattr(sh, name)
    want = sh.tensor_shapes(cfg)
    got = build(cfg).expected_tensors()
    assert set(got) == set(want)
    assert {n: tuple(ts.shape) for n, ts in got.items()} == want


def test_a_size_that_only_the_checkpoint_gives(tmp_path):
    cfg = copy.deepcopy(sh.ONE)
    del cfg["layers"][0]["mixer"]["gate_rank"]
    shapes = {n: tuple(ts.shape) for n, ts in build(cfg).expected_tensors().items()}
    assert shapes["l0.mix.a1"] == (-1, 40) and shapes["l0.mix.a2"] == (40, -1) and shapes["l0.mix.g2"] == (8, -1)
    with pytest.raises(ValueError, match="only a checkpoint gives"):
        write_random_model(tmp_path / "r", SinulixConfig.from_dict(cfg), seed=1)


def test_run_order_and_cache_entries():
    model = build(sh.MIX)
    order = [(e.layer, e.cache, e.writes_cache) for e in model.spec.execution]
    # layer 3 reads what layer 1 caches and has no entry of its own
    assert order == [(0, 0, True), (1, 1, True), (2, 2, True), (3, 1, False), (4, 3, True)]
    needs = model.cache_needs()
    assert len(needs) == 4
    assert needs[0][0] is None and needs[0][1].shape == (3 * 20 * 12,) and needs[0][1].dtype == torch.float32
    pages, state = needs[1]
    assert state is None and (pages.num_kv_heads, pages.head_dim) == (2, 20 + 12)
    # the matrix state, then taps - 1 rows of the convolution's inputs [q | k | v]
    assert needs[2][1].shape == (6 * 20 * 12 + 2 * (2 * 3 * 12 + 6 * 20),)
    assert needs[3][1].shape == (2 * 12 * 28 + 4 * (2 * 2 * 28 + 2 * 12),)
    one = build(sh.ONE)
    assert one.cache_needs()[0][1].shape == (1 * 8 * 40,)          # one tap: no history behind the matrix state


def test_constants_reach_the_specs():
    spec = build(sh.MIX).spec
    assert all(l.streams == 1 and not l.learned_mixing and l.mixer_norm.offset == 1.0 for l in spec.layers)
    r, a, d, reader, last = (l.mixer for l in spec.layers)
    assert r.kind == "retention" and r.decays == (1 - 2.0 ** -3, 1 - 2.0 ** -4, 1 - 2.0 ** -5) and r.position.rotary_dim == 8
    assert a.head_sinks and a.head_gate and not a.shares_cache and reader.shares_cache
    assert (a.scale, a.v_dim, a.position.rotary_dim, a.qk_norm.eps) == (0.3, 12, 12, 1e-5)
    assert (d.conv_taps, d.unit_eps, d.gate_rank, last.conv_taps, last.gate_rank) == (3, 1e-6, 6, 5, 3)
    moe = spec.layers[1].feed_forward
    assert (moe.num_experts, moe.identity_experts, moe.top, moe.glu_limit, moe.glu_alpha) == (5, 2, 2, 1.5, 1.702)
    assert moe.activation == "clamped_glu" and moe.score_correction and not moe.renormalize
    assert spec.layers[3].feed_forward is None and spec.layers[3].feed_forward_norm is None
    assert build(sh.ONE).spec.layers[1].mixer.position.kind == "none"
    cfg = copy.deepcopy(sh.WIDE)
    assert SinulixConfig.from_dict(cfg).logit_softcap is None
    del cfg["embedding"]
    assert SinulixConfig.from_dict(cfg).embedding_scale == 1.0


@pytest.mark.parametrize("edit,message", [
    (lambda c: c["layers"][0].update(type="window"), "unknown mixer type"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=4), "multiple of kv_heads"),
    (lambda c: c["layers"][0]["mixer"].update(decay=[0.9]), "one number per head"),
    (lambda c: c["layers"][2]["mixer"].pop("conv"), "lacks mixer.conv"),
    (lambda c: c["layers"][2]["mixer"].update(conv=0), "at least 1"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=22), "rot needs"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "kv_from must name"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=2), "kv_from must name"),
    (lambda c: c["layers"][3]["mixer"].update(heads=4), "must equal those of layer 1"),
    (lambda c: c["layers"][0]["mixer"].update(kv_from=0), "only an attention layer"),
    (lambda c: c["layers"][0].update(mlp=dict(kind="shared")), "unknown feed-forward"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=8), "top exceeds"),
    (lambda c: c["layers"][1]["mlp"]["expert"].pop("limit"), "needs router.experts"),
    (lambda c: c.pop("norm"), "lacks required keys"),
    (lambda c: c.update(logit_softcap=-1.0), "logit_softcap"),
])
def test_refused_configurations(edit, message):
    cfg = copy.deepcopy(sh.MIX)
    edit(cfg)
    with pytest.raises(ValueError, match=message):
        SinulixConfig.from_dict(cfg)


def test_folder_round_trip_and_loader_errors(tmp_path):
    from tinyinfer_b200.weights import WeightError, load_weights
    folder = sh.write_folder(tmp_path / "m", sh.ONE, seed=1)
    arch, cfg = load_config(folder)
    assert arch.name == "Sinulix" and cfg.to_dict() == SinulixConfig.from_dict(cfg.to_dict()).to_dict()
    model = arch.model_factory(cfg, torch.float32, "cpu")
    load_weights(model, folder)
    assert model.blocks[0].mixer.w_a1.shape == (2, 40) and model.blocks[3].mixer.w_g1.shape == (6, 40)

    def spoil(t):
        del t["l1.mix.sink"]
        t["l0.mix.q.conv"] = torch.zeros(40, 3)
        t["extra"] = torch.zeros(1)
    bad = sh.write_folder(tmp_path / "bad", sh.ONE, seed=1, edit=spoil)
    with pytest.raises(WeightError) as err:
        load_weights(arch.model_factory(cfg, torch.float32, "cpu"), bad)
    assert err.value.missing == ["l1.mix.sink"] and err.value.unexpected == ["extra"]
    assert [n for n, _, _ in err.value.wrong_shape] == ["l0.mix.q.conv"]


def test_random_weights_folder_and_presets(tmp_path):
    cfg = preset_config("sinulix-tiny")
    folder = write_random_model(tmp_path / "r", cfg, seed=3)
    stored = json.loads((folder / "config.json").read_text())
    assert stored["architecture"] == "Sinulix" and stored["layers"][3]["mixer"]["kv_from"] == 2
    arch, again = load_config(folder)
    model = arch.model_factory(again, torch.float32, "cpu")
    from tinyinfer_b200.weights import load_weights
    load_weights(model, folder)
    assert [e.cache for e in model.spec.execution] == [0, 1, 2, 2, 3]
    for name in ("sinulix-1b", "sinulix-2b"):
        assert preset_config(name).model_spec().layers


# ------------------------------------------------------------------ the plain statement against itself
def test_plain_mechanisms_in_closed_form():
    """Retention unrolled as a sum over the past; one token of the delta rule by hand; the sink's share; identity
    experts; the rotation's relative angle."""
    gen = torch.Generator().manual_seed(0)
    m = dict(heads=2, dim=4, vdim=3, decay=[0.5, 0.9], rot=dict(base=100.0, dims=4))
    w = {n: torch.randn(s, 6, generator=gen, dtype=torch.float64) for n, s in (("q", 8), ("k", 8), ("v", 6), ("g", 6))}
    w["o"] = torch.eye(6, dtype=torch.float64)
    hs = torch.randn(5, 6, generator=gen, dtype=torch.float64)
    state = plain.Retention.new_state(m, torch.float64)
    for t in range(5):
        got = plain.Retention.step(w, m, 1e-5, hs[t], t, state)
    o = torch.zeros(2, 3, dtype=torch.float64)
    q = plain.rotate((w["q"] @ hs[4]).view(2, 4), 4, 4, 100.0)
    for j in range(5):
        k = plain.rotate((w["k"] @ hs[j]).view(2, 4), j, 4, 100.0) * 0.5
        o += torch.tensor([0.5, 0.9], dtype=torch.float64)[:, None] ** (4 - j) * (q * k).sum(-1, keepdim=True) * (w["v"] @ hs[j]).view(2, 3)
    want = (o / torch.sqrt((o * o).mean(-1, keepdim=True) + 1e-5)).reshape(-1) * plain.silu(w["g"] @ hs[4])
    assert (got - want).abs().max() < 1e-12
    # a rotated product depends on the distance of the positions only
    a, b = torch.randn(1, 6, generator=gen, dtype=torch.float64), torch.randn(1, 6, generator=gen, dtype=torch.float64)
    near = (plain.rotate(a, 9, 4, 50.0) * plain.rotate(b, 4, 4, 50.0)).sum()
    far = (plain.rotate(a, 105, 4, 50.0) * plain.rotate(b, 100, 4, 50.0)).sum()
    assert abs(near - far) < 1e-12 and torch.equal(plain.rotate(a, 9, 4, 50.0)[:, 4:], a[:, 4:])
    # experts: all weight on the identity output gives score * h
    f = dict(router=dict(experts=1, top=1, identity=1), expert=dict(ff=2, limit=1.0))
    h = torch.randn(6, generator=gen, dtype=torch.float64)
    we = {"router": torch.zeros(2, 6, dtype=torch.float64), "correction": torch.tensor([0.0, 1.0], dtype=torch.float64)}
    assert (plain.experts_mlp(we, f, h) - 0.5 * h).abs().max() < 1e-15


def test_what_the_tests_can_see(tmp_path):
    """Without the sinks, without the corrections, with identity experts that return nothing, with a convolution or a
    state that forgets what lay before a portion, with a reader that sees keys of its own layer instead of its
    writer's, the plain logits move by far more than any tolerance of the GPU tests."""
    folder = sh.write_folder(tmp_path / "m", sh.MIX, seed=11)
    requests = sh.random_requests(sh.MIX, [48], seed=4)
    want = sh.plain_logits(folder, requests)["r0"]
    margin = 1e-2 * np.abs(want).max()

    def moved(edit):
        return np.abs(sh.plain_logits(folder, requests, edit)["r0"] - want).max()

    def no_sink(c, w):
        for n in w:
            if n.endswith("mix.sink"):
                w[n] = torch.full_like(w[n], -1e9)
    assert moved(no_sink) > margin

    def no_correction(c, w):
        for n in w:
            if n.endswith("mlp.correction"):
                w[n] = torch.zeros_like(w[n])
    assert moved(no_correction) > margin

    def no_gate(c, w):
        w["l1.mix.g"] = torch.zeros_like(w["l1.mix.g"])
    assert moved(no_gate) > margin

    def own_keys(c, w):                       # the reader gets projections of its own: not what the design says
        del c["layers"][3]["mixer"]["kv_from"]
        for n in ("k", "v", "k.norm"):
            w[f"l3.mix.{n}"] = w[f"l1.mix.{n}"]
    assert moved(own_keys) > margin
    c, w = sh.read_folder(folder)
    tail = sh.forward(c, w, requests["r0"][20:])          # history, states and keys lost at token 20
    assert np.abs(tail[0] - want[20]).max() > margin and np.abs(tail[-1] - want[-1]).max() > margin
