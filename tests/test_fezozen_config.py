"""The Fezozen design on the CPU: configuration, tensor names and shapes, run order and cache entries, refused
configurations, the random-weights folder, the blended rotary frequencies, and the plain statement against itself (the
premises of the GPU tests: what a window one key off, a forgotten cap or a weight on the wrong side of an expert does
to the logits)."""
import copy
import math

import numpy as np
import pytest
import torch

import fezozen_helpers as fh
import plain_fezozen as plain
from tinyinfer_b200 import models  # noqa: F401
from tinyinfer_b200.config import FezozenConfig, load_config, lookup_architecture, preset_config
from tinyinfer_b200.weights import write_random_model


def build(cfg):
    return lookup_architecture("Fezozen").model_factory(FezozenConfig.from_dict(cfg), torch.float32, "cpu")


@pytest.mark.parametrize("name", ["MIX", "WIDE", "ONE"])
def test_names_and_shapes_follow_the_configuration(name):
    cfg = getattr(fh, name)
    want = fh.tensor_shapes(cfg)
    got = build(cfg).expected_tensors()
    assert set(got) == set(want)
    assert {n: tuple(ts.shape) for n, ts in got.items()} == want


def test_run_order_and_cache_entries():
    model = build(fh.MIX)
    # layers 3 and 5 run the tensors of layers 0 and 1, each on a cache entry of its own; layer 4 has tensors
    assert [(e.layer, e.cache, e.writes_cache) for e in model.spec.execution] == \
        [(0, 0, True), (1, 1, True), (2, 2, True), (0, 3, True), (3, 4, True), (1, 5, True)]
    assert [l.index for l in model.spec.layers] == [0, 1, 2, 4]
    needs = model.cache_needs()
    assert len(needs) == 6 and all(state is None for _, state in needs)
    assert (needs[0][0].num_kv_heads, needs[0][0].head_dim, needs[0][0].window, needs[0][0].planes) == (2, 32, None, 1)
    assert (needs[1][0].num_kv_heads, needs[1][0].head_dim, needs[1][0].window, needs[1][0].planes) == (1, 32, 19, 1)
    assert (needs[2][0].num_kv_heads, needs[2][0].head_dim, needs[2][0].window, needs[2][0].planes) == (4, 16, 11, 2)
    assert needs[3][0] == needs[0][0] and needs[5][0] == needs[1][0] and needs[4][0].window == 5
    one = build(fh.ONE)            # a layer listed before the one whose tensors it runs
    assert [(e.layer, e.cache) for e in one.spec.execution] == [(1, 0), (0, 1), (1, 2), (2, 3), (3, 4)]
    assert [l.index for l in one.spec.layers] == [1, 2, 3, 4]


def test_constants_reach_the_specs():
    spec = build(fh.MIX).spec
    assert all(l.arrangement == "multi_stream" and l.streams == 1 and l.mixer_out_norm.tensor == "norm1b" for l in spec.layers)
    a, lat, w, last = (l.mixer for l in spec.layers)
    assert a.qkv_bias and a.softcap == 5.0 and a.window is None and a.qk_unit_norm is None and a.scale == 0.3
    assert a.position.interleaved and a.position.rotary_dim == 12 and a.position.blend.factor == 3.0 and a.position.blend.original == 24
    assert (lat.q_rank, lat.kv_rank, lat.rot_dim, lat.v_dim, lat.window, lat.output_gate) == (0, 24, 8, 20, 19, True)
    assert lat.position.rotary_dim == 8 and lat.position.blend.fast == 4.0
    assert not w.qkv_bias and w.softcap is None and w.window == 11 and w.qk_unit_norm == 1e-5 and w.position.blend is None
    assert w.position.rotary_dim == 8 and last.window == 5
    moe = spec.layers[0].feed_forward
    assert (moe.num_experts, moe.top, moe.expert_size, moe.activation, moe.scoring) == (5, 2, 24, "silu_glu", "sigmoid")
    assert moe.weight_input and not moe.renormalize and moe.router_input == "input" and moe.identity_experts == 0
    assert spec.layers[3].feed_forward is None and spec.layers[3].feed_forward_norm is None and spec.layers[3].feed_forward_out_norm is None
    one = build(fh.ONE).spec
    assert one.layers[2].mixer.position.kind == "rope" and one.layers[3].mixer.position.kind == "none"
    cfg = copy.deepcopy(fh.WIDE)
    del cfg["embedding"]
    assert FezozenConfig.from_dict(cfg).embedding_scale == 1.0


@pytest.mark.parametrize("edit,message", [
    (lambda c: c["layers"][0].update(type="window"), "unknown mixer type"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=4), "multiple of kv_heads"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "lacks mixer.kv_rank"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=13), "dims even"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].pop("slow"), "factor, original, fast and slow"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=4), "its rot_dim"),
    (lambda c: c["layers"][1]["mixer"].update(softcap=3.0), "not capped"),
    (lambda c: c["layers"][2]["mixer"]["mask"].update(size=0), "at least 1"),
    (lambda c: c["layers"][3].update(weights_of=5), "tensors of its own"),
    (lambda c: c["layers"][3].update(weights_of=3), "tensors of its own"),
    (lambda c: c["layers"][3].update(weights_of=1), "must equal layer"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "unknown feed-forward"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=6), "between 1 and"),
    (lambda c: c.pop("norm"), "required keys"),
])
def test_refused_configurations(edit, message):
    cfg = copy.deepcopy(fh.MIX)
    edit(cfg)
    with pytest.raises(ValueError, match=message):
        FezozenConfig.from_dict(cfg)


def test_round_trip_presets_and_random_folder(tmp_path):
    cfg = FezozenConfig.from_dict(fh.MIX)
    assert FezozenConfig.from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()
    tiny = preset_config("fezozen-tiny")
    assert isinstance(tiny, FezozenConfig) and len(tiny.layers) == 5 and tiny.layers[3]["weights_of"] == 0
    folder = write_random_model(tmp_path / "r", tiny, seed=1)
    arch, again = load_config(folder)
    assert arch.name == "Fezozen" and again.to_dict() == tiny.to_dict()
    from safetensors.torch import load_file
    stored = load_file(str(folder / "model.safetensors"))
    assert {n: tuple(t.shape) for n, t in stored.items()} == fh.tensor_shapes(tiny.to_dict())
    for preset in ("fezozen-1b", "fezozen-2b"):
        assert build(preset_config(preset).to_dict()).weight_bytes() > 5e8


def test_blended_frequencies_follow_the_plain_statement():
    from tinyinfer_b200.parts.position import RotaryEncoding
    for m in (fh.MIX["layers"][0]["mixer"], fh.WIDE["layers"][0]["mixer"], dict(rot=fh.rot(777.0, 10, fh.scaling(7.0, 9, 2.0, 0.3)))):
        spec = build(fh.config([fh.layer("attention", dict(fh.attention(2, 1, 64, 8), rot=m["rot"]), None)])).spec.layers[0].mixer.position
        part = RotaryEncoding(spec, torch.float32, "cpu")
        f, factor = plain.frequencies(m["rot"])
        assert torch.allclose(part.inv_freq.double(), f, rtol=1e-6, atol=0)
        assert abs(part.factor - factor) < 1e-12 and part.interleaved
    # the blend's ends: the fastest pair keeps its frequency, the slowest turns `factor` times slower
    r = fh.rot(10000.0, 64, fh.scaling(4.0, 128, 16.0, 1.0))
    f, factor = plain.frequencies(r)
    assert f[0] == 1.0 and abs(f[-1] * 4.0 / 10000.0 ** (-62 / 64) - 1) < 1e-12 and abs(factor - (0.1 * math.log(4.0) + 1)) < 1e-12
    assert plain.frequencies(fh.rot(10000.0, 8))[1] == 1.0


# ------------------------------------------------------------------ the plain statement against itself
def logits(cfg, w, tokens):
    return fh.forward(cfg, w, tokens)


def test_plain_window_is_exact_to_the_key():
    """One windowed layer, no feed-forward: the logits at position p hang on tokens p - size + 1 .. p and on no other."""
    for kind, mixer in (("attention_2", fh.attention(2, 1, 8, 12, window=6, rot_=fh.rot(100.0, 8))),
                        ("latent_attention", fh.latent(2, 8, 4, 12, 10, window=6))):
        cfg = fh.config([fh.layer(kind, mixer, None)], width=32)
        w = fh.draw_tensors(cfg, 3, torch.float64)
        tokens = fh.random_requests(cfg, [30], seed=1)["r0"]
        base = logits(cfg, w, tokens)
        inside, outside = list(tokens), list(tokens)
        inside[29 - 5] = (inside[29 - 5] + 1) % cfg["vocab"]
        outside[29 - 6] = (outside[29 - 6] + 1) % cfg["vocab"]
        assert np.abs(logits(cfg, w, outside)[29] - base[29]).max() == 0.0
        assert np.abs(logits(cfg, w, inside)[29] - base[29]).max() > 1e-3 * np.abs(base).max()


def test_plain_mechanisms_carry_weight():
    """Leaving one mechanism out of the plain statement moves the logits far beyond the GPU tests' tolerances."""
    cfg = fh.MIX
    w = fh.draw_tensors(cfg, 5, torch.float64)
    tokens = fh.random_requests(cfg, [40], seed=2)["r0"]
    base = logits(cfg, w, tokens)
    scale = np.abs(base).max()

    def moved(edit_cfg=None, edit_w=None):
        c, t = copy.deepcopy(cfg), dict(w)
        if edit_cfg:
            edit_cfg(c)
        if edit_w:
            edit_w(t)
        return np.abs(logits(c, t, tokens) - base).max() / scale

    def both(c, fn):            # a layer and the one that runs its tensors must stay equal
        for l in c["layers"]:
            fn(l)
    assert moved(lambda c: both(c, lambda l: l["mixer"].pop("softcap", None))) > 1e-3
    assert moved(lambda c: both(c, lambda l: l["mixer"]["rot"].pop("scaling", None))) > 1e-3
    assert moved(lambda c: both(c, lambda l: l["mixer"].get("mask", {}).update(size=l["mixer"].get("mask", {}).get("size", 0) + 1))) > 1e-4
    assert moved(edit_w=lambda t: t.update({"l0.mix.k.b": torch.zeros_like(t["l0.mix.k.b"])})) > 1e-3
    assert moved(edit_w=lambda t: t.update({"l1.mix.g": torch.zeros_like(t["l1.mix.g"])})) > 1e-3
    assert moved(edit_w=lambda t: t.update({"l0.norm1b": torch.ones_like(t["l0.norm1b"])})) > 1e-3
    assert moved(lambda c: c["layers"][5].pop("weights_of"), lambda t: t.update(
        {k.replace("l1.", "l5."): torch.roll(v, 1, 0) for k, v in t.items() if k.startswith("l1.")})) > 1e-3


def test_plain_expert_weight_sits_at_the_input():
    cfg = fh.config([fh.layer("attention_2", fh.attention(2, 2, 8, 8, window=4), fh.moe(4, 2, 16))], width=24)
    w = {k[len("l0.mlp."):]: v for k, v in fh.draw_tensors(cfg, 1, torch.float64).items() if k.startswith("l0.mlp.")}
    h = torch.randn(24, dtype=torch.float64, generator=torch.Generator().manual_seed(0))
    got = plain.experts(w, cfg["layers"][0]["mlp"], h)
    s = torch.sigmoid(w["router"] @ h)
    top = sorted(range(4), key=lambda e: -float(s[e]))[:2]
    at_input = sum(w[f"e{e}.down"] @ (plain.silu(w[f"e{e}.gate"] @ (s[e] * h)) * (w[f"e{e}.up"] @ (s[e] * h))) for e in top)
    at_output = sum(s[e] * (w[f"e{e}.down"] @ (plain.silu(w[f"e{e}.gate"] @ h) * (w[f"e{e}.up"] @ h))) for e in top)
    assert torch.allclose(got, at_input, rtol=1e-12, atol=1e-12)
    assert (got - at_output).abs().max() > 1e-2 * got.abs().max()
