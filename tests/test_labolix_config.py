"""The Labolix design without a GPU: its config reader and the errors it raises, the model spec it
becomes (layers that run with another layer's tensors, tensor names, cache and state needs), rotary
frequencies against the plain implementation, and a random model folder."""

import copy

import numpy as np
import pytest

from plain import labolix as plain
from qwen25vl_lite.config import ConfigError, resolve_architecture
from qwen25vl_lite.config.labolix_config import LabolixConfig
from qwen25vl_lite.models.decoder import DecoderModel
from qwen25vl_lite.parts.position import rotary_frequencies
from tiny_labolix import L1, L2, L3, L4, L5, TINY, make_model_dir


def model_of(raw):
    arch = resolve_architecture(raw)
    return DecoderModel(arch.build_spec(arch.config_from_dict(raw)))


def test_config_reads_every_size_and_constant():
    cfg = LabolixConfig.from_dict(L1)
    assert (cfg.vocab_size, cfg.hidden_size, cfg.norm_eps, cfg.logit_softcap, cfg.num_hidden_layers) == (211, 96, 1e-5, 12.0, 5)
    ret, att, lat = cfg.layers[0].mixer, cfg.layers[1].mixer, cfg.layers[2].mixer
    assert (ret.heads, ret.dim, ret.vdim, ret.decay, ret.rot.dims, ret.rot.scaling) == (3, 16, 24, (0.5, 0.96875, 1.0), 8, None)
    assert (att.heads, att.kv_heads, att.dim, att.vdim, att.scale, att.window) == (6, 2, 32, 16, 0.2, None)
    assert dict(att.rot.scaling) == {"kind": "wavelength", "factor": 8.0, "low": 1.0, "high": 4.0, "original": 64.0}
    assert (lat.heads, lat.dim, lat.rot_dim, lat.vdim, lat.kv_rank, lat.scale, lat.window) == (3, 16, 8, 24, 40, 0.25, 24)
    assert dict(lat.rot.scaling)["kind"] == "ramp"
    assert cfg.layers[2].mlp is None and cfg.layers[3].weights_of == 0 and cfg.layers[4].weights_of == 2
    assert LabolixConfig.from_dict(L2).logit_softcap == 0.0


@pytest.mark.parametrize("path,message", [
    (("vocab",), "vocab"), (("norm",), "norm"), (("layers", 1, "mixer", "scale"), "scale"), (("layers", 2, "mixer", "kv_rank"), "kv_rank"),
    (("layers", 0, "mixer", "decay"), "decay"), (("layers", 1, "mixer", "rot", "base"), "base"), (("layers", 0, "mlp", "limit"), "limit"),
    (("layers", 1, "mixer", "rot", "scaling", "high"), "high"), (("layers", 2, "mixer", "rot", "scaling", "fast"), "fast")])
def test_a_missing_key_is_named(path, message):
    raw = copy.deepcopy(L1)
    raw["layers"][3].pop("weights_of"); raw["layers"][4].pop("weights_of")       # so that an edited layer is not compared with its user
    d = raw
    for key in path[:-1]:
        d = d[key]
    del d[path[-1]]
    with pytest.raises(ConfigError, match=message):
        LabolixConfig.from_dict(raw)


def test_config_errors():
    raw = copy.deepcopy(L1)
    raw["layers"][0]["type"] = "convolution"
    with pytest.raises(ConfigError, match="unknown type"):
        LabolixConfig.from_dict(raw)
    raw = copy.deepcopy(L1)
    raw["layers"][0]["mixer"]["decay"] = [0.5, 0.9]
    with pytest.raises(ConfigError, match="decays"):
        LabolixConfig.from_dict(raw)
    raw = copy.deepcopy(L1)
    raw["layers"][4]["weights_of"] = 3                   # layer 3 has no tensors of its own
    with pytest.raises(ConfigError, match="no tensors of its own"):
        LabolixConfig.from_dict(raw)
    raw = copy.deepcopy(L1)
    raw["layers"][3]["weights_of"] = 1                   # a retention layer cannot run with an attention layer's tensors
    with pytest.raises(ConfigError, match="describes another layer"):
        LabolixConfig.from_dict(raw)
    raw = copy.deepcopy(L1)
    raw["layers"][0]["mlp"]["kind"] = "moe"
    with pytest.raises(ConfigError, match="unknown kind"):
        LabolixConfig.from_dict(raw)
    raw = copy.deepcopy(L1)
    raw["layers"][0]["mixer"]["rot"]["scaling"] = {"factor": 2.0}
    with pytest.raises(ConfigError, match="scaling"):
        LabolixConfig.from_dict(raw)


def test_spec_shares_tensors_and_keeps_caches_apart():
    model = model_of(L1)
    assert [s.layer for s in model.spec.schedule] == [0, 1, 2, 0, 2] and len(model.blocks) == 3
    names = set(model.expected_tensors())
    assert {"embed", "final.norm", "final.norm.b", "final.norm.alpha", "l0.mix.g", "l1.mix.q", "l2.mix.dkv.norm", "l2.mix.sink",
            "l2.mix.uk", "l0.mlp.gate", "l1.norm2.alpha"} <= names
    assert not any(n.startswith(("l3.", "l4.")) for n in names) and "l1.mix.sink" not in names
    required = {n for n, ts in model.expected_tensors().items() if not ts.optional}
    assert "l2.norm2" not in required and "head" not in required        # no feed-forward: no second norm; the head is the embedding
    needs = model.stop_needs()
    assert needs[0].state.shape == (3, 16, 24) and needs[0].cache is None and needs[3].state.shape == (3, 16, 24)
    lat = needs[2].cache
    assert (lat.kv_heads, lat.head_dim, lat.v_dim, lat.window, lat.value_in_key) == (1, 48, 40, 24, True) and needs[4].cache == lat
    att = needs[1].cache
    assert (att.kv_heads, att.head_dim, att.v_dim, att.window, att.value_in_key) == (2, 32, 16, None, False)


def test_cache_groups_and_pages_behind_a_window():
    from qwen25vl_lite.cache.manager import CacheManager

    manager = CacheManager(model_of(L1).stop_needs(), num_pages=12, page_size=16, max_requests=2)
    assert len(manager.groups) == 2 and sorted(len(g.stops) for g in manager.groups) == [1, 2]
    windowed = next(g for g in manager.groups if g.window)
    assert windowed.bytes_per_token(2) == 2 * 48 * 2                   # two stops, one row of rank + turned channels each
    req = manager.open()
    manager.ensure(req, 100)
    manager.advance(req, 100)
    held = [len(req.held_pages(g.index)) for g in manager.groups]
    assert held[windowed.index] == 3 and max(held) == 7               # the next token sees keys 77 .. 100: pages 4, 5 and 6 of 16 tokens
    manager.close(req)
    manager.check([])
    assert model_of(L4).stop_needs()[0].cache is None and not CacheManager(model_of(L4).stop_needs(), 4, 16, 2).groups


@pytest.mark.parametrize("rot,kind", [({"dims": 16, "base": 10000.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}}, "wavelength"),
                                      ({"dims": 8, "base": 1000.0, "scaling": {"factor": 4.0, "original": 48, "fast": 8.0, "slow": 1.0}}, "ramp"),
                                      ({"dims": 64, "base": 250000.0, "scaling": {"factor": 40.0, "original": 4096, "fast": 32.0, "slow": 1.0}}, "ramp"),
                                      ({"dims": 128, "base": 500000.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}, "wavelength"),
                                      ({"dims": 12, "base": 77.0}, None)])
def test_rotary_frequencies(rot, kind):
    scaling = dict(rot["scaling"], kind=kind) if kind else None
    got, magnitude = rotary_frequencies(rot["dims"], rot["base"], scaling)
    want, want_magnitude = plain.rotary_table(rot, kind or "none")
    assert np.allclose(got, want, rtol=1e-12) and magnitude == pytest.approx(want_magnitude)
    plain_f = plain.base_frequencies(rot["dims"], rot["base"])
    if kind:
        assert (got <= plain_f * (1 + 1e-12)).all() and (got < plain_f * 0.999).any() and got[0] == plain_f[0]    # the fastest pair is kept
    assert (magnitude > 1.0) == (kind == "ramp")


@pytest.mark.parametrize("name", sorted(TINY))
def test_random_model_folder_loads_into_the_plain_implementation(tmp_path, name):
    folder = make_model_dir(tmp_path, name, "bfloat16")
    cfg, w = plain.load_model_dir(folder)
    assert set(w) == {n for n, ts in model_of(TINY[name][0]).expected_tensors().items() if not ts.optional}
    logits = plain.forward_logits(cfg, w, [1, 2, 3, 4, 5])
    assert logits.shape == (5, cfg["vocab"]) and np.isfinite(logits).all()
    if cfg.get("logit_softcap"):
        assert np.abs(logits).max() < cfg["logit_softcap"]


def test_known_architectures_include_the_design():
    from qwen25vl_lite.config import known_architectures

    assert {"Labolix", "Rirulix"} <= set(known_architectures())
    assert all(c["architecture"] == "Labolix" for c in (L1, L2, L3, L4, L5))
