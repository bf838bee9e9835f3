"""What needs no GPU of the Rirulix design: its config.json reader, the model it describes (parts,
tensor names, cache and state needs), the random model folder, the pages that a window with kept
first tokens holds and gives back, and the attention's work lists."""

import copy
import json
import os

import numpy as np
import pytest

from qwen25vl_lite.cache.manager import CacheManager, StopNeeds
from qwen25vl_lite.config import ConfigError, resolve_architecture
from qwen25vl_lite.engine.runner import HostStep
from qwen25vl_lite.models.decoder import DecoderModel
from qwen25vl_lite.ops.attention import plan_biased
from qwen25vl_lite.parts import KVCacheNeed
from qwen25vl_lite.weights import write_random_model

from plain.decoder import read_safetensors
from tiny_rirulix import R1, R2, R3


def build(raw):
    arch = resolve_architecture(raw)
    return DecoderModel(arch.build_spec(arch.config_from_dict(raw)))


def test_architecture_is_found_by_its_single_name():
    assert resolve_architecture({"architecture": "Rirulix"}).name == "Rirulix"
    with pytest.raises(ValueError, match="unknown architecture"):
        resolve_architecture({"architecture": "NoSuchDesign"})


def test_every_size_comes_from_the_file():
    model = build(R1)
    mixers = [b.mixer for b in model.blocks]
    assert [m.kind for m in mixers] == ["rglru", "biased_window_attention", "biased_window_attention", "biased_window_attention",
                                       "rglru", "biased_window_attention"]
    assert [getattr(m, "value_mix", None) for m in mixers] == [None, "source", "follower", None, None, "follower"]
    assert (mixers[1].window, mixers[1].keep_first, mixers[1].value_dim, mixers[1].scale) == (24, 3, 16, 0.2)
    assert (mixers[3].window, mixers[3].keep_first, mixers[3].num_kv_heads) == (None, 0, 4)
    assert (mixers[0].width, mixers[0].blocks, mixers[0].conv, mixers[4].conv) == (64, 4, 3, 2)
    ffns = [b.feed_forward for b in model.blocks]
    assert ffns[1] is None and ffns[4] is None and [n.optional for n in model.blocks[1].norms] == [False, False, True, True]
    assert not any(n.optional for n in model.blocks[0].norms)
    assert (ffns[0].experts, ffns[0].top, ffns[0].shared_size, ffns[2].shared_size, ffns[3].top) == (6, 2, 56, None, 1)
    assert all(n.groups == 3 and n.eps == 1e-5 for b in model.blocks for n in b.norms)
    needs = model.stop_needs()
    assert needs[0].state.shape == (3, 64) and needs[4].state.shape == (2, 96) and needs[1].state is None
    assert needs[1].cache == KVCacheNeed(2, 32, 24, 16, 3) and needs[3].cache == KVCacheNeed(4, 16, None, 32, 0)


def test_tensor_names_and_shapes():
    names = {k: v.shape for k, v in build(R1).expected_tensors().items()}
    assert names["embed"] == (211, 96) and names["pos"] == (512, 96) and names["embed.norm"] == (96,)
    assert names["l0.mix.ra"] == (4, 16, 16) and names["l0.mix.conv"] == (64, 3) and names["l0.mix.o"] == (96, 64)
    assert names["l1.mix.q"] == (192, 96) and names["l1.mix.v"] == (32, 96) and names["l1.mix.o"] == (96, 96)
    specs = build(R1).expected_tensors()
    assert names["l1.mix.vmix"] == () and names["l1.mix.r1"] == (6,) and specs["l3.mix.vmix"].optional and not specs["l1.mix.vmix"].optional
    assert specs["l1.norm2"].optional and specs["l4.norm2b"].optional and not specs["l0.norm2"].optional     # no feed-forward: never run
    assert "l1.mlp.router" not in names and names["l0.norm2b"] == (96,)
    assert names["l0.mlp.e5.down"] == (96, 40) and names["l0.mlp.shared.sg"] == (1, 96) and "l2.mlp.shared.gate" not in names
    assert names["final.norm"] == (96,) and names["head"] == (211, 96)


def test_config_errors_name_the_key():
    for path, match in ((("norm",), "norm"), (("layers", 0, "mixer", "blocks"), "blocks"), (("layers", 1, "mixer", "scale"), "scale"),
                        (("layers", 0, "mlp", "router"), "router"), (("vocab",), "vocab")):
        raw = copy.deepcopy(R1)
        at = raw
        for key in path[:-1]:
            at = at[key]
        del at[path[-1]]
        with pytest.raises(ConfigError, match=match):
            build(raw)
    raw = copy.deepcopy(R1)
    raw["layers"][0]["type"] = "lstm"
    with pytest.raises(ConfigError, match="unknown type"):
        build(raw)
    raw = copy.deepcopy(R3)
    raw["layers"][2]["mixer"]["vdim"] = 32
    with pytest.raises(ValueError, match="mixes its values"):
        build(raw)


def test_random_model_folder_loads_by_name(tmp_path):
    folder = write_random_model(str(tmp_path / "m"), R2, seed=3, prefix="")
    tensors = read_safetensors(os.path.join(folder, "model.safetensors"))
    assert set(tensors) == {n for n, ts in build(R2).expected_tensors().items() if not ts.optional}
    assert (tensors["l0.mix.r2"] > 0).all() and 0 < float(tensors["l0.mix.r1"].min())
    with open(os.path.join(folder, "config.json")) as fh:
        assert json.load(fh)["architecture"] == "Rirulix"


def test_command_line_writes_a_folder_that_the_loader_accepts(tmp_path):
    """``random-model`` through the program's own entry point; the names in the file are the ones the
    model expects (no prefix for this architecture), which is what ``generate`` and ``replay`` load."""
    from qwen25vl_lite.cli import main
    from qwen25vl_lite.weights.loader import canonical_name

    config = tmp_path / "config.json"
    config.write_text(json.dumps(R3))
    assert main(["random-model", "--config", str(config), "--out", str(tmp_path / "m"), "--seed", "5", "--storage-dtype", "bfloat16"]) == 0
    model = build(R3)
    names = set(read_safetensors(str(tmp_path / "m" / "model.safetensors")))
    assert {canonical_name(n, model.spec)[0] for n in names} == {n for n, ts in model.expected_tensors().items() if not ts.optional} == names


def test_kept_first_pages_stay_while_the_window_releases():
    """Window 20, 5 kept tokens, pages of 4: pages 0 and 1 hold kept tokens and are never given back;
    the pages between them and the window are."""
    cm = CacheManager([StopNeeds(KVCacheNeed(1, 16, 20, 8, 5))], 64, 4, 2)
    r = cm.open()
    cm.ensure(r, 50)
    cm.advance(r, 50)
    table = r.tables[0]
    first_needed = (50 - 20 + 1) // 4
    assert all(p >= 0 for p in table[:2]) and all(p < 0 for p in table[2:first_needed]) and all(p >= 0 for p in table[first_needed:])
    assert cm.pages_in_use() == [2 + len(table) - first_needed]
    cm.check([r])
    for _ in range(30):                         # single tokens: a page goes back every four
        cm.ensure(r, r.num_tokens + 1)
        cm.advance(r, 1)
        cm.check([r])
    assert all(p >= 0 for p in r.tables[0][:2]) and cm.pages_in_use()[0] <= 2 + 20 // 4 + 2
    cm.close(r)
    assert cm.pages_in_use() == [0]
    # a group whose keys and values differ in size keeps two page tensors
    assert cm.groups[0].bytes_per_token(2) == (16 + 8) * 2


def test_attention_work_lists():
    host = HostStep([1, 70, 1, 5], [10, 0, 300, 64], 77, 4)
    plan = plan_biased(host, group=4, window=0, keep_first=0)
    assert plan["decode_items"].tolist() == [0, 2]
    tiles = plan["tiles64"].reshape(-1, 2).tolist()
    assert sorted(tiles) == [[1, t] for t in range(5)] + [[3, 0]]
    assert tiles[:2] == [[1, 4], [3, 0]]                       # the tiles that see the most keys (70, 69) come first
    windowed = plan_biased(host, group=4, window=16, keep_first=2)["tiles64"].reshape(-1, 2).tolist()
    assert sorted(windowed) == sorted(tiles)
