"""The Vuvosun design without a GPU: its config.json reader, the model that is built
from it, the random-weights folder, the cache manager's kept first pages, and the plain
implementation's own rules."""
import copy
import json
import os

import pytest
import torch

import plain_vuvosun as plain
import vuvosun_cases as cases
from crucible_b200.cache import CacheManager, GroupPolicy
from crucible_b200.config.model_config import UNBOUNDED_CONTEXT, ConfigError
from crucible_b200.config.registry import known_architectures, parse_config
from crucible_b200.models.decoder import DecoderModel


def test_architecture_is_registered_beside_the_others():
    assert {"Vuvosun", "CrucibleGPT", "LlamaForCausalLM"} <= set(known_architectures())


@pytest.mark.parametrize("name", sorted(cases.CASES))
def test_parse_builds_the_layers_the_config_lists(name):
    raw = cases.CASES[name]["config"]
    cfg = parse_config(raw)
    assert cfg.architecture == "Vuvosun" and cfg.max_context == UNBOUNDED_CONTEXT
    assert cfg.tie_word_embeddings and cfg.vocab_size == raw["vocab"] and cfg.hidden_size == raw["width"]
    assert [l.mixer.kind for l in cfg.layers] == [e["type"] for e in raw["layers"]]
    assert [l.feed_forward.kind for l in cfg.layers] == \
        ["polynorm" if e["mlp"] else "none" for e in raw["layers"]]
    model = DecoderModel(cfg)
    names = {r.checkpoint_name for r in model.tensor_requests()}
    assert {"embed", "embed.norm", "final.norm", "l0.norm1", "l0.hc1.in", "l0.hc1.mix", "l0.hc1.out"} <= names
    for i, e in enumerate(raw["layers"]):
        assert (f"l{i}.norm2" in names) == (e["mlp"] is not None)
        assert (f"l{i}.hc2.mix" in names) == (e["mlp"] is not None)
        if e["type"] == "parallel":
            assert {f"l{i}.mix.left.sink", f"l{i}.mix.left.g", f"l{i}.mix.right.q.conv",
                    f"l{i}.mix.right.A_log", f"l{i}.mix.right.dt_bias", f"l{i}.mix.right.norm"} <= names
        else:
            assert {f"l{i}.mix.i", f"l{i}.mix.i.b", f"l{i}.mix.f.b", f"l{i}.mix.norm"} <= names


def test_storage_follows_the_layers():
    a = DecoderModel(parse_config(cases.CASES["vu-a"]["config"]))
    group, other = a.cache_groups
    assert group.layers == (0, 2) and group.need.window == 24 and group.need.keep_first == 3
    assert group.need.head_dim == 32 and group.need.value_dim == 16
    assert other.layers == (3,) and other.need.window == 9 and other.need.keep_first == 0
    # per request: delta-rule matrices and convolution tails of three layers, one mLSTM memory
    delta = 4 * 4 * 16 * 24 + 4 * 2 * (2 * 4 * 16 + 4 * 24)
    small = 4 * 2 * 8 * 8 + 4 * 3 * (2 * 1 * 8 + 2 * 8)
    mlstm = 4 * 2 * 16 * 32 + 4 * 2 * 16 + 16
    assert a.state_bytes == 2 * delta + small + mlstm
    b = DecoderModel(parse_config(cases.CASES["vu-b"]["config"]))
    assert b.cache_groups == [] and b.state_bytes > 0
    c = DecoderModel(parse_config(cases.CASES["vu-c"]["config"]))
    assert c.cache_groups[0].need.value_dim is None and c.cache_groups[0].need.keep_first == 0


def test_config_errors_name_the_key():
    raw = cases.CASES["vu-a"]["config"]
    for path, value, word in [(("layers", 0, "type"), "conv", "layer type"),
                              (("layers", 0, "mixer", "left", "rot", "dims"), 7, "dims"),
                              (("layers", 0, "mixer", "left", "mask", "keep_first"), -1, "keep_first"),
                              (("layers", 0, "mlp", "kind"), "routed", "kind"),
                              (("layers", 1, "mixer", "gate_cap"), None, "gate_cap"),
                              (("norm",), None, "norm"), (("width",), 0, "width")]:
        bad = copy.deepcopy(raw)
        at = bad
        for key in path[:-1]:
            at = at[key]
        at[path[-1]] = value
        with pytest.raises(ConfigError, match=word):
            parse_config(bad)
    bad = copy.deepcopy(raw)
    bad["layers"][0]["mixer"]["left"]["kv_heads"] = 3
    with pytest.raises(ValueError, match="divisible"):
        DecoderModel(parse_config(bad))


def test_random_folder_round_trip(tmp_path):
    folder = cases.make_folder(tmp_path, "vu-a")
    config, tensors = plain.read_folder(folder)
    assert config["layers"] == cases.CASES["vu-a"]["config"]["layers"] and config["streams"] == 2
    model = DecoderModel(parse_config(config))
    for r in model.tensor_requests():
        assert tuple(tensors[r.checkpoint_name].shape) == tuple(r.decl.shape)
    mix = tensors["l0.hc1.mix"]
    assert (mix.diagonal() - 1).abs().max() < 0.3 and tensors["l1.mix.f.b"].min() >= 1.0
    logits = plain.forward(config, tensors, [5, 9, 200, 31])
    assert logits.shape == (4, 300) and torch.isfinite(logits).all()


def test_window_releases_pages_but_never_those_of_the_kept_first_tokens():
    m = CacheManager([GroupPolicy(8, window=10, keep_first=9), GroupPolicy(8, window=10)], [12, 12], 2)
    m.add_request("a")
    m.extend("a", 50)
    m.extend("a", 1)                 # releases what positions 50's window (41..50) has passed
    kept, plain_window = m.block_table("a", 0), m.block_table("a", 1)
    assert kept[0] >= 0 and kept[1] >= 0                  # tokens 0..8 live in blocks 0 and 1
    assert kept[2:5] == [-1, -1, -1] and kept[5] >= 0     # block 5 holds position 41
    assert plain_window[:5] == [-1] * 5 and plain_window[5] >= 0
    assert m.pages_for(0, 1000, 1) == m.pages_for(1, 1000, 1) + 2
    m.check_invariants()
    m.remove_request("a")
    assert m.free_pages(0) == 12 and m.free_pages(1) == 12


def test_plain_rules():
    assert [j for j in range(12) if plain.visible(11, j, 4, 2)] == [0, 1, 8, 9, 10, 11]
    assert not plain.visible(3, 4, 100, 100)
    x = torch.arange(12, dtype=torch.float64).view(1, 1, 12) + 1
    y = plain.rotate_interleaved(x, torch.tensor([5]), 100.0, 8)
    assert torch.equal(y[..., 8:], x[..., 8:])            # features from `dims` on pass
    a = 5 * 100.0 ** (-2 * 1 / 8)                         # the second pair's angle
    c, s = torch.cos(torch.tensor(a, dtype=torch.float64)), torch.sin(torch.tensor(a, dtype=torch.float64))
    assert torch.allclose(y[0, 0, 2:4], torch.stack([3 * c - 4 * s, 4 * c + 3 * s]))
    conv = plain.causal_conv(torch.tensor([[1.0], [2.0], [3.0]]), torch.tensor([[10.0, 1.0]]))
    assert conv.flatten().tolist() == [1.0, 12.0, 23.0]
    # a sink takes weight from the keys and gives nothing back
    q = torch.zeros(1, 1, 4, dtype=torch.float64)
    k = torch.zeros(1, 1, 4, dtype=torch.float64)
    v = torch.ones(1, 1, 2, dtype=torch.float64)
    out = plain.attend(q, k, v, torch.tensor([0]), torch.zeros(1, dtype=torch.float64), 1.0, None, 0)
    assert torch.allclose(out, torch.full((1, 1, 2), 0.5, dtype=torch.float64))


def test_cache_pages_may_hold_values_of_another_size():
    from crucible_b200.engine.context import CacheStorage
    same = CacheStorage(2, 5, 8, 3, 16, torch.float32, "cpu")
    assert same.keys(1).shape == (5, 3, 8, 16) and same.values(1).shape == (5, 3, 8, 16)
    other = CacheStorage(2, 5, 8, 3, 16, torch.float32, "cpu", value_dim=40)
    assert other.keys(1).shape == (5, 3, 8, 16) and other.values(1).shape == (5, 3, 8, 40)
    assert other.keys(0).data_ptr() != other.keys(1).data_ptr()


def test_named_shapes_of_the_design_parse():
    from crucible_b200.config import shape
    for name in ("vuvosun-w1024", "vuvosun-w2048"):
        cfg = parse_config(shape(name))
        assert cfg.architecture == "Vuvosun" and len(cfg.layers) == 4
        assert [l.mixer.kind for l in cfg.layers] == ["mlstm", "parallel", "mlstm", "parallel"]
