"""The Futepel design without a GPU: its config reader and the errors it gives, tensor
names and shapes, storage planning, the random folder, and the plain model's own rules."""
import copy
import math

import pytest
import torch

import futepel_cases as cases
import plain_futepel as plain
from crucible_b200.config.model_config import ConfigError
from crucible_b200.config.registry import known_architectures, parse_config
from crucible_b200.models.decoder import DecoderModel


def _config(name="fu-a"):
    return copy.deepcopy(cases.CASES[name]["config"])


def test_the_architecture_is_registered_and_parsed():
    assert "Futepel" in known_architectures()
    cfg = parse_config(_config())
    assert (cfg.vocab_size, cfg.hidden_size, cfg.max_context, cfg.tie_word_embeddings) == (300, 64, 512, False)
    kinds = [(layer.mixer.kind, layer.feed_forward.kind) for layer in cfg.layers]
    assert kinds == [("latent_attention", "moe"), ("wkv", "dense_act"), ("mamba2", "none"),
                     ("latent_attention", "dense_act")]
    first = cfg.layers[0].mixer
    assert (first.n_heads, first.head_dim, first.option("rot_dim"), first.option("value_dim"),
            first.option("kv_rank"), first.softmax_scale) == (2, 24, 8, 16, 40, 0.2)
    assert dict(first.position.scaling) == cases.YARN and first.position.theta == 10000.0
    assert cfg.layers[3].mixer.position.scaling is None
    assert cfg.embedding.option("bigram") == (97, 31, 5) and cfg.embedding.option("scale") == 4.0
    moe = cfg.layers[0].feed_forward
    assert (moe.option("experts"), moe.option("top"), moe.intermediate, moe.option("shared_intermediate")) == (6, 2, 40, 24)
    assert [name for name, _ in cfg.layers[2].norms] == ["mixer_norm"]      # no feed-forward: one norm


@pytest.mark.parametrize("edit,word", [
    (lambda c: c["layers"][0].update(type="conv"), "unknown layer type"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10), "rot_dim"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=7), "top"),
    (lambda c: c["layers"][1]["mlp"].update(kind="glu"), "kind"),
    (lambda c: c["embedding"]["bigram"].pop("mul_cur"), "mul_cur"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c.update(layers=[]), "layers"),
    (lambda c: c["layers"][2]["mixer"].update(conv=0), "conv"),
])
def test_config_errors_name_the_key(edit, word):
    config = _config()
    edit(config)
    with pytest.raises(ConfigError) as e:
        parse_config(config)
    assert word in str(e.value)


def test_sizes_that_do_not_fit_are_refused_when_the_model_is_built():
    config = _config()
    config["layers"][2]["mixer"]["norm_groups"] = 5            # 4 heads x 16 is not divisible by 5
    with pytest.raises(ValueError):
        DecoderModel(parse_config(config))
    config = _config()
    config["layers"][2]["mixer"]["groups"] = 3                 # 4 heads, 3 groups
    with pytest.raises(ValueError):
        DecoderModel(parse_config(config))


def test_tensor_names_shapes_and_storage():
    model = DecoderModel(parse_config(_config()))
    shapes = {r.checkpoint_name: tuple(r.decl.shape) for r in model.tensor_requests()}
    assert shapes["embed"] == (300, 64) and shapes["bigram"] == (98, 64) and shapes["pos"] == (512, 64)
    assert shapes["head"] == (300, 64) and shapes["final.norm"] == (64,)
    assert shapes["l0.mix.q"] == (2 * (24 + 8), 64) and shapes["l0.mix.dkv"] == (40 + 8, 64)
    assert shapes["l0.mix.uk"] == (2 * 24, 40) and shapes["l0.mix.uv"] == (2 * 16, 40) and shapes["l0.mix.g"] == (2, 64)
    assert shapes["l0.mlp.e5.down"] == (64, 40) and shapes["l0.mlp.shared.gate"] == (24, 64)
    assert shapes["l0.mlp.router"] == (6, 64)
    assert shapes["l1.mix.w1"] == (8, 64) and shapes["l1.mix.w2"] == (32, 8) and shapes["l1.mix.u"] == (2, 16)
    assert shapes["l2.mix.in"] == (2 * 64 + 2 * 2 * 24 + 4, 64) and shapes["l2.mix.conv"] == (64 + 96, 3)
    assert "l2.norm2" not in shapes and "l2.norm1" in shapes and "l3.norm2" in shapes
    # the two attention layers differ in their rows: pages of their own, one row per token
    needs = [(g.need.head_dim, g.need.kv_heads, g.need.values_are_keys, g.layers) for g in model.cache_groups]
    assert needs == [(48, 1, True, (0,)), (64, 1, True, (3,))]
    # state: the last token, then the recurrent layers' matrices, rows and tails
    wkv = 4 * 2 * 16 * 16 + 4 * 64
    ssd = 4 * 4 * 24 * 16 + 4 * 2 * (64 + 96)
    assert model.state_bytes == 16 + wkv + ssd
    assert model.embedding.state_binding.state_bytes == 4
    # equal attention layers share a group
    shared = DecoderModel(parse_config(_config("fu-c")))
    assert [g.layers for g in shared.cache_groups] == [(1, 2)]
    assert DecoderModel(parse_config(_config("fu-b"))).cache_groups == []


def test_the_random_folder_loads_back_and_a_rank_is_read_off_the_tensor(tmp_path):
    from crucible_b200.weights.safetensors_io import SafetensorsFile
    folder = cases.make_folder(tmp_path, "fu-a")
    config, tensors = plain.read_folder(folder)
    assert config["architecture"] == "Futepel"
    model = DecoderModel(parse_config(config))
    f = SafetensorsFile(f"{folder}/model.safetensors")
    assert sorted(f.names()) == sorted(r.checkpoint_name for r in model.tensor_requests())
    f.close()
    # a decay of another rank than the configuration's default loads: the axis is free
    from crucible_b200.weights.loader import _shape_fits
    decl = {r.checkpoint_name: r.decl for r in model.tensor_requests()}
    assert _shape_fits((5, 64), decl["l1.mix.w1"]) and _shape_fits((32, 5), decl["l1.mix.w2"])
    assert not _shape_fits((8, 65), decl["l1.mix.w1"]) and not _shape_fits((33, 8), decl["l1.mix.w2"])
    assert not _shape_fits((5, 64), decl["l1.mix.k"])
    logits = plain.forward(config, tensors, [1, 2, 3, 4, 5])
    assert logits.shape == (5, 300) and torch.isfinite(logits).all()


def test_the_frequencies_of_the_stretched_rotation_match_the_plain_ones():
    from crucible_b200.config.model_config import PositionSpec
    from crucible_b200.parts import POSITIONS
    for dims, base, scaling in [(8, 10000.0, cases.YARN), (32, 20000.0, {"factor": 2.0, "original": 128, "fast": 8.0, "slow": 1.0}),
                                (16, 500.0, None), (2, 100.0, cases.YARN)]:
        spec = PositionSpec(kind="rope_yarn", rotary_dim=dims, theta=base, max_positions=0,
                            scaling=tuple(scaling.items()) if scaling else None)
        part = POSITIONS.build("rope_yarn", spec)
        part.bind({}, torch.float32, "cpu")
        freq, mscale = plain.yarn_frequencies(dims, base, scaling, torch.float64)
        assert torch.allclose(part.frequencies()[0].double(), freq, rtol=1e-6)
        assert abs(part.magnitude() - mscale) < 1e-12
    # stretched: the slow frequencies are divided by the factor, the fast ones stay
    freq, mscale = plain.yarn_frequencies(32, 20000.0, {"factor": 2.0, "original": 128, "fast": 8.0, "slow": 1.0}, torch.float64)
    plain_f = 20000.0 ** (-2.0 * torch.arange(16, dtype=torch.float64) / 32)
    assert torch.isclose(freq[0], plain_f[0]) and torch.isclose(freq[-1], plain_f[-1] / 2.0)
    assert mscale == pytest.approx(0.1 * math.log(2.0) + 1.0)


def test_plain_rules():
    # bigram rows: the first token takes the row after the buckets; Python integers do not wrap
    assert plain.bigram_rows([5, 9, 9], 97, 31, 5).tolist() == [97, (5 * 31 + 9 * 5) % 97, (9 * 31 + 9 * 5) % 97]
    assert plain.bigram_rows([200, 210], 1009, 2147483647, 65537).tolist() == [1009, (200 * 2147483647 + 210 * 65537) % 1009]
    # routing: the softmax runs over the chosen logits alone
    idx, weight = plain.route(torch.tensor([[0.0, 3.0, 1.0, 2.0]], dtype=torch.float64), 2)
    assert idx.tolist() == [[1, 3]]
    assert torch.allclose(weight, torch.softmax(torch.tensor([[3.0, 2.0]], dtype=torch.float64), -1))
    # the wkv recurrence against its sum form: o_t = sum_{j<t} (prod_{j<i<t} w_i) (r_t . k_j) v_j + (r_t . u k_t) v_t
    g = torch.Generator().manual_seed(0)
    T, H, D = 6, 1, 3
    r, k, v = (torch.randn(T, H, D, generator=g, dtype=torch.float64) for _ in range(3))
    w = torch.rand(T, H, D, generator=g, dtype=torch.float64)
    u = torch.randn(H, D, generator=g, dtype=torch.float64)
    out = plain.wkv_recurrence(r, k, v, w, u)
    for t in range(T):
        want = (r[t, 0] * u[0] * k[t, 0]).sum() * v[t, 0]
        for j in range(t):
            decay = torch.ones(D, dtype=torch.float64)
            for i in range(j + 1, t):
                decay = decay * w[i, 0]
            want = want + (r[t, 0] * decay * k[j, 0]).sum() * v[j, 0]
        assert torch.allclose(out[t, 0], want)
    # the state-space recurrence with a decay of 1 and unit steps is a running sum
    x = torch.randn(5, 2, 3, generator=g, dtype=torch.float64)
    B = torch.randn(5, 1, 4, generator=g, dtype=torch.float64)
    C = torch.randn(5, 1, 4, generator=g, dtype=torch.float64)
    y = plain.ssd_recurrence(x, B, C, torch.ones(5, 2, dtype=torch.float64), torch.full((2,), -50.0, dtype=torch.float64),
                             torch.zeros(2, dtype=torch.float64), 1)
    want = sum((C[4, 0] * B[j, 0]).sum() * x[j, 1] for j in range(5))
    assert torch.allclose(y[4, 1], want)
    # the causal convolution: the last tap meets the current token, zeros before the start
    conv = plain.causal_conv(torch.tensor([[1.0], [2.0], [4.0]], dtype=torch.float64),
                             torch.tensor([[100.0, 10.0, 1.0]], dtype=torch.float64), torch.tensor([0.5], dtype=torch.float64))
    assert conv[:, 0].tolist() == [1.5, 12.5, 124.5]
