"""The Kerepel configuration and description without a GPU: the round trip of config.json, the errors, which parts a
layer gets, what the cache is asked to hold, the YaRN frequencies and the plain implementation's own small pieces."""
from __future__ import annotations

import copy
import math

import pytest
import torch

from kerepel_models import CONFIGS


def test_round_trip_and_description():
    from thintensor_b200.config.registry import load_config
    from thintensor_b200.engine.model import DecoderModel

    for name, raw in CONFIGS.items():
        arch, config = load_config(copy.deepcopy(raw))
        assert arch.name == "Kerepel" and config.to_dict() == raw, name
        spec = arch.describe(config)
        assert all(layer.arrangement == "pre_norm" for layer in spec.layers)
        assert [run.cache_from for run in spec.schedule] == [layer["mixer"].get("kv_from") for layer in raw["layers"]]
        declared = DecoderModel(spec, torch.float32, None).weight_declarations()
        assert ("bigram" in declared) == ("embedding" in raw) and ("side.embed" in declared) == ("token_side" in raw)
        assert declared["head"].alias_of == "embed" and declared["head"].prefer_alias
        if "token_side" in raw:
            assert declared["side.embed"].shape == (raw["vocab"], len(raw["layers"]) * raw["token_side"]["dim"])
        for index, layer in enumerate(raw["layers"]):
            mixer, mlp = layer["mixer"], layer["mlp"]
            assert (f"l{index}.norm2" in declared) == (mlp is not None)
            assert (f"l{index}.side.gate" in declared) == ("token_side" in raw)
            if layer["type"] == "attention":
                own = "kv_from" not in mixer
                for leaf in ("k", "v", "k.norm", "k.conv", "v.conv"):
                    assert (f"l{index}.mix.{leaf}" in declared) == (own and ("conv" in mixer or "conv" not in leaf)), (name, index, leaf)
                assert declared[f"l{index}.mix.g"].shape == (mixer["heads"] * mixer["vdim"], raw["width"])
                assert (f"l{index}.mix.q.conv" in declared) == ("conv" in mixer)
            else:
                assert declared[f"l{index}.mix.g"].shape == (mixer["heads"], raw["width"])
                assert declared[f"l{index}.mix.dkv"].shape == (mixer["kv_rank"] + mixer["rot_dim"], raw["width"])
            if mlp is not None and mlp["kind"] == "moe":
                assert declared[f"l{index}.mlp.correction"].shape == (mlp["router"]["experts"],)
                assert (f"l{index}.mlp.shared.sg" in declared) == ("shared" in mlp)


def test_what_the_cache_is_asked_for():
    from thintensor_b200.config.registry import load_config
    from thintensor_b200.engine.model import DecoderModel
    from thintensor_b200.parts.base import KVNeed

    arch, config = load_config(copy.deepcopy(CONFIGS["a"]))
    model = DecoderModel(arch.describe(config), torch.float32, None)
    kv, state, source = model.cache_needs()
    # the source keeps what its reader's wider window sees; the reader asks for its own window and keeps nothing
    assert kv[0] == KVNeed(3, 16, 40, 24) and kv[1] == KVNeed(1, 40 + 8, None, 0) and kv[2] == KVNeed(3, 16, 40, 24)
    assert source[:3] == [None, None, 0]
    assert [tuple(s.shape) for s in state[0]] == [(3, 3 * 16 + 3 * 16 + 3 * 24)] and [tuple(s.shape) for s in state[2]] == [(1, 3 * 16)]
    assert [(tuple(s.shape), s.dtype) for s in state[-1]] == [((), torch.int32)]
    cache = model.new_cache(8, 2, device=None)
    assert len(cache.kv_groups) == 2

    # a reader with a narrower window than its source leaves the source's need as it is
    arch, config = load_config(copy.deepcopy(CONFIGS["b"]))
    kv, _, source = DecoderModel(arch.describe(config), torch.float32, None).cache_needs()
    assert kv[1].window == 150 and kv[2].window == 70 and source[2] == 1

    # a reader without a window: the source's cache keeps everything
    raw = copy.deepcopy(CONFIGS["b"])
    del raw["layers"][2]["mixer"]["mask"]
    arch, config = load_config(raw)
    model = DecoderModel(arch.describe(config), torch.float32, None)
    kv, _, _ = model.cache_needs()
    assert kv[1].window is None and kv[2].window is None
    model.new_cache(8, 2, device=None)


@pytest.mark.parametrize("change,needle", [
    (lambda c: c["layers"][0].update(type="retention"), "known"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=10), "rotated part"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=5), "top"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda c: c["layers"][0]["mlp"].update(kind="gated"), "dense"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "earlier attention layer"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "earlier attention layer"),
    (lambda c: c["layers"][2]["mixer"].update(vdim=8), "differ"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=2), "multiple"),
    (lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].update(factor=0.0), "positive"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_errors(change, needle):
    from thintensor_b200.config.base import ConfigError
    from thintensor_b200.config.registry import load_config

    raw = copy.deepcopy(CONFIGS["a"])
    change(raw)
    with pytest.raises(ConfigError) as err:
        load_config(raw)
    assert needle in str(err.value)


def test_yarn_frequencies_against_the_plain_ones():
    """The position encoding's table for scaled and unscaled rotations equals the plain implementation's, and the scaling's
    edges sit where the formula puts them: pairs faster than ``fast`` turns keep their frequency, pairs slower than ``slow``
    turns are divided by the factor."""
    import plain_kerepel
    from thintensor_b200.parts.rope import RotaryEncoding, yarn_attention_scaling

    for rot in ({"dims": 8, "base": 1000.0, "scaling": {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}},
                {"dims": 32, "base": 10000.0, "scaling": {"factor": 2.0, "original": 64, "fast": 16.0, "slow": 2.0}},
                {"dims": 64, "base": 25000.0, "scaling": {"factor": 40.0, "original": 4096, "fast": 24.0, "slow": 1.5}},
                {"dims": 16, "base": 500.0}):
        want, factor = plain_kerepel.yarn_frequencies(rot)
        s = rot.get("scaling")
        scaling = None if not s else {"rope_type": "yarn", **s}
        part = RotaryEncoding(rot["dims"], rot["base"], rot["dims"], scaling, yarn_attention_scaling(s["factor"]) if s else 1.0, True, "float64")
        assert torch.equal(part.inv_freq_host, want), rot
        assert part.attention_scaling == pytest.approx(factor, abs=0.0)
        plain = torch.tensor([rot["base"] ** (-2.0 * i / rot["dims"]) for i in range(rot["dims"] // 2)], dtype=torch.float64)
        if s:
            assert float(want[0]) == pytest.approx(float(plain[0]), rel=1e-6)                       # the fastest pair is kept
            turns = s["original"] * plain / (2 * math.pi)
            slow = turns < s["slow"] * 0.5
            assert torch.allclose(want.double()[slow], (plain / s["factor"])[slow], rtol=1e-6)


def test_the_plain_pieces():
    """The oracle's own mechanisms on cases small enough to check by hand."""
    import plain_kerepel as P

    u = torch.tensor([[1.0, 10.0], [2.0, 20.0], [3.0, 30.0]], dtype=torch.float64)
    w = torch.tensor([[0.5, 1.0, 2.0], [0.0, 0.0, 1.0]], dtype=torch.float64)          # taps: oldest first
    y = P.short_convolution(u, w)
    assert torch.equal(y, torch.tensor([[2.0, 10.0], [5.0, 20.0], [8.5, 30.0]], dtype=torch.float64))
    # six experts in three groups: group scores are the sums of the two best CHOICE scores; weights are the plain scores
    scores = torch.tensor([0.9, 0.1, 0.5, 0.5, 0.2, 0.85], dtype=torch.float64)
    correction = torch.tensor([0.0, 0.0, 0.0, 0.0, 0.6, 0.0], dtype=torch.float64)
    chosen, weights = P.route(scores, correction, 2, 3, 2)
    assert chosen == [0, 5] and [float(x) for x in weights] == [0.9, 0.85]            # groups 0 (1.0) and 2 (1.65) stay, group 1 (1.0) loses the tie to group 0
    chosen, weights = P.route(scores, correction, 3, 3, 1)
    assert chosen == [5, 4] and [float(x) for x in weights] == [0.85, 0.2]            # only group 2 stays: fewer experts than top
    negative = torch.tensor([0.3, 0.2, 0.25, 0.1], dtype=torch.float64)
    chosen, _ = P.route(negative, torch.tensor([-1.0, -1.0, -0.9, -2.0], dtype=torch.float64), 1, 2, 1)
    assert chosen == [0]                                                              # group 0: -1.5 beats group 1: -2.55, though group 1 holds the best expert
    x = torch.arange(8, dtype=torch.float64).reshape(1, 8)
    turned = P.rotate_pairs(x, torch.tensor([3]), {"dims": 4, "base": 100.0})
    assert torch.equal(turned[0, 4:], x[0, 4:])
    a = 3.0 * 1.0
    assert float(turned[0, 0]) == pytest.approx(0.0 * math.cos(a) - 1.0 * math.sin(a), abs=1e-6)
    assert float(turned[0, 1]) == pytest.approx(1.0 * math.cos(a) + 0.0 * math.sin(a), abs=1e-6)
