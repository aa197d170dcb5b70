"""The Regupel configuration without a GPU: reading config.json, what may be absent, what is refused, the spec it turns into,
the tensors it expects, and hand-made numbers for the plain implementation's mechanisms."""
import copy
import json
import math

import pytest
import torch

import plain_regupel as plain
from qwen_triton_b200 import config_from_dict, load_preset
from qwen_triton_b200.config import ConfigError, RegupelConfig
from qwen_triton_b200.engine.model import expected_tensors

RAW = {
    "architecture": "Regupel", "vocab": 50, "width": 24, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0}, "logit_scale": 3.0, "residual_mult": 0.25,
    "layers": [
        {"type": "attention", "mlp": {"kind": "moe", "expert": {"ff": 10}, "router": {"experts": 3, "top": 2}, "shared": {"ff": 6}},
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 6, "scale": 0.3, "mask": {"size": 9},
                   "rot": {"base": 1000.0, "dims": 4, "scaling": {"factor": 2.0, "low": 1.0, "high": 3.0, "original": 16}}}},
        {"type": "parallel", "mlp": None,
         "mixer": {"left": {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 4, "scale": 0.5, "mask": {"size": 5, "keep_first": 2}}, "left_scale": 0.7,
                   "right": {"heads": 3, "dim": 4, "vdim": 2, "decay": [0.5, 0.9, 1.0]}, "right_scale": 1.2}},
        {"type": "attention", "mlp": {"kind": "moe", "expert": {"ff": 10}, "router": {"experts": 3, "top": 2}, "shared": {"ff": 6}},
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 6, "scale": 0.3, "mask": {"size": 9},
                   "rot": {"base": 1000.0, "dims": 4, "scaling": {"factor": 2.0, "low": 1.0, "high": 3.0, "original": 16}}}, "weights_of": 0},
    ],
}


def test_it_is_chosen_by_its_name_and_round_trips():
    config = config_from_dict(RAW)
    assert isinstance(config, RegupelConfig) and config.vocab_size == 50 and config.hidden_size == 24 and config.num_hidden_layers == 3
    assert config_from_dict(json.loads(json.dumps(config.to_hf_dict()))) == config
    for name in ("regupel-tiny-a", "regupel-tiny-b"):
        preset = load_preset(name)
        assert config_from_dict(preset.to_hf_dict()) == preset


def test_the_spec_runs_a_layer_twice_with_one_set_of_tensors():
    spec = config_from_dict(RAW).model_spec()
    assert [call.layer for call in spec.schedule] == [0, 1, 0] and all(call.cache_of is None for call in spec.schedule)
    assert [layer.prefix for layer in spec.layers] == ["l0", "l1"]
    names = expected_tensors(spec)
    assert not any(name.startswith("l2.") for name in names)
    wanted = {"embed": (50, 24), "final.norm": (24,), "final.norm.b": (24,), "l0.norm1": (24,), "l0.norm1.b": (24,), "l0.norm2.b": (24,),
              "l0.mix.q": (32, 24), "l0.mix.k": (16, 24), "l0.mix.v": (12, 24), "l0.mix.sink": (4,), "l0.mix.g": (4, 24), "l0.mix.o": (24, 24),
              "l0.mlp.router": (3, 24), "l0.mlp.e2.gate": (10, 24), "l0.mlp.e0.down": (24, 10), "l0.mlp.shared.up": (6, 24),
              "l1.mix.left.q": (8, 24), "l1.mix.left.q.norm": (8,), "l1.mix.left.k.norm": (4,), "l1.mix.left.o": (24, 8),
              "l1.mix.right.q": (12, 24), "l1.mix.right.v": (6, 24), "l1.mix.right.g": (6, 24), "l1.mix.right.norm": (6,), "l1.mix.right.o": (24, 6)}
    for name, shape in wanted.items():
        assert tuple(names[name].shape) == shape, name
    assert "l1.norm2" not in names or names["l1.norm2"].optional          # a layer without a feed-forward
    assert "l0.mlp.shared.gate_weight" not in names and "l1.mix.left.sink" not in names and "l1.mix.left.g" not in names


def test_a_layer_may_name_one_that_runs_another_layers_tensors():
    raw = copy.deepcopy(RAW)
    raw["layers"].append({**copy.deepcopy(raw["layers"][2]), "weights_of": 2})
    spec = config_from_dict(raw).model_spec()
    assert [call.layer for call in spec.schedule] == [0, 1, 0, 0] and len(spec.layers) == 2


def test_what_may_be_absent():
    raw = copy.deepcopy(RAW)
    del raw["layers"][0]["mixer"]["mask"], raw["layers"][0]["mixer"]["rot"]["scaling"], raw["layers"][0]["mlp"]["shared"]
    del raw["layers"][2]["mixer"]["mask"], raw["layers"][2]["mixer"]["rot"]["scaling"], raw["layers"][2]["mlp"]["shared"]
    del raw["layers"][1]["mixer"]["left"]["mask"], raw["embedding"], raw["residual_mult"], raw["logit_scale"]
    config = config_from_dict(raw)
    first = config.layers[0]
    assert first.attention.window is None and first.attention.rot_scaling is None and first.mlp.shared_ff is None
    assert config.layers[1].attention.window is None and config.embedding_scale == config.residual_mult == config.logit_scale == 1.0
    spec = config.model_spec()
    assert spec.layers[0].mixer["position"].kind == "rope_wavelength" and "factor" not in spec.layers[0].mixer["position"].params
    del raw["layers"][0]["mixer"]["rot"], raw["layers"][2]["mixer"]["rot"]
    assert config_from_dict(raw).model_spec().layers[0].mixer["position"].kind == "none"


@pytest.mark.parametrize("change, words", [
    (lambda r: r["layers"][0].update(type="conv"), "no mixer"),
    (lambda r: r["layers"][0]["mlp"].update(kind="dense"), "no feed-forward"),
    (lambda r: r["layers"][0]["mixer"].update(heads=3), "not a multiple"),
    (lambda r: r["layers"][1]["mixer"]["right"].update(decay=[0.5]), "one decay per head"),
    (lambda r: r["layers"][1]["mixer"]["right"].update(decay=[0.5, 0.9, 1.5]), "decays"),
    (lambda r: r["layers"][0]["mlp"]["router"].update(top=4), "of 3 experts"),
    (lambda r: r["layers"][2].update(weights_of=2), "earlier layer"),
    (lambda r: r["layers"][2].update(weights_of=1), "differs"),
    (lambda r: r["layers"][2]["mixer"].update(scale=0.4), "differs"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=3), "even"),
    (lambda r: r.pop("vocab"), "vocab"),
    (lambda r: r["layers"][1]["mixer"].pop("right"), "right"),
])
def test_refusals_in_words(change, words):
    raw = copy.deepcopy(RAW)
    change(raw)
    with pytest.raises(ConfigError, match=words):
        config_from_dict(raw)


def test_the_plain_mechanisms_on_numbers_made_by_hand():
    # layer norm: mean 2, variance 2/3 for (1, 2, 3)
    out = plain.layer_norm(torch.tensor([[1.0, 2.0, 3.0]], dtype=torch.float64), torch.tensor([2.0, 2.0, 2.0]), torch.tensor([0.5, 0.5, 0.5]), 0.0)
    torch.testing.assert_close(out, torch.tensor([[-2.0 * math.sqrt(1.5) + 0.5, 0.5, 2.0 * math.sqrt(1.5) + 0.5]], dtype=torch.float64))
    # window 2 with one kept first key and a sink of ln 2: query 3 sees keys 0, 2, 3 with equal scores of 0
    q, k = torch.zeros(4, 1, 2, dtype=torch.float64), torch.zeros(4, 1, 2, dtype=torch.float64)
    v = torch.tensor([1.0, 10.0, 100.0, 1000.0], dtype=torch.float64).view(4, 1, 1)
    out = plain.masked_softmax_attention(q, k, v, 1.0, 2, 1, torch.tensor([math.log(2.0)], dtype=torch.float64))
    torch.testing.assert_close(out[:, 0, 0], torch.tensor([1 / 3.0, 11 / 4.0, 111 / 5.0, 1101 / 5.0], dtype=torch.float64))
    # a pair turned by a quarter turn: (1, 0) -> (0, 1); the element behind the rotated ones stays
    turned = plain.rotate(torch.tensor([[[1.0, 0.0, 7.0]]], dtype=torch.float64), torch.tensor([1]), torch.tensor([math.pi / 2], dtype=torch.float64), 2)
    torch.testing.assert_close(turned, torch.tensor([[[0.0, 1.0, 7.0]]], dtype=torch.float64), atol=1e-12, rtol=0)
    # wavelengths: 2 pi (kept: below 32 / 3), 2 pi 1000^(1/2) = 199 (divided: above 32)
    freqs = plain.stretched_frequencies(4, 1000.0, {"factor": 2.0, "low": 1.0, "high": 3.0, "original": 32})
    torch.testing.assert_close(freqs, torch.tensor([1.0, 1000.0 ** -0.5 / 2.0], dtype=torch.float64))
    # a wavelength of 2 pi between 16 / 3 and 16: blended with s = (16 / (2 pi) - 1) / 2
    blend = (16.0 / (2.0 * math.pi) - 1.0) / 2.0
    freqs = plain.stretched_frequencies(2, 1000.0, {"factor": 2.0, "low": 1.0, "high": 3.0, "original": 16})
    torch.testing.assert_close(freqs, torch.tensor([(1.0 - blend) / 2.0 + blend], dtype=torch.float64))
    # the recurrence with decay 0.5: S_1 = k_1 v_1, S_2 = 0.5 S_1 + k_2 v_2
    q = torch.tensor([[[1.0]], [[1.0]]], dtype=torch.float64)
    out = plain.decayed_linear_attention(q, torch.tensor([[[2.0]], [[3.0]]], dtype=torch.float64), torch.tensor([[[5.0]], [[7.0]]], dtype=torch.float64),
                                         torch.tensor([0.5], dtype=torch.float64))
    torch.testing.assert_close(out[:, 0, 0], torch.tensor([10.0, 26.0], dtype=torch.float64))
    # one expert of two chosen, its score on the input: silu(w s) * (w s) with all matrices 1 x 1 ones
    t = {"p.router": torch.tensor([[1.0], [-1.0]], dtype=torch.float64)}
    for e in range(2):
        t.update({f"p.e{e}.gate": torch.ones(1, 1, dtype=torch.float64) * (e + 1), f"p.e{e}.up": torch.ones(1, 1, dtype=torch.float64),
                  f"p.e{e}.down": torch.ones(1, 1, dtype=torch.float64)})
    h = torch.tensor([[2.0], [-2.0]], dtype=torch.float64)
    out = plain.routed_feed_forward(h, t, "p", {"router": {"experts": 2, "top": 1}, "shared": None})
    s = 1.0 / (1.0 + math.exp(-2.0))
    first = (2 * s) / (1.0 + math.exp(-2 * s)) * (2 * s)                       # expert 0 for h = 2
    second = (2 * -2 * s) / (1.0 + math.exp(2 * 2 * s)) * (-2 * s)            # expert 1 (gate matrix 2) for h = -2
    torch.testing.assert_close(out[:, 0], torch.tensor([first, second], dtype=torch.float64))
