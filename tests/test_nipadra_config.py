"""Nipadra on the CPU: configuration keys, the translation into parts, the weight plan and the loader."""
import copy
import json
import os

import pytest
import torch

import nipadra_configs as nc
from geneinfer_b200.config import ConfigError, NipadraConfig, parse_config
from geneinfer_b200.weights import load_model_folder, write_random_model


def test_configuration_round_trip_and_registry():
    for raw in (nc.NIP_P, nc.NIP_Q):
        arch, cfg = parse_config(raw)
        assert arch.name == "Nipadra" and isinstance(cfg, NipadraConfig)
        assert cfg.to_json() == raw
        assert parse_config({**raw, "architectures": ["Nipadra"]})[0].name == "Nipadra"


def test_every_size_and_constant_reaches_the_parts():
    cfg = NipadraConfig.from_json(nc.NIP_P)
    spec = cfg.model_spec()
    assert spec.open_ended and spec.tie_word_embeddings and len(spec.layers) == 4
    first = spec.layers[0]
    assert first.block == "post_norm" and first.block_params == {"alpha": 1.5}
    assert first.mixer_norm.params == {"size": 96, "eps": 1e-5, "weight_offset": 1.0}
    (ln, left, ls), (rn, right, rs) = first.mixer.params["branches"]
    assert (ln, ls, rn, rs) == ("left", 0.7, "right", 1.25)
    assert left.params["window"] == 20 and left.params["scale"] == 0.3 and left.params["values"] == "keys"
    assert left.params["sink"] and left.params["head_gate"] and left.params["qk_norm_eps"] == 1e-5
    assert left.params["position"].params == {"head_dim": 32, "rotary_dim": 16, "theta": 10000.0, "pairing": "interleaved"}
    assert right.params["groups"] == 2 and right.params["conv_taps"] == 4 and right.params["norm_groups"] == 2
    assert first.feed_forward.params == {"hidden_size": 96, "intermediate_size": 136, "activation": "relu"}
    second = spec.layers[1]
    assert second.mixer.kind == "linear_attention" and second.mixer.params["decay"] == [1.0, 0.9, 0.5]
    assert second.feed_forward.params["activation"] == "silu"
    assert spec.layers[3].feed_forward is None and spec.layers[3].feed_forward_norm is None


@pytest.mark.parametrize("change, message", [
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["layers"][0].__setitem__("type", "other"), "unknown type"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("decay", [0.5]), "decay"),
    (lambda c: c["layers"][0]["mixer"]["left"].__setitem__("vdim", 48), "vdim"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].__setitem__("dims", 34), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["right"].__setitem__("groups", 3), "groups"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "routed"), "kind"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("act", "swish"), "act"),
    (lambda c: c.__setitem__("layers", []), "layers"),
])
def test_bad_configurations_are_refused(change, message):
    raw = copy.deepcopy(nc.NIP_P)
    change(raw)
    with pytest.raises(ConfigError, match=message):
        NipadraConfig.from_json(raw)


def test_weight_plan_names_shapes_and_assembly(tmp_path):
    folder = write_random_model(nc.NIP_P, 5, str(tmp_path / "p"), "bfloat16", std=0.1)
    from safetensors_names import names_and_shapes
    shapes = names_and_shapes(os.path.join(folder, "model.safetensors"))
    assert shapes["embed"] == [211, 96] and shapes["final.norm"] == [96]
    assert shapes["l0.mix.left.q"] == [128, 96] and shapes["l0.mix.left.k"] == [128, 96] and shapes["l0.mix.left.g"] == [4, 96]
    assert shapes["l0.mix.left.q.norm"] == [32] and shapes["l0.mix.left.o"] == [96, 128]
    assert shapes["l0.mix.right.in"] == [2 * 96 + 2 * 2 * 16 + 4, 96] and shapes["l0.mix.right.conv"] == [96 + 64, 4]
    assert shapes["l0.mix.right.conv.b"] == [160] and shapes["l0.mix.right.A_log"] == [4] and shapes["l0.mix.right.norm"] == [96]
    assert shapes["l1.mix.q"] == [48, 96] and shapes["l1.mix.v"] == [96, 96] and shapes["l1.mix.norm"] == [96]
    assert shapes["l1.mlp.gate"] == [72, 96] and "l2.norm2" not in shapes and "l3.mlp.up" not in shapes
    _, cfg, params = load_model_folder(folder)
    assert params["head.weight"] is params["embedding.weight"]
    assert tuple(params["layers.0.mixer.left.w_qkv"].shape) == (128 + 128 + 4, 96)
    assert tuple(params["layers.1.mixer.w_in"].shape) == (48 + 48 + 96 + 96, 96)
    assert tuple(params["layers.0.feed_forward.w_gate_up"].shape) == (272, 96)
    assert "layers.2.feed_forward.w_down" not in params
    assert float(params["layers.0.mixer_norm.weight"].float().abs().mean()) < 0.2      # stored around zero
