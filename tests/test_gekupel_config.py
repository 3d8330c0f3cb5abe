"""Gekupel's configuration, weight plan and random-weights writer (no GPU)."""
import copy
import json
import os

import pytest

import gekupel_configs as gc
from geneinfer_b200.config import ConfigError, parse_config
from geneinfer_b200.config.gekupel import distance_slopes
from geneinfer_b200.weights import load_model_folder


def test_config_round_trip_and_translation():
    for raw in (gc.GEK_A, gc.GEK_B, gc.GEK_C):
        arch, cfg = parse_config(raw)
        assert arch.name == "Gekupel" and cfg.to_json() == raw
        spec = cfg.model_spec()
        spec.validate()
        assert len(spec.layers) == len(raw["layers"]) and not spec.tie_word_embeddings and spec.open_ended
        assert spec.embedding_scale == raw["embedding"]["scale"]
        for i, (layer, entry) in enumerate(zip(spec.layers, raw["layers"])):
            assert layer.block == "output_norm"
            assert (layer.feed_forward is None) == (entry["mlp"] is None)
            if entry["type"] == "attention":
                p = layer.mixer.params
                assert layer.mixer.kind == "attention" and p["chunk"] == entry["mixer"]["mask"]["size"] and p["window"] is None
                assert p["value_dim"] == entry["mixer"]["vdim"] and p["sink"] == "learned" and p["distance_slopes"] == distance_slopes(p["num_heads"])
            else:
                p = layer.mixer.params
                assert layer.mixer.kind == "latent_attention" and p["window"] == entry["mixer"]["mask"]["size"]
                second = entry["type"] == "latent_attention_2"
                assert (p["sink"] == "learned") == second and (p["position"].params["ramp_scaling"] is not None) == second
            if entry["mlp"] and entry["mlp"]["kind"] == "moe":
                assert layer.feed_forward.kind == "routed_experts" and layer.feed_forward.params["top"] == entry["mlp"]["router"]["top"]


def test_a_shared_layer_runs_the_owners_parts_on_a_cache_of_its_own():
    _, cfg = parse_config(gc.GEK_A)
    spec = cfg.model_spec()
    assert spec.shared_layers == {3: 1}
    assert (spec.schedule[3].layer, spec.schedule[3].cache_of) == (1, 3) and spec.schedule[1].cache_of is None
    plan_names = {r.name for r in __import__("geneinfer_b200").weights.plan.gekupel_weight_plan(cfg).rules}
    assert not any(n.startswith("l3.") for n in plan_names) and "l1.mlp.e4.down" in plan_names and "l1.mix.sink" in plan_names
    assert "l2.mix.sink" not in plan_names and "l0.mix.sink" in plan_names and "l4.norm2" not in plan_names


def test_slopes_fall_from_head_to_head():
    s = distance_slopes(4)
    assert s == [0.25, 0.0625, 0.015625, 0.00390625] and distance_slopes(1) == [2.0 ** -8]


@pytest.mark.parametrize("change, text", [
    (lambda c: c["layers"][0].update(type="sliding"), "unknown type"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=6), "rot.dims must equal rot_dim"),
    (lambda c: c["layers"][0]["mixer"]["rot"].pop("scaling"), "scaling"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=4), "multiple of kv_heads"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=6), "exceeds the number of experts"),
    (lambda c: c["layers"][1]["mlp"].update(kind="sparse"), "unknown kind"),
    (lambda c: c["layers"][3].update(weights_of=3), "must name another layer"),
    (lambda c: c["layers"][3].update(weights_of=0), "described differently"),
    (lambda c: c["layers"][3]["mixer"].update(scale=0.31), "described differently"),
    (lambda c: c.pop("embedding"), "embedding"),
    (lambda c: c["layers"][2]["mixer"].pop("q_rank"), "q_rank"),
])
def test_bad_configurations_are_refused(change, text):
    raw = copy.deepcopy(gc.GEK_A)
    change(raw)
    with pytest.raises(ConfigError, match=text):
        parse_config(raw)


def test_random_weights_folder_loads_by_name(tmp_path):
    folder = gc.make_model_dir(gc.GEK_A, 3, str(tmp_path / "m"))
    arch, cfg, params = load_model_folder(folder)
    assert arch.name == "Gekupel"
    assert tuple(params["layers.1.feed_forward.w_gate_up"].shape) == (5, 80, 96)
    assert tuple(params["layers.1.feed_forward.w_down"].shape) == (5, 96, 40)
    assert tuple(params["layers.0.mixer.w_down"].shape) == (56 + 48 + 8, 96)
    assert tuple(params["layers.1.mixer.w_qkv"].shape) == (6 * 24 + 2 * 24 + 2 * 40, 96)
    assert not any(k.startswith("layers.3.") for k in params)
    assert json.load(open(os.path.join(folder, "config.json")))["architecture"] == "Gekupel"
