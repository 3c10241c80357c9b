"""The Ramosun configuration reader, its model description and the random-weights writer, without a GPU."""
from __future__ import annotations

import copy

import numpy as np
import pytest
import torch

import plain_ramosun as plain
import ramosun_models as rm


def test_config_is_found_by_its_architecture_key_and_survives_a_round_trip():
    from celeg_b200.config import RamosunConfig, architecture_of
    for raw, _ in rm.CONFIGS.values():
        architecture = architecture_of(raw)
        assert architecture.name == "Ramosun"
        config = architecture.parse_config(raw)
        assert isinstance(config, RamosunConfig)
        again = architecture.parse_config(config.to_dict())
        assert again == config
        assert [index for index, _ in config.run_order()] == [index for index, _ in plain.run_order(raw)]
        assert [begins for _, begins in config.run_order()] == [begins for _, begins in plain.run_order(raw)]


def test_run_order_repeats_layers_with_caches_of_their_own_and_enters_every_pass():
    from celeg_b200.config import architecture_of
    raw, _ = rm.CONFIGS["loop_from_start"]
    spec = architecture_of(raw).build_spec(architecture_of(raw).parse_config(raw))
    assert [entry.layer for entry in spec.order] == [0, 1, 0, 1, 0, 1, 2, 3]
    assert [bool(entry.before) for entry in spec.order] == [True, False, True, False, True, False, False, False]
    assert all(entry.cache_of is None for entry in spec.order)
    straight, _ = rm.CONFIGS["straight"]
    spec = architecture_of(straight).build_spec(architecture_of(straight).parse_config(straight))
    assert not spec.stream_parts and all(not entry.before for entry in spec.order)


@pytest.mark.parametrize("name", list(rm.CONFIGS))
def test_description_names_exactly_the_tensors_of_a_model_folder(name):
    from celeg_b200.config import architecture_of
    from celeg_b200.weights import check_tensors
    raw, seed = rm.CONFIGS[name]
    tensors = rm.make_tensors(raw, seed)
    spec = architecture_of(raw).build_spec(architecture_of(raw).parse_config(raw))
    check_tensors(spec.all_tensors(), {key: tuple(value.shape) for key, value in tensors.items()},
                  {key: "BF16" for key in tensors})


@pytest.mark.parametrize("change,message", [
    (lambda raw: raw["layers"][0].update(type="hyena"), "unknown layer type"),
    (lambda raw: raw["layers"][0]["mixer"].update(vdim=7), "values are the keys"),
    (lambda raw: raw["layers"][0]["mixer"].update(kv_heads=3), "not a multiple"),
    (lambda raw: raw["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda raw: raw.update(loop={"start": 2, "stop": 9, "times": 2}), "loop"),
    (lambda raw: raw["layers"][1].update(mlp={"kind": "experts", "ff": 8}), "unknown kind"),
    (lambda raw: raw.pop("width"), "width"),
])
def test_faulty_configurations_are_refused_with_a_message(change, message):
    from celeg_b200.config import ConfigError, architecture_of
    raw = copy.deepcopy(rm.MIXED)
    change(raw)
    with pytest.raises(ConfigError, match=message):
        architecture_of(raw).parse_config(raw)


@pytest.mark.parametrize("rot", [
    {"base": 10000.0, "dims": 64, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 512}},
    {"base": 500.0, "dims": 16, "scaling": {"factor": 2.0, "low": 2.0, "high": 3.0, "original": 40}},
    {"base": 100.0, "dims": 6},
])
def test_frequencies_scaled_by_wavelength(rot):
    from celeg_b200.parts.positions import scale_by_wavelength
    half = rot["dims"] // 2
    plain_frequencies = torch.tensor([rot["base"] ** (-2.0 * i / rot["dims"]) for i in range(half)], dtype=torch.float64)
    got = plain_frequencies
    if "scaling" in rot:
        s = rot["scaling"]
        got = scale_by_wavelength(plain_frequencies, s["factor"], s["low"], s["high"], s["original"])
        assert not torch.equal(got, plain_frequencies)
    np.testing.assert_allclose(got.numpy(), plain.rotary_frequencies(rot), rtol=1e-12)


def test_random_weights_mode_writes_a_folder_the_plain_model_can_run(tmp_path):
    from safetensors.torch import load_file
    from celeg_b200.weights import write_random_model
    folder = write_random_model(str(tmp_path / "random"), copy.deepcopy(rm.MIXED), seed=3)
    tensors = plain.as_float64(load_file(folder + "/model.safetensors"))
    logits = plain.forward(rm.MIXED, tensors, [1, 2, 3, 4, 5, 6, 7])
    assert logits.shape == (7, rm.MIXED["vocab"]) and np.isfinite(logits).all()
    assert np.abs(logits).max() <= rm.MIXED["logit_softcap"] and logits.std() > 0.05


def test_plain_model_token_by_token_state_equals_whole_sequence():
    """The plain model's own check: a prefix of a sequence gives the prefix of its logits (causality)."""
    raw, seed = rm.CONFIGS["loop_once"]
    tensors = plain.as_float64(rm.make_tensors(raw, seed))
    tokens = list(range(20))
    whole = plain.forward(raw, tensors, tokens)
    np.testing.assert_allclose(plain.forward(raw, tensors, tokens[:11]), whole[:11], rtol=1e-9, atol=1e-9)
