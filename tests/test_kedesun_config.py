"""The Kedesun design without a GPU: its configuration reader, its model description against the tensors a
checkpoint holds, its random-weights mode, and the plain float64 model against itself (the latent attention with
every head's keys and values rebuilt equals the form in which the query is taken to the latent space)."""
from __future__ import annotations

import copy
import json
import math
import os

import numpy as np
import pytest

import kedesun_models as km
import plain_kedesun as plain
from celeg_b200.config import ConfigError, architecture_of
from celeg_b200.config.kedesun import KedesunConfig


def test_configuration_round_trip_and_tensor_table():
    for name, (raw, seed) in km.CONFIGS.items():
        architecture = architecture_of(raw)
        assert architecture.name == "Kedesun"
        config = architecture.parse_config(raw)
        again = KedesunConfig.from_dict(config.to_dict())
        assert again == config
        spec = architecture.build_spec(config)
        wanted = {ref.name: tuple(ref.shape) for ref in spec.all_tensors()}
        made = {key: tuple(value.shape) for key, value in km.make_tensors(raw, seed).items()}
        assert wanted == made, name
        assert len(spec.order) == len(raw["layers"]) and all(entry.cache_of is None for entry in spec.order)


def test_absent_scale_is_one_over_the_root_of_the_whole_key_size():
    raw = copy.deepcopy(km.single_layer(km.latent(2, 24, 8, 8, 16)))
    del raw["layers"][0]["mixer"]["scale"]
    config = architecture_of(raw).parse_config(raw)
    assert config.layers[0].scale == pytest.approx(32 ** -0.5)


@pytest.mark.parametrize("damage,message", [
    (lambda raw: raw["layers"][0].update(type="sliding"), "unknown layer type"),
    (lambda raw: raw["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda raw: raw["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda raw: raw["layers"][0]["mixer"]["rot"].update(dims=64), "at most"),
    (lambda raw: raw["layers"][1]["mixer"].update(decay=[0.5]), "decay"),
    (lambda raw: raw["layers"][1]["mlp"]["router"].update(top=9), "exceeds"),
    (lambda raw: raw["layers"][1]["mlp"].update(kind="sparse"), "unknown kind"),
    (lambda raw: raw.pop("norm"), "norm"),
    (lambda raw: raw.update(layers=[]), "layers"),
])
def test_faulty_configurations_are_refused_with_a_message(damage, message):
    raw = km.config(64, 32, [km.with_mlp(km.latent(2, 8, 8, 8, 16), km.dense(48)),
                             km.with_mlp(km.retention(2, 8, 8), km.moe(8, 2, 16, shared=8))])
    damage(raw)
    with pytest.raises(ConfigError, match=message):
        architecture_of(raw).parse_config(raw)


def test_random_weights_mode_writes_a_loadable_folder(tmp_path):
    from celeg_b200 import write_random_model
    from celeg_b200.weights.safetensors_io import TensorRepository
    raw, _ = km.CONFIGS["mixed"]
    folder = write_random_model(str(tmp_path / "random"), raw, seed=3)
    repository = TensorRepository(folder)
    shapes = repository.shapes()
    architecture = architecture_of(raw)
    wanted = {ref.name: tuple(ref.shape) for ref in architecture.build_spec(architecture.parse_config(raw)).all_tensors()}
    assert {key: tuple(value) for key, value in shapes.items()} == wanted
    average = repository.tensor("l2.dwa").float()
    assert average.shape == (4,) and 0.0 < float(average.mean()) < 1.0
    repository.close()
    assert json.load(open(os.path.join(folder, "config.json")))["architecture"] == "Kedesun"


def test_yarn_frequencies_at_their_limits():
    rot = {"base": 10000.0, "dims": 32}
    plainf, one = plain.yarn_frequencies(rot)
    assert one == 1.0 and plainf[0] == 1.0 and plainf[-1] == pytest.approx(10000.0 ** (-30 / 32))
    scaled, magnitude = plain.yarn_frequencies(dict(rot, scaling={"factor": 4.0, "original": 512, "fast": 32.0, "slow": 1.0}))
    assert magnitude == pytest.approx(0.1 * math.log(4.0) + 1.0)
    assert scaled[0] == plainf[0]                               # fast waves are kept
    assert scaled[-1] == pytest.approx(plainf[-1] / 4.0)        # slow waves are divided by the factor
    assert np.all(np.diff(scaled / plainf) <= 1e-12)            # the share of the divided frequency never falls
    # the engine's table of frequencies is the plain model's
    from celeg_b200.parts.positions import scale_by_turns
    import torch
    table = scale_by_turns(torch.from_numpy(plainf), 10000.0, 32, 4.0, 512.0, 32.0, 1.0).numpy()
    assert np.allclose(table, scaled, rtol=1e-14)


def test_plain_latent_attention_equals_its_absorbed_form():
    """Scores and outputs through the cached vector alone: (U_h^T q_h) . c + q_rot . r and V_h (sum p c)."""
    raw = km.single_layer(km.latent(3, 8, 4, 5, 6, yarn=km.YARN))
    tensors = plain.as_float64(km.make_tensors(raw, 5))
    mixer = raw["layers"][0]["mixer"]
    rng = np.random.default_rng(0)
    h = rng.normal(size=(11, raw["width"]))
    want = plain.latent_attention(tensors, "l0.mix.", mixer, h, 1e-5)
    heads, dim, rot, vdim, rank = 3, 8, 4, 5, 6
    positions = np.arange(11)
    q = (h @ tensors["l0.mix.q"].T).reshape(11, heads, dim + rot)
    down = h @ tensors["l0.mix.dkv"].T
    c = plain.rms_norm(down[:, :rank], tensors["l0.mix.dkv.norm"], 1e-5)
    r = plain.rotate_interleaved(down[:, rank:], positions, mixer["rot"])
    q_rot = plain.rotate_interleaved(q[:, :, dim:], positions, mixer["rot"])
    uk = tensors["l0.mix.uk"].reshape(heads, dim, rank)
    uv = tensors["l0.mix.uv"].reshape(heads, vdim, rank)
    gate = plain.sigmoid(h @ tensors["l0.mix.g"].T)
    out = np.zeros((11, heads, vdim))
    for head in range(heads):
        absorbed = q[:, head, :dim] @ uk[head]
        scores = (absorbed @ c.T + q_rot[:, head] @ r.T) * mixer["scale"]
        scores = np.where(np.tril(np.ones((11, 11), dtype=bool)), scores, -np.inf)
        p = np.exp(scores - scores.max(-1, keepdims=True))
        p /= p.sum(-1, keepdims=True)
        out[:, head] = ((p @ c) @ uv[head].T) * gate[:, head:head + 1]
    assert np.allclose(out.reshape(11, -1) @ tensors["l0.mix.o"].T, want, rtol=1e-10, atol=1e-12)


def test_plain_router_chooses_by_corrected_scores_and_weighs_by_plain_ones():
    raw = km.single_layer(km.retention(1, 8, 8), km.moe(4, 2, 8))
    tensors = plain.as_float64(km.make_tensors(raw, 6))
    tensors["l0.mlp.router"] = np.zeros((4, raw["width"]))
    tensors["l0.mlp.router"][:, 0] = [3.0, 2.0, 1.0, 0.0]
    tensors["l0.mlp.correction"] = np.array([0.0, 0.0, 0.0, 1.0])      # lifts the last expert over all others
    h = np.zeros((1, raw["width"]))
    h[0, 0] = 1.0
    chosen, weights = plain.route(tensors, "l0.mlp.", raw["layers"][0]["mlp"], h)
    assert chosen.tolist() == [[3, 0]]
    s = np.exp([3.0, 2.0, 1.0, 0.0]) / np.exp([3.0, 2.0, 1.0, 0.0]).sum()
    assert np.allclose(weights[0], [s[3] / (s[3] + s[0]), s[0] / (s[3] + s[0])])


def test_plain_retention_equals_its_sum_over_the_past():
    raw = km.single_layer(km.retention(2, 4, 3, [0.5, 0.9]))
    tensors = plain.as_float64(km.make_tensors(raw, 7))
    h = np.random.default_rng(1).normal(size=(9, raw["width"]))
    want = plain.retention(tensors, "l0.mix.", raw["layers"][0]["mixer"], h, 1e-5)
    q = (h @ tensors["l0.mix.q"].T).reshape(9, 2, 4)
    k = (h @ tensors["l0.mix.k"].T).reshape(9, 2, 4) / 2.0
    v = (h @ tensors["l0.mix.v"].T).reshape(9, 2, 3)
    read = np.zeros((9, 2, 3))
    for head, decay in enumerate((0.5, 0.9)):
        for t in range(9):
            for s in range(t + 1):
                read[t, head] += decay ** (t - s) * (q[t, head] @ k[s, head]) * v[s, head]
    read = plain.rms_scaled(read, 1e-5).reshape(9, 6)
    assert np.allclose((read * plain.silu(h @ tensors["l0.mix.g"].T)) @ tensors["l0.mix.o"].T, want, rtol=1e-10, atol=1e-12)
