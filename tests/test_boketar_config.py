"""Boketar without a GPU: configuration reading, the model description's tensor names, and the
plain implementation's own consistency."""
import copy
import json
import os

import pytest
import torch

import boketar_configs as B
from plain import boketar_plain as P

from poor_mans_mamba_b200.config import ConfigError, open_model_dir, resolve_architecture
from poor_mans_mamba_b200.engine.model import Model
from poor_mans_mamba_b200.weights import ModelFiles, write_random_model
from poor_mans_mamba_b200.weights.loader import check_tensors
import poor_mans_mamba_b200.architectures  # noqa: F401


@pytest.mark.parametrize("which", ["A", "B", "C"])
def test_description_names_every_tensor_and_reads_ranks_from_shapes(which, tmp_path):
    d, cfg, weights = B.make_model_dir(which, str(tmp_path))
    assert "decay_rank" not in json.dumps(json.load(open(os.path.join(d, "config.json"))))
    arch, typed = open_model_dir(d)
    assert arch.name == "Boketar"
    model = Model(arch.model_spec(typed))
    specs = model.param_specs()
    assert set(specs) == set(weights)
    for name, spec in specs.items():
        assert tuple(spec.shape) == tuple(weights[name].shape), name
    files = ModelFiles(d)
    try:
        assert check_tensors(specs, model.ignored_names(), files, strict=True) == []
    finally:
        files.close()
    assert typed.streams == cfg.get("streams")
    assert model.spec.residual_lanes == cfg.get("streams")
    kinds = [l.arrangement for l in model.spec.layers]
    assert set(kinds) == ({"hyper_prenorm"} if "streams" in cfg else {"parallel_prenorm"})


def test_states_of_every_layer_kind():
    cfg = B.config("A")
    arch = resolve_architecture(cfg)
    model = Model(arch.model_spec(arch.parse(cfg)))
    states = model.state_specs()
    left = cfg["layers"][0]["mixer"]["left"]
    assert [n for n, _ in states[0]] == ["mix.left.kv", "mix.left.conv", "mix.right.S"]
    kv = dict(states[0])["mix.left.kv"]
    assert kv.kind == "paged" and kv.window == left["mask"]["size"] and kv.width == left["kv_heads"] * 32
    assert dict(states[1])["mix.S"].shape == (4, 24, 16) and dict(states[1])["mix.conv"].shape == (2, 2 * 2 * 24 + 4 * 16)


def test_random_weights_mode_needs_the_ranks_in_the_configuration(tmp_path):
    cfg = B.config("B")
    out = write_random_model(cfg, 3, str(tmp_path / "m"))
    arch, typed = open_model_dir(out)
    assert typed.layers[0].delta.decay_rank == 16 and typed.layers[0].delta.gate_rank == 8
    bare = copy.deepcopy(cfg)
    del bare["layers"][0]["mixer"]["decay_rank"]
    with pytest.raises(ConfigError, match="decay_rank"):
        resolve_architecture(bare).parse(bare)


@pytest.mark.parametrize("edit,message", [
    (lambda c: c["layers"][0].__setitem__("type", "conv"), "unknown layer type"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "routed"), "unknown feed-forward"),
    (lambda c: c["layers"][0]["mixer"]["left"].__setitem__("heads", 3), "no multiple of kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].__setitem__("dims", 7), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["right"].__setitem__("decay", [0.5]), "decay"),
    (lambda c: c.__setitem__("streams", 9), "streams"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["norm"].pop("eps"), "eps"),
])
def test_configurations_that_are_refused(edit, message):
    cfg = B.config("A")
    edit(cfg)
    with pytest.raises(ConfigError, match=message):
        resolve_architecture(cfg).parse(cfg)


def test_one_lane_with_unit_weights_is_the_plain_residual_stream():
    cfg = B.config("C")
    W = B.make_weights(cfg, 5)
    for k in W:
        if ".hc" in k:
            W[k] = torch.ones_like(W[k])
    toks = B.sequences(cfg, (30,))[0]
    with_lanes = P.forward(cfg, W, toks)
    plain = copy.deepcopy(cfg)
    del plain["streams"]
    assert torch.allclose(with_lanes, P.forward(plain, W, toks), atol=1e-12)


def test_plain_recurrences_do_not_depend_on_how_the_sequence_is_told():
    """The delta rule of a prefix equals the prefix of the delta rule (causality of the oracle itself),
    and the window attention of a long sequence equals that of its last window for the last token."""
    torch.manual_seed(0)
    T, H, d, dv = 40, 2, 8, 6
    q, k, v = torch.randn(T, H, d).double(), torch.randn(T, H, d).double(), torch.randn(T, H, dv).double()
    beta, g = torch.rand(T, H).double(), torch.rand(T, H, d).double()
    full = P.gated_delta_rule(q, k, v, beta, g)
    assert torch.allclose(full[:17], P.gated_delta_rule(q[:17], k[:17], v[:17], beta[:17], g[:17]), atol=1e-12)
    sink = torch.tensor([0.3, -1.0]).double()
    a = P.windowed_sink_attention(q, k, v, 0.4, 9, sink)
    b = P.windowed_sink_attention(q[-9:], k[-9:], v[-9:], 0.4, 9, sink)
    assert torch.allclose(a[-1], b[-1], atol=1e-12)
    c = P.windowed_sink_attention(q[-10:], k[-10:], v[-10:], 0.4, 10, sink)
    assert not torch.allclose(a[-1], c[-1], atol=1e-6)
