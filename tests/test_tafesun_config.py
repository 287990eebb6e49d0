"""Tafesun's configuration reader, its description as parts and its tensor names (no GPU)."""
import copy
import json
import os

import pytest
import torch

import tafesun_configs as C
from plain import tafesun_plain as P

import poor_mans_mamba_b200.architectures  # noqa: F401  (registration)
from poor_mans_mamba_b200.config import ConfigError, TafesunConfig, resolve_architecture
from poor_mans_mamba_b200.config.registry import open_model_dir
from poor_mans_mamba_b200.engine.model import Model
from poor_mans_mamba_b200.weights.loader import check_tensors
from poor_mans_mamba_b200.weights.safetensors_io import ModelFiles


@pytest.mark.parametrize("which", ["A", "B", "C", "M"])
def test_every_size_and_constant_is_read(which):
    data = C.config(which)
    cfg = TafesunConfig.from_dict(data)
    assert (cfg.vocab_size, cfg.hidden_size, cfg.norm_eps, cfg.logit_scale) == (
        data["vocab"], data["width"], data["norm"]["eps"], data["logit_scale"])
    for layer, raw in zip(cfg.layers, data["layers"]):
        left, right, m = raw["mixer"]["left"], raw["mixer"]["right"], raw["mixer"]
        assert (layer.left.heads, layer.left.kv_heads, layer.left.dim, layer.left.vdim, layer.left.scale) == (
            left["heads"], left["kv_heads"], left["dim"], left["vdim"], left["scale"])
        assert (layer.left.rot_dims, layer.left.rot_base) == (left["rot"]["dims"], left["rot"]["base"])
        assert layer.left.rot_factor == (left["rot"]["scaling"]["factor"] if "scaling" in left["rot"] else 1.0)
        assert (layer.right.heads, layer.right.vdim, layer.right.state, layer.right.groups, layer.right.conv,
                layer.right.norm_groups) == tuple(right[k] for k in ("heads", "vdim", "state", "groups", "conv", "norm_groups"))
        assert (layer.left_scale, layer.right_scale) == (m["left_scale"], m["right_scale"])
        assert layer.weights_of == raw.get("weights_of")
        if raw["mlp"] is None:
            assert layer.mlp is None
        else:
            assert (layer.mlp.experts, layer.mlp.top, layer.mlp.expert_ff, layer.mlp.expert_limit) == (
                raw["mlp"]["router"]["experts"], raw["mlp"]["router"]["top"], raw["mlp"]["expert"]["ff"],
                raw["mlp"]["expert"]["limit"])
            shared = raw["mlp"].get("shared")
            assert (layer.mlp.shared_ff, layer.mlp.shared_limit) == ((shared["ff"], shared["limit"]) if shared else (0, 0.0))


def test_the_architecture_is_chosen_by_its_name():
    arch = resolve_architecture(C.config("A"))
    assert arch.name == "Tafesun"


@pytest.mark.parametrize("path,value,needle", [
    (("layers", 0, "mixer", "left", "heads"), 3, "layers[0].mixer.left.heads"),
    (("layers", 0, "mixer", "left", "rot", "dims"), 7, "layers[0].mixer.left.rot.dims"),
    (("layers", 0, "mixer", "left", "rot", "dims"), 18, "layers[0].mixer.left.rot.dims"),
    (("layers", 0, "mixer", "right", "groups"), 2, "layers[0].mixer.right.heads"),
    (("layers", 0, "mixer", "right", "norm_groups"), 5, "layers[0].mixer.right.norm_groups"),
    (("layers", 0, "mlp", "router", "top"), 6, "layers[0].mlp.router.top"),
    (("layers", 0, "mlp", "kind"), "dense", "layers[0].mlp.kind"),
    (("layers", 1, "type"), "serial", "layers[1].type"),
    (("layers", 2, "weights_of"), 9, "layers[2].weights_of"),
    (("layers", 2, "mixer", "left_scale"), 0.5, "layers[2].weights_of"),   # differs from the layer it borrows from
    (("width",), 0, "width"),
])
def test_errors_name_the_key(path, value, needle):
    data = C.config("A")
    node = data
    for k in path[:-1]:
        node = node[k]
    node[path[-1]] = value
    with pytest.raises(ConfigError) as exc:
        TafesunConfig.from_dict(data)
    assert needle in str(exc.value)


def test_missing_keys_and_circles_are_refused():
    data = C.config("A")
    del data["logit_scale"]
    with pytest.raises(ConfigError, match="logit_scale"):
        TafesunConfig.from_dict(data)
    data = C.config("A")
    del data["layers"][1]["mixer"]["right"]["state"]
    with pytest.raises(ConfigError, match="state"):
        TafesunConfig.from_dict(data)
    data = C.config("B")
    data["layers"][2]["weights_of"] = 0  # 0 -> 2 -> 0
    with pytest.raises(ConfigError, match="circle"):
        TafesunConfig.from_dict(data)


@pytest.mark.parametrize("which", ["A", "B", "C"])
def test_layers_that_borrow_tensors_run_on_caches_of_their_own(which):
    data = C.config(which)
    cfg = TafesunConfig.from_dict(data)
    spec = resolve_architecture(data).model_spec(cfg)
    own = [i for i, l in enumerate(data["layers"]) if l.get("weights_of") is None]
    assert [l.prefix for l in spec.layers] == [f"l{i}." for i in own]
    assert [c.cache_of for c in spec.order] == list(range(len(data["layers"])))
    assert [spec.layers[c.layer].prefix for c in spec.order] == [f"l{C.owner(data, i)}." for i in range(len(data["layers"]))]
    model = Model(spec)
    states = model.state_specs()
    assert sorted(states) == list(range(len(data["layers"])))
    for i, raw in enumerate(data["layers"]):
        L, R = raw["mixer"]["left"], raw["mixer"]["right"]
        by_name = dict(states[i])
        Dp = (max(L["dim"], L["vdim"]) + 15) // 16 * 16
        assert by_name["mix.left.kv"].kind == "paged" and by_name["mix.left.kv"].width == L["kv_heads"] * Dp
        assert by_name["mix.right.ssm"].shape == (R["heads"], R["vdim"], R["state"]) and by_name["mix.right.ssm"].dtype == "float32"
        assert by_name["mix.right.conv"].shape == (R["conv"] - 1, R["heads"] * R["vdim"] + 2 * R["groups"] * R["state"])
    assert spec.head_name is None and spec.head_multiplier == data["logit_scale"]


@pytest.mark.parametrize("which", ["A", "B", "C"])
def test_tensor_names_and_shapes_match_a_model_folder(which, tmp_path):
    d, cfg, weights = C.make_model_dir(which, str(tmp_path))
    arch, typed = open_model_dir(d)
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


def test_random_weights_mode_writes_a_loadable_folder(tmp_path):
    from poor_mans_mamba_b200.weights import write_random_model
    d = write_random_model(C.config("C"), seed=5, out_dir=str(tmp_path))
    arch, typed = open_model_dir(d)
    model = Model(arch.model_spec(typed))
    files = ModelFiles(d)
    try:
        assert check_tensors(model.param_specs(), model.ignored_names(), files, strict=True) == []
        w = {k: files.tensor(k).float() for k in files.keys()}
    finally:
        files.close()
    logits = P.forward(json.load(open(os.path.join(d, "config.json"))), w, [1, 2, 3, 4, 5])
    assert logits.shape == (5, 97) and bool(torch.isfinite(logits).all())


def test_plain_mechanisms_on_hand_made_cases():
    """The oracle's own pieces on cases small enough to do by hand."""
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 5.0]]], dtype=torch.float64)  # one token, one head, d = 5, 4 rotated
    pos = torch.tensor([3])
    out = P.rotate_halves(x, pos, 4, 100.0, 2.0)
    a0, a1 = 3 * 1.0 / 2.0, 3 * 100.0 ** (-0.5) / 2.0
    want = [1 * torch.cos(torch.tensor(a0)) - 3 * torch.sin(torch.tensor(a0)),
            2 * torch.cos(torch.tensor(a1)) - 4 * torch.sin(torch.tensor(a1)),
            3 * torch.cos(torch.tensor(a0)) + 1 * torch.sin(torch.tensor(a0)),
            4 * torch.cos(torch.tensor(a1)) + 2 * torch.sin(torch.tensor(a1)), 5.0]
    assert torch.allclose(out[0, 0], torch.tensor([float(v) for v in want], dtype=torch.float64))
    # a causal convolution's last column weighs the current token
    y = P.causal_conv(torch.tensor([[1.0], [10.0], [100.0]], dtype=torch.float64),
                      torch.tensor([[2.0, 3.0]], dtype=torch.float64), torch.tensor([0.5], dtype=torch.float64))
    assert y.view(-1).tolist() == [3.5, 32.5, 320.5]
    # the router's weights are a softmax over the chosen logits only
    w = {"r.router": torch.eye(3, dtype=torch.float64), "r.router.b": torch.zeros(3, dtype=torch.float64)}
    for e in range(3):
        w[f"r.e{e}.gate"] = torch.full((1, 3), 10.0, dtype=torch.float64)
        w[f"r.e{e}.up"] = torch.zeros(1, 3, dtype=torch.float64)
        w[f"r.e{e}.down"] = torch.full((3, 1), float(e + 1), dtype=torch.float64)
    h = torch.tensor([[3.0, 1.0, 2.0]], dtype=torch.float64)
    got = P.routed_experts(h, w, "r.", {"router": {"experts": 3, "top": 2}, "expert": {"ff": 1, "limit": 2.0}})
    p0 = 1.0 / (1.0 + torch.exp(torch.tensor(-1.0, dtype=torch.float64)))  # experts 0 and 2, logits 3 and 2
    act = 2.0 * torch.sigmoid(torch.tensor(1.702 * 2.0, dtype=torch.float64))  # gate clamped to 2, up 0 -> (0 + 1)
    assert torch.allclose(got[0], (p0 * 1.0 + (1 - p0) * 3.0) * act * torch.ones(3, dtype=torch.float64))
