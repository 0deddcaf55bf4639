"""The Sapatar configuration gate and spec builder (no GPU): what is read from where, what is refused."""
import copy
import json

import pytest
import torch

import tessweave_engine_b200 as tw
from tessweave_engine_b200.config import ConfigError, resolve, resolve_folder
from tessweave_engine_b200.models import Model
from tessweave_engine_b200.parts import FixedState, PagedKV, Runtime, SeveralNeeds
from tiny_sapatar import SAPATAR_CONFIGS, moe, wkv


def meta_model(cfg):
    typed, spec = resolve(cfg)
    return typed, spec, Model(spec, Runtime(torch.device("meta"), torch.float32), config=typed)


@pytest.mark.parametrize("name", list(SAPATAR_CONFIGS))
def test_tensor_names_and_schedule(name):
    cfg = SAPATAR_CONFIGS[name]
    typed, spec, model = meta_model(cfg)
    owners = [i for i, layer in enumerate(cfg["layers"]) if layer.get("weights_of") is None]
    assert len(spec.layers) == len(owners) and len(spec.schedule) == len(cfg["layers"])
    for i, (layer, entry) in enumerate(zip(cfg["layers"], spec.schedule)):
        assert spec.layers[entry.layer].prefix == f"l{layer.get('weights_of', i)}" and entry.cache_of is None
    names = set(model.weight_decls())
    assert {"embed", "final.norm", "head"} <= names
    for i in owners:
        layer = cfg["layers"][i]
        assert f"l{i}.norm1" in names and (f"l{i}.norm2" in names) == (layer["mlp"] is not None)
        assert (f"l{i}.hc1.mix" in names) == ("streams" in cfg)
        assert (f"l{i}.hc2.in" in names) == ("streams" in cfg and layer["mlp"] is not None)
        if layer["type"] == "parallel":
            assert {f"l{i}.mix.left.q.b", f"l{i}.mix.left.o", f"l{i}.mix.right.i.b", f"l{i}.mix.right.norm"} <= names
        if layer["type"] == "wkv":
            assert {f"l{i}.mix.mu.w", f"l{i}.mix.w1", f"l{i}.mix.w2", f"l{i}.mix.w0", f"l{i}.mix.u", f"l{i}.mix.r"} <= names
        if layer["mlp"] is not None:
            e = layer["mlp"]["router"]["experts"]
            assert f"l{i}.mlp.e{e - 1}.down" in names and f"l{i}.mlp.e{e}.down" not in names
            assert (f"l{i}.mlp.shared.sg" in names) == ("shared" in layer["mlp"])
    for i in set(range(len(cfg["layers"]))) - set(owners):
        assert not any(n.startswith(f"l{i}.") for n in names)


def test_cache_needs_of_every_mixer():
    _, _, model = meta_model(SAPATAR_CONFIGS["A"])
    needs = [n for n, _ in model.cache_needs()]
    assert needs[0] == FixedState(2 * 16 * 16 + 64)                         # wkv: S per head, then the row before
    assert needs[1] == SeveralNeeds((PagedKV(2, 16, 9, 32), FixedState(3 * (16 * 25 + 1))))
    assert needs[2] == FixedState(2 * 16 * 8)
    assert needs[3] == needs[1] and needs[4] == needs[0]                   # same tensors, a cache and state of their own
    assert model.cache_bytes_per_token(2) == 2 * 2 * 2 * (16 + 32)
    assert model.state_bytes_per_request() == 4 * sum(n.numel if isinstance(n, FixedState) else n.needs[1].numel for n in needs)


def test_decay_rank_comes_from_the_checkpoint(tmp_path):
    cfg = copy.deepcopy(SAPATAR_CONFIGS["B"])
    folder = tw.write_random_model(tmp_path / "m", cfg, seed=1)
    written = json.loads((folder / "config.json").read_text())
    del written["layers"][2]["mixer"]["decay_rank"]
    (folder / "config.json").write_text(json.dumps(written))
    typed, _ = resolve_folder(folder)
    assert typed.layers[2].mixer.decay_rank == 4
    with pytest.raises(ValueError):
        resolve(written)                                     # neither the key nor a checkpoint
    written["layers"][2]["mixer"]["decay_rank"] = 7
    (folder / "config.json").write_text(json.dumps(written))
    with pytest.raises(ConfigError):
        resolve_folder(folder)


def broken(change):
    cfg = copy.deepcopy(SAPATAR_CONFIGS["A"])
    change(cfg)
    return cfg


@pytest.mark.parametrize("change", [
    lambda c: c["layers"][0].update(type="conv"),
    lambda c: c["layers"][0]["mlp"].update(kind="dense"),
    lambda c: c["layers"][0]["mlp"]["router"].update(top=7),
    lambda c: c["layers"][1]["mixer"]["left"].update(kv_heads=3),
    lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=18),
    lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=7),
    lambda c: c["layers"][1]["mixer"]["right"].update(gate_cap=0.0),
    lambda c: c["layers"][2]["mixer"].update(decay=[0.9]),
    lambda c: c["layers"][3].update(weights_of=3),
    lambda c: c["layers"][3].update(mixer={**c["layers"][3]["mixer"], "left_scale": 0.71}),    # describes another layer than the one it names
    lambda c: c.update(streams=0),
    lambda c: c["norm"].update(eps=0.0),
    lambda c: c.pop("width"),
])
def test_the_gate_refuses(change):
    with pytest.raises(ConfigError):
        resolve(broken(change))


def test_too_many_copies_and_too_large_heads_are_refused_when_the_parts_are_built():
    with pytest.raises(ValueError):
        meta_model(broken(lambda c: c.update(streams=17)))
    big = {"architecture": "Sapatar", "vocab": 10, "width": 16, "norm": {"eps": 1e-5}, "layers": [wkv(1, 512, 4, mlp=moe(2, 1, 8))]}
    with pytest.raises(ValueError):
        meta_model(big)
