"""The gate on a Linurax config.json, the registry, the weight declarations and the random-weights writer (no GPU)."""
import copy
import json

import pytest
import torch

import plain_linurax as plain
from tiny_linurax import LINURAX_A, LINURAX_B, LINURAX_CONFIGS

import tessweave_engine_b200 as tw
from tessweave_engine_b200.config import ConfigError, LinuraxConfig, architecture_of, resolve
from tessweave_engine_b200.models.model import Model
from tessweave_engine_b200.parts import FixedState, PagedKV, Runtime


def test_registry_finds_the_design_by_its_own_key():
    assert architecture_of(LINURAX_A) == "Linurax"
    cfg, spec = resolve(LINURAX_A)
    assert isinstance(cfg, LinuraxConfig) and spec.architecture == "Linurax" and spec.tie_word_embeddings
    assert [layer.block.kind for layer in spec.layers] == ["output_norm"] * 4
    assert [layer.block.params["mixer"].kind for layer in spec.layers] == ["mingru", "sigmoid_attention", "sigmoid_attention", "mingru"]
    assert ["feed_forward" in layer.block.params for layer in spec.layers] == [True, True, False, False]


def test_every_size_and_constant_comes_from_the_file():
    cfg, spec = resolve(LINURAX_B)
    assert (cfg.vocab, cfg.width, cfg.embedding_scale, cfg.norm_eps) == (97, 40, 1.0, 1e-6)
    att = spec.layers[0].block.params["mixer"].params
    assert (att["n_heads"], att["n_kv_heads"], att["head_dim"], att["scale"], att["eps"]) == (3, 1, 24, 0.25, 1e-6)
    assert att["position"].params == {"theta": 50.0, "dims": 12}
    assert spec.layers[2].block.params["mixer"].params["position"].params["dims"] == 0
    assert spec.layers[1].block.params["mixer"].params == {"hidden": 40, "width": 56}
    assert spec.embedding.params["scale"] == 1.0 and spec.final_norm.params["eps"] == 1e-6


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][1].update(type="conv"), "not implemented"),
    (lambda c: c["layers"][1]["mlp"].update(kind="routed"), "not implemented"),
    (lambda c: c["layers"][1]["mixer"].update(vdim=8), "vdim must equal dim"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "multiple of kv_heads"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "dims must be even"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=18), "at most dim"),
    (lambda c: c["layers"][0]["mixer"].pop("width"), "lacks the key 'width'"),
    (lambda c: c.pop("embedding"), "lacks the key 'embedding'"),
    (lambda c: c["norm"].update(eps=0.0), "eps must be positive"),
    (lambda c: c.update(layers=[]), "non-empty list"),
    (lambda c: c.update(vocab=0), "positive integer"),
])
def test_gate_refuses_what_is_not_implemented(change, message):
    config = copy.deepcopy(LINURAX_A)
    change(config)
    with pytest.raises(ConfigError, match=message):
        resolve(config)


@pytest.mark.parametrize("name", sorted(LINURAX_CONFIGS))
def test_declared_tensors_and_cache_needs(name):
    config = LINURAX_CONFIGS[name]
    cfg, spec = resolve(config)
    model = Model(spec, Runtime(torch.device("meta"), torch.bfloat16), config=cfg)
    decls = model.weight_decls()
    want = {"embed": (config["vocab"], config["width"]), "final.norm": (config["width"],)}
    for i, layer in enumerate(config["layers"]):
        m, width = layer["mixer"], config["width"]
        want[f"l{i}.norm1"] = (width,)
        if layer["type"] == "attention":
            q, k = m["heads"] * m["dim"], m["kv_heads"] * m["dim"]
            want.update({f"l{i}.mix.q": (q, width), f"l{i}.mix.k": (k, width), f"l{i}.mix.q.norm": (q,),
                         f"l{i}.mix.k.norm": (k,), f"l{i}.mix.talk": (m["heads"], m["heads"]), f"l{i}.mix.pb": (m["heads"],),
                         f"l{i}.mix.g": (q, width), f"l{i}.mix.o": (width, q)})
        else:
            w = m["width"]
            want.update({f"l{i}.mix.z": (w, width), f"l{i}.mix.z.b": (w,), f"l{i}.mix.x": (w, width), f"l{i}.mix.x.b": (w,),
                         f"l{i}.mix.g": (w, width), f"l{i}.mix.o": (width, w)})
        if layer["mlp"]:
            ff = layer["mlp"]["ff"]
            want.update({f"l{i}.norm2": (width,), f"l{i}.mlp.gate": (ff, width), f"l{i}.mlp.up": (ff, width),
                         f"l{i}.mlp.down": (width, ff)})
    assert {k: tuple(d.shape) for k, d in decls.items()} == want
    needs = [need for need, _ in model.cache_needs()]
    for layer, need in zip(config["layers"], needs):
        if layer["type"] == "attention":
            assert need == PagedKV(layer["mixer"]["kv_heads"], layer["mixer"]["dim"], None)
        else:
            assert need == FixedState(layer["mixer"]["width"], torch.float32)
    assert model.state_bytes_per_request() == 4 * sum(l["mixer"]["width"] for l in config["layers"] if l["type"] == "mingru")


def test_random_model_folder_is_read_by_the_plain_implementation(tmp_path):
    folder = tw.write_random_model(tmp_path / "m", LINURAX_B, seed=3, std=0.2)
    config, weights = plain.read_folder(folder)
    assert config["architecture"] == "Linurax" and json.loads((folder / "config.json").read_text())["vocab"] == 97
    talk = weights["l0.mix.talk"]
    assert talk.shape == (3, 3) and float((talk - torch.eye(3)).abs().max()) < 1.5      # identity plus noise
    logits = plain.forward(config, weights, [1, 2, 3, 4])
    assert logits.shape == (4, 97) and torch.isfinite(logits).all()
    # a missing tensor is named
    from safetensors.torch import load_file, save_file
    t = load_file(str(folder / "model.safetensors"))
    del t["l1.mix.z.b"]
    save_file(t, str(folder / "model.safetensors"))
    from tessweave_engine_b200.weights.loader import fill_weights
    cfg, spec = resolve(LINURAX_B)
    model = Model(spec, Runtime(torch.device("cpu"), torch.float32), config=cfg)
    with pytest.raises(tw.WeightError, match="l1.mix.z.b"):
        fill_weights(model, folder)
