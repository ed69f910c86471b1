"""Baselix on the host: config.json to the model's description, tensor names, cache needs, errors."""
import copy
import json
import os

import pytest
import torch

import baselix_tiny as BT
from plain import baselix_plain as BP
from zedinfer_b200.cache import CacheManager
from zedinfer_b200.config.registry import ConfigError, load_model_config, resolve_architecture
from zedinfer_b200.engine.model import Model


def spec_of(raw):
    arch = resolve_architecture(raw)
    spec = arch.build_spec(arch.parse(raw))
    spec.validate()
    return spec


def test_the_architecture_is_found_by_its_name():
    assert resolve_architecture({"architecture": "Baselix"}).name == "Baselix"
    assert resolve_architecture({"architectures": ["Baselix"]}).name == "Baselix"
    assert resolve_architecture({"model_type": "baselix"}).name == "Baselix"
    assert resolve_architecture({"architectures": ["Qwen2ForCausalLM"]}).name == "Qwen2ForCausalLM"


def test_layers_schedule_and_shared_latents():
    spec = spec_of(BT.BX_A)
    assert [c.cache_of for c in spec.schedule] == [None, 0, None, 2]
    kinds = [(l.mixer.kind, l.ffn.kind if l.ffn else None) for l in spec.layers]
    assert kinds == [("latent_attention", "squared_relu_mlp"), ("latent_attention", "routed_experts"),
                     ("latent_attention", None), ("latent_attention", "squared_relu_mlp")]
    assert [l.mixer.params["own_latent"] for l in spec.layers] == [True, False, True, False]
    assert [l.mixer.params["window"] for l in spec.layers] == [24, 17, 11, 29]
    # the cache of an owner keeps what the widest window among its users needs
    assert [l.mixer.params["cache_window"] for l in spec.layers] == [24, 24, 29, 29]
    assert all(l.block_params == {"residual_scale": 0.5} for l in spec.layers)
    assert spec.head.params["softcap"] == 10.0 and spec_of(BT.BX_B).head.params["softcap"] is None
    model = Model(spec)
    needs = dict(model.cache_needs())
    assert sorted(needs) == [0, 2] and all(n.planes == 1 and n.n_kv_heads == 1 and n.head_dim == 32 for n in needs.values())
    assert needs[0].window == 24 and needs[2].window == 29
    assert model.capture_safe()


def test_tensor_names_and_shapes():
    names = Model(spec_of(BT.BX_A)).tensor_specs()
    required = {k for k, v in names.items() if not v.optional}
    want = {"embed": (300, 96), "pos": (512, 96), "final.norm": (96,), "l0.norm1": (96,), "l0.norm2": (96,),
            "l0.mix.q": (48, 96), "l0.mix.dkv": (32, 96), "l0.mix.dkv.norm": (32,), "l0.mix.uk": (48, 32),
            "l0.mix.uv": (72, 32), "l0.mix.sink": (3,), "l0.mix.o": (96, 72), "l0.mlp.up": (136, 96),
            "l0.mlp.down": (96, 136), "l1.mlp.router": (6, 96), "l1.mlp.router.b": (6,), "l1.mlp.e5.gate": (40, 96),
            "l1.mlp.e0.down": (96, 40), "l1.mlp.shared.up": (56, 96), "l1.mlp.shared.down": (96, 56),
            "l3.mix.uk": (48, 32), "l3.mix.o": (96, 16)}
    for k, shape in want.items():
        assert tuple(names[k].shape) == shape, k
    assert "l1.mix.dkv" not in names and "l1.mix.dkv.norm" not in names and "l3.mix.dkv" not in names
    assert not any(k.startswith("l2.mlp.") or k == "l2.norm2" for k in names)
    assert not any(k.startswith("l0.mlp.shared") for k in names)
    assert len([k for k in required if k.startswith("l1.mlp.e")]) == 18
    assert not any(k.startswith("l0.mlp.e") for k in Model(spec_of(BT.BX_B)).tensor_specs() if "shared" in k)


def test_one_plane_groups_in_the_cache_manager():
    model = Model(spec_of(BT.BX_A))
    cache = CacheManager(model.cache_needs(), 8, max_requests=4)
    assert [(g.planes, g.head_dim, g.window, len(g.calls)) for g in cache.groups] == [(1, 32, 24, 1), (1, 32, 29, 1)]
    assert cache.groups[0].page_elems(8) == 8 * 32
    cache.set_num_pages(10)
    v = cache.view_for_call(0)
    assert v.kind == "paged" and v.kv_stride == 0 and v.page_stride == 8 * 32 and v.window == 24
    # two-plane and one-plane needs of the same shape do not share a group
    from zedinfer_b200.cache.manager import PagedKVNeed
    both = CacheManager([(0, PagedKVNeed(1, 32, None)), (1, PagedKVNeed(1, 32, None, planes=1))], 8)
    assert len(both.groups) == 2 and both.groups[0].page_elems(8) == 2 * both.groups[1].page_elems(8)
    with pytest.raises(ValueError, match="planes"):
        CacheManager([(0, PagedKVNeed(1, 32, None, planes=3))], 8)


@pytest.mark.parametrize("edit,match", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_from", 1), "earlier layer"),
    (lambda c: c["layers"][3]["mixer"].__setitem__("kv_from", 1), "no latent of its own"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_rank", 64), "kv_rank"),
    (lambda c: c["layers"][0].__setitem__("type", "recurrent"), "not a mixer"),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 7), "exceeds"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "gated"), "dense"),
    (lambda c: c["norm"].__setitem__("eps", 0), "eps"),
    (lambda c: c.__setitem__("logit_softcap", -1.0), "logit_softcap"),
    (lambda c: c["layers"][0]["mixer"]["mask"].__setitem__("size", 0), "size"),
])
def test_config_errors_name_the_key(edit, match):
    raw = copy.deepcopy(BT.BX_A)
    edit(raw)
    with pytest.raises(ConfigError, match=match):
        spec_of(raw)


def test_keys_nobody_knows_are_ignored_and_defaults():
    raw = copy.deepcopy(BT.BX_B)
    raw["torch_dtype"] = "bfloat16"
    raw.pop("residual_mult")
    spec = spec_of(raw)
    assert spec.layers[0].block_params == {"residual_scale": 1.0}
    m = copy.deepcopy(BT.BX_B)
    m["layers"][0]["mixer"].pop("scale")
    assert spec_of(m).layers[0].mixer.params["scale"] == 32 ** -0.5


def test_a_written_folder_loads_and_the_plain_reader_sees_the_same_tensors(tmp_path):
    out = BT.make_model_dir(tmp_path, "A")
    arch, cfg, spec = load_model_config(out)
    assert arch.name == "Baselix" and cfg.residual_mult == 0.5 and len(cfg.layers) == 4
    pcfg, w = BP.read_model(out, torch.float32)
    need = {k for k, v in Model(spec).tensor_specs().items() if not v.optional}
    assert set(w) == need and pcfg["layers"][1]["mlp"]["router"]["top"] == 2
    assert float(w["l0.norm1"].abs().max()) < 0.5 and abs(float(w["l0.mix.dkv.norm"].mean()) - 1.0) < 0.2


def test_the_plain_functions_on_cases_done_by_hand():
    # softmax with a sink and a window: one key, score 0, sink 0 -> half of the value
    q = torch.zeros(1, 1, 2, dtype=torch.float64)
    k = torch.ones(1, 1, 2, dtype=torch.float64)
    v = torch.tensor([[[4.0, 8.0]]], dtype=torch.float64)
    out = BP.windowed_sink_attention(q, k, v, torch.zeros(1, dtype=torch.float64), 1.0, None)
    assert torch.allclose(out, torch.tensor([[[2.0, 4.0]]], dtype=torch.float64))
    # window 2: the third query does not see the first key
    q = torch.zeros(3, 1, 1, dtype=torch.float64)
    v = torch.tensor([[[1.0]], [[10.0]], [[100.0]]], dtype=torch.float64)
    out = BP.windowed_sink_attention(q, torch.zeros(3, 1, 1, dtype=torch.float64), v,
                                     torch.full((1,), -1e9, dtype=torch.float64), 1.0, 2)
    assert torch.allclose(out.flatten(), torch.tensor([1.0, 5.5, 55.0], dtype=torch.float64))
    # the expert's activation at its clamps
    one = torch.ones(1, 1, dtype=torch.float64)
    y = BP.clamped_expert(torch.tensor([[10.0]], dtype=torch.float64), one, -one, one, 2.0)
    g = 2.0
    assert torch.allclose(y, torch.tensor([[g / (1 + torch.exp(torch.tensor(-1.702 * g))) * (-2.0 + 1.0)]], dtype=torch.float64))
    idx, wts = BP.route(torch.tensor([[1.0]], dtype=torch.float64), torch.tensor([[0.0], [2.0], [1.0]], dtype=torch.float64),
                        torch.tensor([0.5, 0.0, 0.0], dtype=torch.float64), 2)
    assert idx.tolist() == [[1, 2]] and torch.allclose(wts, torch.softmax(torch.tensor([[2.0, 1.0]], dtype=torch.float64), -1))
    assert torch.allclose(BP.capped_logits(torch.tensor([[100.0]], dtype=torch.float64), one, 5.0), torch.tensor([[5.0]], dtype=torch.float64))
