"""Gibalorn on the host: config.json to the model's description, run order, tensor names, cache needs, errors; the plain
implementation's own mechanisms against each other."""
import copy
import os

import pytest
import torch

import gibalorn_tiny as GT
from plain import gibalorn_plain as GP
from zedinfer_b200.cache import CacheManager, StateNeed
from zedinfer_b200.cache.manager import PagedKVNeed
from zedinfer_b200.config.registry import ConfigError, resolve_architecture
from zedinfer_b200.engine.model import Model


def spec_of(raw):
    arch = resolve_architecture(raw)
    spec = arch.build_spec(arch.parse(raw))
    spec.validate()
    return spec


def test_the_architecture_is_found_by_its_name():
    assert resolve_architecture({"architecture": "Gibalorn"}).name == "Gibalorn"
    assert resolve_architecture({"model_type": "gibalorn"}).name == "Gibalorn"
    assert "ssm" in resolve_architecture({"architecture": "Gibalorn"}).kernel_libraries


def test_layers_parts_and_run_order():
    spec = spec_of(GT.GB_A)
    kinds = [(l.mixer.kind, l.ffn.kind if l.ffn else None) for l in spec.layers]
    assert kinds == [("latent_attention", "routed_experts"), ("mamba2", None), ("attention", "routed_experts"),
                     ("mamba2", "routed_experts")]
    assert [(c.layer, c.add_embedding) for c in spec.schedule] == [(0, False), (1, False), (2, False), (1, True), (2, False), (3, False)]
    attn = spec.layers[2].mixer.params
    assert attn["value_from_key"] and attn["unit_sink"] and attn["scale"] == 0.2 and not attn["qkv_bias"]
    assert attn["position"].kind == "rope_span" and attn["position"].params["dims"] == 16 and not attn["position"].params["interleaved"]
    lat = spec.layers[0].mixer.params
    assert lat["rot_interleaved"] and lat["out_gate"] and lat["q_rank"] == 40 and lat["rot_dim"] == 8 and not lat["sinks"] and lat["window"] is None
    ffn = spec.layers[0].ffn.params
    assert (ffn["score"], ffn["weight_on"], ffn["activation"], ffn["router_bias"]) == ("sigmoid", "input", "relu2", False)
    assert not spec.tie_word_embeddings and spec.head_name == "head"
    for raw in (GT.GB_B, GT.GB_C, GT.GB_D):
        assert [c.layer for c in spec_of(raw).schedule] == GP.run_order(raw)


def test_caches_and_states_of_every_pass():
    model = Model(spec_of(GT.GB_A))
    needs = dict(model.cache_needs())
    assert sorted(needs) == [0, 1, 2, 3, 4, 5]
    assert needs[0] == PagedKVNeed(1, 32, None, planes=1)                       # latent 24 + turned part 8
    assert needs[2] == needs[4] == PagedKVNeed(2, 32, None, planes=2)           # turned keys, plain keys as values
    inner, channels = 6 * 8, 6 * 8 + 2 * 2 * 16
    assert needs[1] == needs[3] == StateNeed((inner * 16 + 3 * channels,), torch.float32)
    assert needs[5] == StateNeed((2 * 24 * 40 + 1 * (48 + 80),), torch.float32)
    assert model.capture_safe()
    cache = CacheManager(list(needs.items()), 4, max_requests=3)
    assert len(cache.groups) == 2 and cache.slots.num_slots == 3
    # a latent row that is no multiple of 8 is padded: 20 + 6 -> 32
    assert dict(Model(spec_of(GT.GB_C)).cache_needs())[1] == PagedKVNeed(1, 32, None, planes=1)


def test_tensor_names_and_shapes():
    names = Model(spec_of(GT.GB_A)).tensor_specs()
    want = {"embed": (300, 96), "head": (300, 96), "final.norm": (96,), "l0.norm1": (96,), "l0.norm2": (96,),
            "l0.mix.dq": (40, 96), "l0.mix.dq.norm": (40,), "l0.mix.uq": (72, 40), "l0.mix.dkv": (32, 96), "l0.mix.dkv.norm": (24,),
            "l0.mix.uk": (48, 24), "l0.mix.uv": (72, 24), "l0.mix.g": (72, 96), "l0.mix.o": (96, 72),
            "l0.mlp.router": (5, 96), "l0.mlp.e4.up": (40, 96), "l0.mlp.e0.down": (96, 40),
            "l1.mix.in": (2 * 48 + 2 * 32 + 6, 96), "l1.mix.conv": (112, 4), "l1.mix.conv.b": (112,), "l1.mix.dt_bias": (6,),
            "l1.mix.A_log": (6,), "l1.mix.D": (6,), "l1.mix.norm": (48,), "l1.mix.o": (96, 48),
            "l2.mix.q": (128, 96), "l2.mix.k": (64, 96), "l2.mix.o": (96, 128)}
    for k, shape in want.items():
        assert tuple(names[k].shape) == shape, k
    for absent in ("l1.norm2", "l1.mlp.router", "l2.mix.v", "l0.mix.q", "l0.mix.sink", "l0.mlp.router.b", "l0.mlp.e0.gate", "pos"):
        assert absent not in names, absent


@pytest.mark.parametrize("edit,word", [
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][2]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][2]["mixer"].update(vdim=16), "vdim"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=34), "dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10), "dims"),
    (lambda c: c["layers"][1]["mixer"].update(groups=4), "groups"),
    (lambda c: c["layers"][1]["mixer"].update(norm_groups=5), "norm_groups"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=6), "top"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "kind"),
    (lambda c: c["loop"].update(stop=9), "stop"),
    (lambda c: c["loop"].update(start=3, stop=1), "stop"),
    (lambda c: c["loop"].update(times=0), "times"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c["layers"][0]["mixer"].pop("q_rank"), "q_rank"),
])
def test_a_config_that_cannot_be_used_names_the_key(edit, word):
    raw = copy.deepcopy(GT.GB_A)
    edit(raw)
    with pytest.raises(ConfigError, match=word):
        spec_of(raw)


def test_a_written_folder_reads_back_and_the_plain_implementation_runs_it(tmp_path):
    folder = GT.make_model_dir(tmp_path, "C")
    cfg, w = GP.read_model(folder)
    assert {k: v for k, v in cfg.items() if k != "torch_dtype"} == GT.GB_C and set(w) == set(Model(spec_of(GT.GB_C)).tensor_specs())
    logits, layers = [], []
    out = GP.forward(cfg, w, [3, 1, 4, 1, 5, 9, 2, 6], layers)
    assert out.shape == (8, 203) and len(layers) == 9 and bool(torch.isfinite(out).all())
    # causal: a prefix gives the same logits
    assert torch.allclose(GP.forward(cfg, w, [3, 1, 4, 1, 5])[:5], out[:5], atol=1e-12)


def test_plain_mechanisms_agree_with_each_other():
    """The two pairings are one rotation up to a permutation of the entries; a turn by p and then by q is a turn by p + q;
    the convolution's last column meets the current token; the recurrence with a step size of zero keeps its state."""
    g = torch.Generator().manual_seed(0)
    v = torch.randn(5, 2, 12, generator=g, dtype=torch.float64)
    pos = torch.tensor([0, 1, 7, 100, 1000])
    half = GP.rotate(v, pos, 100.0, 8, "half")
    perm = [0, 4, 1, 5, 2, 6, 3, 7]                              # interleaved entry 2i is half's i, 2i + 1 its i + 4
    inter = GP.rotate(v[..., perm + [8, 9, 10, 11]].contiguous(), pos, 100.0, 8, "interleaved")
    assert torch.allclose(inter[..., :8], half[..., perm]) and torch.equal(inter[..., 8:], v[..., 8:]) and torch.equal(half[..., 8:], v[..., 8:])
    assert torch.allclose(GP.rotate(GP.rotate(v, pos, 100.0, 8, "half"), pos + 3, 100.0, 8, "half"), GP.rotate(v, 2 * pos + 3, 100.0, 8, "half"))
    assert torch.equal(GP.rotate(v, torch.zeros(5, dtype=torch.long), 100.0, 12, "interleaved"), v)
    u = torch.randn(6, 3, generator=g, dtype=torch.float64)
    kernel = torch.tensor([[0.0, 0.0, 1.0]] * 3, dtype=torch.float64)
    assert torch.allclose(GP.causal_conv(u, kernel, torch.zeros(3, dtype=torch.float64)), u)
    kernel = torch.tensor([[1.0, 0.0, 0.0]] * 3, dtype=torch.float64)
    assert torch.allclose(GP.causal_conv(u, kernel, torch.ones(3, dtype=torch.float64))[2:], u[:-2] + 1) \
        and torch.allclose(GP.causal_conv(u, kernel, torch.ones(3, dtype=torch.float64))[:2], torch.ones(2, 3, dtype=torch.float64))
    w = GP.causal_weights(torch.zeros(1, 4, 4, dtype=torch.float64), sink_one=True)[0]
    assert torch.allclose(w[3], torch.full((4,), 0.2, dtype=torch.float64)) and torch.allclose(w[0], torch.tensor([0.5, 0, 0, 0], dtype=torch.float64))
    idx, wts = GP.route(torch.zeros(2, 4, dtype=torch.float64), torch.ones(5, 4, dtype=torch.float64), 2)
    assert idx.tolist() == [[0, 1], [0, 1]] and bool((wts == 0.5).all())
    # a router's margin: how far the last chosen logit lies above the first one left out
    h = torch.tensor([[1.0, 0.0], [0.0, 1.0]], dtype=torch.float64)
    wr = torch.tensor([[3.0, 0.0], [1.0, 5.0], [2.5, 4.0]], dtype=torch.float64)
    assert GP.route_margin(h, wr, 1).tolist() == [0.5, 1.0] and GP.route_margin(h, wr, 2).tolist() == [1.5, 4.0]
    assert bool(torch.isinf(GP.route_margin(h, wr, 3)).all())
