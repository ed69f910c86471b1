"""Tiny Gibalorn configurations for the tests.  They differ in every size and option: the three mixers in several
orders, head counts and head sizes (query/key and value sizes that differ, one head, as many key/value heads as query
heads), rotated spans that cover a whole head and only part of one, latent ranks whose cache row (rank + rotated part)
is 64 or 128 (the tensor-core attention kernels), another multiple of 8 (the general kernel) or none at all (padded),
state sizes dealt to 1, 4 and 8 lanes, convolutions of 1 to 4 taps, one and several groups of B/C and of the norm,
routers that choose one, some or all experts, layers without a feed-forward, and run orders without a loop, with a loop
in the middle, at the start, over everything, and with ``times`` 1."""
import copy
import os


def _attn(heads, kv, dim, rot, base, scale):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": scale,
                                           "rot": {"base": base, "dims": rot}}}


def _latent(heads, dim, rot_dim, vdim, rank, q_rank, base, scale, rot=None):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank,
                                                  "q_rank": q_rank, "scale": scale,
                                                  "rot": {"base": base, "dims": rot_dim if rot is None else rot}}}


def _mamba(heads, vdim, state, groups, conv, norm_groups):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                                        "norm_groups": norm_groups}}


def _moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def _with(layer, mlp):
    out = dict(layer)
    out["mlp"] = mlp
    return out


# latent row 24 + 8 = 32 (the general attention kernel); a loop in the middle; a layer without a feed-forward
GB_A = {
    "architecture": "Gibalorn", "vocab": 300, "width": 96, "norm": {"eps": 1e-5},
    "layers": [
        _with(_latent(3, 16, 8, 24, 24, 40, 10000.0, 0.2), _moe(5, 2, 40)),
        _with(_mamba(6, 8, 16, 2, 4, 3), None),
        _with(_attn(4, 2, 32, 16, 5000.0, 0.2), _moe(4, 4, 24)),
        _with(_mamba(2, 24, 40, 1, 2, 1), _moe(3, 1, 56)),
    ],
    "loop": {"start": 1, "stop": 3, "times": 2},
}
# the tensor-core attention kernels: head size 64 with as many key/value heads as query heads and the whole head turned,
# latent rows of 48 + 16 = 64 and 112 + 16 = 128; no loop
GB_B = {
    "architecture": "Gibalorn", "vocab": 777, "width": 128, "norm": {"eps": 1e-6},
    "layers": [
        _with(_attn(2, 2, 64, 64, 1000.0, 0.11), _moe(6, 2, 48)),
        _with(_latent(4, 32, 16, 16, 48, 24, 20000.0, 0.15), None),
        _with(_mamba(8, 16, 64, 1, 3, 2), _moe(2, 2, 72)),
        _with(_latent(2, 48, 16, 40, 112, 64, 300.0, 0.12), _moe(7, 3, 32)),
    ],
    "loop": None,
}
# sizes that fit no vector width: a latent row of 20 + 6 = 26 (padded to 32) of which 4 entries turn, one head, a state
# of 8 on one lane, a convolution of one tap (no history), 7 experts; the loop covers everything, three times
GB_C = {
    "architecture": "Gibalorn", "vocab": 203, "width": 72, "norm": {"eps": 1e-4},
    "layers": [
        _with(_mamba(3, 12, 8, 3, 1, 1), _moe(7, 3, 20)),
        _with(_latent(1, 24, 6, 12, 20, 16, 777.0, 0.25, rot=4), _moe(2, 1, 36)),
        _with(_attn(3, 1, 16, 8, 100.0, 0.3), None),
    ],
    "loop": {"start": 0, "stop": 3, "times": 3},
}
# a loop at the start that runs once (so nothing is added again), a state of 136 on 16 lanes, several groups
GB_D = {
    "architecture": "Gibalorn", "vocab": 150, "width": 64, "norm": {"eps": 1e-5},
    "layers": [
        _with(_mamba(4, 20, 136, 2, 4, 4), _moe(4, 2, 24)),
        _with(_attn(6, 3, 16, 16, 40000.0, 0.25), _moe(3, 2, 40)),
    ],
    "loop": {"start": 0, "stop": 1, "times": 1},
}
def all_chosen(cfg):
    """The same model with every router choosing all of its experts: nothing discrete is left, so bfloat16 can be compared
    position by position (with a choice among experts, rounding turns a close call now and then, and what a turned choice
    changes reaches every later token through keys, values and states)."""
    out = copy.deepcopy(cfg)
    for layer in out["layers"]:
        if layer["mlp"] is not None:
            layer["mlp"]["router"]["top"] = layer["mlp"]["router"]["experts"]
    return out


# state-space layers alone (no paged cache at all), run twice; and a model of attention alone with a head size of 24
GB_E = {
    "architecture": "Gibalorn", "vocab": 120, "width": 48, "norm": {"eps": 1e-5},
    "layers": [_with(_mamba(2, 16, 24, 2, 3, 2), _moe(3, 2, 32)), _with(_mamba(5, 4, 12, 1, 2, 1), None)],
    "loop": {"start": 0, "stop": 2, "times": 2},
}
GB_F = {
    "architecture": "Gibalorn", "vocab": 99, "width": 40, "norm": {"eps": 1e-6},
    "layers": [_with(_attn(2, 1, 24, 12, 64.0, 0.2), _moe(2, 1, 16)), _with(_latent(2, 8, 4, 8, 536, 8, 99.0, 0.3), None)],
    "loop": None,
}
CONFIGS = {"A": (GB_A, 31), "B": (GB_B, 32), "C": (GB_C, 33), "D": (GB_D, 34), "E": (GB_E, 35), "F": (GB_F, 36)}
CONFIGS.update({name + "x": (all_chosen(cfg), seed) for name, (cfg, seed) in list(CONFIGS.items())})
INIT_SCALE = 5.0


def make_model_dir(tmp_root, name, dtype="bfloat16"):
    """Write the folder with the framework's random-weights writer."""
    from zedinfer_b200.weights import write_random_model
    cfg, seed = CONFIGS[name]
    out = os.path.join(str(tmp_root), f"gibalorn_{name}_{dtype}")
    if not os.path.isfile(os.path.join(out, "model.safetensors")):
        write_random_model(cfg, seed, out, dtype=dtype, init_scale=INIT_SCALE, name_prefix="")
    return out
