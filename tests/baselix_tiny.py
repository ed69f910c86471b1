"""Tiny Baselix configurations for the tests.  They differ in every size and option: head counts, query/key and
value sizes that differ from each other, latent ranks (32: the general attention kernel; 64 and 128: the tensor-core
kernels; 320: beyond 256), windows that are no multiple of a page, a borrower whose window is wider than its owner's,
layers without a feed-forward, routed layers with and without a shared expert, top 1 and top = experts, a residual
factor of 1 and others, with and without a logit cap, and one (E) whose sizes fit no vector width."""
import os


def _mixer(heads, dim, vdim, rank, window, scale, kv_from=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "mask": {"size": window}, "scale": scale}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _layer(mixer, mlp):
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


def _moe(ff, limit, experts, top, shared=None):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}, "shared": shared}


BX_A = {
    "architecture": "Baselix", "vocab": 300, "width": 96, "max_positions": 512, "norm": {"eps": 1e-6},
    "residual_mult": 0.5, "logit_softcap": 10.0,
    "layers": [
        _layer(_mixer(3, 16, 24, 32, 24, 0.3), {"kind": "dense", "ff": 136}),
        _layer(_mixer(3, 16, 24, 32, 17, 0.3, kv_from=0), _moe(40, 1.5, 6, 2, {"ff": 56, "limit": 0.75})),
        _layer(_mixer(2, 24, 8, 32, 11, 0.2), None),
        _layer(_mixer(2, 24, 8, 32, 29, 0.2, kv_from=2), {"kind": "dense", "ff": 72}),   # wider window than its owner's
    ],
}
BX_B = {
    "architecture": "Baselix", "vocab": 777, "width": 128, "max_positions": 600, "norm": {"eps": 1e-5},
    "residual_mult": 1.0,
    "layers": [
        _layer(_mixer(4, 32, 16, 64, 40, 0.17), _moe(48, 3.0, 5, 1)),
        _layer(_mixer(4, 32, 16, 64, 9, 0.17, kv_from=0), {"kind": "dense", "ff": 200}),
        _layer(_mixer(4, 32, 16, 64, 40, 0.17, kv_from=0), None),
    ],
}
BX_C = {
    "architecture": "Baselix", "vocab": 411, "width": 64, "max_positions": 700, "norm": {"eps": 1e-4},
    "residual_mult": 0.8, "logit_softcap": 4.0,
    "layers": [
        _layer(_mixer(2, 64, 32, 128, 70, 0.1), _moe(24, 0.5, 3, 3, {"ff": 16, "limit": 2.5})),
        _layer(_mixer(5, 16, 16, 128, 33, 0.25), {"kind": "dense", "ff": 96}),
    ],
}
BX_D = {
    "architecture": "Baselix", "vocab": 150, "width": 80, "max_positions": 256, "norm": {"eps": 1e-5},
    "residual_mult": 0.25, "logit_softcap": 50.0,
    "layers": [
        _layer(_mixer(1, 40, 48, 320, 19, 0.15), {"kind": "dense", "ff": 88}),
        _layer(_mixer(1, 40, 48, 320, 19, 0.15, kv_from=0), _moe(32, 1.0, 4, 2, {"ff": 24, "limit": 1.0})),
    ],
}
# sizes that fit no vector width: a width that is no multiple of 8, 5 heads of 12, values of 20, rank 40, 7 experts
BX_E = {
    "architecture": "Baselix", "vocab": 203, "width": 100, "max_positions": 300, "norm": {"eps": 1e-5},
    "residual_mult": 0.6, "logit_softcap": 8.0,
    "layers": [
        _layer(_mixer(5, 12, 20, 40, 13, 0.3), _moe(36, 1.2, 7, 3, {"ff": 52, "limit": 0.9})),
        _layer(_mixer(5, 12, 20, 40, 26, 0.3, kv_from=0), {"kind": "dense", "ff": 90}),
        _layer(_mixer(3, 20, 12, 24, 8, 0.25), _moe(44, 2.0, 2, 1)),
    ],
}
CONFIGS = {"A": (BX_A, 21), "B": (BX_B, 22), "C": (BX_C, 23), "D": (BX_D, 24), "E": (BX_E, 25)}
INIT_SCALE = 5.0


def make_model_dir(tmp_root, name, dtype="bfloat16"):
    """Write the folder with the framework's random-weights writer."""
    from zedinfer_b200.weights import write_random_model
    cfg, seed = CONFIGS[name]
    out = os.path.join(str(tmp_root), f"baselix_{name}_{dtype}")
    if not os.path.isfile(os.path.join(out, "model.safetensors")):
        write_random_model(cfg, seed, out, dtype=dtype, init_scale=INIT_SCALE)
    return out
