"""Tiny Pemezen configurations for the tests, and their model folders with random weights."""
from __future__ import annotations

ARCH = "Pemezen"


def _latent(kind, heads, dim, rot_dim, vdim, rank, scale, base, dims=None, scaling=None, ff=None):
    rot = dict(base=base, dims=rot_dim if dims is None else dims)
    if scaling:
        rot["scaling"] = scaling
    return dict(type=kind, mixer=dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=rank, scale=scale, rot=rot),
                mlp=None if ff is None else dict(kind="dense", ff=ff))


def _rglru(width, blocks, conv, ff=None):
    return dict(type="rglru", mixer=dict(width=width, blocks=blocks, conv=conv), mlp=None if ff is None else dict(kind="dense", ff=ff))


YARN = dict(factor=4.0, original=16, fast=8.0, slow=1.0)

CONFIGS = {
    # odd sizes all round, nothing a multiple of 8: three norm groups, convolutions of 3 (layers) and 2 / 5 (recurrent
    # blocks) taps, a recurrent layer first, layers without a feed-forward, value width != key width, fewer rotated
    # entries than the rotated part is wide, one layer without frequency scaling, no soft cap
    "odd": dict(config=dict(architecture=ARCH, vocab=97, width=42, norm=dict(eps=1e-5, groups=3), canon=dict(taps=3),
                            embedding=dict(scale=1.7),
                            layers=[_rglru(35, 5, 2, ff=50),
                                    _latent("latent_attention", 3, 10, 6, 9, 21, 0.9, 1000.0, dims=4),
                                    _latent("latent_attention_2", 5, 7, 4, 13, 17, 1.3, 500.0, scaling=YARN, ff=61),
                                    _rglru(44, 1, 5)]),
                seed=11, sigma=0.12),
    # multiples of 8: the bfloat16 engine takes its tensor-core products here; 20 heads (more than one tile of rows),
    # one norm group, one head, a convolution of one tap, the soft cap
    "even": dict(config=dict(architecture=ARCH, vocab=512, width=128, norm=dict(eps=1e-6, groups=1), canon=dict(taps=1),
                             embedding=dict(scale=0.8), logit_softcap=9.0,
                             layers=[_latent("latent_attention_2", 20, 16, 8, 24, 40, 0.5, 10000.0, scaling=YARN, ff=192),
                                     _rglru(96, 3, 4, ff=160),
                                     _latent("latent_attention", 1, 32, 16, 16, 64, 0.4, 20000.0, ff=136)]),
                 seed=12, sigma=0.07),
}


def make_model_dir(folder: str, name: str) -> str:
    from hymt2sharp_b200.config import PemezenConfig
    from hymt2sharp_b200.weights import write_random_model
    spec = CONFIGS[name]
    write_random_model(folder, PemezenConfig.from_dict(spec["config"]), spec["seed"], spec["sigma"])
    return folder
