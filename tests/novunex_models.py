"""Tiny Novunex configurations for the tests, and their model folders with random weights."""
from __future__ import annotations

ARCH = "Novunex"


def _layer(kind, heads, kv_heads, dim, vdim, scale, base, dims, scaling=None, kv_from=None, mlp=None):
    rot = dict(base=base, dims=dims)
    if scaling:
        rot["scaling"] = scaling
    mixer = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, rot=rot)
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return dict(type=kind, mixer=mixer, mlp=mlp)


def _moe(experts, identity, top, ff, shared=None):
    m = dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, identity=identity, top=top))
    if shared is not None:
        m["shared"] = dict(ff=shared)
    return m


# wavelengths of base 1000 over 6 entries: 6.3, 63, 628 positions; with original 64 the three fall into the three ranges
SCALED = dict(factor=4.0, low=1.0, high=4.0, original=64)

CONFIGS = {
    # odd sizes all round, nothing a multiple of 8: values narrower AND wider than keys, one kv head, as many kv heads as
    # heads, a head that is not rotated at all, a layer without a feed-forward, a layer that reads another's keys and values,
    # mixtures with no identity expert, with one real expert, with every output chosen, with and without a shared expert
    "odd": dict(config=dict(architecture=ARCH, vocab=97, width=42, norm=dict(eps=1e-5), layers=[
        _layer("attention", 3, 1, 10, 7, 0.4, 1000.0, 6, mlp=_moe(3, 2, 2, 11, shared=13)),
        _layer("attention_2", 4, 2, 6, 9, 0.5, 1000.0, 6, scaling=SCALED),
        _layer("attention_2", 4, 2, 6, 9, 0.5, 1000.0, 6, scaling=SCALED, kv_from=1, mlp=_moe(5, 0, 1, 8)),
        _layer("attention", 2, 2, 12, 12, 0.3, 300.0, 0, mlp=_moe(1, 3, 4, 5, shared=6)),
    ]), seed=21, sigma=0.15),
    # sizes in multiples of 16 with heads of 64 and 128: the bfloat16 engine takes its tensor-core kernels where it has
    # them; 17 router outputs of which 4 are chosen; a kv_from layer right behind its source and one two layers on
    "even": dict(config=dict(architecture=ARCH, vocab=512, width=128, norm=dict(eps=1e-6), layers=[
        _layer("attention_2", 8, 2, 64, 32, 0.125, 10000.0, 64, scaling=dict(factor=6.0, low=1.0, high=3.0, original=256),
               mlp=_moe(16, 1, 4, 64, shared=96)),
        _layer("attention", 4, 1, 128, 64, 0.09, 40000.0, 48, mlp=_moe(4, 3, 3, 32, shared=64)),
        _layer("attention_2", 8, 2, 64, 32, 0.125, 10000.0, 64, scaling=dict(factor=6.0, low=1.0, high=3.0, original=256),
               kv_from=0, mlp=_moe(16, 1, 4, 64)),
        _layer("attention", 2, 2, 64, 128, 0.11, 5000.0, 64, mlp=_moe(2, 0, 2, 48, shared=32)),
    ]), seed=22, sigma=0.08, spaced_corrections=True),
}


ROUTER_SPREAD = 2.0


def make_model_dir(folder: str, name: str) -> str:
    from hymt2sharp_b200.config import NovunexConfig
    from hymt2sharp_b200.weights import write_random_model
    import os
    import torch
    from safetensors.torch import load_file, save_file
    spec = CONFIGS[name]
    write_random_model(folder, NovunexConfig.from_dict(spec["config"]), spec["seed"], spec["sigma"])
    # routers with a wide spread of outputs: a choice between two experts that rests on the last bits would make the
    # comparison of two precisions a comparison of two different sums
    path = os.path.join(folder, "model.safetensors")
    tensors = load_file(path)
    for k in tensors:
        if k.endswith(".mlp.router"):
            tensors[k] = (tensors[k].float() * ROUTER_SPREAD).to(tensors[k].dtype)
        if k.endswith(".mlp.correction") and spec.get("spaced_corrections"):
            # corrections a whole score apart, in a shuffled order: scores lie between 0 and 1, so the corrections alone decide
            # the choice and the bfloat16 engine chooses as the plain model does; the weights are still the tokens' own scores.
            # (The other model keeps random corrections, and with them a choice that differs from token to token.)
            n = tensors[k].shape[0]
            order = torch.randperm(n, generator=torch.Generator().manual_seed(n + spec["seed"]))
            tensors[k] = order.float().to(tensors[k].dtype)
    save_file(tensors, path)
    return folder
