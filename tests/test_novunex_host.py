"""The Novunex design without a GPU: its configuration, the registry, the tensor list and memory plan, the frequency
table, and the plain implementation's mechanisms against values worked out by hand."""
import copy
import math

import numpy as np
import pytest
import torch

import novunex_models
from plain import novunex_plain as plain


def _cfg(name="odd"):
    return copy.deepcopy(novunex_models.CONFIGS[name]["config"])


def test_configuration_reads_every_size_and_round_trips():
    from hymt2sharp_b200.config import NovunexConfig
    cfg = NovunexConfig.from_dict(_cfg())
    assert (cfg.vocab, cfg.width, cfg.norm_eps, len(cfg.layers)) == (97, 42, 1e-5, 4)
    l0, l1, l2, l3 = cfg.layers
    assert (l0.type, l0.mixer.heads, l0.mixer.kv_heads, l0.mixer.dim, l0.mixer.vdim, l0.mixer.scale) == ("attention", 3, 1, 10, 7, 0.4)
    assert l0.mixer.rot.dims == 6 and l0.mixer.rot.scaling is None and l1.mixer.rot.scaling["original"] == 64
    assert (l0.mlp.experts, l0.mlp.identity, l0.mlp.top, l0.mlp.ff, l0.mlp.shared_ff) == (3, 2, 2, 11, 13)
    assert l1.mlp is None and l2.mixer.kv_from == 1 and l2.mlp.shared_ff is None and l2.mlp.identity == 0
    assert l3.mixer.rot.dims == 0
    assert NovunexConfig.from_dict(cfg.to_dict()) == cfg


@pytest.mark.parametrize("edit, key", [
    (lambda c: c["layers"][0].update(type="attention_3"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("vdim"), "mixer.vdim"),
    (lambda c: c["layers"][0]["mixer"].update(heads=4, kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=5), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=12), "rot.dims"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=0), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=2), "kv_from"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=6), "top"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "mlp.kind"),
    (lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].pop("low"), "low"),
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
])
def test_configuration_errors_name_the_key(edit, key):
    from hymt2sharp_b200.config import ConfigError, NovunexConfig
    c = _cfg()
    edit(c)
    with pytest.raises(ConfigError, match=key.replace(".", r"\.")):
        NovunexConfig.from_dict(c)


def test_registry_tensor_list_and_memory_plan():
    from hymt2sharp_b200.config.registry import get_architecture, known_architectures
    from hymt2sharp_b200.engine.model import DecoderModel
    assert "Novunex" in known_architectures()
    arch = get_architecture("Novunex")
    cfg = arch.config_class.from_dict(_cfg())
    model = DecoderModel(arch.build_spec(cfg))
    t = {k: tuple(v.shape) for k, v in model.tensors().items()}
    assert t["embed"] == (97, 42) and t["head"] == (97, 42) and t["final.norm"] == (42,)
    assert t["l0.mix.q"] == (30, 42) and t["l0.mix.k"] == (10, 42) and t["l0.mix.v"] == (7, 42) and t["l0.mix.o"] == (42, 21)
    assert t["l0.mix.q.norm"] == (10,) and t["l0.mix.k.norm"] == (10,)           # per head: one gain for all heads
    assert t["l1.mix.q.norm"] == (24,) and t["l1.mix.k.norm"] == (12,)           # over the whole projection
    assert "l2.mix.k" not in t and "l2.mix.v" not in t and "l2.mix.k.norm" not in t and t["l2.mix.q.norm"] == (24,)
    assert t["l0.mlp.router"] == (5, 42) and t["l0.mlp.correction"] == (5,) and t["l0.mlp.e2.up"] == (11, 42)
    assert "l0.mlp.e3.up" not in t and t["l0.mlp.shared.down"] == (42, 13) and "l2.mlp.shared.up" not in t
    assert not any(k.startswith("l1.mlp") or k == "l1.norm2" for k in t) and t["l1.norm1"] == (42,)
    # layer 2 reads layer 1's plane; keys and values of different widths get storage of their own
    keys = [(g.kv_heads, g.head_dim, g.value_width, g.planes) for g in model.groups]
    assert keys == [(1, 10, 7, 1), (2, 6, 9, 1), (2, 12, 12, 1)]
    slots = [(r[0].group, r[0].plane, r[0].writes) for r in model.slots]
    assert slots == [(0, 0, True), (1, 0, True), (1, 0, False), (2, 0, True)]
    assert model.state_bytes == 0 and model.graph_safe


def test_frequency_table_in_the_three_ranges():
    from hymt2sharp_b200.parts.rope import WavelengthScaledRotary
    s = dict(factor=4.0, low=1.0, high=4.0, original=64)
    f = [1000.0 ** (-2 * i / 6) for i in range(3)]          # wavelengths 6.28, 62.8, 628
    got = WavelengthScaledRotary(6, 1000.0, s)._host
    mid = (64 / (2 * math.pi / f[1]) - 1.0) / 3.0
    want = [f[0], (1 - mid) * f[1] / 4 + mid * f[1], f[2] / 4]
    assert np.allclose(got, want, rtol=1e-6) and 0.0 < mid < 1.0
    assert np.allclose(plain.rotary_frequencies(6, 1000.0, s).numpy(), want, rtol=1e-12)
    assert np.allclose(WavelengthScaledRotary(6, 1000.0, None)._host, f, rtol=1e-6)
    assert WavelengthScaledRotary(0, 10.0)._host.shape == (0,)


def test_plain_rotation_pairs_and_leaves_the_rest():
    v = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 5.0]]], dtype=torch.float64)        # dims 4: pairs (0, 2) and (1, 3); entry 4 stays
    f = torch.tensor([0.5, 0.25], dtype=torch.float64)
    out = plain.rotate(v, torch.tensor([2]), f)[0, 0]
    a, b = 1.0, 0.5
    want = [1 * math.cos(a) - 3 * math.sin(a), 2 * math.cos(b) - 4 * math.sin(b), 3 * math.cos(a) + 1 * math.sin(a),
            4 * math.cos(b) + 2 * math.sin(b), 5.0]
    assert torch.allclose(out, torch.tensor(want, dtype=torch.float64))


def test_plain_softmax_with_and_without_a_sink():
    q = torch.zeros(2, 1, 2, dtype=torch.float64)
    k = torch.zeros(2, 1, 2, dtype=torch.float64)
    v = torch.tensor([[[1.0]], [[3.0]]], dtype=torch.float64)
    # all scores 0: without a sink the mean of the visible values; with it the sink takes one share of the weight
    assert torch.allclose(plain.causal_attention(q, k, v, 1.0, sink=False)[:, 0, 0], torch.tensor([1.0, 2.0], dtype=torch.float64))
    assert torch.allclose(plain.causal_attention(q, k, v, 1.0, sink=True)[:, 0, 0], torch.tensor([0.5, 4.0 / 3.0], dtype=torch.float64))


def test_plain_router_chooses_with_the_correction_and_weighs_without():
    h = torch.eye(3, dtype=torch.float64)[:1]                                   # one token: z = first column of the router
    router = torch.tensor([[2.0, 0, 0], [1.0, 0, 0], [0.0, 0, 0], [-1.0, 0, 0]], dtype=torch.float64)
    s = torch.softmax(torch.tensor([2.0, 1.0, 0.0, -1.0], dtype=torch.float64), 0)
    chosen, w = plain.route(h, router, torch.zeros(4, dtype=torch.float64), 2)
    assert chosen.tolist() == [[0, 1]] and torch.allclose(w[0], s[:2])
    chosen, w = plain.route(h, router, torch.tensor([0.0, 0.0, 0.0, 5.0], dtype=torch.float64), 2)
    assert chosen.tolist() == [[3, 0]] and torch.allclose(w[0], torch.stack([s[3], s[0]]))      # not renormalised: sum < 1
    assert float(w.sum()) < 1.0


def test_plain_mixture_identity_and_shared_experts():
    torch.manual_seed(0)
    H, F = 4, 3
    w = {"m.router": torch.zeros(3, H, dtype=torch.float64), "m.correction": torch.tensor([0.0, -1.0, 0.0], dtype=torch.float64),
         "m.e0.up": torch.randn(F, H, dtype=torch.float64), "m.e0.down": torch.randn(H, F, dtype=torch.float64),
         "m.e1.up": torch.randn(F, H, dtype=torch.float64), "m.e1.down": torch.randn(H, F, dtype=torch.float64),
         "m.shared.up": torch.randn(2, H, dtype=torch.float64), "m.shared.down": torch.randn(H, 2, dtype=torch.float64)}
    h = torch.randn(2, H, dtype=torch.float64)
    mlp = dict(router=dict(experts=2, identity=1, top=2), expert=dict(ff=F), shared=dict(ff=2))
    out = plain.mixture(h, w, "m.", mlp)
    # uniform scores 1/3; the correction keeps expert 1 out: expert 0 and the identity expert, each with weight 1/3
    e0 = torch.relu(h @ w["m.e0.up"].T) ** 2 @ w["m.e0.down"].T
    shared = torch.relu(h @ w["m.shared.up"].T) ** 2 @ w["m.shared.down"].T
    assert torch.allclose(out, e0 / 3 + h / 3 + shared)
    del mlp["shared"]
    assert torch.allclose(plain.mixture(h, w, "m.", mlp), e0 / 3 + h / 3)


def test_plain_model_runs_and_a_kv_from_layer_reads_the_source():
    import tempfile
    with tempfile.TemporaryDirectory() as d:
        novunex_models.make_model_dir(d, "odd")
        cfg, w = plain.read_model(d)
    toks = [5, 17, 3, 60, 2, 9]
    logits, layers = plain.forward(cfg, w, toks, layers_out=True)
    assert logits.shape == (6, 97) and layers.shape == (4, 6, 42) and torch.isfinite(logits).all()
    # causal: a later token changes nothing before it
    again = plain.forward(cfg, w, toks[:4] + [11, 12])
    assert torch.allclose(again[:4], logits[:4]) and not torch.allclose(again[4:], logits[4:])
    # changing layer 1's key projection changes layer 2's output too (it has no keys of its own)
    w2 = dict(w)
    w2["l1.mix.k"] = w["l1.mix.k"] * 1.5
    x1 = plain.forward(cfg, w2, toks, layers_out=True)[1]
    assert not torch.allclose(x1[1], layers[1]) and torch.allclose(x1[0], layers[0])
