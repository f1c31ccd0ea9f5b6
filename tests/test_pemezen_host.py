"""Pemezen without a GPU: its configuration, its place in the registry, its tensor list and memory plan, and the plain
implementation's own mechanisms against values worked out by hand."""
import json
import math

import pytest
import torch

import pemezen_models
from plain import pemezen_plain as plain


def test_config_reads_every_size_and_refuses_what_it_does_not_know():
    from hymt2sharp_b200.config import ConfigError, PemezenConfig, load_config
    data = pemezen_models.CONFIGS["odd"]["config"]
    cfg = PemezenConfig.from_dict(data)
    assert cfg.width == 42 and cfg.norm_groups == 3 and cfg.canon_taps == 3 and cfg.logit_softcap is None
    assert [l.type for l in cfg.layers] == ["rglru", "latent_attention", "latent_attention_2", "rglru"]
    assert cfg.layers[1].mixer.gate == "element" and cfg.layers[2].mixer.gate == "head"
    assert cfg.layers[1].mixer.rot.dims == 4 and cfg.layers[1].mixer.rot.scaling is None and cfg.layers[1].ff is None
    assert cfg.layers[2].mixer.rot.scaling["factor"] == 4.0 and cfg.layers[0].mixer.conv == 2
    assert PemezenConfig.from_dict(cfg.to_dict()) == cfg
    for path, value, word in ((("layers", 0, "type"), "mamba", "type"), (("norm", "groups"), 5, "groups"),
                              (("layers", 1, "mixer", "rot", "dims"), 3, "rot.dims"), (("layers", 0, "mixer", "blocks"), 4, "blocks"),
                              (("layers", 0, "mlp", "kind"), "experts", "mlp.kind")):
        bad = json.loads(json.dumps(data))
        node = bad
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        with pytest.raises(ConfigError, match=word):
            PemezenConfig.from_dict(bad)
    missing = json.loads(json.dumps(data))
    del missing["layers"][1]["mixer"]["kv_rank"]
    with pytest.raises(ConfigError, match="kv_rank"):
        PemezenConfig.from_dict(missing)


def test_registry_picks_the_design_by_its_name(tmp_path):
    from hymt2sharp_b200.config import known_architectures, load_config
    assert "Pemezen" in known_architectures() and "HunYuanDenseV1ForCausalLM" in known_architectures()
    (tmp_path / "config.json").write_text(json.dumps(pemezen_models.CONFIGS["even"]["config"]))
    arch, cfg = load_config(str(tmp_path))
    assert arch.name == "Pemezen" and cfg.logit_softcap == 9.0


def test_tensor_list_and_memory_plan():
    from hymt2sharp_b200.config import PemezenConfig, get_architecture
    from hymt2sharp_b200.engine.model import DecoderModel
    cfg = PemezenConfig.from_dict(pemezen_models.CONFIGS["odd"]["config"])
    model = DecoderModel(get_architecture("Pemezen").build_spec(cfg))
    t = {n: s.shape for n, s in model.tensors().items()}
    assert t["embed"] == (97, 42) and t["head"] == (97, 42) and t["final.norm"] == (42,)
    assert t["l0.mix.ra"] == (5, 7, 7) and t["l0.mix.conv"] == (35, 2) and t["l0.mix.lam"] == (35,) and t["l0.canon2"] == (42, 3)
    assert t["l1.mix.q"] == (3 * 16, 42) and t["l1.mix.dkv"] == (27, 42) and t["l1.mix.g"] == (27, 42) and t["l1.mix.uv"] == (27, 21)
    assert t["l2.mix.g"] == (5, 42) and t["l2.mix.o"] == (42, 65) and t["l2.mlp.act"] == (2,)
    assert "l1.norm2" not in t and "l1.canon2" not in t and "l3.mlp.up" not in t and "l3.canon1" in t
    import re
    unread = model.spec.ignorable_tensors       # what a checkpoint may still hold for the layers without a feed-forward
    assert any(re.fullmatch(p, "l1.norm2b") for p in unread) and any(re.fullmatch(p, "l3.canon2") for p in unread)
    assert not any(re.fullmatch(p, "l0.norm2") or re.fullmatch(p, "l1.norm1") for p in unread)
    # two attention layers with different row widths: a cache group each, one stream (a single vector per token)
    assert [(g.kv_heads, g.head_dim, g.planes, g.streams) for g in model.groups] == [(1, 27, 1, 1), (1, 21, 1, 1)]
    # state: per layer the mixer's (S and its convolution's inputs for a recurrent block), then the block's convolutions
    sizes = [[s.state_bytes for s in row] for row in model.slots]
    assert sizes == [[4 * 35 + 4 * 1 * 35, 4 * 2 * 42, 4 * 2 * 42], [0, 4 * 2 * 42], [0, 4 * 2 * 42, 4 * 2 * 42], [4 * 44 + 4 * 4 * 44, 4 * 2 * 42]]
    offsets = [s.state_offset for row in model.slots for s in row if s.state_bytes]
    assert offsets == sorted(offsets) and all(o % 16 == 0 for o in offsets) and model.state_bytes >= sum(map(sum, sizes))


def test_plain_norm_conv_and_recurrence_by_hand():
    x = torch.tensor([[3.0, 4.0, 0.0, 2.0]], dtype=torch.float64)
    y = plain.grouped_rms_norm(x, torch.tensor([1.0, 1.0, 2.0, 2.0], dtype=torch.float64), 2, 0.0)
    assert torch.allclose(y, torch.tensor([[3 / math.sqrt(12.5), 4 / math.sqrt(12.5), 0.0, 2 * 2 / math.sqrt(2.0)]], dtype=torch.float64))
    h = torch.tensor([[1.0], [2.0], [3.0]], dtype=torch.float64)
    out = plain.causal_conv(h, torch.tensor([[10.0, 1.0]], dtype=torch.float64))           # last column: the current token
    assert out.reshape(-1).tolist() == [1.0, 12.0, 23.0]
    z = torch.tensor([2.0, -1.0], dtype=torch.float64)
    sp = lambda v: math.log1p(math.exp(v))
    got = plain.xielu(z, torch.tensor(0.3, dtype=torch.float64), torch.tensor(-0.2, dtype=torch.float64))
    assert torch.allclose(got, torch.tensor([sp(0.3) * 4 + 1.0, (0.5 + sp(-0.2)) * (math.exp(-1) - 1 + 1) - 0.5], dtype=torch.float64))


def test_plain_frequencies():
    f, m = plain.yarn_frequencies(8, 100.0, None)
    assert m == 1.0 and torch.allclose(f, torch.tensor([1.0, 100 ** -0.25, 100 ** -0.5, 100 ** -0.75], dtype=torch.float64))
    f2, m2 = plain.yarn_frequencies(8, 100.0, dict(factor=4.0, original=16, fast=8.0, slow=1.0))
    # dim(8 turns) < 0 -> lo 0; dim(1 turn) = 8 ln(16 / 2 pi) / (2 ln 100) = 0.81 -> hi 1: pair 0 keeps its frequency, the others / 4
    assert m2 == pytest.approx(0.1 * math.log(4.0) + 1.0) and torch.allclose(f2, f * torch.tensor([1.0, 0.25, 0.25, 0.25], dtype=torch.float64))
    from hymt2sharp_b200.parts.rope import YarnInterleavedRotary
    part = YarnInterleavedRotary(8, 100.0, dict(factor=4.0, original=16, fast=8.0, slow=1.0))
    assert torch.allclose(torch.from_numpy(part._host).double(), f2, rtol=1e-7) and part.amplitude == pytest.approx(m2)
