"""Novunex: from its configuration to a ModelSpec.

Every layer has its norms BEHIND the sublayers only, x += norm1(mixer(x)), x += norm2(ff(x)) (the sandwich block without
its front norms), around grouped-query attention with values narrower or wider than keys, in one of two forms chosen layer
by layer: 'attention' norms q and k per head before the rotation and has a sink in its softmax; 'attention_2' norms the
whole q and k projections before the rotation and scales the rotation's frequencies by their wavelength.  A layer with
`kv_from` has no key/value projections and reads the cache plane of the layer it names (the order's `cache_from`).  The
feed-forward is a mixture of experts with the square of relu, identity experts, a correction of the choice and a shared
expert, or absent.  Tensor names are those of the design's checkpoints: 'l<i>.' in front of a layer's, '.mix.' for its
mixer, '.mlp.' for its feed-forward.
"""
from __future__ import annotations

from ..config.novunex import ARCHITECTURE, NovunexConfig
from ..config.registry import register_architecture
from ..parts.base import PartSpec
from .spec import ModelSpec, Run

EXPERT_ACTIVATION = "relu2"   # act(z) = max(z, 0)^2: a constant of the design


def build_spec(cfg: NovunexConfig) -> ModelSpec:
    H = cfg.width

    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", dict(dim=H, eps=cfg.norm_eps, weight=name))

    layers, order, unread = [], [], []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        x = p + "mix."
        second = layer.type == "attention_2"
        position = PartSpec("wavelength_scaled_rope", dict(dims=m.rot.dims, base=m.rot.base, scaling=m.rot.scaling if second else None))
        own = m.kv_from is None
        mixer = PartSpec("gqa_attention", dict(
            hidden=H, heads=m.heads, kv_heads=m.kv_heads, head_dim=m.dim, value_dim=m.vdim, scale=m.scale, eps=cfg.norm_eps,
            qk_norm="all" if second else "head", norm_first=True, sink=not second, own_kv=own, position=position,
            q_proj=x + "q", k_proj=x + "k" if own else None, v_proj=x + "v" if own else None, o_proj=x + "o",
            q_norm=x + "q.norm", k_norm=x + "k.norm" if own else None))
        params = dict(norm1=None, mixer=mixer, norm1_after=norm(p + "norm1"))
        if not own:
            unread.append(rf"l{i}\.mix\.(k|v)(\..*)?")
        if layer.mlp is not None:
            f = layer.mlp
            shared = None
            if f.shared_ff is not None:
                shared = PartSpec("dense_mlp", dict(hidden=H, intermediate=f.shared_ff, activation=EXPERT_ACTIVATION,
                                                    up_proj=p + "mlp.shared.up", down_proj=p + "mlp.shared.down"))
            params.update(norm2=None, norm2_after=norm(p + "norm2"),
                          feed_forward=PartSpec("routed_experts", dict(
                              hidden=H, experts=f.experts, identity=f.identity, top=f.top, intermediate=f.ff,
                              activation=EXPERT_ACTIVATION, router=p + "mlp.router", correction=p + "mlp.correction",
                              up_proj=p + "mlp.e{}.up", down_proj=p + "mlp.e{}.down", shared=shared)))
        else:
            # a layer without a feed-forward reads none of the second sublayer's tensors, should a checkpoint hold them
            unread.append(rf"l{i}\.(norm2|mlp\..*)")
        layers.append(PartSpec("sandwich", params))
        order.append(Run(i, cache_from=m.kv_from))
    return ModelSpec(vocab=cfg.vocab, hidden=H, embedding="embed", layers=layers, order=order, final_norm=norm("final.norm"), head="head",
                     ignorable_tensors=unread)


def tensor_shapes(cfg: NovunexConfig):
    from .model import DecoderModel
    return DecoderModel(build_spec(cfg)).tensors()


register_architecture(ARCHITECTURE, NovunexConfig, build_spec, tensor_shapes)
