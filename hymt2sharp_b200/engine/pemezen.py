"""Pemezen: from its configuration to a ModelSpec.

Every layer is a sandwich block (a grouped RMSNorm before and after each sublayer, a short causal convolution in front
of each sublayer's input) around one of three mixers, chosen layer by layer: latent attention with an output gate per
entry, latent attention with an output gate per head, or a recurrent block with a real-gated linear recurrence; and a
dense feed-forward with the xIELU activation, or none.  The embedding rows are scaled, the final norm is grouped too,
the output head is a tensor of its own and the logits are soft-capped.  Tensor names are those of the design's
checkpoints: 'l<i>.' in front of a layer's, '.mix.' for its mixer, '.mlp.' for its feed-forward.
"""
from __future__ import annotations

from ..config.pemezen import ARCHITECTURE, PemezenConfig
from ..config.registry import register_architecture
from ..parts.base import PartSpec
from .spec import ModelSpec

RECURRENCE_DECAY = 8.0   # log a = -8 * r * softplus(lam): a constant of the design's recurrent block


def build_spec(cfg: PemezenConfig) -> ModelSpec:
    H = cfg.width

    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", dict(dim=H, eps=cfg.norm_eps, weight=name, groups=cfg.norm_groups))

    layers, unread = [], []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        x = p + "mix."
        if layer.type == "rglru":
            mixer = PartSpec("rglru", dict(hidden=H, width=m.width, blocks=m.blocks, taps=m.conv, decay=RECURRENCE_DECAY,
                                           y_proj=x + "y", y_bias=x + "y.b", x_proj=x + "x", x_bias=x + "x.b", conv=x + "conv",
                                           conv_bias=x + "conv.b", r_gate=x + "ra", r_bias=x + "ra.b", i_gate=x + "ri",
                                           i_bias=x + "ri.b", lam=x + "lam", o_proj=x + "o"))
        else:
            position = PartSpec("yarn_interleaved", dict(dims=m.rot.dims, base=m.rot.base, scaling=m.rot.scaling))
            mixer = PartSpec("latent_attention", dict(hidden=H, heads=m.heads, dim=m.dim, rot_dim=m.rot_dim, vdim=m.vdim,
                                                      kv_rank=m.kv_rank, scale=m.scale, eps=cfg.norm_eps, position=position,
                                                      gate=m.gate, q_proj=x + "q", dkv_proj=x + "dkv", dkv_norm=x + "dkv.norm",
                                                      uk_proj=x + "uk", uv_proj=x + "uv", o_proj=x + "o", g_proj=x + "g"))
        params = dict(norm1=norm(p + "norm1"), mixer=mixer, norm1_after=norm(p + "norm1b"),
                      conv1=dict(channels=H, taps=cfg.canon_taps, weight=p + "canon1"))
        if layer.ff is not None:
            params.update(norm2=norm(p + "norm2"), norm2_after=norm(p + "norm2b"),
                          feed_forward=PartSpec("dense_mlp", dict(hidden=H, intermediate=layer.ff, activation="xielu",
                                                                  up_proj=p + "mlp.up", down_proj=p + "mlp.down",
                                                                  act_params=p + "mlp.act")),
                          conv2=dict(channels=H, taps=cfg.canon_taps, weight=p + "canon2"))
        else:
            # a layer without a feed-forward reads none of the second sublayer's tensors, should a checkpoint hold them
            unread.append(rf"l{i}\.(norm2|norm2b|canon2|mlp\..*)")
        layers.append(PartSpec("sandwich", params))
    return ModelSpec(vocab=cfg.vocab, hidden=H, embedding="embed", layers=layers, final_norm=norm("final.norm"), head="head",
                     embed_scale=cfg.embedding_scale, logit_softcap=cfg.logit_softcap, ignorable_tensors=unread)


def tensor_shapes(cfg: PemezenConfig):
    from .model import DecoderModel
    return DecoderModel(build_spec(cfg)).tensors()


register_architecture(ARCHITECTURE, PemezenConfig, build_spec, tensor_shapes)
