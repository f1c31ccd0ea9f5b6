"""A recurrent block around a real-gated linear recurrent unit, as a mixer part.

Two branches of `width` channels read the mixer's input h: y = gelu_tanh(W_y h + b_y) and u = conv(W_x h + b_x), a
short causal convolution over time per channel (parts.conv.ShortConv, with a bias).  u is cut into `blocks` equal
parts; in part b the recurrence gate and the input gate are r = sigmoid(A_r[b] u_b + b_r[b]) and
i = sigmoid(A_i[b] u_b + b_i[b]) with square matrices [out, in].  Per channel

    a = exp(-decay * r * softplus(lam)),   S_t = a * S_(t-1) + sqrt(1 - a^2) * i * u,   S_(-1) = 0

and the block's output is W_o (S * y).  The gates, the decay and the state S are float32; S and the convolution's last
inputs are the sequence's state, carried from step to step in the cache's state row.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import MixerSlot, register_part
from .conv import ShortConv
from .linear import Linear, compute_form, matmul_batched


class RGLRU:
    graph_safe = True
    can_store = True   # forward(..., store=True) overwrites `residual` with its output instead of adding to it

    def __init__(self, hidden: int, width: int, blocks: int, taps: int, decay: float, y_proj: str, y_bias: str, x_proj: str,
                 x_bias: str, conv: str, conv_bias: str, r_gate: str, r_bias: str, i_gate: str, i_bias: str, lam: str,
                 o_proj: str):
        if width % blocks:
            raise ValueError(f"{width} channels cannot be cut into {blocks} equal parts")
        self.hidden, self.width, self.blocks, self.decay = int(hidden), int(width), int(blocks), float(decay)
        self.names = dict(y=y_proj, yb=y_bias, x=x_proj, xb=x_bias, ra=r_gate, rb=r_bias, ia=i_gate, ib=i_bias, lam=lam, o=o_proj)
        self.conv = ShortConv(width, taps, conv, conv_bias, add_input=False)
        self.yx = self.out = self.bias = self.ra = self.ia = self.rb = self.ib = self.lam = None

    def tensors(self):
        n, W, B, h = self.names, self.width, self.blocks, self.hidden
        bw = W // B
        t = {n["y"]: TensorSpec((W, h)), n["yb"]: TensorSpec((W,)), n["x"]: TensorSpec((W, h)), n["xb"]: TensorSpec((W,)),
             n["ra"]: TensorSpec((B, bw, bw)), n["rb"]: TensorSpec((B, bw)), n["ia"]: TensorSpec((B, bw, bw)),
             n["ib"]: TensorSpec((B, bw)), n["lam"]: TensorSpec((W,)), n["o"]: TensorSpec((h, W))}
        t.update(self.conv.tensors())
        return t

    def cache_need(self):
        return None

    def state_bytes(self) -> int:
        # S float32 [width], then the convolution's last inputs
        return 4 * self.width + self.conv.state_bytes()

    def load(self, weights, device, dtype):
        n = self.names
        small = lambda name: weights[name].to(device).float().reshape(-1).contiguous()
        self.yx = Linear(compute_form(torch.cat([weights[n["y"]], weights[n["x"]]], dim=0), device, dtype), role="yx")
        self.bias = torch.cat([small(n["yb"]), small(n["xb"])])
        self.ra, self.ia = compute_form(weights[n["ra"]], device, dtype), compute_form(weights[n["ia"]], device, dtype)
        self.rb, self.ib, self.lam = small(n["rb"]), small(n["ib"]), small(n["lam"])
        self.out = Linear(compute_form(weights[n["o"]], device, dtype), ops.EPILOGUE_ACCUMULATE, role="o_proj")
        self.out_store = Linear(self.out.weight, ops.EPILOGUE_STORE, role="o_proj")
        self.conv.load(weights, device, dtype)

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, slot: MixerSlot, store: bool = False) -> None:
        T, W, B = ctx.num_tokens, self.width, self.blocks
        bw = W // B
        yx = self.yx(x, ctx=ctx)                        # [T, y | x] before their biases
        ops.bias_act(yx, self.bias, W)                  # y = gelu_tanh(. + b_y);  x = . + b_x
        conv_slot = MixerSlot(state_offset=slot.state_offset + 4 * W, state_bytes=self.conv.state_bytes())
        u = self.conv.forward(yx[:, W:], ctx, conv_slot)
        gates = torch.empty((T, 2 * W), dtype=torch.float32, device=u.device)
        ops.tag = "gates"
        matmul_batched(gates[:, :W], u, self.ra, bw, bw)
        matmul_batched(gates[:, W:], u, self.ia, bw, bw)
        ops.tag = None
        mixed = torch.empty((T, W), dtype=u.dtype, device=u.device)
        ops.rglru_scan(mixed, gates, u, yx[:, :W], self.rb, self.ib, self.lam, self.decay, ctx.cache.state, slot.state_offset,
                       ctx.cu_seqlens, ctx.slot_ids, ctx.kv_lens, ctx.num_seqs, ctx.max_new_tokens)
        if store:
            self.out_store(mixed, out=residual)
        else:
            self.out.add_then_norm(mixed, residual, getattr(ctx, "norm_ahead", None), ctx)


register_part("mixer", "rglru", RGLRU)
