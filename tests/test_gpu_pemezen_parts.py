"""The mechanisms that the Pemezen design brought, each alone, against the plain functions: the grouped norm (stored and
added), the short convolution with its state, the recurrent block, the feed-forward's activation, latent attention in
prompts and in decoding (keys far back, at the borders of cache blocks and of the decode kernel's chunks, the first
tokens, a window's edge), and the sandwich block."""
import numpy as np
import pytest
import torch

from plain import pemezen_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64


@pytest.fixture(autouse=True)
def _same_numbers_every_run():
    torch.manual_seed(20240)


def _context(cache, slot_tokens, dtype):
    from hymt2sharp_b200.engine.engine import StepEntry, make_context
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    ctx, _, _, plan = make_context(cache, [StepEntry(s, [0] * n, []) for s, n in slot_tokens], 10, dtype, DEV, status)
    return ctx, plan


def _cache(dtype, need=None, state_bytes=0, tokens=2048, slots=4):
    from hymt2sharp_b200.cache import GroupSpec, PagedCache
    groups = [] if need is None else [GroupSpec(need.kind, need.kv_heads, need.head_dim, 1, need.window, need.streams)]
    return PagedCache(groups, dtype, DEV, tokens, max_slots=slots, state_bytes=state_bytes)


def _tol(dtype):
    return dict(atol=4e-2, rtol=4e-2) if dtype == torch.bfloat16 else dict(atol=3e-5, rtol=3e-5)


def _close(got, ref, dtype, loose: float = 1.0) -> bool:
    """Against the largest value of the reference: 32-bit differs by the order of its sums, bfloat16 by a few roundings
    of 2^-9 on the way."""
    scale = float(ref.abs().max())
    err, limit = float((got.to(F64) - ref).abs().max()), loose * (7e-2 if dtype == torch.bfloat16 else 5e-5) * max(scale, 1e-3)
    assert err <= limit, f"largest error {err:.3e} is over {limit:.3e} (largest value {scale:.3f})"
    return True


def _weights(shapes, sigma=0.2, seed=0):
    gen = torch.Generator().manual_seed(seed)
    return {n: (torch.randn(s.shape, generator=gen) * sigma + (1.0 if s.init == "gain" else 0.0)).to(torch.bfloat16)
            for n, s in shapes.items()}


def _run_cuts(part_forward, cache, slots, inputs, cuts, dtype, width):
    """Feeds every sequence's rows through `part_forward(x, residual, ctx)` in steps of the given sizes
    (cuts[step][sequence], 0 = the sequence rests); returns each sequence's output rows."""
    at = [0] * len(inputs)
    outs = [[] for _ in inputs]
    for step in cuts:
        live = [(i, n) for i, n in enumerate(step) if n]
        ctx, plan = _context(cache, [(slots[i], n) for i, n in live], dtype)
        x = torch.cat([inputs[i][at[i]:at[i] + n] for i, n in live]).to(DEV).to(dtype)
        residual = torch.zeros(x.shape[0], width, device=DEV)
        part_forward(x, residual, ctx)
        cache.end_step(plan)
        o = 0
        for i, n in live:
            outs[i].append(residual[o:o + n].cpu()); o += n; at[i] += n
    return [torch.cat(o) if o else torch.zeros(0, width) for o in outs]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dim, groups", [(42, 3), (320, 2), (64, 1), (30, 30)])
def test_grouped_norm_stores_and_adds(dtype, dim, groups):
    from hymt2sharp_b200.parts import PartSpec, build_part
    part = build_part("norm", PartSpec("rmsnorm", dict(dim=dim, eps=1e-3, weight="w", groups=groups)))
    assert part.foldable == (groups == 1)
    gain = (1 + 0.2 * torch.randn(dim)).to(torch.bfloat16)
    part.load({"w": gain}, DEV, dtype)
    x = torch.randn(11, dim) * 3
    ref = plain.grouped_rms_norm(x.to(F64), gain.to(F64), groups, 1e-3)
    y = part.forward(x.to(DEV), None, dtype, fresh=True)
    assert y.dtype == dtype and torch.allclose(y.cpu().to(F64), ref, **_tol(dtype))
    rows = torch.tensor([7, 0, 7], dtype=torch.int32, device=DEV)
    assert torch.allclose(part.forward(x.to(DEV), None, dtype, rows_index=rows, fresh=True).cpu().to(F64), ref[[7, 0, 7]], **_tol(dtype))
    residual = torch.full((11, dim), 0.5, device=DEV)
    part.add_into(x.to(DEV).to(dtype), residual)
    ref_in = plain.grouped_rms_norm(x.to(dtype).to(F64), gain.to(F64), groups, 1e-3)
    assert torch.allclose(residual.cpu().to(F64) - 0.5, ref_in, atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps, bias, add", [(4, False, True), (1, True, False), (2, True, False), (7, False, False)])
def test_short_convolution_carries_its_inputs_across_steps(dtype, taps, bias, add):
    from hymt2sharp_b200.parts import MixerSlot
    from hymt2sharp_b200.parts.conv import ShortConv
    C = 37
    conv = ShortConv(C, taps, "w", "b" if bias else None, add_input=add)
    w = _weights(conv.tensors(), 0.5)
    conv.load(w, DEV, dtype)
    cache = _cache(dtype, state_bytes=16 + conv.state_bytes())
    slot = MixerSlot(state_offset=16, state_bytes=conv.state_bytes())
    xs = [torch.randn(n, C).to(torch.bfloat16).float() for n in (75, 9)]
    refs = []
    for x in xs:
        r = plain.causal_conv(x.to(F64), w["w"].to(F64), w["b"].to(F64) if bias else None)
        refs.append(r + x.to(F64) if add else r)

    def forward(x, residual, ctx):
        residual += conv.forward(x, ctx, slot).float()

    # whole; portions down to one and two tokens (shorter than the filter), unequal sequences resting in between
    for cuts in ([(75, 9)], [(40, 2), (1, 1), (2, 0), (1, 2), (31, 4)], [(1, 1)] * 9 + [(66, 0)]):
        slots = cache.alloc_slots(2)
        got = _run_cuts(forward, cache, slots, xs, cuts, dtype, C)
        cache.free_slots(slots)    # the next round takes the same slots: their state rows start from zero again
        for g, r in zip(got, refs):
            assert _close(g, r, dtype), cuts


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden, width, blocks, taps", [(40, 35, 5, 2), (64, 96, 1, 4), (48, 24, 24, 1)])
def test_recurrent_block_against_plain(dtype, hidden, width, blocks, taps):
    from hymt2sharp_b200.parts import MixerSlot, PartSpec, build_part
    names = dict(y_proj="y", y_bias="y.b", x_proj="x", x_bias="x.b", conv="conv", conv_bias="conv.b", r_gate="ra", r_bias="ra.b",
                 i_gate="ri", i_bias="ri.b", lam="lam", o_proj="o")
    part = build_part("mixer", PartSpec("rglru", dict(hidden=hidden, width=width, blocks=blocks, taps=taps, decay=8.0, **names)))
    w = _weights(part.tensors(), 0.3, seed=width)
    w["lam"] = (torch.randn(width) * 2 - 3).to(torch.bfloat16)      # decays from nearly 1 (a long memory) down to small ones
    part.load(w, DEV, dtype)
    assert part.cache_need() is None and part.state_bytes() == 4 * width + 4 * (taps - 1) * width
    cache = _cache(dtype, state_bytes=part.state_bytes())
    slot = MixerSlot(state_offset=0, state_bytes=part.state_bytes())
    xs = [torch.randn(n, hidden).to(torch.bfloat16).float() for n in (90, 13, 1)]
    mixer = dict(width=width, blocks=blocks)
    refs = [plain.rglru(x.to(F64), {k: v.to(F64) for k, v in w.items()}, mixer) for x in xs]
    assert refs[0][-1].abs().max() > 1e-3
    forward = lambda x, residual, ctx: part.forward(x, residual, ctx, slot)
    for cuts in ([(90, 13, 1)], [(50, 2, 1), (1, 1, 0), (1, 1, 0), (2, 9, 0), (36, 0, 0)], [(1, 1, 1)] + [(1, 1, 0)] * 12 + [(77, 0, 0)]):
        slots = cache.alloc_slots(3)
        got = _run_cuts(forward, cache, slots, xs, cuts, dtype, hidden)
        cache.free_slots(slots)
        for g, r in zip(got, refs):
            assert _close(g, r, dtype), cuts


def test_recurrent_state_is_float32_and_long_lived():
    """A decay close to 1 keeps what the first token wrote alive over hundreds of single-token steps."""
    from hymt2sharp_b200.parts import MixerSlot, PartSpec, build_part
    names = dict(y_proj="y", y_bias="y.b", x_proj="x", x_bias="x.b", conv="conv", conv_bias="conv.b", r_gate="ra", r_bias="ra.b",
                 i_gate="ri", i_bias="ri.b", lam="lam", o_proj="o")
    part = build_part("mixer", PartSpec("rglru", dict(hidden=16, width=16, blocks=2, taps=2, decay=8.0, **names)))
    w = _weights(part.tensors(), 0.3, seed=5)
    w["lam"] = torch.full((16,), -9.0).to(torch.bfloat16)     # a = exp(-8 r softplus(-9)): about 0.9995 a step
    part.load(w, DEV, torch.bfloat16)
    cache = _cache(torch.bfloat16, state_bytes=part.state_bytes())
    slot = MixerSlot(state_offset=0, state_bytes=part.state_bytes())
    x = torch.randn(400, 16).to(torch.bfloat16).float()
    x[1:] *= 0.01                                              # after the first token almost nothing comes in
    ref = plain.rglru(x.to(F64), {k: v.to(F64) for k, v in w.items()}, dict(width=16, blocks=2))
    slots = cache.alloc_slots(1)
    got = _run_cuts(lambda a, r, c: part.forward(a, r, c, slot), cache, slots, [x], [(1,)] * 400, torch.bfloat16, 16)[0]
    assert ref[-1].abs().max() > 0.05 * ref[0].abs().max()
    assert torch.allclose(got[-40:].to(F64), ref[-40:], atol=0.03 * float(ref[-40:].abs().max()), rtol=0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dense_feed_forward_with_xielu(dtype):
    from hymt2sharp_b200.parts import PartSpec, build_part
    part = build_part("feed_forward", PartSpec("dense_mlp", dict(hidden=40, intermediate=72, activation="xielu", up_proj="up",
                                                                 down_proj="down", act_params="act")))
    w = _weights(part.tensors(), 0.3)
    w["act"] = torch.tensor([0.7, -0.4]).to(torch.bfloat16)
    part.load(w, DEV, dtype)
    x = (torch.randn(19, 40) * 2).to(torch.bfloat16).float()
    residual = torch.full((19, 40), 1.0, device=DEV)
    part.forward(x.to(DEV).to(dtype), residual, None)
    ref = plain.dense_ff(x.to(F64), {k: v.to(F64) for k, v in w.items()})
    assert _close(residual.cpu() - 1.0, ref, dtype)


LATENT = dict(q_proj="q", dkv_proj="dkv", dkv_norm="dkv.norm", uk_proj="uk", uv_proj="uv", o_proj="o", g_proj="g")
YARN = dict(factor=4.0, original=16, fast=8.0, slow=1.0)


def _latent_part(hidden, heads, dim, rot, vdim, rank, scale, gate, dims=None, scaling=None, window=None, base=1000.0):
    from hymt2sharp_b200.parts import PartSpec, build_part
    position = PartSpec("yarn_interleaved", dict(dims=rot if dims is None else dims, base=base, scaling=scaling))
    part = build_part("mixer", PartSpec("latent_attention", dict(hidden=hidden, heads=heads, dim=dim, rot_dim=rot, vdim=vdim,
                                                                 kv_rank=rank, scale=scale, eps=1e-5, position=position, gate=gate,
                                                                 window=window, **LATENT)))
    mixer = dict(heads=heads, dim=dim, rot_dim=rot, vdim=vdim, kv_rank=rank, scale=scale,
                 rot=dict(dims=rot if dims is None else dims, base=base, scaling=scaling))
    return part, mixer


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden, heads, dim, rot, vdim, rank, gate, dims, scaling, window",
                         [(42, 3, 10, 6, 9, 21, "element", 4, None, None), (64, 20, 16, 16, 32, 48, "head", None, YARN, None),
                          (48, 1, 32, 16, 16, 64, None, None, YARN, None), (40, 4, 8, 8, 8, 24, "head", None, None, 70),
                          (64, 2, 192, 32, 144, 64, "element", 16, None, None), (64, 3, 48, 16, 32, 32, "head", None, None, 90)])
def test_latent_attention_prompts_then_decoding(dtype, hidden, heads, dim, rot, vdim, rank, gate, dims, scaling, window):
    from hymt2sharp_b200.parts import MixerSlot
    part, mixer = _latent_part(hidden, heads, dim, rot, vdim, rank, 1.5 / (dim + rot) ** 0.5, gate, dims, scaling, window)
    shapes = part.tensors()
    assert shapes["q"].shape == (heads * (dim + rot), hidden) and shapes["dkv"].shape == (rank + rot, hidden)
    assert ("g" in shapes) == (gate is not None)
    need = part.cache_need()
    assert (need.kv_heads, need.head_dim, need.streams, need.kind) == (1, rank + rot, 1, "window" if window else "full")
    w = _weights(shapes, 0.3, seed=heads)
    part.load(w, DEV, dtype)
    cache = _cache(dtype, need)
    slot = MixerSlot(group=0, plane=0)
    xs = [torch.randn(n, hidden).to(torch.bfloat16).float() for n in (300, 70, 3)]
    wf = {k: v.to(F64) for k, v in w.items()}
    refs = [plain.latent_attention(x.to(F64), wf, mixer, gate, 1e-5, window or 0) for x in xs]
    forward = lambda x, residual, ctx: part.forward(x, residual, ctx, slot)
    # whole prompts; prompts in portions; a prompt and then 45 single tokens (past 256 keys the decode step folds chunks)
    for cuts in ([(300, 70, 3)], [(130, 64, 2), (2, 1, 1), (62, 5, 0), (106, 0, 0)], [(255, 60, 1)] + [(1, 1, 1)] * 2 + [(1, 1, 0)] * 8 + [(1, 0, 0)] * 35):
        slots = cache.alloc_slots(3)
        got = _run_cuts(forward, cache, slots, xs, cuts, dtype, hidden)
        cache.free_slots(slots)
        for g, r in zip(got, refs):
            assert _close(g, r, dtype), cuts


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_attention_finds_one_key_wherever_it_lies(dtype):
    """The query weights are built so that a query token t meets, with nearly all of its softmax weight, the ONE earlier
    token s whose input it was made from (q(x_t) is parallel to k(x_s) when x_t = R^T x_s): keys far back, the first
    token, the last and first rows of cache blocks (63 | 64), the edges of the decode kernel's chunks (255 | 256) and the
    token just before the query.  A kernel that misses or misplaces one key gives another token's value."""
    from hymt2sharp_b200.parts import MixerSlot
    hidden, heads, dim, rot, vdim, rank = 48, 2, 32, 16, 16, 32      # (pieces of 16 everywhere: bfloat16 runs the tensor-core kernels)
    part, mixer = _latent_part(hidden, heads, dim, rot, vdim, rank, 1.0, None)
    w = _weights(part.tensors(), 0.3, seed=3)
    w["dkv.norm"] = torch.ones(rank).to(torch.bfloat16)
    pairs = {330: 0, 331: 63, 332: 64, 333: 255, 334: 256, 335: 1, 336: 127, 337: 128, 338: 319, 339: 320, 340: 339, 200: 3, 129: 64}
    q0 = w["q"].to(F64).reshape(heads, dim + rot, hidden) * 0.05
    for seed in range(300):      # (a random key may happen to lie nearly as well as the planted one: the first draw without such a key)
        gen = torch.Generator().manual_seed(seed)
        R = torch.linalg.qr(torch.randn(hidden, hidden, generator=gen, dtype=F64))[0]
        x = torch.randn(341, hidden, generator=gen, dtype=F64)
        for t, s in pairs.items():
            x[t] = R.T @ x[s]
        x = x.to(torch.bfloat16).float()
        q = q0.clone()
        for h in range(heads):
            q[h, :dim] = 6.0 * w["uk"].to(F64)[h * dim:(h + 1) * dim] @ w["dkv"].to(F64)[:rank] @ R
        w["q"] = q.reshape(heads * (dim + rot), hidden).to(torch.bfloat16)
        wf = {k: v.to(F64) for k, v in w.items()}
        p = plain.latent_attention(x.to(F64), wf, mixer, None, 1e-5, return_weights=True)
        if all(float(p[:, t, s].min()) > 0.97 for t, s in pairs.items()):
            break
    for t, s in pairs.items():
        assert float(p[:, t, s].min()) > 0.97, (t, s, p[:, t, s])
    part.load(w, DEV, dtype)
    ref = plain.latent_attention(x.to(F64), wf, mixer, None, 1e-5)
    cache = _cache(dtype, part.cache_need())
    slot = MixerSlot(group=0, plane=0)
    forward = lambda a, residual, ctx: part.forward(a, residual, ctx, slot)
    other = torch.randn(20, hidden).to(torch.bfloat16).float()
    # the probes inside one prompt; inside portions; and decoded one by one beside a second, short sequence
    for cuts in ([(341, 0)], [(100, 20), (29, 0), (1, 0), (199, 0), (12, 0)], [(325, 4)] + [(1, 1)] * 16):
        slots = cache.alloc_slots(2)
        got = _run_cuts(forward, cache, slots, [x, other], cuts, dtype, hidden)[0]
        cache.free_slots(slots)
        assert _close(got, ref, dtype, loose=4.0), cuts     # (a softmax this sharp magnifies a rounding of its scores)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_attention_window_edge(dtype):
    """With a window of 50 the key 50 back is out and the key 49 back is in: each probe's query is built to meet one of them."""
    from hymt2sharp_b200.parts import MixerSlot
    hidden, heads, dim, rot, vdim, rank, window = 32, 2, 16, 16, 16, 32, 50
    part, mixer = _latent_part(hidden, heads, dim, rot, vdim, rank, 1.0, None, window=window)
    w = _weights(part.tensors(), 0.3, seed=4)
    gen = torch.Generator().manual_seed(2)
    R = torch.linalg.qr(torch.randn(hidden, hidden, generator=gen, dtype=F64))[0]
    w["dkv.norm"] = torch.ones(rank).to(torch.bfloat16)
    q = w["q"].to(F64).reshape(heads, dim + rot, hidden) * 0.05
    for h in range(heads):
        q[h, :dim] = 4.0 * w["uk"].to(F64)[h * dim:(h + 1) * dim] @ w["dkv"].to(F64)[:rank] @ R
    w["q"] = q.reshape(heads * (dim + rot), hidden).to(torch.bfloat16)
    part.load(w, DEV, dtype)
    pairs = {150: 101, 151: 101, 152: 103, 153: 103, 120: 71, 121: 71}      # 49 back (seen), 50 back (not seen), ...
    x = torch.randn(160, hidden, generator=gen, dtype=F64)
    for t, s in pairs.items():
        x[t] = R.T @ x[s]
    x = x.to(torch.bfloat16).float()
    wf = {k: v.to(F64) for k, v in w.items()}
    p = plain.latent_attention(x.to(F64), wf, mixer, None, 1e-5, window, return_weights=True)
    assert float(p[:, 150, 101].min()) > 0.8 and float(p[:, 151, 101].max()) == 0.0 and float(p[:, 152, 103].min()) > 0.8
    ref = plain.latent_attention(x.to(F64), wf, mixer, None, 1e-5, window)
    cache = _cache(dtype, part.cache_need())
    slot = MixerSlot(group=0, plane=0)
    forward = lambda a, residual, ctx: part.forward(a, residual, ctx, slot)
    for cuts in ([(160,)], [(99,), (3,)] + [(1,)] * 58, [(145,)] + [(1,)] * 15):
        slots = cache.alloc_slots(1)
        got = _run_cuts(forward, cache, slots, [x], cuts, dtype, hidden)[0]
        cache.free_slots(slots)
        assert _close(got, ref, dtype, loose=4.0), cuts     # (a softmax this sharp magnifies a rounding of its scores)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sandwich_block_without_a_feed_forward_and_with_one(dtype):
    from hymt2sharp_b200.parts import MixerSlot, PartSpec, build_part
    H, groups, taps = 36, 3, 3
    norm = lambda n: PartSpec("rmsnorm", dict(dim=H, eps=1e-5, weight=n, groups=groups))
    names = dict(y_proj="m.y", y_bias="m.y.b", x_proj="m.x", x_bias="m.x.b", conv="m.conv", conv_bias="m.conv.b", r_gate="m.ra",
                 r_bias="m.ra.b", i_gate="m.ri", i_bias="m.ri.b", lam="m.lam", o_proj="m.o")
    mixer = PartSpec("rglru", dict(hidden=H, width=20, blocks=2, taps=2, decay=8.0, **names))
    ff = PartSpec("dense_mlp", dict(hidden=H, intermediate=50, activation="xielu", up_proj="f.up", down_proj="f.down", act_params="f.act"))
    for with_ff in (False, True):
        params = dict(norm1=norm("n1"), mixer=mixer, norm1_after=norm("n1b"), conv1=dict(channels=H, taps=taps, weight="c1"))
        if with_ff:
            params.update(norm2=norm("n2"), feed_forward=ff, norm2_after=norm("n2b"), conv2=dict(channels=H, taps=taps, weight="c2"))
        block = build_part("block", PartSpec("sandwich", params))
        assert ("n2" in block.tensors()) == with_ff and len(block.state_bytes()) == (3 if with_ff else 2)
        assert block.cache_needs() == [None] * len(block.state_bytes())
        w = _weights(block.tensors(), 0.3, seed=1)
        block.load(w, DEV, dtype)
        slots_of, offset = [], 0
        for sb in block.state_bytes():
            slots_of.append(MixerSlot(state_offset=offset, state_bytes=sb)); offset += -(-sb // 16) * 16
        cache = _cache(dtype, state_bytes=offset)
        x0 = torch.randn(40, H).to(torch.bfloat16).float()
        wf = {k: v.to(F64) for k, v in w.items()}
        x = x0.to(F64)
        h = plain.grouped_rms_norm(x, wf["n1"], groups, 1e-5)
        h = h + plain.causal_conv(h, wf["c1"])
        x = x + plain.grouped_rms_norm(plain.rglru(h, plain.sub(wf, "m."), dict(width=20, blocks=2)), wf["n1b"], groups, 1e-5)
        if with_ff:
            h = plain.grouped_rms_norm(x, wf["n2"], groups, 1e-5)
            h = h + plain.causal_conv(h, wf["c2"])
            x = x + plain.grouped_rms_norm(plain.dense_ff(h, plain.sub(wf, "f.")), wf["n2b"], groups, 1e-5)
        for cuts in ([40], [17, 1, 2, 20]):
            slot = cache.alloc_slots(1)
            rows, at = [], 0
            for n in cuts:
                ctx, plan = _context(cache, [(slot[0], n)], dtype)
                residual = x0[at:at + n].to(DEV).clone()
                block.forward(residual, ctx, slots_of)
                cache.end_step(plan)
                rows.append(residual.cpu()); at += n
            cache.free_slots(slot)
            assert _close(torch.cat(rows), x, dtype), (with_ff, cuts)
