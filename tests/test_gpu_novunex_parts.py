"""The mechanisms of the Novunex design one by one, each built from its own parameters with weights of its own, against the
plain functions: norms before the rotation (per head, over the whole projection), values of another width than keys, the
sink, keys that one query must find wherever they lie, a layer that reads another's keys and values, routing, the
mixture's grouped products, the block with norms behind its sublayers only."""
import math

import numpy as np
import pytest
import torch

import helpers
from plain import novunex_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64


def _context(cache, slot_tokens, dtype):
    from hymt2sharp_b200.engine.engine import StepEntry, make_context
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    entries = [StepEntry(s, [0] * n, []) for s, n in slot_tokens]
    ctx, _, _, plan = make_context(cache, entries, 10, dtype, DEV, status)
    return ctx, plan


def _cache_for(mixer, dtype, tokens=2048, slots=4):
    from hymt2sharp_b200.cache import GroupSpec, PagedCache
    n = mixer.cache_need()
    return PagedCache([GroupSpec(n.kind, n.kv_heads, n.head_dim, 1, n.window, n.streams, n.value_dim)], dtype, DEV, tokens, max_slots=slots)


def _weights(part, scale=0.1):
    return {n: (torch.randn(s.shape) * (scale if len(s.shape) == 2 else 0.1) + (0 if len(s.shape) == 2 else 1)).to(torch.bfloat16)
            for n, s in part.tensors().items()}


def _attention(kind, hidden, heads, kv, d, dv, dims, base, scale, scaling=None, own_kv=True):
    from hymt2sharp_b200.parts import PartSpec, build_part
    return build_part("mixer", PartSpec("gqa_attention", dict(
        hidden=hidden, heads=heads, kv_heads=kv, head_dim=d, value_dim=dv, scale=scale, eps=1e-5,
        qk_norm="all" if kind == "attention_2" else "head", norm_first=True, sink=kind == "attention", own_kv=own_kv,
        position=PartSpec("wavelength_scaled_rope", dict(dims=dims, base=base, scaling=scaling)),
        q_proj="q", k_proj="k" if own_kv else None, v_proj="v" if own_kv else None, o_proj="o", q_norm="q.norm",
        k_norm="k.norm" if own_kv else None)))


def _run_mixer(part, cache, slot, steps, xs, dtype, mslot=None):
    """Feeds xs [T, hidden] in portions `steps` through the mixer alone; returns what it adds to a zero residual."""
    from hymt2sharp_b200.parts import MixerSlot
    mslot = mslot or MixerSlot(group=0, plane=0)
    out, at = [], 0
    for n in steps:
        ctx, plan = _context(cache, [(slot, n)], dtype)
        res = torch.zeros(n, xs.shape[1], dtype=torch.float32, device=DEV)
        part.forward(xs[at:at + n].to(DEV).to(dtype), res, ctx, mslot)
        cache.end_step(plan)
        out.append(res.cpu())
        at += n
    return torch.cat(out)


SCALED = dict(factor=4.0, low=1.0, high=4.0, original=64)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind, hidden, heads, kv, d, dv, dims, scaling", [
    ("attention", 40, 3, 1, 10, 7, 6, None),            # odd sizes, values narrower than keys, part of a head rotated
    ("attention_2", 40, 4, 2, 6, 9, 6, SCALED),         # values wider than keys, the whole head rotated, scaled frequencies
    ("attention", 64, 4, 4, 16, 16, 0, None),           # no rotation at all, as many kv heads as heads
    ("attention_2", 96, 8, 2, 64, 32, 64, SCALED),
    ("attention", 128, 6, 3, 128, 64, 48, None),         # from here on the bfloat16 engine runs its tensor-core prompt kernel and
    ("attention_2", 128, 8, 2, 64, 64, 64, SCALED),      # its streaming decode kernel: keys and values of 64 and 128 in every pairing,
    ("attention", 64, 2, 1, 64, 128, 16, None),          # with and without the sink
    ("attention_2", 128, 4, 4, 128, 128, 128, None),
    ("attention", 128, 12, 2, 128, 128, 64, None),       # six heads on a kv head
])
def test_attention_forms_in_prompts_portions_and_decoding(dtype, kind, hidden, heads, kv, d, dv, dims, scaling):
    torch.manual_seed(hidden + d)
    part = _attention(kind, hidden, heads, kv, d, dv, dims, 1000.0, 0.7 / math.sqrt(d), scaling)
    w = _weights(part)
    part.load(w, DEV, dtype)
    T = 300
    xs = torch.randn(T, hidden).to(torch.bfloat16).float()
    m = dict(heads=heads, kv_heads=kv, dim=d, vdim=dv, scale=0.7 / math.sqrt(d), rot=dict(dims=dims, base=1000.0, scaling=scaling))
    w64 = {k: v.to(F64) for k, v in w.items()}
    pos = torch.arange(T)
    kvs = plain.keys_and_values(xs.to(F64), w64, "", m, kind, 1e-5, pos)
    ref = plain.attention_mixer(xs.to(F64), w64, "", m, kind, 1e-5, pos, kvs).numpy()
    name = "float32" if dtype == torch.float32 else "bfloat16"
    for steps in ([T], [2, 3, 59, 1, 63, 130, 42], [258] + [1] * 42):       # a whole prompt; portions down to one token; decoding past
        cache = _cache_for(part, dtype)                                      # a block's end and past the first chunk of keys (256)
        slot = cache.alloc_slots(1)[0]
        got = _run_mixer(part, cache, slot, steps, xs, dtype).numpy()
        helpers.assert_close(got, ref, name, f"{kind} d={d} dv={dv} steps {steps[:3]}", factor=2.0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_layer_without_keys_reads_the_plane_of_another(dtype):
    """Two mixers on one cache plane: the first writes keys and values, the second has no such projections and attends with
    its own queries; in prompts and in decoding."""
    from hymt2sharp_b200.parts import MixerSlot
    torch.manual_seed(3)
    a = _attention("attention_2", 48, 4, 2, 8, 12, 8, 500.0, 0.3, SCALED)
    b = _attention("attention_2", 48, 4, 2, 8, 12, 8, 500.0, 0.3, SCALED, own_kv=False)
    assert sorted(b.tensors()) == ["o", "q", "q.norm"] and a.cache_need().key() == b.cache_need().key()
    wa, wb = _weights(a), _weights(b)
    a.load(wa, DEV, dtype); b.load(wb, DEV, dtype)
    T = 90
    xa, xb = (torch.randn(T, 48).to(torch.bfloat16).float() for _ in range(2))
    m = dict(heads=4, kv_heads=2, dim=8, vdim=12, scale=0.3, rot=dict(dims=8, base=500.0, scaling=SCALED))
    pos = torch.arange(T)
    kvs = plain.keys_and_values(xa.to(F64), {k: v.to(F64) for k, v in wa.items()}, "", m, "attention_2", 1e-5, pos)
    ref = plain.attention_mixer(xb.to(F64), {k: v.to(F64) for k, v in wb.items()}, "", m, "attention_2", 1e-5, pos, kvs).numpy()
    cache = _cache_for(a, dtype)
    slot = cache.alloc_slots(1)[0]
    got, at = [], 0
    for n in [60] + [1] * 30:
        ctx, plan = _context(cache, [(slot, n)], dtype)
        ra, rb = (torch.zeros(n, 48, dtype=torch.float32, device=DEV) for _ in range(2))
        a.forward(xa[at:at + n].to(DEV).to(dtype), ra, ctx, MixerSlot(group=0, plane=0))
        b.forward(xb[at:at + n].to(DEV).to(dtype), rb, ctx, MixerSlot(group=0, plane=0, writes=False))
        cache.end_step(plan)
        got.append(rb.cpu()); at += n
    helpers.assert_close(torch.cat(got).numpy(), ref, "float32" if dtype == torch.float32 else "bfloat16", "shared plane", factor=2.0)
    with pytest.raises(ValueError, match="cache plane"):
        ctx, plan = _context(cache, [(slot, 1)], dtype)
        b.forward(xb[:1].to(DEV).to(dtype), torch.zeros(1, 48, device=DEV), ctx, MixerSlot(group=0, plane=0, writes=True))


def _planted(dtype, sink, d, dv, nkv, g, length, key_at, decode_from=None, second=None):
    """Keys of small random entries except ONE, which is the query's direction made long: the row's output must be that
    key's value (less the sink's share).  Written into the cache through the appending kernel, read by the attention."""
    from hymt2sharp_b200.cache import GroupSpec, PagedCache
    from hymt2sharp_b200.kernels import fast, ops
    torch.manual_seed(key_at + length)
    nh = nkv * g
    cache = PagedCache([GroupSpec("full", nkv, d, 1, 0, 2, 0 if dv == d else dv)], dtype, DEV, 4096, max_slots=4)
    slots = cache.alloc_slots(2)
    lens = [length] + ([second] if second else [])
    direction = torch.nn.functional.normalize(torch.randn(nkv, d), dim=-1)
    outs = {}
    at = [0] * len(lens)
    steps = [[n for n in lens]] if decode_from is None else [[min(decode_from, n) for n in lens]] + [[1 if decode_from + i < n else 0 for n in lens] for i in range(max(lens) - decode_from)]
    ks = [torch.randn(n, nkv, d) * 0.05 for n in lens]
    vs = [torch.randn(n, nkv, dv) for n in lens]
    for s, k in enumerate(ks):
        k[min(key_at, lens[s] - 1)] = direction * 4.0
    qs = [direction[:, None, :].expand(nkv, g, d).reshape(1, nh * d).repeat(n, 1) * 4.0 for n in lens]
    k_plane, v_plane = cache.plane(0, 0)
    for step in steps:
        live = [(slots[i], n) for i, n in enumerate(step) if n]
        idx = [i for i, n in enumerate(step) if n]
        ctx, plan = _context(cache, live, dtype)
        proj = torch.cat([torch.cat([qs[i][at[i]:at[i] + step[i]], ks[i][at[i]:at[i] + step[i]].reshape(step[i], -1),
                                     vs[i][at[i]:at[i] + step[i]].reshape(step[i], -1)], dim=1) for i in idx]).to(DEV).to(dtype)
        T = proj.shape[0]
        q = torch.empty(T, nh * d, dtype=dtype, device=DEV)
        ops.rope_kv_general(proj, q, k_plane, v_plane, cache.tables[0], cache.block_tokens, ctx.token_seq, ctx.token_pos, ctx.slot_ids,
                            None, 0, None, None, ops.NORM_NONE, 1e-5, nh, nkv, d, dv, True)
        out = torch.empty(T, nh * dv, dtype=dtype, device=DEV)
        split, ms, acc, ml = 0, 0, None, None
        if ctx.decode and ctx.max_kv_len > 256:
            split, ms = 256, -(-ctx.max_kv_len // 256)
            na, nm = ops.attention_simt_scratch(T, nh, dv, ms)
            acc, ml = torch.empty(na, device=DEV), torch.empty(nm, device=DEV)
        # the engine's own choice of kernels: tensor cores where they take the shape, else the general kernel
        if not fast.try_attention_kv(out, q, k_plane, v_plane, cache.tables[0], ctx, nh, nkv, d, dv, 1.0, 0, sink):
            ops.attention_simt_kv(out, q, k_plane, v_plane, cache.tables[0], ctx.cu_seqlens, ctx.slot_ids, ctx.kv_lens, ctx.num_seqs,
                                  ctx.max_new_tokens, nh, nkv, d, dv, 1.0, 0, sink, split, ms, acc, ml)
        cache.end_step(plan)
        o = 0
        for i in idx:
            for j in range(step[i]):
                outs[(i, at[i] + j)] = out[o + j].float().cpu().reshape(nkv, g, dv)
            o += step[i]; at[i] += step[i]
    return outs, vs


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sink", [False, True])
@pytest.mark.parametrize("d, dv", [(16, 24), (128, 64)])
@pytest.mark.parametrize("key_at", [0, 1, 63, 64, 127, 128, 255, 256, 319, 320, 511])
def test_one_far_key_is_found_in_prompts_and_in_decoding(dtype, sink, key_at, d, dv):
    """The key stands at the first token, at both sides of a block's end (64 tokens), of a query tile's end (128 rows of the
    tensor-core kernel) and of a chunk's end (256 keys in decoding), and hundreds of tokens back, beside a second, shorter
    sequence in the same batch.  Heads of 16 and 24 run the general kernels; heads of 128 and 64 the fast ones in bfloat16."""
    length = 600
    for decode_from in (None, 590):
        outs, vs = _planted(dtype, sink, d, dv, 3, 2, length, key_at, decode_from, second=70)
        for t in (length - 1, length - 5):
            got = outs[(0, t)]
            want = vs[0][key_at][:, None, :].expand_as(got)
            # score 16 against scores near 0: the key holds all but e^-16 * 600 of the weight
            assert torch.allclose(got, want, atol=0.05 if dtype == torch.bfloat16 else 2e-3), (key_at, t, decode_from)
        # a query in FRONT of the key does not see it
        if key_at > 3:
            early = outs.get((0, key_at - 1))
            if early is not None:
                assert not torch.allclose(early, vs[0][key_at][:, None, :].expand_as(early), atol=0.2)
        got = outs[(1, 69)]
        assert torch.allclose(got, vs[1][min(key_at, 69)][:, None, :].expand_as(got), atol=0.05 if dtype == torch.bfloat16 else 2e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_sink_takes_its_share_when_every_score_is_low(dtype):
    """Queries that point AWAY from every key: scores of -16 and near 0.  Without a sink the softmax still sums to one; with
    it the output shrinks by 1 / (1 + sum exp(s)), in a prompt, in decoding below and above the first chunk of keys."""
    from hymt2sharp_b200.cache import GroupSpec, PagedCache
    from hymt2sharp_b200.kernels import ops
    torch.manual_seed(9)
    d, dv, T = 8, 8, 300
    k = torch.randn(T, 1, d).to(torch.bfloat16).float()
    v = torch.randn(T, 1, dv).to(torch.bfloat16).float()
    q = (-0.7 * k[:, 0] + 0.1 * torch.randn(T, d)).to(torch.bfloat16).float().reshape(T, 1, d)
    for sink in (False, True):
        ref = plain.causal_attention(q.to(F64), k.to(F64), v.to(F64), 1.0, sink).numpy().reshape(T, dv)
        for steps in ([T], [40] + [1] * 260):
            cache = PagedCache([GroupSpec("full", 1, d, 1)], dtype, DEV, 1024, max_slots=2)
            slot = cache.alloc_slots(1)[0]
            kp, vp = cache.plane(0, 0)
            got, at = [], 0
            for n in steps:
                ctx, plan = _context(cache, [(slot, n)], dtype)
                proj = torch.cat([q[at:at + n, 0], k[at:at + n, 0], v[at:at + n, 0]], dim=1).to(DEV).to(dtype)
                qq = torch.empty(n, d, dtype=dtype, device=DEV)
                ops.rope_kv_general(proj, qq, kp, vp, cache.tables[0], 64, ctx.token_seq, ctx.token_pos, ctx.slot_ids, None, 0, None, None,
                                    ops.NORM_NONE, 1e-5, 1, 1, d, dv, True)
                out = torch.empty(n, dv, dtype=dtype, device=DEV)
                split, ms, acc, ml = 0, 0, None, None
                if ctx.decode and ctx.max_kv_len > 256:
                    split, ms = 256, 2
                    acc, ml = torch.empty(n * 2 * dv, device=DEV), torch.empty(n * 4, device=DEV)
                ops.attention_simt_kv(out, qq, kp, vp, cache.tables[0], ctx.cu_seqlens, ctx.slot_ids, ctx.kv_lens, 1, ctx.max_new_tokens,
                                      1, 1, d, dv, 1.0, 0, sink, split, ms, acc, ml)
                cache.end_step(plan)
                got.append(out.float().cpu()); at += n
            helpers.assert_close(torch.cat(got).numpy(), ref, "float32" if dtype == torch.float32 else "bfloat16", f"sink={sink} {steps[:2]}",
                                 factor=2.0)
    # the two differ by much: the test would see a sink that is left out
    a = plain.causal_attention(q.to(F64), k.to(F64), v.to(F64), 1.0, False)
    b = plain.causal_attention(q.to(F64), k.to(F64), v.to(F64), 1.0, True)
    assert float((a - b).abs().max()) > 0.3


@pytest.mark.parametrize("outputs, top", [(5, 2), (12, 3), (4, 4), (70, 8), (1, 1)])
def test_routing_against_the_plain_choice(outputs, top):
    from hymt2sharp_b200.kernels import ops
    torch.manual_seed(outputs)
    T = 77
    logits = (torch.randn(T, outputs) * 3).to(DEV)
    corr = (torch.randn(outputs) * 0.3).to(DEV)
    chosen = torch.empty(T, top, dtype=torch.int32, device=DEV)
    weight = torch.empty(T, top, dtype=torch.float32, device=DEV)
    ops.moe_route(chosen, weight, logits, corr)
    s = torch.softmax(logits.cpu().to(F64), -1)
    want = torch.topk(s + corr.cpu().to(F64), top, dim=-1).indices
    assert torch.equal(chosen.cpu().long(), want)
    assert torch.allclose(weight.cpu().to(F64), torch.gather(s, -1, want), rtol=1e-5, atol=1e-7)
    ops.moe_route(chosen, weight, logits, None)
    assert torch.equal(chosen.cpu().long(), torch.topk(s, top, dim=-1).indices)
    # equal scores: the lower index first
    ops.moe_route(chosen, weight, torch.zeros(T, outputs, device=DEV), None)
    assert torch.equal(chosen.cpu()[0].long(), torch.arange(top))


@pytest.mark.parametrize("kernel", ["simt", "skinny", "tc"])
@pytest.mark.parametrize("tokens, top, experts, identity", [(1, 1, 1, 0), (5, 2, 3, 2), (300, 3, 8, 4), (129, 4, 1, 3), (64, 2, 0, 3), (3000, 3, 8, 4)])
def test_sorted_rows_hold_every_pair_once_in_token_order(tokens, top, experts, identity, kernel):
    from hymt2sharp_b200.kernels import ops
    rng = np.random.default_rng(tokens)
    chosen = np.stack([rng.permutation(experts + identity)[:top] for _ in range(tokens)]).astype(np.int32)
    tile = ops.gemm_group_tile(kernel)          # row tiles of 64, 8 and 128 rows
    assert tile == {"simt": 64, "skinny": 8, "tc": 128}[kernel]
    tiles = ops.moe_tiles(tokens, top, experts, tile)
    c = torch.from_numpy(chosen).to(DEV)
    pair_row = torch.full((tokens, top), -7, dtype=torch.int32, device=DEV)
    row_token = torch.full((tiles * tile,), -7, dtype=torch.int32, device=DEV)
    tile_group = torch.full((tiles + 1,), -7, dtype=torch.int32, device=DEV)
    counts = torch.zeros(max(experts, 1), dtype=torch.int32, device=DEV)
    ops.moe_place(pair_row, row_token, tile_group, counts, c, experts, tile)
    pr, rt, tg = pair_row.cpu().numpy(), row_token.cpu().numpy(), tile_group.cpu().numpy()
    assert ((pr == -1) == (chosen >= experts)).all()
    used = 0
    for e in range(experts):
        ts = [t for t in range(tokens) for k in range(top) if chosen[t, k] == e]
        n = -(-len(ts) // tile) * tile
        assert list(rt[used:used + len(ts)]) == ts and (rt[used + len(ts):used + n] == -1).all()       # token order, then padding
        assert (tg[used // tile:(used + n) // tile] == e).all()
        for t in range(tokens):
            for k in range(top):
                if chosen[t, k] == e:
                    assert rt[pr[t, k]] == t and used <= pr[t, k] < used + len(ts)
        used += n
    assert (tg[used // tile:tiles] == -1).all() and (rt[used:] == -1).all() and tg[tiles] == used // tile


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden, experts, identity, top, ff, shared, tokens", [
    (42, 3, 2, 2, 11, 13, 70), (64, 6, 3, 2, 56, 120, 300), (40, 5, 0, 1, 8, None, 9), (48, 1, 3, 4, 5, 6, 1), (32, 0, 3, 2, 8, None, 20),
    (42, 3, 2, 2, 11, 13, 400), (128, 6, 1, 2, 72, None, 700), (64, 6, 3, 2, 56, 120, 30)])
def test_mixture_of_experts_against_plain(dtype, hidden, experts, identity, top, ff, shared, tokens):
    """Few (token, choice) pairs run the grouped product for few rows; more run the tensor-core one in bfloat16 where rows are
    whole 16-byte pieces (the cases of 300 and 700 tokens, and 30 tokens of 64 entries) and the general one otherwise (400
    tokens of 42 entries, and every 32-bit case with many pairs)."""
    from hymt2sharp_b200.parts import PartSpec, build_part
    torch.manual_seed(hidden + tokens)
    sh = None if shared is None else PartSpec("dense_mlp", dict(hidden=hidden, intermediate=shared, activation="relu2",
                                                                up_proj="m.shared.up", down_proj="m.shared.down"))
    part = build_part("feed_forward", PartSpec("routed_experts", dict(
        hidden=hidden, experts=experts, identity=identity, top=top, intermediate=ff, activation="relu2", router="m.router",
        correction="m.correction", up_proj="m.e{}.up", down_proj="m.e{}.down", shared=sh)))
    w = {n: (torch.randn(s.shape) * 0.3).to(torch.bfloat16) for n, s in part.tensors().items()}
    w["m.router"] = (w["m.router"].float() * 4).to(torch.bfloat16)
    part.load(w, DEV, dtype)
    tc = dtype == torch.bfloat16 and hidden % 8 == 0 and ff % 8 == 0
    want = "skinny" if tokens * top <= (64 if tc else 512) else ("tc" if tc else "simt")
    assert experts == 0 or part._grouped_kernel(torch.empty(1, dtype=dtype, device=DEV), tokens) == want
    x = torch.randn(tokens, hidden).to(torch.bfloat16).float()
    mlp = dict(router=dict(experts=experts, identity=identity, top=top), expert=dict(ff=ff), shared=None if shared is None else dict(ff=shared))
    ref = plain.mixture(x.to(F64), {k: v.to(F64) for k, v in w.items()}, "m.", mlp).numpy()
    from types import SimpleNamespace
    ctx = SimpleNamespace(norm_ahead=None, prenormed=None)
    name = "float32" if dtype == torch.float32 else "bfloat16"
    xs = x.to(DEV).to(dtype)
    res = torch.full((tokens, hidden), 0.5, dtype=torch.float32, device=DEV)
    part.forward(xs, res, ctx)                              # adds
    helpers.assert_close(res.cpu().numpy() - 0.5, ref, name, "mixture added", factor=2.0)
    res2 = torch.full((tokens, hidden), float("nan"), dtype=torch.float32, device=DEV)
    part.forward(xs, res2, ctx, store=True)                 # overwrites
    helpers.assert_close(res2.cpu().numpy(), ref, name, "mixture stored", factor=2.0)
    # a token's row does not depend on the other tokens of the step beyond rounding (few pairs and many run different
    # grouped products, whose sums run in different orders)
    one = torch.zeros((1, hidden), dtype=torch.float32, device=DEV)
    part.forward(xs[tokens // 2: tokens // 2 + 1], one, ctx, store=True)
    helpers.assert_close(one[0].cpu().numpy(), res2[tokens // 2].cpu().numpy(), name, "one token alone", factor=0.5)
    half = torch.zeros((tokens // 2 + 1, hidden), dtype=torch.float32, device=DEV)
    part.forward(xs[: tokens // 2 + 1], half, ctx, store=True)
    helpers.assert_close(half[-1].cpu().numpy(), res2[tokens // 2].cpu().numpy(), name, "half the tokens", factor=0.5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_block_with_norms_behind_the_sublayers_only(dtype):
    """x += norm1(mixer(x)); x += norm2(ff(x)), with and without a feed-forward, two blocks in a row (the second takes the
    rounded rows that the first leaves behind)."""
    from hymt2sharp_b200.parts import PartSpec, build_part
    torch.manual_seed(5)
    H = 48

    def block(p, ff):
        att = PartSpec("gqa_attention", dict(hidden=H, heads=4, kv_heads=2, head_dim=8, value_dim=6, scale=0.35, eps=1e-5, qk_norm="head",
                                             norm_first=True, sink=True, position=PartSpec("wavelength_scaled_rope", dict(dims=4, base=100.0)),
                                             q_proj=p + "mix.q", k_proj=p + "mix.k", v_proj=p + "mix.v", o_proj=p + "mix.o",
                                             q_norm=p + "mix.q.norm", k_norm=p + "mix.k.norm"))
        params = dict(norm1=None, mixer=att, norm1_after=PartSpec("rmsnorm", dict(dim=H, eps=1e-5, weight=p + "norm1")))
        if ff:
            params.update(norm2=None, norm2_after=PartSpec("rmsnorm", dict(dim=H, eps=1e-5, weight=p + "norm2")),
                          feed_forward=PartSpec("routed_experts", dict(hidden=H, experts=2, identity=1, top=2, intermediate=16, activation="relu2",
                                                                       router=p + "mlp.router", correction=p + "mlp.correction",
                                                                       up_proj=p + "mlp.e{}.up", down_proj=p + "mlp.e{}.down")))
        return build_part("block", PartSpec("sandwich", params))

    blocks = [block("l0.", True), block("l1.", False)]
    w = {}
    for b in blocks:
        w.update(_weights(b, 0.2))
    for k in w:
        if k.endswith("router"):
            w[k] = (w[k].float() * 5).to(torch.bfloat16)
    for b in blocks:
        b.load(w, DEV, dtype)
    T = 50
    x = torch.randn(T, H).to(torch.bfloat16).float()
    w64 = {k: v.to(F64) for k, v in w.items()}
    m = dict(heads=4, kv_heads=2, dim=8, vdim=6, scale=0.35, rot=dict(dims=4, base=100.0))
    pos = torch.arange(T)
    r = x.to(F64)
    for i, ff in enumerate((True, False)):
        p = f"l{i}."
        kv = plain.keys_and_values(r, w64, p + "mix.", m, "attention", 1e-5, pos)
        r = r + plain.rms_norm(plain.attention_mixer(r, w64, p + "mix.", m, "attention", 1e-5, pos, kv), w64[p + "norm1"], 1e-5)
        if ff:
            r = r + plain.rms_norm(plain.mixture(r, w64, p + "mlp.", dict(router=dict(experts=2, identity=1, top=2), expert=dict(ff=16))),
                                   w64[p + "norm2"], 1e-5)
    from hymt2sharp_b200.cache import GroupSpec, PagedCache
    from hymt2sharp_b200.parts import MixerSlot
    n = blocks[0].cache_needs()[0]
    cache = PagedCache([GroupSpec(n.kind, n.kv_heads, n.head_dim, 2, n.window, n.streams, n.value_dim)], dtype, DEV, 256, max_slots=2)
    slot = cache.alloc_slots(1)[0]
    ctx, plan = _context(cache, [(slot, T)], dtype)
    res = x.to(DEV).clone()
    for i, b in enumerate(blocks):
        b.forward(res, ctx, [MixerSlot(group=0, plane=i)])
        if dtype == torch.bfloat16:
            left = ctx.shared.get("residual_rows")
            assert left is not None and left[0] is res and torch.equal(left[1], res.to(torch.bfloat16))
    helpers.assert_close(res.cpu().numpy(), r.numpy(), "float32" if dtype == torch.float32 else "bfloat16", "two blocks", factor=2.0)


@pytest.mark.parametrize("tokens, top, experts, identity", [(1, 1, 1, 0), (5, 2, 3, 2), (16, 4, 32, 2), (20, 3, 0, 4), (9, 4, 1, 3)])
def test_one_launch_for_few_tokens_leaves_what_the_three_kernels_leave(tokens, top, experts, identity):
    from hymt2sharp_b200.kernels import ops
    torch.manual_seed(tokens)
    outputs = experts + identity
    logits = (torch.randn(tokens, outputs) * 2).to(DEV)
    corr = (torch.randn(outputs) * 0.2).to(DEV)
    for kernel in ("skinny", "simt"):
        tile = ops.gemm_group_tile(kernel)
        tiles = ops.moe_tiles(tokens, top, experts, tile)
        made = []
        for fused in (False, True):
            chosen = torch.full((tokens, top), -7, dtype=torch.int32, device=DEV)
            weight = torch.full((tokens, top), -7.0, device=DEV)
            pair_row = torch.full((tokens, top), -7, dtype=torch.int32, device=DEV)
            row_token = torch.full((tiles * tile,), -7, dtype=torch.int32, device=DEV)
            tile_group = torch.full((tiles + 1,), -7, dtype=torch.int32, device=DEV)
            if fused:
                ops.moe_route_place(chosen, weight, pair_row, row_token, tile_group, logits, corr, experts, tile)
            else:
                ops.moe_route(chosen, weight, logits, corr)
                ops.moe_place(pair_row, row_token, tile_group, torch.zeros(max(experts, 1), dtype=torch.int32, device=DEV), chosen, experts, tile)
            made.append([t.cpu() for t in (chosen, weight, pair_row, row_token, tile_group)])
        for a, b in zip(*made):
            assert torch.equal(a, b)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_norm_behind_a_mixture_in_one_kernel(dtype):
    """forward_then_norm against forward followed by the norm's own kernel, with and without a shared expert, with the rounded
    rows asked for and not."""
    from types import SimpleNamespace
    from hymt2sharp_b200.parts import PartSpec, build_part
    torch.manual_seed(1)
    H = 72
    norm = build_part("norm", PartSpec("rmsnorm", dict(dim=H, eps=1e-5, weight="n")))
    for shared in (None, 40):
        sh = None if shared is None else PartSpec("dense_mlp", dict(hidden=H, intermediate=shared, activation="relu2", up_proj="m.shared.up",
                                                                    down_proj="m.shared.down"))
        part = build_part("feed_forward", PartSpec("routed_experts", dict(hidden=H, experts=4, identity=2, top=3, intermediate=24, activation="relu2",
                                                                          router="m.router", correction="m.correction", up_proj="m.e{}.up",
                                                                          down_proj="m.e{}.down", shared=sh)))
        w = {n: (torch.randn(s.shape) * 0.3).to(torch.bfloat16) for n, s in part.tensors().items()}
        w["n"] = (1 + 0.1 * torch.randn(H)).to(torch.bfloat16)
        part.load(w, DEV, dtype); norm.load(w, DEV, dtype)
        for tokens in (3, 200):
            x = torch.randn(tokens, H).to(torch.bfloat16).to(DEV).to(dtype)
            start = torch.randn(tokens, H, device=DEV)
            ctx = SimpleNamespace(norm_ahead=None, prenormed=None)
            long_way, branch = start.clone(), torch.empty(tokens, H, device=DEV)
            part.forward(x, branch, ctx, store=True)
            norm.add_into(branch, long_way)
            for want in (None, torch.bfloat16):
                res = start.clone()
                rows = part.forward_then_norm(x, res, norm, ctx, want)
                helpers.assert_close(res.cpu().numpy(), long_way.cpu().numpy(), "float32", "one kernel against two", factor=2.0 if dtype == torch.float32 else 20.0)
                assert (rows is None) == (want is None)
                if rows is not None:
                    assert torch.equal(rows, res.to(torch.bfloat16))
