"""Losorax through the engine against the plain implementation (``plain_losorax``): every
mechanism alone, every way of cutting requests into steps, the edges of the distance rows,
far memory, reused slots, greedy generation through the library's own entry point."""
import json
import math
import os

import numpy as np
import pytest
import torch

import losorax_tiny as tiny
import plain_losorax as plain
from replay_cuts import (rel_err, run_batch, run_chunks, run_schedule, run_tail_by_one,
                         run_whole)

pytestmark = pytest.mark.gpu

# Relative to the largest plain logit.  The float32 runs are the sharp ones; in bfloat16 the
# bound is on the mean over the positions, with a loose one on the worst (a router's close call
# may send a token to another expert there).
TOL = {"float32": 1e-4, "bfloat16": 4e-2}
BF16_WORST = 0.5


def close(got, want, dtype):
    if dtype == "float32":
        return rel_err(got, want) <= TOL[dtype]
    want = np.asarray(want, dtype=np.float64)
    per_row = np.abs(np.asarray(got, dtype=np.float64) - want).max(axis=-1) / np.abs(want).max()
    return per_row.mean() <= TOL[dtype] and per_row.max() <= BF16_WORST


LENGTHS = {"A": [1, 2, 3, 10, 23, 75, 140], "B": [1, 5, 64, 65, 131, 200], "C": [1, 2, 9, 40],
           "D": [1, 4, 31, 70, 100]}


def _write(tmp_path_factory, name, cfg, seed, edit=None):
    """A model folder for ``cfg`` with seeded random weights; ``edit(tensors)`` may change
    tensors before they are written."""
    from cretif_b200.config import build_losorax_spec, losorax_config_from_dict
    from cretif_b200.engine.model import manifest
    from cretif_b200.weights.loader import random_weights, write_model_folder
    d = str(tmp_path_factory.mktemp(f"losorax_{name}"))
    names, _ = manifest(build_losorax_spec(losorax_config_from_dict(cfg)))
    tensors = random_weights(names, seed, torch.bfloat16)
    # wider projections than the default draw: scores, gates and routers that are not all alike
    for k in tensors:
        if k.endswith((".q", ".k", ".v", ".r", ".g", ".a", ".w1", ".gate", ".up", ".down", ".o")) \
                or k in ("embed", "head"):
            tensors[k] = (tensors[k].float() * 4.0).to(torch.bfloat16)
    if edit is not None:
        edit(tensors)
    write_model_folder(d, cfg, tensors)
    return d


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {n: _write(tmp_path_factory, n, c, tiny.SEEDS[n]) for n, c in tiny.CONFIGS.items()}


@pytest.fixture(scope="module")
def engines(folders):
    from cretif_b200.engine import Engine
    made = {}

    def get(name, dtype, max_tokens=2048):
        key = (name, dtype, max_tokens)
        if key not in made:
            made[key] = Engine(folders[name], dtype=dtype, max_tokens=max_tokens)
        return made[key]
    return get


@pytest.fixture(scope="module")
def plain_logits(folders):
    models, memo = {}, {}

    def get(name, toks):
        key = (name, tuple(toks))
        if key not in memo:
            if name not in models:
                models[name] = plain.read_model_folder(folders[name])
            cfg, w = models[name]
            memo[key] = plain.forward(cfg, w, list(toks)).numpy()
        return memo[key]
    return get


# ------------------------------------------------------------------ registry and loading
def test_the_configuration_picks_the_model_and_its_parts(folders):
    from cretif_b200.config import load_config
    from cretif_b200.engine import Engine
    arch, cfg, spec = load_config(folders["A"])
    assert arch.name == "Losorax" and spec.vocab_size == 96 and spec.hidden_size == 64
    kinds = [spec.layers[e.layer].branches[0].part.kind for e in spec.schedule]
    assert kinds == ["attention", "general_delta_rule", "attention"]
    assert [b.part.kind for b in spec.layers[1].branches] == ["general_delta_rule", "routed_experts"]
    eng = Engine(folders["A"], dtype="float32", max_tokens=256)
    groups = eng.cache.stats()["groups"]
    # one set of keys and values for the writer and its reader
    assert [(g["head_dim"], g["value_dim"], g["layers"]) for g in groups] == [(16, 24, 1)]
    assert eng.cache.stats()["state_bytes"] > 0


# ------------------------------------------------------------------ kernels of the mechanisms
def test_dynamic_tanh_rows_and_addition():
    from cretif_b200.csrc import ops
    g = torch.Generator().manual_seed(1)
    for R, H in ((1, 8), (5, 100), (67, 1030), (300, 64)):
        h = torch.randn(R, H, generator=g) * 2
        y = torch.randn(R, H, generator=g) * 3
        w, b, gain = (torch.randn(H, generator=g) for _ in range(3))
        alpha = torch.tensor([0.7])
        W = {"n": w.double(), "n.b": b.double(), "n.alpha": alpha.double()[0]}
        for dt, tol in ((torch.float32, 1e-5), (torch.bfloat16, 3e-2)):
            out = torch.empty(R, H, dtype=dt, device="cuda")
            ops.dyt_rows(h.cuda(), None, w.cuda(), b.cuda(), alpha.cuda(), out)
            assert (out.cpu().double() - plain.dyt(h.double(), W, "n")).abs().max() < tol
        # with a delta that is added to the stream first, a gain, and gathered rows
        hs = h.cuda()
        out = torch.empty(R, H, device="cuda")
        ops.dyt_rows(hs, y.cuda(), w.cuda(), b.cuda(), alpha.cuda(), out, gain=gain.cuda())
        assert (hs.cpu() - (h + y)).abs().max() < 1e-6
        assert (out.cpu().double() - plain.dyt((h + y).double(), W, "n") * gain.double()
                ).abs().max() < 1e-5
        rows = torch.tensor([R - 1, 0], dtype=torch.int32, device="cuda")
        out2 = torch.empty(2, H, device="cuda")
        ops.dyt_rows(hs, None, w.cuda(), b.cuda(), alpha.cuda(), out2, gain=gain.cuda(), rows=rows)
        assert torch.equal(out2.cpu(), out.cpu()[[R - 1, 0]])
        for ydt in (torch.float32, torch.bfloat16):
            got = h.cuda()
            ops.dyt_add(got, y.cuda().to(ydt), w.cuda(), b.cuda(), alpha.cuda(), gain=gain.cuda())
            want = h.double() + plain.dyt(y.to(ydt).double(), W, "n") * gain.double()
            assert (got.cpu().double() - want).abs().max() < 1e-5


def test_token_shift_in_pieces_and_batches():
    """Rows blended with the row before, over sequences fed in pieces into their slots' saved
    rows, two sequences a step, against the whole-sequence formula; a third slot stays as it is."""
    from cretif_b200.csrc import ops
    g = torch.Generator().manual_seed(2)
    H, S0, S1 = 40, 50, 37
    hs = [torch.randn(S0, H, generator=g), torch.randn(S1, H, generator=g)]
    w, b = torch.randn(H, generator=g), torch.randn(H, generator=g)
    alpha, shift = torch.tensor([0.6]), torch.rand(H, generator=g) * 1.4 - 0.2
    W = {"n": w.double(), "n.b": b.double(), "n.alpha": alpha.double()[0]}
    for normed in (True, False):
        want = [plain.blend_with_previous(plain.dyt(x.double(), W, "n") if normed else x.double(),
                                          shift.double()) for x in hs]
        state = torch.zeros(4, H, device="cuda")
        state[1] = 5.0
        slots = torch.tensor([3, 0], dtype=torch.int32, device="cuda")
        at, got = [0, 0], [[], []]
        for n0, n1 in ((1, 2), (1, 1), (17, 1), (2, 30), (29, 3)):
            rows = torch.cat([hs[0][at[0]:at[0] + n0], hs[1][at[1]:at[1] + n1]]).cuda()
            seq = torch.tensor([0] * n0 + [1] * n1, dtype=torch.int32, device="cuda")
            cu = torch.tensor([0, n0, n0 + n1], dtype=torch.int32, device="cuda")
            out = torch.empty(n0 + n1, H, device="cuda")
            kw = dict(weight=w.cuda(), bias=b.cuda(), alpha=alpha.cuda()) if normed else {}
            ops.shift_rows(rows, shift.cuda(), state, seq, slots, cu, out, **kw)
            got[0].append(out[:n0].cpu())
            got[1].append(out[n0:].cpu())
            at = [at[0] + n0, at[1] + n1]
        assert at == [S0, S1]
        for r in range(2):
            assert (torch.cat(got[r]).double() - want[r]).abs().max() < 1e-5
        assert bool((state[1] == 5.0).all()) and bool((state[2] == 0.0).all())


def _cache_for(positions, nkv, hd, dtype, bt=64):
    n_blocks = (positions + bt - 1) // bt + 1
    kc = torch.zeros(n_blocks, nkv, bt, hd, dtype=dtype, device="cuda")
    table = torch.arange(1, n_blocks + 1, dtype=torch.int32, device="cuda").flip(0)[None, :] - 1
    return kc, table.contiguous()


def _gather(cache, table, positions, bt=64):
    t = table[0].cpu()
    return torch.stack([cache[t[p // bt], :, p % bt].cpu() for p in range(positions)])


@pytest.mark.parametrize("H,G,d,e,taps", [(4, 2, 16, 24, 3), (2, 1, 32, 16, 1), (1, 1, 8, 8, 2),
                                          (3, 3, 12, 20, 5), (2, 1, 96, 40, 4), (4, 0, 16, 16, 3),
                                          (2, 1, 16, 16, 9), (1, 1, 160, 300, 2)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_convolution_head_norm_gain_and_cache_write_in_pieces(H, G, d, e, taps, dtype):
    from cretif_b200.csrc import ops
    g = torch.Generator().manual_seed(3)
    S = 150
    C = H * d + G * (d + e)
    proj = torch.randn(S, C + 8, generator=g) * 2
    conv_w = torch.randn(C, taps, generator=g) * 0.5
    coef, every, eps = 0.4, 9, 1e-5
    cv = plain.causal_conv(proj[:, :C].double(), conv_w.double())
    gains = torch.tensor([plain.query_gain(t, coef, every) for t in range(S)])
    q_want = plain.unit(cv[:, :H * d].reshape(S, H, d), eps) * gains[:, None, None]
    kc, table = _cache_for(S, max(G, 1), d, dtype)
    vc, _ = _cache_for(S, max(G, 1), e, dtype)
    # the sequence lives in slot 1: the block table has a row per slot, the others map nothing
    table = torch.cat([torch.full_like(table, -1), table, torch.full_like(table, -1)]).contiguous()
    state = torch.zeros(3, C * (taps - 1), device="cuda")
    state[0] = 3.0
    slot = torch.tensor([1], dtype=torch.int32, device="cuda")
    fault = torch.zeros(1, dtype=torch.int32, device="cuda")
    got, at = [], 0
    for n in (1, 2, 1, 61, 3, 70, 40):
        n = min(n, S - at)
        rows = proj[at:at + n].cuda().contiguous()
        pos = torch.arange(at, at + n, dtype=torch.int32, device="cuda")
        zeros = torch.zeros(n, dtype=torch.int32, device="cuda")
        start = torch.tensor([at], dtype=torch.int32, device="cuda")
        cu = torch.tensor([0, n], dtype=torch.int32, device="cuda")
        q = torch.empty(n, H * d, dtype=dtype, device="cuda")
        ops.conv_headnorm_kv_append(rows, conv_w.cuda(), state, pos, zeros, slot, start, H, G, d,
                                    e, eps, coef, every, q, table=table, kc=kc, vc=vc,
                                    block_tokens=64, write_cache=True, fault=fault)
        if taps > 1:
            ops.delta_conv_state(rows, state, taps, C, cu, slot, 1)
        got.append(q.cpu())
        at += n
    assert at == S and int(fault.item()) == 0
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    # (bfloat16 rounds relative to a value's size; the gained queries reach several units)
    assert (torch.cat(got).double().reshape(S, H, d) - q_want).abs().max() \
        < tol * max(1.0, float(q_want.abs().max()))
    if G:
        k_want = plain.unit(cv[:, H * d:H * d + G * d].reshape(S, G, d), eps)
        v_want = cv[:, H * d + G * d:].reshape(S, G, e)
        assert (_gather(kc, table[1:2], S).double() - k_want).abs().max() < tol
        assert (_gather(vc, table[1:2], S).double() - v_want).abs().max() < tol * max(1.0, v_want.abs().max())
    assert bool((state[0] == 3.0).all()) and bool((state[2] == 0.0).all())


@pytest.mark.parametrize("H,G,d,e,rows,far", [(4, 2, 16, 24, 12, 40), (2, 1, 32, 16, 7, 100),
                                              (1, 1, 8, 8, 2, 3), (3, 3, 12, 20, 64, 500),
                                              (5, 1, 112, 112, 28, 200)])
def test_attention_with_distance_rows_other_value_size_and_one_added(H, G, d, e, rows, far):
    """The plain kernel against the formula.  The bias table is large, so that a key one
    distance row off shows, and one key per query is made to stand out at the first distance of
    a row, alternately just inside and just outside it."""
    from cretif_b200.csrc import ops
    from cretif_b200.parts.attention import distance_edges
    g = torch.Generator().manual_seed(4)
    S = 330
    q = torch.randn(S, H, d, generator=g)
    k = torch.randn(S, G, d, generator=g)
    v = torch.randn(S, G, e, generator=g)
    rel = torch.randn(rows, H, generator=g) * 3
    edges = distance_edges(rows, far)
    for i in range(S):
        n = int(edges[(i * 7) % rows]) - (i % 2)
        if 0 <= n <= i:
            k[i - n, :, 0] += 3.0
            q[i, :, 0] += 2.0
    gains = torch.ones(S, dtype=torch.float64)
    want = plain.attention_scores_to_output(q.double(), k.double(), v.double(), 0.5, rel.double(),
                                            far, gains).reshape(S, H * e)
    kc, table = _cache_for(S, G, d, torch.float32)
    vc, _ = _cache_for(S, G, e, torch.float32)
    t = table[0].cpu()
    for p in range(S):
        kc[t[p // 64], :, p % 64] = k[p].cuda()
        vc[t[p // 64], :, p % 64] = v[p].cuda()
    out = torch.empty(S, H * e, device="cuda")
    pos = torch.arange(S, dtype=torch.int32, device="cuda")
    zeros = torch.zeros(S, dtype=torch.int32, device="cuda")
    sink = torch.zeros(H, device="cuda")
    ops.attn_simt(q.reshape(S, H * d).cuda(), out, kc, vc, table, pos, zeros, zeros[:1], H, G, d,
                  0.5, 0, 64, sink=sink, vd=e, bias=rel.cuda(),
                  bias_edges=torch.from_numpy(edges).cuda())
    assert (out.cpu().double() - want).abs().max() < 5e-5
    # neither the added one nor the bias is a detail here
    ops.attn_simt(q.reshape(S, H * d).cuda(), out, kc, vc, table, pos, zeros, zeros[:1], H, G, d,
                  0.5, 0, 64, vd=e, bias=rel.cuda(), bias_edges=torch.from_numpy(edges).cuda())
    assert (out.cpu().double() - want).abs().max() > 1e-2
    ops.attn_simt(q.reshape(S, H * d).cuda(), out, kc, vc, table, pos, zeros, zeros[:1], H, G, d,
                  0.5, 0, 64, sink=sink, vd=e)
    assert (out.cpu().double() - want).abs().max() > 1e-2


@pytest.mark.parametrize("H,G,d,rows,far", [(5, 1, 112, 28, 200), (8, 2, 64, 12, 40),
                                            (4, 4, 128, 64, 500), (2, 1, 16, 7, 100),
                                            (16, 2, 32, 2, 3), (3, 1, 80, 20, 1000)])
def test_fast_attention_kernels_with_distance_rows(H, G, d, rows, far):
    """The bfloat16 attention kernels the engine picks (prompt, a further portion, single
    tokens) with the bias by distance and the added one, against the formula on the same rounded
    inputs; a key at a row's first distance, or just before it, stands out in every query."""
    from cretif_b200.csrc import ops
    from cretif_b200.parts.attention import distance_edges, run_attention
    from cretif_b200.parts.base import StepContext
    g = torch.Generator().manual_seed(7)
    S = 700
    q = torch.randn(S, H, d, generator=g)
    k = torch.randn(S, G, d, generator=g)
    edges = distance_edges(rows, far)
    for i in range(S):
        n = int(edges[(i * 5) % rows]) - (i % 2)
        if 0 <= n <= i:
            k[i - n, :, 0] += 3.0
            q[i, :, 0] += 2.0
    q, k = q.bfloat16(), k.bfloat16()
    v = torch.randn(S, G, d, generator=g).bfloat16()
    rel = (torch.randn(rows, H, generator=g) * 3).bfloat16().float()
    scale = 0.7 / d ** 0.5
    want = plain.attention_scores_to_output(q.double(), k.double(), v.double(), scale,
                                            rel.double(), far, torch.ones(S, dtype=torch.float64)
                                            ).reshape(S, H * d)
    kc, table = _cache_for(S, G, d, torch.bfloat16)
    vc = torch.zeros_like(kc)
    t = table[0].cpu()
    for p in range(S):
        kc[t[p // 64], :, p % 64] = k[p].cuda()
        vc[t[p // 64], :, p % 64] = v[p].cuda()

    class KV:
        pass
    kv = KV()
    kv.k, kv.v, kv.table, kv.block_tokens, kv.window = kc, vc, table, 64, 0
    dev = torch.device("cuda")
    i32 = dict(dtype=torch.int32, device=dev)
    fault = torch.zeros(1, **i32)
    n_far = int(edges[-1])
    row_of = np.searchsorted(edges, np.arange(n_far), side="right") - 1
    log2e = 1.4426950408889634
    dense = ((rel[torch.from_numpy(row_of)].t() * log2e).contiguous().cuda(),
             (rel[-1] * log2e).contiguous().cuda())
    sink = torch.zeros(H, device=dev)

    def ctx(T, first, decode):
        return StepContext(T=T, B=1, tok_ids=torch.zeros(T, **i32),
                           tok_pos=torch.arange(first, first + T, **i32),
                           tok_seq=torch.zeros(T, **i32), seq_slot=torch.zeros(1, **i32),
                           seq_start=torch.tensor([first], **i32),
                           cu_seqlens=torch.tensor([0, T], **i32), is_decode=decode, max_new=T,
                           max_context=1024 if decode else first + T, fault=fault,
                           dtype=torch.bfloat16, device=dev)
    before = ops.variant_counts()
    for first, T, decode in ((0, S, False), (300, S - 300, False), (S - 1, 1, True),
                             (150, 1, True), (int(edges[-1]), 1, True)):
        out = torch.zeros(T, H * d, dtype=torch.bfloat16, device=dev)
        run_attention(q[first:first + T].reshape(T, H * d).cuda(), out, ctx(T, first, decode), kv,
                      H, G, d, scale, 0, torch.bfloat16, sink, bias=rel.cuda(),
                      bias_edges=torch.from_numpy(edges).cuda(), bias_dense=dense)
        err = (out.cpu().double() - want[first:first + T]).abs().max()
        assert err <= 2e-2 * want.abs().max(), (first, T, decode, float(err))
    after = ops.variant_counts()
    ran = {k: after[k] - before[k] for k in ("prefill_attn", "prefill_attn_pair",
                                             "prefill_attn_split")}
    assert sum(ran.values()) == 2                                       # the tensor-core kernels ran
    # head sizes up to 64 take the kernel with a thread per row, which has the bias as well
    assert (ran["prefill_attn"] == 0) == (d <= 64)
    assert (after["decode_cluster"] + after["decode_split"]
            - before["decode_cluster"] - before["decode_split"]) == 3
    assert int(fault.item()) == 0


def test_a_sink_in_the_thread_per_row_prompt_kernel():
    """Head size 64 without a window: the prompt kernel with a thread per row and a lazy
    reference, with a sink of any value per head (both of its forms: two query tiles a CTA, and
    one tile split between the CTA's slots), against the formula."""
    import plain_rigozen
    from cretif_b200.csrc import ops
    from cretif_b200.parts.attention import run_attention
    from cretif_b200.parts.base import StepContext
    g = torch.Generator().manual_seed(8)
    S, H, G, d = 500, 4, 2, 64
    q = torch.randn(S, H, d, generator=g).bfloat16()
    k = torch.randn(S, G, d, generator=g).bfloat16()
    v = torch.randn(S, G, d, generator=g).bfloat16()
    sink = torch.randn(H, generator=g) * 2
    want = plain_rigozen.windowed_softmax_attention(q.double(), k.double(), v.double(), 0.2, S,
                                                    sink.double()).reshape(S, H * d)
    kc, table = _cache_for(S, G, d, torch.bfloat16)
    vc = torch.zeros_like(kc)
    t = table[0].cpu()
    for p in range(S):
        kc[t[p // 64], :, p % 64] = k[p].cuda()
        vc[t[p // 64], :, p % 64] = v[p].cuda()

    class KV:
        pass
    kv = KV()
    kv.k, kv.v, kv.table, kv.block_tokens, kv.window = kc, vc, table, 64, 0
    dev = torch.device("cuda")
    i32 = dict(dtype=torch.int32, device=dev)
    fault = torch.zeros(1, **i32)
    for mode, name in ((1, "prefill_attn_pair"), (2, "prefill_attn_split")):
        was = ops.set_prefill_pairing(mode)
        try:
            for first in (0, 130):
                T = S - first
                ctx = StepContext(T=T, B=1, tok_ids=torch.zeros(T, **i32),
                                  tok_pos=torch.arange(first, S, **i32),
                                  tok_seq=torch.zeros(T, **i32), seq_slot=torch.zeros(1, **i32),
                                  seq_start=torch.tensor([first], **i32),
                                  cu_seqlens=torch.tensor([0, T], **i32), is_decode=False,
                                  max_new=T, max_context=S, fault=fault, dtype=torch.bfloat16,
                                  device=dev)
                before = ops.variant_counts()[name]
                out = torch.zeros(T, H * d, dtype=torch.bfloat16, device=dev)
                run_attention(q[first:].reshape(T, H * d).cuda(), out, ctx, kv, H, G, d, 0.2, 0,
                              torch.bfloat16, sink.cuda())
                assert ops.variant_counts()[name] == before + 1
                err = (out.cpu().double() - want[first:]).abs().max()
                assert err <= 2e-2 * want.abs().max(), (mode, first, float(err))
        finally:
            ops.set_prefill_pairing(was)
    assert int(fault.item()) == 0


@pytest.mark.parametrize("H,d,e,R", [(2, 16, 16, 6), (3, 24, 24, 5), (1, 8, 8, 1), (3, 10, 10, 4),
                                     (2, 128, 128, 16), (1, 72, 130, 2), (1, 256, 32, 3),
                                     (4, 32, 32, 16)])
def test_general_delta_rule_kernels_in_pieces(H, d, e, R):
    """Unit keys, removal rates, low-rank decays and the recurrence over a sequence fed in pieces
    of 1 to 40 tokens into a slot's state, against the recurrence written out token by token."""
    from cretif_b200.csrc import ops
    g = torch.Generator().manual_seed(5)
    S = 97
    width = 3 * H * d + 2 * H * e + R
    proj = torch.randn(S, width, generator=g)
    a_bias, w0 = torch.randn(H * d, generator=g), torch.randn(H * d, generator=g)
    w2 = torch.randn(H * d, R, generator=g)
    norm_w = torch.randn(H * e, generator=g)
    P = proj.double()
    o_r, o_k, o_v, o_g, o_a, o_w = 0, H * d, 2 * H * d, 2 * H * d + H * e, 2 * H * d + 2 * H * e, \
        3 * H * d + 2 * H * e
    r = P[:, o_r:o_k].reshape(S, H, d)
    k = P[:, o_k:o_v].reshape(S, H, d)
    v = P[:, o_v:o_g].reshape(S, H, e)
    scale = math.exp(-0.5)
    w = torch.exp(-scale * plain.sigmoid(torch.tanh(P[:, o_w:]) @ w2.double().T + w0.double())
                  ).reshape(S, H, d)
    a = plain.sigmoid(P[:, o_a:o_w] + a_bias.double()).reshape(S, H, d)
    o = plain.general_delta_rule(r, k, v, w, a)
    want = (plain.unit(o, 1e-5).reshape(S, H * e) * norm_w.double() * plain.sigmoid(P[:, o_g:o_a]))

    slots, slot = 3, 2
    state = torch.zeros(slots, H * d * e, device="cuda")
    state[1] = 7.0                                     # a neighbour's state must not be touched
    seq_slot = torch.tensor([slot], dtype=torch.int32, device="cuda")
    got, at = [], 0
    for n in (1, 2, 1, 17, 40, 3, 33):
        n = min(n, S - at)
        rows = proj[at:at + n].cuda().contiguous()
        prep = torch.empty(n, 3 * H * d, device="cuda")
        cu = torch.tensor([0, n], dtype=torch.int32, device="cuda")
        low = torch.empty(n, R, device="cuda")
        ops.tanh_cols(rows[:, o_w:], low)
        z = torch.empty(n, H * d, device="cuda")
        ops.gemm_simt(low, w2.cuda(), z)
        ops.general_delta_prepare(rows, prep, a_bias.cuda(), z, w0.cuda(), H, d, e, 1e-6, scale)
        out = torch.empty(n, H * e, device="cuda")
        ops.general_delta_recurrence(rows, prep, rows[:, o_g:o_a], state, cu, seq_slot, 1, H, d, e,
                                     norm_w.cuda(), 1e-5, out)
        got.append(out.cpu())
        at += n
    assert at == S
    got = torch.cat(got).double()
    assert (got - want).abs().max() <= 2e-4 * max(1.0, want.abs().max())
    assert bool((state[1] == 7.0).all()) and bool((state[0] == 0.0).all())


@pytest.mark.parametrize("T,H,F,E,top", [(1, 64, 32, 6, 2), (70, 96, 40, 5, 3), (9, 48, 48, 1, 1),
                                         (8, 100, 36, 9, 4), (3, 70, 30, 4, 2),
                                         (300, 64, 64, 7, 2), (1000, 128, 192, 12, 3),
                                         (40, 256, 128, 33, 4), (9, 64, 64, 3, 2),
                                         (300, 40, 24, 7, 2), (130, 64, 100, 11, 1),
                                         (33, 72, 20, 40, 4)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_routed_experts_kernels(T, H, F, E, top, dtype):
    """Routing, grouping and the two grouped products (on the CUDA cores, and in bfloat16 on the
    tensor cores as well) against every token's experts computed one by one."""
    from cretif_b200.csrc import ops
    from cretif_b200.parts.experts import RoutedExperts
    g = torch.Generator().manual_seed(6)
    params = {"num_experts": E, "top": top, "intermediate_size": F, "weight_on": "input",
              "names": {"router": "router", "gate": "e{e}.gate", "up": "e{e}.up",
                        "down": "e{e}.down"}}
    tensors, W = {}, {}
    for key, (name, spec) in RoutedExperts.weight_specs(params, H).items():
        t = torch.randn(spec.shape, generator=g) * (1.0 if key == "router" else 0.3)
        tensors[key] = t.to(dtype)
        W["m." + name] = tensors[key].double()
    part = RoutedExperts(params, H, dtype, "cuda")
    part.load(tensors)
    x = torch.randn(T, H, generator=g).to(dtype)
    want = plain.routed_experts(x.double(), W, "m.", {"router": {"experts": E, "top": top}})
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    from cretif_b200.parts import experts
    ways = [(True, True)] + ([(False, True)] if dtype == torch.bfloat16 else [])
    if T * top <= experts.FEW_PAIRS:
        ways.append((True, False))                     # the few-pairs kernel
    for simt, sorted_tiles in ways:
        ops.moe_simt_only(simt)
        experts.few_pairs_off(sorted_tiles)
        before = ops.variant_counts()
        try:
            got = part.forward(x.cuda(), None)
        finally:
            ops.moe_simt_only(False)
            experts.few_pairs_off(False)
        after = ops.variant_counts()
        ran_tc = sum(after[k] - before[k] for k in ("tc64", "tc128", "tc256"))
        # bfloat16 experts whose width is a multiple of 64 take the tcgen05 grouped products
        # (the router's logits of a long step may be one more tcgen05 product)
        if not simt and sorted_tiles and F % 64 == 0 and H % 8 == 0:
            assert ran_tc >= 2
        else:
            assert ran_tc <= 1
        err = (got.cpu().double() - want).abs().max(dim=1).values / want.abs().max()
        # (in bfloat16 the activation between the products is rounded)
        assert err.max() <= tol, (simt, sorted_tiles, float(err.max()))
    # the weight on the output instead is another function
    part_out = RoutedExperts({**params, "weight_on": "output"}, H, dtype, "cuda")
    part_out.load(tensors)
    other = part_out.forward(x.cuda(), None).cpu().double()
    s = plain.sigmoid(x.double() @ W["m.router"].T)
    best = torch.topk(s, top, dim=-1)
    want_out = torch.zeros_like(want)
    for t in range(T):
        for score, e in zip(best.values[t], best.indices[t]):
            want_out[t] += score * plain.swiglu(x[t].double()[None], W, f"m.e{int(e)}.")[0]
    assert (other - want_out).abs().max() <= tol * max(1.0, want_out.abs().max())


# ------------------------------------------------------------------ each mixer alone in a model
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["attention", "general_delta"])
def test_one_layer_of_each_mixer(tmp_path_factory, kind, dtype):
    from cretif_b200.engine import Engine
    cfg = tiny.one_layer(kind)
    d = _write(tmp_path_factory, "one_" + kind, cfg, seed=9)
    eng = Engine(d, dtype=dtype, max_tokens=1024)
    pcfg, w = plain.read_model_folder(d)
    rng = np.random.default_rng(3)
    for n in (1, 2, 13, 90):
        toks = rng.integers(0, cfg["vocab"], size=n).tolist()
        want = plain.forward(pcfg, w, toks).numpy()
        assert close(run_whole(eng, toks), want, dtype), (kind, n)
        assert close(run_tail_by_one(eng, toks, tail=n), want, dtype), (kind, n)
        assert close(run_chunks(eng, toks, [2, 5, 2, 30]), want, dtype), (kind, n)
    eng.cache.check()


# ------------------------------------------------------------------ ways of cutting the work
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_whole_and_token_by_token(engines, plain_logits, name, dtype):
    eng = engines(name, dtype)
    for n in LENGTHS[name]:
        toks = tiny.tokens(name, n, 1)
        want = plain_logits(name, toks)
        got = run_whole(eng, toks)
        assert got.shape == want.shape
        assert close(got, want, dtype), (name, n)
        assert close(run_tail_by_one(eng, toks, tail=32), want, dtype), (name, n)
    toks = tiny.tokens(name, 20, 2)                    # nothing but single tokens
    assert close(run_tail_by_one(eng, toks, tail=20), plain_logits(name, toks), dtype)
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_portions_of_a_prompt(engines, plain_logits, name, dtype):
    eng = engines(name, dtype)
    n = LENGTHS[name][-1]
    toks = tiny.tokens(name, n, 3)
    want = plain_logits(name, toks)
    for cuts in ([2, 2, 2, 2], [63, 2, 64], [1, 70, 1, 2], [5] * 12, [n - 2, 2]):
        assert close(run_chunks(eng, toks, cuts), want, dtype), (name, cuts)
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_unequal_batches_against_each_alone_and_reused_slots(engines, plain_logits, name, dtype):
    """Batches of unequal requests on a cache too small for two batches: the second and third
    rounds get slots, blocks and states (matrices, saved inputs, shifted rows) that were used
    before."""
    eng = engines(name, dtype, max_tokens=640)
    lens = LENGTHS[name]
    for round_ in range(3):
        reqs = [tiny.tokens(name, n + 6 + 2 * i, 20 + round_) for i, n in enumerate(lens[:5])]
        prompts = [min(lens[i], len(r)) for i, r in enumerate(reqs)]
        outs = run_batch(eng, reqs, prompts)
        for r, got in zip(reqs, outs):
            assert close(got, plain_logits(name, r), dtype), (name, round_, len(r))
        eng.cache.check()
        assert eng.cache.stats()["slots_live"] == 0
    # a mixture: fresh prompts, further portions and single tokens in the same steps
    reqs = [tiny.tokens(name, n, 30) for n in (40, 9, 27)]
    outs = run_schedule(eng, reqs, [[(0, 18)], [(0, 2), (1, 9)], [(0, 1), (2, 25)],
                                    [(0, 19), (2, 2)]])
    for r, got in zip(reqs, outs):
        assert close(got, plain_logits(name, r), dtype), name
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(engines, plain_logits, dtype):
    """A short prompt and then 230 single tokens: the distance rows of B's layers (up to 100 and
    33 positions back), the steps of its query gain and block borders pass over decoded tokens."""
    eng = engines("B", dtype)
    toks = tiny.tokens("B", 240, 5)
    got = run_tail_by_one(eng, toks, tail=230)
    assert close(got, plain_logits("B", toks), dtype)
    eng.cache.check()


# ------------------------------------------------------------------ what a position depends on
def _one_layer_engine(tmp_path_factory, kind, tag, edit=None, dtype="float32", mixer=None, mlp=None):
    from cretif_b200.engine import Engine
    cfg = tiny.one_layer(kind, mixer=mixer, mlp=mlp)
    d = _write(tmp_path_factory, f"edge_{kind}_{tag}", cfg, seed=13, edit=edit)
    return Engine(d, dtype=dtype, max_tokens=2048), plain.read_model_folder(d), cfg


def test_the_edge_of_every_distance_row_in_prompts_and_decoded(tmp_path_factory):
    """One attention layer whose bias table alone decides the weights (a large table, small
    scores): each row's first distance lies once just inside and once just outside, far keys
    share the last row, and a model whose table has one row shifted is another function."""
    def loud(tensors):
        tensors["l0.mix.rel"] = (tensors["l0.mix.rel"].float() * 4.0).to(torch.bfloat16)
        tensors["l0.mix.q"] = (tensors["l0.mix.q"].float() * 0.1).to(torch.bfloat16)
    mixer = tiny._att(2, 1, 16, 8, 2, 10, 150, 0.3, 64, 0.3)
    eng, (pcfg, w), cfg = _one_layer_engine(tmp_path_factory, "attention", "rows", edit=loud,
                                            mixer=mixer)
    toks = np.random.default_rng(4).integers(0, cfg["vocab"], size=260).tolist()
    want = plain.forward(pcfg, w, toks).numpy()
    assert close(run_whole(eng, toks), want, "float32")
    assert close(run_tail_by_one(eng, toks, tail=120), want, "float32")
    assert close(run_chunks(eng, toks, [100, 2, 64, 1, 50]), want, "float32")
    # the rows matter: with the table rolled by one row the logits move a lot
    w2 = dict(w)
    w2["l0.mix.rel"] = torch.roll(w["l0.mix.rel"], 1, dims=0)
    other = plain.forward(pcfg, w2, toks).numpy()
    assert np.abs(other - want).max() > 5e-3 * np.abs(want).max()      # fifty times the bound


def test_a_far_key_among_hundreds(tmp_path_factory):
    """Sharpened queries: most of a row's weight lies on one key, often far back and beyond
    block borders, where every far key shares the table's last row."""
    def sharpen(tensors):
        tensors["l0.mix.q"] = (tensors["l0.mix.q"].float() * 8.0).to(torch.bfloat16)
    eng, (pcfg, w), cfg = _one_layer_engine(tmp_path_factory, "attention", "far", edit=sharpen)
    toks = np.random.default_rng(2).integers(0, cfg["vocab"], size=420).tolist()
    want = plain.forward(pcfg, w, toks).numpy()
    assert close(run_whole(eng, toks), want, "float32")
    assert close(run_tail_by_one(eng, toks, tail=50), want, "float32")


def test_memory_of_a_token_far_back(tmp_path_factory):
    """A delta layer alone whose decay is made slow and whose removal is made weak: the first
    token still shows in the logits hundreds of tokens later, across prompt portions and single
    tokens, and the engine carries it as the recurrence written out does."""
    def slow(tensors):
        tensors["l0.mix.w0"] = torch.full_like(tensors["l0.mix.w0"], -9.0)
        tensors["l0.mix.w2"] = torch.zeros_like(tensors["l0.mix.w2"])
        tensors["l0.mix.a.b"] = torch.full_like(tensors["l0.mix.a.b"], -6.0)
        tensors["l0.mix.a"] = torch.zeros_like(tensors["l0.mix.a"])
    eng, (pcfg, w), cfg = _one_layer_engine(tmp_path_factory, "general_delta", "slow", edit=slow,
                                            mixer=tiny._delta(2, 64, 4))
    rng = np.random.default_rng(8)
    n = 300
    base = rng.integers(0, cfg["vocab"], size=n).tolist()
    other = [(base[0] + 3) % cfg["vocab"]] + base[1:]
    want, want_other = (plain.forward(pcfg, w, t).numpy() for t in (base, other))
    assert np.abs(want[-1] - want_other[-1]).max() > 5e-4 * np.abs(want).max()
    for toks, ref in ((base, want), (other, want_other)):
        assert close(run_whole(eng, toks), ref, "float32")
        assert close(run_chunks(eng, toks, [3, 2, 150, 1, 1, 100]), ref, "float32")
        assert close(run_tail_by_one(eng, toks, tail=60), ref, "float32")


def test_the_first_tokens_of_a_sequence(engines, plain_logits):
    """Positions 0..5 alone and as the start of longer requests: zeros stand before the first
    token for the shift and for every tap, and the added one keeps the first softmax below 1."""
    for name in ("A", "D"):
        eng = engines(name, "float32")
        toks = tiny.tokens(name, 6, 9)
        want = plain_logits(name, toks)
        for n in range(1, 7):
            assert rel_err(run_whole(eng, toks[:n]), want[:n]) <= 1e-4
        assert rel_err(run_tail_by_one(eng, toks, tail=5), want) <= 1e-4


# ------------------------------------------------------------------ generation
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_entry_point(folders, name):
    """``load(...).generate(...)``: batching, the decode graph (whose warm-up must not advance a
    state twice) and the run-ahead of the host, against re-running the plain model on the
    growing sequence."""
    import cretif_b200
    eng = cretif_b200.load(folders[name], dtype="float32", max_tokens=2048)
    pcfg, w = plain.read_model_folder(folders[name])
    prompts = [tiny.tokens(name, n, 40) for n in (3, 11, 30)]
    for use_graph in (True, False):
        got = eng.generate(prompts, max_tokens=12, stop_ids=[], use_graph=use_graph)
        for p, r in zip(prompts, got):
            seq = list(p)
            for tok in r.tokens:        # every token is the plain model's best, or tied with it
                row = plain.forward(pcfg, w, seq)[-1].numpy()
                assert row.max() - row[tok] <= 1e-4 * np.abs(row).max(), (name, use_graph)
                seq.append(tok)
            assert len(r.tokens) == 12
    eng.cache.check()
    assert eng.cache.stats()["slots_live"] == 0


def test_the_replay_program_runs_a_losorax_folder(folders, tmp_path):
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    toks = tiny.tokens("A", 30, 50)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": toks[:20], "want": [0, 19]},
                                     {"id": "y", "tokens": toks[:7], "want": [6]}], "end": ["y"]},
             {"step": 1, "entries": [{"id": "x", "tokens": toks[20:21], "want": [0]}], "end": []},
             {"step": 2, "entries": [{"id": "x", "tokens": toks[21:22], "want": []}],
              "end": ["x"]}]
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model",
                        folders["A"], "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "64"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", text=True,
                       capture_output=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == \
        ["done 0", "done 1", "done 2"]
    cfg, w = plain.read_model_folder(folders["A"])
    want = plain.forward(cfg, w, toks).numpy()
    got0 = np.fromfile(out / "0.f32", dtype="<f4").reshape(3, -1)
    got1 = np.fromfile(out / "1.f32", dtype="<f4").reshape(1, -1)
    assert not (out / "2.f32").exists()
    assert rel_err(got0, want[[0, 19, 6]]) <= 1e-4 and rel_err(got1, want[[20]]) <= 1e-4


def test_the_command_line_writes_and_runs_a_losorax_folder(tmp_path):
    """``python -m cretif_b200``: a folder with random weights from a config.json, then greedy
    generation from token ids, the same tokens as the entry point gives."""
    import subprocess
    import sys
    import cretif_b200
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg_file = tmp_path / "cfg.json"
    cfg_file.write_text(json.dumps(tiny.L_D))
    folder = str(tmp_path / "model")
    env = dict(os.environ, PYTHONPATH=root)
    r = subprocess.run([sys.executable, "-m", "cretif_b200", folder, "5,6,7,8", "6", "--dtype",
                        "float32", "--random-weights", "21", "--config", str(cfg_file)],
                       capture_output=True, text=True, timeout=600, env=env, cwd=root)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "model: Losorax, 3 layers, hidden 40" in r.stdout
    line = [l for l in r.stdout.splitlines() if l.startswith("generated ids:")][0]
    got = json.loads(line[len("generated ids:"):line.index("(")].strip())
    eng = cretif_b200.load(folder, dtype="float32", max_tokens=512)
    want = eng.generate([[5, 6, 7, 8]], max_tokens=6, stop_ids=[])[0].tokens
    assert got == want and len(got) == 6
