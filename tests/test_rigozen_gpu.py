"""Rigozen through the engine against the plain implementation (``plain_rigozen``): every
mechanism alone, every way of cutting requests into steps, windows' edges, far memory, reused
slots, greedy generation through the library's own entry point."""
import json
import os

import numpy as np
import pytest
import torch

import plain_rigozen as plain
import rigozen_tiny as tiny
from replay_cuts import (rel_err, run_batch, run_chunks, run_schedule, run_tail_by_one,
                         run_whole)

pytestmark = pytest.mark.gpu

# Relative to the largest plain logit.  bfloat16 rounds activations, keys and latents to eight
# bits several times a layer and every sublayer's output is normed before it is added, so a
# position whose sublayer output is small or whose scores are nearly tied moves by tens of per
# cent whichever kernels run and however the request is cut (the plain attention kernel and the
# tensor-core ones, whole prompts and single tokens all land within a few per cent of each
# other there); the bound is on the mean over the positions, with a loose one on the worst.
# The float32 runs are the sharp ones.
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
    from cretif_b200.config import rigozen_config_from_dict, build_rigozen_spec
    from cretif_b200.engine.model import manifest
    from cretif_b200.weights.loader import random_weights, write_model_folder
    d = str(tmp_path_factory.mktemp(f"rigozen_{name}"))
    names, _ = manifest(build_rigozen_spec(rigozen_config_from_dict(cfg)))
    tensors = random_weights(names, seed, torch.bfloat16)
    # wider projections than the default draw: scores and gates that are not all alike
    for k in tensors:
        if k.endswith((".q", ".k", ".v", ".uk", ".uv", ".dkv", ".g", ".b", ".a", ".gate",
                       ".up", ".down", ".o")) or k == "embed":
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

    def get(name, dtype, max_tokens=2048, folder=None):
        key = (name, dtype, max_tokens)
        if key not in made:
            made[key] = Engine(folder or folders[name], dtype=dtype, max_tokens=max_tokens)
        return made[key]
    return get


@pytest.fixture(scope="module")
def plain_logits(folders):
    models, memo = {}, {}

    def get(name, toks, folder=None):
        key = (name, tuple(toks))
        if key not in memo:
            if name not in models:
                models[name] = plain.read_model_folder(folder or folders[name])
            cfg, w = models[name]
            memo[key] = plain.forward(cfg, w, list(toks)).numpy()
        return memo[key]
    return get


# ------------------------------------------------------------------ registry and loading
def test_the_configuration_picks_the_model_and_its_parts(folders):
    from cretif_b200.config import load_config
    from cretif_b200.engine import Engine
    arch, cfg, spec = load_config(folders["A"])
    assert arch.name == "Rigozen" and spec.vocab_size == 96 and spec.hidden_size == 64
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 1] and len(spec.layers) == 3
    kinds = [spec.layers[e.layer].branches[0].part.kind for e in spec.schedule]
    assert kinds == ["gated_delta_rule", "attention", "latent_attention", "attention"]
    eng = Engine(folders["A"], dtype="float32", max_tokens=256)
    groups = eng.cache.stats()["groups"]
    # the attention layer and its second run share a group (two caches), the latent has its own
    assert sorted((g["head_dim"], g["layers"], g["window"]) for g in groups) == \
        [(16, 2, 9), (40, 1, 21)]
    assert eng.cache.stats()["state_bytes"] > 0


# ------------------------------------------------------------------ kernels of the mechanisms
def test_output_norm_added_to_the_stream():
    from cretif_b200.csrc import ops
    g = torch.Generator().manual_seed(1)
    for R, H in ((1, 8), (5, 100), (67, 1030), (300, 64)):
        h = torch.randn(R, H, generator=g)
        y = torch.randn(R, H, generator=g) * 3
        w = torch.randn(H, generator=g)
        want = h.double() + plain.norm_plain(y.double(), w.double(), 1e-5)
        got = h.cuda()
        ops.rmsnorm_add(got, y.cuda(), w.cuda(), 1e-5)
        assert (got.cpu().double() - want).abs().max() < 1e-5
        got = h.cuda()
        ops.rmsnorm_add(got, y.cuda().bfloat16(), w.cuda(), 1e-5)
        want = h.double() + plain.norm_plain(y.bfloat16().double(), w.double(), 1e-5)
        assert (got.cpu().double() - want).abs().max() < 1e-5


def test_a_matrix_per_head():
    from cretif_b200.csrc import ops
    g = torch.Generator().manual_seed(2)
    for M, Z, K, N in ((1, 3, 8, 40), (70, 2, 24, 8), (130, 5, 40, 72)):
        rows = torch.randn(M, Z * K + 16, generator=g)
        w = torch.randn(Z, N, K, generator=g)
        a = rows[:, :Z * K].unflatten(1, (Z, K))
        want = torch.einsum("mzk,znk->mzn", a.double(), w.double())
        for dt, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
            r = rows.cuda().to(dt)
            c = torch.empty(M, Z, N, dtype=dt, device="cuda")
            ops.gemm_batched(r[:, :Z * K].unflatten(1, (Z, K)), w.cuda().to(dt), c)
            ref = want if dt == torch.float32 else torch.einsum(
                "mzk,znk->mzn", a.bfloat16().double(), w.bfloat16().double())
            assert (c.cpu().double() - ref).abs().max() <= tol * ref.abs().max()


def _cache_for(positions, nkv, hd, dtype, bt=64):
    n_blocks = (positions + bt - 1) // bt + 1
    kc = torch.zeros(n_blocks, nkv, bt, hd, dtype=dtype, device="cuda")
    table = torch.arange(1, n_blocks + 1, dtype=torch.int32, device="cuda").flip(0)[None, :] - 1
    return kc, table.contiguous()


def _gather(cache, table, positions, bt=64):
    t = table[0].cpu()
    return torch.stack([cache[t[p // bt], :, p % bt].cpu() for p in range(positions)])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_over_whole_projections_and_keys_stored_as_values(dtype):
    from cretif_b200.csrc import ops
    g = torch.Generator().manual_seed(3)
    S, H, G, d = 70, 4, 2, 16
    rows = (torch.randn(S, H * d + G * d, generator=g) * 2).to(dtype)
    wq, wk = torch.randn(H * d, generator=g), torch.randn(G * d, generator=g)
    kc, table = _cache_for(S, G, d, dtype)
    vc = torch.zeros_like(kc)
    pos = torch.arange(S, dtype=torch.int32, device="cuda")
    zeros = torch.zeros(S, dtype=torch.int32, device="cuda")
    fault = torch.zeros(1, dtype=torch.int32, device="cuda")
    buf = rows.cuda().clone()
    ops.proj_norm_kv_append(buf, H * d, wq.cuda(), G, d, wk.cuda(), 1e-5, pos, zeros, zeros[:1],
                            table, kc, vc, 64, True, fault)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    r = rows.double()
    assert (buf[:, :H * d].cpu().double() - plain.norm_plain(r[:, :H * d], wq.double(), 1e-5)
            ).abs().max() < tol
    k_want = plain.norm_plain(r[:, H * d:], wk.double(), 1e-5).reshape(S, G, d)
    assert (_gather(kc, table, S).double() - k_want).abs().max() < tol
    assert torch.equal(_gather(vc, table, S), rows[:, H * d:].reshape(S, G, d))   # as projected
    assert int(fault.item()) == 0


@pytest.mark.parametrize("window", [1, 5, 64, 65, 200])
def test_windowed_attention_with_a_sink(window):
    """The plain kernel with a sink against the formula; one score per row is made to stand out
    at the window's first key, so that a window one key too short or too long shows."""
    from cretif_b200.csrc import ops
    g = torch.Generator().manual_seed(4)
    S, H, G, d = 150, 4, 2, 16
    q = torch.randn(S, H, d, generator=g)
    k = torch.randn(S, G, d, generator=g)
    v = torch.randn(S, G, d, generator=g)
    for i in range(S):                       # the key at the window's edge answers the query
        j = max(0, i - window + 1)
        k[j, :, 0] += 3.0
        q[i, :, 0] += 2.0
    sink = torch.randn(H, generator=g) * 2
    want = plain.windowed_softmax_attention(q.double(), k.double(), v.double(), 0.5, window,
                                            sink.double())
    kc, table = _cache_for(S, G, d, torch.float32)
    vc = torch.zeros_like(kc)
    t = table[0].cpu()
    for p in range(S):
        kc[t[p // 64], :, p % 64] = k[p].cuda()
        vc[t[p // 64], :, p % 64] = v[p].cuda()
    out = torch.empty(S, H * d, device="cuda")
    pos = torch.arange(S, dtype=torch.int32, device="cuda")
    zeros = torch.zeros(S, dtype=torch.int32, device="cuda")
    ops.attn_simt(q.reshape(S, H * d).cuda(), out, kc, vc, table, pos, zeros, zeros[:1], H, G, d,
                  0.5, window, 64, sink=sink.cuda())
    assert (out.cpu().double().reshape(S, H, d) - want).abs().max() < 2e-5
    no_sink = plain.windowed_softmax_attention(q.double(), k.double(), v.double(), 0.5, window)
    assert (no_sink - want).abs().max() > 1e-2          # the sink is not a detail here


@pytest.mark.parametrize("H,G,d,window", [(8, 1, 128, 70), (4, 2, 64, 300), (16, 1, 32, 129),
                                          (2, 2, 16, 1), (3, 1, 256, 40)])
def test_fast_attention_kernels_with_a_sink(H, G, d, window):
    """The bfloat16 attention kernels the engine picks (prompt, single tokens) with a sink,
    against the formula on the same rounded inputs; a key at each window's edge stands out."""
    from cretif_b200.parts.attention import run_attention
    from cretif_b200.parts.base import StepContext
    g = torch.Generator().manual_seed(6)
    S = 333
    q = torch.randn(S, H, d, generator=g)
    k = torch.randn(S, G, d, generator=g)
    for i in range(S):
        k[max(0, i - window + 1), :, 0] += 3.0
        q[i, :, 0] += 2.0
    q, k = q.bfloat16(), k.bfloat16()
    v = torch.randn(S, G, d, generator=g).bfloat16()
    sink = torch.randn(H, generator=g) * 2
    scale = 0.7 / d ** 0.5
    want = plain.windowed_softmax_attention(q.double(), k.double(), v.double(), scale, window,
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
    kv.k, kv.v, kv.table, kv.block_tokens, kv.window = kc, vc, table, 64, window
    dev = torch.device("cuda")
    i32 = dict(dtype=torch.int32, device=dev)
    fault = torch.zeros(1, **i32)

    def ctx(T, first, decode):
        return StepContext(T=T, B=1, tok_ids=torch.zeros(T, **i32),
                           tok_pos=torch.arange(first, first + T, **i32),
                           tok_seq=torch.zeros(T, **i32), seq_slot=torch.zeros(1, **i32),
                           seq_start=torch.tensor([first], **i32),
                           cu_seqlens=torch.tensor([0, T], **i32), is_decode=decode, max_new=T,
                           max_context=512 if decode else first + T, fault=fault,
                           dtype=torch.bfloat16, device=dev)
    # a whole prompt, a further portion at a cached position, single tokens
    for first, T, decode in ((0, S, False), (200, S - 200, False), (S - 1, 1, True),
                             (150, 1, True)):
        out = torch.zeros(T, H * d, dtype=torch.bfloat16, device=dev)
        run_attention(q[first:first + T].reshape(T, H * d).cuda(), out, ctx(T, first, decode), kv,
                      H, G, d, scale, window, torch.bfloat16, sink.cuda())
        err = (out.cpu().double() - want[first:first + T]).abs().max()
        assert err <= 2e-2 * want.abs().max(), (first, T, decode, float(err))
    assert int(fault.item()) == 0


@pytest.mark.parametrize("H,G,d,e,taps", [(4, 2, 16, 24, 3), (2, 2, 32, 32, 4), (1, 1, 8, 8, 1),
                                          (3, 1, 40, 12, 2), (2, 1, 128, 64, 4), (1, 1, 72, 130, 2),
                                          (1, 1, 256, 32, 2)])
def test_delta_rule_kernels_in_pieces(H, G, d, e, taps):
    """Convolution, gates and recurrence over a sequence fed in pieces of 1 to 40 tokens into
    a slot's state, against the recurrence written out token by token."""
    from cretif_b200.csrc import ops
    g = torch.Generator().manual_seed(5)
    S, C = 97, 2 * G * d + H * e
    proj = torch.randn(S, C + H * e + 2 * H, generator=g)
    conv_w = torch.randn(C, taps, generator=g) * 0.5
    a_log, dt_bias = torch.randn(H, generator=g) * 0.5 - 3.0, torch.randn(H, generator=g)
    norm_w = torch.randn(e, generator=g)
    P = proj.double()
    cv = plain.silu(plain.causal_conv(P[:, :C], conv_w.double()))
    qq = cv[:, :G * d].reshape(S, G, d)
    kk = cv[:, G * d:2 * G * d].reshape(S, G, d)
    vv = cv[:, 2 * G * d:].reshape(S, H, e)
    qq = qq / torch.sqrt((qq * qq).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    kk = kk / torch.sqrt((kk * kk).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(P[:, C + H * e:C + H * e + H])
    decay = torch.exp(-torch.exp(a_log.double()) * plain.softplus(P[:, C + H * e + H:]
                                                                   + dt_bias.double()))
    o = plain.delta_rule(qq.repeat_interleave(H // G, 1), kk.repeat_interleave(H // G, 1), vv,
                         beta, decay)
    want = (plain.unit(o, 1e-5) * norm_w.double()
            * plain.silu(P[:, C:C + H * e]).reshape(S, H, e)).reshape(S, H * e)

    slots, slot = 3, 2
    state = torch.zeros(slots, H * d * e + C * (taps - 1), device="cuda")
    state[1] = 7.0                                     # a neighbour's state must not be touched
    mats, inputs = state[:, :H * d * e], state[:, H * d * e:]
    seq_slot = torch.tensor([slot], dtype=torch.int32, device="cuda")
    got, at = [], 0
    for n in (1, 2, 1, 17, 40, 3, 33):
        n = min(n, S - at)
        rows = proj[at:at + n].cuda().contiguous()
        prep = torch.empty(n, C + 2 * H, device="cuda")
        pos = torch.arange(at, at + n, dtype=torch.int32, device="cuda")
        zeros = torch.zeros(n, dtype=torch.int32, device="cuda")
        start = torch.tensor([at], dtype=torch.int32, device="cuda")
        cu = torch.tensor([0, n], dtype=torch.int32, device="cuda")
        ops.delta_prepare(rows, prep, conv_w.cuda(), inputs, a_log.cuda(), dt_bias.cuda(), pos,
                          zeros, seq_slot, start, H, G, d, e, 1e-6)
        out = torch.empty(n, H * e, device="cuda")
        ops.delta_recurrence(prep, rows[:, C:C + H * e], mats, cu, seq_slot, 1, H, G, d, e,
                             norm_w.cuda(), 1e-5, out)
        ops.delta_conv_state(rows, inputs, taps, C, cu, seq_slot, 1)
        got.append(out.cpu())
        at += n
    assert at == S
    got = torch.cat(got).double()
    assert (got - want).abs().max() <= 2e-4 * max(1.0, want.abs().max())
    assert bool((state[1] == 7.0).all()) and bool((state[0] == 0.0).all())


# ------------------------------------------------------------------ each mixer alone in a model
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["attention", "latent_attention", "delta"])
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
@pytest.mark.parametrize("name", ["A", "B", "C"])
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
    rounds get slots, blocks and states that were used before."""
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
def test_long_decoding_past_every_window(engines, plain_logits, dtype):
    """A short prompt and then 230 single tokens: both windows of B (70 and 130 keys) pass over
    decoded tokens and over block borders, and window blocks are given back on the way."""
    eng = engines("B", dtype)
    toks = tiny.tokens("B", 240, 5)
    got = run_tail_by_one(eng, toks, tail=230)
    assert close(got, plain_logits("B", toks), dtype)
    eng.cache.check()


# ------------------------------------------------------------------ what a position may depend on
def _one_layer_engine(tmp_path_factory, kind, window, edit=None, dtype="float32", mixer=None):
    from cretif_b200.engine import Engine
    cfg = tiny.one_layer(kind, window)
    if mixer is not None:
        cfg["layers"][0]["mixer"] = mixer
    d = _write(tmp_path_factory, f"edge_{kind}_{window}", cfg, seed=13, edit=edit)
    return Engine(d, dtype=dtype, max_tokens=2048), plain.read_model_folder(d), cfg


@pytest.mark.parametrize("kind", ["attention", "latent_attention"])
@pytest.mark.parametrize("window", [1, 7, 64, 65, 129])
def test_a_window_ends_where_it_should(tmp_path_factory, kind, window):
    """One attention layer alone: the logits at position i depend on the tokens i-window+1 .. i
    and on nothing else.  Changing the token just inside the window changes them, changing the
    token just outside does not, for a position inside a prompt and for a decoded one."""
    eng, (pcfg, w), cfg = _one_layer_engine(tmp_path_factory, kind, window)
    rng = np.random.default_rng(window)
    n = window + 70
    base = rng.integers(0, cfg["vocab"], size=n).tolist()
    want = plain.forward(pcfg, w, base).numpy()
    for run in (run_whole, lambda e, t: run_tail_by_one(e, t, tail=40)):
        ref = run(eng, base)
        assert close(ref, want, "float32")
        for i in (n - 1, n - 17):
            inside, outside = i - window + 1, i - window
            for j, seen in ((inside, True), (outside, False)):
                other = list(base)
                other[j] = (other[j] + 1 + j % 5) % cfg["vocab"]
                got = run(eng, other)
                moved = float(np.abs(got[i] - ref[i]).max())
                # outside the window nothing of position i's arithmetic changes at all
                assert (moved > 1e-6) if seen else (moved == 0.0), (kind, window, i, j, moved)
    eng.cache.check()


def test_memory_of_a_token_far_back(tmp_path_factory):
    """A delta layer alone whose decay is made slow: the first token still shows in the logits
    hundreds of tokens later, across prompt portions and single tokens, and the engine carries
    it as the recurrence written out does."""
    def slow(tensors):
        tensors["l0.mix.A_log"] = torch.full_like(tensors["l0.mix.A_log"], -7.0)
    # wide keys, so that three hundred later writes leave something of the first
    eng, (pcfg, w), cfg = _one_layer_engine(
        tmp_path_factory, "delta", 1, edit=slow,
        mixer={"heads": 2, "kv_heads": 1, "dim": 64, "vdim": 8, "conv": 4})
    rng = np.random.default_rng(8)
    n = 300
    base = rng.integers(0, cfg["vocab"], size=n).tolist()
    other = [(base[0] + 3) % cfg["vocab"]] + base[1:]
    want, want_other = (plain.forward(pcfg, w, t).numpy() for t in (base, other))
    assert np.abs(want[-1] - want_other[-1]).max() > 1e-3 * np.abs(want).max()
    for toks, ref in ((base, want), (other, want_other)):
        assert close(run_whole(eng, toks), ref, "float32")
        assert close(run_chunks(eng, toks, [3, 2, 150, 1, 1, 100]), ref, "float32")
        assert close(run_tail_by_one(eng, toks, tail=60), ref, "float32")


def test_a_far_key_among_hundreds(tmp_path_factory):
    """Attention with a window of 300 whose queries are sharpened: most of a row's weight lies
    on one key, often far back and beyond block borders."""
    def sharpen(tensors):
        tensors["l0.mix.q"] = (tensors["l0.mix.q"].float() * 6.0).to(torch.bfloat16)
    for kind in ("attention", "latent_attention"):
        eng, (pcfg, w), cfg = _one_layer_engine(tmp_path_factory, kind, 300, edit=sharpen)
        toks = np.random.default_rng(2).integers(0, cfg["vocab"], size=420).tolist()
        want = plain.forward(pcfg, w, toks).numpy()
        assert close(run_whole(eng, toks), want, "float32")
        assert close(run_tail_by_one(eng, toks, tail=50), want, "float32")


# ------------------------------------------------------------------ generation
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_entry_point(folders, name):
    """``load(...).generate(...)``: batching, the decode graph (whose warm-up must not advance
    a recurrent state twice) and the run-ahead of the host, against re-running the plain model
    on the growing sequence."""
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


def test_the_replay_program_runs_a_rigozen_folder(folders, tmp_path):
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
