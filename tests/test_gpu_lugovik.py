"""GPU: the Lugovik model family and its mechanisms against the plain restatement in tests/lugovik_oracle.py
(float64, token by token), on small random models of several shapes: each mechanism alone, whole prompts against
token-by-token decoding and portions of many sizes, interleaved requests, reused state slots, block edges, long
decoding, greedy generation through the engine's scheduler."""
import ctypes as C
import math

import pytest
import torch

import lugovik_oracle as O

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _pkg():
    import lit_llama_b200 as P
    from lit_llama_b200 import _seqlib as S
    from lit_llama_b200 import mixers as M
    return P, S, M


_KEEP = []


def dev(t):
    """Device copy that stays alive (a temporary's pointer could be handed to the next allocation)."""
    t = t.to(DEV).contiguous()
    _KEEP.append(t)
    del _KEEP[:-64]
    return t


def rel(got, want):
    got, want = got.double().cpu(), want.double().cpu()
    return float((got - want).norm() / (want.norm() + 1e-30))


# ----------------------------------------------------------------------------- configurations (none is a served model's)
def cfg_a():
    return {"architecture": "Lugovik", "vocab": 160, "width": 96, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0}, "layers": [
        {"type": "parallel", "mlp": {"kind": "dense", "ff": 128}, "mixer": {
            "left": {"heads": 4, "kv_heads": 2, "dim": 24, "vdim": 16, "mask": {"size": 8}, "scale": 0.3, "softcap": 5.0,
                     "rot": {"base": 1000.0, "dims": 16, "scaling": {"factor": 4.0, "original": 16, "fast": 8.0, "slow": 1.0}}},
            "right": {"heads": 2, "dim": 24, "vdim": 40, "tau": 4.0, "rank": 6}, "left_scale": 0.7, "right_scale": 1.3}},
        {"type": "mamba2", "mlp": None, "mixer": {"conv": 2, "groups": 2, "heads": 4, "norm_groups": 2, "state": 24, "vdim": 12}},
        {"type": "channel_delta", "mlp": {"kind": "dense", "ff": 64},
         "mixer": {"conv": 4, "dim": 20, "heads": 4, "kv_heads": 2, "vdim": 28, "rank": 5}},
    ]}


def cfg_b():
    return {"architecture": "Lugovik", "vocab": 77, "width": 64, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0}, "layers": [
        {"type": "mamba2", "mlp": {"kind": "dense", "ff": 96}, "mixer": {"conv": 3, "groups": 1, "heads": 2, "norm_groups": 1, "state": 64, "vdim": 80}},
        {"type": "channel_delta", "mlp": None, "mixer": {"conv": 2, "dim": 72, "heads": 1, "kv_heads": 1, "vdim": 8, "rank": 3}},
        {"type": "parallel", "mlp": {"kind": "dense", "ff": 40}, "mixer": {
            "left": {"heads": 2, "kv_heads": 2, "dim": 12, "vdim": 36, "mask": {"size": 5}, "scale": 0.5, "rot": {"base": 50.0, "dims": 12}},
            "right": {"heads": 1, "dim": 8, "vdim": 8, "tau": 1.0, "rank": 2}, "left_scale": 1.0, "right_scale": 1.0}},
        {"type": "mamba2", "mlp": None, "mixer": {"conv": 4, "groups": 1, "heads": 1, "norm_groups": 4, "state": 8, "vdim": 16}},
    ]}


def cfg_c():
    """Shapes that take the tiled attention kernel, the chunk-parallel scans and two value columns per lane."""
    return {"architecture": "Lugovik", "vocab": 200, "width": 160, "norm": {"eps": 1e-6}, "embedding": {"scale": 12.0}, "layers": [
        {"type": "mamba2", "mlp": {"kind": "dense", "ff": 192}, "mixer": {"conv": 4, "groups": 1, "heads": 3, "norm_groups": 3, "state": 40, "vdim": 64}},
        {"type": "parallel", "mlp": {"kind": "dense", "ff": 192}, "mixer": {
            "left": {"heads": 4, "kv_heads": 1, "dim": 40, "vdim": 64, "mask": {"size": 100}, "scale": 0.16, "softcap": 30.0,
                     "rot": {"base": 5000.0, "dims": 32, "scaling": {"factor": 4.0, "original": 128, "fast": 16.0, "slow": 2.0}}},
            "right": {"heads": 2, "dim": 16, "vdim": 48, "tau": 8.0, "rank": 4}, "left_scale": 1.5, "right_scale": 0.5}},
        {"type": "channel_delta", "mlp": {"kind": "dense", "ff": 192}, "mixer": {"conv": 3, "dim": 48, "heads": 2, "kv_heads": 1, "vdim": 64, "rank": 12}},
    ]}


CONFIGS = {"a": cfg_a, "b": cfg_b, "c": cfg_c}


def build(cfg, dtype, seed=1, n_slots=3, **kw):
    P, _, _ = _pkg()
    W = O.random_weights(cfg, seed=seed)
    model = P.Lugovik(P.LugovikConfig.from_dict(cfg), {k: v.to(DEV, dtype) for k, v in W.items()}, max_positions=256)
    return P.Engine(model, n_slots=n_slots, **kw), {k: v.double() for k, v in W.items()}


def tokens_for(cfg, n, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


def run_schedule(engine, rid, toks, cuts, release=True):
    """Feed toks in portions of the given sizes (every place wanted); returns logits [len(toks), vocab]."""
    outs, at = [], 0
    for c in cuts:
        outs.append(engine.step([{"id": rid, "tokens": toks[at:at + c], "want": list(range(c))}])[0])
        at += c
    assert at == len(toks)
    if release:
        engine.step([], [rid])
    return torch.cat(outs).cpu()


def cuts_of(n, sizes):
    out, at, k = [], 0, 0
    while at < n:
        c = min(sizes[k % len(sizes)], n - at)
        out.append(c)
        at += c
        k += 1
    return out


F32_TOL, BF16_TOL = 2e-4, 4e-2


# ----------------------------------------------------------------------------- whole models
@pytest.mark.parametrize("name", ["a", "b"])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, F32_TOL), (torch.bfloat16, BF16_TOL)])
def test_whole_prompt_matches_the_plain_model(name, dtype, tol):
    cfg = CONFIGS[name]()
    engine, W = build(cfg, dtype)
    toks = tokens_for(cfg, 45)
    want, layers = O.forward(cfg, W, toks, return_layers=True)
    engine.model.capture_layers = []
    got = run_schedule(engine, "r", toks, [len(toks)])
    for i, x in enumerate(engine.model.capture_layers):
        assert rel(x, layers[i]) < tol, (i, cfg["layers"][i]["type"], rel(x, layers[i]))
    assert rel(got, want) < tol, rel(got, want)
    worst = max(rel(got[t], want[t]) for t in range(len(toks)))
    assert worst < 4 * tol, worst


@pytest.mark.parametrize("name", ["a", "b"])
def test_prefill_decode_and_portions_agree(name):
    """f32: whole prompt == token by token == portions of many sizes (down to two, across block edges), to rounding;
    every one of them matches the plain model."""
    cfg = CONFIGS[name]()
    engine, W = build(cfg, torch.float32)
    toks = tokens_for(cfg, 70, seed=3)
    want = O.forward(cfg, W, toks)
    whole = run_schedule(engine, "w", toks, [len(toks)])
    assert rel(whole, want) < F32_TOL
    for sizes in ([1], [2], [3, 1, 2, 7, 1, 1, 5], [33, 2, 35], [8, 8, 8], [9, 40, 1, 1, 1, 2, 16]):
        got = run_schedule(engine, "p", toks, cuts_of(len(toks), sizes))
        assert rel(got, whole) < 2e-5, (sizes, rel(got, whole))
        assert max(rel(got[t], want[t]) for t in range(len(toks))) < 4 * F32_TOL, sizes


def test_bf16_schedules_agree_within_rounding():
    cfg = cfg_a()
    engine, W = build(cfg, torch.bfloat16)
    toks = tokens_for(cfg, 50, seed=4)
    want = O.forward(cfg, W, toks)
    for sizes in ([50], [1], [2], [7, 1, 13, 2]):
        got = run_schedule(engine, "p", toks, cuts_of(len(toks), sizes))
        assert max(rel(got[t], want[t]) for t in range(len(toks))) < 3 * BF16_TOL, sizes


def test_interleaved_requests_and_reused_slots():
    """Three requests of unequal length take turns in portions; each equals its run alone.  Then more requests than
    slots pass through one after the other: a slot that held another sequence behaves like a fresh one."""
    cfg = cfg_a()
    engine, W = build(cfg, torch.float32, n_slots=3)
    reqs = {k: tokens_for(cfg, n, seed=10 + i) for i, (k, n) in enumerate([("x", 31), ("y", 9), ("z", 50)])}
    alone = {k: run_schedule(engine, "alone", t, [len(t)]) for k, t in reqs.items()}
    at = {k: 0 for k in reqs}
    outs = {k: [] for k in reqs}
    sizes = {"x": [4, 1, 9], "y": [2], "z": [17, 3, 1]}
    turn = 0
    while any(at[k] < len(reqs[k]) for k in reqs):
        for k in reqs:
            if at[k] >= len(reqs[k]):
                continue
            c = min(sizes[k][turn % len(sizes[k])], len(reqs[k]) - at[k])
            end = [k] if at[k] + c == len(reqs[k]) else []
            outs[k].append(engine.step([{"id": k, "tokens": reqs[k][at[k]:at[k] + c], "want": list(range(c))}], end)[0].cpu())
            at[k] += c
        turn += 1
    for k in reqs:
        assert rel(torch.cat(outs[k]), alone[k]) < 2e-5, k
    before = engine.pool.reused
    for i in range(7):
        t = tokens_for(cfg, 12 + i, seed=30 + i)
        got = run_schedule(engine, f"s{i}", t, cuts_of(len(t), [5, 1, 2]))
        assert rel(got, O.forward(cfg, W, t)) < F32_TOL, i
    assert engine.pool.reused > before and engine.pool.free_slots() == 3


def test_a_long_prompt_in_one_portion_and_in_pieces():
    """600 tokens: the recurrences without the delta rule take the chunk-parallel path in the whole-prompt run and
    the sequential one in the small portions; both match the plain model."""
    cfg = cfg_a()
    engine, W = build(cfg, torch.float32)
    toks = tokens_for(cfg, 600, seed=8)
    want = O.forward(cfg, W, toks)
    whole = run_schedule(engine, "w", toks, [600])
    parts = run_schedule(engine, "p", toks, cuts_of(600, [100, 3, 270, 1]))
    assert rel(whole, parts) < 2e-5
    assert max(rel(whole[t], want[t]) for t in range(0, 600, 7)) < 4 * F32_TOL


@pytest.mark.parametrize("dtype,tol", [(torch.float32, F32_TOL), (torch.bfloat16, BF16_TOL)])
def test_long_prompt_on_the_prompt_kernels(dtype, tol):
    """500 tokens of a model whose shapes select the tiled attention kernel and the chunk-parallel scans, whole and cut
    inside blocks and chunks, then decoded tokens, against the plain model."""
    cfg = cfg_c()
    engine, W = build(cfg, dtype)
    toks = tokens_for(cfg, 520, seed=6)
    want = O.forward(cfg, W, toks)
    for cuts in ([500] + [1] * 20, [130, 270, 3, 97] + [1] * 20):
        got = run_schedule(engine, "r", toks, cuts)
        assert max(rel(got[t], want[t]) for t in list(range(0, 520, 9)) + list(range(495, 520))) < 4 * tol, cuts[:4]


def test_long_decoding_across_many_blocks():
    cfg = cfg_b()                      # block of 5 positions: 120 decoded tokens pass 24 block edges
    engine, W = build(cfg, torch.float32)
    toks = tokens_for(cfg, 130, seed=5)
    want = O.forward(cfg, W, toks)
    got = run_schedule(engine, "d", toks, [10] + [1] * 120)
    assert max(rel(got[t], want[t]) for t in range(len(toks))) < 4 * F32_TOL


def test_greedy_generation_through_the_scheduler():
    """Engine.add_request / run: several requests, fewer slots than requests, prompts longer than a prefill portion;
    tokens equal greedy decoding with the plain model."""
    cfg = cfg_a()
    engine, W = build(cfg, torch.float32, n_slots=2, prefill_chunk=7)
    prompts = {i: tokens_for(cfg, n, seed=40 + i) for i, n in enumerate([5, 19, 1, 12])}
    for i, p in prompts.items():
        engine.add_request(i, p, max_new_tokens=6)
    got = engine.run()
    assert engine.pool.free_slots() == 2 and not engine.live and not engine.waiting
    for i, p in prompts.items():
        seq = list(p)
        for _ in range(6):
            logits = O.forward(cfg, W, seq)[-1]
            top = torch.topk(logits, 2).values
            assert float(top[0] - top[1]) > 1e-3, "test model has a near-tie: pick another seed"
            seq.append(int(torch.argmax(logits)))
        assert got[i] == seq[len(p):], i
    again = engine.generate(prompts[1], 6)
    assert again == prompts[1] + got[1]


def test_sampled_generation_runs_and_respects_eos():
    cfg = cfg_b()
    engine, _ = build(cfg, torch.bfloat16)
    torch.manual_seed(0)
    out = engine.generate(tokens_for(cfg, 9), 12, temperature=0.8, top_k=5)
    assert len(out) == 21 and all(0 <= t < cfg["vocab"] for t in out)
    first = engine.generate(tokens_for(cfg, 9), 4)[9]
    assert engine.generate(tokens_for(cfg, 9), 12, eos_id=first) == tokens_for(cfg, 9) + [first]


def test_registry_loads_a_saved_model(tmp_path):
    import json

    P, _, _ = _pkg()
    from lit_llama_b200.checkpoint_io import write_safetensors

    cfg = cfg_b()
    W = O.random_weights(cfg, seed=9)
    write_safetensors(str(tmp_path / "model.safetensors"), W)
    (tmp_path / "config.json").write_text(json.dumps({k: v for k, v in cfg.items()}))
    model = P.load_model(str(tmp_path), dtype=torch.float32, device=DEV, max_positions=64)
    assert isinstance(model, P.Lugovik)
    engine = P.Engine(model, n_slots=1)
    toks = tokens_for(cfg, 11)
    assert rel(run_schedule(engine, "r", toks, [11]), O.forward(cfg, {k: v.double() for k, v in W.items()}, toks)) < F32_TOL


# ----------------------------------------------------------------------------- mechanisms alone
def _ctx(T, slot=0, pos0=0, dtype=torch.float32, state=None):
    _, _, M = _pkg()
    meta = torch.tensor([slot, pos0], dtype=torch.int32, device=DEV)
    return M.StepContext(T, meta, state or {}, dtype)


def _scan_call(q, k, v, decay, state, *, beta=None, vscale=None, skip=None, qk_heads=None, q_mult=1.0, slot=0):
    """q, k [T, Hq, K], v [T, H, V] f32 on the device; state [slots, H, V, K]."""
    _, S, M = _pkg()
    T, H, V = v.shape
    K = q.shape[2]
    out = torch.empty((T, H * V), dtype=torch.float32, device=DEV)
    ctx = _ctx(T, slot=slot, state={"S": state})
    M._scan(ctx, q=M._p(q), ldq=q.shape[1] * K, k=M._p(k), ldk=k.shape[1] * K, v=M._p(v), ldv=H * V, q_mult=q_mult,
            decay=M._p(decay), ldd=decay.shape[1] * (decay.shape[2] if decay.dim() == 3 else 1), per_channel=decay.dim() == 3,
            beta=M._p(beta), ldb=H, vscale=M._p(vscale), ldvs=H, skip=M._p(skip), state=state, out=M._p(out), ldo=H * V, heads=H,
            qk_heads=qk_heads or q.shape[1], K=K, V=V)
    return out.view(T, H, V)


@pytest.mark.parametrize("K,V,H,G", [(16, 8, 2, 2), (20, 28, 4, 2), (72, 5, 1, 1), (128, 64, 2, 1), (200, 33, 1, 1), (1, 1, 1, 1)])
def test_delta_rule_scan_alone(K, V, H, G):
    T = 37
    q, k = torch.randn(T, G, K), O.unit(torch.randn(T, G, K))
    v, beta = torch.randn(T, H, V), torch.randn(T, H)
    g = torch.rand(T, H, K) * 0.5 + 0.5
    want = torch.stack([O.delta_rule_head(q[:, h // (H // G)].double(), k[:, h // (H // G)].double(), v[:, h].double(),
                                          torch.sigmoid(beta[:, h].double()), g[:, h].double()) for h in range(H)], dim=1)
    state = torch.zeros(2, H, V, K, device=DEV)
    dq, dk, dv, dg, db = (t.to(DEV).contiguous() for t in (q, k, v, g, beta))
    got = _scan_call(dq, dk, dv, dg, state, beta=db, qk_heads=G, slot=1)
    assert rel(got, want) < 2e-5
    assert float(state[0].abs().max()) == 0.0          # the other slot is untouched
    # the same tokens in two portions continue from the carried state
    state.zero_()
    a = _scan_call(dq[:13].contiguous(), dk[:13].contiguous(), dv[:13].contiguous(), dg[:13].contiguous(), state, beta=db[:13].contiguous(), qk_heads=G)
    b = _scan_call(dq[13:].contiguous(), dk[13:].contiguous(), dv[13:].contiguous(), dg[13:].contiguous(), state, beta=db[13:].contiguous(), qk_heads=G)
    assert rel(torch.cat([a, b]), want) < 2e-5


@pytest.mark.parametrize("K,V,H,G,per_channel", [(24, 40, 2, 2, True), (8, 8, 1, 1, True), (24, 12, 4, 2, False), (64, 80, 2, 1, False)])
def test_decayed_outer_product_scan_alone(K, V, H, G, per_channel):
    T = 77                             # above 64 tokens wide heads take the two-columns-per-lane form
    q, k, v = torch.randn(T, G, K), torch.randn(T, G, K) * 0.3, torch.randn(T, H, V)
    a = torch.rand(T, H, K) * 0.4 + 0.6 if per_channel else torch.rand(T, H) * 0.4 + 0.6
    dt, D = torch.rand(T, H) + 0.1, torch.randn(H)
    want = []
    for h in range(H):
        j = h // (H // G)
        y = O.decayed_outer_head(q[:, j].double() * 0.5, k[:, j].double(), (dt[:, h, None] * v[:, h]).double(), a[:, h].double())
        want.append(y + D[h].double() * v[:, h].double())
    want = torch.stack(want, dim=1)
    state = torch.zeros(1, H, V, K, device=DEV)
    got = _scan_call(q.to(DEV), k.to(DEV), v.to(DEV), a.to(DEV).contiguous(), state, vscale=dt.to(DEV), skip=D.to(DEV), qk_heads=G, q_mult=0.5)
    assert rel(got, want) < 2e-5


@pytest.mark.parametrize("K,V,H,per_channel", [(24, 40, 2, True), (128, 64, 3, False), (7, 5, 1, True)])
def test_long_portions_run_in_parallel_chunks_and_carry_the_state(K, V, H, per_channel):
    """Portions of 256 tokens or more (no delta rule) are cut into chunks that run in parallel; the result and the
    carried state equal the token-by-token recurrence, also when a chunked portion follows another portion."""
    _, S, _ = _pkg()
    T = 700
    assert S.lib().b2l_seq_scan_chunks(300, 0) > 1 and S.lib().b2l_seq_scan_chunks(300, 1) == 1 and S.lib().b2l_seq_scan_chunks(255, 0) == 1
    q, k, v = torch.randn(T, H, K), torch.randn(T, H, K) * 0.3, torch.randn(T, H, V)
    a = torch.rand(T, H, K) * 0.2 + 0.8 if per_channel else torch.rand(T, H) * 0.2 + 0.8
    want = torch.stack([O.decayed_outer_head(q[:, h].double(), k[:, h].double(), v[:, h].double(), a[:, h].double()) for h in range(H)], dim=1)
    for cuts in ([T], [300, 400], [1, 699], [37, 263, 1, 399]):
        state = torch.zeros(1, H, V, K, device=DEV)
        outs, at = [], 0
        for c in cuts:
            outs.append(_scan_call(dev(q[at:at + c]), dev(k[at:at + c]), dev(v[at:at + c]), dev(a[at:at + c]), state))
            at += c
        assert rel(torch.cat(outs), want) < 2e-5, cuts


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps,C", [(1, 8), (2, 5), (3, 64), (4, 130)])
def test_causal_convolution_carries_its_inputs(taps, C, dtype):
    _, S, M = _pkg()
    T = 75
    x = torch.randn(T, C).to(dtype)
    w, b = (torch.randn(C, taps) * 0.5).to(dtype), torch.randn(C).to(dtype)
    want = O.silu(O.causal_conv(x.double(), w.double(), b.double()))
    for cuts in ([T], [1] * T, [2, 40, 1, 32], [33, 42]):
        state = torch.zeros(2, taps - 1, C, dtype=dtype, device=DEV)
        outs, at = [], 0
        for c in cuts:
            xin = dev(x[at:at + c])
            out = torch.empty(c, C, dtype=torch.float32, device=DEV)
            ctx = _ctx(c, slot=1, dtype=dtype)
            S.check(S.lib().b2l_seq_conv_silu(M._p(xin), C, M._p(dev(w)), M._p(dev(b)), M._p(state), M._p(ctx.meta), M._p(out), C, c, C, taps,
                                              ctx.act, ctx.stream), "conv")
            outs.append(out)
            at += c
        assert rel(torch.cat(outs), want) < 1e-5, cuts
        if taps > 1:                                   # a single tap carries nothing
            assert float(state[0].abs().max()) == 0.0
            assert torch.equal(state[1].cpu(), x[T - (taps - 1):])


def _attention_call(q, k, v, pos0, block, cache_k, cache_v, *, scale, softcap, sink=True, gate=None, mult=1.0, dtype=torch.float32):
    """q [T, H, K] f32, k [T, G, K], v [T, G, V] in dtype; caches [1, block, G, K|V]."""
    _, S, M = _pkg()
    T, H, K = q.shape
    G, V = k.shape[1], v.shape[2]
    out = torch.empty(T, H * V, dtype=dtype, device=DEV)
    ctx = _ctx(T, pos0=pos0, dtype=dtype)
    a = S.AttnArgs(q=M._p(q), k_new=M._p(k), v_new=M._p(v), ldv=G * V, cache_k=M._p(cache_k), cache_v=M._p(cache_v), meta=M._p(ctx.meta),
                   gate=M._p(gate), ldg=H, out=M._p(out), ldo=H * V, scale=scale, softcap=softcap or 0.0, out_mult=mult, has_sink=int(sink),
                   block=block, T=T, heads=H, kv_heads=G, K=K, V=V, act_dtype=ctx.act)
    S.check(S.lib().b2l_seq_block_attention(C.byref(a), ctx.stream), "attention")
    return out.view(T, H, V).float()


@pytest.mark.parametrize("H,G,K,V,block,dtype", [
    (4, 2, 24, 16, 8, torch.float32), (2, 2, 12, 36, 5, torch.float32), (6, 2, 80, 96, 37, torch.float32), (1, 1, 128, 256, 64, torch.float32),
    (3, 3, 7, 3, 1, torch.float32), (2, 1, 32, 32, 8, torch.float32), (4, 2, 64, 64, 50, torch.bfloat16), (8, 2, 128, 128, 100, torch.float32),
    (8, 8, 40, 128, 300, torch.bfloat16), (2, 2, 12, 36, 5, torch.bfloat16)])
def test_block_attention_alone_whole_and_through_the_ring(H, G, K, V, block, dtype):
    """Both kernels (the tiled one for prompt portions with value sizes 32..128, the warp-per-query one otherwise and
    for single tokens), whole, token by token and in ragged portions, with stale ring entries that must never be read."""
    T = 150
    q, k, v = torch.randn(T, H, K), torch.randn(T, G, K).to(dtype).float(), torch.randn(T, G, V).to(dtype).float()
    gate = torch.randn(T, H)
    pos = torch.arange(T)
    want = O.chunked_sink_attention(q.double(), k.double(), v.double(), pos, 0.4, 3.0, block) * torch.sigmoid(gate.double())[:, :, None] * 0.7
    gate = gate.to(dtype).float()
    want = O.chunked_sink_attention(q.double(), k.double(), v.double(), pos, 0.4, 3.0, block) * torch.sigmoid(gate.double())[:, :, None] * 0.7
    dq, dk, dv, dg = q.to(DEV).contiguous(), k.to(DEV, dtype).contiguous(), v.to(DEV, dtype).contiguous(), gate.to(DEV, dtype).contiguous()
    tol = 1e-5 if dtype == torch.float32 else 4e-3          # bf16: only the output is rounded
    for cuts in ([T], [1] * T, cuts_of(T, [2, 9, 1, 40, 3]), [70, 80]):
        ck, cv = torch.full((1, block, G, K), 1e4, device=DEV, dtype=dtype), torch.full((1, block, G, V), 1e4, device=DEV, dtype=dtype)
        outs, at = [], 0
        for c in cuts:
            outs.append(_attention_call(dq[at:at + c].contiguous(), dk[at:at + c].contiguous(), dv[at:at + c].contiguous(), at, block, ck, cv,
                                        scale=0.4, softcap=3.0, gate=dg[at:at + c].contiguous(), mult=0.7, dtype=dtype))
            at += c
        assert rel(torch.cat(outs), want) < tol, cuts[:4]


@pytest.mark.parametrize("decode", [False, True])
def test_a_key_one_place_outside_the_block_is_not_seen_and_the_first_one_inside_is(decode):
    """One key gets a score that dwarfs all others.  Placed on the first position of the query's block it owns the
    output; placed one position earlier (the last of the previous block) it must not matter at all."""
    H = G = 1
    K, V, block, T = 16, 8, 10, 40
    torch.manual_seed(5)
    base_k, v = torch.randn(T, G, K) * 0.1, torch.randn(T, G, V)
    qdir = torch.nn.functional.normalize(torch.randn(K), dim=0)
    q = qdir.repeat(T, 1).view(T, H, K) * 4.0
    for hot, seen_by in ((30, range(30, 40)), (29, range(20, 30))):
        k = base_k.clone()
        k[hot, 0] = qdir * 8.0                       # score 32 * scale against scores of order one
        want = O.chunked_sink_attention(q.double(), k.double(), v.double(), torch.arange(T), 1.0, None, block)
        ck, cv = torch.zeros(1, block, G, K, device=DEV), torch.zeros(1, block, G, V, device=DEV)
        cuts = [25] + [1] * 15 if decode else [T]
        outs, at = [], 0
        for c in cuts:
            outs.append(_attention_call(q[at:at + c].to(DEV).contiguous(), k[at:at + c].to(DEV).contiguous(), v[at:at + c].to(DEV).contiguous(), at,
                                        block, ck, cv, scale=1.0, softcap=None))
            at += c
        got = torch.cat(outs).cpu()
        assert rel(got, want) < 1e-5
        for t in range(T):
            owned = float((got[t, 0] - v[hot, 0]).norm() / v[hot, 0].norm()) < 1e-3
            assert owned == (t in seen_by and t >= hot), (hot, t)


def test_the_sink_takes_its_share():
    """One key with score 0: weights are 1/2 with the sink, 1 without; very negative scores leave nothing."""
    q, k, v = torch.zeros(1, 1, 8, device=DEV), torch.randn(1, 1, 8, device=DEV), torch.randn(1, 1, 4, device=DEV)
    ck, cv = torch.zeros(1, 4, 1, 8, device=DEV), torch.zeros(1, 4, 1, 4, device=DEV)
    assert rel(_attention_call(q, k, v, 0, 4, ck, cv, scale=1.0, softcap=None, sink=True), 0.5 * v) < 1e-6
    assert rel(_attention_call(q, k, v, 0, 4, ck, cv, scale=1.0, softcap=None, sink=False), v) < 1e-6
    got = _attention_call(-k * 100, k, v, 0, 4, ck, cv, scale=1.0, softcap=None, sink=True)
    assert float(got.abs().max()) < 1e-20
    capped = _attention_call(-k * 100, k, v, 0, 4, ck, cv, scale=1.0, softcap=2.0, sink=True)      # tanh saturates at -2
    assert rel(capped, v * math.exp(-2.0) / (1 + math.exp(-2.0))) < 1e-5


@pytest.mark.parametrize("rot", [{"base": 1000.0, "dims": 16, "scaling": {"factor": 4.0, "original": 16, "fast": 8.0, "slow": 1.0}},
                                 {"base": 20000.0, "dims": 24}, {"base": 10.0, "dims": 2, "scaling": {"factor": 32.0, "original": 4096, "fast": 32.0, "slow": 1.0}}])
def test_head_norm_and_rotation(rot):
    _, S, M = _pkg()
    T, H, K, pos0 = 9, 3, 24, 1000
    x, w = torch.randn(T, H, K), torch.rand(K) + 0.5
    want = O.rotate(O.rms_norm(x.double(), w.double(), 1e-5), torch.arange(pos0, pos0 + T), rot)
    f, mult = M.rope_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
    fo, mo = O.rope_frequencies(rot)
    assert rel(f, fo) < 1e-7 and abs(mult - mo) < 1e-12
    out = torch.empty(T, H * K, device=DEV)
    ctx = _ctx(T, pos0=pos0)
    S.check(S.lib().b2l_seq_headnorm_rope(M._p(dev(x)), H * K, M._p(dev(w)), 1e-5, M._p(dev(f)), rot["dims"], mult, M._p(ctx.meta), M._p(out), 1,
                                          T, H, K, ctx.act, ctx.stream), "rope")
    assert rel(out.view(T, H, K), want) < 2e-5     # f32 angles at position ~1000


@pytest.mark.parametrize("D", [50, 1030, 2048, 3000, 5000])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_post_norm_residual_pre_norm_all_widths(D, dtype):
    _, S, M = _pkg()
    T = 3
    ctx = _ctx(T, dtype=dtype)
    x, y, w1, w2 = torch.randn(T, D), (torch.randn(T, D) * 3).to(dtype), (torch.rand(D) + 0.5).to(dtype), (torch.rand(D) + 0.5).to(dtype)
    for nxt in (True, False):
        dx, h = dev(x.clone()), torch.zeros(T, D, device=DEV, dtype=dtype)
        S.check(S.lib().b2l_seq_norm_add_norm(M._p(dev(y)), M._p(dev(w1)), 1e-5, M._p(dx), M._p(dev(w2)) if nxt else None, M._p(h) if nxt else None, T, D,
                                              ctx.act, ctx.stream), "nan")
        x2 = x.double() + O.rms_norm(y.double(), w1.double(), 1e-5)
        assert rel(dx, x2) < 1e-6
        if nxt:
            assert rel(h, O.rms_norm(x2, w2.double(), 1e-5)) < (1e-6 if dtype == torch.float32 else 4e-3)


@pytest.mark.parametrize("group,n", [(12, 48), (512, 1024), (2000, 2000)])
def test_grouped_read_out_norm_small_and_large_groups(group, n):
    _, S, M = _pkg()
    T = 4
    ctx = _ctx(T)
    o, gate, wn = torch.randn(T, n), torch.randn(T, n), torch.rand(n) + 0.5
    res = torch.empty(T, n, device=DEV)
    S.check(S.lib().b2l_seq_group_norm_gate(M._p(dev(o)), n, M._p(dev(wn)), 0, M._p(dev(gate)), n, S.ACT_SILU, 1, 1e-5, 0.5, M._p(res), n, T, n, group, ctx.act,
                                            ctx.stream), "gng")
    ref = O.rms_norm((o.double() * O.silu(gate.double())).view(T, n // group, group), None, 1e-5).reshape(T, n) * wn.double() * 0.5
    assert rel(res, ref) < 1e-6


@pytest.mark.parametrize("F,dtype", [(33, torch.float32), (64, torch.float32), (4096, torch.bfloat16), (40, torch.bfloat16), (36, torch.bfloat16)])
def test_gated_activation_both_forms(F, dtype):
    _, S, M = _pkg()
    T = 5
    ctx = _ctx(T, dtype=dtype)
    gu = (torch.randn(T, 2 * F) * 3).to(dtype)
    mid = torch.empty(T, F, device=DEV, dtype=dtype)
    for act, fn in ((S.ACT_GELU_TANH, O.gelu_tanh), (S.ACT_SILU, O.silu)):
        S.check(S.lib().b2l_seq_gated_act(M._p(dev(gu)), 2 * F, M._p(mid), T, F, act, 0.0, ctx.act, ctx.stream), "act")
        assert rel(mid, fn(gu[:, :F].double()) * gu[:, F:].double()) < (1e-6 if dtype == torch.float32 else 4e-3)


def test_row_kernels():
    """Embedding scale, RMS norm with row selection, post-norm + residual + next pre-norm, gated activation, grouped
    read-out norm with its gate in both orders, both decay forms (including arguments where exp or sigmoid saturate)."""
    _, S, M = _pkg()
    lib, T, D = S.lib(), 6, 50
    ctx = _ctx(T)
    x, y, w1, w2 = torch.randn(T, D), torch.randn(T, D) * 3, torch.rand(D) + 0.5, torch.rand(D) + 0.5
    dx, h = x.to(DEV), torch.empty(T, D, device=DEV)
    S.check(lib.b2l_seq_norm_add_norm(M._p(dev(y)), M._p(dev(w1)), 1e-5, M._p(dx), M._p(dev(w2)), M._p(h), T, D, ctx.act, ctx.stream), "nan")
    x2 = x.double() + O.rms_norm(y.double(), w1.double(), 1e-5)
    assert rel(dx, x2) < 1e-6 and rel(h, O.rms_norm(x2, w2.double(), 1e-5)) < 1e-6
    rows = torch.tensor([4, 0, 4], dtype=torch.int32, device=DEV)
    out = torch.empty(3, D, device=DEV)
    S.check(lib.b2l_seq_rmsnorm(M._p(dx), M._p(dev(w1)), 1e-5, M._p(out), M._p(rows), 3, D, ctx.act, ctx.stream), "norm")
    assert rel(out, O.rms_norm(x2[[4, 0, 4]], w1.double(), 1e-5)) < 1e-6
    gu = torch.randn(T, 2 * 33) * 3
    mid = torch.empty(T, 33, device=DEV)
    S.check(lib.b2l_seq_gated_act(M._p(dev(gu)), 66, M._p(mid), T, 33, S.ACT_GELU_TANH, 0.0, ctx.act, ctx.stream), "act")
    assert rel(mid, O.gelu_tanh(gu[:, :33].double()) * gu[:, 33:].double()) < 1e-6
    tab, tok = torch.randn(11, D), torch.tensor([3, 10, 0, 3, 7, 1])
    emb = torch.empty(T, D, device=DEV)
    S.check(lib.b2l_seq_embed(M._p(dev(tok)), 1, M._p(dev(tab)), ctx.act, 2.5, M._p(emb), T, D, 11, ctx.stream), "embed")
    assert torch.equal(emb.cpu(), tab[tok] * 2.5)
    n, group = 48, 12
    o, gate, wn = torch.randn(T, n), torch.randn(T, n), torch.rand(n) + 0.5
    for shared, first, act, fn in ((1, 0, S.ACT_SIGMOID, torch.sigmoid), (0, 1, S.ACT_SILU, O.silu), (1, 0, S.ACT_SILU, O.silu)):
        res = torch.empty(T, n, device=DEV)
        wv = wn[:group] if shared else wn
        S.check(lib.b2l_seq_group_norm_gate(M._p(dev(o)), n, M._p(dev(wv)), shared, M._p(dev(gate)), n, act, first, 1e-5, 1.5, M._p(res), n, T, n,
                                            group, ctx.act, ctx.stream), "gng")
        od, gd = o.double().view(T, n // group, group), fn(gate.double()).view(T, n // group, group)
        wd = (wn[:group].double() if shared else wn.double().view(n // group, group))
        ref = O.rms_norm(od * gd, None, 1e-5) * wd if first else O.rms_norm(od, None, 1e-5) * wd * gd
        assert rel(res, 1.5 * ref.reshape(T, n)) < 1e-6
    Hh, Kk = 3, 7
    a = torch.cat([torch.randn(T - 2, Hh * Kk) * 3, torch.full((1, Hh * Kk), 60.0), torch.full((1, Hh * Kk), -60.0)])
    bias, A_log = torch.randn(Hh * Kk), torch.randn(Hh)
    dec, dt = torch.empty(T, Hh * Kk, device=DEV), torch.empty(T, Hh * Kk, device=DEV)
    S.check(lib.b2l_seq_decay(M._p(dev(a)), Hh * Kk, M._p(dev(bias)), M._p(dev(A_log)), S.DECAY_EXP_SOFTPLUS, 0.0, M._p(dec), M._p(dt), T, Hh, Kk,
                              ctx.act, ctx.stream), "decay")
    sp = O.softplus(a.double() + bias.double())
    assert rel(dt, sp) < 1e-6
    assert rel(dec, torch.exp(-torch.exp(A_log.double()).repeat_interleave(Kk) * sp)) < 1e-5
    S.check(lib.b2l_seq_decay(M._p(dev(a)), Hh * Kk, M._p(dev(bias)), None, S.DECAY_SIGMOID_ROOT, 16.0, M._p(dec), None, T, Hh, Kk, ctx.act,
                              ctx.stream), "decay")
    assert rel(dec, torch.sigmoid(a.double() + bias.double()) ** (1 / 16.0)) < 1e-6
    assert float(dec.min()) > 0.0


def test_bad_arguments_are_refused():
    _, S, M = _pkg()
    lib = S.lib()
    assert lib.b2l_seq_scan(None, None) == -1 and b"null" in lib.b2l_seq_last_error()
    assert lib.b2l_seq_conv_silu(C.c_void_p(16), 4, C.c_void_p(16), None, C.c_void_p(16), C.c_void_p(16), C.c_void_p(16), 4, 1, 4, 9, 0, None) == -2
    with pytest.raises(RuntimeError):
        S.act_code(torch.float16)
    with pytest.raises(ValueError):
        _pkg()[0].LugovikConfig.from_dict({"architecture": "Lugovik", "vocab": 1, "width": 1, "norm": {"eps": 1e-6}, "layers": [{"type": "nope"}]})


def test_llama_is_served_by_the_same_engine():
    """The package's LLaMA behind the engine: greedy tokens equal its own generate() with top_k = 1."""
    import lit_llama_b200 as P
    from gpu_util import build_tiny
    from lit_llama_b200.registry import LLaMASequenceModel

    cfg = dict(block_size=64, vocab_size=96, n_layer=2, n_head=4, n_embd=128)
    model, _, _ = build_tiny(torch.device(DEV), cfg)
    prompt = [3, 17, 40, 41, 2, 77, 5]
    want = P.generate(model, torch.tensor(prompt, dtype=torch.int64, device=DEV), 8, max_seq_length=32, top_k=1).tolist()
    model.reset_cache()
    engine = P.Engine(LLaMASequenceModel(model, 32), n_slots=1)
    assert engine.generate(prompt, 8) == want
