"""GPU: the Rinirax model family and its mechanisms against the plain restatement in tests/rinirax_oracle.py (float64),
on small random models of several shapes: each mechanism alone, whole prompts against token-by-token decoding and
portions of many sizes, interleaved requests, reused slots, loud keys far back and just inside and just outside the
window (in prompts, across portions and in decoding), the first tokens of a sequence, long decoding through the captured
step, greedy generation through the engine's scheduler."""
import ctypes as C
import json
import math

import pytest
import torch

import rinirax_oracle as O

pytestmark = pytest.mark.gpu

DEV = "cuda"
TOL = 3e-5


def _pkg():
    import lit_llama_b200 as P
    from lit_llama_b200 import _seqlib as S
    from lit_llama_b200 import mixers as M
    return P, S, M


def rel(got, want):
    got, want = got.double().cpu(), want.double().cpu()
    return float((got - want).norm() / (want.norm() + 1e-30))


# ----------------------------------------------------------------------------- configurations (none is a served model's)
def attn(heads, kv_heads, dim, vdim, scale, diff, conv=None, rot=None, kv_from=None):
    c = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if conv:
        c["conv"] = conv
    if rot:
        c["rot"] = {"base": rot[0], "dims": rot[1]}
    if kv_from is not None:
        c["kv_from"] = kv_from
    return {"type": "attention", "mixer": c}


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, window=None, base=10000.0, scaling=None):
    c = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale}
    if rot_dim:
        c["rot"] = {"base": base, "dims": rot_dim}
        if scaling:
            c["rot"]["scaling"] = scaling
    if window:
        c["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": c}


def gru(width):
    return {"type": "mingru", "mixer": {"width": width}}


def moe(experts, top, ff, count=1, keep=1, scale=None):
    r = {"experts": experts, "top": top}
    if count > 1:
        r["groups"] = {"count": count, "keep": keep}
    if scale is not None:
        r["scale"] = scale
    return {"kind": "moe", "expert": {"ff": ff}, "router": r}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def with_mlp(layer, mlp):
    return dict(layer, mlp=mlp)


YARN = {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0}


def cfg_a():
    """Odd sizes; a recurrent layer first; partial rotation; four taps; two layers that read the keys and values of layer 1;
    three groups of which two are kept; a window of 7; a layer without feed-forward."""
    return {"architecture": "Rinirax", "vocab": 131, "width": 72, "norm": {"eps": 1e-5}, "layers": [
        with_mlp(gru(40), dense(50)),
        with_mlp(attn(6, 2, 10, 12, 0.3, 0.3, conv=4, rot=(1000.0, 6)), moe(6, 2, 40, count=3, keep=2, scale=2.5)),
        with_mlp(latent(3, 12, 8, 10, 20, 24, 0.2, window=7, base=5000.0, scaling=YARN), None),
        with_mlp(attn(6, 2, 10, 12, 0.25, 0.3, conv=4, rot=(1000.0, 6), kv_from=1), moe(5, 3, 24, scale=0.5)),
        with_mlp(attn(2, 2, 8, 6, 0.35, 0.7, conv=2), dense(30)),
        with_mlp(attn(6, 2, 10, 12, 0.3, 0.1, conv=2, rot=(1000.0, 6), kv_from=1), moe(8, 2, 16, count=4, keep=1)),
    ]}


def cfg_b():
    """Shapes that take the tiled attention kernel, the expanded latent form, the chunked recurrence and the sorted expert
    path: 16-byte rows, portions of hundreds of tokens; windows of 40 and 150."""
    return {"architecture": "Rinirax", "vocab": 200, "width": 128, "norm": {"eps": 1e-6}, "layers": [
        with_mlp(attn(6, 2, 24, 48, 0.14, 0.45, conv=3, rot=(3e5, 24)), moe(8, 3, 64, count=4, keep=2, scale=1.25)),
        with_mlp(latent(4, 32, 16, 32, 48, 64, 0.1, window=40, base=2e5, scaling={"factor": 6.0, "original": 128, "fast": 24.0, "slow": 1.0}), dense(160)),
        with_mlp(gru(96), moe(8, 2, 64, count=2, keep=1)),
        with_mlp(attn(6, 2, 24, 48, 0.14, 0.45, conv=3, rot=(3e5, 24), kv_from=0), moe(8, 3, 64, count=4, keep=2, scale=1.25)),
        with_mlp(latent(2, 16, 16, 48, 32, 40, 0.15, window=150), None),
    ]}


def cfg_c():
    """What a served model may happen to make equal or one: one head, kv heads = heads, no convolution, no rotation, one
    tap, one expert per token, no groups, every group kept, a window of one position, a window longer than any prompt, no
    window at all, no YaRN, no rotated part, no router scale, no selection bias."""
    return {"architecture": "Rinirax", "vocab": 90, "width": 64, "norm": {"eps": 1e-6}, "layers": [
        with_mlp(attn(1, 1, 16, 16, 0.25, 0.8), moe(4, 1, 24)),
        with_mlp(latent(2, 8, 8, 8, 16, 16, 0.25, window=1), moe(6, 2, 16, count=3, keep=3)),
        with_mlp(attn(4, 4, 8, 16, 0.3, 0.2, conv=1, rot=(100.0, 8)), dense(40)),
        with_mlp(latent(2, 16, 4, 8, 12, 20, 0.2, window=100000), None),
        with_mlp(latent(3, 8, 0, 16, 16, 8, 0.3), moe(4, 4, 8, count=2, keep=2, scale=1.0)),
        with_mlp(gru(64), None),
        with_mlp(attn(4, 4, 8, 16, 0.3, 0.5, conv=3, kv_from=2), None),
        with_mlp(latent(1, 8, 8, 8, 8, 8, 0.3), dense(16)),
    ]}


CONFIGS = {"a": cfg_a, "b": cfg_b, "c": cfg_c}


def random_weights(cfg, seed=1, no_bias=()):
    """bf16-representable float32 tensors on the CPU under the family's tensor names.  no_bias: layers whose experts get no
    selection bias tensor."""
    g = torch.Generator().manual_seed(seed)
    D, W = cfg["width"], {}

    def rnd(*shape, std=1.0, mean=0.0):
        return (mean + std * torch.randn(*shape, generator=g)).bfloat16().float()

    def lin(o, i, gain=1.0):
        return rnd(o, i, std=gain / math.sqrt(i))

    W["embed"], W["head"] = rnd(cfg["vocab"], D), lin(cfg["vocab"], D)
    W["final.norm"], W["final.norm.b"] = rnd(D, std=0.2, mean=1.0), rnd(D, std=0.2)
    for i, layer in enumerate(cfg["layers"]):
        p, m, c = f"l{i}.", f"l{i}.mix.", layer["mixer"]
        W[p + "norm1"], W[p + "norm1.b"] = rnd(D, std=0.2, mean=1.0), rnd(D, std=0.2)
        if layer["type"] == "attention":
            H, G, K, V = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
            parts = {"q": H * 2 * K} if c.get("kv_from") is not None else {"q": H * 2 * K, "k": G * 2 * K, "v": G * V}
            for n, rows in parts.items():
                W[m + n], W[m + n + ".b"] = lin(rows, D, 2.0 if n != "v" else 1.0), rnd(rows, std=0.3)
                if c.get("conv"):
                    W[m + n + ".conv"] = rnd(rows, c["conv"], std=0.6)
            for n in ("lq1", "lk1", "lq2", "lk2"):
                W[m + n] = rnd(K, std=0.35)
            W[m + "o"] = lin(D, H * V)
        elif layer["type"] == "mingru":
            n = c["width"]
            W[m + "z"], W[m + "x"], W[m + "g"], W[m + "o"] = lin(n, D, 2.0), lin(n, D, 2.0), lin(n, D), lin(D, n)
            W[m + "z.b"], W[m + "x.b"] = rnd(n, std=0.7), rnd(n, std=0.7)
        else:
            H, dn, dr, dv, rq, rk = c["heads"], c["dim"], c["rot_dim"], c["vdim"], c["q_rank"], c["kv_rank"]
            W[m + "dq"], W[m + "dq.norm"], W[m + "uq"] = lin(rq, D), rnd(rq, std=0.3, mean=1.5), lin(H * (dn + dr), rq, 2.0)
            W[m + "dkv"], W[m + "dkv.norm"] = lin(rk + dr, D, 2.0), rnd(rk, std=0.3, mean=1.5)
            W[m + "uk"], W[m + "uv"], W[m + "o"] = lin(H * dn, rk, 2.0), lin(H * dv, rk), lin(D, H * dv)
        f = layer.get("mlp")
        if f and f["kind"] == "dense":
            W[p + "mlp.up"], W[p + "mlp.down"], W[p + "mlp.act"] = lin(f["ff"], D, 1.5), lin(D, f["ff"]), rnd(2, std=0.8)
        elif f:
            E, ff = f["router"]["experts"], f["expert"]["ff"]
            W[p + "mlp.router"] = lin(E, D, 3.0)
            if i not in no_bias:
                W[p + "mlp.correction"] = rnd(E, std=0.15)
            for e in range(E):
                q = f"{p}mlp.e{e}."
                W[q + "gate"], W[q + "up"], W[q + "down"] = lin(ff, D, 2.0), lin(ff, D, 2.0), lin(D, ff)
        d = 0.3 * torch.randn(i + 2, generator=g)
        d[-1] += 1.0
        W[p + "dwa"] = d.bfloat16().float()
    return W


def build(cfg, dtype, seed=1, n_slots=3, max_positions=512, no_bias=()):
    P, S, M = _pkg()
    W = random_weights(cfg, seed, no_bias)
    model = P.Rinirax(P.RiniraxConfig.from_dict(cfg), {k: v.to(DEV, dtype) for k, v in W.items()}, max_positions=max_positions)
    return model, P.Engine(model, n_slots=n_slots), W


def tokens_of(cfg, n, seed=5):
    return torch.randint(0, cfg["vocab"], (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def run_whole(engine, toks, rid="w"):
    return engine.step([{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], [rid])[0]


def run_pieces(engine, toks, sizes, rid="p"):
    """The prompt in portions of the given sizes (cycled), every position's logits."""
    outs, at, i = [], 0, 0
    while at < len(toks):
        n = min(sizes[i % len(sizes)], len(toks) - at)
        outs.append(engine.step([{"id": rid, "tokens": toks[at:at + n], "want": list(range(n))}], [rid] if at + n == len(toks) else [])[0])
        at, i = at + n, i + 1
    return torch.cat(outs)


# ----------------------------------------------------------------------------- whole models against the oracle
@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_model_matches_the_oracle_layer_by_layer_f32(name):
    cfg = CONFIGS[name]()
    model, engine, W = build(cfg, torch.float32, no_bias=(4,) if name == "c" else ())
    toks = tokens_of(cfg, 100 if name == "b" else 45)
    cap = []
    want = O.model(toks, cfg, W, capture=cap)
    model.capture_layers = []
    got = run_whole(engine, toks)
    assert len(model.capture_layers) == len(cap) == len(cfg["layers"])
    for i, (g, w) in enumerate(zip(model.capture_layers, cap)):
        assert rel(g, w) < TOL, (name, "layer", i, rel(g, w))
    assert rel(got, want) < TOL


@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_model_bf16_is_close_to_the_oracle(name):
    cfg = CONFIGS[name]()
    model, engine, W = build(cfg, torch.bfloat16)
    toks = tokens_of(cfg, 60)
    want = O.model(toks, cfg, W)
    got = run_whole(engine, toks)
    assert rel(got, want) < 0.12, rel(got, want)
    again = run_pieces(engine, toks, [7, 1, 2, 13])
    per_token = (again.double() - got.double()).norm(dim=-1) / got.double().norm(dim=-1)
    assert int((per_token > 0.06).sum()) <= 3, per_token      # a routing flip on a close call moves one token a lot, rounding none


@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_portions_and_single_tokens_equal_the_whole_prompt(name):
    cfg = CONFIGS[name]()
    n = 420 if name == "b" else 80          # b: several query tiles, chunks of the recurrence, windows that start in older portions
    model, engine, W = build(cfg, torch.float32)
    toks = tokens_of(cfg, n)
    whole = run_whole(engine, toks)
    if name != "b":
        assert rel(whole, O.model(toks, cfg, W)) < TOL
    for sizes in ([1], [2], [3, 2, 17, 1, 5], [33, 64], [n - 9, 1, 1, 2]):
        if name == "b" and sizes == [1]:
            sizes = [n - 170, 1]            # a long first portion, then 170 tokens one by one: both windows pass over decoded tokens
        got = run_pieces(engine, toks, sizes)
        assert rel(got, whole) < TOL, (name, sizes, rel(got, whole))


def test_long_prompt_matches_the_oracle():
    cfg = cfg_b()
    model, engine, W = build(cfg, torch.float32)
    toks = tokens_of(cfg, 300, seed=9)
    want = O.model(toks, cfg, W)
    assert rel(run_whole(engine, toks), want) < TOL
    assert rel(run_pieces(engine, toks, [261, 1, 2, 1, 1]), want) < TOL


def test_interleaved_requests_and_reused_slots():
    cfg = cfg_a()
    model, engine, W = build(cfg, torch.float32, n_slots=2)
    prompts = [tokens_of(cfg, n, seed=s) for n, s in ((23, 1), (5, 2), (41, 3), (1, 4), (12, 5))]
    alone = [run_whole(engine, p, rid=("alone", i)) for i, p in enumerate(prompts)]
    for i, p in enumerate(prompts):
        assert rel(alone[i], O.model(p, cfg, W)) < TOL
    # two at a time in the two slots, unequal portions in turns; finished requests hand their slot to the next one
    got = {i: [] for i in range(len(prompts))}
    at = {i: 0 for i in range(len(prompts))}
    waiting, live = list(range(len(prompts))), []
    step = 0
    while waiting or live:
        while waiting and len(live) < 2:
            live.append(waiting.pop(0))
        for i in list(live):
            n = min([3, 1, 7, 2][step % 4], len(prompts[i]) - at[i])
            step += 1
            end = at[i] + n == len(prompts[i])
            got[i].append(engine.step([{"id": i, "tokens": prompts[i][at[i]:at[i] + n], "want": list(range(n))}], [i] if end else [])[0])
            at[i] += n
            if end:
                live.remove(i)
    assert engine.pool.reused >= 3
    for i in range(len(prompts)):
        assert rel(torch.cat(got[i]), alone[i]) < TOL, i
    # one step with several entries of unequal length against each alone
    outs = engine.step([{"id": ("m", i), "tokens": p, "want": list(range(len(p)))} for i, p in enumerate(prompts[:2])], [("m", 0), ("m", 1)])
    for i in range(2):
        assert rel(outs[i], alone[i]) < TOL


def test_long_decoding_through_the_captured_step():
    cfg = cfg_a()                            # the window of 7 passes over decoded tokens many times; the recurrence runs 200 steps
    model, engine, W = build(cfg, torch.float32)
    toks = tokens_of(cfg, 230)
    want = O.model(toks, cfg, W)
    first = engine.step([{"id": "d", "tokens": toks[:20], "want": [19]}])[0]
    outs = [first] + [engine.step([{"id": "d", "tokens": [t], "want": [0]}])[0] for t in toks[20:]]
    assert engine._graph is not None
    assert rel(torch.cat(outs), want[19:]) < TOL
    # the same captured step serves another request in another slot from its first token on
    outs2 = [engine.step([{"id": "e", "tokens": [t], "want": [0]}])[0] for t in toks[:40]]
    assert rel(torch.cat(outs2), want[:40]) < TOL


def test_first_tokens_of_a_sequence():
    """One-token and two-token sequences in a slot that another request used before: the convolution's carried rows and the
    recurrence start from zero, the first tokens see no key before position 0."""
    cfg = cfg_a()
    model, engine, W = build(cfg, torch.float32, n_slots=1)
    run_whole(engine, tokens_of(cfg, 30, seed=2))
    for toks in ([7], [7, 7], [130, 0], tokens_of(cfg, 3), tokens_of(cfg, 5)):
        want = O.model(toks, cfg, W)
        assert rel(run_whole(engine, toks), want) < TOL
        assert rel(run_pieces(engine, toks, [1]), want) < TOL
        assert rel(run_pieces(engine, toks, [2, 1]), want) < TOL
    assert engine.pool.reused >= 10


def test_position_limit_is_reported():
    P, S, M = _pkg()
    cfg = cfg_c()
    model, engine, W = build(cfg, torch.float32, max_positions=16)
    toks = tokens_of(cfg, 20)
    engine.step([{"id": "x", "tokens": toks[:16], "want": []}])
    with pytest.raises(P.state.PoolFull):
        engine.step([{"id": "x", "tokens": toks[16:], "want": [0]}])


def test_greedy_generation_through_the_scheduler():
    cfg = cfg_a()
    model, engine, W = build(cfg, torch.float32, n_slots=2)
    engine.prefill_chunk = 6
    prompts = [tokens_of(cfg, n, seed=s) for n, s in ((9, 11), (17, 12), (3, 13))]
    for i, p in enumerate(prompts):
        engine.add_request(i, p, 12)
    out = engine.run()
    for i, p in enumerate(prompts):
        seq = list(p)
        for _ in range(12):
            lg = O.model(seq, cfg, W)[-1]
            top2 = lg.topk(2).values
            if float(top2[0] - top2[1]) < 1e-3:          # a close call decides nothing about the framework
                break
            seq.append(int(lg.argmax()))
        n = len(seq) - len(p)
        assert out[i][:n] == seq[len(p):], (i, out[i], seq[len(p):])
    assert engine.generate(prompts[0], 4)[:len(prompts[0])] == prompts[0]


def test_sampled_generation_runs_and_respects_eos():
    cfg = cfg_c()
    model, engine, W = build(cfg, torch.bfloat16)
    torch.manual_seed(0)
    prompt = tokens_of(cfg, 9)
    out = engine.generate(prompt, 12, temperature=0.8, top_k=5)
    assert len(out) == 21 and all(0 <= t < cfg["vocab"] for t in out)
    first = engine.generate(prompt, 4)[9]
    assert engine.generate(prompt, 12, eos_id=first) == prompt + [first]


def test_registry_loads_a_saved_model(tmp_path):
    P, S, M = _pkg()
    from lit_llama_b200.checkpoint_io import write_safetensors

    cfg = cfg_a()
    W = random_weights(cfg, seed=3)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    write_safetensors(str(tmp_path / "model.safetensors"), {k: v.bfloat16() for k, v in W.items()})
    toks = tokens_of(cfg, 12)
    want = O.model(toks, cfg, W)
    for dtype, tol in ((torch.float32, TOL), (torch.bfloat16, 0.12)):
        model = P.load_model(str(tmp_path), dtype=dtype, device=DEV, max_positions=64)
        assert type(model).__name__ == "Rinirax" and model.max_positions == 64
        assert rel(run_whole(P.Engine(model, n_slots=1), toks), want) < tol


# ----------------------------------------------------------------------------- mechanisms alone
def _ctx(M, P, specs, T, pos0, dtype, slot=0, pool=None, n_slots=2):
    pool = pool or P.SequenceStatePool(specs, n_slots, torch.device(DEV))
    meta = torch.tensor([slot, pos0], dtype=torch.int32, device=DEV)
    return M.StepContext(T, meta, pool.tensors, dtype, pos_hint=pos0, slot_hint=slot), pool


def _run_mixer(M, P, mixer, h, sizes, dtype=torch.float32, slot=1, extra=None):
    """A mixer over h [T, width] in portions of the given sizes (cycled) in one slot of a fresh pool; `extra`: mixers that must
    run ahead of it on the same input in every step (a layer whose keys and values it reads)."""
    specs = dict(mixer.state_specs())
    for e in extra or []:
        specs.update(e.state_specs())
    pool = P.SequenceStatePool(specs, 2, torch.device(DEV))
    pool.acquire("other")
    pool.acquire("it")
    assert pool.slot("it") == slot
    outs, at, i = [], 0, 0
    while at < h.shape[0]:
        n = min(sizes[i % len(sizes)], h.shape[0] - at)
        ctx, _ = _ctx(M, P, None, n, at, dtype, slot=slot, pool=pool)
        part = h[at:at + n].to(DEV, dtype).contiguous()
        for e in extra or []:
            e.forward(part, ctx)
        outs.append(mixer.forward(part, ctx))
        at, i = at + n, i + 1
    return torch.cat(outs).float().cpu()


def _mixer_weights(layer, D, seed):
    cfg = {"vocab": 8, "width": D, "norm": {"eps": 1e-6}, "layers": [layer]}
    W = random_weights(cfg, seed)
    return {k[len("l0.mix."):]: v for k, v in W.items() if k.startswith("l0.mix.")}


def loud_rows(h, rows, factor=5.0):
    h = h.clone()
    for r in rows:
        if 0 <= r < h.shape[0]:
            h[r] *= factor
    return h.bfloat16().float()


@pytest.mark.parametrize("shape", [(6, 2, 10, 12, 4, 6), (4, 2, 40, 72, 3, 40), (2, 2, 16, 24, 0, 0), (3, 1, 64, 128, 2, 16)])
def test_differential_attention_alone_with_loud_far_keys(shape):
    P, S, M = _pkg()
    H, G, K, V, taps, rd = shape
    D, T = 48, 330
    layer = attn(H, G, K, V, 1.0 / math.sqrt(K), 0.4, conv=taps or None, rot=(700.0, rd) if rd else None)
    c = layer["mixer"]
    W = _mixer_weights(layer, D, 3)
    g = torch.Generator().manual_seed(1)
    # positions 2 and 65 are loud: they dominate queries hundreds of positions later, at a tile's and a chunk's border
    h = loud_rows(torch.randn(T, D, generator=g), [2, 65, 255, 256, 320])
    want, _ = O.differential_attention(h.double(), W, "", c, 1e-6)
    Wd = {k: v.to(DEV) for k, v in W.items()}
    mixer = M.DifferentialAttention("m", Wd, "", heads=H, kv_heads=G, dim=K, vdim=V, scale=c["scale"], diff=c["diff"], eps=1e-6, conv=c.get("conv", 0),
                                    rot=c.get("rot"), max_positions=T + 7)
    for sizes in ([T], [1], [64, 1, 2, 37], [300, 1]):
        got = _run_mixer(M, P, mixer, h, sizes)
        assert rel(got, want) < TOL, (shape, sizes, rel(got, want))
    Wb = {k: v.to(DEV, torch.bfloat16) for k, v in W.items()}
    mixer = M.DifferentialAttention("m", Wb, "", heads=H, kv_heads=G, dim=K, vdim=V, scale=c["scale"], diff=c["diff"], eps=1e-6, conv=c.get("conv", 0),
                                    rot=c.get("rot"), max_positions=T + 7)
    assert rel(_run_mixer(M, P, mixer, h, [100, 1, 29], dtype=torch.bfloat16), want) < 0.06


def test_differential_attention_over_another_layers_keys_and_values():
    P, S, M = _pkg()
    H, G, K, V, D, T = 4, 2, 8, 12, 40, 90
    src_l, dst_l = attn(H, G, K, V, 0.3, 0.4, conv=3, rot=(50.0, 8)), attn(H, G, K, V, 0.2, 0.6, conv=2, rot=(50.0, 8), kv_from=0)
    Ws, Wt = _mixer_weights(src_l, D, 5), _mixer_weights(dst_l, D, 6)
    assert "k" not in Wt and "v.conv" not in Wt
    h = torch.randn(T, D, generator=torch.Generator().manual_seed(2)).bfloat16().float()
    _, kv = O.differential_attention(h.double(), Ws, "", src_l["mixer"], 1e-6)
    want, _ = O.differential_attention(h.double(), Wt, "", dst_l["mixer"], 1e-6, kv=kv)
    kw = dict(heads=H, kv_heads=G, dim=K, vdim=V, eps=1e-6, rot={"base": 50.0, "dims": 8}, max_positions=128)
    src = M.DifferentialAttention("s", {k: v.to(DEV) for k, v in Ws.items()}, "", scale=0.3, diff=0.4, conv=3, **kw)
    dst = M.DifferentialAttention("t", {k: v.to(DEV) for k, v in Wt.items()}, "", scale=0.2, diff=0.6, conv=2, kv_from=src, **kw)
    assert set(dst.state_specs()) == {"t.conv"}
    for sizes in ([T], [1], [40, 1, 2, 5]):
        assert rel(_run_mixer(M, P, dst, h, sizes, extra=[src]), want) < TOL, sizes
    with pytest.raises(ValueError):
        M.DifferentialAttention("u", {k: v.to(DEV) for k, v in Wt.items()}, "", scale=0.2, diff=0.6, conv=2, kv_from=dst, **kw)


@pytest.mark.parametrize("shape", [(3, 12, 8, 10, 20, 24, 7), (4, 32, 16, 32, 48, 64, 40), (2, 16, 16, 48, 32, 40, 150), (2, 8, 0, 8, 8, 8, 3),
                                   (4, 64, 32, 48, 80, 128, 64)])
def test_latent_attention_window_edges_with_loud_keys(shape):
    P, S, M = _pkg()
    H, dn, dr, dv, rq, rk, win = shape
    D, T = 56, 260
    layer = latent(H, dn, dr, dv, rq, rk, 1.0 / math.sqrt(dn + dr), window=win, base=3000.0, scaling=YARN if dr else None)
    c = layer["mixer"]
    W = _mixer_weights(layer, D, 4)
    g = torch.Generator().manual_seed(3)
    # loud positions: for the queries at 200 and 259 (a portion's last token, a decoded token) the key just outside the window
    # and the one just inside it; for position win the key at 0 (the first one a window drops)
    h = loud_rows(torch.randn(T, D, generator=g), [0, 200 - win, 200 - win + 1, 259 - win, 259 - win + 1, 128])
    want = O.latent_attention(h.double(), W, "", c, 1e-6)
    Wd = {k: v.to(DEV) for k, v in W.items()}
    mixer = M.LatentAttention("m", Wd, "", heads=H, dim=dn, rot_dim=dr, vdim=dv, q_rank=rq, kv_rank=rk, scale=c["scale"], eps=1e-6, rot=c.get("rot"),
                              max_positions=T + 3, interleaved=False, window=win)
    assert mixer.sink is None
    for sizes in ([T], [1], [201, 1], [64, 1, 2, 37], [199, 2, 70]):
        got = _run_mixer(M, P, mixer, h, sizes)
        assert rel(got, want) < TOL, (shape, sizes, rel(got, want))
    # without the window the same weights give something else: the edge matters in this test
    free = dict(c)
    del free["mask"]
    assert rel(O.latent_attention(h.double(), W, "", free, 1e-6), want) > 1e-2
    Wb = {k: v.to(DEV, torch.bfloat16) for k, v in W.items()}
    mixer = M.LatentAttention("m", Wb, "", heads=H, dim=dn, rot_dim=dr, vdim=dv, q_rank=rq, kv_rank=rk, scale=c["scale"], eps=1e-6, rot=c.get("rot"),
                              max_positions=T + 3, interleaved=False, window=win)
    assert rel(_run_mixer(M, P, mixer, h, [100, 1, 29], dtype=torch.bfloat16), want) < 0.06


@pytest.mark.parametrize("width", [40, 232, 1000])
def test_mingru_alone_sequential_and_chunked(width):
    P, S, M = _pkg()
    D, T = 48, 600
    W = _mixer_weights(gru(width), D, 7)
    h = loud_rows(torch.randn(T, D, generator=torch.Generator().manual_seed(4)), [5, 300, 301])
    want = O.mingru(h.double(), W, "")
    mixer = M.MinGRUMixer("m", {k: v.to(DEV) for k, v in W.items()}, "", width=width)
    assert S.lib().b2l_seq_mingru_chunks(T) > 1 and S.lib().b2l_seq_mingru_chunks(100) == 1
    for sizes in ([T], [1], [100, 1, 2, 63], [599, 1], [257, 343]):
        assert rel(_run_mixer(M, P, mixer, h, sizes), want) < TOL, (width, sizes)
    mixer = M.MinGRUMixer("m", {k: v.to(DEV, torch.bfloat16) for k, v in W.items()}, "", width=width)
    assert rel(_run_mixer(M, P, mixer, h, [300, 1, 100], dtype=torch.bfloat16), want) < 0.05


def test_convolution_and_rotation_kernel_alone():
    P, S, M = _pkg()
    lib = S.lib()
    g = torch.Generator().manual_seed(6)
    for (Hq, Hk, K, nv, taps, rd, inter, mult) in ((6, 2, 10, 12, 4, 6, 1, 1.0), (4, 2, 16, 24, 3, 16, 0, 1.3), (2, 0, 8, 0, 2, 4, 1, 1.0), (3, 3, 12, 6, 1, 0, 1, 1.0)):
        T, pos0 = 70, 11
        parts = [torch.randn(T + pos0, Hq * K, generator=g)] + ([torch.randn(T + pos0, Hk * K, generator=g), torch.randn(T + pos0, nv, generator=g)] if Hk else [])
        ws = [torch.randn(p.shape[1], taps, generator=g) for p in parts]
        freqs = [700.0 ** (-2.0 * i / rd) for i in range(rd // 2)] if rd else []
        # the oracle: convolve every part over the whole sequence, rotate the heads
        want = []
        for n, (u, w) in enumerate(zip(parts, ws)):
            y = O.causal_conv(u.double(), w.double())
            if n < 2 and rd:
                y = y.view(T + pos0, -1, K).clone()
                for t in range(T + pos0):
                    for hd in range(y.shape[1]):
                        y[t, hd] = O.rotate(y[t, hd], t, freqs, mult, bool(inter))
                y = y.reshape(T + pos0, -1)
            want.append(y)
        stacked, offs = M.stack_rows([p.t().contiguous() for p in parts])          # columns of a stacked projection
        proj = stacked.t().contiguous().to(DEV)
        wc = M.stack_rows(ws)[0].to(DEV)
        Cn = proj.shape[1]
        freq = torch.tensor(freqs, dtype=torch.float32, device=DEV) if rd else None
        state = torch.zeros(2, max(taps - 1, 1), Cn, device=DEV)
        outs = [[], [], []]
        at = 0
        for n_tok in (pos0, 1, 40, T - 41):          # the state carries rows over a single token, a tile and several tiles
            meta = torch.tensor([1, at], dtype=torch.int32, device=DEV)
            q = torch.empty(n_tok, Hq * K, device=DEV)
            k = torch.empty(n_tok, max(Hk * K, 1), device=DEV)
            v = torch.empty(n_tok, max(nv, 1), device=DEV)
            a = S.ConvRopeArgs(proj=proj[at:at + n_tok].data_ptr(), ld=Cn, c_off=0, C=Cn, taps=taps, w=wc.data_ptr(), state=state.data_ptr() if taps > 1 else None,
                               meta=meta.data_ptr(), q_off=offs[0], q_heads=Hq, k_off=offs[1] if Hk else -1, k_heads=Hk, K=K, v_off=offs[2] if Hk else -1, n_v=nv,
                               freq=freq.data_ptr() if rd else None, rot_dims=rd, interleaved=inter, rot_mult=mult, q_out=q.data_ptr(),
                               k_out=k.data_ptr() if Hk else None, v_out=v.data_ptr() if Hk else None, T=n_tok, act_dtype=S.B2L_F32)
            S.check(lib.b2l_seq_conv_rope(C.byref(a), None), "conv_rope")
            for o, t in zip(outs, (q, k, v)):
                o.append(t.cpu())
            at += n_tok
        assert float(state[0].abs().max()) == 0.0                       # the other slot's rows are untouched
        for n in range(len(parts)):
            assert rel(torch.cat(outs[n]), want[n]) < 1e-5, (Hq, Hk, K, n)


def test_depth_step_norm_and_activation_kernels_alone():
    P, S, M = _pkg()
    lib = S.lib()
    g = torch.Generator().manual_seed(8)
    for D in (72, 328, 1500, 3000):
        T, n_hist = 9, 4
        hist = torch.randn(n_hist, T, D, generator=g)
        y1, y2, x_in = torch.randn(T, D, generator=g), torch.randn(T, D, generator=g), torch.randn(T, D, generator=g)
        avg, w, b = torch.randn(n_hist, generator=g), torch.randn(D, generator=g), torch.randn(D, generator=g)
        own = x_in + y1 + y2
        x_want = sum(float(avg[j]) * hist[j].double() for j in range(n_hist - 1)) + float(avg[-1]) * own.double()
        y1d, y2d, avgd, wd, bd = (t.to(DEV) for t in (y1, y2, avg, w, b))      # held: a temporary's memory may be handed out again
        for kind, code in (("layer", S.NORM_LAYER), ("rms", S.NORM_RMS)):
            h_want = O.layer_norm(x_want, w.double(), b.double(), 1e-5) if kind == "layer" else O.rms_norm(x_want, w.double(), 1e-5) + b.double()
            hd, xd, out = hist.clone().to(DEV), x_in.to(DEV), torch.empty(T, D, device=DEV)
            S.check(lib.b2l_seq_depth_step(y1d.data_ptr(), y2d.data_ptr(), xd.data_ptr(), hd.data_ptr(), n_hist, avgd.data_ptr(), xd.data_ptr(),
                                           wd.data_ptr(), bd.data_ptr(), code, 1e-5, out.data_ptr(), T, D, S.B2L_F32, None), "depth_step")
            assert rel(hd[-1], own) < 1e-6 and rel(xd, x_want) < 1e-6 and rel(out, h_want) < 1e-5, (D, kind)
            assert torch.equal(hd[:-1].cpu(), hist[:-1])
            rows = torch.tensor([T - 1, 0, 3], dtype=torch.int32, device=DEV)
            picked = torch.empty(3, D, device=DEV)
            S.check(lib.b2l_seq_norm(xd.data_ptr(), wd.data_ptr(), bd.data_ptr(), code, 1e-5, picked.data_ptr(), rows.data_ptr(), 3, D, S.B2L_F32, None), "norm")
            assert rel(picked, h_want[[T - 1, 0, 3]]) < 1e-5
        # no average: the ordinary residual stream
        hd, xo, xi = hist.clone().to(DEV), torch.empty(T, D, device=DEV), x_in.to(DEV)
        S.check(lib.b2l_seq_depth_step(y1d.data_ptr(), None, xi.data_ptr(), hd.data_ptr(), n_hist, None, xo.data_ptr(), None, None, 0, 0.0, None,
                                       T, D, S.B2L_F32, None), "depth_step")
        assert rel(xo, x_in + y1) < 1e-6
    # a constant offset must not change a layer norm: the variance is of the deviations, not E[x^2] - mean^2
    x = (torch.randn(4, 312, generator=g) * 0.01 + 30.0).to(DEV)
    one, zero, out = torch.ones(312, device=DEV), torch.zeros(312, device=DEV), torch.empty(4, 312, device=DEV)
    S.check(lib.b2l_seq_norm(x.data_ptr(), one.data_ptr(), zero.data_ptr(), S.NORM_LAYER, 1e-6, out.data_ptr(), None, 4, 312, S.B2L_F32, None), "norm")
    assert rel(out, O.layer_norm(x.double().cpu(), 1.0, 0.0, 1e-6)) < 2e-3
    for F, dtype in ((50, torch.float32), (392, torch.float32), (392, torch.bfloat16)):
        z = (3.0 * torch.randn(7, F, generator=g)).bfloat16().float()
        z[0, :8] = torch.tensor([0.0, -1e-4, -0.2490, -0.2501, -0.25, 1e-4, -30.0, -100.0])     # both forms of the negative side and their border
        pq = torch.tensor([0.3, -0.6]).bfloat16().float()
        zd = z.to(DEV, dtype)
        coef = torch.tensor([O.softplus(float(pq[0])), 0.5 + O.softplus(float(pq[1]))], dtype=torch.float32, device=DEV)
        S.check(lib.b2l_seq_unary_act(zd.data_ptr(), F, zd.data_ptr(), F, 7, F, S.ACT_XIELU, coef.data_ptr(), S.act_code(dtype), None), "act")
        assert rel(zd, O.xielu(z.double(), float(pq[0]), float(pq[1]))) < (1e-6 if dtype == torch.float32 else 4e-3)


def test_router_groups_worth_their_two_best():
    P, S, M = _pkg()
    n, T = 24, 64
    g = torch.Generator().manual_seed(9)
    z = (2.0 * torch.randn(T, n, generator=g)).float()
    corr = (0.3 * torch.randn(n, generator=g)).float()
    # a group with the single best expert but a poor second loses against a group with two good ones
    z[0] = torch.tensor([4.0] + [-9.0] * 7 + [2.0, 2.0] + [-9.0] * 14)
    for count, keep, top, scale in ((3, 1, 2, 1.25), (4, 2, 3, 1.0), (2, 1, 6, 0.25), (24, 5, 3, 2.0), (6, 6, 4, 1.0)):
        r = {"experts": n, "top": top, "groups": {"count": count, "keep": keep}, "scale": scale}
        W = {"router": torch.eye(n), "correction": corr if count not in (3, 4) else torch.zeros(n)}
        want_idx, want_w = O.route(z.double(), W, "", r)
        idx = torch.empty(T, top, dtype=torch.int32, device=DEV)
        wgt = torch.empty(T, top, dtype=torch.float32, device=DEV)
        zd, cd, eye = z.to(DEV), W["correction"].to(DEV), torch.eye(n, device=DEV)
        S.check(S.lib().b2l_seq_moe_route(zd.data_ptr(), n, cd.data_ptr(), n, count, keep, top, S.SCORE_SIGMOID, 1, 2, scale,
                                          idx.data_ptr(), wgt.data_ptr(), T, None), "route")
        assert idx.cpu().tolist() == want_idx.tolist(), (count, keep, top)
        assert rel(wgt, want_w) < 1e-6
        if count == 3:
            assert sorted(idx[0].tolist()) == [8, 9]
        # the fused form of a few tokens: logits from the product with an identity router
        idx2, wgt2 = torch.empty(3, top, dtype=torch.int32, device=DEV), torch.empty(3, top, dtype=torch.float32, device=DEV)
        S.check(S.lib().b2l_seq_moe_route_fused(zd.data_ptr(), n, eye.data_ptr(), cd.data_ptr(), n, n, count, keep,
                                                top, S.SCORE_SIGMOID, 1, 2, scale, idx2.data_ptr(), wgt2.data_ptr(), 3, S.B2L_F32, None), "route_fused")
        assert idx2.cpu().tolist() == want_idx[:3].tolist() and rel(wgt2, want_w[:3]) < 1e-6


def test_feed_forwards_alone():
    P, S, M = _pkg()
    D, T = 64, 40
    for layer_mlp in (dense(100), moe(8, 3, 24, count=4, keep=2, scale=1.25), moe(5, 1, 16), moe(6, 6, 8, count=2, keep=2, scale=0.5)):
        cfg = {"vocab": 8, "width": D, "norm": {"eps": 1e-6}, "layers": [with_mlp(gru(8), layer_mlp)]}
        W = {k[len("l0.mlp."):]: v for k, v in random_weights(cfg, 11).items() if k.startswith("l0.mlp.")}
        h = torch.randn(T, D, generator=torch.Generator().manual_seed(10)).bfloat16().float()
        want = O.dense_ff(h.double(), W, "") if layer_mlp["kind"] == "dense" else O.routed_ff(h.double(), W, "", layer_mlp)
        from lit_llama_b200.rinirax import build_feed_forward
        ff = build_feed_forward(layer_mlp, {k: v.to(DEV) for k, v in W.items()}, "")
        for n in (T, 3):                       # the sorted path of long portions and the device-indexed one of a few tokens
            ctx, _ = _ctx(M, P, {}, n, 0, torch.float32)
            assert rel(ff.forward(h[:n].to(DEV), ctx), want[:n]) < TOL, (layer_mlp, n)


def test_differential_readout_kernel_alone():
    P, S, M = _pkg()
    g = torch.Generator().manual_seed(12)
    for H, V in ((3, 12), (4, 56), (1, 200)):
        T = 11
        a = torch.randn(T, H, 2, V, generator=g)
        o = a[:, :, 0].double() - 0.37 * a[:, :, 1].double()
        want = O.rms_norm(o, None, 1e-5) * 0.6
        out, ad = torch.empty(T, H * V, device=DEV), a.to(DEV)
        S.check(S.lib().b2l_seq_diff_combine(ad.data_ptr(), H * 2 * V, 0.37, 1e-5, 0.6, out.data_ptr(), H * V, T, H, V, S.B2L_F32, None), "diff_combine")
        assert rel(out, want.reshape(T, H * V)) < 1e-6
