"""GPU: the Zuvevik model family and its mechanisms against the plain restatement in tests/zuvevik_oracle.py
(float64), on small random models of several shapes: each mechanism alone, whole prompts against token-by-token
decoding and portions of many sizes, interleaved requests, reused slots, dominant keys just inside and just outside the
window (in prompts, across portions and in decoding, at ring and tile borders), the first tokens of a sequence, long
decoding over many turns of the ring, greedy generation through the engine's scheduler."""
import ctypes as C
import json
import math

import pytest
import torch

import zuvevik_oracle as O

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _pkg():
    import lit_llama_b200 as P
    from lit_llama_b200 import _seqlib as S
    from lit_llama_b200 import mixers as M
    return P, S, M


def rel(got, want):
    got, want = got.double().cpu(), want.double().cpu()
    return float((got - want).norm() / (want.norm() + 1e-30))


# ----------------------------------------------------------------------------- configurations (none is a served model's)
def attn(heads, kv_heads, dim, vdim, window, scale, rot_dims, base=10000.0, v_mix=True):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window}, "scale": scale, "v_mix": v_mix,
            "rot": {"base": base, "dims": rot_dims}}


def moe(experts, top, ff, limit):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


def cfg_a():
    """Odd sizes; two experts per token; partial rotation; a layer without value mixing ahead of the first mixing one; a
    layer without feed-forward; windows of 5, 9 and 1 positions; two streams."""
    return {"architecture": "Zuvevik", "vocab": 131, "width": 72, "norm": {"eps": 1e-5}, "streams": 2, "logit_scale": 0.7,
            "embedding": {"bigram": {"buckets": 37, "mul_prev": 5, "mul_cur": 11}},
            "layers": [
                {"type": "attention", "mixer": attn(3, 3, 20, 12, 5, 0.21, 12, 1000.0, v_mix=False), "mlp": moe(6, 2, 40, 1.0)},
                {"type": "attention", "mixer": attn(6, 2, 10, 18, 9, 0.4, 10), "mlp": None},
                {"type": "attention", "mixer": attn(6, 2, 14, 18, 1, 0.3, 6), "mlp": {"kind": "dense", "ff": 50}},
                {"type": "attention", "mixer": attn(2, 2, 24, 18, 9, 0.2, 24, 50.0), "mlp": moe(5, 3, 24, 0.6)},
            ]}


def cfg_b():
    """Four streams, one expert per token, a dense layer last, no rotation in one layer, kv heads = 1, logit scale 1."""
    return {"architecture": "Zuvevik", "vocab": 90, "width": 64, "norm": {"eps": 1e-6}, "streams": 4, "logit_scale": 1.0,
            "embedding": {"bigram": {"buckets": 64, "mul_prev": 1, "mul_cur": 1}},
            "layers": [
                {"type": "attention", "mixer": attn(4, 1, 16, 16, 33, 0.25, 8), "mlp": moe(4, 1, 24, 2.5)},
                {"type": "attention", "mixer": attn(2, 2, 32, 8, 64, 0.18, 0), "mlp": moe(7, 4, 16, 1.75)},
                {"type": "attention", "mixer": attn(4, 1, 16, 16, 17, 0.25, 16), "mlp": {"kind": "dense", "ff": 96}},
            ]}


def cfg_c():
    """Shapes that take the tiled attention kernel (16-byte rows, many queries) and the sorted expert path; one stream
    with hyper-connection weights; a window of 40 over portions of hundreds of tokens."""
    return {"architecture": "Zuvevik", "vocab": 200, "width": 128, "norm": {"eps": 1e-6}, "streams": 1, "logit_scale": 3.0,
            "embedding": {"bigram": {"buckets": 101, "mul_prev": 7, "mul_cur": 3}},
            "layers": [
                {"type": "attention", "mixer": attn(8, 2, 32, 40, 40, 0.15, 16, 3e5), "mlp": moe(8, 3, 64, 1.2)},
                {"type": "attention", "mixer": attn(8, 4, 32, 64, 70, 0.15, 32, 3e5, v_mix=False), "mlp": {"kind": "dense", "ff": 160}},
                {"type": "attention", "mixer": attn(8, 2, 32, 40, 40, 0.15, 16, 3e5), "mlp": moe(8, 2, 64, 0.9)},
            ]}


def cfg_d():
    """No hyper-connection tensors and no pair table: the ordinary pre-norm residual layer; five streams elsewhere."""
    return {"architecture": "Zuvevik", "vocab": 77, "width": 40, "norm": {"eps": 1e-6},
            "layers": [
                {"type": "attention", "mixer": attn(2, 2, 10, 6, 7, 0.3, 4), "mlp": {"kind": "dense", "ff": 30}},
                {"type": "attention", "mixer": attn(1, 1, 10, 12, 3, 0.3, 10), "mlp": moe(3, 2, 12, 1.0)},
            ]}


def cfg_e():
    d = cfg_d()
    d["streams"] = 5
    d["embedding"] = {"bigram": {"buckets": 11, "mul_prev": 1000003, "mul_cur": (1 << 61) - 1}}
    return d


CONFIGS = {"a": cfg_a, "b": cfg_b, "c": cfg_c, "d": cfg_d, "e": cfg_e}


def random_weights(cfg, seed=1):
    """bf16-representable float32 tensors on the CPU under the family's tensor names."""
    g = torch.Generator().manual_seed(seed)
    D, s, W = cfg["width"], int(cfg.get("streams", 1)), {}

    def rnd(*shape, std=1.0, mean=0.0):
        return (mean + std * torch.randn(*shape, generator=g)).bfloat16().float()

    def lin(o, i, gain=1.0):
        return rnd(o, i, std=gain / math.sqrt(i))

    W["embed"], W["head"], W["final.norm"] = rnd(cfg["vocab"], D), lin(cfg["vocab"], D), rnd(D, std=0.2, mean=1.0)
    b = (cfg.get("embedding") or {}).get("bigram")
    if b:
        W["bigram"] = rnd(b["buckets"] + 1, D, std=0.7)
    for i, layer in enumerate(cfg["layers"]):
        p, m, c = f"l{i}.", f"l{i}.mix.", layer["mixer"]
        H, G, K, V = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
        W[p + "norm1"] = rnd(D, std=0.2, mean=1.0)
        W[m + "q"], W[m + "k"], W[m + "v"], W[m + "g"], W[m + "o"] = lin(H * K, D, 2.0), lin(G * K, D, 2.0), lin(G * V, D), lin(H * V, D), lin(D, H * V)
        W[m + "q.norm"], W[m + "k.norm"] = rnd(H * K, std=0.3, mean=1.5), rnd(G * K, std=0.3, mean=1.5)
        W[m + "vmix"] = rnd((), std=0.15, mean=0.4)
        f = layer.get("mlp")
        if f:
            W[p + "norm2"] = rnd(D, std=0.2, mean=1.0)
            if f["kind"] == "dense":
                W[p + "mlp.gate"], W[p + "mlp.up"], W[p + "mlp.down"] = lin(f["ff"], D), lin(f["ff"], D), lin(D, f["ff"])
            else:
                W[p + "mlp.router"] = lin(f["router"]["experts"], D, 3.0)
                for e in range(f["router"]["experts"]):
                    q, ff = f"{p}mlp.e{e}.", f["expert"]["ff"]
                    W[q + "gate"], W[q + "up"], W[q + "down"] = lin(ff, D, 2.0), lin(ff, D, 2.0), lin(D, ff)
        if "streams" in cfg:
            for q in ("1", "2") if f else ("1",):
                W[p + f"hc{q}.in"] = rnd(s, std=0.3, mean=0.6)
                W[p + f"hc{q}.out"] = rnd(s, std=0.4, mean=0.8)
                W[p + f"hc{q}.mix"] = (torch.eye(s) * 0.8 + 0.25 * torch.randn(s, s, generator=g)).bfloat16().float()
    return W


def build(cfg, dtype, seed=1, n_slots=3):
    P, S, M = _pkg()
    W = random_weights(cfg, seed)
    model = P.Zuvevik(P.ZuvevikConfig.from_dict(cfg), {k: v.to(DEV, dtype) for k, v in W.items()})
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
@pytest.mark.parametrize("name", ["a", "b", "c", "d", "e"])
def test_model_matches_the_oracle_layer_by_layer_f32(name):
    cfg = CONFIGS[name]()
    model, engine, W = build(cfg, torch.float32)
    toks = tokens_of(cfg, 90 if name == "c" else 45)
    cap = []
    want = O.model(toks, cfg, W, capture=cap)
    model.capture_layers = []
    got = run_whole(engine, toks)
    assert len(model.capture_layers) == len(cap) == len(cfg["layers"])
    for i, (g, w) in enumerate(zip(model.capture_layers, cap)):
        assert rel(g, w) < 2e-5, (name, "layer", i, rel(g, w))
    assert rel(got, want) < 2e-5


@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_model_bf16_is_close_to_the_oracle(name):
    cfg = CONFIGS[name]()
    model, engine, W = build(cfg, torch.bfloat16)
    toks = tokens_of(cfg, 60)
    want = O.model(toks, cfg, W)
    got = run_whole(engine, toks)
    assert rel(got, want) < 0.1, rel(got, want)
    again = run_pieces(engine, toks, [7, 1, 2, 13])
    per_token = (again.double() - got.double()).norm(dim=-1) / got.double().norm(dim=-1)
    assert int((per_token > 0.05).sum()) <= 2, per_token      # a routing flip on a close call moves one token a lot, rounding none


@pytest.mark.parametrize("name", ["a", "b", "c", "e"])
def test_portions_and_single_tokens_equal_the_whole_prompt(name):
    cfg = CONFIGS[name]()
    n = 330 if name == "c" else 80          # c: several 64-query tiles, windows that start in older portions
    model, engine, W = build(cfg, torch.float32)
    toks = tokens_of(cfg, n)
    whole = run_whole(engine, toks)
    if name != "c":
        assert rel(whole, O.model(toks, cfg, W)) < 2e-5
    for sizes in ([1], [2], [3, 2, 17, 1, 5], [33, 64], [n - 9, 1, 1, 2]):
        if name == "c" and sizes == [1]:
            sizes = [n - 100, 1]            # a long first portion, then 100 tokens one by one through the captured step
        got = run_pieces(engine, toks, sizes)
        assert rel(got, whole) < 2e-5, (name, sizes, rel(got, whole))


def test_interleaved_requests_and_reused_slots():
    cfg = cfg_a()
    model, engine, W = build(cfg, torch.float32, n_slots=2)
    prompts = [tokens_of(cfg, n, seed=s) for n, s in ((23, 1), (5, 2), (41, 3), (1, 4), (12, 5))]
    alone = [run_whole(engine, p, rid=("alone", i)) for i, p in enumerate(prompts)]
    for i, p in enumerate(prompts):
        assert rel(alone[i], O.model(p, cfg, W)) < 2e-5
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
        assert rel(torch.cat(got[i]), alone[i]) < 2e-5, i
    # one step with several entries of unequal length against each alone
    outs = engine.step([{"id": ("m", i), "tokens": p, "want": list(range(len(p)))} for i, p in enumerate(prompts[:2])], [("m", 0), ("m", 1)])
    for i in range(2):
        assert rel(outs[i], alone[i]) < 2e-5


def test_long_decoding_through_the_captured_step():
    cfg = cfg_b()                            # windows of 33, 64 and 17: the rings turn several times
    model, engine, W = build(cfg, torch.float32)
    toks = tokens_of(cfg, 230)
    want = O.model(toks, cfg, W)
    first = engine.step([{"id": "d", "tokens": toks[:20], "want": [19]}])[0]
    outs = [first] + [engine.step([{"id": "d", "tokens": [t], "want": [0]}])[0] for t in toks[20:]]
    assert engine._graph is not None
    assert rel(torch.cat(outs), want[19:]) < 2e-5
    # the same captured step serves another request in another slot from its first token on
    outs2 = [engine.step([{"id": "e", "tokens": [t], "want": [0]}])[0] for t in toks[:40]]
    assert rel(torch.cat(outs2), want[:40]) < 2e-5


def test_first_tokens_of_a_sequence():
    """One-token and two-token sequences, and the first-token row of the pair table after a slot was used before."""
    cfg = cfg_a()
    model, engine, W = build(cfg, torch.float32, n_slots=1)
    for toks in ([7], [7, 7], [130, 0], tokens_of(cfg, 3)):
        want = O.model(toks, cfg, W)
        assert rel(run_whole(engine, toks), want) < 2e-5
        assert rel(run_pieces(engine, toks, [1]), want) < 2e-5
    assert engine.pool.reused >= 5


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
    cfg = cfg_b()
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

    cfg = cfg_b()
    W = random_weights(cfg, seed=3)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    write_safetensors(str(tmp_path / "model.safetensors"), {k: v.bfloat16() for k, v in W.items()})
    toks = tokens_of(cfg, 12)
    want = O.model(toks, cfg, W)
    for dtype, tol in ((torch.float32, 2e-5), (torch.bfloat16, 0.1)):
        model = P.load_model(str(tmp_path), dtype=dtype, device=DEV, max_positions=64)
        assert type(model).__name__ == "Zuvevik"
        assert rel(run_whole(P.Engine(model, n_slots=1), toks), want) < tol
        if dtype == torch.float32:                   # a ring per layer: no position limit, whatever max_positions said
            long = tokens_of(cfg, 150)
            assert rel(run_whole(P.Engine(model, n_slots=1), long), O.model(long, cfg, W)) < 2e-5


# ----------------------------------------------------------------------------- mechanisms alone
def _ctx(M, P, specs, T, pos0, dtype, slot=0, pool=None, n_slots=2):
    pool = pool or P.SequenceStatePool(specs, n_slots, torch.device(DEV))
    meta = torch.tensor([slot, pos0], dtype=torch.int32, device=DEV)
    return M.StepContext(T, meta, pool.tensors, dtype, pos_hint=pos0, slot_hint=slot), pool


def test_pair_embedding_alone():
    P, S, M = _pkg()
    V, D, buckets = 50, 24, 13
    g = torch.Generator().manual_seed(0)
    emb, pair = torch.randn(V, D, generator=g).bfloat16().float(), torch.randn(buckets + 1, D, generator=g).bfloat16().float()
    toks = torch.randint(0, V, (40,), generator=g).tolist()
    cfg = {"embedding": {"bigram": {"buckets": buckets, "mul_prev": 29, "mul_cur": 13}}}
    want = O.embedding(toks, {"embed": emb, "bigram": pair}, cfg)
    for dtype in (torch.float32, torch.bfloat16):
        e = M.PairHashEmbedding("pe", emb.to(DEV, dtype), pair.to(DEV, dtype), buckets=buckets, mul_prev=29, mul_cur=13, streams=3)
        pool = None
        for slot, cuts in ((1, [40]), (0, [1, 1, 5, 2, 31]), (1, [13, 27])):       # slot 1 is used twice: the stale last token must not be read
            outs, at = [], 0
            for n in cuts:
                ctx, pool = _ctx(M, P, e.state_specs(), n, at, dtype, slot=slot, pool=pool)
                tk = torch.tensor(toks[at:at + n], dtype=torch.int64 if n % 2 else torch.int32, device=DEV)
                x = e.forward(tk, ctx)
                assert x.shape == (n, 3, D) and bool((x[:, 0] == x[:, 1]).all()) and bool((x[:, 0] == x[:, 2]).all())
                outs.append(x[:, 0])
                at += n
            assert float((torch.cat(outs).double().cpu() - want).abs().max()) < 1e-6
    plain = M.PairHashEmbedding("pe", emb.to(DEV), None, streams=1)
    ctx, _ = _ctx(M, P, {}, 40, 0, torch.float32)
    assert float((plain.forward(torch.tensor(toks, device=DEV), ctx)[:, 0].cpu() - emb[torch.tensor(toks)]).abs().max()) == 0.0


@pytest.mark.parametrize("streams", [1, 2, 3, 4, 6, 11])
def test_hyper_connection_step_alone(streams):
    P, S, M = _pkg()
    T, D, eps = 9, 200, 1e-5
    g = torch.Generator().manual_seed(streams)
    X = torch.randn(T, streams, D, generator=g)
    y = torch.randn(T, D, generator=g).bfloat16().float()
    a = M.HyperConnection(*(torch.randn(*s, generator=g).to(DEV) for s in ((streams,), (streams, streams), (streams,))))
    b = M.HyperConnection(*(torch.randn(*s, generator=g).to(DEV) for s in ((streams,), (streams, streams), (streams,))))
    w = torch.randn(D, generator=g).bfloat16().float()
    old = [X[:, s].double() for s in range(streams)]
    new = O.hyper_step(old, y.double(), a.read.cpu(), a.mix.cpu(), a.write.cpu())
    want_h = O.rms_norm(O.hyper_read(new, b.read.cpu()), w.double(), eps)
    for dtype, tol in ((torch.float32, 1e-6), (torch.bfloat16, 6e-3)):
        ctx, _ = _ctx(M, P, {}, T, 0, dtype)
        x = X.to(DEV).clone()
        h = M.HyperConnection.step(x, ctx, y=y.to(DEV, dtype), wrote=a, reads=b, norm=w.to(DEV, dtype), eps=eps)
        for s in range(streams):
            assert rel(x[:, s], new[s]) < 1e-6
        assert rel(h, want_h) < tol
        # the read alone on picked rows, and the write alone
        rows = torch.tensor([8, 0, 3], dtype=torch.int32, device=DEV)
        h2 = M.HyperConnection.step(x, ctx, reads=b, norm=w.to(DEV, dtype), eps=eps, rows=rows, n_rows=3)
        assert rel(h2, want_h[[8, 0, 3]]) < tol
        x2 = X.to(DEV).clone()
        assert M.HyperConnection.step(x2, ctx, y=y.to(DEV, dtype), wrote=a) is None
        assert float((x2 - x).abs().max()) == 0.0
        out = torch.empty(T, D, device=DEV)
        S.check(S.lib().b2l_seq_hc_sum(x.data_ptr(), out.data_ptr(), T, D, streams, None), "sum")
        assert rel(out, sum(new)) < 1e-6


@pytest.mark.parametrize("per_head", [False, True])
def test_attention_operands_alone(per_head):
    """q/k norm over the whole projection or per head, partial rotation from a device position, value mixing."""
    P, S, M = _pkg()
    H, G, K, V, D, T, eps, pos0 = 5, 1, 12, 7, 40, 11, 1e-5, 37
    c = attn(H, G, K, V, 4, 0.3, 8, 123.0)
    g = torch.Generator().manual_seed(3)
    W = {"q": torch.randn(H * K, D, generator=g), "k": torch.randn(G * K, D, generator=g), "v": torch.randn(G * V, D, generator=g),
         "q.norm": torch.randn(K if per_head else H * K, generator=g), "k.norm": torch.randn(K if per_head else G * K, generator=g)}
    W = {k: v.bfloat16().float() for k, v in W.items()}
    h = torch.randn(T, D, generator=g).bfloat16().float()
    q, k, v = O.attention_operands(h.double(), W, "", c, eps, pos0=pos0, per_head_norm=per_head)
    v_first = torch.randn(T, G * V + 3, generator=g).bfloat16().float()
    lam = torch.tensor([0.3125])
    want_v = (1 - 0.3125) * v + 0.3125 * v_first[:, 2:2 + G * V].double()
    proj = torch.cat([torch.zeros(T, 8), h @ W["q"].T, h @ W["k"].T, torch.zeros(T, 4), h @ W["v"].T], dim=1).to(DEV)
    o_q, o_k, o_v = 8, 8 + H * K, 8 + H * K + G * K + 4
    f = M.rope_frequencies(8, 123.0, None)[0].to(DEV)
    qn, kn, lam_d = W["q.norm"].to(DEV), W["k.norm"].to(DEV), lam.to(DEV)
    meta = torch.tensor([0, pos0], dtype=torch.int32, device=DEV)
    qo, ko, vo = torch.empty(T, H * K, device=DEV), torch.empty(T, G * K, device=DEV), torch.empty(T, G * V, device=DEV)
    vf = v_first.to(DEV)
    a = S.QkvPrepArgs(proj=proj.data_ptr(), ld=proj.shape[1], q_off=o_q, k_off=o_k, v_off=o_v, q_norm=qn.data_ptr(),
                      k_norm=kn.data_ptr(), whole_row=int(not per_head), eps=eps, freq=f.data_ptr(), rot_dims=8, rot_mult=1.0,
                      meta=meta.data_ptr(), q_out=qo.data_ptr(), k_out=ko.data_ptr(), v_first=vf.data_ptr() + 2 * 4, ldvf=vf.shape[1],
                      lambda_=lam_d.data_ptr(), v_out=vo.data_ptr(), T=T, heads=H, kv_heads=G, K=K, V=V, act_dtype=S.B2L_F32)
    S.check(S.lib().b2l_seq_qkv_prep(C.byref(a), None), "prep")
    assert rel(qo, q.reshape(T, -1)) < 2e-6 and rel(ko, k.reshape(T, -1)) < 2e-6 and rel(vo, want_v) < 1e-6


def _window_attention(S, q, k, v, cache_k, cache_v, gate, pos0, window, ring, scale, dtype, slot=0, work=True):
    """The attention kernel on operands made by the test: q [T, H, K] f32, k [T, G, K], v [T, G, V], caches
    [slots, ring, G, K or V], gate [T, H*V]; returns [T, H*V] and appends to the ring.  `work`: give the call the work
    space it asks for (few queries then run as parallel key chunks with a merge), else it runs its form without one."""
    T, H, K = q.shape
    G, V = k.shape[1], v.shape[2]
    out = torch.empty(T, H * V, dtype=dtype, device=DEV)
    meta = torch.tensor([slot, pos0], dtype=torch.int32, device=DEV)
    qd, kd, vd, gd = q.to(DEV).contiguous(), k.to(DEV, dtype).contiguous(), v.to(DEV, dtype).contiguous(), gate.to(DEV, dtype).contiguous()
    a = S.AttnArgs(q=qd.data_ptr(), k_new=kd.data_ptr(), v_new=vd.data_ptr(), ldv=G * V, cache_k=cache_k.data_ptr(), cache_v=cache_v.data_ptr(),
                   meta=meta.data_ptr(), gate=gd.data_ptr(), ldg=H * V, out=out.data_ptr(), ldo=H * V, scale=scale, softcap=0.0, out_mult=1.0,
                   has_sink=0, block=ring, T=T, heads=H, kv_heads=G, K=K, V=V, act_dtype=S.act_code(dtype), window=window, gate_per_channel=1)
    n = S.lib().b2l_seq_block_attention_work_floats(C.byref(a)) if work else 0
    buf = torch.full((max(n, 1),), float("nan"), device=DEV)
    if n:
        a.work, a.work_floats = buf.data_ptr(), n
    S.check(S.lib().b2l_seq_block_attention(C.byref(a), None), "attention")
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("shape", [(4, 2, 16, 24, 40, 40), (6, 2, 32, 56, 70, 70), (3, 1, 10, 6, 5, 8), (8, 8, 64, 64, 33, 64), (2, 1, 20, 128, 100, 100)])
def test_sliding_window_attention_alone(shape):
    """Both attention kernels (a warp per query and head; 64-query tiles) against the oracle: whole, in portions whose
    windows reach into the ring, and token by token, in f32 and bf16; the ring may be larger than the window."""
    P, S, M = _pkg()
    H, G, K, V, window, ring = shape
    T, scale = 333, 0.4 / math.sqrt(K)
    g = torch.Generator().manual_seed(7)
    q, k, v = (torch.randn(T, n, d, generator=g).bfloat16().float() for n, d in ((H, K), (G, K), (G, V)))
    gate = torch.randn(T, H * V, generator=g).bfloat16().float()
    want = O.windowed_softmax_attention(q.double(), k.double(), v.double(), scale, window) * torch.sigmoid(gate.double())
    for dtype, tol in ((torch.float32, 3e-6), (torch.bfloat16, 6e-3)):
        for slot, cuts, work in ((0, [T], True), (1, [130, 1, 2, 64, 17, 119], True), (0, [200] + [1] * 133, True), (1, [150, 3, 20] + [1] * 160, False)):
            ck = torch.full((2, ring, G, K), float("nan"), dtype=dtype, device=DEV)      # stale entries must never be read
            cv = torch.full((2, ring, G, V), float("nan"), dtype=dtype, device=DEV)
            outs, at = [], 0
            for n in cuts:
                outs.append(_window_attention(S, q[at:at + n], k[at:at + n], v[at:at + n], ck, cv, gate[at:at + n], at, window, ring, scale, dtype, slot,
                                              work=work))
                at += n
            assert rel(torch.cat(outs), want) < tol, (shape, dtype, cuts[:3], rel(torch.cat(outs), want))


@pytest.mark.parametrize("V,work", [(8, True), (6, True), (8, False)])
@pytest.mark.parametrize("window", [1, 2, 31, 32, 33, 63, 64, 65, 80, 128, 129])
def test_a_dominant_key_just_inside_and_just_outside_the_window(window, V, work):
    """One key is made to stand out (long, along every query); its value is a marker.  A query sees the marker exactly
    when 0 <= distance < window: in one portion (both kernels), across a portion border, and when decoding from the ring."""
    P, S, M = _pkg()
    H, G, K, ring = 8, 2, 16, window + 3              # V = 6: rows that the tiled kernel does not take
    g = torch.Generator().manual_seed(window)
    direction = torch.randn(K, generator=g)
    direction /= direction.norm()
    for T, star in ((300, 150), (300, 0), (300, 63), (300, 64), (40, 7)):
        q = 0.1 * torch.randn(T, H, K, generator=g) + 6.0 * direction
        k = 0.1 * torch.randn(T, G, K, generator=g)
        k[star] += 6.0 * direction                   # score of the marked key: ~36 above the others
        v = 0.01 * torch.randn(T, G, V, generator=g)
        v[star] = 100.0
        gate = torch.full((T, H * V), 30.0)           # sigmoid = 1
        checks = [star, star + 1, star + window - 1, star + window, star + window + 1, T - 1]
        upto = min(T, star + window + 3)              # later queries are like the last one checked
        for cuts in ([T], [star + 1, T - star - 1], [star + 1] + [1] * (upto - star - 1), [star + window - 1, 2, T]):
            ck = torch.zeros((1, ring, G, K), device=DEV)
            cv = torch.zeros((1, ring, G, V), device=DEV)
            outs, at = [], 0
            for n in cuts:
                n = min(n, T - at)
                if n <= 0:
                    continue
                outs.append(_window_attention(S, q[at:at + n], k[at:at + n], v[at:at + n], ck, cv, gate[at:at + n], at, window, ring, 1.0, torch.float32,
                                              work=work))
                at += n
            out = torch.cat(outs).cpu()
            for i in checks:
                if i >= out.shape[0]:
                    continue
                seen = 0 <= i - star < window
                val = float(out[i].mean())
                assert (val > 99.0) == seen and (seen or abs(val) < 1.0), (window, T, star, cuts[:2], i, val)


def test_routed_experts_alone():
    """Sigmoid scores, several experts per token, the score as weight on the expert's input, the clamped unit: the
    device-indexed form (a few tokens) and the sorted form (many), f32 and bf16."""
    P, S, M = _pkg()
    for (E, top, ff, D, limit) in ((6, 2, 40, 72, 1.0), (4, 1, 24, 64, 2.5), (9, 4, 20, 50, 0.5), (3, 3, 16, 32, 1.25)):
        m = moe(E, top, ff, limit)
        g = torch.Generator().manual_seed(E)
        W = {"router": (3.0 * torch.randn(E, D, generator=g) / math.sqrt(D)).bfloat16().float()}
        for e in range(E):
            for nm, shp in (("gate", (ff, D)), ("up", (ff, D)), ("down", (D, ff))):
                W[f"e{e}.{nm}"] = (2.0 * torch.randn(*shp, generator=g) / math.sqrt(shp[1])).bfloat16().float()
        h = torch.randn(37, D, generator=g).bfloat16().float()
        want = O.routed_ff(h.double(), W, "", m)
        widx, wwgt = O.route(h.double(), W, "", m)
        for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
            ff_ = M.MoEFeedForward({k: v.to(DEV, dtype) for k, v in W.items()}, "", experts=E, identity=0, top=top, groups=1, keep=1, ff=ff,
                                   act="clamped_swish", limit=limit, score="sigmoid", renormalize=False, weight_on="input")
            for lo, hi in ((0, 37), (0, 3), (3, 4), (4, 6)):
                ctx, _ = _ctx(M, P, {}, hi - lo, 0, dtype)
                got = ff_.forward(h[lo:hi].to(DEV, dtype), ctx)
                if dtype == torch.float32:
                    assert ff_.last_idx.cpu().tolist() == widx[lo:hi].tolist()
                assert rel(got, want[lo:hi]) < tol, (E, top, dtype, lo, hi, rel(got, want[lo:hi]))
        # the saturating side of the unit: large products are clamped
        big = (40.0 * h).bfloat16().float()
        ff_ = M.MoEFeedForward({k: v.to(DEV) for k, v in W.items()}, "", experts=E, identity=0, top=top, groups=1, keep=1, ff=ff,
                               act="clamped_swish", limit=limit, score="sigmoid", renormalize=False, weight_on="input")
        ctx, _ = _ctx(M, P, {}, 37, 0, torch.float32)
        assert rel(ff_.forward(big.to(DEV), ctx), O.routed_ff(big.double(), W, "", m)) < 1e-5


def test_sigmoid_scores_without_renormalisation():
    P, S, M = _pkg()
    T, n = 7, 10
    z = torch.randn(T, n)
    idx = torch.empty(T, 3, dtype=torch.int32, device=DEV)
    wgt = torch.empty(T, 3, dtype=torch.float32, device=DEV)
    zd = z.to(DEV)
    S.check(S.lib().b2l_seq_moe_route(zd.data_ptr(), n, None, n, 1, 1, 3, S.SCORE_SIGMOID, 0, 1, 1.0, idx.data_ptr(), wgt.data_ptr(), T, None), "route")
    want = torch.sigmoid(z).topk(3, dim=-1)
    assert idx.cpu().tolist() == want.indices.tolist()
    assert float((wgt.cpu() - want.values).abs().max()) < 1e-6
    S.check(S.lib().b2l_seq_moe_route(zd.data_ptr(), n, None, n, 1, 1, 3, S.SCORE_SIGMOID, 1, 1, 1.0, idx.data_ptr(), wgt.data_ptr(), T, None), "route")
    assert float((wgt.cpu() - want.values / want.values.sum(-1, keepdim=True)).abs().max()) < 1e-6


def test_clamped_unit_and_scale():
    P, S, M = _pkg()
    T, F = 5, 24
    gu = (3.0 * torch.randn(T, 2 * F)).bfloat16().float()
    want = O.clamped_unit(gu[:, :F].double(), gu[:, F:].double(), 1.25)
    for dtype, tol in ((torch.float32, 1e-6), (torch.bfloat16, 5e-3)):
        for f, ld in ((F, 2 * F), (F - 1, 2 * F)):          # the 16-byte form and the plain one
            src = gu if f == F else torch.cat([gu[:, :f], gu[:, F:F + f], gu[:, :2]], dim=1)
            d = src.to(DEV, dtype).contiguous()
            mid = torch.empty(T, f, dtype=dtype, device=DEV)
            S.check(S.lib().b2l_seq_gated_act(d.data_ptr(), ld, mid.data_ptr(), T, f, S.ACT_CLAMPED_SWISH, 1.25, S.act_code(dtype), None), "act")
            assert rel(mid, want[:, :f]) < tol
    z = torch.randn(1000, device=DEV)
    zz = z.clone()
    S.check(S.lib().b2l_seq_scale(zz.data_ptr(), zz.numel(), 0.37, None), "scale")
    assert float((zz - z * 0.37).abs().max()) < 1e-7
