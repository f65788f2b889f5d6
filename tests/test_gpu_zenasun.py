"""GPU: the Zenasun model family and its mechanisms against the plain restatement in tests/zenasun_oracle.py
(float64), on small random models of several shapes: each mechanism alone, whole prompts against token-by-token
decoding and portions of many sizes, interleaved requests, reused cache slots, far keys and the causal edge at tile
and split borders, the sink, long decoding, greedy generation through the engine's scheduler."""
import ctypes as C
import json
import math

import pytest
import torch

import zenasun_oracle as O

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
def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base=10000.0):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale,
            "rot": {"base": base, "dims": rot_dim}}


def moe(experts, identity, top, count, keep, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top,
                                                             "groups": {"count": count, "keep": keep}}}


def cfg_a():
    """Odd sizes everywhere; a shared layer; a layer without feed-forward; partial rotation in the retention."""
    la = latent(3, 20, 12, 28, 40, 36, 0.21, 1000.0)
    m = moe(6, 3, 2, 3, 2, 40)
    return {"architecture": "Zenasun", "vocab": 131, "width": 72, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0}, "logit_softcap": 12.0,
            "layers": [
                {"type": "retention", "mlp": m, "mixer": {"heads": 2, "dim": 24, "vdim": 40, "decay": [0.9, 0.995], "rot": {"base": 300.0, "dims": 16}}},
                {"type": "latent_attention", "mlp": m, "mixer": la},
                {"type": "latent_attention", "mlp": None, "mixer": latent(5, 8, 4, 8, 16, 12, 0.4)},
                {"type": "latent_attention", "mlp": m, "mixer": la, "weights_of": 1},
                {"type": "retention", "mlp": None, "mixer": {"heads": 3, "dim": 10, "vdim": 6, "decay": [1.0, 0.5, 0.97], "rot": {"base": 50.0, "dims": 10}}},
            ]}


def cfg_b():
    """One expert per token, one group, no identity experts, no soft cap, embedding scale 1, a latent above 64 and 128."""
    return {"architecture": "Zenasun", "vocab": 90, "width": 64, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
            "layers": [
                {"type": "latent_attention", "mlp": moe(4, 0, 1, 1, 1, 24), "mixer": latent(2, 16, 8, 16, 24, 72, 0.25)},
                {"type": "retention", "mlp": moe(5, 1, 3, 2, 2, 16), "mixer": {"heads": 1, "dim": 48, "vdim": 16, "decay": [0.99], "rot": {"base": 1e4, "dims": 48}}},
                {"type": "latent_attention", "mlp": moe(8, 4, 4, 4, 2, 32), "mixer": latent(4, 12, 6, 10, 20, 136, 0.3)},
            ]}


def cfg_c():
    """Shapes that take the chunk-parallel retention, the sorted expert path with many tokens and 16-byte weight rows."""
    return {"architecture": "Zenasun", "vocab": 200, "width": 128, "norm": {"eps": 1e-6}, "embedding": {"scale": 5.0}, "logit_softcap": 20.0,
            "layers": [
                {"type": "latent_attention", "mlp": moe(8, 2, 3, 5, 3, 64), "mixer": latent(4, 32, 16, 24, 48, 40, 0.15, 3e5)},
                {"type": "retention", "mlp": moe(8, 2, 3, 5, 3, 64), "mixer": {"heads": 4, "dim": 32, "vdim": 64, "decay": [0.97, 0.99, 0.995, 0.999],
                                                                             "rot": {"base": 2e5, "dims": 32}}},
                {"type": "retention", "mlp": moe(8, 2, 3, 5, 3, 64), "mixer": {"heads": 4, "dim": 32, "vdim": 64, "decay": [0.97, 0.99, 0.995, 0.999],
                                                                             "rot": {"base": 2e5, "dims": 32}}, "weights_of": 1},
            ]}


def cfg_d():
    """Nothing is a multiple of 4 or 8 where it need not be: rows of weights, caches and products start unaligned."""
    la = latent(3, 10, 6, 14, 18, 30, 0.27, 2000.0)
    m = moe(5, 1, 2, 3, 2, 26)
    return {"architecture": "Zenasun", "vocab": 101, "width": 70, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.5}, "logit_softcap": 9.0,
            "layers": [
                {"type": "latent_attention", "mlp": m, "mixer": la},
                {"type": "retention", "mlp": m, "mixer": {"heads": 3, "dim": 14, "vdim": 10, "decay": [0.99, 0.9, 0.999], "rot": {"base": 77.0, "dims": 6}}},
                {"type": "latent_attention", "mlp": m, "mixer": la, "weights_of": 0},
            ]}


CONFIGS = {"a": cfg_a, "b": cfg_b, "c": cfg_c, "d": cfg_d}


def random_weights(cfg, seed=1):
    """bf16-representable float32 tensors on the CPU under the family's tensor names."""
    g = torch.Generator().manual_seed(seed)
    D, W = cfg["width"], {}

    def rnd(*shape, std=1.0, mean=0.0):
        return (mean + std * torch.randn(*shape, generator=g)).bfloat16().float()

    def lin(o, i, gain=1.0):
        return rnd(o, i, std=gain / math.sqrt(i))

    W["embed"], W["final.norm"] = rnd(cfg["vocab"], D, std=0.5), rnd(D, std=0.2)
    for i, layer in enumerate(cfg["layers"]):
        if layer.get("weights_of") is not None:
            continue
        p, m, c = f"l{i}.", f"l{i}.mix.", layer["mixer"]
        W[p + "norm1"] = rnd(D, std=0.2)
        if layer["type"] == "latent_attention":
            H, dn, dr, dv, rq, rk = c["heads"], c["dim"], c["rot_dim"], c["vdim"], c["q_rank"], c["kv_rank"]
            W[m + "dq"], W[m + "dq.norm"], W[m + "uq"] = lin(rq, D), rnd(rq, std=0.2, mean=1.0), lin(H * (dn + dr), rq, 2.0)
            W[m + "dkv"], W[m + "dkv.norm"] = lin(rk + dr, D), rnd(rk, std=0.2, mean=1.0)
            W[m + "uk"], W[m + "uv"], W[m + "sink"], W[m + "o"] = lin(H * dn, rk, 2.0), lin(H * dv, rk), rnd(H, std=1.0), lin(D, H * dv)
        else:
            H, K, V = c["heads"], c["dim"], c["vdim"]
            W[m + "q"], W[m + "k"], W[m + "v"], W[m + "g"], W[m + "o"] = lin(H * K, D), lin(H * K, D), lin(H * V, D), lin(H * V, D), lin(D, H * V)
        if layer.get("mlp"):
            r, ff = layer["mlp"]["router"], layer["mlp"]["expert"]["ff"]
            n = r["experts"] + r["identity"]
            W[p + "norm2"], W[p + "mlp.router"], W[p + "mlp.correction"] = rnd(D, std=0.2), lin(n, D, 3.0), rnd(n, std=0.05)
            for e in range(r["experts"]):
                q = f"{p}mlp.e{e}."
                W[q + "gate"], W[q + "up"], W[q + "down"] = lin(ff, D), lin(ff, D), lin(D, ff)
    return W


def build(cfg, dtype, seed=1, n_slots=3, max_positions=512):
    P, S, M = _pkg()
    W = random_weights(cfg, seed)
    model = P.Zenasun(P.ZenasunConfig.from_dict(cfg), {k: v.to(DEV, dtype) for k, v in W.items()}, max_positions=max_positions)
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
@pytest.mark.parametrize("name", ["a", "b", "c", "d"])
def test_model_matches_the_oracle_layer_by_layer_f32(name):
    cfg = CONFIGS[name]()
    model, engine, W = build(cfg, torch.float32)
    toks = tokens_of(cfg, 75 if name == "d" else 45)     # d: long enough for the expanded attention form
    cap = []
    want = O.model(toks, cfg, W, capture=cap)
    model.capture_layers = []
    got = run_whole(engine, toks)
    for i, (g, w) in enumerate(zip(model.capture_layers, cap)):
        assert rel(g, w) < 2e-5, (name, "layer", i, rel(g, w))
    assert rel(got, want) < 2e-5


@pytest.mark.parametrize("name", ["a", "b", "c", "d"])
def test_model_bf16_is_close_to_the_oracle(name):
    cfg = CONFIGS[name]()
    model, engine, W = build(cfg, torch.bfloat16)
    toks = tokens_of(cfg, 80 if name == "d" else 40)
    want = O.model(toks, cfg, W)
    got = run_whole(engine, toks)
    assert rel(got, want) < 0.1, rel(got, want)      # a routing flip on a close call moves one token a lot
    again = run_pieces(engine, toks, [7, 1, 2, 13])
    assert rel(again, got) < 0.05


@pytest.mark.parametrize("name", ["a", "b", "c", "d"])
def test_portions_and_single_tokens_equal_the_whole_prompt(name):
    cfg = CONFIGS[name]()
    n = 300 if name == "c" else 70          # c: long enough for the chunk-parallel retention and key splits
    model, engine, W = build(cfg, torch.float32)
    toks = tokens_of(cfg, n)
    whole = run_whole(engine, toks)
    if name != "c":
        assert rel(whole, O.model(toks, cfg, W)) < 2e-5
    for sizes in ([1], [2], [3, 2, 17, 1, 5], [33, 64], [n - 9, 1, 1, 2]):
        if name == "c" and sizes == [1]:
            sizes = [n - 40, 1]             # a long first portion, then token by token through the captured step
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


def test_long_decoding_through_the_captured_step():
    cfg = cfg_b()
    model, engine, W = build(cfg, torch.float32)
    toks = tokens_of(cfg, 210)
    want = O.model(toks, cfg, W)
    first = engine.step([{"id": "d", "tokens": toks[:20], "want": [19]}])[0]
    outs = [first] + [engine.step([{"id": "d", "tokens": [t], "want": [0]}])[0] for t in toks[20:]]
    assert engine._graph is not None
    assert rel(torch.cat(outs), want[19:]) < 2e-5
    # the same captured step serves another request in another slot from position 0
    outs2 = [engine.step([{"id": "e", "tokens": [t], "want": [0]}])[0] for t in toks[:30]]
    assert rel(torch.cat(outs2), want[:30]) < 2e-5


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
        assert type(model).__name__ == "Zenasun" and model.max_positions == 64
        assert rel(run_whole(P.Engine(model, n_slots=1), toks), want) < tol
    with pytest.raises(Exception):
        P.Engine(model, n_slots=1).step([{"id": 0, "tokens": [1] * 65, "want": []}])      # more positions than a slot holds


# ----------------------------------------------------------------------------- mechanisms alone
def _ctx(M, P, mixer, T, pos0, dtype, slot=0, pool=None, hint=True):
    pool = pool or P.SequenceStatePool(mixer.state_specs(), 2, torch.device(DEV))
    meta = torch.tensor([slot, pos0], dtype=torch.int32, device=DEV)
    return M.StepContext(T, meta, pool.tensors, dtype, pos_hint=pos0 if hint else None, slot_hint=slot if hint else None), pool, meta


@pytest.mark.parametrize("sizes", [(3, 20, 12, 28, 40, 36), (1, 8, 2, 4, 8, 70), (6, 16, 16, 16, 32, 150), (2, 4, 6, 300, 12, 260)])
def test_latent_attention_alone(sizes):
    P, S, M = _pkg()
    H, dn, dr, dv, rq, rk = sizes
    D, T, eps = 48, 90, 1e-5          # 90 x 3 heads: the latent form takes 8 rows per warp at the first shape
    m = latent(H, dn, dr, dv, rq, rk, 0.2, 777.0)
    W = {k[len("l0."):]: v for k, v in random_weights({"vocab": 8, "width": D, "layers": [{"type": "latent_attention", "mixer": m, "mlp": None}]}, 2).items()
         if k.startswith("l0.mix.")}
    h = torch.randn(T, D).bfloat16().float()
    want = O.latent_attention(h.double(), {k: v.double() for k, v in W.items()}, "mix.", m, eps)
    mixer = M.LatentAttention("x", {k: v.to(DEV) for k, v in W.items()}, "mix.", heads=H, dim=dn, rot_dim=dr, vdim=dv, q_rank=rq, kv_rank=rk,
                              scale=0.2, eps=eps, rot=m["rot"], max_positions=128)
    ctx, pool, meta = _ctx(M, P, mixer, T, 0, torch.float32, slot=1)
    got = mixer.forward(h.to(DEV), ctx)                                   # a long portion: expanded keys and values per head
    assert rel(got, want) < 2e-5
    mixer.expand_from = 10 ** 9
    assert rel(mixer.forward(h.to(DEV), ctx), want) < 2e-5                # the same portion in the latent space
    mixer.expand_from = 40
    # the same in three portions on the other slot (latent, expanded over older positions, latent on a fixed grid)
    outs, at = [], 0
    for n, hint in ((31, True), (58, True), (1, False)):
        ctx, pool, meta = _ctx(M, P, mixer, n, at, torch.float32, slot=0, pool=pool, hint=hint)
        outs.append(mixer.forward(h[at:at + n].to(DEV), ctx))
        at += n
    assert rel(torch.cat(outs), want) < 2e-5


def _latent_kernel(S, cache, q_lat, q_rot, sink, scale, pos0, splits, slot=0):
    """The attention kernel in its latent form on a cache filled by the test: q_lat [T, H, rank], q_rot [T, H, rot];
    returns [T, H, rank]."""
    T, H, rank = q_lat.shape
    rot = q_rot.shape[2]
    out = torch.empty(T, H * rank, device=DEV)
    work = torch.empty(max(splits, 1), T * H, rank + 2, device=DEV)
    meta = torch.tensor([slot, pos0], dtype=torch.int32, device=DEV)
    ql, qr = q_lat.to(DEV).contiguous(), q_rot.to(DEV).contiguous()
    Kd = rank + rot
    a = S.LatentAttnArgs(q_a=ql.data_ptr(), ldqa_t=H * rank, ldqa_h=rank, q_b=qr.data_ptr(), ldqb_t=H * rot, ldqb_h=rot, key_a=cache.data_ptr(), ldka=Kd,
                         hska=0, slot_stride_a=cache.shape[1] * Kd, key_b=cache.data_ptr() + 4 * rank, ldkb=Kd, slot_stride_b=cache.shape[1] * Kd,
                         sink=sink.data_ptr(), meta=meta.data_ptr(), out=out.data_ptr(), ldo=H * rank, work=work.data_ptr(), scale=scale, T=T, heads=H,
                         heads_per_group=H, n_a=rank, n_b=rot, vdim=rank, score_off=0, splits=splits, act_dtype=S.B2L_F32)
    S.check(S.lib().b2l_seq_latent_attention(C.byref(a), torch.cuda.current_stream().cuda_stream), "b2l_seq_latent_attention")
    torch.cuda.synchronize()
    return out.view(T, H, rank).cpu()


def _latent_plain(cache, q_lat, q_rot, sink, scale, pos0):
    T, H, rank = q_lat.shape
    out = torch.zeros(T, H, rank, dtype=torch.float64)
    for t in range(T):
        keys = cache[: pos0 + t + 1].double()
        for h in range(H):
            s = (keys[:, :rank] @ q_lat[t, h].double() + keys[:, rank:] @ q_rot[t, h].double()) * scale
            mx = max(float(s.max()), float(sink[h]))
            e = torch.exp(s - mx)
            out[t, h] = (e / (e.sum() + math.exp(float(sink[h]) - mx))) @ keys[:, :rank]
    return out


@pytest.mark.parametrize("splits", [1, 3, 7])
def test_latent_attention_far_keys_and_the_causal_edge(splits):
    """One key made dominant by a large matching query: far back among hundreds, on both sides of tile borders (32
    keys) and of split borders, on the query's own position (seen) and one after it (not seen)."""
    P, S, M = _pkg()
    rank, rot, H, n = 20, 6, 3, 400
    g = torch.Generator().manual_seed(9)
    base = torch.randn(2, 512, rank + rot, generator=g)
    sink = torch.tensor([-30.0, 0.0, 2.0])
    sink_d = sink.to(DEV)
    pos0 = n - 2                               # two queries at positions n-2 and n-1
    for target in (0, 1, 31, 32, 33, 63, 64, 133, 134, 255, 256, n - 3, n - 2, n - 1):
        q_lat = 0.05 * torch.randn(2, H, rank, generator=g)
        q_rot = 0.05 * torch.randn(2, H, rot, generator=g)
        cache = base.clone()
        cache[1, target, :rank] *= 3.0                               # a long key, and a query along it: its score stands out by > 30
        q_lat[:, 0] += 4.0 * cache[1, target, :rank] / cache[1, target, :rank].norm()
        cache_d = cache.to(DEV)
        got = _latent_kernel(S, cache_d, q_lat, q_rot, sink_d, 1.0, pos0, splits, slot=1)
        want = _latent_plain(cache[1], q_lat, q_rot, sink, 1.0, pos0)
        assert rel(got, want) < 2e-5, (target, rel(got, want))
        hit = [float(torch.dist(got[t, 0], cache[1, target, :rank]) / cache[1, target, :rank].norm()) for t in range(2)]
        if target <= n - 2:
            assert hit[0] < 0.05 and hit[1] < 0.05, (target, hit)
        else:                                                       # position n-1 is after the first query: it must not see it
            assert hit[0] > 0.5 and hit[1] < 0.05, (target, hit)


def test_latent_attention_sink_takes_its_share():
    P, S, M = _pkg()
    rank, rot, H = 8, 2, 4
    cache = torch.randn(1, 64, rank + rot)
    q_lat, q_rot = torch.zeros(1, H, rank), torch.zeros(1, H, rot)       # all scores 0: weights 1 / (n + exp(sink))
    sink = torch.tensor([-100.0, 0.0, math.log(10.0), 50.0])
    for pos0 in (0, 9, 40):
        got = _latent_kernel(S, cache.to(DEV), q_lat, q_rot, sink.to(DEV), 0.3, pos0, 1)
        keys = cache[0, : pos0 + 1, :rank].double()
        for h in range(H):
            want = keys.sum(0) / (pos0 + 1 + math.exp(float(sink[h])))
            assert torch.allclose(got[0, h].double(), want, rtol=1e-5, atol=1e-7), (pos0, h)


@pytest.mark.parametrize("H,K,V,dims", [(2, 24, 40, 16), (1, 48, 16, 48), (3, 10, 6, 10), (4, 32, 64, 32)])
def test_retention_alone(H, K, V, dims):
    P, S, M = _pkg()
    D, T, eps = 40, 300, 1e-5
    m = {"heads": H, "dim": K, "vdim": V, "decay": [1.0, 0.9, 0.99, 0.999][:H], "rot": {"base": 123.0, "dims": dims}}
    W = {k[len("l0."):]: v for k, v in random_weights({"vocab": 8, "width": D, "layers": [{"type": "retention", "mixer": m, "mlp": None}]}, 4).items()
         if k.startswith("l0.mix.")}
    h = torch.randn(T, D).bfloat16().float()
    want, S_want = O.retention(h.double(), {k: v.double() for k, v in W.items()}, "mix.", m, eps)
    mixer = M.RetentionMixer("r", {k: v.to(DEV) for k, v in W.items()}, "mix.", heads=H, dim=K, vdim=V, decay=m["decay"], eps=eps, rot=m["rot"])
    ctx, pool, meta = _ctx(M, P, mixer, T, 0, torch.float32, slot=1)
    got = mixer.forward(h.to(DEV), ctx)                                  # one portion: chunk-parallel form
    assert rel(got, want) < 2e-5
    assert rel(pool.tensors["r.S"][1].transpose(1, 2), S_want) < 2e-5     # the state is stored [heads][vdim][dim]
    outs, at = [], 0
    for n in (1, 2, 60, 1, 236):                                         # carried state, sequential form
        ctx, pool, meta = _ctx(M, P, mixer, n, at, torch.float32, slot=0, pool=pool)
        outs.append(mixer.forward(h[at:at + n].to(DEV), ctx))
        at += n
    assert rel(torch.cat(outs), want) < 2e-5


@pytest.mark.parametrize("E,I,top,count,keep", [(6, 3, 2, 3, 2), (4, 0, 1, 1, 1), (8, 4, 4, 4, 2), (30, 10, 6, 8, 3), (5, 1, 3, 2, 2), (12, 4, 4, 4, 3)])
def test_router_and_experts(E, I, top, count, keep):
    P, S, M = _pkg()
    D, ff, T = 40, 24, 50
    mlp = moe(E, I, top, count, keep, ff)
    cfg = {"vocab": 8, "width": D, "layers": [{"type": "retention", "mixer": {"heads": 1, "dim": 2, "vdim": 2, "decay": [1.0]}, "mlp": mlp}]}
    W = {k[len("l0."):]: v for k, v in random_weights(cfg, 6).items() if k.startswith("l0.mlp.")}
    W["mlp.correction"] = (0.3 * torch.randn(E + I)).bfloat16().float()          # large enough to change choices, also negative
    h = torch.randn(T, D).bfloat16().float()
    Wd = {k: v.double() for k, v in W.items()}
    idx_want, w_want = O.route(h.double(), Wd, "mlp.", mlp["router"])
    choice = torch.softmax(h.double() @ Wd["mlp.router"].T, -1) + Wd["mlp.correction"]
    ff_layer = M.MoEFeedForward({k: v.to(DEV) for k, v in W.items()}, "mlp.", experts=E, identity=I, top=top, groups=count, keep=keep, ff=ff)
    ctx = M.StepContext(T, torch.zeros(2, dtype=torch.int32, device=DEV), {}, torch.float32)
    idx, wgt = ff_layer.route(h.to(DEV), ctx)
    srt = choice.sort(dim=-1).values
    clear = (srt[:, 1:] - srt[:, :-1]).min(dim=-1).values > 1e-5             # no two choice scores nearly equal
    assert int(clear.sum()) > T // 2
    assert torch.equal(idx.cpu().long()[clear], idx_want[clear])
    assert torch.allclose(wgt.cpu().double()[clear], w_want[clear], rtol=1e-5, atol=1e-7)
    c3 = M.StepContext(3, ctx.meta, {}, torch.float32)                         # a few tokens: logits and routing in one launch
    idx3, wgt3 = ff_layer.route(h[:3].to(DEV), c3)
    assert torch.equal(idx3.cpu().long()[clear[:3]], idx_want[:3][clear[:3]])
    assert torch.allclose(wgt3.cpu().double()[clear[:3]], w_want[:3][clear[:3]], rtol=1e-5, atol=1e-7)
    if I:
        assert int((idx_want >= E).sum()) > 0                                 # identity experts are exercised
    want = O.moe(h.double(), Wd, "mlp.", mlp)
    got_sorted = ff_layer.forward(h.to(DEV), ctx)
    assert rel(got_sorted[clear.to(DEV)], want[clear]) < 2e-5
    outs = []
    for t in range(0, 12, 3):                                                 # a few tokens: indices read on the device
        c = M.StepContext(3, ctx.meta, {}, torch.float32)
        outs.append(ff_layer.forward(h[t:t + 3].to(DEV), c))
    small = torch.cat(outs)
    assert rel(small[clear[:12].to(DEV)], want[:12][clear[:12]]) < 2e-5


def test_group_limit_and_negative_choice_scores():
    """The best expert of a group that is not kept is never chosen, also when every allowed choice score is negative."""
    P, S, M = _pkg()
    n, T = 8, 1
    z = torch.tensor([[0.0, 0.1, 5.0, 0.2, 0.3, 0.0, 0.1, 0.2]])                # expert 2 has by far the largest score
    corr = torch.tensor([-2.0, -2.0, -3.0, -3.0, -2.0, -2.0, -2.0, -1.5])       # ... but its group (2, 3) ends up worst
    idx = torch.empty(T, 2, dtype=torch.int32, device=DEV)
    wgt = torch.empty(T, 2, device=DEV)
    zd, cd = z.to(DEV), corr.to(DEV)
    S.check(S.lib().b2l_seq_moe_route(zd.data_ptr(), n, cd.data_ptr(), n, 4, 3, 2, S.SCORE_SOFTMAX, 1, 1, 1.0, idx.data_ptr(), wgt.data_ptr(), T, None), "route")
    s = torch.softmax(z.double(), -1)[0]
    choice = s + corr.double()
    assert float(choice[2]) < float(choice.max()) and 2 not in idx.cpu().tolist()[0]
    allowed = [i for i in range(n) if i // 2 != 1]
    best = sorted(allowed, key=lambda i: -float(choice[i]))[:2]
    assert idx.cpu().tolist()[0] == best
    assert torch.allclose(wgt.cpu().double()[0], s[best] / s[best].sum(), rtol=1e-5)
    # with every group kept the same expert wins on its choice score only if the correction lets it
    S.check(S.lib().b2l_seq_moe_route(zd.data_ptr(), n, None, n, 4, 4, 2, S.SCORE_SOFTMAX, 1, 1, 1.0, idx.data_ptr(), wgt.data_ptr(), T, None), "route")
    assert idx.cpu().tolist()[0][0] == 2


def test_norm_pair_and_softcap_and_rotation():
    P, S, M = _pkg()
    lib = S.lib()
    T, D = 7, 50
    x = torch.randn(T, D)
    y1, y2 = torch.randn(T, D), torch.randn(T, D)
    w1, w2 = 0.2 * torch.randn(D), 0.2 * torch.randn(D)
    xd, h1, h2 = x.to(DEV), torch.empty(T, D, device=DEV), torch.empty(T, D, device=DEV)
    a, b, c, d = y1.to(DEV), y2.to(DEV), w1.to(DEV), w2.to(DEV)
    S.check(lib.b2l_seq_add_norm2(a.data_ptr(), b.data_ptr(), xd.data_ptr(), c.data_ptr(), h1.data_ptr(), d.data_ptr(), h2.data_ptr(), 1.0, 1e-5,
                                  None, T, D, S.B2L_F32, None), "add_norm2")
    xs = x.double() + (y1.double() + y2.double())
    assert rel(xd, xs) < 1e-6
    assert rel(h1, O.norm_around_zero(xs, w1.double(), 1e-5)) < 1e-6 and rel(h2, O.norm_around_zero(xs, w2.double(), 1e-5)) < 1e-6
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
    hn = torch.empty(3, D, device=DEV)
    S.check(lib.b2l_seq_add_norm2(None, None, xd.data_ptr(), c.data_ptr(), hn.data_ptr(), None, None, 1.0, 1e-5, rows.data_ptr(), 3, D, S.B2L_F32,
                                  None), "add_norm2 rows")
    assert rel(hn, O.norm_around_zero(xs[[5, 0, 5]], w1.double(), 1e-5)) < 1e-6
    z = (40 * torch.randn(1000)).to(DEV)
    want = 7.0 * torch.tanh(z.double().cpu() / 7.0)
    S.check(lib.b2l_seq_softcap(z.data_ptr(), z.numel(), 7.0, None), "softcap")
    assert rel(z, want) < 1e-6
    # rotation: both layouts, an offset inside the head, a multiplier, positions from the device pair
    H, size, off, dims = 3, 14, 4, 8
    v = torch.randn(T, H * size)
    meta = torch.tensor([0, 100], dtype=torch.int32, device=DEV)
    freq = torch.tensor([100.0 ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float32, device=DEV)
    for inter in (0, 1):
        out = torch.empty(T, H * size, device=DEV)
        vd = v.to(DEV)
        S.check(lib.b2l_seq_rope(vd.data_ptr(), H * size, 1, freq.data_ptr(), dims, inter, off, 0.5, 1.0, meta.data_ptr(), out.data_ptr(), H * size, 1, T, H,
                                 size, size, size, S.B2L_F32, None), "rope")
        want = v.double().view(T, H, size).clone()
        for hd in range(H):
            want[:, hd, off:] = O.rotate(want[:, hd, off:], torch.arange(100, 100 + T), dims, 100.0, bool(inter))
        assert rel(out, 0.5 * want.view(T, H * size)) < 2e-5       # the angle itself is an f32 product
