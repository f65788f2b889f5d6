"""Throughput of the Zuvevik family beside the package's Lugovik family at equal width and depth
(`bench.py --family zuvevik`).

Random weights, bf16, one sequence: prefill of a `prompt`-token prompt in one portion, then single-token decoding
through the engine (CUDA-graph replay).  The Lugovik arm is the closest served model: the same engine, state pool,
library products and attention kernels (block-local there, a sliding window here), a dense gated feed-forward.  A
second table times the family's mechanisms alone at the model's shapes with their algorithmic bytes and flops, each
next to the like kernel of the closest model run on the same operands: the attention kernel in its block-local form
with a sink and a gate per head, the residual step of one stream, routed experts with softmax scores and weights on the
outputs.  CUDA events, warm-up, L2 flushed between iterations."""
import ctypes as C
import json
import os
import time
from typing import List

import torch

from . import seq_bench

SIZES = {
    # a dense first layer, routed experts in the others; the window is half the default prompt
    "1k": dict(width=1024, layers=8, heads=8, kv_heads=2, dim=128, vdim=128, window=1024, streams=4, ff=4096, experts=16, top=2, eff=1024,
               vocab=32000),
    "2k": dict(width=2048, layers=8, heads=16, kv_heads=4, dim=128, vdim=128, window=1024, streams=4, ff=8192, experts=32, top=4, eff=1024,
               vocab=32000),
    "4k": dict(width=4096, layers=8, heads=32, kv_heads=8, dim=128, vdim=128, window=1024, streams=4, ff=11008, experts=32, top=4, eff=2048,
               vocab=32000),
}


def zuvevik_config(width, layers, heads, kv_heads, dim, vdim, window, streams, ff, experts, top, eff, vocab) -> dict:
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window}, "scale": dim ** -0.5, "v_mix": True,
             "rot": {"base": 1e6, "dims": dim}}
    dense = {"kind": "dense", "ff": ff}
    routed = {"kind": "moe", "expert": {"ff": eff, "limit": 7.0}, "router": {"experts": experts, "top": top}}
    return {"architecture": "Zuvevik", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "streams": streams, "logit_scale": 1.0,
            "embedding": {"bigram": {"buckets": 65521, "mul_prev": 40503, "mul_cur": 2654435}},
            "layers": [{"type": "attention", "mixer": mixer, "mlp": dense if i == 0 else routed} for i in range(layers)]}


def _throughput(engine, toks, prompt, decode_steps, device, timer):
    n = [0]

    def prefill():
        n[0] += 1
        engine.step([{"id": n[0], "tokens": toks[:prompt], "want": [prompt - 1]}], end=[n[0]])

    t_pre = timer(prefill, iters=3, warmup=2)
    engine.step([{"id": "d", "tokens": toks[:prompt], "want": []}])
    for i in range(4):                                    # warm the single-token graph
        engine.step([{"id": "d", "tokens": [toks[prompt + i]], "want": [0]}])
    torch.cuda.synchronize(device)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(4, decode_steps):
        engine.step([{"id": "d", "tokens": [toks[prompt + i]], "want": [0]}])
    b.record()
    torch.cuda.synchronize(device)
    engine.step([], end=["d"])
    return t_pre, a.elapsed_time(b) * 1e-3 / (decode_steps - 4)


def kernel_table(model, engine, T: int, device, timer, peaks: dict) -> List[dict]:
    """The family's mechanisms alone at this model's shapes, each followed by the like kernel of the closest model on
    the same operands: a T-token portion from position 0 and one token at position T - 1 (a full window, and the last
    position of a block)."""
    from . import _seqlib as S
    from . import mixers as M

    rows, hbm, es = [], peaks["hbm_gbs"] * 1e9, 2
    slot = engine.pool.acquire("kernels")
    D, dt, lib, n_s, eps = model.width, model.dtype, S.lib(), model.streams, model.eps
    att = model.layers[1].mixer                          # a layer that mixes its values with the first layer's
    moe = next(l.mlp for l in model.layers if isinstance(l.mlp, M.MoEFeedForward))
    dense = next(l.mlp for l in model.layers if isinstance(l.mlp, M.GatedMLP))
    hc = model.sublayers[0].hc
    H, G, K, V, Wn = att.H, att.G, att.K, att.V, att.window

    def add(name, tt, t, nbytes, flops=0.0, note=""):
        rows.append({"kernel": name, "tokens": int(tt), "us": t * 1e6, "GB_s": nbytes / t / 1e9, "frac_of_measured_hbm": nbytes / t / hbm,
                     "GFLOP_s": flops / t / 1e9, "note": note})

    # fill the ring of the slot, so that a single token at position T has a full window to read
    full = M.StepContext(T, torch.tensor([slot, 0], dtype=torch.int32, device=device), engine.pool.tensors, dt, pos_hint=0, slot_hint=slot)
    att.forward(torch.randn(T, D, device=device).to(dt), full)
    ck, cv = engine.pool.tensors[att.name + ".k"], engine.pool.tensors[att.name + ".v"]
    for tt, pos0 in ((T, 0), (1, T - 1)):
        meta = torch.tensor([slot, pos0], dtype=torch.int32, device=device)
        ctx = M.StepContext(tt, meta, engine.pool.tensors, dt, pos_hint=pos0 if tt > 1 else None, slot_hint=slot if tt > 1 else None)
        hh = torch.randn(tt, D, device=device).to(dt)
        y = torch.randn(tt, D, device=device).to(dt)
        w = torch.ones(D, dtype=dt, device=device)
        # ---- residual step: the write of one sublayer, the read and the norm of the next
        X = torch.randn(tt, n_s, D, device=device)
        t = timer(lambda: M.HyperConnection.step(X, ctx, y=y, wrote=hc, reads=hc, norm=w, eps=eps))
        add(f"seq_hc_step_kernel ({n_s} streams: write + read + norm)", tt, t, tt * D * (es + 8 * n_s + es))
        x1 = torch.randn(tt, D, device=device)
        h1 = torch.empty(tt, D, dtype=dt, device=device)
        t = timer(lambda: S.check(lib.b2l_seq_norm_add_norm(M._p(y), M._p(w), eps, M._p(x1), M._p(w), M._p(h1), tt, D, ctx.act, ctx.stream), "k"))
        add("  like: seq_norm_add_norm_kernel (one stream: post-norm + add + norm)", tt, t, tt * D * (es + 4 + 4 + es))
        # ---- embedding: the token row plus the hashed pair row into every stream, against the plain embedding
        emb = model.embedding
        tk = torch.randint(0, emb.vocab, (tt,), device=device)
        t = timer(lambda: emb.forward(tk, ctx))
        add(f"seq_embed_pair_kernel (token + pair rows into {n_s} streams)", tt, t, tt * D * (2 * es + 4 * n_s))
        t = timer(lambda: S.check(lib.b2l_seq_embed(M._p(tk), 1, M._p(emb.embed), ctx.act, 1.0, M._p(x1), tt, D, emb.vocab, ctx.stream), "k"))
        add("  like: seq_embed_kernel (token row into one stream)", tt, t, tt * D * (es + 4))
        # ---- attention operands
        proj = torch.randn(tt, att.w_in.shape[0], device=device).to(dt)
        ld = proj.shape[1]
        q = torch.empty(tt, H * K, device=device)
        kn = torch.empty(tt, G * K, dtype=dt, device=device)
        vm = torch.empty(tt, G * V, dtype=dt, device=device)
        vf = torch.randn(tt, G * V, device=device).to(dt)
        a = S.QkvPrepArgs(proj=M._p(proj), ld=ld, q_off=att.o_q, k_off=att.o_k, v_off=att.o_v, q_norm=M._p(att.q_norm), k_norm=M._p(att.k_norm),
                          whole_row=1, eps=eps, freq=M._p(att.freq), rot_dims=att.rot_dims, rot_mult=1.0, meta=M._p(meta), q_out=M._p(q),
                          k_out=M._p(kn), v_first=M._p(vf), ldvf=G * V, lambda_=M._p(att.lam), v_out=M._p(vm), T=tt, heads=H, kv_heads=G, K=K, V=V,
                          act_dtype=ctx.act)
        t = timer(lambda: S.check(lib.b2l_seq_qkv_prep(C.byref(a), ctx.stream), "k"))
        add("seq_qkv_prep_kernel (q/k norm over the projection + rotation + value mixing)", tt, t,
            tt * ((H + G) * K * es + H * K * 4 + G * K * es + 3 * G * V * es))
        wk = torch.ones(K, dtype=dt, device=device)

        def two_norms():
            S.check(lib.b2l_seq_headnorm_rope(M._p(proj, att.o_q), ld, M._p(wk), eps, M._p(att.freq), att.rot_dims, 1.0, M._p(meta), M._p(q), 1, tt,
                                              H, K, ctx.act, ctx.stream), "k")
            S.check(lib.b2l_seq_headnorm_rope(M._p(proj, att.o_k), ld, M._p(wk), eps, M._p(att.freq), att.rot_dims, 1.0, M._p(meta), M._p(kn), 0, tt,
                                              G, K, ctx.act, ctx.stream), "k")

        t = timer(two_norms)
        add("  like: 2 x seq_headnorm_rope_kernel (per-head norm + rotation, no value mixing)", tt, t, tt * ((H + G) * K * es + H * K * 4 + G * K * es))
        # ---- the attention kernel alone: sliding window against the block-local form on the same operands
        out = torch.empty(tt, H * V, dtype=dt, device=device)
        qr = torch.randn(tt, H * K, device=device)
        kr = torch.randn(tt, G * K, device=device).to(dt)
        if tt > 1:
            keys = (min(T, Wn) * (min(T, Wn) + 1) / 2 + max(0, T - Wn) * Wn) / T
            keys_block = sum(min(Wn, T - b0) * (min(Wn, T - b0) + 1) / 2 for b0 in range(0, T, Wn)) / T
        else:
            keys, keys_block = min(T, Wn), (T - 1) % Wn + 1
        for name, window, sink, per_channel, gate, ldg, kq in (
                ("seq_block_attention (sliding window, softmax, gate per channel) + ring append", Wn, 0, 1, M._p(proj, att.o_g), ld, keys),
                ("  like: seq_block_attention (block-local, sink, gate per head) + ring append", 0, 1, 0, M._p(proj, att.o_g), ld, keys_block)):
            b = S.AttnArgs(q=M._p(qr), k_new=M._p(kr), v_new=M._p(vm), ldv=G * V, cache_k=M._p(ck), cache_v=M._p(cv), meta=M._p(meta), gate=gate,
                           ldg=ldg, out=M._p(out), ldo=H * V, scale=att.scale, softcap=0.0, out_mult=1.0, has_sink=sink, block=Wn, T=tt, heads=H,
                           kv_heads=G, K=K, V=V, act_dtype=ctx.act, window=window, gate_per_channel=per_channel)
            t = timer(lambda: M.local_attention(b, ctx))
            nb = tt * (H * K * 4 + G * (K + V) * es * 2 + H * V * es * (2 if per_channel else 1)) + (kq * G * (K + V) * es if tt == 1 else 0)
            add(name, tt, t, nb, 2.0 * tt * H * kq * (K + V), f"f32 scores on CUDA cores, {kq:.0f} keys per query")
        t = timer(lambda: att.forward(hh, ctx))
        wb = (att.w_in.numel() + att.w_o.numel()) * es
        add("SlidingWindowAttention whole (2 products + operands + attention)", tt, t, wb + 2 * tt * D * es, 2.0 * tt * H * keys * (K + V) + 2.0 * tt * wb / es)
        # ---- feed-forward
        t = timer(lambda: moe.forward(hh, ctx))
        active = moe.top * 3 * moe.ff * D
        wb = min(moe.E, tt * moe.top) * 3 * moe.ff * D * es
        form = "device-indexed expert products" if tt <= moe.SMALL else "sort + weighted gather + grouped library products + combine"
        add("MoEFeedForward whole (sigmoid scores, weights on the input, clamped unit)", tt, t, wb + 2 * tt * D * es, 2.0 * tt * active, form)
        like = M.MoEFeedForward.__new__(M.MoEFeedForward)
        like.__dict__.update(moe.__dict__)
        like.act, like.limit, like.score, like.renorm, like.weight_input, like.correction = S.ACT_SILU, 0.0, S.SCORE_SOFTMAX, 1, 0, None
        t = timer(lambda: like.forward(hh, ctx))
        add("  like: MoEFeedForward whole (softmax scores renormalised, weights on the output, silu unit)", tt, t, wb + 2 * tt * D * es, 2.0 * tt * active, form)
        t = timer(lambda: dense.forward(hh, ctx))
        wb = (dense.w_in.numel() + dense.w_down.numel()) * es
        add("GatedMLP whole (silu; the closest model's feed-forward with another activation)", tt, t, wb + 2 * tt * D * es, 2.0 * tt * wb / es)
    engine.pool.release("kernels")
    return rows


def run_size(name: str, prompt: int, decode_steps: int, device, timer, peaks: dict) -> dict:
    import lit_llama_b200 as P
    from .zuvevik import random_weights

    sz = SIZES[name]
    cfg = zuvevik_config(**sz)
    W = random_weights(cfg, device)
    model = P.Zuvevik(P.ZuvevikConfig.from_dict(cfg), W)
    del W
    engine = P.Engine(model, n_slots=2, prefill_chunk=prompt)
    toks = torch.randint(0, sz["vocab"], (prompt + decode_steps,), generator=torch.Generator().manual_seed(1)).tolist()
    t_pre, t_dec = _throughput(engine, toks, prompt, decode_steps, device, timer)
    params, active = model.n_parameters()
    active -= model.embedding.embed.numel() + (model.embedding.pair.numel() if model.embedding.pair is not None else 0)    # a token reads two rows of them
    state = engine.pool.bytes() // engine.pool.n_slots
    out = {"zuvevik": {"params": params, "active_params_per_token": active, "state_bytes_per_sequence": state,
                       "prefill_tok_s": prompt / t_pre, "prefill_ms": t_pre * 1e3, "decode_tok_s": 1.0 / t_dec, "decode_us": t_dec * 1e6,
                       "decode_frac_of_measured_hbm": (2 * active + state) / t_dec / (peaks["hbm_gbs"] * 1e9)}}
    out["kernels"] = kernel_table(model, engine, prompt, device, timer, peaks)
    del engine, model
    torch.cuda.empty_cache()

    # ---- the closest served family at the same width and depth
    lsz = seq_bench.SIZES[name]
    lcfg = seq_bench.lugovik_config(**lsz)
    LW = seq_bench.random_weights(lcfg, device)
    lug = P.Lugovik(P.LugovikConfig.from_dict(lcfg), LW, max_positions=prompt + decode_steps + 8)
    del LW
    lengine = P.Engine(lug, n_slots=2, prefill_chunk=prompt)
    t_pre2, t_dec2 = _throughput(lengine, toks, prompt, decode_steps, device, timer)
    lp, lstate = lug.n_parameters(), lengine.pool.bytes() // 2
    out["lugovik"] = {"params": lp, "state_bytes_per_sequence": lstate, "prefill_tok_s": prompt / t_pre2, "prefill_ms": t_pre2 * 1e3,
                      "decode_tok_s": 1.0 / t_dec2, "decode_us": t_dec2 * 1e6,
                      "decode_frac_of_measured_hbm": (2 * lp + 2 * lstate) / t_dec2 / (peaks["hbm_gbs"] * 1e9)}
    del lengine, lug
    torch.cuda.empty_cache()
    return out


def run(args, sizes: List[str]) -> dict:
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            peaks = json.load(f)
        peaks["source"] = "measured"
    except OSError:
        peaks = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    timer = seq_bench._Timer(device)
    out = {"metric": "zuvevik_vs_lugovik_throughput", "unit": "tokens/s", "dtype": "bf16", "data": "synthetic (random weights)", "prompt": args.prompt,
           "decode_steps": args.decode_steps, "peaks": {k: peaks[k] for k in ("hbm_gbs", "bf16_tflops", "source")}, "l2": "flushed between timed iterations",
           "sizes": {}}
    t0 = time.time()
    for name in sizes:
        out["sizes"][name] = run_size(name, args.prompt, args.decode_steps, device, timer, peaks)
    out["seconds"] = round(time.time() - t0, 1)
    return out
