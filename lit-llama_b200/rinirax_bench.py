"""Throughput of the Rinirax family beside the package's Zenasun family at equal width and depth
(`bench.py --family rinirax`).

Random weights, bf16, one sequence: prefill of a `prompt`-token prompt in one portion, then single-token decoding
through the engine (CUDA-graph replay).  The Zenasun arm is the closest served model: parallel layers on an f32 residual
stream, latent attention, routed experts, the same engine, state pool and library products.  A second table times the
family's mechanisms alone at the model's shapes with their algorithmic bytes and flops, each next to the like kernel of
the closest model run on operands of the same size: the attention kernel with one map per head, latent attention without a
window and with a sink, the residual step without history, the matrix-state recurrence, the gated activation, the router
whose groups are worth their best member.  CUDA events, warm-up, L2 flushed between iterations."""
import ctypes as C
import json
import os
import time
from typing import List

import torch

from . import seq_bench, zenasun_bench

SIZES = {
    # the layer pattern repeats: attention (dense feed-forward), mingru, attention, latent attention, attention over the keys
    # and values of the attention layer two before it; the others have routed experts.  Two maps of `dim` entries per head.
    "1k": dict(width=1024, layers=8, heads=8, kv_heads=2, dim=64, vdim=128, conv=4, gru=2048, l_heads=8, l_dim=128, l_rot=64, l_vdim=128, q_rank=384,
               kv_rank=256, window=1024, ff=4096, experts=16, top=4, groups=4, keep=2, eff=512, vocab=32000),
    "2k": dict(width=2048, layers=8, heads=16, kv_heads=4, dim=64, vdim=128, conv=4, gru=4096, l_heads=16, l_dim=128, l_rot=64, l_vdim=128, q_rank=768,
               kv_rank=512, window=1024, ff=8192, experts=32, top=6, groups=8, keep=4, eff=1024, vocab=32000),
}


def rinirax_config(width, layers, heads, kv_heads, dim, vdim, conv, gru, l_heads, l_dim, l_rot, l_vdim, q_rank, kv_rank, window, ff, experts, top, groups,
                   keep, eff, vocab) -> dict:
    att = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "diff": 0.4, "scale": dim ** -0.5, "rot": {"base": 1e5, "dims": dim}}
    lat = {"heads": l_heads, "dim": l_dim, "rot_dim": l_rot, "vdim": l_vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": (l_dim + l_rot) ** -0.5,
           "mask": {"size": window}, "rot": {"base": 1e6, "dims": l_rot, "scaling": {"factor": 8.0, "original": 2048, "fast": 32.0, "slow": 1.0}}}
    routed = {"kind": "moe", "expert": {"ff": eff}, "router": {"experts": experts, "top": top, "scale": 2.0, "groups": {"count": groups, "keep": keep}}}
    out = []
    for i in range(layers):
        k = i % 5
        if k == 0:
            out.append({"type": "attention", "mixer": dict(att), "mlp": {"kind": "dense", "ff": ff}})
        elif k == 1:
            out.append({"type": "mingru", "mixer": {"width": gru}, "mlp": routed})
        elif k == 2:
            out.append({"type": "attention", "mixer": dict(att), "mlp": routed})
        elif k == 3:
            out.append({"type": "latent_attention", "mixer": lat, "mlp": routed})
        else:
            out.append({"type": "attention", "mixer": dict(att, kv_from=i - 2), "mlp": routed})
    return {"architecture": "Rinirax", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "layers": out}


def kernel_table(model, engine, T: int, device, timer, peaks: dict) -> List[dict]:
    """The family's mechanisms alone at this model's shapes, each followed by the like kernel of the closest model: a
    T-token portion from position 0 and one token at position T."""
    from . import _seqlib as S
    from . import mixers as M

    rows, hbm, es = [], peaks["hbm_gbs"] * 1e9, 2
    slot = engine.pool.acquire("kernels")
    D, dt, lib, eps, L = model.width, model.dtype, S.lib(), model.eps, len(model.layers)
    att = next(l.mixer for l in model.layers if isinstance(l.mixer, M.DifferentialAttention) and l.mixer.src is None)
    lat = next(l.mixer for l in model.layers if isinstance(l.mixer, M.LatentAttention))
    gru = next(l.mixer for l in model.layers if isinstance(l.mixer, M.MinGRUMixer))
    moe = next(l.mlp for l in model.layers if isinstance(l.mlp, M.MoEFeedForward))
    dense = next(l.mlp for l in model.layers if isinstance(l.mlp, M.DenseMLP))
    H, G, K, V = att.H, att.G, att.K, att.V

    def add(name, tt, t, nbytes, flops=0.0, note=""):
        rows.append({"kernel": name, "tokens": int(tt), "us": t * 1e6, "GB_s": nbytes / t / 1e9, "frac_of_measured_hbm": nbytes / t / hbm,
                     "GFLOP_s": flops / t / 1e9, "note": note})

    # fill the caches of the slot once, so that a single token at position T has T keys (a full window) to read
    full = M.StepContext(T, torch.tensor([slot, 0], dtype=torch.int32, device=device), engine.pool.tensors, dt, pos_hint=0, slot_hint=slot)
    hfull = torch.randn(T, D, device=device).to(dt)
    att.forward(hfull, full)
    lat.forward(hfull, full)
    ck, cv = engine.pool.tensors[att.name + ".k"], engine.pool.tensors[att.name + ".v"]
    for tt, pos0 in ((T, 0), (1, T)):
        meta = torch.tensor([slot, pos0], dtype=torch.int32, device=device)
        ctx = M.StepContext(tt, meta, engine.pool.tensors, dt, pos_hint=pos0 if tt > 1 else None, slot_hint=slot if tt > 1 else None)
        hh = torch.randn(tt, D, device=device).to(dt)
        y1, y2 = torch.randn(tt, D, device=device).to(dt), torch.randn(tt, D, device=device).to(dt)
        w, b = torch.ones(D, dtype=dt, device=device), torch.zeros(D, dtype=dt, device=device)
        # ---- residual step: own result, the average over the history, the next layer norm
        n_hist = L // 2 + 1                                     # a layer in the middle of the stack
        hist = torch.randn(n_hist, tt, D, device=device)
        avg = torch.randn(n_hist, device=device)
        x = torch.randn(tt, D, device=device)
        hn = torch.empty(tt, D, dtype=dt, device=device)
        t = timer(lambda: S.check(lib.b2l_seq_depth_step(M._p(y1), M._p(y2), M._p(x), M._p(hist), n_hist, M._p(avg), M._p(x), M._p(w), M._p(b),
                                                         S.NORM_LAYER, eps, M._p(hn), tt, D, ctx.act, ctx.stream), "k"))
        add(f"seq_depth_step_kernel (sum + average over {n_hist} results + layer norm)", tt, t, tt * D * (2 * es + 4 + 4 + 4 * n_hist + es))
        h2 = torch.empty(tt, D, dtype=dt, device=device)
        t = timer(lambda: S.check(lib.b2l_seq_add_norm2(M._p(y1), M._p(y2), M._p(x), M._p(w), M._p(hn), M._p(w), M._p(h2), 1.0, eps, None, tt, D,
                                                        ctx.act, ctx.stream), "k"))
        add("  like: seq_add_norm2_kernel (sum + two RMS norms, no history)", tt, t, tt * D * (2 * es + 4 + 4 + 2 * es))
        # ---- attention operands: convolution + rotation against norm + rotation
        proj = torch.randn(tt, att.C, device=device).to(dt)
        q = torch.empty(tt, H * 2 * K, device=device)
        kn = torch.empty(tt, G * 2 * K, dtype=dt, device=device)
        vn = torch.empty(tt, G * V, dtype=dt, device=device)
        a = S.ConvRopeArgs(proj=M._p(proj), ld=att.C, c_off=0, C=att.C, taps=att.taps, w=M._p(att.w_conv), state=M._p(ctx.state[att.name + ".conv"]),
                           meta=M._p(meta), q_off=att.o_q, q_heads=2 * H, k_off=att.o_k, k_heads=2 * G, K=K, v_off=att.o_v, n_v=G * V, freq=M._p(att.freq),
                           rot_dims=att.rot_dims, interleaved=1, rot_mult=1.0, q_out=M._p(q), k_out=M._p(kn), v_out=M._p(vn), T=tt, act_dtype=ctx.act)
        t = timer(lambda: S.check(lib.b2l_seq_conv_rope(C.byref(a), ctx.stream), "k"))
        nbq = tt * (att.C * es + H * 2 * K * 4 + G * 2 * K * es + G * V * es)
        add(f"seq_conv_rope_kernel ({att.taps} taps + rotation of q and k, v convolved)", tt, t, nbq)
        wk = torch.ones(K, dtype=dt, device=device)

        def two_norms():
            S.check(lib.b2l_seq_headnorm_rope(M._p(proj, att.o_q), att.C, M._p(wk), eps, M._p(att.freq), att.rot_dims, 1.0, M._p(meta), M._p(q), 1, tt,
                                              2 * H, K, ctx.act, ctx.stream), "k")
            S.check(lib.b2l_seq_headnorm_rope(M._p(proj, att.o_k), att.C, M._p(wk), eps, M._p(att.freq), att.rot_dims, 1.0, M._p(meta), M._p(kn), 0, tt,
                                              2 * G, K, ctx.act, ctx.stream), "k")

        t = timer(two_norms)
        add("  like: 2 x seq_headnorm_rope_kernel (per-head norm + rotation of q and k, v untouched)", tt, t,
            tt * ((H + G) * 2 * K * es + H * 2 * K * 4 + G * 2 * K * es))
        # ---- the attention kernel: two maps per head over shared values + read-out, against one map per head of twice the size
        keys = (tt + 1) / 2 if tt > 1 else pos0 + 1
        qr = torch.randn(tt, H * 2 * K, device=device)
        kr = torch.randn(tt, G * 2 * K, device=device).to(dt)
        maps = torch.empty(tt, H * 2 * V, device=device)
        y = torch.empty(tt, H * V, dtype=dt, device=device)
        bA = S.AttnArgs(q=M._p(qr), k_new=M._p(kr), v_new=M._p(vn), ldv=G * V, cache_k=M._p(ck), cache_v=M._p(cv), meta=M._p(meta), gate=None, ldg=0,
                        out=M._p(maps), ldo=H * 2 * V, scale=att.scale, softcap=0.0, out_mult=1.0, has_sink=0, block=att.max_positions, T=tt, heads=2 * H,
                        kv_heads=G, K=K, V=V, act_dtype=ctx.act, window=0, gate_per_channel=0, maps=2, out_f32=1, no_append=0, diff_out=M._p(y), ldd=H * V,
                        diff_lambda=att.lam, diff_eps=eps, diff_mult=1.0 - att.diff)
        t = timer(lambda: M.local_attention(bA, ctx))
        nb = tt * (H * 2 * K * 4 + G * (2 * K + V) * es * 2 + H * V * es) + (keys * G * (2 * K + V) * es if tt == 1 else 0)
        add("seq_block_attention (2 maps per head + differential read-out) + append", tt, t, nb, 2.0 * tt * 2 * H * keys * (K + V),
            f"f32 scores on CUDA cores, {keys:.0f} keys per query")
        t = timer(lambda: S.check(lib.b2l_seq_diff_combine(M._p(maps), H * 2 * V, att.lam, eps, 1.0 - att.diff, M._p(y), H * V, tt, H, V, ctx.act, ctx.stream), "k"))
        add("  seq_diff_combine_kernel alone (the read-out as a kernel of its own: prompt portions)", tt, t, tt * H * V * (8 + es))
        gate = torch.randn(tt, H, device=device).to(dt)
        bB = S.AttnArgs(q=M._p(qr), k_new=M._p(kr), v_new=M._p(vn), ldv=G * V, cache_k=M._p(ck), cache_v=M._p(cv), meta=M._p(meta), gate=M._p(gate), ldg=H,
                        out=M._p(y), ldo=H * V, scale=att.scale, softcap=0.0, out_mult=1.0, has_sink=1, block=att.max_positions, T=tt, heads=H, kv_heads=G,
                        K=2 * K, V=V, act_dtype=ctx.act, window=0, gate_per_channel=0, maps=0, out_f32=0, no_append=0)
        t = timer(lambda: M.local_attention(bB, ctx))
        nb = tt * (H * 2 * K * 4 + G * (2 * K + V) * es * 2 + H * V * es) + (keys * G * (2 * K + V) * es if tt == 1 else 0)
        add("  like: seq_block_attention (one map of twice the size per head, sink, gate per head) + append", tt, t, nb, 2.0 * tt * H * keys * (2 * K + V),
            "the same keys and values; half the value products")
        t = timer(lambda: att.forward(hh, ctx))
        wb = (att.w_in.numel() + att.w_o.numel()) * es
        add("DifferentialAttention whole (2 products + convolution/rotation + attention + read-out)", tt, t, wb + 2 * tt * D * es,
            2.0 * tt * 2 * H * keys * (K + V) + 2.0 * tt * wb / es)
        # ---- latent attention: sliding window without a sink against the unbounded form with a sink
        Hl, rk, dr, dn, dv, Wn = lat.H, lat.rk, lat.dr, lat.dn, lat.dv, lat.window
        n_keys = pos0 + tt
        Kd = rk + dr
        cache = ctx.state[lat.name + ".kv"]
        shared_b = dict(key_b=M._p(cache, rk), ldkb=Kd, slot_stride_b=lat.max_positions * Kd, n_b=dr)
        keys_w = ((min(tt, Wn) * (min(tt, Wn) + 1) / 2 + max(0, tt - Wn) * Wn) / tt) if tt > 1 else min(n_keys, Wn)
        sink = torch.zeros(Hl, device=device)
        for name, window, sk, kq in (("seq_latent_attention_kernel (window %d, no sink" % Wn, Wn, None, keys_w),
                                     ("  like: seq_latent_attention_kernel (every earlier position, sink", 0, sink, keys)):
            lat.window, lat.sink = window, sk
            if tt >= lat.expand_from:
                q32 = torch.randn(tt, Hl * (dn + dr), device=device)
                kv = torch.randn(n_keys, Hl * (dv + dn), device=device).to(dt)
                out_a = torch.empty(tt, Hl * dv, dtype=dt, device=device)
                splits = lat._splits(ctx, 1)
                t = timer(lambda: lat._attend(ctx, out_a, dv, splits, q_a=M._p(q32), ldqa_t=Hl * (dn + dr), ldqa_h=dn + dr, q_b=M._p(q32, dn),
                                              ldqb_t=Hl * (dn + dr), ldqb_h=dn + dr, key_a=M._p(kv), ldka=Hl * (dv + dn), hska=dv + dn, slot_stride_a=0,
                                              n_a=dv + dn, score_off=dv, heads_per_group=1, **shared_b))
                fl, form = 2.0 * tt * Hl * kq * (dn + dr + dv), "expanded"
                nbl = n_keys * (Hl * (dv + dn) + dr) * es + tt * Hl * ((dn + dr) * 4 + dv * es)
            else:
                q_lat = torch.randn(Hl, tt, rk, device=device)
                q_rot = torch.randn(tt, Hl, dr, device=device)
                out_a = torch.empty(tt, Hl * rk, dtype=dt, device=device)
                splits = lat._splits(ctx, Hl)
                t = timer(lambda: lat._attend(ctx, out_a, rk, splits, q_a=M._p(q_lat), ldqa_t=rk, ldqa_h=tt * rk, q_b=M._p(q_rot), ldqb_t=Hl * dr,
                                              ldqb_h=dr, key_a=M._p(cache), ldka=Kd, hska=0, slot_stride_a=lat.max_positions * Kd, n_a=rk, score_off=0,
                                              heads_per_group=Hl, **shared_b))
                fl, form = 2.0 * tt * Hl * kq * (2 * rk + dr), "latent"
                nbl = kq * Kd * es + tt * Hl * (Kd * 4 + rk * es)
            add(f"{name}, {form} form)", tt, t, nbl, fl, f"f32 scores on CUDA cores, {kq:.0f} keys per query, {splits} key split(s)")
        lat.window, lat.sink = Wn, None
        t = timer(lambda: lat.forward(hh, ctx))
        wb = (lat.w_in.numel() + lat.w_uq.numel() + lat.w_uk.numel() + lat.w_uv_t.numel() + lat.w_o.numel()) * es
        add("LatentAttention whole (5 products + prep + rotation + attention)", tt, t, wb + 2 * tt * D * es)
        # ---- the recurrence: a state per channel against a matrix state per head
        n = gru.width
        pj = torch.randn(tt, gru.w_in.shape[0], device=device).to(dt)
        og = torch.empty(tt, n, dtype=dt, device=device)
        n_chunks = lib.b2l_seq_mingru_chunks(tt)
        work = torch.empty(n_chunks, 2, n, device=device) if n_chunks > 1 else None
        t = timer(lambda: S.check(lib.b2l_seq_mingru(M._p(pj), pj.shape[1], gru.o_z, gru.o_x, gru.o_g, M._p(ctx.state[gru.name + ".S"]), M._p(meta), M._p(og), n,
                                                     M._p(work), n_chunks, tt, n, ctx.act, ctx.stream), "k"))
        add(f"seq_mingru_kernel ({n_chunks} chunk(s))", tt, t, tt * n * 4 * es + 8 * n, 6.0 * tt * n,
            "chunked: gates and candidates are read twice" if n_chunks > 1 else "")
        Hs, Ks, Vs = max(1, n // 128), 64, 128                   # a matrix state of the closest model at the same read-out width
        qkv = torch.randn(tt, 2 * Hs * Ks + Hs * Vs, device=device)
        st = torch.zeros(engine.pool.n_slots, Hs, Vs, Ks, device=device)
        dec = torch.full((Hs,), 0.97, device=device)
        o32 = torch.empty(tt, Hs * Vs, device=device)
        t = timer(lambda: M._scan(ctx, q=M._p(qkv), ldq=qkv.shape[1], k=M._p(qkv, Hs * Ks), ldk=qkv.shape[1], v=M._p(qkv, 2 * Hs * Ks), ldv=qkv.shape[1],
                                  q_mult=1.0, decay=M._p(dec), ldd=0, per_channel=False, state=st, out=M._p(o32), ldo=Hs * Vs, heads=Hs, qk_heads=Hs,
                                  K=Ks, V=Vs))
        add("  like: seq_scan (retention: a 64 x 128 state per head, fixed decay)", tt, t, tt * (2 * Hs * Ks + 2 * Hs * Vs) * 4 + 2 * Hs * Ks * Vs * 4,
            6.0 * tt * Hs * Ks * Vs)
        t = timer(lambda: gru.forward(hh, ctx))
        wb = (gru.w_in.numel() + gru.w_o.numel()) * es
        add("MinGRUMixer whole (2 products + recurrence)", tt, t, wb + 2 * tt * D * es, 2.0 * tt * wb / es)
        # ---- feed-forward
        u = torch.randn(tt, dense.ff, device=device).to(dt)
        t = timer(lambda: S.check(lib.b2l_seq_unary_act(M._p(u), dense.ff, M._p(u), dense.ff, tt, dense.ff, dense.act, M._p(dense.coef), ctx.act, ctx.stream), "k"))
        add("seq_unary_act_kernel (xIELU in place)", tt, t, tt * dense.ff * 2 * es)
        gu = torch.randn(tt, 2 * dense.ff, device=device).to(dt)
        t = timer(lambda: S.check(lib.b2l_seq_gated_act(M._p(gu), 2 * dense.ff, M._p(u), tt, dense.ff, S.ACT_SILU, 0.0, ctx.act, ctx.stream), "k"))
        add("  like: seq_gated_act_kernel (silu gate)", tt, t, tt * dense.ff * 3 * es)
        t = timer(lambda: dense.forward(hh, ctx))
        wb = (dense.w_up.numel() + dense.w_down.numel()) * es
        add("DenseMLP whole (2 products + xIELU)", tt, t, wb + 2 * tt * D * es, 2.0 * tt * wb / es)
        t = timer(lambda: moe.forward(hh, ctx))
        active = moe.top * 3 * moe.ff * D
        wb = min(moe.E, tt * moe.top) * 3 * moe.ff * D * es
        form = "device-indexed expert products" if tt <= moe.SMALL else "sort + gather + grouped library products + combine"
        add("MoEFeedForward whole (sigmoid scores, groups worth their two best, scaled weights)", tt, t, wb + 2 * tt * D * es, 2.0 * tt * active, form)
        like = M.MoEFeedForward.__new__(M.MoEFeedForward)
        like.__dict__.update(moe.__dict__)
        like.score, like.group_top, like.weight_scale = S.SCORE_SOFTMAX, 1, 1.0
        t = timer(lambda: like.forward(hh, ctx))
        add("  like: MoEFeedForward whole (softmax scores, groups worth their best)", tt, t, wb + 2 * tt * D * es, 2.0 * tt * active, form)
        idx, wgt = moe.route(hh, ctx)
        z = torch.randn(tt, moe.n, device=device)
        for nm, gt in (("seq_moe_route_kernel (groups worth their two best)", 2), ("  like: seq_moe_route_kernel (groups worth their best)", 1)):
            t = timer(lambda: S.check(lib.b2l_seq_moe_route(M._p(z), moe.n, M._p(moe.correction), moe.n, moe.groups, moe.keep, moe.top, moe.score, moe.renorm, gt,
                                                            moe.weight_scale, M._p(idx), M._p(wgt), tt, ctx.stream), "k"))
            add(nm, tt, t, tt * (moe.n * 4 + moe.top * 8))
    engine.pool.release("kernels")
    return rows


def run_size(name: str, prompt: int, decode_steps: int, device, timer, peaks: dict) -> dict:
    import lit_llama_b200 as P
    from .rinirax import random_weights
    from .zenasun import random_weights as zenasun_weights

    sz = SIZES[name]
    cfg = rinirax_config(**sz)
    W = random_weights(cfg, device)
    model = P.Rinirax(P.RiniraxConfig.from_dict(cfg), W, max_positions=prompt + decode_steps + 8)
    del W
    engine = P.Engine(model, n_slots=2, prefill_chunk=prompt)
    toks = torch.randint(0, sz["vocab"], (prompt + decode_steps,), generator=torch.Generator().manual_seed(1)).tolist()
    t_pre, t_dec = zenasun_bench._throughput(engine, toks, prompt, decode_steps, device, timer)
    params, active = model.n_parameters()
    active -= model.embed.numel()                                # a token reads one row of it
    cache = sum(t[0].numel() * t.element_size() * (prompt / model.max_positions if k.endswith((".kv", ".k", ".v")) else 1.0)
                for k, t in engine.pool.tensors.items())
    # a decoded token reads the caches of the own-key attention layers twice: the layers that share them read them again
    shared = sum(engine.pool.tensors[l.mixer.src.name + s][0].numel() * 2 * prompt / model.max_positions
                 for l in model.layers if getattr(l.mixer, "src", None) is not None for s in (".k", ".v"))
    out = {"rinirax": {"params": params, "active_params_per_token": active, "state_bytes_per_sequence": engine.pool.bytes() // engine.pool.n_slots,
                       "cache_bytes_read_per_token": int(cache + shared), "prefill_tok_s": prompt / t_pre, "prefill_ms": t_pre * 1e3,
                       "decode_tok_s": 1.0 / t_dec, "decode_us": t_dec * 1e6,
                       "decode_frac_of_measured_hbm": (2 * active + cache + shared) / t_dec / (peaks["hbm_gbs"] * 1e9)}}
    out["kernels"] = kernel_table(model, engine, prompt, device, timer, peaks)
    del engine, model
    torch.cuda.empty_cache()

    # ---- the closest served family at the same width and depth
    zsz = zenasun_bench.SIZES[name]
    zcfg = zenasun_bench.zenasun_config(**zsz)
    ZW = zenasun_weights(zcfg, device)
    zen = P.Zenasun(P.ZenasunConfig.from_dict(zcfg), ZW, max_positions=prompt + decode_steps + 8)
    del ZW
    zengine = P.Engine(zen, n_slots=2, prefill_chunk=prompt)
    t_pre2, t_dec2 = zenasun_bench._throughput(zengine, toks, prompt, decode_steps, device, timer)
    zp = zen.n_parameters()
    zmoe = zen.layers[0].mlp
    zactive = zp - sum(1 for l in zen.layers if l.mlp is not None) * (zmoe.E - zmoe.top) * 3 * zmoe.ff * zsz["width"] - zen.embed.numel()
    zcache = sum(t[0].numel() * t.element_size() * (prompt / zen.max_positions if k.endswith(".kv") else 1.0) for k, t in zengine.pool.tensors.items())
    out["zenasun"] = {"params": zp, "active_params_per_token": zactive, "state_bytes_per_sequence": zengine.pool.bytes() // 2,
                      "cache_bytes_read_per_token": int(zcache), "prefill_tok_s": prompt / t_pre2, "prefill_ms": t_pre2 * 1e3,
                      "decode_tok_s": 1.0 / t_dec2, "decode_us": t_dec2 * 1e6,
                      "decode_frac_of_measured_hbm": (2 * zactive + zcache) / t_dec2 / (peaks["hbm_gbs"] * 1e9)}
    del zengine, zen
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
    out = {"metric": "rinirax_vs_zenasun_throughput", "unit": "tokens/s", "dtype": "bf16", "data": "synthetic (random weights)", "prompt": args.prompt,
           "decode_steps": args.decode_steps, "peaks": {k: peaks[k] for k in ("hbm_gbs", "bf16_tflops", "source")}, "l2": "flushed between timed iterations",
           "sizes": {}}
    t0 = time.time()
    for name in sizes:
        out["sizes"][name] = run_size(name, args.prompt, args.decode_steps, device, timer, peaks)
    out["seconds"] = round(time.time() - t0, 1)
    return out
