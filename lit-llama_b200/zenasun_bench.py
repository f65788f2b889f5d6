"""Throughput of the Zenasun family beside the package's Lugovik family at equal width and depth
(`bench.py --family zenasun`).

Random weights, bf16, one sequence: prefill of a `prompt`-token prompt in one portion, then single-token decoding
through the engine (CUDA-graph replay).  The Lugovik arm is the closest served model: the same engine, state pool and
library products, its own block-local attention, recurrences and dense gated feed-forward.  A second table times the
family's mechanisms alone at the model's shapes with their algorithmic bytes and flops, next to the Lugovik kernel that
does the like job.  CUDA events, warm-up, L2 flushed between iterations."""
import ctypes as C
import json
import math
import os
import time
from typing import List

import torch

from . import seq_bench

SIZES = {
    # three latent-attention layers, then one retention layer, repeated; every layer has routed experts
    "1k": dict(width=1024, layers=8, heads=8, dim=128, rot_dim=64, vdim=128, q_rank=384, kv_rank=256, experts=20, identity=4, top=4, groups=6,
               keep=4, ff=512, vocab=32000),
    "2k": dict(width=2048, layers=8, heads=16, dim=128, rot_dim=64, vdim=128, q_rank=768, kv_rank=512, experts=28, identity=4, top=6, groups=8,
               keep=4, ff=1024, vocab=32000),
}


def zenasun_config(width, layers, heads, dim, rot_dim, vdim, q_rank, kv_rank, experts, identity, top, groups, keep, ff, vocab) -> dict:
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top, "groups": {"count": groups, "keep": keep}}}
    out = []
    for i in range(layers):
        if i % 4 == 3:
            decay = [1.0 - 2.0 ** (-5 - 5 * h / max(1, heads - 1)) for h in range(heads)]
            mixer, kind = {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay, "rot": {"base": 1e5, "dims": dim}}, "retention"
        else:
            mixer, kind = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
                           "scale": (dim + rot_dim) ** -0.5, "rot": {"base": 1e4, "dims": rot_dim}}, "latent_attention"
        out.append({"type": kind, "mixer": mixer, "mlp": mlp})
    return {"architecture": "Zenasun", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "embedding": {"scale": math.sqrt(width)},
            "logit_softcap": 50.0, "layers": out}


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
    """The family's mechanisms alone at this model's shapes: a T-token portion from position 0 and one token at
    position T."""
    from . import _seqlib as S
    from . import mixers as M

    rows, hbm, es = [], peaks["hbm_gbs"] * 1e9, 2
    slot = engine.pool.acquire("kernels")
    D, dt, lib = model.width, model.dtype, S.lib()
    att = next(l.mixer for l in model.layers if isinstance(l.mixer, M.LatentAttention))
    ret = next(l.mixer for l in model.layers if isinstance(l.mixer, M.RetentionMixer))
    moe = model.layers[0].mlp

    def add(name, like, tt, t, nbytes, flops=0.0, note=""):
        rows.append({"kernel": name, "like": like, "tokens": int(tt), "us": t * 1e6, "GB_s": nbytes / t / 1e9, "frac_of_measured_hbm": nbytes / t / hbm,
                     "GFLOP_s": flops / t / 1e9, "note": note})

    # fill the cache of the slot once, so that a single token at position T has T keys to read
    full = M.StepContext(T, torch.tensor([slot, 0], dtype=torch.int32, device=device), engine.pool.tensors, dt, pos_hint=0, slot_hint=slot)
    att.forward(torch.randn(T, D, device=device).to(dt), full)
    for tt, pos0 in ((T, 0), (1, T)):
        meta = torch.tensor([slot, pos0], dtype=torch.int32, device=device)
        ctx = M.StepContext(tt, meta, engine.pool.tensors, dt, pos_hint=pos0 if tt > 1 else None, slot_hint=slot if tt > 1 else None)
        hh = torch.randn(tt, D, device=device).to(dt)
        x = torch.randn(tt, D, device=device)
        y1, y2 = torch.randn(tt, D, device=device).to(dt), torch.randn(tt, D, device=device).to(dt)
        h1, h2 = torch.empty(tt, D, dtype=dt, device=device), torch.empty(tt, D, dtype=dt, device=device)
        w = torch.zeros(D, dtype=dt, device=device)
        t = timer(lambda: S.check(lib.b2l_seq_add_norm2(M._p(y1), M._p(y2), M._p(x), M._p(w), M._p(h1), M._p(w), M._p(h2), 1.0, 1e-6, None, tt, D,
                                                        ctx.act, ctx.stream), "k"))
        add("seq_add_norm2_kernel", "seq_norm_add_norm_kernel", tt, t, tt * D * (2 * es + 4 + 4 + 2 * es))
        # the attention kernel alone, in the form the mixer picks for this portion (its own products excluded)
        H, rk, dr, dn, dv = att.H, att.rk, att.dr, att.dn, att.dv
        n_keys = pos0 + tt
        expanded = tt >= att.expand_from
        keys = (tt + 1) / 2 if tt > 1 else n_keys
        Kd = rk + dr
        shared_b = dict(key_b=M._p(ctx.state[att.name + ".kv"], rk), ldkb=Kd, slot_stride_b=att.max_positions * Kd, n_b=dr)
        if expanded:
            q32 = torch.randn(tt, H * (dn + dr), device=device)
            kv = torch.randn(n_keys, H * (dv + dn), device=device).to(dt)
            out_a = torch.empty(tt, H * dv, dtype=dt, device=device)
            ctx.slot_hint = slot
            splits = att._splits(ctx, 1)
            t = timer(lambda: att._attend(ctx, out_a, dv, splits, q_a=M._p(q32), ldqa_t=H * (dn + dr), ldqa_h=dn + dr, q_b=M._p(q32, dn),
                                          ldqb_t=H * (dn + dr), ldqb_h=dn + dr, key_a=M._p(kv), ldka=H * (dv + dn), hska=dv + dn, slot_stride_a=0,
                                          n_a=dv + dn, score_off=dv, heads_per_group=1, **shared_b))
            fl = 2.0 * tt * H * keys * (dn + dr + dv)
            nb = n_keys * (H * (dv + dn) + dr) * es + tt * H * ((dn + dr) * 4 + dv * es)
        else:
            q_lat = torch.randn(H, tt, rk, device=device)
            q_rot = torch.randn(tt, H, dr, device=device)
            out_a = torch.empty(tt, H * rk, dtype=dt, device=device)
            splits = att._splits(ctx, H)
            t = timer(lambda: att._attend(ctx, out_a, rk, splits, q_a=M._p(q_lat), ldqa_t=rk, ldqa_h=tt * rk, q_b=M._p(q_rot), ldqb_t=H * dr, ldqb_h=dr,
                                          key_a=M._p(ctx.state[att.name + ".kv"]), ldka=Kd, hska=0, slot_stride_a=att.max_positions * Kd, n_a=rk,
                                          score_off=0, heads_per_group=H, **shared_b))
            fl = 2.0 * tt * H * keys * (2 * rk + dr)
            nb = n_keys * Kd * es + tt * H * (Kd * 4 + rk * es)
        add("seq_latent_attention_kernel (" + ("expanded" if expanded else "latent") + " form)",
            "seq_block_attention_tile_kernel" if tt > 1 else "seq_block_attention_kernel", tt, t, nb, fl,
            f"f32 scores on CUDA cores, {splits} key split(s)")
        t = timer(lambda: att.forward(hh, ctx))
        wb = (att.w_in.numel() + att.w_uq.numel() + att.w_uk.numel() + att.w_uv_t.numel() + att.w_o.numel()) * es
        add("LatentAttention whole (5 products + prep + rotation + attention)", "attention branch", tt, t, wb + nb, fl + 2.0 * tt * wb / es)
        t = timer(lambda: ret.forward(hh, ctx))
        st = ret.H * ret.K * ret.V * 4 * 2
        wb = (ret.w_in.numel() + ret.w_o.numel()) * es
        add("RetentionMixer whole (2 products + rotation + seq_scan + read-out)", "linear-attention branch", tt, t, st + wb + 2 * tt * D * es,
            6.0 * tt * ret.H * ret.K * ret.V + 2.0 * tt * wb / es, "the recurrence kernel is the one the closest model uses")
        t = timer(lambda: moe.forward(hh, ctx))
        active = moe.top * 3 * moe.ff * D
        wb = (min(moe.E, tt * moe.top) * 3 * moe.ff * D) * es
        add("MoEFeedForward whole (router + experts)", "GatedMLP (2 products + seq_gated_act)", tt, t, wb + 2 * tt * D * es, 2.0 * tt * active,
            "device-indexed expert products" if tt <= moe.SMALL else "sort + gather + per-expert library products + combine")
        idx, wgt = moe.route(hh, ctx)
        z = torch.randn(tt, moe.n, device=device)
        t = timer(lambda: S.check(lib.b2l_seq_moe_route(M._p(z), moe.n, M._p(moe.correction), moe.n, moe.groups, moe.keep, moe.top, moe.score, moe.renorm, moe.group_top, moe.weight_scale,
                                                        M._p(idx), M._p(wgt),
                                                        tt, ctx.stream), "k"))
        add("seq_moe_route_kernel", "-", tt, t, tt * (moe.n * 4 + moe.top * 8))
    engine.pool.release("kernels")
    return rows


def run_size(name: str, prompt: int, decode_steps: int, device, timer, peaks: dict) -> dict:
    import lit_llama_b200 as P
    from .zenasun import random_weights

    sz = SIZES[name]
    cfg = zenasun_config(**sz)
    W = random_weights(cfg, device)
    model = P.Zenasun(P.ZenasunConfig.from_dict(cfg), W, max_positions=prompt + decode_steps + 8)
    del W
    engine = P.Engine(model, n_slots=2, prefill_chunk=prompt)
    toks = torch.randint(0, sz["vocab"], (prompt + decode_steps,), generator=torch.Generator().manual_seed(1)).tolist()
    t_pre, t_dec = _throughput(engine, toks, prompt, decode_steps, device, timer)
    params = model.n_parameters()
    moe = model.layers[0].mlp
    n_moe = sum(1 for l in model.layers if l.mlp is not None)
    active = params - n_moe * (moe.E - moe.top) * 3 * moe.ff * sz["width"]
    cache_bytes = sum(t[0].numel() * t.element_size() * (prompt / model.max_positions if k.endswith(".kv") else 1.0)
                      for k, t in engine.pool.tensors.items())
    out = {"zenasun": {"params": params, "active_params_per_token": active, "cache_and_state_bytes_at_prompt": cache_bytes,
                       "prefill_tok_s": prompt / t_pre, "prefill_ms": t_pre * 1e3, "decode_tok_s": 1.0 / t_dec, "decode_us": t_dec * 1e6,
                       "decode_frac_of_measured_hbm": (2 * active + cache_bytes) / t_dec / (peaks["hbm_gbs"] * 1e9)}}
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
    out["lugovik_kernels"] = seq_bench.kernel_table(lug, lengine, prompt, device, timer, peaks)
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
    out = {"metric": "zenasun_vs_lugovik_throughput", "unit": "tokens/s", "dtype": "bf16", "data": "synthetic (random weights)", "prompt": args.prompt,
           "decode_steps": args.decode_steps, "peaks": {k: peaks[k] for k in ("hbm_gbs", "bf16_tflops", "source")}, "l2": "flushed between timed iterations",
           "sizes": {}}
    t0 = time.time()
    for name in sizes:
        out["sizes"][name] = run_size(name, args.prompt, args.decode_steps, device, timer, peaks)
    out["seconds"] = round(time.time() - t0, 1)
    return out
