"""Throughput of the Lugovik family beside the package's LLaMA at equal width and depth (`bench.py --family lugovik`).

Random weights, bf16, one sequence: prefill of a `prompt`-token prompt in one portion, then single-token decoding
through the engine (CUDA-graph replay).  The LLaMA arm is the package's dense bf16 LLaMA (module path: the same
library products, its own attention / norm kernels) at the same width, layer count and head size.  A second table
times the family's kernels alone at the model's shapes, with their algorithmic bytes, against the measured copy
bandwidth, next to the LLaMA kernel that does the like job.  CUDA events, warm-up, L2 flushed between iterations."""
import ctypes as C
import json
import math
import os
import time
from typing import Callable, Dict, List

import torch

SIZES = {
    # width, layers, head size, ff; the layer pattern repeats: channel_delta, mamba2, mamba2, parallel
    "1k": dict(width=1024, layers=8, ff=4096, hs=128, block=1024, vocab=32000),
    "2k": dict(width=2048, layers=8, ff=8192, hs=128, block=2048, vocab=32000),
    "4k": dict(width=4096, layers=8, ff=11008, hs=128, block=2048, vocab=32000),
}


def lugovik_config(width: int, layers: int, ff: int, hs: int, block: int, vocab: int) -> dict:
    H = width // hs
    kinds = ["channel_delta", "mamba2", "mamba2", "parallel"]
    out = []
    for i in range(layers):
        kind = kinds[i % 4]
        if kind == "channel_delta":
            mixer = {"conv": 4, "dim": hs, "heads": H, "kv_heads": H, "vdim": hs}
        elif kind == "mamba2":
            mixer = {"conv": 4, "groups": 1, "heads": 2 * width // 64, "norm_groups": 1, "state": 128, "vdim": 64}
        else:
            mixer = {"left": {"heads": H, "kv_heads": max(1, H // 4), "dim": hs, "vdim": hs, "mask": {"size": block}, "scale": hs ** -0.5,
                              "softcap": 50.0, "rot": {"base": 1e6, "dims": hs, "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}}},
                     "right": {"heads": max(1, H // 2), "dim": hs, "vdim": hs, "tau": 16.0}, "left_scale": 1.0, "right_scale": 1.0}
        out.append({"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff}})
    return {"architecture": "Lugovik", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "embedding": {"scale": math.sqrt(width)}, "layers": out}


def random_weights(cfg: dict, device, dtype=torch.bfloat16, rank: int = 64, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Random tensors with the family's names and shapes (projections ~ N(0, 1/in), norms ~ 1, decays in a range where
    the recurrences neither die nor blow up)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    D, W = cfg["width"], {}

    def lin(o, i):
        return (torch.randn(o, i, generator=g) / math.sqrt(i)).to(device, dtype)

    def vec(n, mean=1.0, std=0.1):
        return (mean + std * torch.randn(n, generator=g)).to(device, dtype)

    W["embed"], W["head"], W["final.norm"] = (torch.randn(cfg["vocab"], D, generator=g) / math.sqrt(D)).to(device, dtype), lin(cfg["vocab"], D), vec(D)
    for i, layer in enumerate(cfg["layers"]):
        p, m, c = f"l{i}.", f"l{i}.mix.", layer["mixer"]
        for n in ("norm1", "norm2"):
            W[p + n] = vec(D)
        for n in ("norm1b", "norm2b"):
            W[p + n] = vec(D, 0.5)
        if layer["type"] == "channel_delta":
            H, G, K, V = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
            for n, ch in (("q", G * K), ("k", G * K), ("v", H * V)):
                W[m + n], W[m + n + ".conv"] = lin(ch, D), (torch.randn(ch, c["conv"], generator=g) * 0.5).to(device, dtype)
            W[m + "b"], W[m + "A_log"], W[m + "norm"] = lin(H, D), vec(H, -0.5, 0.5), vec(V)
            W[m + "a1"], W[m + "a2"], W[m + "dt_bias"] = lin(rank, D), lin(H * K, rank), vec(H * K, 0.0, 0.5)
            W[m + "g1"], W[m + "g2"], W[m + "o"] = lin(rank, D), lin(H * V, rank), lin(D, H * V)
        elif layer["type"] == "mamba2":
            H, P, N, G = c["heads"], c["vdim"], c["state"], c["groups"]
            ch = H * P + 2 * G * N
            W[m + "in"], W[m + "conv"], W[m + "conv.b"] = lin(2 * H * P + 2 * G * N + H, D), (torch.randn(ch, c["conv"], generator=g) * 0.5).to(device, dtype), vec(ch, 0.0)
            W[m + "dt_bias"], W[m + "A_log"], W[m + "D"] = vec(H, 0.0, 0.5), vec(H, -0.5, 0.5), vec(H)
            W[m + "norm"], W[m + "o"] = vec(H * P), lin(D, H * P)
        else:
            a, b = c["left"], c["right"]
            H, G, K, V = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            W[m + "left.q"], W[m + "left.k"], W[m + "left.v"] = lin(H * K, D), lin(G * K, D), lin(G * V, D)
            W[m + "left.q.norm"], W[m + "left.k.norm"], W[m + "left.g"], W[m + "left.o"] = vec(K), vec(K), lin(H, D), lin(D, H * V)
            H, K, V = b["heads"], b["dim"], b["vdim"]
            W[m + "right.q"], W[m + "right.k"], W[m + "right.v"], W[m + "right.g"] = lin(H * K, D), lin(H * K, D), lin(H * V, D), lin(H * V, D)
            W[m + "right.o"], W[m + "right.norm"] = lin(D, H * V), vec(V)
            W[m + "right.a1"], W[m + "right.a2"], W[m + "right.a2.b"] = lin(rank, D), lin(H * K, rank), vec(H * K, 2.0, 0.5)
        F = layer["mlp"]["ff"]
        W[p + "mlp.gate"], W[p + "mlp.up"], W[p + "mlp.down"] = lin(F, D), lin(F, D), lin(D, F)
    return W


class _Timer:
    def __init__(self, device):
        self.device = device
        self.flush = torch.empty(192 * 1024 * 1024, dtype=torch.uint8, device=device)     # larger than the 126 MB L2

    def __call__(self, fn: Callable[[], None], iters: int = 5, warmup: int = 3) -> float:
        """Median seconds of fn() over `iters` runs, L2 flushed before each."""
        for _ in range(warmup):
            fn()
        times = []
        for _ in range(iters):
            self.flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize(self.device)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize(self.device)
            times.append(a.elapsed_time(b) * 1e-3)
        return sorted(times)[len(times) // 2]


def _llama(width: int, layers: int, hs: int, vocab: int, block_size: int, device):
    import lit_llama_b200 as P

    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(device):
            model = P.LLaMA(P.LLaMAConfig(block_size=block_size, vocab_size=vocab, n_layer=layers, n_head=width // hs, n_embd=width))
    finally:
        torch.set_default_dtype(prev)
    g = torch.Generator(device="cpu").manual_seed(0)
    with torch.no_grad():
        for prm in model.parameters():
            if prm.dim() == 2:
                prm.copy_((torch.randn(prm.shape, generator=g) / math.sqrt(prm.shape[1])).to(prm.dtype))
            else:
                prm.fill_(1.0)
    return model.eval()


def run_size(name: str, prompt: int, decode_steps: int, device, timer: _Timer, peaks: dict) -> dict:
    import lit_llama_b200 as P

    sz = SIZES[name]
    cfg = lugovik_config(**sz)
    W = random_weights(cfg, device)
    model = P.Lugovik(P.LugovikConfig.from_dict(cfg), W, max_positions=prompt + decode_steps + 8)
    del W
    engine = P.Engine(model, n_slots=1, prefill_chunk=prompt)
    toks = torch.randint(0, sz["vocab"], (prompt + decode_steps,), generator=torch.Generator().manual_seed(1)).tolist()
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
    t_dec = a.elapsed_time(b) * 1e-3 / (decode_steps - 4)
    engine.step([], end=["d"])
    params = model.n_parameters()
    state_bytes = engine.pool.bytes()
    out = {"lugovik": {"params": params, "state_bytes_per_sequence": state_bytes, "prefill_tok_s": prompt / t_pre, "prefill_ms": t_pre * 1e3,
                       "decode_tok_s": 1.0 / t_dec, "decode_us": t_dec * 1e6,
                       "decode_frac_of_measured_hbm": (2 * params + 2 * state_bytes) / t_dec / (peaks["hbm_gbs"] * 1e9)}}
    out["kernels"] = kernel_table(model, engine, prompt, device, timer, peaks)
    del engine, model
    torch.cuda.empty_cache()

    # ---- the package's LLaMA (dense bf16, module path) at the same width / depth / head size
    S = (prompt + decode_steps + 8 + 63) // 64 * 64
    llama = _llama(sz["width"], sz["layers"], sz["hs"], sz["vocab"], S, device)
    idx = torch.tensor(toks[:prompt], dtype=torch.int64, device=device).view(1, -1)
    pos = torch.arange(prompt, device=device)

    def llama_prefill():
        llama.reset_cache()
        llama(idx, S, pos)

    with torch.no_grad():
        t_pre2 = timer(llama_prefill, iters=3, warmup=2)
        llama.reset_cache()
        llama(idx, S, pos)
        one = torch.zeros((1, 1), dtype=torch.int64, device=device)
        for i in range(4):
            llama(one, S, torch.tensor([prompt + i], device=device))
        torch.cuda.synchronize(device)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(4, decode_steps):
            llama(one, S, torch.tensor([prompt + i], device=device))
        b.record()
        torch.cuda.synchronize(device)
    t_dec2 = a.elapsed_time(b) * 1e-3 / (decode_steps - 4)
    lp = sum(p.numel() for p in llama.parameters())
    kv = 2 * sz["layers"] * sz["width"] * 2 * prompt
    out["llama_dense_bf16"] = {"params": lp, "prefill_tok_s": prompt / t_pre2, "prefill_ms": t_pre2 * 1e3, "decode_tok_s": 1.0 / t_dec2,
                               "decode_us": t_dec2 * 1e6, "decode_frac_of_measured_hbm": (2 * lp + kv) / t_dec2 / (peaks["hbm_gbs"] * 1e9)}
    out["llama_kernels"] = llama_kernel_table(llama, sz, prompt, device, timer, peaks)
    del llama
    torch.cuda.empty_cache()
    return out


def kernel_table(model, engine, T: int, device, timer: _Timer, peaks: dict) -> List[dict]:
    """The family's kernels alone at this model's shapes: prefill (T tokens) and decode (1 token), seconds,
    algorithmic bytes / flops and the fraction of the measured copy bandwidth."""
    from . import _seqlib as S
    from . import mixers as M

    rows = []
    hbm = peaks["hbm_gbs"] * 1e9
    slot = engine.pool.acquire("kernels")
    metas = {T: torch.tensor([slot, 0], dtype=torch.int32, device=device)}
    D, dt = model.width, model.dtype
    es = 2

    def add(name, like, t, nbytes, flops=0.0, note=""):
        rows.append({"kernel": name, "like": like, "tokens": int(tt), "us": t * 1e6, "GB_s": nbytes / t / 1e9, "frac_of_measured_hbm": nbytes / t / hbm,
                     "GFLOP_s": flops / t / 1e9, "note": note})

    by_kind = {}
    for layer in model.layers:
        by_kind.setdefault(type(layer.mixer).__name__, layer.mixer)
    for tt in (T, 1):
        if tt not in metas:      # a decoded token deep inside its block
            blocks = [b.block for l in model.layers for b in getattr(l.mixer, "branches", []) if hasattr(b, "block")]
            metas[tt] = torch.tensor([slot, min([T] + blocks) - 1], dtype=torch.int32, device=device)
        ctx = M.StepContext(tt, metas[tt], engine.pool.tensors, dt)
        lib = S.lib()
        x = torch.randn(tt, D, device=device)
        y = torch.randn(tt, D, device=device).to(dt)
        h = torch.empty(tt, D, dtype=dt, device=device)
        w = torch.ones(D, dtype=dt, device=device)
        t = timer(lambda: S.check(lib.b2l_seq_norm_add_norm(M._p(y), M._p(w), 1e-6, M._p(x), M._p(w), M._p(h), tt, D, ctx.act, ctx.stream), "k"))
        add("seq_norm_add_norm_kernel", "rmsnorm_kernel + add_kernel", t, tt * D * (es + 4 + 4 + es))
        mlp = model.layers[0].mlp
        gu = torch.randn(tt, 2 * mlp.ff, device=device).to(dt)
        mid = torch.empty(tt, mlp.ff, dtype=dt, device=device)
        t = timer(lambda: S.check(lib.b2l_seq_gated_act(M._p(gu), 2 * mlp.ff, M._p(mid), tt, mlp.ff, S.ACT_GELU_TANH, 0.0, ctx.act, ctx.stream), "k"))
        add("seq_gated_act_kernel", "silu_mul_kernel", t, tt * mlp.ff * 3 * es)
        for kind, mx in by_kind.items():
            hh = torch.randn(tt, D, device=device).to(dt)
            if kind == "ParallelMixer":
                att, gla = mx.branches
                proj = torch.randn(tt, mx.w_in.shape[0], device=device).to(dt)
                out = torch.empty(tt, sum(mx.widths), dtype=dt, device=device)
                t = timer(lambda: att.run(proj, mx.offs[:4], ctx, out, 0, 1.0))
                keys = (min(T, att.block) + 1) / 2 if tt > 1 else min(T, att.block)     # mean keys per query
                fl = 2.0 * tt * att.H * keys * (att.K + att.V)
                nb = tt * (att.H * att.K * (es + 4) + att.G * (att.K + att.V) * es * 3 + att.H * att.V * es) + \
                    (min(T, att.block) * att.G * (att.K + att.V) * es if tt == 1 else 0)
                add("attention branch (2 x seq_headnorm_rope + seq_block_attention + seq_ring_append)", "b2l_attention (prefill: mma.sync tiles)", t, nb, fl,
                    "f32 scores on CUDA cores")
                t = timer(lambda: gla.run(proj, mx.offs[4:], ctx, out, mx.widths[0], 1.0))
                st = gla.H * gla.K * gla.V * 4 * 2
                add("linear-attention branch (product + seq_decay + seq_scan + seq_group_norm_gate)", "-", t, st + tt * gla.H * (3 * gla.K + 2 * gla.V) * 4,
                    6.0 * tt * gla.H * gla.K * gla.V, "sequential over tokens")
            else:
                t = timer(lambda: mx.forward(hh, ctx))
                if kind == "Mamba2Mixer":
                    st, fl = mx.H * mx.P * mx.N * 4 * 2, 6.0 * tt * mx.H * mx.P * mx.N
                    wb = (mx.w_in.numel() + mx.w_o.numel()) * es
                else:
                    st, fl = mx.H * mx.K * mx.V * 4 * 2, 8.0 * tt * mx.H * mx.K * mx.V
                    wb = (mx.w_in.numel() + mx.w_o.numel() + mx.w_a2.numel() + mx.w_g2.numel()) * es
                add(f"{kind} whole (products + conv + scan + read-out)", "CausalSelfAttention whole", t, st + wb + 2 * tt * D * es, fl + 2.0 * tt * wb / es,
                    "state + weights + in/out")
    engine.pool.release("kernels")
    return rows


def llama_kernel_table(llama, sz: dict, T: int, device, timer: _Timer, peaks: dict) -> List[dict]:
    """The LLaMA kernels that do the like jobs, timed the same way."""
    from . import _lib as L

    rows, hbm = [], peaks["hbm_gbs"] * 1e9
    D = sz["width"]
    blk = llama.transformer.h[0]
    for tt in (T, 1):
        x = torch.randn(1, tt, D, device=device).to(torch.bfloat16)
        y = torch.randn(1, tt, D, device=device).to(torch.bfloat16)
        from .model import _add

        t = timer(lambda: _add(x, blk.rms_1(y)))
        rows.append({"kernel": "rmsnorm_kernel + add_kernel", "tokens": tt, "us": t * 1e6, "GB_s": tt * D * 2 * 5 / t / 1e9,
                     "frac_of_measured_hbm": tt * D * 2 * 5 / t / hbm})
        nh = blk.mlp.c_fc1.out_features
        a, b = torch.randn(tt, nh, device=device).to(torch.bfloat16), torch.randn(tt, nh, device=device).to(torch.bfloat16)
        hcat = torch.empty_like(a)
        t = timer(lambda: L.check(L.lib().b2l_silu_mul(a.data_ptr(), b.data_ptr(), hcat.data_ptr(), a.numel(), L.stream_ptr()), "k"))
        rows.append({"kernel": "silu_mul_kernel", "tokens": tt, "us": t * 1e6, "GB_s": tt * nh * 6 / t / 1e9, "frac_of_measured_hbm": tt * nh * 6 / t / hbm})
    S = llama.kv_caches[0][0].shape[2]
    qkv = torch.randn(1, T, 3 * D, device=device).to(torch.bfloat16)
    att = blk.attn
    rope = llama.rope_cache
    kvc = llama.kv_caches[0]
    yb = torch.empty((1, T, D), device=device, dtype=torch.bfloat16)
    nh, hs = att.n_head, D // att.n_head
    lib = L.lib()
    work = torch.zeros(lib.b2l_attn_workspace_bytes(1, nh, hs, T, S) // 4 + 1, device=device, dtype=torch.float32)
    pos = torch.arange(T, device=device)
    ring = torch.zeros(1, dtype=torch.int32, device=device)

    def attn():
        L.check(lib.b2l_attention(qkv.data_ptr(), kvc[0].data_ptr(), kvc[1].data_ptr(), rope.data_ptr(), pos.data_ptr(), ring.data_ptr(), yb.data_ptr(),
                                  work.data_ptr(), 1, T, nh, hs, S, rope.shape[0], 0, L.stream_ptr()), "b2l_attention")

    t = timer(attn)
    fl = 2.0 * T * nh * (T + 1) / 2 * 2 * hs
    rows.append({"kernel": "b2l_attention (prefill, rope + append + causal attention)", "tokens": T, "us": t * 1e6, "GFLOP_s": fl / t / 1e9,
                 "frac_of_measured_bf16": fl / t / (peaks["bf16_tflops"] * 1e12)})
    return rows


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
    timer = _Timer(device)
    out = {"metric": "lugovik_vs_llama_throughput", "unit": "tokens/s", "dtype": "bf16", "data": "synthetic (random weights)", "prompt": args.prompt,
           "decode_steps": args.decode_steps, "peaks": {k: peaks[k] for k in ("hbm_gbs", "bf16_tflops", "source")}, "l2": "flushed between timed iterations",
           "sizes": {}}
    t0 = time.time()
    for name in sizes:
        out["sizes"][name] = run_size(name, args.prompt, args.decode_steps, device, timer, peaks)
    out["seconds"] = round(time.time() - t0, 1)
    return out
