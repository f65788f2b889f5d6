"""A plain float64 restatement of the Zuvevik design, one function per mechanism, written token by token wherever a
loop is the plainest form.  It shares no code with the package: torch on the CPU only.  Weights are a dict
name -> tensor; configurations are the dicts of config.json."""
import math

import torch

F64 = torch.float64


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


def pair_rows(tokens, buckets, mul_prev, mul_cur, before=None):
    """Row of the pair table for every token; `before` is the token ahead of the first one (None: the sequence starts here)."""
    rows, prev = [], before
    for t in tokens:
        rows.append(buckets if prev is None else (prev * mul_prev + t * mul_cur) % buckets)
        prev = t
    return rows


def embedding(tokens, W, cfg, before=None):
    x = W["embed"].to(F64)[torch.tensor(tokens)]
    b = (cfg.get("embedding") or {}).get("bigram")
    if b:
        x = x + W["bigram"].to(F64)[torch.tensor(pair_rows(tokens, b["buckets"], b["mul_prev"], b["mul_cur"], before))]
    return x


def rotate_half(vec, position, dims, base):
    """vec [n]: entry i < dims/2 is paired with entry i + dims/2; the rest is untouched."""
    out = vec.clone()
    half = dims // 2
    for i in range(half):
        angle = position * float(base) ** (-2.0 * i / dims)
        c, s = math.cos(angle), math.sin(angle)
        out[i] = vec[i] * c - vec[i + half] * s
        out[i + half] = vec[i + half] * c + vec[i] * s
    return out


def attention_operands(h, W, p, c, eps, pos0=0, per_head_norm=False):
    """q [T, H, K], k [T, G, K] (normalised, rotated) and v [T, G*V] (not yet mixed) of inputs h [T, width]."""
    H, G, K = c["heads"], c.get("kv_heads", c["heads"]), c["dim"]
    T = h.shape[0]
    q, k, v = h @ W[p + "q"].to(F64).T, h @ W[p + "k"].to(F64).T, h @ W[p + "v"].to(F64).T
    if per_head_norm:
        q = rms_norm(q.view(T, H, K), W[p + "q.norm"].to(F64), eps)
        k = rms_norm(k.view(T, G, K), W[p + "k.norm"].to(F64), eps)
    else:
        q = rms_norm(q, W[p + "q.norm"].to(F64), eps).view(T, H, K)
        k = rms_norm(k, W[p + "k.norm"].to(F64), eps).view(T, G, K)
    rot = c.get("rot")
    if rot and rot.get("dims"):
        q = torch.stack([torch.stack([rotate_half(q[t, i], pos0 + t, rot["dims"], rot["base"]) for i in range(H)]) for t in range(T)])
        k = torch.stack([torch.stack([rotate_half(k[t, i], pos0 + t, rot["dims"], rot["base"]) for i in range(G)]) for t in range(T)])
    return q, k, v


def windowed_softmax_attention(q, k, v, scale, window):
    """q [T, H, K], k [T, G, K], v [T, G, V] of one whole sequence from position 0 -> [T, H*V].  Query i sees the keys
    j with 0 <= i - j < window."""
    T, H, _ = q.shape
    G, V = k.shape[1], v.shape[2]
    out = torch.zeros(T, H, V, dtype=F64)
    for i in range(T):
        lo = max(0, i - window + 1)
        for hd in range(H):
            g = hd // (H // G)
            s = (k[lo:i + 1, g] @ q[i, hd]) * scale
            w = torch.exp(s - s.max())
            w = w / w.sum()
            out[i, hd] = (w[:, None] * v[lo:i + 1, g]).sum(dim=0)
    return out.reshape(T, H * V)


def attention_mixer(h, W, p, c, eps, carry):
    """h [T, width] of a whole sequence -> [T, width].  `carry` is a dict that holds the first value-mixing layer's values."""
    G, V = c.get("kv_heads", c["heads"]), c.get("vdim", c["dim"])
    q, k, v = attention_operands(h, W, p, c, eps)
    if c.get("v_mix"):
        if "v_first" in carry:
            lam = float(W[p + "vmix"])
            v = (1.0 - lam) * v + lam * carry["v_first"]
        else:
            carry["v_first"] = v
    heads = windowed_softmax_attention(q, k, v.view(h.shape[0], G, V), c["scale"], c["mask"]["size"])
    gate = torch.sigmoid(h @ W[p + "g"].to(F64).T)
    return (heads * gate) @ W[p + "o"].to(F64).T


def dense_ff(h, W, p):
    a, b = h @ W[p + "gate"].to(F64).T, h @ W[p + "up"].to(F64).T
    return (a * torch.sigmoid(a) * b) @ W[p + "down"].to(F64).T


def clamped_unit(a, b, limit):
    g = torch.clamp(a, max=limit)
    u = torch.clamp(b, min=-limit, max=limit)
    return g * torch.sigmoid(1.702 * g) * (u + 1.0)


def route(h, W, p, m):
    """Sigmoid scores, the `top` largest (ties to the lower index); returns (indices [T, top], weights [T, top])."""
    z = h.to(torch.float32).to(F64) @ W[p + "router"].to(F64).T
    s = torch.sigmoid(z.to(torch.float32)).to(F64)           # the router is a 32-bit computation
    top = m["router"]["top"]
    idx = torch.zeros(h.shape[0], top, dtype=torch.long)
    for t in range(h.shape[0]):
        order = sorted(range(s.shape[1]), key=lambda e: (-float(s[t, e]), e))
        idx[t] = torch.tensor(order[:top])
    return idx, torch.gather(s, 1, idx)


def routed_ff(h, W, p, m):
    idx, wgt = route(h, W, p, m)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(idx[t].tolist(), wgt[t].tolist()):
            x = w * h[t]                                     # the weight scales the expert's input
            q = f"{p}e{e}."
            mid = clamped_unit(W[q + "gate"].to(F64) @ x, W[q + "up"].to(F64) @ x, m["expert"]["limit"])
            out[t] += W[q + "down"].to(F64) @ mid
    return out


def hyper_step(streams, y, read, mix, write):
    """streams: list of [T, width]; returns the new list: x_t <- sum_s mix[s, t] x_s + write[t] y."""
    n = len(streams)
    return [sum(float(mix[s, t]) * streams[s] for s in range(n)) + float(write[t]) * y for t in range(n)]


def hyper_read(streams, read):
    return sum(float(read[s]) * streams[s] for s in range(len(streams)))


def model(tokens, cfg, W, capture=None):
    """Logits [T, vocab] of a whole sequence.  `capture` (a list) receives the sum of the streams after every layer."""
    eps, n = cfg["norm"]["eps"], int(cfg.get("streams", 1))
    x = embedding(tokens, W, cfg)
    streams = [x.clone() for _ in range(n)]
    carry = {}
    one = torch.ones(n, dtype=F64)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        subs = [("1", lambda u, p=p, layer=layer: attention_mixer(u, W, p + "mix.", layer["mixer"], eps, carry))]
        f = layer.get("mlp")
        if f:
            if f.get("kind", "dense") == "dense":
                subs.append(("2", lambda u, p=p: dense_ff(u, W, p + "mlp.")))
            else:
                subs.append(("2", lambda u, p=p, f=f: routed_ff(u, W, p + "mlp.", f)))
        for q, fn in subs:
            has = (p + f"hc{q}.in") in W
            read = W[p + f"hc{q}.in"].to(F64) if has else one
            mix = W[p + f"hc{q}.mix"].to(F64) if has else torch.eye(n, dtype=F64)
            write = W[p + f"hc{q}.out"].to(F64) if has else one
            y = fn(rms_norm(hyper_read(streams, read), W[p + f"norm{q}"].to(F64), eps))
            streams = hyper_step(streams, y, read, mix, write)
        if capture is not None:
            capture.append(sum(streams))
    x = rms_norm(sum(streams), W["final.norm"].to(F64), eps)
    return x @ W["head"].to(F64).T * float(cfg.get("logit_scale", 1.0))
