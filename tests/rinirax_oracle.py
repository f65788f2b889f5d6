"""A plain float64 restatement of the Rinirax design, one function per mechanism, written token by token wherever a
loop is the plainest form.  It shares no code with the package: torch on the CPU only.  Weights are a dict
name -> tensor; configurations are the dicts of config.json.  Every function takes a whole sequence from position 0."""
import math

import torch

F64 = torch.float64


def w64(W, name):
    return W[name].to(F64)


# ---------------------------------------------------------------------------------------------- norms
def rms_norm(x, w, eps):
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if w is None else y * w


def layer_norm(x, w, b, eps):
    mu = x.mean(dim=-1, keepdim=True)
    var = ((x - mu) ** 2).mean(dim=-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


# ---------------------------------------------------------------------------------------------- short convolution
def causal_conv(u, w):
    """u [T, C], w [C, taps]: y[t] = sum_j w[:, j] * u[t - (taps - 1) + j], zeros before the start."""
    T, taps = u.shape[0], w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            s = t - (taps - 1) + j
            if s >= 0:
                y[t] += w[:, j] * u[s]
    return y


# ---------------------------------------------------------------------------------------------- rotations
def plain_frequencies(dims, base):
    return [float(base) ** (-2.0 * i / dims) for i in range(dims // 2)], 1.0


def yarn_frequencies(dims, base, scaling):
    """Frequencies stretched by `factor` where a pair turns slowly, kept where it turns fast, blended between."""
    f, _ = plain_frequencies(dims, base)
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def turns_to_dim(t):
        return dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(float(base)))

    lo = max(math.floor(turns_to_dim(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turns_to_dim(float(scaling["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate(vec, position, freqs, mult, interleaved):
    """vec [n]: the first 2 * len(freqs) entries turn by position * freqs[i]; pair (2i, 2i+1) or (i, i + half)."""
    out = vec.clone()
    half = len(freqs)
    for i, f in enumerate(freqs):
        a, b = (2 * i, 2 * i + 1) if interleaved else (i, i + half)
        c, s = math.cos(position * f) * mult, math.sin(position * f) * mult
        out[a] = vec[a] * c - vec[b] * s
        out[b] = vec[b] * c + vec[a] * s
    return out


# ---------------------------------------------------------------------------------------------- differential attention
def diff_lambda(W, p, diff):
    return math.exp(float((w64(W, p + "lq1") * w64(W, p + "lk1")).sum())) - math.exp(float((w64(W, p + "lq2") * w64(W, p + "lk2")).sum())) + diff


def diff_queries(h, W, p, c):
    """[T, H, 2, dim]: projection + bias, convolution, rotation."""
    T, H, K = h.shape[0], c["heads"], c["dim"]
    q = h @ w64(W, p + "q").T + w64(W, p + "q.b")
    if c.get("conv"):
        q = causal_conv(q, w64(W, p + "q.conv"))
    q = q.view(T, H, 2, K).clone()
    rot = c.get("rot")
    if rot and rot.get("dims"):
        f, mult = plain_frequencies(rot["dims"], rot["base"])
        for t in range(T):
            for i in range(H):
                for m in range(2):
                    q[t, i, m] = rotate(q[t, i, m], t, f, mult, True)
    return q


def diff_keys_values(h, W, p, c):
    """k [T, G, 2, dim] (convolved, rotated) and v [T, G, vdim] (convolved)."""
    T, G, K, V = h.shape[0], c.get("kv_heads", c["heads"]), c["dim"], c.get("vdim", c["dim"])
    k = h @ w64(W, p + "k").T + w64(W, p + "k.b")
    v = h @ w64(W, p + "v").T + w64(W, p + "v.b")
    if c.get("conv"):
        k, v = causal_conv(k, w64(W, p + "k.conv")), causal_conv(v, w64(W, p + "v.conv"))
    k = k.view(T, G, 2, K).clone()
    rot = c.get("rot")
    if rot and rot.get("dims"):
        f, mult = plain_frequencies(rot["dims"], rot["base"])
        for t in range(T):
            for g in range(G):
                for m in range(2):
                    k[t, g, m] = rotate(k[t, g, m], t, f, mult, True)
    return k, v.view(T, G, V)


def differential_attention(h, W, p, c, eps, kv=None):
    """h [T, width] -> ([T, width], (k, v)).  `kv`: keys and values of another layer instead of this layer's own."""
    T, H, G, V = h.shape[0], c["heads"], c.get("kv_heads", c["heads"]), c.get("vdim", c["dim"])
    q = diff_queries(h, W, p, c)
    k, v = kv if kv is not None else diff_keys_values(h, W, p, c)
    lam, diff = diff_lambda(W, p, c["diff"]), c["diff"]
    heads = torch.zeros(T, H, V, dtype=F64)
    for i in range(T):
        for hd in range(H):
            g = hd // (H // G)
            maps = []
            for m in range(2):
                s = (k[:i + 1, g, m] @ q[i, hd, m]) * c["scale"]
                w = torch.exp(s - s.max())
                w = w / w.sum()
                maps.append((w[:, None] * v[:i + 1, g]).sum(dim=0))
            o = maps[0] - lam * maps[1]
            heads[i, hd] = rms_norm(o, None, eps) * (1.0 - diff)
    return heads.reshape(T, H * V) @ w64(W, p + "o").T, (k, v)


# ---------------------------------------------------------------------------------------------- minGRU
def mingru(h, W, p):
    z = torch.sigmoid(h @ w64(W, p + "z").T + w64(W, p + "z.b"))
    u = h @ w64(W, p + "x").T + w64(W, p + "x.b")
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    g = h @ w64(W, p + "g").T
    state = torch.zeros(z.shape[1], dtype=F64)
    out = torch.zeros_like(z)
    for t in range(h.shape[0]):
        state = (1.0 - z[t]) * state + z[t] * cand[t]
        out[t] = state * (g[t] * torch.sigmoid(g[t]))
    return out @ w64(W, p + "o").T


# ---------------------------------------------------------------------------------------------- latent attention
def latent_attention(h, W, p, c, eps):
    T, H, dn, dr, dv, rk = h.shape[0], c["heads"], c["dim"], c.get("rot_dim", 0), c["vdim"], c["kv_rank"]
    cq = rms_norm(h @ w64(W, p + "dq").T, w64(W, p + "dq.norm"), eps)
    q = (cq @ w64(W, p + "uq").T).view(T, H, dn + dr)
    down = h @ w64(W, p + "dkv").T
    lat = rms_norm(down[:, :rk], w64(W, p + "dkv.norm"), eps)
    kr = down[:, rk:rk + dr].clone()
    kn = (lat @ w64(W, p + "uk").T).view(T, H, dn)
    v = (lat @ w64(W, p + "uv").T).view(T, H, dv)
    qr = q[:, :, dn:].clone()
    rot = c.get("rot")
    if rot and dr:
        f, mult = yarn_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        for t in range(T):
            kr[t] = rotate(kr[t], t, f, mult, False)
            for i in range(H):
                qr[t, i] = rotate(qr[t, i], t, f, mult, False)
    window = (c.get("mask") or {}).get("size")
    out = torch.zeros(T, H, dv, dtype=F64)
    for i in range(T):
        lo = max(0, i - window + 1) if window else 0
        for hd in range(H):
            s = (kn[lo:i + 1, hd] @ q[i, hd, :dn] + kr[lo:i + 1] @ qr[i, hd]) * c["scale"]
            w = torch.exp(s - s.max())
            w = w / w.sum()
            out[i, hd] = (w[:, None] * v[lo:i + 1, hd]).sum(dim=0)
    return out.reshape(T, H * dv) @ w64(W, p + "o").T


# ---------------------------------------------------------------------------------------------- feed-forward
def softplus(x):
    return math.log1p(math.exp(x)) if x < 30 else x


def xielu(z, a_pos, a_neg):
    pos = softplus(a_pos) * z * z + 0.5 * z
    neg = (0.5 + softplus(a_neg)) * (torch.expm1(torch.clamp(z, max=0.0)) - z) + 0.5 * z
    return torch.where(z > 0, pos, neg)


def dense_ff(h, W, p):
    a = w64(W, p + "act")
    return xielu(h @ w64(W, p + "up").T, float(a[0]), float(a[1])) @ w64(W, p + "down").T


def route(h, W, p, r):
    """Indices [T, top] and weights [T, top].  Sigmoid scores; choice = score + correction; a group of neighbours is
    worth the sum of its two largest choice scores and only the best groups' experts can be chosen."""
    z = (h.to(torch.float32).to(F64) @ w64(W, p + "router").T).to(torch.float32)
    s = torch.sigmoid(z).to(F64)
    corr = w64(W, p + "correction") if (p + "correction") in W else torch.zeros(s.shape[1], dtype=F64)
    E, top = s.shape[1], r["top"]
    groups = r.get("groups") or {}
    count, keep = int(groups.get("count", 1)), int(groups.get("keep", 1))
    per = E // count
    idx = torch.zeros(h.shape[0], top, dtype=torch.long)
    wgt = torch.zeros(h.shape[0], top, dtype=F64)
    for t in range(h.shape[0]):
        choice = [float(s[t, e] + corr[e]) for e in range(E)]
        if count > 1:
            worth = []
            for g in range(count):
                best = sorted(choice[g * per:(g + 1) * per], reverse=True)[:2]
                worth.append(sum(best))
            kept = sorted(range(count), key=lambda g: (-worth[g], g))[:keep]
            for e in range(E):
                if e // per not in kept:
                    choice[e] = -math.inf
        order = sorted(range(E), key=lambda e: (-choice[e], e))[:top]
        idx[t] = torch.tensor(order)
        chosen = s[t, order]
        wgt[t] = chosen / (chosen.sum() + 1e-20) * float(r.get("scale", 1.0))
    return idx, wgt


def routed_ff(h, W, p, m):
    idx, wgt = route(h, W, p, m["router"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(idx[t].tolist(), wgt[t].tolist()):
            q = f"{p}e{e}."
            a, b = w64(W, q + "gate") @ h[t], w64(W, q + "up") @ h[t]
            out[t] += w * (w64(W, q + "down") @ (a * torch.sigmoid(a) * b))
    return out


# ---------------------------------------------------------------------------------------------- the model
def model(tokens, cfg, W, capture=None):
    """Logits [T, vocab] of a whole sequence.  `capture` (a list) receives the residual stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = w64(W, "embed")[torch.tensor(tokens)]
    history = [x]                                  # the embedding output and every layer's own result
    kv = {}
    for i, layer in enumerate(cfg["layers"]):
        p, c = f"l{i}.", layer["mixer"]
        h = layer_norm(x, w64(W, p + "norm1"), w64(W, p + "norm1.b"), eps)
        if layer["type"] == "attention":
            src = c.get("kv_from")
            y, kv[i] = differential_attention(h, W, p + "mix.", c, eps, kv=kv[src] if src is not None else None)
        elif layer["type"] == "mingru":
            y = mingru(h, W, p + "mix.")
        elif layer["type"] == "latent_attention":
            y = latent_attention(h, W, p + "mix.", c, eps)
        else:
            raise ValueError(layer["type"])
        f = layer.get("mlp")
        if f:
            y = y + (dense_ff(h, W, p + "mlp.") if f.get("kind", "dense") == "dense" else routed_ff(h, W, p + "mlp.", f))
        history.append(x + y)
        if (p + "dwa") in W:
            d = w64(W, p + "dwa")
            x = sum(float(d[j]) * history[j] for j in range(len(history)))
        else:
            x = history[-1]
        if capture is not None:
            capture.append(x)
    x = layer_norm(x, w64(W, "final.norm"), w64(W, "final.norm.b"), eps)
    return x @ w64(W, "head").T
