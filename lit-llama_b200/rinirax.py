"""Rinirax: a decoder-only language model of parallel layers over a depth-averaged residual stream.

    X_0 = embed[token]
    per layer i, with its input x_i (x_0 = X_0) and h = layernorm_i(x_i):
        X_(i+1) = x_i + (mixer_i(h) + feed_forward_i(h))              one norm, both sublayers read it
        x_(i+1) = sum_(j <= i+1) dwa_i[j] X_j                          a learned average over all results so far
    logits = head(layernorm(x_L))

Layer norms have a weight and a bias.  The mixer of a layer is one of
    attention         `DifferentialAttention`: two softmax maps per head over the same values, biases and short
                      convolutions on q / k / v, interleaved rotation, grouped kv heads; with "kv_from": j the layer has
                      queries only and attends over layer j's keys and values
    mingru            `MinGRUMixer`: a gated recurrence per channel whose gates read only the current token
    latent_attention  `LatentAttention`: sliding-window softmax attention over a cached latent, rotate-half rotation with
                      YaRN-scaled frequencies
and its feed-forward (a layer may have none) is dense (`DenseMLP` with xIELU) or routed (`MoEFeedForward`: sigmoid
scores, selection bias, groups worth their two best members, top-k, weights renormalised and scaled).

Everything about a model comes from its config.json (`RiniraxConfig`) and from the shapes of its tensors.  Tensor names:
`embed`, `l<i>.norm1[.b]`, `l<i>.mix.*`, `l<i>.mlp.up|down|act` or `l<i>.mlp.router|correction|e<k>.gate|up|down`,
`l<i>.dwa`, `final.norm[.b]`, `head`; linear weights are [out, in].  The residual stream, norms, angles, attention scores
and weights, the router and the recurrence are f32 in both number formats.  What a sequence carries between steps is
declared through `state_specs()` and lives in a `SequenceStatePool`, so the `Engine` serves this model like any other."""
import json
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

from . import _seqlib as S
from .mixers import DenseMLP, DepthAverage, DifferentialAttention, LatentAttention, MinGRUMixer, MoEFeedForward, StepContext, _p, linear_f32, norm_rows
from .state import StateSpec

MIXERS = ("attention", "mingru", "latent_attention")
FEED_FORWARDS = ("dense", "moe")
DEFAULT_MAX_POSITIONS = 4096
GROUP_TOP = 2              # a group of experts is worth the sum of this many of its best choice scores


@dataclass
class RiniraxConfig:
    vocab: int
    width: int
    eps: float
    layers: List[dict] = field(default_factory=list)

    @classmethod
    def from_dict(cls, d: dict) -> "RiniraxConfig":
        if d.get("architecture") not in (None, "Rinirax"):
            raise ValueError(f"not a Rinirax configuration: architecture = {d.get('architecture')!r}")
        layers = list(d["layers"])
        for i, layer in enumerate(layers):
            if layer["type"] not in MIXERS:
                raise ValueError(f"layer {i}: unknown layer type {layer['type']!r}")
            mlp = layer.get("mlp")
            if mlp and mlp.get("kind", "dense") not in FEED_FORWARDS:
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
            j = layer["mixer"].get("kv_from")
            if j is not None:
                ok = layer["type"] == "attention" and 0 <= int(j) < i and layers[int(j)]["type"] == "attention" and \
                    layers[int(j)]["mixer"].get("kv_from") is None
                if not ok:
                    raise ValueError(f"layer {i}: kv_from = {j!r} does not name an earlier attention layer with keys and values of its own")
        return cls(vocab=int(d["vocab"]), width=int(d["width"]), eps=float(d["norm"]["eps"]), layers=layers)

    @classmethod
    def from_json(cls, path: str) -> "RiniraxConfig":
        with open(path) as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> dict:
        return {"architecture": "Rinirax", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps}, "layers": self.layers}


def build_mixer(name: str, kind: str, c: dict, W: Dict[str, torch.Tensor], p: str, eps: float, max_positions: int, earlier: List["_Layer"]):
    if kind == "attention":
        j = c.get("kv_from")
        return DifferentialAttention(name, W, p, heads=c["heads"], kv_heads=c.get("kv_heads", c["heads"]), dim=c["dim"], vdim=c.get("vdim", c["dim"]),
                                     scale=c["scale"], diff=c["diff"], eps=eps, conv=c.get("conv", 0), rot=c.get("rot"), max_positions=max_positions,
                                     kv_from=earlier[int(j)].mixer if j is not None else None, interleaved=True)
    if kind == "mingru":
        return MinGRUMixer(name, W, p, width=c["width"])
    if kind == "latent_attention":
        return LatentAttention(name, W, p, heads=c["heads"], dim=c["dim"], rot_dim=c.get("rot_dim", 0), vdim=c["vdim"], q_rank=c["q_rank"],
                               kv_rank=c["kv_rank"], scale=c["scale"], eps=eps, rot=c.get("rot"), max_positions=max_positions, interleaved=False,
                               window=(c.get("mask") or {}).get("size"))
    raise ValueError(kind)


def build_feed_forward(m: dict, W: Dict[str, torch.Tensor], p: str):
    if m.get("kind", "dense") == "dense":
        return DenseMLP(W[p + "up"], W[p + "down"], act="xielu", params=W[p + "act"])
    r = m["router"]
    g = r.get("groups") or {}
    return MoEFeedForward(W, p, experts=r["experts"], identity=0, top=r["top"], groups=g.get("count", 1), keep=g.get("keep", 1), ff=m["expert"]["ff"],
                          act="silu", score="sigmoid", renormalize=True, weight_on="output", group_top=GROUP_TOP, weight_scale=r.get("scale", 1.0))


class _Layer:
    def __init__(self, i: int, spec: dict, W: Dict[str, torch.Tensor], eps: float, max_positions: int, earlier: List["_Layer"]) -> None:
        p = f"l{i}."
        self.mixer = build_mixer(f"l{i}", spec["type"], spec["mixer"], W, p + "mix.", eps, max_positions, earlier)
        self.mlp = build_feed_forward(spec["mlp"], W, p + "mlp.") if spec.get("mlp") else None
        self.norm, self.norm_b = W[p + "norm1"].contiguous(), W[p + "norm1.b"].contiguous()
        self.dwa = W.get(p + "dwa")


class Rinirax:
    """The model over a dict of device tensors in the activation dtype (torch.bfloat16, or torch.float32 for true
    32-bit arithmetic throughout).  `max_positions`: the most positions a sequence may reach (the attention layers cache
    every position)."""

    graph_safe = True

    def __init__(self, config: RiniraxConfig, weights: Dict[str, torch.Tensor], max_positions: int = 0) -> None:
        self.config = config
        self.embed = weights["embed"].contiguous()
        self.dtype, self.device = self.embed.dtype, self.embed.device
        if not self.embed.is_cuda:
            raise RuntimeError("Rinirax runs on CUDA only (no CPU fallback)")
        S.act_code(self.dtype)
        if tuple(self.embed.shape) != (config.vocab, config.width):
            raise ValueError(f"embed is {tuple(self.embed.shape)}, the configuration says {(config.vocab, config.width)}")
        self.vocab, self.width, self.eps = config.vocab, config.width, config.eps
        self.max_positions = int(max_positions) if max_positions and max_positions > 0 else DEFAULT_MAX_POSITIONS
        self.layers: List[_Layer] = []
        for i, spec in enumerate(config.layers):
            self.layers.append(_Layer(i, spec, weights, config.eps, self.max_positions, self.layers))
        self.depth = DepthAverage([layer.dwa for layer in self.layers])
        self.final_norm, self.final_norm_b = weights["final.norm"].contiguous(), weights["final.norm.b"].contiguous()
        self.head = weights["head"].contiguous()
        self.capture_layers: Optional[List[torch.Tensor]] = None     # set to [] to record the residual stream after every layer

    # ------------------------------------------------------------------ framework interface
    def state_specs(self) -> Dict[str, StateSpec]:
        out: Dict[str, StateSpec] = {}
        for layer in self.layers:
            out.update(layer.mixer.state_specs())
        return out

    def n_parameters(self) -> Tuple[int, int]:
        """(all parameters, parameters a token uses): matrices only."""
        total = active = self.embed.numel() + self.head.numel()
        for layer in self.layers:
            m = layer.mixer
            n = sum(v.numel() for k, v in vars(m).items() if isinstance(v, torch.Tensor) and v.dim() >= 2 and k not in ("w_expand", "w_conv"))
            total, active = total + n, active + n
            f = layer.mlp
            if isinstance(f, DenseMLP):
                n = f.w_up.numel() + f.w_down.numel()
                total, active = total + n, active + n
            elif f is not None:
                per = (f.w_gu.numel() + f.w_down.numel()) // max(f.E, 1)
                total, active = total + per * f.E + f.w_router.numel(), active + per * f.top + f.w_router.numel()
        return total, active

    @torch.no_grad()
    def forward_portion(self, tokens: torch.Tensor, ctx: StepContext, want: Optional[torch.Tensor] = None) -> torch.Tensor:
        """tokens: device int32/int64 [T], the next T tokens of the sequence in ctx's slot.  want: device int32 indices
        into the portion (None = every token).  Returns f32 logits [len(want), vocab]."""
        lib, T, D, dev = S.lib(), ctx.T, self.width, self.device
        if torch.backends.cuda.matmul.allow_tf32:
            raise RuntimeError("32-bit products of this model (router, float32 mode) must be true f32: torch.backends.cuda.matmul.allow_tf32 is on")
        hist = self.depth.history(ctx, D, dev)                      # [layers + 1, T, D]: the embedding output, then every layer's own result
        x = hist[0]
        S.check(lib.b2l_seq_embed(_p(tokens), int(tokens.dtype == torch.int64), _p(self.embed), ctx.act, 1.0, _p(x), T, D, self.vocab, ctx.stream),
                "b2l_seq_embed")
        n = T if want is None else int(want.numel())
        L = len(self.layers)
        fuse_last = T == 1 and n == 1 and L > 0                     # a single token: the last residual step and the final norm in one launch
        h = norm_rows(x, self.layers[0].norm, self.layers[0].norm_b, "layer", self.eps, ctx) if L else None
        xbuf = torch.empty((T, D), dtype=torch.float32, device=dev) if L else x
        hn = None
        for i, layer in enumerate(self.layers):
            y1 = layer.mixer.forward(h, ctx)
            y2 = layer.mlp.forward(h, ctx) if layer.mlp is not None else None
            if i + 1 < L:
                nxt = self.layers[i + 1]
                h = self.depth.step(i, hist, x, xbuf, y1, y2, ctx, norm=nxt.norm, bias=nxt.norm_b, kind="layer", eps=self.eps)
            elif fuse_last:
                hn = self.depth.step(i, hist, x, xbuf, y1, y2, ctx, norm=self.final_norm, bias=self.final_norm_b, kind="layer", eps=self.eps)
            else:
                self.depth.step(i, hist, x, xbuf, y1, y2, ctx)
            x = xbuf
            if self.capture_layers is not None:
                self.capture_layers.append(x.clone())
        if n == 0:
            return torch.empty((0, self.vocab), dtype=torch.float32, device=dev)
        if hn is None:
            hn = norm_rows(x, self.final_norm, self.final_norm_b, "layer", self.eps, ctx, rows=want, n_rows=n)
        return linear_f32(hn, self.head)


def load(model_dir: str, dtype: torch.dtype = torch.bfloat16, device: Optional[torch.device] = None, max_positions: int = 0) -> Rinirax:
    """config.json + model.safetensors of `model_dir` -> a model on `device`."""
    from .checkpoint_io import read_safetensors

    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    config = RiniraxConfig.from_json(os.path.join(model_dir, "config.json"))
    weights = read_safetensors(os.path.join(model_dir, "model.safetensors"), device=device, float_dtype=dtype)
    return Rinirax(config, weights, max_positions=max_positions)


def random_weights(cfg: dict, device, dtype: torch.dtype = torch.bfloat16, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Random tensors with the family's names and shapes (projections ~ N(0, 1/in), norm weights around one, depth weights
    that favour the newest result), for benchmarks, tests and smoke runs."""
    import math

    g = torch.Generator(device="cpu").manual_seed(seed)
    D, W = cfg["width"], {}

    def lin(o, i):
        return (torch.randn(o, i, generator=g) / math.sqrt(i)).to(device, dtype)

    def vec(n, mean=1.0, std=0.1):
        return (mean + std * torch.randn(n, generator=g)).to(device, dtype)

    W["embed"], W["head"] = torch.randn(cfg["vocab"], D, generator=g).to(device, dtype), lin(cfg["vocab"], D)
    W["final.norm"], W["final.norm.b"] = vec(D), vec(D, 0.0)
    for i, layer in enumerate(cfg["layers"]):
        p, m, c = f"l{i}.", f"l{i}.mix.", layer["mixer"]
        W[p + "norm1"], W[p + "norm1.b"] = vec(D), vec(D, 0.0)
        if layer["type"] == "attention":
            H, G, K = c["heads"], c.get("kv_heads", c["heads"]), c["dim"]
            V, taps = c.get("vdim", K), c.get("conv", 0)
            parts = {"q": H * 2 * K} if c.get("kv_from") is not None else {"q": H * 2 * K, "k": G * 2 * K, "v": G * V}
            for n, rows in parts.items():
                W[m + n], W[m + n + ".b"] = lin(rows, D), vec(rows, 0.0)
                if taps:
                    W[m + n + ".conv"] = (torch.randn(rows, taps, generator=g) / math.sqrt(taps) + torch.eye(taps)[-1]).to(device, dtype)
            for n in ("lq1", "lk1", "lq2", "lk2"):
                W[m + n] = vec(K, 0.0, 0.3)
            W[m + "o"] = lin(D, H * V)
        elif layer["type"] == "mingru":
            n = c["width"]
            W[m + "z"], W[m + "x"], W[m + "g"], W[m + "o"] = lin(n, D), lin(n, D), lin(n, D), lin(D, n)
            W[m + "z.b"], W[m + "x.b"] = vec(n, 0.0, 0.5), vec(n, 0.0, 0.5)
        else:
            H, dn, dr, dv, rq, rk = c["heads"], c["dim"], c.get("rot_dim", 0), c["vdim"], c["q_rank"], c["kv_rank"]
            W[m + "dq"], W[m + "dq.norm"], W[m + "uq"] = lin(rq, D), vec(rq), lin(H * (dn + dr), rq)
            W[m + "dkv"], W[m + "dkv.norm"] = lin(rk + dr, D), vec(rk)
            W[m + "uk"], W[m + "uv"], W[m + "o"] = lin(H * dn, rk), lin(H * dv, rk), lin(D, H * dv)
        f = layer.get("mlp")
        if f and f.get("kind", "dense") == "dense":
            W[p + "mlp.up"], W[p + "mlp.down"], W[p + "mlp.act"] = lin(f["ff"], D), lin(D, f["ff"]), vec(2, 0.0, 0.5)
        elif f:
            r, ff = f["router"], f["expert"]["ff"]
            W[p + "mlp.router"], W[p + "mlp.correction"] = lin(r["experts"], D), vec(r["experts"], 0.0, 0.05)
            for e in range(r["experts"]):
                q = f"{p}mlp.e{e}."
                W[q + "gate"], W[q + "up"], W[q + "down"] = lin(ff, D), lin(ff, D), lin(D, ff)
        d = 0.15 * torch.randn(i + 2, generator=g) / (i + 2)
        d[-1] += 1.0
        W[p + "dwa"] = d.to(device, dtype)
    return W
