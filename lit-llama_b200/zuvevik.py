"""Zuvevik: a decoder-only language model over several residual streams.

    x_1 = ... = x_S = embed[token] + pair[hash(previous token, token)]          (`PairHashEmbedding`)
    per layer, for the mixer and then for the feed-forward (a layer may have none), with that sublayer's
    hyper-connection weights (read r, mix M indexed [from, to], write o):
        u = sum_s r[s] x_s;   y = sublayer(rmsnorm(u) * w);   x_t <- sum_s M[s, t] x_s + o[t] y   for all t at once
    logits = head(rmsnorm(sum_s x_s) * w_final) * logit_scale

The mixer is sliding-window attention (`SlidingWindowAttention`: q/k norm over the whole projection, partial
rotation, grouped kv heads, values mixed with those of the first value-mixing layer, a sigmoid gate per output channel).
The feed-forward is a dense gated unit with silu (`GatedMLP`) or routed experts (`MoEFeedForward`: sigmoid scores,
the `top` largest chosen, the score itself as weight on the expert's INPUT, clamped gated unit).  With one stream and
no hyper-connection tensors a layer is the ordinary pre-norm residual layer.

Everything about a model comes from its config.json (`ZuvevikConfig`) and from the shapes of its tensors.  Tensor
names: `embed`, `bigram`, `l<i>.norm1|norm2`, `l<i>.hc1|hc2.in|mix|out`, `l<i>.mix.q|k|v|g|o|q.norm|k.norm|vmix`,
`l<i>.mlp.gate|up|down` or `l<i>.mlp.router|e<k>.gate|up|down`, `final.norm`, `head`; linear weights are [out, in].
The residual streams, norms, angles, attention scores and weights and the router are f32 in both number formats.  What
a sequence carries between steps (a ring of keys and values per attention layer, its last token) is declared through
`state_specs()` and lives in a `SequenceStatePool`, so the `Engine` serves this model like any other."""
import json
import os
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Tuple

import torch

from . import _seqlib as S
from .mixers import GatedMLP, HyperConnection, MoEFeedForward, PairHashEmbedding, SlidingWindowAttention, StepContext, _p, linear_f32
from .state import StateSpec

MIXERS = ("attention",)
FEED_FORWARDS = ("dense", "moe")


@dataclass
class ZuvevikConfig:
    vocab: int
    width: int
    eps: float
    streams: int
    logit_scale: float
    bigram: Optional[dict]
    layers: List[dict] = field(default_factory=list)

    @classmethod
    def from_dict(cls, d: dict) -> "ZuvevikConfig":
        if d.get("architecture") not in (None, "Zuvevik"):
            raise ValueError(f"not a Zuvevik configuration: architecture = {d.get('architecture')!r}")
        layers = list(d["layers"])
        for i, layer in enumerate(layers):
            if layer["type"] not in MIXERS:
                raise ValueError(f"layer {i}: unknown layer type {layer['type']!r}")
            mlp = layer.get("mlp")
            if mlp and mlp.get("kind", "dense") not in FEED_FORWARDS:
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
            if not (layer["mixer"].get("mask") or {}).get("size"):
                raise ValueError(f"layer {i}: attention without a window size")
        bigram = (d.get("embedding") or {}).get("bigram")
        streams = int(d.get("streams", 1))
        if streams < 1:
            raise ValueError(f"streams = {streams}")
        return cls(vocab=int(d["vocab"]), width=int(d["width"]), eps=float(d["norm"]["eps"]), streams=streams,
                   logit_scale=float(d.get("logit_scale", 1.0)), bigram=dict(bigram) if bigram else None, layers=layers)

    @classmethod
    def from_json(cls, path: str) -> "ZuvevikConfig":
        with open(path) as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> dict:
        out = {"architecture": "Zuvevik", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps}, "streams": self.streams,
               "logit_scale": self.logit_scale, "layers": self.layers}
        if self.bigram:
            out["embedding"] = {"bigram": self.bigram}
        return out


def build_mixer(name: str, c: dict, W: Dict[str, torch.Tensor], p: str, eps: float) -> SlidingWindowAttention:
    return SlidingWindowAttention(name, W, p, heads=c["heads"], kv_heads=c.get("kv_heads", c["heads"]), dim=c["dim"], vdim=c.get("vdim", c["dim"]),
                                  scale=c["scale"], window=c["mask"]["size"], eps=eps, rot=c.get("rot"), v_mix=bool(c.get("v_mix")),
                                  norm_over="row")


def build_feed_forward(m: dict, W: Dict[str, torch.Tensor], p: str):
    if m.get("kind", "dense") == "dense":
        return GatedMLP(W[p + "gate"], W[p + "up"], W[p + "down"], act="silu")
    r = m["router"]
    return MoEFeedForward(W, p, experts=r["experts"], identity=0, top=r["top"], groups=1, keep=1, ff=m["expert"]["ff"], act="clamped_swish",
                          limit=m["expert"]["limit"], score="sigmoid", renormalize=False, weight_on="input")


class _Sublayer:
    def __init__(self, hc: HyperConnection, norm: torch.Tensor, run: Callable[[torch.Tensor, StepContext], torch.Tensor]) -> None:
        self.hc, self.norm, self.run = hc, norm, run


class _Layer:
    def __init__(self, i: int, spec: dict, W: Dict[str, torch.Tensor], eps: float, streams: int) -> None:
        p = f"l{i}."
        self.mixer = build_mixer(f"l{i}", spec["mixer"], W, p + "mix.", eps)
        self.mlp = build_feed_forward(spec["mlp"], W, p + "mlp.") if spec.get("mlp") else None
        dev = self.mixer.w_o.device

        def hc(q: int) -> HyperConnection:
            if (p + f"hc{q}.in") in W:
                return HyperConnection(W[p + f"hc{q}.in"], W[p + f"hc{q}.mix"], W[p + f"hc{q}.out"])
            return HyperConnection.plain(dev, streams)

        self.sublayers = [_Sublayer(hc(1), W[p + "norm1"].contiguous(), self.mixer.forward)]
        if self.mlp is not None:
            self.sublayers.append(_Sublayer(hc(2), W[p + "norm2"].contiguous(), self.mlp.forward))
        for sub in self.sublayers:
            if sub.hc.streams != streams:
                raise ValueError(f"layer {i}: hyper-connection weights for {sub.hc.streams} streams, the model has {streams}")


class Zuvevik:
    """The model over a dict of device tensors in the activation dtype (torch.bfloat16, or torch.float32 for true
    32-bit arithmetic throughout).  Attention keeps a ring of its window per sequence, so a sequence has no position
    limit."""

    graph_safe = True

    def __init__(self, config: ZuvevikConfig, weights: Dict[str, torch.Tensor], max_positions: int = 0) -> None:
        self.config = config
        embed = weights["embed"]
        self.dtype, self.device = embed.dtype, embed.device
        if not embed.is_cuda:
            raise RuntimeError("Zuvevik runs on CUDA only (no CPU fallback)")
        S.act_code(self.dtype)
        if tuple(embed.shape) != (config.vocab, config.width):
            raise ValueError(f"embed is {tuple(embed.shape)}, the configuration says {(config.vocab, config.width)}")
        self.vocab, self.width, self.eps, self.streams = config.vocab, config.width, config.eps, config.streams
        b = config.bigram
        self.embedding = PairHashEmbedding("bigram", embed, weights["bigram"] if b else None, buckets=b["buckets"] if b else 0,
                                           mul_prev=b["mul_prev"] if b else 0, mul_cur=b["mul_cur"] if b else 0, streams=config.streams)
        self.layers = [_Layer(i, spec, weights, config.eps, config.streams) for i, spec in enumerate(config.layers)]
        self.sublayers: List[_Sublayer] = [s for layer in self.layers for s in layer.sublayers]
        self._layer_end = set()                                   # indices of the sublayers that end a layer
        at = 0
        for layer in self.layers:
            at += len(layer.sublayers)
            self._layer_end.add(at - 1)
        self.final_norm, self.head = weights["final.norm"].contiguous(), weights["head"].contiguous()
        self.ones = torch.ones(config.streams, dtype=torch.float32, device=self.device)      # read weights of the final sum
        self.capture_layers: Optional[List[torch.Tensor]] = None     # set to [] to record the sum of the streams after every layer

    # ------------------------------------------------------------------ framework interface
    def state_specs(self) -> Dict[str, StateSpec]:
        out: Dict[str, StateSpec] = dict(self.embedding.state_specs())
        for layer in self.layers:
            out.update(layer.mixer.state_specs())
        return out

    def n_parameters(self) -> Tuple[int, int]:
        """(all parameters, parameters a token uses)."""
        total = active = self.embedding.embed.numel() + self.head.numel() + (self.embedding.pair.numel() if self.embedding.pair is not None else 0)
        for layer in self.layers:
            m = layer.mixer
            n = m.w_in.numel() + m.w_o.numel()
            total, active = total + n, active + n
            f = layer.mlp
            if isinstance(f, GatedMLP):
                n = f.w_in.numel() + f.w_down.numel()
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
        x = self.embedding.forward(tokens, ctx)                    # [T, streams, D] f32
        subs = self.sublayers
        h = HyperConnection.step(x, ctx, reads=subs[0].hc, norm=subs[0].norm, eps=self.eps) if subs else None
        n = T if want is None else int(want.numel())
        hn = None
        for j, sub in enumerate(subs):
            y = sub.run(h, ctx)
            last = j + 1 == len(subs)
            if last and T == 1 and n == 1:                          # a single token: the last write, the sum and the final norm in one launch
                hn = HyperConnection.step(x, ctx, y=y, wrote=sub.hc, read_weights=self.ones, norm=self.final_norm, eps=self.eps)
            elif last:
                HyperConnection.step(x, ctx, y=y, wrote=sub.hc)
            else:
                h = HyperConnection.step(x, ctx, y=y, wrote=sub.hc, reads=subs[j + 1].hc, norm=subs[j + 1].norm, eps=self.eps)
            if self.capture_layers is not None and j in self._layer_end:
                xs = torch.empty((T, D), dtype=torch.float32, device=dev)
                S.check(lib.b2l_seq_hc_sum(_p(x), _p(xs), T, D, self.streams, ctx.stream), "b2l_seq_hc_sum")
                self.capture_layers.append(xs)
        if n == 0:
            return torch.empty((0, self.vocab), dtype=torch.float32, device=dev)
        if hn is None:
            hn = HyperConnection.step(x, ctx, read_weights=self.ones, norm=self.final_norm, eps=self.eps, rows=want, n_rows=n)
        logits = linear_f32(hn, self.head)
        if self.config.logit_scale != 1.0:
            S.check(lib.b2l_seq_scale(_p(logits), logits.numel(), self.config.logit_scale, ctx.stream), "b2l_seq_scale")
        return logits


def load(model_dir: str, dtype: torch.dtype = torch.bfloat16, device: Optional[torch.device] = None, max_positions: int = 0) -> Zuvevik:
    """config.json + model.safetensors of `model_dir` -> a model on `device`."""
    from .checkpoint_io import read_safetensors

    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    config = ZuvevikConfig.from_json(os.path.join(model_dir, "config.json"))
    weights = read_safetensors(os.path.join(model_dir, "model.safetensors"), device=device, float_dtype=dtype)
    return Zuvevik(config, weights, max_positions=max_positions)


def random_weights(cfg: dict, device, dtype: torch.dtype = torch.bfloat16, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Random tensors with the family's names and shapes (projections ~ N(0, 1/in), norm weights around one, stream
    mixing near the identity), for benchmarks, tests and smoke runs."""
    import math

    g = torch.Generator(device="cpu").manual_seed(seed)
    D, s, W = cfg["width"], int(cfg.get("streams", 1)), {}

    def lin(o, i):
        return (torch.randn(o, i, generator=g) / math.sqrt(i)).to(device, dtype)

    def vec(n, mean=1.0, std=0.1):
        return (mean + std * torch.randn(n, generator=g)).to(device, dtype)

    W["embed"], W["head"], W["final.norm"] = torch.randn(cfg["vocab"], D, generator=g).to(device, dtype), lin(cfg["vocab"], D), vec(D)
    b = (cfg.get("embedding") or {}).get("bigram")
    if b:
        W["bigram"] = (0.5 * torch.randn(b["buckets"] + 1, D, generator=g)).to(device, dtype)
    for i, layer in enumerate(cfg["layers"]):
        p, m, c = f"l{i}.", f"l{i}.mix.", layer["mixer"]
        H, G, K = c["heads"], c.get("kv_heads", c["heads"]), c["dim"]
        V = c.get("vdim", K)
        W[p + "norm1"] = vec(D)
        W[m + "q"], W[m + "k"], W[m + "v"], W[m + "g"], W[m + "o"] = lin(H * K, D), lin(G * K, D), lin(G * V, D), lin(H * V, D), lin(D, H * V)
        W[m + "q.norm"], W[m + "k.norm"] = vec(H * K), vec(G * K)
        W[m + "vmix"] = (0.3 + 0.4 * torch.rand((), generator=g)).to(device, dtype)
        f = layer.get("mlp")
        if f:
            W[p + "norm2"] = vec(D)
            if f.get("kind", "dense") == "dense":
                W[p + "mlp.gate"], W[p + "mlp.up"], W[p + "mlp.down"] = lin(f["ff"], D), lin(f["ff"], D), lin(D, f["ff"])
            else:
                W[p + "mlp.router"] = lin(f["router"]["experts"], D)
                for e in range(f["router"]["experts"]):
                    q, ff = f"{p}mlp.e{e}.", f["expert"]["ff"]
                    W[q + "gate"], W[q + "up"], W[q + "down"] = lin(ff, D), lin(ff, D), lin(D, ff)
        if "streams" in cfg:
            for q in (1, 2) if f else (1,):
                W[p + f"hc{q}.in"] = (1.0 / s + 0.2 * torch.randn(s, generator=g)).to(device, dtype)
                W[p + f"hc{q}.out"] = (1.0 + 0.3 * torch.randn(s, generator=g)).to(device, dtype) / s
                W[p + f"hc{q}.mix"] = (torch.eye(s) + 0.15 * torch.randn(s, s, generator=g)).to(device, dtype)
    return W
