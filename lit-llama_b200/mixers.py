"""Sequence-mixer mechanisms over libb200seq (include/b2l_seq.h), each usable by any model: its sizes and
constants are constructor parameters.

    GatedMLP             act(W_gate h) * (W_up h) -> W_down, both halves from one product
    ChannelDeltaMixer    gated delta rule with one decay per key channel, short convolutions on q / k / v
    BlockSinkAttention   block-local causal softmax attention: q/k norm, partial rotation (YaRN-scaled), soft-capped
                         scores, a sink in the denominator, grouped kv heads, per-head sigmoid output gate, ring cache
    GatedLinearAttention S_t = diag(alpha_t) S_(t-1) + k_t v_t^T with a low-rank decay projection
    ParallelMixer        two mixers on the same input, one output product over their concatenated read-outs
    Mamba2Mixer          state-space duality layer: scalar decay per head, convolution on x | B | C, gated grouped norm
    LatentAttention      causal softmax attention whose keys and values are linear images of one cached latent per position
                         (+ one rotated key part shared by the heads), low-rank queries, a learned sink per head
    RetentionMixer       linear attention with a fixed decay per head, rotated q / k, per-head unit-RMS read-out, silu gate
    MoEFeedForward       routed gated experts: softmax or sigmoid scores, selection bias, expert groups, top-k, identity
                         experts, weights renormalised or not, on an expert's output or on its input, clamped gated unit
    SlidingWindowAttention  causal softmax attention over the last `window` positions: q/k norm over the whole projection
                         or per head, partial rotation, grouped kv heads, values mixed with an earlier layer's, a sigmoid
                         gate per output channel, ring cache of `window` positions
    PairHashEmbedding    token embedding plus a hashed (previous token, token) embedding, into several residual streams
    HyperConnection      one sublayer's read weights, stream-mixing matrix and write weights over several residual streams
    DenseMLP             W_down act(W_up h) without a gate: gelu_tanh, silu, or xIELU with its two learned numbers
    DifferentialAttention  causal softmax attention with two score maps per head over the same values, combined as
                         a0 - lambda a1 and divided by its root mean square; biases and short convolutions on q / k / v,
                         interleaved rotation, grouped kv heads, keys and values of its own or of an earlier layer
    MinGRUMixer          S_t = (1 - z_t) S_(t-1) + z_t c_t per channel with gates that read only the current token, silu gate
    DepthAverage         the residual step of layers whose input is a learned average over all earlier layers' results

A mixer is built from a dict of weight tensors (`from_weights`) and runs one portion of one sequence:
`forward(h, ctx)` with h [T, width] in the model's activation dtype.  Products go through torch (cuBLAS), as the
dense linears of the package's LLaMA do; everything else is a kernel of libb200seq.  What a mixer carries between
tokens is declared by `state_specs()` and lives in a `SequenceStatePool`.  CUDA only; no CPU fallback."""
import ctypes as C
import math
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn.functional as F

from . import _seqlib as S
from .state import StateSpec


class StepContext:
    """One portion of one sequence: T tokens, the device pair {slot, first position} and the slot pool's tensors.
    `pos_hint` / `slot_hint` are the first position and the slot as the host knows them (None inside a captured step,
    which must not depend on them): kernels never read them, they size grids and pick between equivalent forms."""

    def __init__(self, T: int, meta: torch.Tensor, state: Dict[str, torch.Tensor], dtype: torch.dtype, pos_hint: Optional[int] = None,
                 slot_hint: Optional[int] = None) -> None:
        self.T, self.meta, self.state, self.dtype, self.pos_hint, self.slot_hint = T, meta, state, dtype, pos_hint, slot_hint
        self.act = S.act_code(dtype)
        self.shared: Dict[str, object] = {}      # what one layer of this step hands to later ones (values of an earlier layer, ...)

    @property
    def stream(self) -> int:
        """The current CUDA stream at the time of each launch (the capturing stream while a graph is recorded)."""
        return S.stream_ptr()


def _p(t: Optional[torch.Tensor], offset: int = 0) -> Optional[int]:
    """Device address of element `offset` of a tensor's storage view."""
    if t is None:
        return None
    return S.ptr(t) + offset * t.element_size()


def pad8(n: int) -> int:
    return (n + 7) // 8 * 8


def stack_rows(parts: List[torch.Tensor]) -> Tuple[torch.Tensor, List[int]]:
    """Linear weights that read the same input, stacked into one [sum, in] matrix.  Every part starts at a multiple
    of 8 rows (zero rows between), so each part's columns of the product start 16-byte aligned.  Returns the matrix
    and the first row of every part."""
    offs, rows, at = [], [], 0
    for w in parts:
        offs.append(at)
        rows.append(w)
        gap = pad8(w.shape[0]) - w.shape[0]
        if gap:
            rows.append(w.new_zeros((gap,) + tuple(w.shape[1:])))
        at += pad8(w.shape[0])
    return torch.cat(rows, dim=0).contiguous(), offs


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    return F.linear(x, w)


def linear_f32(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x W^T with the f32 accumulator kept (bf16 operands), or the plain f32 product."""
    if x.dtype == torch.float32:
        return F.linear(x, w)
    return torch.mm(x, w.t(), out_dtype=torch.float32)


# ------------------------------------------------------------------------------------------------ feed-forward
class GatedMLP:
    ACTS = {"gelu_tanh": S.ACT_GELU_TANH, "silu": S.ACT_SILU, "clamped_swish": S.ACT_CLAMPED_SWISH}

    def __init__(self, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, act: str = "gelu_tanh", limit: float = 0.0) -> None:
        self.ff = gate.shape[0]
        self.w_in = torch.cat([gate, up], dim=0).contiguous()
        self.w_down = down.contiguous()
        self.act, self.limit = self.ACTS[act], float(limit)

    def state_specs(self) -> Dict[str, StateSpec]:
        return {}

    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        gu = linear(h, self.w_in)
        mid = torch.empty((ctx.T, self.ff), dtype=h.dtype, device=h.device)
        S.check(S.lib().b2l_seq_gated_act(_p(gu), 2 * self.ff, _p(mid), ctx.T, self.ff, self.act, self.limit, ctx.act, ctx.stream),
                "b2l_seq_gated_act")
        return linear(mid, self.w_down)


class DenseMLP:
    """W_down act(W_up h), no gate.  act: gelu_tanh, silu, sigmoid, or xIELU with its two learned numbers `params` = (p, q):
    softplus(p) z^2 + z/2 for z > 0, (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2 otherwise."""

    ACTS = {"gelu_tanh": S.ACT_GELU_TANH, "silu": S.ACT_SILU, "sigmoid": S.ACT_SIGMOID, "xielu": S.ACT_XIELU}

    def __init__(self, up: torch.Tensor, down: torch.Tensor, act: str = "gelu_tanh", params: Optional[torch.Tensor] = None) -> None:
        if act not in self.ACTS:
            raise ValueError(f"dense feed-forward: unknown activation {act!r}")
        self.ff = up.shape[0]
        self.w_up, self.w_down = up.contiguous(), down.contiguous()
        self.act = self.ACTS[act]
        self.coef = None
        if self.act == S.ACT_XIELU:
            if params is None or params.numel() != 2:
                raise ValueError("dense feed-forward: xIELU needs its two numbers")
            pq = params.detach().reshape(-1).double().cpu()
            sp = torch.nn.functional.softplus(pq)                       # the two coefficients, once, in 64-bit; kept as f32
            self.coef = torch.stack([sp[0], 0.5 + sp[1]]).to(torch.float32).to(up.device)

    def state_specs(self) -> Dict[str, StateSpec]:
        return {}

    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        u = linear(h, self.w_up)
        S.check(S.lib().b2l_seq_unary_act(_p(u), self.ff, _p(u), self.ff, ctx.T, self.ff, self.act, _p(self.coef), ctx.act, ctx.stream),
                "b2l_seq_unary_act")                      # in place: every element is read and written by the same thread
        return linear(u, self.w_down)


# ------------------------------------------------------------------------------------------------ recurrences
def _scan(ctx: StepContext, *, q, ldq, k, ldk, v, ldv, q_mult, decay, ldd, per_channel, state, out, ldo, heads, qk_heads,
          K, V, beta=None, ldb=0, vscale=None, ldvs=0, skip=None) -> None:
    lib = S.lib()
    n_chunks = lib.b2l_seq_scan_chunks(ctx.T, int(beta is not None))
    ws = wd = None
    if n_chunks > 1:      # long portion, no delta rule: chunks in parallel (local states, combine, outputs)
        ws = torch.empty((n_chunks, heads, V, K), dtype=torch.float32, device=state.device)
        wd = torch.empty((n_chunks, heads, K if per_channel else 1), dtype=torch.float32, device=state.device)
    a = S.ScanArgs(q=q, ldq=ldq, k=k, ldk=ldk, v=v, ldv=ldv, q_mult=float(q_mult), decay=decay, ldd=ldd,
                   decay_per_channel=int(per_channel), beta=beta, ldb=ldb, delta=int(beta is not None), vscale=vscale, ldvs=ldvs,
                   skip=skip, state=_p(state), meta=_p(ctx.meta), out=out, ldo=ldo, T=ctx.T, heads=heads, qk_heads=qk_heads, K=K, V=V,
                   act_dtype=ctx.act, work_state=_p(ws), work_decay=_p(wd), n_chunks=n_chunks)
    S.check(lib.b2l_seq_scan(C.byref(a), ctx.stream), "b2l_seq_scan")


class ChannelDeltaMixer:
    """Gated delta rule, one decay per head and key channel.

        q, k, v = silu(conv(W h)); q, k unit vectors per head (q times dim^-1/2); beta = sigmoid(W_b h)
        g = exp(-exp(A_log) softplus(W_a2 W_a1 h + dt_bias))              [heads x dim]
        S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
        y = W_o (o / rms(o) * w_norm * sigmoid(W_g2 W_g1 h))
    State per sequence: S (f32, heads x vdim x dim) and the last taps-1 inputs of the convolutions."""

    def __init__(self, name: str, W: Dict[str, torch.Tensor], p: str, *, heads: int, kv_heads: int, dim: int, vdim: int, conv: int,
                 eps: float, unit_eps: float = 1e-6) -> None:
        self.name, self.H, self.G, self.K, self.V, self.taps, self.eps, self.unit_eps = name, heads, kv_heads, dim, vdim, conv, eps, unit_eps
        parts = [W[p + "q"], W[p + "k"], W[p + "v"], W[p + "b"], W[p + "a1"], W[p + "g1"]]
        self.w_in, (self.o_q, self.o_k, self.o_v, self.o_b, self.o_a1, self.o_g1) = stack_rows(parts)
        self.n_in = self.w_in.shape[0]
        self.rank_a, self.rank_g = W[p + "a1"].shape[0], W[p + "g1"].shape[0]
        self.C = self.o_b                                  # conv channels: q | k | v with their alignment gaps
        self.w_conv, _ = stack_rows([W[p + "q.conv"], W[p + "k.conv"], W[p + "v.conv"]])
        assert self.w_conv.shape == (self.C, conv)
        self.w_a2, self.w_g2 = W[p + "a2"].contiguous(), W[p + "g2"].contiguous()
        self.dt_bias, self.A_log, self.w_norm = W[p + "dt_bias"].contiguous(), W[p + "A_log"].contiguous(), W[p + "norm"].contiguous()
        self.w_o = W[p + "o"].contiguous()

    def state_specs(self) -> Dict[str, StateSpec]:
        return {self.name + ".S": StateSpec((self.H, self.V, self.K), torch.float32),
                self.name + ".conv": StateSpec((self.taps - 1, self.C), self.w_in.dtype)}

    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        lib, T, dev = S.lib(), ctx.T, h.device
        proj = linear(h, self.w_in)                                         # [T, n_in]
        a = linear(proj[:, self.o_a1:self.o_a1 + self.rank_a], self.w_a2)    # [T, H*K]
        gate = linear(proj[:, self.o_g1:self.o_g1 + self.rank_g], self.w_g2)  # [T, H*V]
        qkv = torch.empty((T, self.C), dtype=torch.float32, device=dev)
        S.check(lib.b2l_seq_conv_silu(_p(proj), self.n_in, _p(self.w_conv), None, _p(ctx.state[self.name + ".conv"]), _p(ctx.meta),
                                      _p(qkv), self.C, T, self.C, self.taps, ctx.act, ctx.stream), "b2l_seq_conv_silu")
        S.check(lib.b2l_seq_unit_norm(_p(qkv, self.o_q), self.C, T, self.G, self.K, self.unit_eps, self.K ** -0.5, ctx.stream), "b2l_seq_unit_norm")
        S.check(lib.b2l_seq_unit_norm(_p(qkv, self.o_k), self.C, T, self.G, self.K, self.unit_eps, 1.0, ctx.stream), "b2l_seq_unit_norm")
        g = torch.empty((T, self.H * self.K), dtype=torch.float32, device=dev)
        S.check(lib.b2l_seq_decay(_p(a), self.H * self.K, _p(self.dt_bias), _p(self.A_log), S.DECAY_EXP_SOFTPLUS, 0.0, _p(g), None, T,
                                  self.H, self.K, ctx.act, ctx.stream), "b2l_seq_decay")
        o = torch.empty((T, self.H * self.V), dtype=torch.float32, device=dev)
        _scan(ctx, q=_p(qkv, self.o_q), ldq=self.C, k=_p(qkv, self.o_k), ldk=self.C, v=_p(qkv, self.o_v), ldv=self.C,
              q_mult=1.0, decay=_p(g), ldd=self.H * self.K, per_channel=True, beta=_p(proj, self.o_b), ldb=self.n_in,
              state=ctx.state[self.name + ".S"], out=_p(o), ldo=self.H * self.V, heads=self.H, qk_heads=self.G, K=self.K, V=self.V)
        y = torch.empty((T, self.H * self.V), dtype=h.dtype, device=dev)
        S.check(lib.b2l_seq_group_norm_gate(_p(o), self.H * self.V, _p(self.w_norm), 1, _p(gate), self.H * self.V, S.ACT_SIGMOID, 0, self.eps,
                                            1.0, _p(y), self.H * self.V, T, self.H * self.V, self.V, ctx.act, ctx.stream), "b2l_seq_group_norm_gate")
        return linear(y, self.w_o)


class Mamba2Mixer:
    """State-space duality layer.  W_in h = [z | x | B | C | dt]; x | B | C pass a causal convolution (+ bias) and silu;
    dt = softplus(dt + dt_bias); per head S <- exp(-exp(A_log) dt) S + dt B x^T, y = S^T C + D x; then y silu(z),
    RMS norm in `norm_groups` equal parts, W_o.  State: S (f32, heads x vdim x state) and the convolution's inputs."""

    def __init__(self, name: str, W: Dict[str, torch.Tensor], p: str, *, heads: int, vdim: int, state: int, groups: int, norm_groups: int,
                 conv: int, eps: float) -> None:
        self.name, self.H, self.P, self.N, self.G, self.parts, self.taps, self.eps = name, heads, vdim, state, groups, norm_groups, conv, eps
        self.inner = heads * vdim
        self.C = self.inner + 2 * groups * state
        self.w_in = W[p + "in"].contiguous()
        self.n_in = self.w_in.shape[0]
        assert self.n_in == 2 * self.inner + 2 * groups * state + heads, "mamba2: the input projection does not fit z|x|B|C|dt"
        self.w_conv, self.b_conv = W[p + "conv"].contiguous(), W[p + "conv.b"].contiguous()
        self.dt_bias, self.A_log, self.D = W[p + "dt_bias"].contiguous(), W[p + "A_log"].contiguous(), W[p + "D"].contiguous()
        self.w_norm, self.w_o = W[p + "norm"].contiguous(), W[p + "o"].contiguous()

    def state_specs(self) -> Dict[str, StateSpec]:
        return {self.name + ".S": StateSpec((self.H, self.P, self.N), torch.float32),
                self.name + ".conv": StateSpec((self.taps - 1, self.C), self.w_in.dtype)}

    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        lib, T, dev = S.lib(), ctx.T, h.device
        u = linear(h, self.w_in)
        xbc = torch.empty((T, self.C), dtype=torch.float32, device=dev)
        S.check(lib.b2l_seq_conv_silu(_p(u, self.inner), self.n_in, _p(self.w_conv), _p(self.b_conv), _p(ctx.state[self.name + ".conv"]),
                                      _p(ctx.meta), _p(xbc), self.C, T, self.C, self.taps, ctx.act, ctx.stream), "b2l_seq_conv_silu")
        decay = torch.empty((T, self.H), dtype=torch.float32, device=dev)
        dt = torch.empty((T, self.H), dtype=torch.float32, device=dev)
        S.check(lib.b2l_seq_decay(_p(u, self.inner + self.C), self.n_in, _p(self.dt_bias), _p(self.A_log), S.DECAY_EXP_SOFTPLUS, 0.0, _p(decay),
                                  _p(dt), T, self.H, 1, ctx.act, ctx.stream), "b2l_seq_decay")
        y = torch.empty((T, self.inner), dtype=torch.float32, device=dev)
        GN = self.G * self.N
        _scan(ctx, q=_p(xbc, self.inner + GN), ldq=self.C, k=_p(xbc, self.inner), ldk=self.C, v=_p(xbc), ldv=self.C, q_mult=1.0,
              decay=_p(decay), ldd=self.H, per_channel=False, vscale=_p(dt), ldvs=self.H, skip=_p(self.D), state=ctx.state[self.name + ".S"],
              out=_p(y), ldo=self.inner, heads=self.H, qk_heads=self.G, K=self.N, V=self.P)
        out = torch.empty((T, self.inner), dtype=h.dtype, device=dev)
        S.check(lib.b2l_seq_group_norm_gate(_p(y), self.inner, _p(self.w_norm), 0, _p(u), self.n_in, S.ACT_SILU, 1, self.eps, 1.0, _p(out),
                                            self.inner, T, self.inner, self.inner // self.parts, ctx.act, ctx.stream), "b2l_seq_group_norm_gate")
        return linear(out, self.w_o)


class MinGRUMixer:
    """A gated recurrence whose gates read only the current token, channel by channel:

        z = sigmoid(W_z h + b_z);  u = W_x h + b_x;  c = u + 1/2 where u >= 0, sigmoid(u) where u < 0
        S_t = (1 - z) S_(t-1) + z c;   y = W_o (S_t * silu(W_g h))

    The three projections are one product; everything after it is f32.  State per sequence: S (f32, width), zero at the
    start.  Long portions run as chunks in parallel (the recurrence is linear in S)."""

    def __init__(self, name: str, W: Dict[str, torch.Tensor], p: str, *, width: int) -> None:
        self.name, self.width = name, int(width)
        parts = [W[p + "z"], W[p + "x"], W[p + "g"]]
        assert all(w.shape[0] == self.width for w in parts) and W[p + "o"].shape[1] == self.width, "minGRU: projections do not fit the width"
        self.w_in, (self.o_z, self.o_x, self.o_g) = stack_rows(parts)
        zero = torch.zeros_like(W[p + "z.b"])
        self.b_in, _ = stack_rows([W[p + "z.b"] if (p + "z.b") in W else zero, W[p + "x.b"] if (p + "x.b") in W else zero, zero])
        self.w_o = W[p + "o"].contiguous()

    def state_specs(self) -> Dict[str, StateSpec]:
        return {self.name + ".S": StateSpec((self.width,), torch.float32)}

    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        lib, T = S.lib(), ctx.T
        proj = F.linear(h, self.w_in, self.b_in)
        out = torch.empty((T, self.width), dtype=h.dtype, device=h.device)
        n_chunks = lib.b2l_seq_mingru_chunks(T)
        work = torch.empty((n_chunks, 2, self.width), dtype=torch.float32, device=h.device) if n_chunks > 1 else None
        S.check(lib.b2l_seq_mingru(_p(proj), proj.shape[1], self.o_z, self.o_x, self.o_g, _p(ctx.state[self.name + ".S"]), _p(ctx.meta), _p(out),
                                   self.width, _p(work), n_chunks, T, self.width, ctx.act, ctx.stream), "b2l_seq_mingru")
        return linear(out, self.w_o)


# ------------------------------------------------------------------------------------------------ rotation
def rope_frequencies(dims: int, base: float, scaling: Optional[dict]) -> Tuple[torch.Tensor, float]:
    """Per-pair rotation frequencies f_i = base^(-2i/dims), i < dims/2, optionally YaRN-scaled: with
    d(t) = dims ln(original / (2 pi t)) / (2 ln base), lo = max(floor(d(fast)), 0), hi = min(ceil(d(slow)), dims - 1) and
    ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1) the frequency becomes f_i / factor * ramp_i + f_i (1 - ramp_i),
    and cos / sin are multiplied by 0.1 ln(factor) + 1.  Returns (f32 frequencies on the CPU, multiplier)."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = float(base) ** (-2.0 * i / dims)
    mult = 1.0
    if scaling:
        factor, orig = float(scaling["factor"]), float(scaling["original"])

        def d(t: float) -> float:
            return dims * math.log(orig / (2 * math.pi * t)) / (2 * math.log(float(base)))

        lo = max(math.floor(d(float(scaling["fast"]))), 0)
        hi = min(math.ceil(d(float(scaling["slow"]))), dims - 1)
        ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0, 1)
        f = f / factor * ramp + f * (1 - ramp)
        mult = 0.1 * math.log(factor) + 1.0
    return f.to(torch.float32), mult


# ------------------------------------------------------------------------------------------------ attention
def local_attention(a: "S.AttnArgs", ctx: StepContext) -> None:
    """b2l_seq_block_attention with the work space its few-query form asks for."""
    lib = S.lib()
    n = lib.b2l_seq_block_attention_work_floats(C.byref(a))
    work = None
    if n:
        work = torch.empty((n,), dtype=torch.float32, device=ctx.meta.device)
        a.work, a.work_floats = _p(work), n
    S.check(lib.b2l_seq_block_attention(C.byref(a), ctx.stream), "b2l_seq_block_attention")


class BlockSinkAttention:
    """Softmax attention inside blocks of `block` positions (query p sees j <= p with j // block == p // block; block
    None: the whole sequence up to `max_positions`), weights exp(s_j) / (1 + sum exp(s_j)) when `sink`.  As a branch of
    a ParallelMixer it shares the input product: `parts()` lists its projection weights, `run()` consumes columns of
    the shared product and writes its gated heads into a slice of the shared read-out buffer."""

    def __init__(self, name: str, W: Dict[str, torch.Tensor], p: str, *, heads: int, kv_heads: int, dim: int, vdim: int, scale: float,
                 eps: float, softcap: Optional[float] = None, block: Optional[int] = None, rot: Optional[dict] = None, sink: bool = True,
                 max_positions: int = 0) -> None:
        self.name, self.H, self.G, self.K, self.V, self.scale, self.eps = name, heads, kv_heads, dim, vdim, float(scale), eps
        self.softcap = float(softcap) if softcap else 0.0
        self.block = int(block) if block else int(max_positions)
        if self.block <= 0:
            raise ValueError("attention without a block size needs max_positions")
        self.sink = bool(sink)
        self.w = [W[p + "q"], W[p + "k"], W[p + "v"], W[p + "g"]]
        self.q_norm, self.k_norm = W[p + "q.norm"].contiguous(), W[p + "k.norm"].contiguous()
        self.w_o = W[p + "o"]
        self.rot_dims, self.rot_mult, self.freq = 0, 1.0, None
        if rot:
            self.rot_dims = int(rot["dims"])
            f, self.rot_mult = rope_frequencies(self.rot_dims, float(rot["base"]), rot.get("scaling"))
            self.freq = f.to(self.w_o.device)

    def parts(self) -> List[torch.Tensor]:
        return self.w

    def out_width(self) -> int:
        return self.H * self.V

    def state_specs(self) -> Dict[str, StateSpec]:
        dt = self.w_o.dtype
        return {self.name + ".k": StateSpec((self.block, self.G, self.K), dt, zero_on_acquire=False),
                self.name + ".v": StateSpec((self.block, self.G, self.V), dt, zero_on_acquire=False)}

    def run(self, proj: torch.Tensor, offs: List[int], ctx: StepContext, out: torch.Tensor, out_off: int, out_mult: float) -> None:
        lib, T, dev, ld = S.lib(), ctx.T, proj.device, proj.shape[1]
        o_q, o_k, o_v, o_g = offs
        q = torch.empty((T, self.H * self.K), dtype=torch.float32, device=dev)
        kn = torch.empty((T, self.G * self.K), dtype=proj.dtype, device=dev)
        S.check(lib.b2l_seq_headnorm_rope(_p(proj, o_q), ld, _p(self.q_norm), self.eps, _p(self.freq), self.rot_dims, self.rot_mult, _p(ctx.meta),
                                          _p(q), 1, T, self.H, self.K, ctx.act, ctx.stream), "b2l_seq_headnorm_rope")
        S.check(lib.b2l_seq_headnorm_rope(_p(proj, o_k), ld, _p(self.k_norm), self.eps, _p(self.freq), self.rot_dims, self.rot_mult, _p(ctx.meta),
                                          _p(kn), 0, T, self.G, self.K, ctx.act, ctx.stream), "b2l_seq_headnorm_rope")
        a = S.AttnArgs(q=_p(q), k_new=_p(kn), v_new=_p(proj, o_v), ldv=ld, cache_k=_p(ctx.state[self.name + ".k"]),
                       cache_v=_p(ctx.state[self.name + ".v"]), meta=_p(ctx.meta), gate=_p(proj, o_g), ldg=ld, out=_p(out, out_off),
                       ldo=out.shape[1], scale=self.scale, softcap=self.softcap, out_mult=float(out_mult), has_sink=int(self.sink),
                       block=self.block, T=T, heads=self.H, kv_heads=self.G, K=self.K, V=self.V, act_dtype=ctx.act)
        local_attention(a, ctx)


class GatedLinearAttention:
    """S_t = diag(alpha_t) S_(t-1) + k_t v_t^T, o_t = S_t^T (q_t dim^-1/2), alpha = sigmoid(W_a2 W_a1 h + b)^(1/tau);
    read-out: per-head RMS norm (shared weight), times silu(W_g h).  A branch like BlockSinkAttention."""

    def __init__(self, name: str, W: Dict[str, torch.Tensor], p: str, *, heads: int, dim: int, vdim: int, tau: float, eps: float) -> None:
        self.name, self.H, self.K, self.V, self.tau, self.eps = name, heads, dim, vdim, float(tau), eps
        self.w = [W[p + "q"], W[p + "k"], W[p + "v"], W[p + "g"], W[p + "a1"]]
        self.rank = W[p + "a1"].shape[0]
        self.w_a2, self.b_a2 = W[p + "a2"].contiguous(), W[p + "a2.b"].contiguous()
        self.w_norm, self.w_o = W[p + "norm"].contiguous(), W[p + "o"]

    def parts(self) -> List[torch.Tensor]:
        return self.w

    def out_width(self) -> int:
        return self.H * self.V

    def state_specs(self) -> Dict[str, StateSpec]:
        return {self.name + ".S": StateSpec((self.H, self.V, self.K), torch.float32)}

    def run(self, proj: torch.Tensor, offs: List[int], ctx: StepContext, out: torch.Tensor, out_off: int, out_mult: float) -> None:
        lib, T, dev, ld = S.lib(), ctx.T, proj.device, proj.shape[1]
        o_q, o_k, o_v, o_g, o_a1 = offs
        a = linear(proj[:, o_a1:o_a1 + self.rank], self.w_a2)
        n = self.H * self.K
        alpha = torch.empty((T, n), dtype=torch.float32, device=dev)
        S.check(lib.b2l_seq_decay(_p(a), n, _p(self.b_a2), None, S.DECAY_SIGMOID_ROOT, self.tau, _p(alpha), None, T, self.H, self.K, ctx.act,
                                  ctx.stream), "b2l_seq_decay")
        o = torch.empty((T, self.H * self.V), dtype=torch.float32, device=dev)
        nq = o_g - o_q                                   # q | k | v are consecutive columns of the product
        qkv = torch.empty((T, nq), dtype=torch.float32, device=dev)
        S.check(lib.b2l_seq_cast_f32(_p(proj, o_q), ld, _p(qkv), nq, T, nq, ctx.act, ctx.stream), "b2l_seq_cast_f32")
        _scan(ctx, q=_p(qkv), ldq=nq, k=_p(qkv, o_k - o_q), ldk=nq, v=_p(qkv, o_v - o_q), ldv=nq, q_mult=self.K ** -0.5, decay=_p(alpha),
              ldd=n, per_channel=True, state=ctx.state[self.name + ".S"], out=_p(o), ldo=self.H * self.V, heads=self.H, qk_heads=self.H,
              K=self.K, V=self.V)
        S.check(lib.b2l_seq_group_norm_gate(_p(o), self.H * self.V, _p(self.w_norm), 1, _p(proj, o_g), ld, S.ACT_SILU, 0, self.eps, float(out_mult),
                                            _p(out, out_off), out.shape[1], T, self.H * self.V, self.V, ctx.act, ctx.stream),
                "b2l_seq_group_norm_gate")


class ParallelMixer:
    """y = sum_b scale_b * W_o,b branch_b(h): the branches' input projections are one product, and so are their
    output projections (the branches write scale_b * read-out into one buffer that meets [W_o,1 | W_o,2 | ...])."""

    def __init__(self, branches: List[Tuple[object, float]]) -> None:
        self.branches = [b for b, _ in branches]
        self.scales = [float(s) for _, s in branches]
        parts, self.counts = [], []
        for b in self.branches:
            parts += b.parts()
            self.counts.append(len(b.parts()))
        self.w_in, self.offs = stack_rows(parts)
        self.widths = [b.out_width() for b in self.branches]
        self.w_o = torch.cat([b.w_o for b in self.branches], dim=1).contiguous()

    def state_specs(self) -> Dict[str, StateSpec]:
        out: Dict[str, StateSpec] = {}
        for b in self.branches:
            out.update(b.state_specs())
        return out

    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        proj = linear(h, self.w_in)
        out = torch.empty((ctx.T, sum(self.widths)), dtype=h.dtype, device=h.device)
        at, col = 0, 0
        for b, n, s, w in zip(self.branches, self.counts, self.scales, self.widths):
            b.run(proj, self.offs[at:at + n], ctx, out, col, s)
            at += n
            col += w
        return linear(out, self.w_o)


class SlidingWindowAttention:
    """Causal softmax attention over the last `window` positions (the query's own and the window - 1 before it).

        q, k, v = W_q h, W_k h, W_v h (one stacked product, with the gate);  q, k: RMS norm, over the whole projection
        with a weight of its size (`norm_over` = "row") or per head with one weight of `dim` entries ("head"), then
        rotation of the first rot.dims entries of every head (entry i with entry i + dims/2)
        v <- (1 - lambda) v + lambda v_first in every layer with `v_mix` but the first of them, whose v is v_first
        weights = softmax(q . k * scale) over the visible keys (ordinary softmax, no sink); query head h reads
        key / value head h // (heads / kv_heads)
        y = W_o (concat_h(sum_j weight_j v_j) * sigmoid(W_g h))            a gate per output channel

    State per sequence: a ring of `window` positions of rotated keys and (mixed) values, entry position % window.  The
    first value-mixing layer of a step leaves its values in `ctx.shared` for the later ones."""

    def __init__(self, name: str, W: Dict[str, torch.Tensor], p: str, *, heads: int, kv_heads: int, dim: int, vdim: int, scale: float, window: int,
                 eps: float, rot: Optional[dict] = None, v_mix: bool = False, norm_over: str = "row", mix_key: str = "v_first") -> None:
        self.name, self.H, self.G, self.K, self.V, self.scale, self.eps = name, int(heads), int(kv_heads), int(dim), int(vdim), float(scale), eps
        self.window = int(window)
        if self.window < 1 or self.H % self.G:
            raise ValueError("sliding-window attention: the window must hold at least the query's own position, heads a multiple of kv_heads")
        if norm_over not in ("row", "head"):
            raise ValueError(f"sliding-window attention: norm over {norm_over!r}")
        self.whole_row, self.v_mix, self.mix_key = int(norm_over == "row"), bool(v_mix), mix_key
        assert W[p + "q"].shape[0] == heads * dim and W[p + "k"].shape[0] == kv_heads * dim and W[p + "v"].shape[0] == kv_heads * vdim, \
            "sliding-window attention: projections do not fit the head sizes"
        assert W[p + "g"].shape[0] == heads * vdim and W[p + "o"].shape[1] == heads * vdim, "sliding-window attention: gate / output do not fit"
        self.w_in, (self.o_q, self.o_k, self.o_v, self.o_g) = stack_rows([W[p + "q"], W[p + "k"], W[p + "v"], W[p + "g"]])
        self.q_norm = W[p + "q.norm"].contiguous() if (p + "q.norm") in W else None
        self.k_norm = W[p + "k.norm"].contiguous() if (p + "k.norm") in W else None
        self.lam = W[p + "vmix"].reshape(1).contiguous() if self.v_mix else None
        self.w_o = W[p + "o"].contiguous()
        self.rot_dims, self.rot_mult, self.freq = 0, 1.0, None
        if rot and int(rot.get("dims", 0)):
            self.rot_dims = int(rot["dims"])
            f, self.rot_mult = rope_frequencies(self.rot_dims, float(rot["base"]), rot.get("scaling"))
            self.freq = f.to(self.w_o.device)

    def state_specs(self) -> Dict[str, StateSpec]:
        dt = self.w_o.dtype
        return {self.name + ".k": StateSpec((self.window, self.G, self.K), dt, zero_on_acquire=False),
                self.name + ".v": StateSpec((self.window, self.G, self.V), dt, zero_on_acquire=False)}

    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        lib, T, dev = S.lib(), ctx.T, h.device
        proj = linear(h, self.w_in)
        ld = proj.shape[1]
        q = torch.empty((T, self.H * self.K), dtype=torch.float32, device=dev)
        kn = torch.empty((T, self.G * self.K), dtype=proj.dtype, device=dev)
        first = ctx.shared.get(self.mix_key) if self.v_mix else None          # (tensor, column, leading dimension, width) of the first layer's values
        if first is not None and first[3] != self.G * self.V:
            raise ValueError(f"{self.name}: values of {self.G * self.V} entries cannot be mixed with the first layer's {first[3]}")
        v, v_off, ldv = proj, self.o_v, ld
        vm = None
        if first is not None:
            vm = torch.empty((T, self.G * self.V), dtype=proj.dtype, device=dev)
            v, v_off, ldv = vm, 0, self.G * self.V
        elif self.v_mix:
            ctx.shared[self.mix_key] = (proj, self.o_v, ld, self.G * self.V)
        a = S.QkvPrepArgs(proj=_p(proj), ld=ld, q_off=self.o_q, k_off=self.o_k, v_off=self.o_v, q_norm=_p(self.q_norm), k_norm=_p(self.k_norm),
                          whole_row=self.whole_row, eps=self.eps, freq=_p(self.freq), rot_dims=self.rot_dims, rot_mult=self.rot_mult,
                          meta=_p(ctx.meta), q_out=_p(q), k_out=_p(kn), v_first=_p(first[0], first[1]) if first is not None else None,
                          ldvf=first[2] if first is not None else 0, lambda_=_p(self.lam) if first is not None else None, v_out=_p(vm), T=T,
                          heads=self.H, kv_heads=self.G, K=self.K, V=self.V, act_dtype=ctx.act)
        S.check(lib.b2l_seq_qkv_prep(C.byref(a), ctx.stream), "b2l_seq_qkv_prep")
        att = torch.empty((T, self.H * self.V), dtype=h.dtype, device=dev)
        b = S.AttnArgs(q=_p(q), k_new=_p(kn), v_new=_p(v, v_off), ldv=ldv, cache_k=_p(ctx.state[self.name + ".k"]),
                       cache_v=_p(ctx.state[self.name + ".v"]), meta=_p(ctx.meta), gate=_p(proj, self.o_g), ldg=ld, out=_p(att), ldo=self.H * self.V,
                       scale=self.scale, softcap=0.0, out_mult=1.0, has_sink=0, block=self.window, T=T, heads=self.H, kv_heads=self.G, K=self.K,
                       V=self.V, act_dtype=ctx.act, window=self.window, gate_per_channel=1)
        local_attention(b, ctx)
        return linear(att, self.w_o)


class DifferentialAttention:
    """Causal softmax attention with two score maps per head over the same values.

        q = conv(W_q h + b_q) [heads x 2 x dim], k = conv(W_k h + b_k) [kv_heads x 2 x dim], v = conv(W_v h + b_v) [kv_heads x vdim]
        conv: a causal convolution of `conv` taps over time on every channel (no bias, no activation)
        q, k: the first rot.dims entries of every map of every head turn by position, pairs (2i, 2i+1) when `interleaved`
        a_m = softmax_j(q_m . k_m,j * scale) v_j over all j <= i, for the maps m = 0, 1;  query head h reads key/value head
        h // (heads / kv_heads)
        o = a_0 - lambda a_1,  lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff  (one number per layer)
        y = W_o concat_h(o / sqrt(mean(o^2) + eps) * (1 - diff))

    The three projections are one product.  State per sequence: the last conv - 1 projected rows, and every position's
    rotated keys and convolved values (`max_positions` of them).  With `kv_from` (an earlier DifferentialAttention with the
    same head counts and rotation) the layer has only queries of its own: it attends over that layer's keys and values, read
    from that layer's cache and, for the portion's own tokens, from what that layer left in `ctx.shared` in this step."""

    def __init__(self, name: str, W: Dict[str, torch.Tensor], p: str, *, heads: int, kv_heads: int, dim: int, vdim: int, scale: float, diff: float,
                 eps: float, conv: int = 0, rot: Optional[dict] = None, max_positions: int = 0, kv_from: Optional["DifferentialAttention"] = None,
                 interleaved: bool = True) -> None:
        if max_positions <= 0:
            raise ValueError("differential attention caches every position: it needs max_positions")
        self.name, self.H, self.G, self.K, self.V = name, int(heads), int(kv_heads), int(dim), int(vdim)
        self.scale, self.diff, self.eps, self.max_positions, self.interleaved = float(scale), float(diff), eps, int(max_positions), bool(interleaved)
        if self.H % self.G or self.K % 2:
            raise ValueError("differential attention: heads must be a multiple of kv_heads, the map size even")
        self.src = kv_from
        if kv_from is not None and (kv_from.src is not None or (kv_from.H, kv_from.G, kv_from.K, kv_from.V) != (self.H, self.G, self.K, self.V)):
            raise ValueError(f"{name}: keys and values must come from a layer with projections of its own and the same head sizes")
        names = ["q"] if kv_from is not None else ["q", "k", "v"]
        rows = {"q": self.H * 2 * self.K, "k": self.G * 2 * self.K, "v": self.G * self.V}
        for n in names:
            assert W[p + n].shape[0] == rows[n], f"differential attention: projection {n} does not fit the head sizes"
        assert W[p + "o"].shape[1] == self.H * self.V, "differential attention: output projection does not fit"
        self.w_in, offs = stack_rows([W[p + n] for n in names])
        self.b_in, _ = stack_rows([W[p + n + ".b"] if (p + n + ".b") in W else torch.zeros_like(W[p + n][:, 0]) for n in names])
        self.o_q, self.o_k, self.o_v = offs[0], (offs[1] if len(offs) > 1 else -1), (offs[2] if len(offs) > 2 else -1)
        self.C = self.w_in.shape[0]
        self.taps = int(conv) if conv else 1
        if conv:
            self.w_conv, _ = stack_rows([W[p + n + ".conv"] for n in names])
            assert self.w_conv.shape == (self.C, self.taps), "differential attention: convolution weights do not fit"
        else:                                   # no convolution: one tap of weight one
            self.w_conv = torch.ones((self.C, 1), dtype=self.w_in.dtype, device=self.w_in.device)
        lam = [float((W[p + f"lq{m}"].double() * W[p + f"lk{m}"].double()).sum()) for m in (1, 2)]
        self.lam = math.exp(lam[0]) - math.exp(lam[1]) + self.diff
        self.w_o = W[p + "o"].contiguous()
        self.rot_dims, self.rot_mult, self.freq = 0, 1.0, None
        if rot and int(rot.get("dims", 0)):
            self.rot_dims = int(rot["dims"])
            f, self.rot_mult = rope_frequencies(self.rot_dims, float(rot["base"]), rot.get("scaling"))
            self.freq = f.to(self.w_o.device)

    def state_specs(self) -> Dict[str, StateSpec]:
        dt = self.w_o.dtype
        out = {self.name + ".conv": StateSpec((self.taps - 1, self.C), dt)} if self.taps > 1 else {}
        if self.src is None:
            out[self.name + ".k"] = StateSpec((self.max_positions, self.G * 2 * self.K), dt, zero_on_acquire=False)
            out[self.name + ".v"] = StateSpec((self.max_positions, self.G * self.V), dt, zero_on_acquire=False)
        return out

    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        lib, T, dev, H, G, K, V = S.lib(), ctx.T, h.device, self.H, self.G, self.K, self.V
        proj = F.linear(h, self.w_in, self.b_in)
        q = torch.empty((T, H * 2 * K), dtype=torch.float32, device=dev)
        own = self.src is None
        kn = torch.empty((T, G * 2 * K), dtype=proj.dtype, device=dev) if own else None
        vn = torch.empty((T, G * V), dtype=proj.dtype, device=dev) if own else None
        a = S.ConvRopeArgs(proj=_p(proj), ld=proj.shape[1], c_off=0, C=self.C, taps=self.taps, w=_p(self.w_conv),
                           state=_p(ctx.state[self.name + ".conv"]) if self.taps > 1 else None, meta=_p(ctx.meta), q_off=self.o_q, q_heads=2 * H,
                           k_off=self.o_k, k_heads=2 * G, K=K, v_off=self.o_v, n_v=G * V, freq=_p(self.freq), rot_dims=self.rot_dims,
                           interleaved=int(self.interleaved), rot_mult=self.rot_mult, q_out=_p(q), k_out=_p(kn), v_out=_p(vn), T=T, act_dtype=ctx.act)
        S.check(lib.b2l_seq_conv_rope(C.byref(a), ctx.stream), "b2l_seq_conv_rope")
        if own:
            ctx.shared["kv:" + self.name] = (kn, vn)
            holder = self.name
        else:
            if ("kv:" + self.src.name) not in ctx.shared:
                raise RuntimeError(f"{self.name}: layer {self.src.name} has not run in this step")
            kn, vn = ctx.shared["kv:" + self.src.name]
            holder = self.src.name
        maps = torch.empty((T, H * 2 * V), dtype=torch.float32, device=dev)      # scratch of the forms that do not merge the maps themselves
        y = torch.empty((T, H * V), dtype=h.dtype, device=dev)
        b = S.AttnArgs(q=_p(q), k_new=_p(kn), v_new=_p(vn), ldv=G * V, cache_k=_p(ctx.state[holder + ".k"]), cache_v=_p(ctx.state[holder + ".v"]),
                       meta=_p(ctx.meta), gate=None, ldg=0, out=_p(maps), ldo=H * 2 * V, scale=self.scale, softcap=0.0, out_mult=1.0, has_sink=0,
                       block=self.max_positions, T=T, heads=2 * H, kv_heads=G, K=K, V=V, act_dtype=ctx.act, window=0, gate_per_channel=0, maps=2,
                       out_f32=1, no_append=int(not own), diff_out=_p(y), ldd=H * V, diff_lambda=self.lam, diff_eps=self.eps,
                       diff_mult=1.0 - self.diff)
        local_attention(b, ctx)                 # attention of both maps and the differential read-out
        return linear(y, self.w_o)


# ------------------------------------------------------------------------------------------------ residual streams
def norm_rows(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], kind: str, eps: float, ctx: StepContext,
              rows: Optional[torch.Tensor] = None, n_rows: Optional[int] = None) -> torch.Tensor:
    """RMS norm ("rms") or layer norm with a bias ("layer") of rows of the f32 stream x [T, width] -> act [n_rows, width]."""
    n = x.shape[0] if n_rows is None else n_rows
    out = torch.empty((n, x.shape[1]), dtype=ctx.dtype, device=x.device)
    S.check(S.lib().b2l_seq_norm(_p(x), _p(w), _p(b), DepthAverage.NORMS[kind], eps, _p(out), _p(rows), n, x.shape[1], ctx.act, ctx.stream), "b2l_seq_norm")
    return out


class DepthAverage:
    """The residual stream of layers that read a learned average over everything before them.  With X_0 the embedding
    output and X_(i+1) = x_i + (what layer i's sublayers add to their input x_i), the next layer's input is
    x_(i+1) = sum_(j <= i+1) avg_i[j] X_j (avg_i None: X_(i+1) itself, the ordinary residual stream).  `history` holds the
    X_j of one portion ([layers + 1, T, width] f32); `step` writes X_(i+1), forms x_(i+1) and the next norm in one launch."""

    NORMS = {"rms": S.NORM_RMS, "layer": S.NORM_LAYER}

    def __init__(self, weights: List[Optional[torch.Tensor]]) -> None:
        self.avg = []
        for i, w in enumerate(weights):
            if w is not None and w.numel() != i + 2:
                raise ValueError(f"layer {i}: {w.numel()} depth weights, {i + 2} earlier results")
            self.avg.append(w.to(torch.float32).contiguous() if w is not None else None)

    def history(self, ctx: StepContext, width: int, device) -> torch.Tensor:
        return torch.empty((len(self.avg) + 1, ctx.T, width), dtype=torch.float32, device=device)

    def step(self, i: int, hist: torch.Tensor, x_in: torch.Tensor, x_out: torch.Tensor, y1: torch.Tensor, y2: Optional[torch.Tensor], ctx: StepContext, *,
             norm: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None, kind: str = "layer", eps: float = 0.0) -> Optional[torch.Tensor]:
        """Layer i's results y1 (+ y2) on its input x_in -> the next input in x_out (may be x_in), and its norm (act) when `norm` is given."""
        T, D = x_in.shape
        h = torch.empty((T, D), dtype=ctx.dtype, device=x_in.device) if norm is not None else None
        S.check(S.lib().b2l_seq_depth_step(_p(y1), _p(y2), _p(x_in), _p(hist), i + 2, _p(self.avg[i]), _p(x_out), _p(norm), _p(bias), self.NORMS[kind],
                                           eps, _p(h), T, D, ctx.act, ctx.stream), "b2l_seq_depth_step")
        return h


class PairHashEmbedding:
    """x = embed[token] * scale + pair[(previous token * mul_prev + token * mul_cur) mod buckets], the first token of a
    sequence reading the pair table's last row (number `buckets`); written into `streams` equal residual streams
    [T, streams, width] (f32).  `pair` None: the token embedding alone.  State per sequence: its last token."""

    def __init__(self, name: str, embed: torch.Tensor, pair: Optional[torch.Tensor], *, buckets: int = 0, mul_prev: int = 0, mul_cur: int = 0,
                 scale: float = 1.0, streams: int = 1) -> None:
        self.name, self.embed, self.pair = name, embed.contiguous(), pair.contiguous() if pair is not None else None
        self.vocab, self.width = self.embed.shape
        self.buckets, self.mul_prev, self.mul_cur, self.scale, self.streams = int(buckets), int(mul_prev), int(mul_cur), float(scale), int(streams)
        if self.pair is not None and tuple(self.pair.shape) != (self.buckets + 1, self.width):
            raise ValueError(f"pair embedding is {tuple(self.pair.shape)}, {self.buckets} buckets and a first-token row need {(self.buckets + 1, self.width)}")

    def state_specs(self) -> Dict[str, StateSpec]:
        return {self.name + ".prev": StateSpec((1,), torch.int32)} if self.pair is not None else {}

    def forward(self, tokens: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        x = torch.empty((ctx.T, self.streams, self.width), dtype=torch.float32, device=self.embed.device)
        prev = ctx.state[self.name + ".prev"] if self.pair is not None else None
        S.check(S.lib().b2l_seq_embed_pair(_p(tokens), int(tokens.dtype == torch.int64), _p(self.embed), _p(self.pair), self.scale, _p(prev),
                                           _p(ctx.meta), self.mul_prev, self.mul_cur, self.buckets, _p(x), ctx.T, self.width, self.vocab,
                                           self.streams, ctx.act, ctx.stream), "b2l_seq_embed_pair")
        return x


class HyperConnection:
    """One sublayer over `streams` residual streams: it reads u = sum_s read[s] x_s, and its result y is written as
    x_t <- sum_s mix[s, t] x_s + write[t] y for all streams at once (mix indexed [from, to]).  The weights are f32 on
    the device; `plain(streams)` is the ordinary residual step (one stream, all weights 1).  `step()` fuses the write
    of one sublayer with the read and the RMS norm of the next."""

    def __init__(self, read: torch.Tensor, mix: torch.Tensor, write: torch.Tensor) -> None:
        self.streams = int(read.numel())
        if tuple(mix.shape) != (self.streams, self.streams) or write.numel() != self.streams:
            raise ValueError(f"hyper-connection: read {tuple(read.shape)}, mix {tuple(mix.shape)}, write {tuple(write.shape)} do not fit")
        self.read, self.mix, self.write = (t.to(torch.float32).contiguous() for t in (read, mix, write))

    @classmethod
    def plain(cls, device, streams: int = 1) -> "HyperConnection":
        if streams != 1:
            raise ValueError("a plain residual step has one stream")
        one = torch.ones(1, dtype=torch.float32, device=device)
        return cls(one, one.reshape(1, 1), one)

    @staticmethod
    def step(x: torch.Tensor, ctx: StepContext, *, y: Optional[torch.Tensor] = None, wrote: Optional["HyperConnection"] = None,
             reads: Optional["HyperConnection"] = None, read_weights: Optional[torch.Tensor] = None, norm: Optional[torch.Tensor] = None,
             eps: float = 0.0, rows: Optional[torch.Tensor] = None, n_rows: Optional[int] = None) -> Optional[torch.Tensor]:
        """x [T, streams, width] f32, updated in place with sublayer `wrote`'s result y; then, with `norm`, the input of
        the next sublayer `reads` (or any read weights, e.g. ones for the sum of the streams): act [n_rows, width]."""
        T, n_s, D = x.shape
        n = T if n_rows is None else n_rows
        rw = reads.read if reads is not None else read_weights
        h = torch.empty((n, D), dtype=ctx.dtype, device=x.device) if norm is not None else None
        S.check(S.lib().b2l_seq_hc_step(_p(y), _p(x), _p(wrote.mix) if y is not None else None, _p(wrote.write) if y is not None else None,
                                        _p(rw) if norm is not None else None, _p(norm), _p(h), eps, _p(rows), n, D, n_s, ctx.act, ctx.stream),
                "b2l_seq_hc_step")
        return h


# ------------------------------------------------------------------------------------------------ latent attention
class LatentAttention:
    """Causal softmax attention over a cached latent.

        c_q = rmsnorm(W_dq h) w_q;  q = W_uq c_q, per head [dim unrotated | rot_dim rotated]
        [c' | k_r] = W_dkv h;  c = rmsnorm(c') w_kv (kv_rank);  k_r rotated by position, shared by all heads
        key_h = [W_uk,h c | k_r],  value_h = W_uv,h c,  score = q . key * scale
        weights exp(s_j) / (exp(sink_h) + sum_j exp(s_j)),  y = W_o concat_h(sum_j weight_j value_j)

    over every earlier position, or with `window` over the query's own position and the window - 1 before it; without a
    `sink` tensor the softmax is the ordinary one.  A YaRN `scaling` of the rotation stretches the slow frequencies and
    multiplies cos and sin of q_r and k_r; `scale` is taken as given.

    Only [c | k_r] is cached per position.  Single tokens and short portions attend in the latent space: the query is
    multiplied by W_uk once (q' = W_uk,h^T q_h), scores are q' . c + q_r . k_r, the weighted sum of latents is mapped
    through W_uv afterwards; every head reads the same cached row, once.  Portions of `expand_from` tokens or more
    expand [value_h | key_h] of every cached position with one product and attend per head, which costs several times
    fewer operations per (query, key) pair.  Both forms run the same kernel.  `rot`: {"base", "dims"} on the first
    `dims` entries of the rotated part, pairs (2i, 2i+1) when `interleaved`."""

    expand_from: int = 64                 # portions at least this long take the expanded form
    expand_limit: int = 1 << 31           # ... unless the expansion would have more elements than this

    def __init__(self, name: str, W: Dict[str, torch.Tensor], p: str, *, heads: int, dim: int, rot_dim: int, vdim: int, q_rank: int,
                 kv_rank: int, scale: float, eps: float, rot: Optional[dict], max_positions: int, interleaved: bool = True,
                 window: Optional[int] = None) -> None:
        if max_positions <= 0:
            raise ValueError("latent attention caches every position: it needs max_positions")
        self.window = int(window) if window else 0
        if self.window < 0:
            raise ValueError("latent attention: negative window")
        self.name, self.H, self.dn, self.dr, self.dv, self.rq, self.rk = name, heads, dim, rot_dim, vdim, q_rank, kv_rank
        self.scale, self.eps, self.max_positions, self.interleaved = float(scale), eps, int(max_positions), bool(interleaved)
        self.w_in, (self.o_q, self.o_kv) = stack_rows([W[p + "dq"], W[p + "dkv"]])
        assert W[p + "dq"].shape[0] == q_rank and W[p + "dkv"].shape[0] == kv_rank + rot_dim, "latent attention: down-projections do not fit"
        self.q_norm, self.kv_norm = W[p + "dq.norm"].contiguous(), W[p + "dkv.norm"].contiguous()
        self.w_uq = W[p + "uq"].contiguous()
        assert self.w_uq.shape == (heads * (dim + rot_dim), q_rank), "latent attention: query up-projection does not fit"
        uk, uv = W[p + "uk"].reshape(heads, dim, kv_rank), W[p + "uv"].reshape(heads, vdim, kv_rank)
        self.w_uk = uk.contiguous()                                                            # q' = q_h W_uk,h
        self.w_uv_t = uv.transpose(1, 2).contiguous()                                          # value = o' W_uv,h^T
        self.w_expand = torch.cat([uv, uk], dim=1).reshape(heads * (vdim + dim), kv_rank).contiguous()   # per head [value | key] rows
        self.sink = W[p + "sink"].to(torch.float32).contiguous() if (p + "sink") in W else None
        self.w_o = W[p + "o"].contiguous()
        self.rot_dims, self.rot_mult, self.freq = 0, 1.0, None
        if rot and rot_dim:
            self.rot_dims = int(rot["dims"])
            if self.rot_dims > rot_dim:
                raise ValueError(f"latent attention: {self.rot_dims} rotated entries in a part of {rot_dim}")
            f, self.rot_mult = rope_frequencies(self.rot_dims, float(rot["base"]), rot.get("scaling"))
            self.freq = f.to(self.w_o.device)

    def state_specs(self) -> Dict[str, StateSpec]:
        return {self.name + ".kv": StateSpec((self.max_positions, self.rk + self.dr), self.w_o.dtype, zero_on_acquire=False)}

    def _splits(self, ctx: StepContext, hpg: int) -> int:
        """Key splits: fill the machine when there are few rows; never a function of the position inside a captured step."""
        T = ctx.T
        n_keys = self.max_positions if ctx.pos_hint is None else min(self.max_positions, ctx.pos_hint + T)
        if self.window:
            n_keys = min(n_keys, self.window + 4 * S.lib().b2l_seq_latent_attention_warps(T, hpg) // hpg)     # what one CTA's rows see
        warps = S.lib().b2l_seq_latent_attention_warps(T, hpg)
        ctas = -(-T * hpg // (4 * warps)) * (self.H // hpg)
        if ctas >= 444:                       # a full wave of three CTAs per SM
            return 1
        return max(1, min(-(-444 // ctas), -(-n_keys // 32)))

    def _attend(self, ctx: StepContext, out: torch.Tensor, vdim: int, splits: int, **kw) -> None:
        work = torch.empty((splits, ctx.T * self.H, vdim + 2), dtype=torch.float32, device=out.device) if splits > 1 else None
        a = S.LatentAttnArgs(sink=_p(self.sink), meta=_p(ctx.meta), out=_p(out), ldo=self.H * vdim, work=_p(work), scale=self.scale, T=ctx.T,
                             heads=self.H, vdim=vdim, splits=splits, act_dtype=ctx.act, window=self.window, **kw)
        S.check(S.lib().b2l_seq_latent_attention(C.byref(a), ctx.stream), "b2l_seq_latent_attention")

    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        lib, T, dev, H = S.lib(), ctx.T, h.device, self.H
        proj = linear_f32(h, self.w_in)
        cq = torch.empty((T, self.rq), dtype=h.dtype, device=dev)
        cache = ctx.state[self.name + ".kv"]
        Kd = self.rk + self.dr
        S.check(lib.b2l_seq_latent_prep(_p(proj), proj.shape[1], self.o_q, self.rq, _p(self.q_norm), _p(cq), self.o_kv, self.rk, _p(self.kv_norm),
                                        self.dr, _p(self.freq), self.rot_dims, int(self.interleaved), self.rot_mult, self.eps, _p(ctx.meta), _p(cache),
                                        self.max_positions, T, ctx.act, ctx.stream), "b2l_seq_latent_prep")
        dq, f32 = self.dn + self.dr, h.dtype == torch.float32
        q = linear(cq, self.w_uq)                                                   # [T, H * (dim + rot_dim)]
        shared_b = dict(key_b=_p(cache, self.rk), ldkb=Kd, slot_stride_b=self.max_positions * Kd, n_b=self.dr)
        n_pos = None if ctx.pos_hint is None or ctx.slot_hint is None else ctx.pos_hint + T
        if n_pos is not None and T >= self.expand_from and n_pos * H * (self.dv + self.dn) <= self.expand_limit:
            # expanded form: [value_h | key_h] of positions 0 .. n_pos-1 from the cached latents, one product
            q32 = torch.empty((T, H * dq), dtype=torch.float32, device=dev)
            S.check(lib.b2l_seq_rope(_p(q), H * dq, int(f32), _p(self.freq), self.rot_dims, int(self.interleaved), self.dn, 1.0, self.rot_mult, _p(ctx.meta),
                                     _p(q32), H * dq, 1, T, H, dq, dq, dq, ctx.act, ctx.stream), "b2l_seq_rope")
            lo = max(0, ctx.pos_hint - self.window + 1) if self.window else 0       # the first position any query of the portion sees
            kv = linear(cache[ctx.slot_hint, lo:n_pos, :self.rk], self.w_expand)     # [n_pos - lo, H * (vdim + dim)]: row j - lo is position j
            att = torch.empty((T, H * self.dv), dtype=h.dtype, device=dev)
            self._attend(ctx, att, self.dv, self._splits(ctx, 1), q_a=_p(q32), ldqa_t=H * dq, ldqa_h=dq, q_b=_p(q32, self.dn), ldqb_t=H * dq,
                         ldqb_h=dq, key_a=_p(kv, -lo * H * (self.dv + self.dn)), ldka=H * (self.dv + self.dn), hska=self.dv + self.dn, slot_stride_a=0, n_a=self.dv + self.dn,
                         score_off=self.dv, heads_per_group=1, **shared_b)
            return linear(att, self.w_o)
        # latent form
        qn = q.view(T, H, dq)[:, :, :self.dn].transpose(0, 1)                        # [H, T, dim]
        q_lat = torch.bmm(qn, self.w_uk) if f32 else torch.bmm(qn, self.w_uk, out_dtype=torch.float32)     # [H, T, rank] f32
        q_rot = torch.empty((T, H, max(self.dr, 1)), dtype=torch.float32, device=dev)
        if self.dr:
            S.check(lib.b2l_seq_rope(_p(q, self.dn), H * dq, int(f32), _p(self.freq), self.rot_dims, int(self.interleaved), 0, 1.0, self.rot_mult, _p(ctx.meta),
                                     _p(q_rot), H * self.dr, 1, T, H, self.dr, dq, self.dr, ctx.act, ctx.stream), "b2l_seq_rope")
        o_lat = torch.empty((T, H * self.rk), dtype=h.dtype, device=dev)
        self._attend(ctx, o_lat, self.rk, self._splits(ctx, H), q_a=_p(q_lat), ldqa_t=self.rk, ldqa_h=T * self.rk, q_b=_p(q_rot),
                     ldqb_t=H * max(self.dr, 1), ldqb_h=max(self.dr, 1), key_a=_p(cache), ldka=Kd, hska=0, slot_stride_a=self.max_positions * Kd,
                     n_a=self.rk, score_off=0, heads_per_group=H, **shared_b)
        v = torch.bmm(o_lat.view(T, H, self.rk).transpose(0, 1), self.w_uv_t)        # [H, T, vdim]
        return linear(v.transpose(0, 1).reshape(T, H * self.dv), self.w_o)


# ------------------------------------------------------------------------------------------------ retention
class RetentionMixer:
    """Linear attention with one fixed decay per head, no softmax and no denominator:

        q, k rotated by position (first rot.dims entries of each head; entry i with entry i + dims/2), k times dim^-1/2
        S_t = decay_h S_(t-1) + k_t v_t^T;  o_t = S_t^T q_t
        y = W_o (concat_h(o_t,h / rms(o_t,h)) * silu(W_g h))

    State per sequence: S (f32, heads x vdim x dim), zero at the start."""

    def __init__(self, name: str, W: Dict[str, torch.Tensor], p: str, *, heads: int, dim: int, vdim: int, decay: List[float], eps: float,
                 rot: Optional[dict], interleaved: bool = False) -> None:
        self.name, self.H, self.K, self.V, self.eps, self.interleaved = name, heads, dim, vdim, eps, bool(interleaved)
        if len(decay) != heads:
            raise ValueError(f"retention: {len(decay)} decays for {heads} heads")
        self.w_in, (self.o_q, self.o_k, self.o_v, self.o_g) = stack_rows([W[p + "q"], W[p + "k"], W[p + "v"], W[p + "g"]])
        assert W[p + "q"].shape[0] == heads * dim and W[p + "v"].shape[0] == heads * vdim and W[p + "g"].shape[0] == heads * vdim
        self.w_o = W[p + "o"].contiguous()
        dev = self.w_o.device
        self.decay = torch.tensor([float(d) for d in decay], dtype=torch.float32, device=dev)
        self.ones = torch.ones(vdim, dtype=self.w_o.dtype, device=dev)
        self.rot_dims, self.freq = 0, None
        if rot:
            self.rot_dims = int(rot["dims"])
            f, _ = rope_frequencies(self.rot_dims, float(rot["base"]), rot.get("scaling"))
            self.freq = f.to(dev)

    def state_specs(self) -> Dict[str, StateSpec]:
        return {self.name + ".S": StateSpec((self.H, self.V, self.K), torch.float32)}

    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        lib, T, dev, H, K, V = S.lib(), ctx.T, h.device, self.H, self.K, self.V
        proj = linear(h, self.w_in)
        ld, f32in = proj.shape[1], int(proj.dtype == torch.float32)
        qkv = torch.empty((T, 2 * H * K + H * V), dtype=torch.float32, device=dev)
        n = qkv.shape[1]
        for off_in, off_out, mult in ((self.o_q, 0, 1.0), (self.o_k, H * K, K ** -0.5)):
            S.check(lib.b2l_seq_rope(_p(proj, off_in), ld, f32in, _p(self.freq), self.rot_dims, int(self.interleaved), 0, mult, 1.0, _p(ctx.meta),
                                     _p(qkv, off_out), n, 1, T, H, K, K, K, ctx.act, ctx.stream), "b2l_seq_rope")
        S.check(lib.b2l_seq_cast_f32(_p(proj, self.o_v), ld, _p(qkv, 2 * H * K), n, T, H * V, ctx.act, ctx.stream), "b2l_seq_cast_f32")
        o = torch.empty((T, H * V), dtype=torch.float32, device=dev)
        _scan(ctx, q=_p(qkv), ldq=n, k=_p(qkv, H * K), ldk=n, v=_p(qkv, 2 * H * K), ldv=n, q_mult=1.0, decay=_p(self.decay), ldd=0,
              per_channel=False, state=ctx.state[self.name + ".S"], out=_p(o), ldo=H * V, heads=H, qk_heads=H, K=K, V=V)
        y = torch.empty((T, H * V), dtype=h.dtype, device=dev)
        S.check(lib.b2l_seq_group_norm_gate(_p(o), H * V, _p(self.ones), 1, _p(proj, self.o_g), ld, S.ACT_SILU, 0, self.eps, 1.0, _p(y), H * V, T,
                                            H * V, V, ctx.act, ctx.stream), "b2l_seq_group_norm_gate")
        return linear(y, self.w_o)


# ------------------------------------------------------------------------------------------------ routed experts
class MoEFeedForward:
    """y = sum over the chosen experts of weight_e * expert_e(h).

        s = softmax(W_router h) over all experts, or sigmoid of each logit (`score`), f32;  choice = s + correction
        (steers the choice only); experts form `groups` equal groups of neighbours; a group is worth the sum of its
        `group_top` largest choice scores (1: its best); only experts of the `keep` best groups can be chosen; the `top`
        largest choice scores win;  weight = s / (sum of the chosen s + 1e-20) when `renormalize`, else s itself, times
        `weight_scale`
        expert e < experts: W_down unit(W_gate x, W_up x) with unit(a, b) = act(a) * b, or the clamped unit
        min(a, limit) * sigmoid(1.702 min(a, limit)) * (clamp(b, -limit, limit) + 1) (`act` = "clamped_swish");
        x = h and the weight scales the expert's output, or (`weight_on` = "input") x = weight * h and the outputs are
        summed unweighted;  the last `identity` outputs of the router: h itself

    A few tokens (also the captured single-token step) run with the expert index read on the device; longer portions
    sort the assignments by expert and run one pair of products per expert that received tokens."""

    SMALL = 4
    grouped = True        # bf16, 16-byte rows: the library's grouped product instead of one product per expert

    SCORES = {"softmax": S.SCORE_SOFTMAX, "sigmoid": S.SCORE_SIGMOID}

    def __init__(self, W: Dict[str, torch.Tensor], p: str, *, experts: int, identity: int, top: int, groups: int, keep: int, ff: int,
                 act: str = "silu", limit: float = 0.0, score: str = "softmax", renormalize: bool = True, weight_on: str = "output",
                 group_top: int = 1, weight_scale: float = 1.0) -> None:
        self.group_top, self.weight_scale = int(group_top), float(weight_scale)
        if self.group_top < 1:
            raise ValueError("routed experts: a group's score needs at least its best member")
        self.E, self.I, self.top, self.groups, self.keep, self.ff = int(experts), int(identity), int(top), int(groups), int(keep), int(ff)
        self.n = self.E + self.I
        if self.n % self.groups or not (1 <= self.keep <= self.groups) or self.keep * (self.n // self.groups) < self.top:
            raise ValueError("routed experts: groups / keep / top do not fit the expert count")
        self.act, self.limit = GatedMLP.ACTS[act], float(limit)
        if self.act == S.ACT_CLAMPED_SWISH and not self.limit > 0.0:
            raise ValueError("routed experts: the clamped unit needs a positive limit")
        if score not in self.SCORES or weight_on not in ("output", "input"):
            raise ValueError(f"routed experts: unknown score function {score!r} or weight placement {weight_on!r}")
        self.score, self.renorm, self.weight_input = self.SCORES[score], int(bool(renormalize)), int(weight_on == "input")
        if self.weight_input and self.I:
            raise ValueError("routed experts: identity experts with weights on the input are not built")
        self.w_router = W[p + "router"].contiguous()
        assert self.w_router.shape[0] == self.n, "routed experts: the router does not have experts + identity outputs"
        self.correction = W[p + "correction"].to(torch.float32).contiguous() if (p + "correction") in W else None
        dev, dt = self.w_router.device, W[p + "router"].dtype
        if self.E:
            self.w_gu = torch.stack([torch.cat([W[f"{p}e{e}.gate"], W[f"{p}e{e}.up"]], dim=0) for e in range(self.E)]).contiguous()
            self.w_down = torch.stack([W[f"{p}e{e}.down"] for e in range(self.E)]).contiguous()
            assert self.w_gu.shape[1] == 2 * self.ff, "routed experts: expert size does not fit"
        else:
            self.w_gu = self.w_down = torch.zeros(0, dtype=dt, device=dev)
        self.last_idx: Optional[torch.Tensor] = None       # the routing of the last call (tests, diagnostics)

    def state_specs(self) -> Dict[str, StateSpec]:
        return {}

    def route(self, h: torch.Tensor, ctx: StepContext) -> Tuple[torch.Tensor, torch.Tensor]:
        lib, T, dev, D = S.lib(), ctx.T, h.device, h.shape[1]
        if torch.backends.cuda.matmul.allow_tf32:
            raise RuntimeError("router logits need true 32-bit products: torch.backends.cuda.matmul.allow_tf32 is on")
        idx = torch.empty((T, self.top), dtype=torch.int32, device=dev)
        wgt = torch.empty((T, self.top), dtype=torch.float32, device=dev)
        if T <= self.SMALL:        # a few tokens: the logits and the routing in one launch
            S.check(lib.b2l_seq_moe_route_fused(_p(h), D, _p(self.w_router), _p(self.correction), D, self.n, self.groups, self.keep, self.top,
                                                self.score, self.renorm, self.group_top, self.weight_scale, _p(idx), _p(wgt), T, ctx.act,
                                                ctx.stream), "b2l_seq_moe_route_fused")
            self.last_idx = idx
            return idx, wgt
        # f32 logits: bf16 activations and router weights are exact in f32, the product keeps its f32 accumulator
        z = linear_f32(h, self.w_router)
        S.check(lib.b2l_seq_moe_route(_p(z), self.n, _p(self.correction), self.n, self.groups, self.keep, self.top, self.score, self.renorm,
                                      self.group_top, self.weight_scale, _p(idx), _p(wgt), T, ctx.stream), "b2l_seq_moe_route")
        self.last_idx = idx
        return idx, wgt

    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        lib, T, dev, D, E, top, ff = S.lib(), ctx.T, h.device, h.shape[1], self.E, self.top, self.ff
        idx, wgt = self.route(h, ctx)
        y = torch.empty((T, D), dtype=h.dtype, device=dev)
        N = T * top
        if T <= self.SMALL or E == 0:
            mid = torch.empty((N, ff), dtype=h.dtype, device=dev)
            S.check(lib.b2l_seq_moe_experts_small(_p(h), D, _p(self.w_gu) if E else None, _p(self.w_down) if E else None, _p(idx), _p(wgt), _p(mid),
                                                  _p(y), D, T, D, ff, E, top, self.act, self.limit, self.weight_input, ctx.act, ctx.stream),
                    "b2l_seq_moe_experts_small")
            return y
        meta = torch.empty((2 * (E + 1) + 2 * N,), dtype=torch.int32, device=dev)
        offsets, cursor, perm, inv = meta[:E + 1], meta[E + 1:2 * E + 2], meta[2 * E + 2:2 * E + 2 + N], meta[2 * E + 2 + N:]
        S.check(lib.b2l_seq_moe_sort(_p(idx), N, E, _p(offsets), _p(cursor), _p(perm), _p(inv), ctx.stream), "b2l_seq_moe_sort")
        xg = torch.empty((N + 8, D), dtype=h.dtype, device=dev)       # rows past the last group's end are never read
        S.check(lib.b2l_seq_moe_gather(_p(h), D, _p(perm), _p(offsets, E), _p(wgt) if self.weight_input else None, top, _p(xg), N, D, ctx.act,
                                       ctx.stream), "b2l_seq_moe_gather")
        gu = torch.empty((N, 2 * ff), dtype=h.dtype, device=dev)
        mid = torch.empty((N + 8, ff), dtype=h.dtype, device=dev)
        if self.grouped and h.dtype == torch.bfloat16 and D % 8 == 0 and ff % 8 == 0:
            # the library's grouped product: every expert's rows in one launch, group ends read on the device
            ends = offsets[1:]
            gu = F.grouped_mm(xg, self.w_gu.transpose(1, 2), offs=ends)
            S.check(lib.b2l_seq_gated_act(_p(gu), 2 * ff, _p(mid), N, ff, self.act, self.limit, ctx.act, ctx.stream), "b2l_seq_gated_act")
            yg = F.grouped_mm(mid, self.w_down.transpose(1, 2), offs=ends)
        else:
            off = offsets.cpu().tolist()                               # the one host read of a long portion
            for e in range(E):
                if off[e + 1] > off[e]:
                    torch.mm(xg[off[e]:off[e + 1]], self.w_gu[e].t(), out=gu[off[e]:off[e + 1]])
            S.check(lib.b2l_seq_gated_act(_p(gu), 2 * ff, _p(mid), off[E], ff, self.act, self.limit, ctx.act, ctx.stream), "b2l_seq_gated_act")
            yg = torch.empty((N, D), dtype=h.dtype, device=dev)
            for e in range(E):
                if off[e + 1] > off[e]:
                    torch.mm(mid[off[e]:off[e + 1]], self.w_down[e].t(), out=yg[off[e]:off[e + 1]])
        S.check(lib.b2l_seq_moe_combine(_p(yg), _p(inv), None if self.weight_input else _p(wgt), _p(h), D, _p(y), D, T, D, top, ctx.act,
                                        ctx.stream), "b2l_seq_moe_combine")
        return y
