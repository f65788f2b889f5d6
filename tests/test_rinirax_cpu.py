"""CPU: the Rinirax configuration reader and registry entry, the argument blocks of its kernels against a C compiler,
and the plain restatement's own invariants (tests/rinirax_oracle.py)."""
import ctypes as C
import math
import os
import subprocess

import pytest
import torch

import rinirax_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def small_config():
    att = {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 6, "scale": 0.3, "diff": 0.4, "conv": 3, "rot": {"base": 100.0, "dims": 4}}
    lat = {"heads": 2, "dim": 8, "rot_dim": 4, "vdim": 6, "q_rank": 10, "kv_rank": 12, "scale": 0.3, "mask": {"size": 5},
           "rot": {"base": 100.0, "dims": 4, "scaling": {"factor": 2.0, "original": 16, "fast": 4.0, "slow": 1.0}}}
    experts = {"kind": "moe", "expert": {"ff": 8}, "router": {"experts": 6, "top": 2, "scale": 1.25, "groups": {"count": 3, "keep": 2}}}
    return {"architecture": "Rinirax", "vocab": 30, "width": 16, "norm": {"eps": 1e-5},
            "layers": [{"type": "attention", "mixer": att, "mlp": {"kind": "dense", "ff": 20}},
                       {"type": "mingru", "mixer": {"width": 12}, "mlp": experts},
                       {"type": "latent_attention", "mixer": lat, "mlp": None},
                       {"type": "attention", "mixer": dict(att, kv_from=0), "mlp": experts}]}


def test_config_reader_and_registry():
    from lit_llama_b200 import RiniraxConfig, registry

    assert "Rinirax" in registry.architectures()
    c = RiniraxConfig.from_dict(small_config())
    assert (c.vocab, c.width, c.eps, len(c.layers)) == (30, 16, 1e-5, 4)
    assert RiniraxConfig.from_dict(c.to_dict()) == c
    for breaker in (lambda d: d["layers"][0].update(type="convolution"), lambda d: d["layers"][1]["mlp"].update(kind="maxout"),
                    lambda d: d["layers"][3]["mixer"].update(kv_from=3), lambda d: d["layers"][3]["mixer"].update(kv_from=1),
                    lambda d: d["layers"][0]["mixer"].update(kv_from=0), lambda d: d.update(architecture="Other")):
        d = small_config()
        breaker(d)
        with pytest.raises(ValueError):
            RiniraxConfig.from_dict(d)


def test_argument_blocks_match_the_header(tmp_path):
    from lit_llama_b200 import _seqlib as S

    prog = tmp_path / "layout.c"
    prog.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "b2l_seq.h"\nint main(void){printf("%zu %zu %zu %zu %zu %zu %zu %zu %zu %zu\\n", '
                    "sizeof(b2l_seq_conv_rope_args), offsetof(b2l_seq_conv_rope_args, w), offsetof(b2l_seq_conv_rope_args, freq), "
                    "offsetof(b2l_seq_conv_rope_args, rot_mult), offsetof(b2l_seq_conv_rope_args, act_dtype), sizeof(b2l_seq_attn_args), "
                    "offsetof(b2l_seq_attn_args, no_append), offsetof(b2l_seq_attn_args, diff_mult), sizeof(b2l_seq_latent_attn_args), "
                    "offsetof(b2l_seq_latent_attn_args, window));return 0;}\n")
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), str(prog), "-o", str(exe)], check=True)
    out = [int(v) for v in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()]
    A, B, L = S.ConvRopeArgs, S.AttnArgs, S.LatentAttnArgs
    assert out == [C.sizeof(A), A.w.offset, A.freq.offset, A.rot_mult.offset, A.act_dtype.offset, C.sizeof(B), B.no_append.offset, B.diff_mult.offset, C.sizeof(L),
                   L.window.offset]


def test_oracle_rotation_frequencies_match_the_package():
    from lit_llama_b200.mixers import rope_frequencies

    for dims, base, scaling in ((8, 100.0, None), (32, 3e5, {"factor": 6.0, "original": 512, "fast": 24.0, "slow": 1.0}),
                                (16, 1e4, {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0})):
        f, mult = O.yarn_frequencies(dims, base, scaling)
        g, m = rope_frequencies(dims, base, scaling)
        assert mult == pytest.approx(m) and torch.allclose(torch.tensor(f, dtype=torch.float32), g, rtol=1e-6)
        if scaling:
            assert f[0] == pytest.approx(1.0) and f[-1] < base ** (-2.0 * (dims // 2 - 1) / dims)      # fast pairs kept, slow ones stretched


def test_oracle_invariants():
    g = torch.Generator().manual_seed(0)
    # a convolution whose last tap is one and the rest zero is the identity; taps before the start read zeros
    u = torch.randn(6, 3, generator=g, dtype=torch.float64)
    w = torch.zeros(3, 4, dtype=torch.float64)
    w[:, -1] = 1.0
    assert torch.equal(O.causal_conv(u, w), u)
    w[:, -1], w[:, 0] = 0.0, 1.0
    assert torch.equal(O.causal_conv(u, w)[3:], u[:3]) and float(O.causal_conv(u, w)[:3].abs().max()) == 0.0
    # rotations keep the length; both layouts turn pair i by the same angle
    v = torch.randn(8, generator=g, dtype=torch.float64)
    f, _ = O.plain_frequencies(8, 50.0)
    a, b = O.rotate(v, 7, f, 1.0, True), O.rotate(v[[0, 2, 4, 6, 1, 3, 5, 7]], 7, f, 1.0, False)
    assert float(a.norm()) == pytest.approx(float(v.norm())) and torch.allclose(a[[0, 2, 4, 6, 1, 3, 5, 7]], b)
    # xIELU is continuous at zero with slope 1/2 on both sides
    z = torch.tensor([-1e-6, 0.0, 1e-6], dtype=torch.float64)
    y = O.xielu(z, 0.3, -0.2)
    assert float(y[1]) == 0.0 and float((y[2] - y[0]) / 2e-6) == pytest.approx(0.5, rel=1e-4)
    # the recurrence with an open gate copies the candidate, with a closed one keeps the state
    W = {"z": torch.zeros(2, 2), "x": torch.eye(2), "g": torch.zeros(2, 2), "o": torch.eye(2), "z.b": torch.tensor([40.0, -40.0]), "x.b": torch.zeros(2)}
    h = torch.tensor([[1.0, 1.0], [3.0, 3.0]], dtype=torch.float64)
    W["g"] = torch.eye(2) * 50.0                     # silu(50 h) = 50 h to many digits
    out = O.mingru(h, W, "")
    assert out[1, 0] == pytest.approx(3.5 * 150.0) and abs(float(out[1, 1])) < 1e-10
    # group scores are sums of the two best; a lone strong expert loses its group
    Wr = {"router": torch.eye(6), "correction": torch.zeros(6)}
    idx, wgt = O.route(torch.tensor([[5.0, -9, -9, 1.0, 1.0, -9]], dtype=torch.float64), Wr, "", {"experts": 6, "top": 2, "scale": 3.0, "groups": {"count": 2, "keep": 1}})
    assert sorted(idx[0].tolist()) == [3, 4] and float(wgt.sum()) == pytest.approx(3.0)


def test_oracle_whole_model_runs_and_shares_keys():
    cfg = small_config()
    g = torch.Generator().manual_seed(1)
    D, W = cfg["width"], {}

    def lin(o, i):
        return torch.randn(o, i, generator=g) / math.sqrt(i)

    W["embed"], W["head"], W["final.norm"], W["final.norm.b"] = torch.randn(30, D, generator=g), lin(30, D), torch.ones(D), torch.zeros(D)
    for i, layer in enumerate(cfg["layers"]):
        p, m, c = f"l{i}.", f"l{i}.mix.", layer["mixer"]
        W[p + "norm1"], W[p + "norm1.b"] = torch.ones(D), torch.zeros(D)
        W[p + "dwa"] = torch.tensor([0.0] * (i + 1) + [1.0])
        if layer["type"] == "attention":
            rows = {"q": 64} if "kv_from" in c else {"q": 64, "k": 32, "v": 12}
            for n, r in rows.items():
                W[m + n], W[m + n + ".b"], W[m + n + ".conv"] = lin(r, D), torch.zeros(r), torch.randn(r, 3, generator=g)
            for n in ("lq1", "lk1", "lq2", "lk2"):
                W[m + n] = 0.1 * torch.randn(8, generator=g)
            W[m + "o"] = lin(D, 24)
        elif layer["type"] == "mingru":
            W[m + "z"], W[m + "x"], W[m + "g"], W[m + "o"], W[m + "z.b"], W[m + "x.b"] = lin(12, D), lin(12, D), lin(12, D), lin(D, 12), torch.zeros(12), torch.zeros(12)
        else:
            W[m + "dq"], W[m + "dq.norm"], W[m + "uq"], W[m + "dkv"], W[m + "dkv.norm"] = lin(10, D), torch.ones(10), lin(24, 10), lin(16, D), torch.ones(12)
            W[m + "uk"], W[m + "uv"], W[m + "o"] = lin(16, 12), lin(12, 12), lin(D, 12)
        f = layer["mlp"]
        if f and f["kind"] == "dense":
            W[p + "mlp.up"], W[p + "mlp.down"], W[p + "mlp.act"] = lin(20, D), lin(D, 20), torch.zeros(2)
        elif f:
            W[p + "mlp.router"], W[p + "mlp.correction"] = lin(6, D), torch.zeros(6)
            for e in range(6):
                W[f"{p}mlp.e{e}.gate"], W[f"{p}mlp.e{e}.up"], W[f"{p}mlp.e{e}.down"] = lin(8, D), lin(8, D), lin(D, 8)
    toks = [3, 1, 4, 1, 5, 9, 2, 6, 5, 3, 5, 8]
    cap = []
    out = O.model(toks, cfg, W, capture=cap)
    assert out.shape == (12, 30) and len(cap) == 4 and bool(torch.isfinite(out).all())
    # causal: a later token changes nothing before it; the window of the latent layer does not reach back past 5 positions
    again = O.model(toks[:7] + [0] + toks[8:], cfg, W)
    assert torch.allclose(again[:7], out[:7]) and not torch.allclose(again[7:], out[7:])
