"""CPU: the Zuvevik configuration reader and registry entry, the argument blocks of its kernels against a C compiler,
and the plain restatement's own invariants (tests/zuvevik_oracle.py)."""
import ctypes as C
import os
import subprocess

import pytest
import torch

import zuvevik_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def small_config():
    mixer = {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 6, "mask": {"size": 5}, "scale": 0.3, "v_mix": True, "rot": {"base": 100.0, "dims": 4}}
    return {"architecture": "Zuvevik", "vocab": 30, "width": 16, "norm": {"eps": 1e-5}, "streams": 2, "logit_scale": 1.5,
            "embedding": {"bigram": {"buckets": 7, "mul_prev": 3, "mul_cur": 5}},
            "layers": [{"type": "attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": 20}},
                       {"type": "attention", "mixer": mixer, "mlp": {"kind": "moe", "expert": {"ff": 8, "limit": 1.0}, "router": {"experts": 3, "top": 2}}},
                       {"type": "attention", "mixer": mixer, "mlp": None}]}


def test_config_reader_and_registry():
    from lit_llama_b200 import ZuvevikConfig, registry

    assert "Zuvevik" in registry.architectures()
    c = ZuvevikConfig.from_dict(small_config())
    assert (c.vocab, c.width, c.streams, c.logit_scale, c.bigram["buckets"]) == (30, 16, 2, 1.5, 7)
    assert ZuvevikConfig.from_dict(c.to_dict()) == c
    d = small_config()
    del d["streams"], d["embedding"], d["logit_scale"]
    c = ZuvevikConfig.from_dict(d)
    assert (c.streams, c.logit_scale, c.bigram) == (1, 1.0, None)
    for breaker in (lambda d: d["layers"][0].update(type="convolution"), lambda d: d["layers"][1]["mlp"].update(kind="maxout"),
                    lambda d: d["layers"][2]["mixer"].update(mask={}), lambda d: d.update(architecture="Other"), lambda d: d.update(streams=0)):
        d = small_config()
        breaker(d)
        with pytest.raises(ValueError):
            ZuvevikConfig.from_dict(d)


def test_argument_blocks_match_the_header(tmp_path):
    from lit_llama_b200 import _seqlib as S

    prog = tmp_path / "layout.c"
    prog.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "b2l_seq.h"\nint main(void){printf("%zu %zu %zu %zu %zu %zu %zu\\n", '
                    "sizeof(b2l_seq_qkv_prep_args), offsetof(b2l_seq_qkv_prep_args, eps), offsetof(b2l_seq_qkv_prep_args, q_out), "
                    "offsetof(b2l_seq_qkv_prep_args, lambda), offsetof(b2l_seq_qkv_prep_args, act_dtype), sizeof(b2l_seq_attn_args), "
                    "offsetof(b2l_seq_attn_args, gate_per_channel));return 0;}\n")
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), str(prog), "-o", str(exe)], check=True)
    out = [int(v) for v in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()]
    A, B = S.QkvPrepArgs, S.AttnArgs
    assert out == [C.sizeof(A), A.eps.offset, A.q_out.offset, A.lambda_.offset, A.act_dtype.offset, C.sizeof(B), B.gate_per_channel.offset]


def test_oracle_window_and_pair_rows():
    g = torch.Generator().manual_seed(0)
    T, H, G, K, V = 12, 4, 2, 6, 5
    q, k, v = (torch.randn(T, n, d, generator=g, dtype=torch.float64) for n, d in ((H, K), (G, K), (G, V)))
    full = O.windowed_softmax_attention(q, k, v, 0.5, T)
    wider = O.windowed_softmax_attention(q, k, v, 0.5, T + 9)
    assert torch.allclose(full, wider)
    causal = torch.softmax((torch.einsum("thk,sk->hts", q[:, :2], k[:, 0]) * 0.5).masked_fill(torch.ones(T, T).triu(1).bool(), -1e300), dim=-1)
    assert torch.allclose(full.view(T, H, V)[:, 1], causal[1] @ v[:, 0])
    own = O.windowed_softmax_attention(q, k, v, 0.5, 1)                 # a window of one position: the query's own value
    assert torch.allclose(own.view(T, H, V)[:, 3], v[:, 1])
    near = O.windowed_softmax_attention(q, k, v, 0.5, 3)
    assert torch.allclose(near[:3], full[:3]) and not torch.allclose(near[3:], full[3:])
    rows = O.pair_rows([4, 9, 2], 7, 3, 5)
    assert rows == [7, (4 * 3 + 9 * 5) % 7, (9 * 3 + 2 * 5) % 7]
    assert O.pair_rows([9, 2], 7, 3, 5, before=4) == rows[1:]


def test_oracle_streams_reduce_to_the_plain_residual():
    """With one stream and unit weights a hyper-connection step is x + y; mixing conserves what the weights say."""
    x, y = torch.randn(3, 8, dtype=torch.float64), torch.randn(3, 8, dtype=torch.float64)
    one = torch.ones(1, dtype=torch.float64)
    assert torch.allclose(O.hyper_step([x], y, one, one.reshape(1, 1), one)[0], x + y)
    mix = torch.tensor([[0.5, 2.0], [1.0, -1.0]], dtype=torch.float64)
    a, b = O.hyper_step([x, 2 * x], y, None, mix, torch.tensor([0.0, 3.0], dtype=torch.float64))
    assert torch.allclose(a, 0.5 * x + 1.0 * 2 * x) and torch.allclose(b, 2.0 * x - 2 * x + 3 * y)
    unit = O.clamped_unit(torch.tensor([-9.0, 0.5, 9.0], dtype=torch.float64), torch.tensor([9.0, -9.0, 0.25], dtype=torch.float64), 2.0)
    want = [-9.0 * torch.sigmoid(torch.tensor(-9.0 * 1.702, dtype=torch.float64)) * 3.0, 0.5 * torch.sigmoid(torch.tensor(0.5 * 1.702, dtype=torch.float64)) * -1.0,
            2.0 * torch.sigmoid(torch.tensor(2.0 * 1.702, dtype=torch.float64)) * 1.25]
    assert torch.allclose(unit, torch.stack(want))
