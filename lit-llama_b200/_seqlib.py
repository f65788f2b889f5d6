"""ctypes binding of libb200seq.so (include/b2l_seq.h): the sequence-mixer kernels.  The library is compiled on
first use when it is missing (only this library, not the quantized-LLaMA one).  No CPU or PyTorch fallback."""
import ctypes as C
import threading

import torch

from . import _build

B2L_BF16, B2L_F32 = 0, 1
ACT_GELU_TANH, ACT_SILU, ACT_SIGMOID, ACT_CLAMPED_SWISH, ACT_XIELU, ACT_NONE = 0, 1, 2, 3, 4, 5
NORM_RMS, NORM_LAYER = 0, 1
SCORE_SOFTMAX, SCORE_SIGMOID = 0, 1
DECAY_EXP_SOFTPLUS, DECAY_SIGMOID_ROOT = 0, 1

c_void_p, c_int, c_float, c_size_t = C.c_void_p, C.c_int, C.c_float, C.c_size_t


class ScanArgs(C.Structure):
    _fields_ = [
        ("q", c_void_p), ("ldq", c_int),
        ("k", c_void_p), ("ldk", c_int),
        ("v", c_void_p), ("ldv", c_int),
        ("q_mult", c_float),
        ("decay", c_void_p), ("ldd", c_int), ("decay_per_channel", c_int),
        ("beta", c_void_p), ("ldb", c_int), ("delta", c_int),
        ("vscale", c_void_p), ("ldvs", c_int),
        ("skip", c_void_p),
        ("state", c_void_p), ("meta", c_void_p),
        ("out", c_void_p), ("ldo", c_int),
        ("T", c_int), ("heads", c_int), ("qk_heads", c_int), ("K", c_int), ("V", c_int), ("act_dtype", c_int),
        ("work_state", c_void_p), ("work_decay", c_void_p), ("n_chunks", c_int),
    ]


class AttnArgs(C.Structure):
    _fields_ = [
        ("q", c_void_p),
        ("k_new", c_void_p),
        ("v_new", c_void_p), ("ldv", c_int),
        ("cache_k", c_void_p), ("cache_v", c_void_p),
        ("meta", c_void_p),
        ("gate", c_void_p), ("ldg", c_int),
        ("out", c_void_p), ("ldo", c_int),
        ("scale", c_float), ("softcap", c_float), ("out_mult", c_float),
        ("has_sink", c_int), ("block", c_int), ("T", c_int), ("heads", c_int), ("kv_heads", c_int), ("K", c_int), ("V", c_int),
        ("act_dtype", c_int),
        ("window", c_int), ("gate_per_channel", c_int),
        ("work", c_void_p), ("work_floats", c_int),
        ("maps", c_int), ("out_f32", c_int), ("no_append", c_int),
        ("diff_out", c_void_p), ("ldd", c_int),
        ("diff_lambda", c_float), ("diff_eps", c_float), ("diff_mult", c_float),
    ]


class LatentAttnArgs(C.Structure):
    _fields_ = [
        ("q_a", c_void_p), ("ldqa_t", C.c_longlong), ("ldqa_h", C.c_longlong),
        ("q_b", c_void_p), ("ldqb_t", C.c_longlong), ("ldqb_h", C.c_longlong),
        ("key_a", c_void_p), ("ldka", C.c_longlong), ("hska", C.c_longlong), ("slot_stride_a", C.c_longlong),
        ("key_b", c_void_p), ("ldkb", C.c_longlong), ("slot_stride_b", C.c_longlong),
        ("sink", c_void_p),
        ("meta", c_void_p),
        ("out", c_void_p), ("ldo", c_int),
        ("work", c_void_p),
        ("scale", c_float),
        ("T", c_int), ("heads", c_int), ("heads_per_group", c_int), ("n_a", c_int), ("n_b", c_int), ("vdim", c_int), ("score_off", c_int),
        ("splits", c_int), ("act_dtype", c_int),
        ("window", c_int),
    ]


class ConvRopeArgs(C.Structure):
    _fields_ = [
        ("proj", c_void_p), ("ld", c_int),
        ("c_off", c_int), ("C", c_int), ("taps", c_int),
        ("w", c_void_p), ("state", c_void_p), ("meta", c_void_p),
        ("q_off", c_int), ("q_heads", c_int), ("k_off", c_int), ("k_heads", c_int), ("K", c_int), ("v_off", c_int), ("n_v", c_int),
        ("freq", c_void_p), ("rot_dims", c_int), ("interleaved", c_int), ("rot_mult", c_float),
        ("q_out", c_void_p), ("k_out", c_void_p), ("v_out", c_void_p),
        ("T", c_int), ("act_dtype", c_int),
    ]


class QkvPrepArgs(C.Structure):
    _fields_ = [
        ("proj", c_void_p), ("ld", c_int), ("q_off", c_int), ("k_off", c_int), ("v_off", c_int),
        ("q_norm", c_void_p), ("k_norm", c_void_p), ("whole_row", c_int), ("eps", c_float),
        ("freq", c_void_p), ("rot_dims", c_int), ("rot_mult", c_float),
        ("meta", c_void_p),
        ("q_out", c_void_p), ("k_out", c_void_p),
        ("v_first", c_void_p), ("ldvf", c_int), ("lambda_", c_void_p), ("v_out", c_void_p),
        ("T", c_int), ("heads", c_int), ("kv_heads", c_int), ("K", c_int), ("V", c_int), ("act_dtype", c_int),
    ]


_SIGS = {
    "b2l_seq_version": (c_int, []),
    "b2l_seq_last_error": (C.c_char_p, []),
    "b2l_seq_embed": (c_int, [c_void_p, c_int, c_void_p, c_int, c_float, c_void_p, c_int, c_int, c_int, c_void_p]),
    "b2l_seq_rmsnorm": (c_int, [c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "b2l_seq_norm_add_norm": (c_int, [c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "b2l_seq_gated_act": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float, c_int, c_void_p]),
    "b2l_seq_conv_silu": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                  c_void_p]),
    "b2l_seq_unit_norm": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p]),
    "b2l_seq_decay": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_float, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                              c_void_p]),
    "b2l_seq_scan": (c_int, [C.POINTER(ScanArgs), c_void_p]),
    "b2l_seq_scan_chunks": (c_int, [c_int, c_int]),
    "b2l_seq_group_norm_gate": (c_int, [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float, c_float, c_void_p,
                                        c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "b2l_seq_headnorm_rope": (c_int, [c_void_p, c_int, c_void_p, c_float, c_void_p, c_int, c_float, c_void_p, c_void_p, c_int, c_int,
                                      c_int, c_int, c_int, c_void_p]),
    "b2l_seq_block_attention": (c_int, [C.POINTER(AttnArgs), c_void_p]),
    "b2l_seq_block_attention_work_floats": (C.c_longlong, [C.POINTER(AttnArgs)]),
    "b2l_seq_cast_f32": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "b2l_seq_zero_slot": (c_int, [c_void_p, c_size_t, c_int, c_void_p]),
    "b2l_seq_add_norm2": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_float, c_void_p, c_int,
                                  c_int, c_int, c_void_p]),
    "b2l_seq_softcap": (c_int, [c_void_p, c_size_t, c_float, c_void_p]),
    "b2l_seq_rope": (c_int, [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_float, c_float, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                             c_int, c_int, c_int, c_int, c_void_p]),
    "b2l_seq_latent_prep": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_int,
                                    c_float, c_float, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "b2l_seq_latent_attention": (c_int, [C.POINTER(LatentAttnArgs), c_void_p]),
    "b2l_seq_latent_attention_warps": (c_int, [c_int, c_int]),
    "b2l_seq_moe_route": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_int,
                                  c_void_p]),
    "b2l_seq_moe_route_fused": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                        c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "b2l_seq_moe_experts_small": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                          c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p]),
    "b2l_seq_moe_sort": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "b2l_seq_moe_gather": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p]),
    "b2l_seq_moe_combine": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "b2l_seq_embed_pair": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_float, c_void_p, c_void_p, C.c_longlong, C.c_longlong, c_int, c_void_p,
                                   c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "b2l_seq_hc_step": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_int,
                                c_int, c_void_p]),
    "b2l_seq_hc_sum": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "b2l_seq_scale": (c_int, [c_void_p, c_size_t, c_float, c_void_p]),
    "b2l_seq_qkv_prep": (c_int, [C.POINTER(QkvPrepArgs), c_void_p]),
    "b2l_seq_unary_act": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p]),
    "b2l_seq_conv_rope": (c_int, [C.POINTER(ConvRopeArgs), c_void_p]),
    "b2l_seq_diff_combine": (c_int, [c_void_p, c_int, c_float, c_float, c_float, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "b2l_seq_mingru_chunks": (c_int, [c_int]),
    "b2l_seq_mingru": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                               c_void_p]),
    "b2l_seq_norm": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "b2l_seq_depth_step": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float,
                                   c_void_p, c_int, c_int, c_int, c_void_p]),
}

EXPORTS = tuple(_SIGS)
LIB_PATH = _build.LIBRARIES["seq"]["out"]

_lib = None
_lock = threading.Lock()


def lib():
    """The loaded library; built first (nvcc, sm_100a) when it is missing or older than its sources."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                handle = C.CDLL(_build.ensure("seq"))
                for name, (res, args) in _SIGS.items():
                    fn = getattr(handle, name)
                    fn.restype = res
                    fn.argtypes = args
                _lib = handle
    return _lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = lib().b2l_seq_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"{what} failed (rc={rc}): {msg}")


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def act_code(dtype: torch.dtype) -> int:
    if dtype == torch.bfloat16:
        return B2L_BF16
    if dtype == torch.float32:
        return B2L_F32
    raise RuntimeError(f"dtype {dtype} unsupported: the sequence kernels take torch.bfloat16 or torch.float32")


def ptr(t) -> int:
    """Device pointer of a CUDA tensor (None -> null)."""
    if t is None:
        return None
    if not t.is_cuda:
        raise RuntimeError(f"tensor on {t.device}: the sequence kernels run on CUDA only (no CPU fallback)")
    return t.data_ptr()
