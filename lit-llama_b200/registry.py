"""Model registry: config.json's "architecture" picks the loader, as `llama_model_lookup` picks a LLaMA size from
a checkpoint.  A loader returns an object the Engine can serve (state_specs / vocab / dtype / device /
forward_portion)."""
import json
import os
from typing import Callable, Dict, Optional

import torch

_LOADERS: Dict[str, Callable] = {}


def register(architecture: str):
    def deco(fn: Callable) -> Callable:
        _LOADERS[architecture] = fn
        return fn
    return deco


def architectures():
    return sorted(_LOADERS)


@register("Lugovik")
def _load_lugovik(model_dir: str, dtype: torch.dtype, device: torch.device, max_positions: int, config: dict):
    from . import lugovik

    return lugovik.load(model_dir, dtype=dtype, device=device, max_positions=max_positions)


@register("Zenasun")
def _load_zenasun(model_dir: str, dtype: torch.dtype, device: torch.device, max_positions: int, config: dict):
    from . import zenasun

    return zenasun.load(model_dir, dtype=dtype, device=device, max_positions=max_positions)


@register("Zuvevik")
def _load_zuvevik(model_dir: str, dtype: torch.dtype, device: torch.device, max_positions: int, config: dict):
    from . import zuvevik

    return zuvevik.load(model_dir, dtype=dtype, device=device, max_positions=max_positions)


@register("Rinirax")
def _load_rinirax(model_dir: str, dtype: torch.dtype, device: torch.device, max_positions: int, config: dict):
    from . import rinirax

    return rinirax.load(model_dir, dtype=dtype, device=device, max_positions=max_positions)


@register("LLaMA")
def _load_llama(model_dir: str, dtype: torch.dtype, device: torch.device, max_positions: int, config: dict):
    """config.json: {"architecture": "LLaMA", "name": "7B" | sizes..., "quantize": null | "gptq.int4" | ..., "checkpoint": file}."""
    from .model import LLaMA, LLaMAConfig
    from .utils import EmptyInitOnDevice, lazy_load

    if dtype != torch.bfloat16:
        raise RuntimeError("the LLaMA path runs in bfloat16 only")
    cfg = LLaMAConfig.from_name(config["name"]) if "name" in config else LLaMAConfig(
        **{k: config[k] for k in ("block_size", "vocab_size", "n_layer", "n_head", "n_embd") if k in config})
    with EmptyInitOnDevice(device=device, dtype=torch.bfloat16, quantization_mode=config.get("quantize")):
        model = LLaMA(cfg)
    with lazy_load(os.path.join(model_dir, config.get("checkpoint", "lit-llama.pth"))) as sd:
        model.load_state_dict(sd)
    return LLaMASequenceModel(model.eval(), max_positions or cfg.block_size)


class LLaMASequenceModel:
    """The package's LLaMA behind the Engine's model interface.  Its KV cache lives inside the module (one sequence
    at a time), so it declares no pooled state; a portion that starts at position 0 resets the cache."""
    graph_safe = False     # LLaMA.forward replays its own decode graph

    def __init__(self, model, max_seq_length: int) -> None:
        self.model, self.max_seq_length = model, int(max_seq_length)
        self.vocab = model.config.padded_vocab_size
        self.dtype = torch.bfloat16
        self.device = next(model.parameters()).device
        self._pos = 0

    def state_specs(self):
        return {}

    @torch.no_grad()
    def forward_portion(self, tokens: torch.Tensor, ctx, want: Optional[torch.Tensor] = None) -> torch.Tensor:
        pos0 = int(ctx.meta[1])
        if pos0 == 0:
            self.model.reset_cache()
        T = tokens.numel()
        input_pos = torch.arange(pos0, pos0 + T, device=tokens.device)
        logits = self.model(tokens.view(1, -1).to(torch.int64), self.max_seq_length, input_pos)[0]
        return (logits if want is None else logits.index_select(0, want.to(torch.int64))).float()


def read_config(model_dir: str) -> dict:
    with open(os.path.join(model_dir, "config.json")) as f:
        return json.load(f)


def load_model(model_dir: str, dtype: torch.dtype = torch.bfloat16, device: Optional[torch.device] = None, max_positions: int = 0):
    """The model of `model_dir` (config.json + weights) on `device`, chosen by config.json's architecture."""
    config = read_config(model_dir)
    arch = config.get("architecture")
    if arch not in _LOADERS:
        raise ValueError(f"unknown architecture {arch!r}; registered: {architectures()}")
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    return _LOADERS[arch](model_dir, dtype, device, max_positions, config)
