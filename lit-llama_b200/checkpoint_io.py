"""Checkpoint readers.  A `.safetensors` file is an 8-byte little-endian header length, that many bytes of JSON
(name -> dtype, shape, data_offsets) and the raw little-endian data; it is read here with the standard library and
torch only.  `.pth` checkpoints of the LLaMA path keep going through `torch.load` (utils.lazy_load)."""
import json
import mmap
import struct
from typing import Dict, Optional

import torch

_DTYPES = {
    "BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "F64": torch.float64,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool,
}


def read_safetensors(path: str, device: Optional[torch.device] = None, float_dtype: Optional[torch.dtype] = None) -> Dict[str, torch.Tensor]:
    """Every tensor of the file, on `device`; floating tensors converted to `float_dtype` when given (integer
    tables keep their type)."""
    out: Dict[str, torch.Tensor] = {}
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n).decode("utf-8"))
        base = 8 + n
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        try:
            for name, info in header.items():
                if name == "__metadata__":
                    continue
                dt = _DTYPES.get(info["dtype"])
                if dt is None:
                    raise ValueError(f"{path}: tensor {name!r} has unsupported dtype {info['dtype']}")
                lo, hi = info["data_offsets"]
                shape = tuple(info["shape"])
                count = 1
                for s in shape:
                    count *= s
                if hi - lo != count * torch.empty((), dtype=dt).element_size():
                    raise ValueError(f"{path}: tensor {name!r}: {hi - lo} bytes do not fit shape {shape}")
                if count == 0:
                    t = torch.empty(shape, dtype=dt)
                else:
                    t = torch.frombuffer(bytearray(mm[base + lo: base + hi]), dtype=dt).reshape(shape)
                if float_dtype is not None and t.is_floating_point():
                    t = t.to(float_dtype)
                out[name] = t.to(device) if device is not None else t
        finally:
            mm.close()
    return out


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor]) -> None:
    """The inverse of read_safetensors (used to save synthetic models)."""
    names = {v: k for k, v in _DTYPES.items()}
    header, blobs, at = {}, [], 0
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": names[t.dtype], "shape": list(t.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    h = json.dumps(header, separators=(",", ":")).encode("utf-8")
    h += b" " * (-len(h) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)))
        f.write(h)
        for b in blobs:
            f.write(b)
