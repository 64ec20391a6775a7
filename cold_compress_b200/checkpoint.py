"""Checkpoint folders: `config.json` + `model.safetensors`, and the registry that maps config.json's `architecture`
to a model class.  A safetensors file is an 8-byte little-endian header length, that many bytes of JSON
(name -> dtype, shape, data_offsets) and the raw little-endian data; it is parsed here directly (no extra package)."""
from __future__ import annotations

import json
import struct
from pathlib import Path
from typing import Callable, Dict

import torch

_DTYPES = {"BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "F64": torch.float64,
           "I32": torch.int32, "I64": torch.int64, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool}


def read_safetensors(path) -> Dict[str, torch.Tensor]:
    """name -> CPU tensor (a copy; the file is not kept mapped)."""
    out = {}
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) != 8:
            raise ValueError(f"{path}: not a safetensors file")
        (n,) = struct.unpack("<Q", head)
        header = json.loads(f.read(n).decode("utf-8"))
        base = 0
        mm = bytearray(f.read())
        if True:
            for name, meta in header.items():
                if name == "__metadata__":
                    continue
                dtype = _DTYPES.get(meta["dtype"])
                if dtype is None:
                    raise ValueError(f"{path}: tensor {name!r} has unsupported dtype {meta['dtype']}")
                lo, hi = meta["data_offsets"]
                shape = tuple(meta["shape"])
                count = 1
                for s in shape:
                    count *= s
                if count == 0:
                    out[name] = torch.empty(shape, dtype=dtype)
                    continue
                if hi - lo != count * torch.empty((), dtype=dtype).element_size():
                    raise ValueError(f"{path}: tensor {name!r}: {hi - lo} bytes do not fit shape {shape}")
                t = torch.frombuffer(mm, dtype=dtype, count=count, offset=base + lo).clone()
                out[name] = t.reshape(shape)
    return out


# architecture name (config.json "architecture") -> builder(config dict, dtype) returning a model with load_tensors()
MODEL_REGISTRY: Dict[str, Callable] = {}


def register_model(architecture: str, builder: Callable):
    MODEL_REGISTRY[architecture] = builder


def _builtin():
    if "Tidelorn" not in MODEL_REGISTRY:
        from .tidelorn import TidelornTransformer
        register_model("Tidelorn", TidelornTransformer.from_config)
    if "Detatar" not in MODEL_REGISTRY:
        from .detatar import DetatarTransformer
        register_model("Detatar", DetatarTransformer.from_config)
    if "Tefovik" not in MODEL_REGISTRY:
        from .tefovik import TefovikTransformer
        register_model("Tefovik", TefovikTransformer.from_config)
    if "Nevodra" not in MODEL_REGISTRY:
        from .nevodra import NevodraTransformer
        register_model("Nevodra", NevodraTransformer.from_config)


def is_checkpoint_folder(path) -> bool:
    p = Path(path)
    return p.is_dir() and (p / "config.json").exists()


def load_checkpoint_folder(path, device, precision=torch.bfloat16):
    """Builds the model class that config.json names, fills it from model.safetensors and moves it to `device`."""
    _builtin()
    p = Path(path)
    cfg = json.loads((p / "config.json").read_text())
    arch = cfg.get("architecture")
    if arch not in MODEL_REGISTRY:
        raise ValueError(f"{p / 'config.json'}: unknown architecture {arch!r} (known: {sorted(MODEL_REGISTRY)})")
    model = MODEL_REGISTRY[arch](cfg, precision)
    unused = model.load_tensors(read_safetensors(p / "model.safetensors"))
    if unused:
        print(f"note: {len(unused)} checkpoint tensors are not used by {arch}: {unused[:8]}")
    return model.to(device).eval()


def write_safetensors(path, tensors: Dict[str, torch.Tensor]):
    """The inverse of read_safetensors (used to export random-init checkpoints for benchmarks and tests)."""
    names = {v: k for k, v in _DTYPES.items()}
    header, blobs, off = {}, [], 0
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        raw = t.view(torch.uint8).numpy().tobytes() if t.dim() else t.reshape(1).view(torch.uint8).numpy().tobytes()
        header[name] = {"dtype": names[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    head = json.dumps(header, separators=(",", ":")).encode("utf-8")
    head += b" " * (-len(head) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(head)))
        f.write(head)
        for b in blobs:
            f.write(b)
