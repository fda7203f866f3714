"""Reader / writer of the safetensors container: 8-byte little-endian header length, a JSON header
{name: {dtype, shape, data_offsets}}, then the raw little-endian tensor bytes.  Standard library + torch only.
Tensors come back as torch CPU tensors (bfloat16 stays bfloat16)."""
import json
import struct

import numpy as np
import torch

_DTYPES = {
    "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2), "F32": (torch.float32, 4), "F64": (torch.float64, 8),
    "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "I16": (torch.int16, 2), "I32": (torch.int32, 4),
    "I64": (torch.int64, 8), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


def load_file(path):
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) != 8:
            raise RuntimeError(f"{path}: not a safetensors file")
        n = struct.unpack("<Q", head)[0]
        meta = json.loads(f.read(n).decode("utf-8"))
        data = np.frombuffer(f.read(), dtype=np.uint8)
    out = {}
    for name, info in meta.items():
        if name == "__metadata__":
            continue
        if info["dtype"] not in _DTYPES:
            raise RuntimeError(f"{path}: tensor {name} has unsupported dtype {info['dtype']}")
        dt, size = _DTYPES[info["dtype"]]
        a, b = info["data_offsets"]
        shape = [int(s) for s in info["shape"]]
        count = int(np.prod(shape)) if shape else 1
        if b - a != count * size or b > data.size:
            raise RuntimeError(f"{path}: tensor {name} does not fit its byte range")
        raw = torch.from_numpy(data[a:b].copy())
        out[name] = raw.view(dt).reshape(shape)
    return out


def save_file(tensors, path):
    meta, blobs, off = {}, [], 0
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        meta[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    head = json.dumps(meta, separators=(",", ":")).encode("utf-8")
    head += b" " * (-len(head) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(head)))
        f.write(head)
        for raw in blobs:
            f.write(raw)
