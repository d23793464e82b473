"""Reading and writing the safetensors container: 8 bytes of little-endian
header length, a JSON header {name: {dtype, shape, data_offsets}}, then the
tensors' bytes.  Tensors come back as CPU torch tensors that view a memory map
of the file, in the dtype the file stores."""
from __future__ import annotations

import json
import os
import struct
import warnings
from typing import Dict

import numpy as np
import torch


class WeightError(ValueError):
    """A weight file that is malformed or does not fit the model."""


# file dtype -> (numpy dtype of the raw bytes, torch dtype to view them as)
_FILE_DTYPES = {
    "BF16": (np.uint16, torch.bfloat16),
    "F16": (np.float16, torch.float16),
    "F32": (np.float32, torch.float32),
    "F64": (np.float64, torch.float64),
    "I64": (np.int64, torch.int64),
    "I32": (np.int32, torch.int32),
    "I16": (np.int16, torch.int16),
    "I8": (np.int8, torch.int8),
    "U8": (np.uint8, torch.uint8),
    "BOOL": (np.bool_, torch.bool),
}
_TORCH_TO_FILE = {torch_dtype: name for name, (_, torch_dtype) in _FILE_DTYPES.items()}


def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    try:
        size = os.path.getsize(path)
    except OSError:
        raise WeightError(f"{path} does not exist") from None
    if size < 8:
        raise WeightError(f"{path} is too short to be a safetensors file")
    with open(path, "rb") as fh:
        (header_len,) = struct.unpack("<Q", fh.read(8))
        if header_len > size - 8:
            raise WeightError(f"{path}: header length {header_len} exceeds the file")
        try:
            header = json.loads(fh.read(header_len))
        except (json.JSONDecodeError, UnicodeDecodeError) as err:
            raise WeightError(f"{path}: header is not JSON ({err})") from None
    data_start = 8 + header_len
    raw = np.memmap(path, dtype=np.uint8, mode="r", offset=data_start) if size > data_start \
        else np.zeros(0, dtype=np.uint8)
    tensors: Dict[str, torch.Tensor] = {}
    for name, entry in header.items():
        if name == "__metadata__":
            continue
        if entry["dtype"] not in _FILE_DTYPES:
            raise WeightError(f"{path}: tensor {name} has unsupported dtype {entry['dtype']}")
        np_dtype, torch_dtype = _FILE_DTYPES[entry["dtype"]]
        begin, end = entry["data_offsets"]
        shape = tuple(entry["shape"])
        count = int(np.prod(shape, dtype=np.int64)) if shape else 1
        if end - begin != count * np.dtype(np_dtype).itemsize or end > raw.size:
            raise WeightError(f"{path}: tensor {name} has {end - begin} bytes for shape {shape}")
        array = np.frombuffer(raw, dtype=np_dtype, count=count, offset=begin)
        if count == 0 or begin % np.dtype(np_dtype).itemsize:
            array = array.copy()
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)  # the map is read-only by design
            tensor = torch.from_numpy(array)
        if torch_dtype == torch.bfloat16:
            tensor = tensor.view(torch.bfloat16)
        tensors[name] = tensor.reshape(shape)
    return tensors


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor]) -> None:
    header = {}
    offset = 0
    flats = []
    for name in sorted(tensors):
        tensor = tensors[name].detach().cpu().contiguous()
        if tensor.dtype not in _TORCH_TO_FILE:
            raise WeightError(f"tensor {name}: dtype {tensor.dtype} cannot be stored")
        flat = tensor.reshape(-1)
        if tensor.dtype == torch.bfloat16:
            flat = flat.view(torch.int16)
        size = flat.numel() * flat.element_size()
        header[name] = {
            "dtype": _TORCH_TO_FILE[tensor.dtype],
            "shape": list(tensor.shape),
            "data_offsets": [offset, offset + size],
        }
        offset += size
        flats.append(flat)
    encoded = json.dumps(header, separators=(",", ":")).encode()
    encoded += b" " * (-len(encoded) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as fh:
        fh.write(struct.pack("<Q", len(encoded)))
        fh.write(encoded)
        for flat in flats:
            if flat.numel():
                fh.write(memoryview(flat.numpy()).cast("B"))     # straight from the tensor's memory
    os.replace(tmp, path)
