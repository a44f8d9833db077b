"""PyTorch ``.bin`` / ``.pt`` checkpoints (zip archive + pickle) read without executing arbitrary code.

Reference parity: pure-Rust zip + pickle reader (src/loader/pytorch.rs). Here the pickle is interpreted by a
restricted unpickler that only rebuilds tensors (``torch._utils._rebuild_tensor_v2`` over typed storages) and
plain containers; any other global raises.
"""
from __future__ import annotations

import pickle
import zipfile
from collections import OrderedDict
from typing import Dict

import numpy as np
import torch

from .loader import TensorProvider
from .name_map import match_tensor_role

_STORAGE_DTYPES = {
    "FloatStorage": torch.float32, "HalfStorage": torch.float16, "BFloat16Storage": torch.bfloat16,
    "DoubleStorage": torch.float64, "LongStorage": torch.int64, "IntStorage": torch.int32,
    "ShortStorage": torch.int16, "CharStorage": torch.int8, "ByteStorage": torch.uint8, "BoolStorage": torch.bool,
}


class _StorageType:
    def __init__(self, dtype):
        self.dtype = dtype


def _rebuild_tensor_v2(storage, storage_offset, size, stride, requires_grad=False, backward_hooks=None, metadata=None):
    if len(size) == 0:
        return storage[storage_offset:storage_offset + 1].reshape(())
    return torch.as_strided(storage, tuple(size), tuple(stride), storage_offset)


class _Unpickler(pickle.Unpickler):
    def __init__(self, f, zf, prefix):
        super().__init__(f)
        self.zf, self.prefix = zf, prefix

    def find_class(self, module, name):
        if module == "collections" and name == "OrderedDict":
            return OrderedDict
        if module == "torch._utils" and name in ("_rebuild_tensor_v2", "_rebuild_tensor"):
            return _rebuild_tensor_v2
        if module == "torch" and name in _STORAGE_DTYPES:
            return _StorageType(_STORAGE_DTYPES[name])
        if module == "torch._utils" and name == "_rebuild_parameter":
            return lambda data, requires_grad, hooks: data
        raise pickle.UnpicklingError(f"refusing to load global {module}.{name}")

    def persistent_load(self, pid):
        # ('storage', storage_type, key, location, numel)
        _, st, key, _, numel = pid
        dtype = st.dtype if isinstance(st, _StorageType) else torch.float32
        raw = self.zf.read(f"{self.prefix}/data/{key}")
        return torch.frombuffer(bytearray(raw), dtype=dtype, count=numel) if numel else torch.empty(0, dtype=dtype)


def load_state_dict(path) -> Dict[str, torch.Tensor]:
    with zipfile.ZipFile(path) as zf:
        pkl = next(n for n in zf.namelist() if n.endswith("data.pkl"))
        prefix = pkl.rsplit("/", 1)[0]
        with zf.open(pkl) as f:
            obj = _Unpickler(f, zf, prefix).load()
    if isinstance(obj, dict) and "state_dict" in obj and isinstance(obj["state_dict"], dict):
        obj = obj["state_dict"]
    return {k: v for k, v in obj.items() if isinstance(v, torch.Tensor)}


class PytorchProvider(TensorProvider):
    def __init__(self, files, dtype=torch.bfloat16):
        super().__init__()
        self.dtype = dtype
        self.tensors: Dict[str, torch.Tensor] = {}
        for f in files:
            self.tensors.update(load_state_dict(f))
        for n, t in self.tensors.items():
            self.shapes[n] = tuple(t.shape)
            canon = match_tensor_role(n)[2]
            if canon:
                self.canon_to_external[canon] = n

    def get(self, name):
        t = self.tensors[self.canon_to_external[name]]
        if name.rsplit(".", 1)[-1].endswith("norm"):
            return t.float()
        return t.to(self.dtype) if t.is_floating_point() else t
