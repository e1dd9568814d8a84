"""GGUF file reader over the native library: host-side mirror of the reference's
``GGUF`` class (warpforge-data/src/main/java/io/surfworks/warpforge/data/format/GGUF.java):
``open`` / ``version`` / ``tensor_names`` / ``tensor_info`` / ``tensor`` / ``metadata`` /
``close`` keep the reference's names, argument meaning and failures (``GGUFFormatError`` where
the reference throws ``IOException``, ``KeyError`` -> ``ValueError("No tensor named: ...")``
for an unknown tensor).  Parsing and the memory mapping live in the library
(``wf_gguf_*``); nothing here reads the file itself.  ``upload`` hands a quantized tensor
from the mapping to the device without copying it through Python.
"""
from __future__ import annotations

import ctypes
import dataclasses
from typing import Dict, List, Tuple

import numpy as np

from . import _native as N


class GGUFFormatError(IOError):
    pass


@dataclasses.dataclass(frozen=True)
class TensorInfo:
    """GGUF.java:72-94: shape is in file order, shape[0] varies fastest."""

    name: str
    ggml_type: int
    shape: Tuple[int, ...]
    offset: int
    size: int

    def element_count(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n


class GGUF:
    def __init__(self, handle: int, path: str):
        self._lib = N.load()
        self.handle, self.path = handle, path
        v, nt, nm, off, al, fs = ctypes.c_int(), ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int(), ctypes.c_int64()
        N.check("wf_gguf_info", self._lib.wf_gguf_info(handle, ctypes.byref(v), ctypes.byref(nt), ctypes.byref(nm),
                                                       ctypes.byref(off), ctypes.byref(al), ctypes.byref(fs)))
        self._version, self._n_tensors, self._n_meta = v.value, nt.value, nm.value
        self.data_offset, self.alignment, self.file_size = off.value, al.value, fs.value

    @classmethod
    def open(cls, path) -> "GGUF":
        lib = N.load()
        h = ctypes.c_int64()
        err = ctypes.create_string_buffer(512)
        st = lib.wf_gguf_open(str(path).encode(), ctypes.byref(h), err, len(err))
        if st != N.WF_OK:
            raise GGUFFormatError(err.value.decode(errors="replace") or N.error_name(st))
        return cls(h.value, str(path))

    def version(self) -> int:
        return self._version

    def tensor_count(self) -> int:
        return self._n_tensors

    def tensor_names(self) -> List[str]:
        buf = ctypes.create_string_buffer(1024)
        names = []
        for i in range(self._n_tensors):
            N.check("wf_gguf_tensor_name", self._lib.wf_gguf_tensor_name(self.handle, i, buf, len(buf)))
            names.append(buf.value.decode())
        return names

    def has_tensor(self, name: str) -> bool:
        return self._lib.wf_gguf_tensor_info(self.handle, name.encode(), None, None, None, None, None) == N.WF_OK

    def tensor_info(self, name: str) -> TensorInfo:
        t, nd, off, size = ctypes.c_int(), ctypes.c_int(), ctypes.c_int64(), ctypes.c_int64()
        dims = (ctypes.c_int64 * 8)()
        st = self._lib.wf_gguf_tensor_info(self.handle, name.encode(), ctypes.byref(t), ctypes.byref(nd), dims,
                                           ctypes.byref(off), ctypes.byref(size))
        if st == N.WF_ERR_INVALID_ARGUMENT:
            raise ValueError(f"No tensor named: {name}")
        N.check("wf_gguf_tensor_info", st)
        return TensorInfo(name, t.value, tuple(dims[i] for i in range(nd.value)), off.value, size.value)

    def tensor(self, name: str) -> np.ndarray:
        """The tensor's bytes as a read-only view of the mapping (valid until ``close``)."""
        p, size = ctypes.c_void_p(), ctypes.c_int64()
        st = self._lib.wf_gguf_tensor_data(self.handle, name.encode(), ctypes.byref(p), ctypes.byref(size))
        if st == N.WF_ERR_INVALID_ARGUMENT:
            raise ValueError(f"No tensor named: {name}")
        if st == N.WF_ERR_GGUF:
            raise GGUFFormatError(f"tensor {name} lies outside the file")
        N.check("wf_gguf_tensor_data", st)
        if size.value == 0:
            return np.empty(0, np.uint8)
        a = np.ctypeslib.as_array(ctypes.cast(p, ctypes.POINTER(ctypes.c_uint8)), shape=(size.value,))
        a.flags.writeable = False
        return a

    def metadata(self) -> Dict[str, str]:
        key, val = ctypes.create_string_buffer(1024), ctypes.create_string_buffer(4096)
        out = {}
        for i in range(self._n_meta):
            N.check("wf_gguf_metadata", self._lib.wf_gguf_metadata(self.handle, i, key, len(key), val, len(val)))
            out[key.value.decode(errors="replace")] = val.value.decode(errors="replace")
        return out

    def upload(self, context, name: str, shard_rank: int = 0, shard_world: int = 1,
               q4_0_order: int = N.WF_Q4_0_ORDER_REFERENCE):
        """Device-resident row shard of the linear weight ``name`` ({k, n_rows} in the file)."""
        from .backend import QuantizedWeight

        return QuantizedWeight.from_gguf(context, self, name, shard_rank, shard_world, q4_0_order)

    def close(self) -> None:
        if self.handle:
            h, self.handle = self.handle, 0
            N.check("wf_gguf_close", self._lib.wf_gguf_close(h))

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
