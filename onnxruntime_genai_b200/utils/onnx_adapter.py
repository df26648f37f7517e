"""Reader and writer for `.onnx_adapter` files (the LoRA adapter container that the reference loads through
OrtLoraAdapter, src/models/adapters.cpp:10-87, and that its tests write with onnxruntime.AdapterFormat,
test/python/test_onnxruntime_genai_api.py:785-800).

The container is a FlatBuffers file with the schema

    table Parameter { name:string; dims:[int64]; data_type:int32 (ONNX TensorProto.DataType); raw_data:[ubyte] (force_align: 8); }
    table Adapter   { format_version:int; adapter_version:int; model_version:int; parameters:[Parameter]; }
    root_type Adapter;

There is no flatbuffers package in this environment, and only this one schema is needed, so the few rules of the wire format
are applied directly: a table starts with a signed offset back to its vtable (u16 vtable size, u16 table size, one u16 offset per
field, 0 = absent), scalars are stored inline, strings / vectors / tables are reached through unsigned 32-bit offsets relative to
the position of the offset itself, vectors and strings are prefixed by a u32 element count.
"""
from __future__ import annotations

import struct
from typing import Dict, Tuple

import numpy as np

# ONNX TensorProto.DataType -> numpy dtype (bfloat16 is carried as uint16 and flagged)
_ONNX_TO_NP = {1: np.float32, 2: np.uint8, 3: np.int8, 4: np.uint16, 5: np.int16, 6: np.int32, 7: np.int64, 9: np.bool_, 10: np.float16,
               11: np.float64, 12: np.uint32, 13: np.uint64, 16: np.uint16}
_NP_TO_ONNX = {np.dtype(np.float32): 1, np.dtype(np.uint8): 2, np.dtype(np.int8): 3, np.dtype(np.int16): 5, np.dtype(np.int32): 6,
               np.dtype(np.int64): 7, np.dtype(np.bool_): 9, np.dtype(np.float16): 10, np.dtype(np.float64): 11}
BFLOAT16 = 16
FORMAT_VERSION = 1


class _Reader:
    def __init__(self, buf: bytes):
        self.b = memoryview(buf)

    def u16(self, p): return struct.unpack_from("<H", self.b, p)[0]
    def i32(self, p): return struct.unpack_from("<i", self.b, p)[0]
    def u32(self, p): return struct.unpack_from("<I", self.b, p)[0]

    def field(self, table: int, index: int) -> int:
        """Position of field `index` of the table at `table`, 0 when absent."""
        vt = table - self.i32(table)
        if 4 + 2 * index >= self.u16(vt):
            return 0
        off = self.u16(vt + 4 + 2 * index)
        return table + off if off else 0

    def indirect(self, p: int) -> int:
        return p + self.u32(p)

    def scalar_i32(self, table, index, default=0):
        p = self.field(table, index)
        return self.i32(p) if p else default

    def vector(self, table, index) -> Tuple[int, int]:
        """(position of the first element, element count)"""
        p = self.field(table, index)
        if not p:
            return 0, 0
        v = self.indirect(p)
        return v + 4, self.u32(v)


def read_adapter(path: str) -> Tuple[Dict[str, Tuple[np.ndarray, int]], Dict[str, int]]:
    """-> ({parameter name: (array, onnx data type)}, {format_version, adapter_version, model_version}).
    bfloat16 parameters come back as uint16 arrays with data type 16."""
    with open(path, "rb") as f:
        buf = f.read()
    if len(buf) < 16:
        raise RuntimeError(f"{path}: not an adapter file (too short)")
    r = _Reader(buf)
    try:
        root = r.indirect(0)
        meta = {"format_version": r.scalar_i32(root, 0), "adapter_version": r.scalar_i32(root, 1), "model_version": r.scalar_i32(root, 2)}
        first, count = r.vector(root, 3)
        out: Dict[str, Tuple[np.ndarray, int]] = {}
        for i in range(count):
            t = r.indirect(first + 4 * i)
            np_, n = r.vector(t, 0)
            name = bytes(r.b[np_:np_ + n]).decode("utf-8")
            dp, dn = r.vector(t, 1)
            dims = list(struct.unpack_from(f"<{dn}q", r.b, dp)) if dn else []
            dtype = r.scalar_i32(t, 2)
            rp, rn = r.vector(t, 3)
            if dtype not in _ONNX_TO_NP:
                raise RuntimeError(f"{path}: parameter {name} has unsupported data type {dtype}")
            arr = np.frombuffer(bytes(r.b[rp:rp + rn]), dtype=_ONNX_TO_NP[dtype])
            want = int(np.prod(dims)) if dims else arr.size
            if arr.size != want:
                raise RuntimeError(f"{path}: parameter {name}: {arr.size} elements for shape {dims}")
            out[name] = (arr.reshape(dims) if (dims or arr.size == 1) else arr, dtype)
    except (struct.error, IndexError, ValueError) as e:
        raise RuntimeError(f"{path}: malformed adapter file ({e})") from None
    return out, meta


def write_adapter(path: str, parameters: Dict[str, np.ndarray], adapter_version: int = 1, model_version: int = 1,
                  bfloat16: Tuple[str, ...] = ()) -> None:
    """Writes the parameters (name -> array) in the same container.  Names listed in `bfloat16` hold uint16 arrays that are to be
    tagged as bfloat16."""
    names = list(parameters)
    n = len(names)
    out = bytearray()

    def pad(align):
        while len(out) % align:
            out.append(0)

    def put(fmt, *v):
        out.extend(struct.pack(fmt, *v))

    # ---- header: root offset (patched below) + an identifier slot (ignored by readers that do not ask for one)
    put("<I", 0)
    out.extend(b"OGAD")
    # ---- Adapter: vtable (4 fields) then the table
    pad(4)
    vt = len(out)
    put("<HHHHHH", 12, 20, 4, 8, 12, 16)
    pad(4)
    root = len(out)
    put("<i", root - vt)
    put("<iii", FORMAT_VERSION, adapter_version, model_version)
    params_ref = len(out)
    put("<I", 0)
    struct.pack_into("<I", out, 0, root)
    # ---- vector of parameter tables
    pad(4)
    vec = len(out)
    struct.pack_into("<I", out, params_ref, vec - params_ref)
    put("<I", n)
    elem = len(out)
    out.extend(b"\0" * (4 * n))
    refs = []
    for i, name in enumerate(names):
        pad(4)
        pvt = len(out)
        put("<HHHHHH", 12, 20, 4, 8, 12, 16)
        pad(4)
        t = len(out)
        struct.pack_into("<I", out, elem + 4 * i, t - (elem + 4 * i))
        put("<i", t - pvt)
        arr = np.require(parameters[name], requirements="C")       # (ascontiguousarray would turn a scalar into a vector)
        dtype = BFLOAT16 if name in bfloat16 else _NP_TO_ONNX.get(arr.dtype)
        if dtype is None:
            raise RuntimeError(f"parameter {name}: unsupported dtype {arr.dtype}")
        name_ref = len(out); put("<I", 0)
        dims_ref = len(out); put("<I", 0)
        put("<i", dtype)
        raw_ref = len(out); put("<I", 0)
        refs.append((name, arr, name_ref, dims_ref, raw_ref))
    for name, arr, name_ref, dims_ref, raw_ref in refs:
        pad(4)
        struct.pack_into("<I", out, name_ref, len(out) - name_ref)
        nb = name.encode("utf-8")
        put("<I", len(nb)); out.extend(nb); out.append(0)
        # int64 elements: the element data (after the 4-byte count) is 8-byte aligned
        while (len(out) + 4) % 8:
            out.append(0)
        struct.pack_into("<I", out, dims_ref, len(out) - dims_ref)
        put("<I", arr.ndim)
        for d in arr.shape:
            put("<q", int(d))
        while (len(out) + 4) % 8:
            out.append(0)
        struct.pack_into("<I", out, raw_ref, len(out) - raw_ref)
        raw = arr.tobytes()
        put("<I", len(raw)); out.extend(raw)
    with open(path, "wb") as f:
        f.write(bytes(out))
