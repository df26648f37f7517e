"""Minimal ONNX protobuf wire-format codec (no `onnx` package needed).

The checkpoint format is a directory holding `genai_config.json`, `model.onnx`
and one external-data file `model.onnx.data` (reference:
src/python/py/models/builders/base.py:1418-1459).  This runtime does not
interpret ONNX graphs; it uses the file as a *weight container plus
architecture descriptor*: initializer names / dtypes / shapes / external-data
offsets, and a handful of node attributes (MatMulNBits K/N/bits/block_size,
GroupQueryAttention num_heads/kv_num_heads/local_window_size/scale/softcap,
MoE k/activation...).  Only the messages needed for that are implemented:
ModelProto, GraphProto, NodeProto, AttributeProto, TensorProto,
ValueInfoProto, TypeProto, OperatorSetIdProto.

Field numbers follow the public onnx.proto3 schema.
"""
from __future__ import annotations

import mmap
import os
import struct
from dataclasses import dataclass, field
from typing import Any, Dict, Iterator, List, Optional, Tuple

import numpy as np

# --------------------------------------------------------------------------- dtypes
FLOAT, UINT8, INT8, UINT16, INT16, INT32, INT64, STRING, BOOL = 1, 2, 3, 4, 5, 6, 7, 8, 9
FLOAT16, DOUBLE, UINT32, UINT64 = 10, 11, 12, 13
BFLOAT16 = 16
FLOAT8E4M3FN = 17
UINT4, INT4 = 21, 22

_NP_OF = {
    FLOAT: np.float32, UINT8: np.uint8, INT8: np.int8, UINT16: np.uint16, INT16: np.int16,
    INT32: np.int32, INT64: np.int64, BOOL: np.bool_, FLOAT16: np.float16, DOUBLE: np.float64,
    UINT32: np.uint32, UINT64: np.uint64,
    BFLOAT16: np.uint16,  # carried as raw 16-bit words
    FLOAT8E4M3FN: np.uint8,
}
_ITEMSIZE = {k: np.dtype(v).itemsize for k, v in _NP_OF.items()}


def numpy_dtype(onnx_dtype: int):
    return _NP_OF[onnx_dtype]


def itemsize(onnx_dtype: int) -> int:
    return _ITEMSIZE[onnx_dtype]


# --------------------------------------------------------------------------- wire primitives
def _enc_varint(v: int) -> bytes:
    if v < 0:
        v += 1 << 64
    out = bytearray()
    while True:
        b = v & 0x7F
        v >>= 7
        if v:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


def _dec_varint(buf, pos: int) -> Tuple[int, int]:
    result = 0
    shift = 0
    while True:
        b = buf[pos]
        pos += 1
        result |= (b & 0x7F) << shift
        if not (b & 0x80):
            return result, pos
        shift += 7


def _signed(v: int) -> int:
    return v - (1 << 64) if v >= (1 << 63) else v


def _tag(field_no: int, wire: int) -> bytes:
    return _enc_varint((field_no << 3) | wire)


def _f_varint(field_no: int, v: int) -> bytes:
    return _tag(field_no, 0) + _enc_varint(v)


def _f_bytes(field_no: int, b: bytes) -> bytes:
    return _tag(field_no, 2) + _enc_varint(len(b)) + b


def _f_str(field_no: int, s: str) -> bytes:
    return _f_bytes(field_no, s.encode("utf-8"))


def _f_float(field_no: int, v: float) -> bytes:
    return _tag(field_no, 5) + struct.pack("<f", v)


def _iter_fields(buf, start: int = 0, end: Optional[int] = None) -> Iterator[Tuple[int, int, Any]]:
    """Yield (field_no, wire_type, value); length-delimited values are (start, end) spans."""
    pos = start
    end = len(buf) if end is None else end
    while pos < end:
        key, pos = _dec_varint(buf, pos)
        fno, wire = key >> 3, key & 7
        if wire == 0:
            v, pos = _dec_varint(buf, pos)
            yield fno, wire, v
        elif wire == 1:
            yield fno, wire, bytes(buf[pos:pos + 8])
            pos += 8
        elif wire == 2:
            ln, pos = _dec_varint(buf, pos)
            yield fno, wire, (pos, pos + ln)
            pos += ln
        elif wire == 5:
            yield fno, wire, bytes(buf[pos:pos + 4])
            pos += 4
        else:
            raise ValueError(f"unsupported protobuf wire type {wire}")


# --------------------------------------------------------------------------- data model
@dataclass
class Tensor:
    name: str
    dtype: int
    dims: Tuple[int, ...]
    raw: Optional[bytes] = None  # inline payload
    ext_location: Optional[str] = None  # external file name (relative)
    ext_offset: int = 0
    ext_length: int = 0

    @property
    def nbytes(self) -> int:
        n = 1
        for d in self.dims:
            n *= d
        return n * itemsize(self.dtype)


@dataclass
class Attribute:
    name: str
    value: Any  # int | float | bytes/str | list | Tensor


@dataclass
class Node:
    op_type: str
    name: str = ""
    inputs: List[str] = field(default_factory=list)
    outputs: List[str] = field(default_factory=list)
    domain: str = ""
    attrs: Dict[str, Any] = field(default_factory=dict)


@dataclass
class ValueInfo:
    name: str
    dtype: int
    shape: Tuple[Any, ...]  # ints or symbolic strings


@dataclass
class Model:
    graph_name: str = "main_graph"
    ir_version: int = 10
    producer_name: str = "onnxruntime_genai_b200"
    opsets: Dict[str, int] = field(default_factory=lambda: {"": 21, "com.microsoft": 1})
    nodes: List[Node] = field(default_factory=list)
    initializers: Dict[str, Tensor] = field(default_factory=dict)
    inputs: List[ValueInfo] = field(default_factory=list)
    outputs: List[ValueInfo] = field(default_factory=list)


# --------------------------------------------------------------------------- encoding
def _enc_tensor(t: Tensor) -> bytes:
    out = bytearray()
    for d in t.dims:
        out += _f_varint(1, int(d))
    out += _f_varint(2, t.dtype)
    out += _f_str(8, t.name)
    if t.ext_location is not None:
        for k, v in (("location", t.ext_location), ("offset", str(t.ext_offset)), ("length", str(t.ext_length))):
            out += _f_bytes(13, _f_str(1, k) + _f_str(2, v))
        out += _f_varint(14, 1)
    else:
        out += _f_bytes(9, t.raw or b"")
    return bytes(out)


def _enc_attr(name: str, v: Any) -> bytes:
    out = bytearray(_f_str(1, name))
    if isinstance(v, bool):
        out += _f_varint(3, int(v)) + _f_varint(20, 2)
    elif isinstance(v, int):
        out += _f_varint(3, v) + _f_varint(20, 2)
    elif isinstance(v, float):
        out += _f_float(2, v) + _f_varint(20, 1)
    elif isinstance(v, (str, bytes)):
        b = v.encode() if isinstance(v, str) else v
        out += _f_bytes(4, b) + _f_varint(20, 3)
    elif isinstance(v, Tensor):
        out += _f_bytes(5, _enc_tensor(v)) + _f_varint(20, 4)
    elif isinstance(v, (list, tuple)):
        if all(isinstance(x, int) for x in v):
            for x in v:
                out += _f_varint(8, x)
            out += _f_varint(20, 7)
        elif all(isinstance(x, (int, float)) for x in v):
            for x in v:
                out += _f_float(7, float(x))
            out += _f_varint(20, 6)
        else:
            for x in v:
                out += _f_bytes(9, x.encode() if isinstance(x, str) else x)
            out += _f_varint(20, 8)
    else:
        raise TypeError(f"attribute {name}: unsupported value {type(v)}")
    return bytes(out)


def _enc_value_info(vi: ValueInfo) -> bytes:
    shape = bytearray()
    for d in vi.shape:
        if isinstance(d, int):
            shape += _f_bytes(1, _f_varint(1, d))
        else:
            shape += _f_bytes(1, _f_str(2, str(d)))
    tensor_type = _f_varint(1, vi.dtype) + _f_bytes(2, bytes(shape))
    return _f_str(1, vi.name) + _f_bytes(2, _f_bytes(1, tensor_type))


def _enc_node(n: Node) -> bytes:
    out = bytearray()
    for s in n.inputs:
        out += _f_str(1, s)
    for s in n.outputs:
        out += _f_str(2, s)
    out += _f_str(3, n.name) + _f_str(4, n.op_type)
    for k, v in n.attrs.items():
        out += _f_bytes(5, _enc_attr(k, v))
    if n.domain:
        out += _f_str(7, n.domain)
    return bytes(out)


def encode_model(m: Model) -> bytes:
    g = bytearray()
    for n in m.nodes:
        g += _f_bytes(1, _enc_node(n))
    g += _f_str(2, m.graph_name)
    for t in m.initializers.values():
        g += _f_bytes(5, _enc_tensor(t))
    for vi in m.inputs:
        g += _f_bytes(11, _enc_value_info(vi))
    for vi in m.outputs:
        g += _f_bytes(12, _enc_value_info(vi))
    out = bytearray(_f_varint(1, m.ir_version) + _f_str(2, m.producer_name))
    out += _f_bytes(7, bytes(g))
    for dom, ver in m.opsets.items():
        out += _f_bytes(8, _f_str(1, dom) + _f_varint(2, ver))
    return bytes(out)


# --------------------------------------------------------------------------- decoding
def _dec_tensor(buf, s: int, e: int) -> Tensor:
    dims: List[int] = []
    dtype = 0
    name = ""
    raw = None
    ext: Dict[str, str] = {}
    external = False
    typed: Optional[np.ndarray] = None
    for fno, wire, v in _iter_fields(buf, s, e):
        if fno == 1:
            if wire == 0:
                dims.append(_signed(v))
            else:  # packed
                p, pe = v
                while p < pe:
                    d, p = _dec_varint(buf, p)
                    dims.append(_signed(d))
        elif fno == 2:
            dtype = v
        elif fno == 8:
            name = bytes(buf[v[0]:v[1]]).decode()
        elif fno == 9:
            raw = bytes(buf[v[0]:v[1]])
        elif fno == 13:
            k = val = ""
            for f2, _, v2 in _iter_fields(buf, v[0], v[1]):
                if f2 == 1:
                    k = bytes(buf[v2[0]:v2[1]]).decode()
                elif f2 == 2:
                    val = bytes(buf[v2[0]:v2[1]]).decode()
            ext[k] = val
        elif fno == 14:
            external = v == 1
        elif fno == 4 and wire == 2:  # packed float_data
            typed = np.frombuffer(bytes(buf[v[0]:v[1]]), dtype="<f4")
        elif fno == 7 and wire == 2:  # packed int64_data
            vals = []
            p, pe = v
            while p < pe:
                d, p = _dec_varint(buf, p)
                vals.append(_signed(d))
            typed = np.asarray(vals, dtype=np.int64)
        elif fno == 5 and wire == 2:  # packed int32_data
            vals = []
            p, pe = v
            while p < pe:
                d, p = _dec_varint(buf, p)
                vals.append(_signed(d))
            typed = np.asarray(vals, dtype=np.int64)
    t = Tensor(name=name, dtype=dtype, dims=tuple(dims))
    if external or ext:
        t.ext_location = ext.get("location")
        t.ext_offset = int(ext.get("offset", "0"))
        t.ext_length = int(ext.get("length", str(t.nbytes)))
    elif raw is not None:
        t.raw = raw
    elif typed is not None:
        t.raw = typed.astype(numpy_dtype(dtype)).tobytes()
    else:
        t.raw = b""
    return t


def _dec_attr(buf, s: int, e: int) -> Tuple[str, Any]:
    name = ""
    atype = 0
    f = i = None
    sbytes = None
    tensor = None
    floats: List[float] = []
    ints: List[int] = []
    strings: List[bytes] = []
    for fno, wire, v in _iter_fields(buf, s, e):
        if fno == 1:
            name = bytes(buf[v[0]:v[1]]).decode()
        elif fno == 2:
            f = struct.unpack("<f", v)[0]
        elif fno == 3:
            i = _signed(v)
        elif fno == 4:
            sbytes = bytes(buf[v[0]:v[1]])
        elif fno == 5:
            tensor = _dec_tensor(buf, v[0], v[1])
        elif fno == 7:
            if wire == 5:
                floats.append(struct.unpack("<f", v)[0])
            else:
                floats.extend(np.frombuffer(bytes(buf[v[0]:v[1]]), dtype="<f4").tolist())
        elif fno == 8:
            if wire == 0:
                ints.append(_signed(v))
            else:
                p, pe = v
                while p < pe:
                    d, p = _dec_varint(buf, p)
                    ints.append(_signed(d))
        elif fno == 9:
            strings.append(bytes(buf[v[0]:v[1]]))
        elif fno == 20:
            atype = v
    if atype == 1 or (atype == 0 and f is not None):
        return name, f
    if atype == 2 or (atype == 0 and i is not None):
        return name, i
    if atype == 3 or (atype == 0 and sbytes is not None):
        try:
            return name, sbytes.decode()
        except UnicodeDecodeError:
            return name, sbytes
    if atype == 4:
        return name, tensor
    if atype == 6:
        return name, floats
    if atype == 7:
        return name, ints
    if atype == 8:
        return name, [x.decode(errors="replace") for x in strings]
    return name, None


def _dec_node(buf, s: int, e: int) -> Node:
    n = Node(op_type="")
    for fno, _, v in _iter_fields(buf, s, e):
        if fno == 1:
            n.inputs.append(bytes(buf[v[0]:v[1]]).decode())
        elif fno == 2:
            n.outputs.append(bytes(buf[v[0]:v[1]]).decode())
        elif fno == 3:
            n.name = bytes(buf[v[0]:v[1]]).decode()
        elif fno == 4:
            n.op_type = bytes(buf[v[0]:v[1]]).decode()
        elif fno == 5:
            k, val = _dec_attr(buf, v[0], v[1])
            n.attrs[k] = val
        elif fno == 7:
            n.domain = bytes(buf[v[0]:v[1]]).decode()
    return n


def _dec_value_info(buf, s: int, e: int) -> ValueInfo:
    name = ""
    dtype = 0
    shape: List[Any] = []
    for fno, _, v in _iter_fields(buf, s, e):
        if fno == 1:
            name = bytes(buf[v[0]:v[1]]).decode()
        elif fno == 2:
            for f2, _, v2 in _iter_fields(buf, v[0], v[1]):
                if f2 != 1:
                    continue
                for f3, _, v3 in _iter_fields(buf, v2[0], v2[1]):
                    if f3 == 1:
                        dtype = v3
                    elif f3 == 2:
                        for f4, _, v4 in _iter_fields(buf, v3[0], v3[1]):
                            if f4 != 1:
                                continue
                            dim: Any = "?"
                            for f5, _, v5 in _iter_fields(buf, v4[0], v4[1]):
                                if f5 == 1:
                                    dim = _signed(v5)
                                elif f5 == 2:
                                    dim = bytes(buf[v5[0]:v5[1]]).decode()
                            shape.append(dim)
    return ValueInfo(name, dtype, tuple(shape))


def decode_model(buf) -> Model:
    m = Model(opsets={})
    for fno, _, v in _iter_fields(buf):
        if fno == 1:
            m.ir_version = v
        elif fno == 2:
            m.producer_name = bytes(buf[v[0]:v[1]]).decode()
        elif fno == 8:
            dom, ver = "", 0
            for f2, _, v2 in _iter_fields(buf, v[0], v[1]):
                if f2 == 1:
                    dom = bytes(buf[v2[0]:v2[1]]).decode()
                elif f2 == 2:
                    ver = v2
            m.opsets[dom] = ver
        elif fno == 7:
            for f2, _, v2 in _iter_fields(buf, v[0], v[1]):
                if f2 == 1:
                    m.nodes.append(_dec_node(buf, v2[0], v2[1]))
                elif f2 == 2:
                    m.graph_name = bytes(buf[v2[0]:v2[1]]).decode()
                elif f2 == 5:
                    t = _dec_tensor(buf, v2[0], v2[1])
                    m.initializers[t.name] = t
                elif f2 == 11:
                    m.inputs.append(_dec_value_info(buf, v2[0], v2[1]))
                elif f2 == 12:
                    m.outputs.append(_dec_value_info(buf, v2[0], v2[1]))
    return m


# --------------------------------------------------------------------------- file helpers
class ExternalDataWriter:
    """Appends tensors to one external-data file with 64-byte aligned offsets."""

    ALIGN = 64

    def __init__(self, path: str):
        self.path = path
        self.location = os.path.basename(path)
        self._f = open(path, "wb")
        self._pos = 0

    def add(self, name: str, dtype: int, arr: np.ndarray, dims=None) -> Tensor:
        data = np.ascontiguousarray(arr)
        pad = (-self._pos) % self.ALIGN
        if pad:
            self._f.write(b"\0" * pad)
            self._pos += pad
        off = self._pos
        mv = memoryview(data).cast("B")
        self._f.write(mv)
        self._pos += len(mv)
        return Tensor(name=name, dtype=dtype, dims=tuple(dims if dims is not None else data.shape),
                      ext_location=self.location, ext_offset=off, ext_length=len(mv))

    def close(self):
        self._f.close()


def save_model(m: Model, path: str) -> None:
    with open(path, "wb") as f:
        f.write(encode_model(m))


class LoadedModel:
    """A decoded model plus mmap'ed access to its external-data files."""

    def __init__(self, path: str):
        self.path = path
        self.dir = os.path.dirname(os.path.abspath(path))
        with open(path, "rb") as f:
            self.model = decode_model(f.read())
        self._maps: Dict[str, mmap.mmap] = {}

    def _map(self, location: str) -> mmap.mmap:
        if os.path.isabs(location) or ".." in location.replace("\\", "/").split("/"):
            raise ValueError(f"external data location must be a relative path inside the model dir: {location}")
        mm = self._maps.get(location)
        if mm is None:
            with open(os.path.join(self.dir, location), "rb") as f:
                mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
            self._maps[location] = mm
        return mm

    def names(self) -> List[str]:
        return list(self.model.initializers)

    def has(self, name: str) -> bool:
        return name in self.model.initializers

    def info(self, name: str) -> Tensor:
        return self.model.initializers[name]

    def array(self, name: str) -> np.ndarray:
        """Return a read-only numpy view (zero copy for external data)."""
        t = self.model.initializers[name]
        npdt = numpy_dtype(t.dtype)
        if t.ext_location is not None:
            mm = self._map(t.ext_location)
            arr = np.frombuffer(mm, dtype=npdt, count=t.ext_length // np.dtype(npdt).itemsize, offset=t.ext_offset)
        else:
            arr = np.frombuffer(t.raw, dtype=npdt)
        return arr.reshape(t.dims) if t.dims else arr.reshape(())

    def close(self):
        for mm in self._maps.values():
            try:
                mm.close()
            except BufferError:
                pass  # numpy views still alive; the map closes with them
        self._maps.clear()
