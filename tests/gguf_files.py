"""Test-side GGUF writer: lays a file out the way the reference's GGUFTest builds its fixtures
(warpforge-data/src/test/java/io/surfworks/warpforge/data/format/GGUFTest.java: magic, version,
counts, key/values, tensor infos, padding to the alignment, tensor data), with the knobs the
parser tests need (format version, custom alignment, raw overrides for corrupt files)."""
import struct

MAGIC = 0x46554747
T_U8, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STR, T_ARR, T_U64, T_I64, T_F64 = range(13)
_SCALAR = {T_U8: "<B", T_I8: "<b", T_U16: "<H", T_I16: "<h", T_U32: "<I", T_I32: "<i", T_F32: "<f", T_BOOL: "<B",
           T_U64: "<Q", T_I64: "<q", T_F64: "<d"}


def _string(s: str, version: int) -> bytes:
    b = s.encode()
    return struct.pack("<Q" if version >= 2 else "<I", len(b)) + b


def _value(vtype: int, value, version: int) -> bytes:
    if vtype == T_STR:
        return _string(value, version)
    if vtype == T_ARR:
        etype, items = value
        out = struct.pack("<I", etype) + struct.pack("<Q" if version >= 2 else "<I", len(items))
        return out + b"".join(_value(etype, v, version) for v in items)
    return struct.pack(_SCALAR[vtype], value)


def gguf_bytes(tensors, metadata=(), version=3, alignment=None, magic=MAGIC):
    """tensors: [(name, dims, ggml_type, data bytes)], dims in file order (dims[0] fastest);
    metadata: [(key, value type, value)].  Returns (file bytes, data offset, {name: offset})."""
    align = 32
    meta = list(metadata)
    if alignment is not None:
        meta.append(("general.alignment", T_U32, alignment))
        align = alignment
    head = struct.pack("<IIqq", magic, version, len(tensors), len(meta))
    for key, vtype, value in meta:
        head += _string(key, version) + struct.pack("<I", vtype) + _value(vtype, value, version)
    offsets, off = {}, 0
    for name, dims, ggml_type, data in tensors:
        off = (off + align - 1) // align * align
        offsets[name] = off
        head += _string(name, version) + struct.pack("<i", len(dims)) + b"".join(struct.pack("<q", d) for d in dims)
        head += struct.pack("<iq", ggml_type, off)
        off += len(data)
    data_offset = (len(head) + align - 1) // align * align
    body = bytearray(off)
    for name, dims, ggml_type, data in tensors:
        body[offsets[name]:offsets[name] + len(data)] = data
    return head + b"\0" * (data_offset - len(head)) + bytes(body), data_offset, offsets


def write_gguf(path, tensors, metadata=(), version=3, alignment=None, magic=MAGIC):
    blob, data_offset, offsets = gguf_bytes(tensors, metadata, version, alignment, magic)
    with open(path, "wb") as f:
        f.write(blob)
    return data_offset, offsets
