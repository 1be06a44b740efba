"""A minimal GGUF writer for the tests: header, typed metadata, tensor infos, aligned tensor data — the layout
Gguf::open reads (crates/ksearch_gguf/src/gguf_impl.rs:216-260).  Test infrastructure only."""
import struct

import numpy as np

# value type ids of the format
U8, I8, U16, I16, U32, I32, F32, BOOL, STR, ARR, U64, I64, F64 = range(13)
_FMT = {U8: "<B", I8: "<b", U16: "<H", I16: "<h", U32: "<I", I32: "<i", F32: "<f", BOOL: "<B", U64: "<Q", I64: "<q", F64: "<d"}


def _gstr(s: str) -> bytes:
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def _scalar(vt: int, v) -> bytes:
    return _gstr(v) if vt == STR else struct.pack(_FMT[vt], v)


def write_gguf(path, metadata, tensors, version=3, alignment=None, magic=0x46554747):
    """metadata: list of (key, value type id, value) — for ARR the value is (element type id, [values]);
    tensors: list of (name, ggml type id, dims (ne0 first), bytes-like).  Returns {name: absolute file offset}."""
    md = list(metadata)
    if alignment is not None:
        md.append(("general.alignment", U32, alignment))
    align = alignment or 32
    head = struct.pack("<IIQQ", magic, version, len(tensors), len(md))
    for key, vt, val in md:
        head += _gstr(key) + struct.pack("<I", vt)
        if vt == ARR:
            et, vals = val
            head += struct.pack("<IQ", et, len(vals)) + b"".join(_scalar(et, v) for v in vals)
        else:
            head += _scalar(vt, val)
    offs, off = [], 0
    blobs = [np.ascontiguousarray(t[3]).tobytes() for t in tensors]
    for b in blobs:
        offs.append(off)
        off = (off + len(b) + align - 1) // align * align
    for (name, gt, dims, _), o in zip(tensors, offs):
        head += _gstr(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        head += struct.pack("<IQ", gt, o)
    data_off = (len(head) + align - 1) // align * align
    with open(path, "wb") as f:
        f.write(head + b"\0" * (data_off - len(head)))
        for b, o in zip(blobs, offs):
            f.seek(data_off + o)
            f.write(b)
        f.seek(0, 2)
        end = f.tell()
        f.write(b"\0" * ((end + align - 1) // align * align - end))
    return {t[0]: data_off + o for t, o in zip(tensors, offs)}
