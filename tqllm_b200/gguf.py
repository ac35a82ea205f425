"""Host-side mirror of the library's GGUF expert reader (b2moe_gguf_*): opens a checkpoint, lists tensors, slices experts
and packs a block of experts into a finished bank (numpy arrays ready for one upload). `write_gguf` is a minimal GGUF v3
writer for tests and for packing synthetic layers into files."""
from __future__ import annotations

import ctypes as C
import struct

import numpy as np

from . import capi
from .capi import check, lib


class GgufExperts:
    def __init__(self, path: str):
        self._h = C.c_void_p()
        check(lib.b2moe_gguf_open(path.encode(), C.byref(self._h)), f"b2moe_gguf_open({path})")

    def close(self):
        if self._h:
            lib.b2moe_gguf_close(self._h)
            self._h = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def names(self):
        out, buf = [], C.create_string_buffer(512)
        for i in range(lib.b2moe_gguf_tensor_count(self._h)):
            check(lib.b2moe_gguf_tensor_name(self._h, i, buf, 512), "b2moe_gguf_tensor_name")
            out.append(buf.value.decode())
        return out

    def tensor(self, name: str):
        """(type, (cols, rows, experts), offset, bytes)"""
        t, dims, off, nb = C.c_uint32(), (C.c_int64 * 3)(), C.c_uint64(), C.c_uint64()
        check(lib.b2moe_gguf_tensor(self._h, name.encode(), C.byref(t), dims, C.byref(off), C.byref(nb)), f"b2moe_gguf_tensor({name})")
        return t.value, tuple(dims), off.value, nb.value

    def expert_slice(self, name: str, first: int, count: int = 1):
        """(type, rows, cols, raw bytes of the experts as a numpy view of the mapped file)"""
        t, rows, cols, raw, nb = C.c_uint32(), C.c_int32(), C.c_int32(), C.c_void_p(), C.c_uint64()
        check(lib.b2moe_gguf_expert_slice(self._h, name.encode(), first, count, C.byref(t), C.byref(rows), C.byref(cols), C.byref(raw),
                                          C.byref(nb)), f"b2moe_gguf_expert_slice({name})")
        view = np.ctypeslib.as_array(C.cast(raw, C.POINTER(C.c_uint8)), shape=(nb.value,))
        return t.value, rows.value, cols.value, view

    def expert_bank(self, name: str, first: int, count: int, iq3s_as_codes: bool = True):
        """(bank type, rows per expert, cols, data uint8 array, aux float32 array or None) of experts [first, first + count)"""
        t, (cols, rows, _), _, _ = self.tensor(name)
        bank_type = capi.IQ3_S_X4 if (t == 21 and iq3s_as_codes) else t
        data = np.empty(lib.b2moe_bank_bytes(bank_type, count * rows, cols), np.uint8)
        aux_bytes = lib.b2moe_bank_aux_bytes(bank_type, count * rows, cols)
        aux = np.empty(aux_bytes // 4, np.float32) if aux_bytes else None
        check(lib.b2moe_gguf_expert_bank(self._h, name.encode(), first, count, bank_type, data.ctypes.data,
                                         aux.ctypes.data if aux is not None else None), f"b2moe_gguf_expert_bank({name})")
        return bank_type, rows, cols, data, aux


def _gstr(s: str) -> bytes:
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def write_gguf(path: str, tensors, alignment: int = 32, kv=()):
    """tensors: [(name, ggml type, dims (cols, rows[, experts]), raw bytes)]; kv: [(key, value)] with str / int / float /
    list-of-int values (enough to exercise the reader's key/value skipping)."""
    head = struct.pack("<IIQQ", 0x46554747, 3, len(tensors), len(kv) + 1)
    head += _gstr("general.alignment") + struct.pack("<II", 4, alignment)
    for key, val in kv:
        head += _gstr(key)
        if isinstance(val, str):
            head += struct.pack("<I", 8) + _gstr(val)
        elif isinstance(val, float):
            head += struct.pack("<If", 6, val)
        elif isinstance(val, (list, tuple)):
            head += struct.pack("<IIQ", 9, 5, len(val)) + b"".join(struct.pack("<i", v) for v in val)
        else:
            head += struct.pack("<IQ", 10, int(val))
    infos, blobs, off = b"", [], 0
    for name, ttype, dims, raw in tensors:
        raw = bytes(raw)
        infos += _gstr(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", ttype, off)
        pad = (-len(raw)) % alignment
        blobs.append(raw + b"\0" * pad)
        off += len(raw) + pad
    body = head + infos
    body += b"\0" * ((-len(body)) % alignment)
    with open(path, "wb") as f:
        f.write(body)
        for b in blobs:
            f.write(b)
