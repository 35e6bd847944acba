"""A writer of small GGUF v3 buffers for the tests (the layout is the one
crates/xabe-gguf/src/file.rs:1-24 documents).  Test infrastructure only."""
import struct

import numpy as np

TYPE = {"f32": (0, 1, 4), "f16": (1, 1, 2), "q4_0": (2, 32, 18), "q8_0": (8, 32, 34), "q4_K": (12, 256, 144),
        "q5_K": (13, 256, 176), "q6_K": (14, 256, 210), "bf16": (30, 1, 2)}


def _s(text) -> bytes:
    b = text if isinstance(text, bytes) else text.encode()
    return struct.pack("<Q", len(b)) + b


class Builder:
    def __init__(self, alignment: int = 32, version: int = 3):
        self.kv = []
        self.infos = []
        self.data = bytearray()
        self.alignment = alignment
        self.version = version

    def kv_raw(self, key, tag: int, payload: bytes):
        self.kv.append(_s(key) + struct.pack("<i", tag) + payload)
        return self

    def kv_u32(self, key, v):
        return self.kv_raw(key, 4, struct.pack("<I", v))

    def kv_u64(self, key, v):
        return self.kv_raw(key, 10, struct.pack("<Q", v))

    def kv_f32(self, key, v):
        return self.kv_raw(key, 6, struct.pack("<f", v))

    def kv_bool(self, key, v):
        return self.kv_raw(key, 7, struct.pack("<b", 1 if v else 0))

    def kv_str(self, key, v):
        return self.kv_raw(key, 8, _s(v))

    def kv_array(self, key, elem_tag: int, fmt: str, values):
        return self.kv_raw(key, 9, struct.pack("<iQ", elem_tag, len(values)) + b"".join(struct.pack("<" + fmt, v) for v in values))

    def kv_string_array(self, key, values):
        return self.kv_raw(key, 9, struct.pack("<iQ", 8, len(values)) + b"".join(_s(v) for v in values))

    def tensor(self, name, dims, type_name: str, data: bytes | None = None, type_id: int | None = None):
        tid, block, size = TYPE[type_name]
        n = int(np.prod(dims, dtype=np.uint64)) if len(dims) else 1
        n_bytes = (n // block) * size
        pad = (-len(self.data)) % self.alignment
        self.data += b"\0" * pad
        offset = len(self.data)
        self.infos.append(_s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<q", d) for d in dims) +
                          struct.pack("<iQ", tid if type_id is None else type_id, offset))
        self.data += bytes(n_bytes) if data is None else bytes(data)
        return self

    def build(self) -> bytes:
        head = b"GGUF" + struct.pack("<Iqq", self.version, len(self.infos), len(self.kv))
        meta = head + b"".join(self.kv) + b"".join(self.infos)
        pad = (-len(meta)) % self.alignment
        return meta + b"\0" * pad + bytes(self.data)
