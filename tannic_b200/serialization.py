"""`.tannic` tensor files: the on-disk record of include/tannic/serialization.hpp:26-66 of the reference.

The reference tree defines the two packed records and how their fields are filled (`headerof`,
`metadataof`) but holds no writer or reader, so the order of the parts is taken from the header's own
byte count (`nbytes = payload + sizeof(Metadata<Tensor>) + rank * sizeof(size_t)`):

    Header    <I B H Q   magic 0x43495245, version 1, checksum 0xABCD, nbytes of everything after the header
    Metadata  <B Q Q B   dtype code (include/tannic/types.hpp:206-221), byte offset of the view, payload bytes, rank
    sizes     rank x <Q
    payload   the tensor's bytes, dense row-major; boolean tensors are bit-packed, element i in bit
              i % 8 of byte i / 8 ((n + 7) / 8 bytes: `nbytesof`, include/tannic/types.hpp:149-154, and the
              bit order of `Tensor::assign(bool const*, index)`, src/tensor.cpp:48-61)

Used here as the fixture format shared by host-side tests; nothing on the device path depends on it.
"""
from __future__ import annotations

import struct
from pathlib import Path

import numpy as np
import torch

MAGIC = 0x43495245
HEADER = struct.Struct("<IBHQ")
METADATA = struct.Struct("<BQQB")

DCODE = {torch.bool: 1, torch.int8: 12, torch.int16: 13, torch.int32: 14, torch.int64: 15, torch.float16: 23,
         torch.bfloat16: 231, torch.float32: 24, torch.float64: 25, torch.complex64: 35, torch.complex128: 36}
DTYPE = {v: k for k, v in DCODE.items()}


def dumps(t: torch.Tensor) -> bytes:
    if t.dtype not in DCODE:
        raise ValueError(f"{t.dtype} has no Tannic dtype code")
    dense = t.detach().cpu().contiguous()
    if dense.dtype == torch.bool:
        payload = np.packbits(dense.reshape(-1).numpy(), bitorder="little").tobytes() if dense.numel() else b""
    else:
        payload = dense.reshape(-1).view(torch.uint8).numpy().tobytes() if dense.numel() else b""
    sizes = b"".join(struct.pack("<Q", s) for s in dense.shape)
    body = METADATA.pack(DCODE[t.dtype], 0, len(payload), dense.dim()) + sizes + payload
    return HEADER.pack(MAGIC, 1, 0xABCD, len(body)) + body


def loads(blob: bytes) -> torch.Tensor:
    if len(blob) < HEADER.size:
        raise ValueError("truncated header")
    magic, version, _checksum, nbytes = HEADER.unpack_from(blob, 0)
    if magic != MAGIC:
        raise ValueError(f"bad magic {magic:#x}")
    if version != 1:
        raise ValueError(f"unsupported version {version}")
    if len(blob) < HEADER.size + nbytes or nbytes < METADATA.size:
        raise ValueError("truncated body")
    dcode, _offset, payload_bytes, rank = METADATA.unpack_from(blob, HEADER.size)
    if dcode not in DTYPE:
        raise ValueError(f"unknown dtype code {dcode}")
    at = HEADER.size + METADATA.size
    shape = struct.unpack_from(f"<{rank}Q", blob, at) if rank else ()
    at += 8 * rank
    if nbytes != METADATA.size + 8 * rank + payload_bytes:
        raise ValueError("byte counts of header and metadata disagree")
    dtype = DTYPE[dcode]
    count = 1
    for s in shape:
        count *= s
    expected = (count + 7) // 8 if dtype == torch.bool else count * torch.empty((), dtype=dtype).element_size()
    if expected != payload_bytes:
        raise ValueError("payload size does not match shape and dtype")
    if count == 0:
        return torch.empty(shape, dtype=dtype)
    if dtype == torch.bool:
        bits = np.unpackbits(np.frombuffer(blob, dtype=np.uint8, count=payload_bytes, offset=at), bitorder="little")[:count]
        return torch.from_numpy(bits.astype(np.bool_)).reshape(shape)
    raw = torch.frombuffer(bytearray(blob[at:at + payload_bytes]), dtype=torch.uint8)
    return raw.view(dtype).reshape(shape)


def save(t: torch.Tensor, path) -> None:
    Path(path).write_bytes(dumps(t))


def load(path) -> torch.Tensor:
    return loads(Path(path).read_bytes())
