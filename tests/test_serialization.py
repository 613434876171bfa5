"""Round trips and rejects of the `.tannic` record (include/tannic/serialization.hpp:26-66 of the reference)."""
import struct

import pytest
import torch

from tannic_b200 import serialization as ser


@pytest.mark.parametrize("dtype", [torch.int8, torch.int16, torch.int32, torch.int64, torch.float16, torch.bfloat16, torch.float32,
                                   torch.float64, torch.complex64, torch.bool])
@pytest.mark.parametrize("shape", [(), (7,), (3, 4, 5), (2, 0, 3)])
def test_round_trip(dtype, shape, tmp_path):
    g = torch.Generator().manual_seed(1)
    x = (torch.randn(shape, generator=g) * 10).to(dtype) if dtype != torch.bool else torch.rand(shape, generator=g) > 0.5
    blob = ser.dumps(x)
    magic, version, checksum, nbytes = ser.HEADER.unpack_from(blob, 0)
    assert (magic, version, checksum) == (0x43495245, 1, 0xABCD)
    payload = (x.numel() + 7) // 8 if dtype == torch.bool else x.numel() * x.element_size()  # booleans are bit-packed
    assert nbytes == len(blob) - ser.HEADER.size == payload + ser.METADATA.size + 8 * len(shape)
    assert ser.HEADER.size == 15 and ser.METADATA.size == 18  # packed records
    y = ser.loads(blob)
    assert y.dtype == x.dtype and y.shape == x.shape
    raw = lambda t: t.contiguous().reshape(-1).view(torch.uint8)
    assert torch.equal(raw(y), raw(x))
    ser.save(x, tmp_path / "t.tannic")
    assert torch.equal(raw(ser.load(tmp_path / "t.tannic")), raw(x))


def test_boolean_payload_is_bit_packed_lsb_first():
    """nbytesof(boolean, n) = (n + 7) / 8 (include/tannic/types.hpp:149-154); element i is bit i % 8 of
    byte i / 8 (src/tensor.cpp:48-61)."""
    x = torch.tensor([True, False, False, True, False, False, False, False, True, True, False])  # 11 elements
    blob = ser.dumps(x)
    _, _, payload_bytes, rank = ser.METADATA.unpack_from(blob, ser.HEADER.size)
    assert (payload_bytes, rank) == (2, 1)
    assert blob[-2:] == bytes([0b00001001, 0b00000011])
    assert torch.equal(ser.loads(blob), x)
    wide = torch.rand((5, 13), generator=torch.Generator().manual_seed(3)) > 0.5
    assert torch.equal(ser.loads(ser.dumps(wide)), wide)


def test_views_are_stored_dense():
    x = torch.arange(24, dtype=torch.float32).reshape(4, 6)
    assert torch.equal(ser.loads(ser.dumps(x.t()[1:, ::2])), x.t()[1:, ::2].contiguous())


def test_rejects():
    blob = bytearray(ser.dumps(torch.ones(3)))
    with pytest.raises(ValueError):
        ser.loads(bytes(blob[:10]))
    bad = bytearray(blob)
    struct.pack_into("<I", bad, 0, 0xDEADBEEF)
    with pytest.raises(ValueError):
        ser.loads(bytes(bad))
    with pytest.raises(ValueError):
        ser.loads(bytes(blob[:-2]))
    bad = bytearray(blob)
    bad[ser.HEADER.size] = 99  # dtype code
    with pytest.raises(ValueError):
        ser.loads(bytes(bad))
