"""The CGB2 container: header layout and validation on CPU; GPU round trips in test_gpu_flat.py."""
import struct

import pytest
import torch

from cachegen_b200.serde import flat_format as ff


def make_blob(T=300, table_kind=ff.TABLES_CDF):
    L, H, D, lp = 2, 2, 64, 33
    nsub = (T + 255) // 256
    sub_off = [0] + [100 * (j + 1) for j in range(nsub)]
    tb = 2 * L * H * D * lp * 2 if table_kind == ff.TABLES_CDF else 1000
    h = ff.layout(L, H, D, T, lp, torch.bfloat16, table_kind, tb, ff.LENGTHS_U16, sub_off)
    blob = torch.zeros(h.total, dtype=torch.uint8)
    hb = h.pack()
    blob[:len(hb)] = torch.frombuffer(bytearray(hb), dtype=torch.uint8)
    return h, blob


def test_layout_sections_are_aligned_and_typed():
    h, blob = make_blob()
    assert all(off % ff.ALIGN == 0 for off in (h.off_scales, h.off_tables, h.off_lengths, h.off_payload))
    c = ff.FlatChunk(blob)
    assert c.header == h
    assert c.scales().shape == (4, 300) and c.scales().dtype == torch.bfloat16
    assert c.tables().shape == (4, 128, 33) and c.tables().dtype == torch.int16
    assert c.lengths(1).shape == (4, 128) and c.lengths(1).dtype == torch.int16
    assert c.payload(0).numel() == 100 and c.payload(1).numel() == 100
    assert [c.sub_tokens(j) for j in range(2)] == [256, 44]
    assert c.num_heads == 2 and c.head_size == 64 and c.num_tokens == 300
    back = ff.from_bytes(c.tobytes())
    assert back.header == h and ff.is_flat(c.tobytes()) and not ff.is_flat(b"\x80\x04pickle")


def test_counts_tables_are_a_byte_view():
    h, blob = make_blob(table_kind=ff.TABLES_COUNTS)
    c = ff.FlatChunk(blob)
    assert c.tables().dtype == torch.uint8 and c.tables().numel() >= 1000


def test_row_offsets_follow_the_bins():
    bins = torch.tensor([32.0, 16.0, 12.0, 8.0])
    assert ff.table_row_offsets(bins, 10) == [0, 300, 440, 540, 600]  # 2*(b//2-1) symbols per row


@pytest.mark.parametrize("mutate", ["magic", "version", "total", "nsub", "order", "payload", "truncate", "kind"])
def test_corrupt_headers_are_rejected(mutate):
    h, blob = make_blob()
    raw = bytearray(blob.numpy().tobytes())
    if mutate == "magic":
        raw[0:4] = b"XXXX"
    elif mutate == "version":
        raw[4:8] = struct.pack("<I", 9)
    elif mutate == "total":
        raw += b"\0"
    elif mutate == "nsub":
        raw[28:32] = struct.pack("<I", 7)
    elif mutate == "order":
        raw[48:56] = struct.pack("<Q", h.off_tables + 256)  # scales after tables
    elif mutate == "payload":
        raw[128 + 8:128 + 16] = struct.pack("<Q", 10 ** 9)
    elif mutate == "truncate":
        raw = raw[:100]
    elif mutate == "kind":
        raw[36:40] = struct.pack("<I", 5)
    with pytest.raises(ValueError):
        ff.from_bytes(bytes(raw))


def test_sparse_table_geometry():
    bins = torch.tensor([32.0, 16.0, 16.0, 32.0])
    # odd channel count: a 2-byte row of 7 channels takes 16 bytes so that the next row stays 4-byte aligned
    assert ff.mask_row_offsets(bins, 7) == [0, 28, 44, 60, 88]
    assert ff.mask_row_offsets(bins, 128) == [0, 512, 768, 1024, 1536]
    off_masks, off_counts = ff.sparse_parts(4, 300, 1000)
    assert off_masks == 64 and off_counts == 64 + 1008      # 4 rows x 3 groups + 1 offsets = 52 bytes -> 64
    assert ff.sparse_representable(torch.tensor([34.0, 8.0])) and not ff.sparse_representable(torch.tensor([36.0]))
    h, blob = make_blob(table_kind=ff.TABLES_SPARSE)
    assert ff.FlatHeader.parse(blob.numpy().tobytes()).table_kind == ff.TABLES_SPARSE


def test_bins_checksum_travels_in_the_header():
    a, b = ff.bins_checksum(torch.tensor([32.0, 16.0])), ff.bins_checksum(torch.tensor([16.0, 8.0]))
    assert a != b and a != 0 and b != 0
    h = ff.layout(2, 2, 64, 10, 33, torch.float16, ff.TABLES_COUNTS, 100, ff.LENGTHS_U16, [0, 5], bins_checksum=a)
    assert ff.FlatHeader.parse_head(h.pack(), h.total).bins_checksum == a
    assert ff.FlatHeader.parse_head(make_blob()[0].pack(), make_blob()[0].total).bins_checksum == 0  # not recorded
