"""CPU-only checks of the offline packed-weight file: the writer quantizes exactly as the
oracle's per-channel weight quantizer, the documented byte layout can be read back with
numpy alone, and damaged files are refused."""
import struct

import numpy as np
import pytest
import torch

D, NQKV, HID, LAYERS = 128, 384, 256, 2
HEADER = struct.Struct("<8sIIIIIIQQ16s")


def unslab(codes, n, k):
    return np.ascontiguousarray(codes.reshape(k // 128, n, 128).transpose(1, 0, 2)).reshape(n, k)


def fnv1a(data: bytes) -> int:
    h = 1469598103934665603
    for b in data:
        h = ((h ^ b) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return h


@pytest.fixture()
def written(pkg, ref, tmp_path):
    path = tmp_path / "stack.w8a8"
    layers = [ref.make_layer_fp32(l, D, NQKV, HID) for l in range(LAYERS)]
    pkg.write_weight_file(path, D, NQKV, HID, layers, threads=2)
    return path, layers


def test_header_and_layout_match_the_oracle_quantizer(pkg, ref, written):
    path, layers = written
    assert pkg.weight_file_info(path) == (D, NQKV, HID, LAYERS)
    raw = path.read_bytes()
    magic, version, layout, d, nq, hid, nl, payload, checksum, _ = HEADER.unpack_from(raw)
    assert HEADER.size == 64 and magic == b"B2W8A8WF" and version == 1 and layout == pkg.W_SLAB128
    assert (d, nq, hid, nl) == (D, NQKV, HID, LAYERS)
    assert payload == len(raw) - 64 and checksum == fnv1a(raw[64:])
    off = 64
    for ws, gs in layers:
        for w in ws:
            n, k = w.shape
            q_ref, s_ref = ref.quantize_weight(w)
            codes = np.frombuffer(raw, np.int8, n * k, off)
            off += n * k
            scales = np.frombuffer(raw, np.float32, n, off)
            off += 4 * n
            assert np.array_equal(unslab(codes, n, k), q_ref.numpy())
            assert np.array_equal(scales.view(np.uint32), s_ref.numpy().view(np.uint32))
        for g in gs:
            got = np.frombuffer(raw, np.float32, D, off)
            off += 4 * D
            assert np.array_equal(got.view(np.uint32), g.float().numpy().view(np.uint32))
    assert off == len(raw)


def test_damaged_files_are_refused(pkg, written, tmp_path):
    path, _ = written
    raw = bytearray(path.read_bytes())
    cases = {}
    flipped = bytearray(raw)
    flipped[64 + 1000] ^= 0x40
    cases["checksum"] = bytes(flipped)
    cases["truncated"] = bytes(raw[:-17])
    cases["trailing"] = bytes(raw) + b"\0"
    bad_magic = bytearray(raw)
    bad_magic[0:2] = b"XX"
    cases["not a packed"] = bytes(bad_magic)
    bad_dims = bytearray(raw)
    struct.pack_into("<I", bad_dims, 16, 130)  # d not a multiple of 128
    cases["invalid dimensions"] = bytes(bad_dims)
    bad_ver = bytearray(raw)
    struct.pack_into("<I", bad_ver, 8, 7)
    cases["unsupported version"] = bytes(bad_ver)
    for word, blob in cases.items():
        p = tmp_path / "damaged.w8a8"
        p.write_bytes(blob)
        with pytest.raises(pkg.W8A8Error, match=word):
            pkg.weight_file_info(p)
    # a flipped payload byte passes the header-only check
    p = tmp_path / "damaged.w8a8"
    p.write_bytes(cases["checksum"])
    assert pkg.weight_file_info(p, verify=False) == (D, NQKV, HID, LAYERS)
    with pytest.raises(pkg.W8A8Error, match="cannot open"):
        pkg.weight_file_info(tmp_path / "missing.w8a8")


def test_writer_rejects_bad_input(pkg, ref, tmp_path):
    layers = [ref.make_layer_fp32(0, D, NQKV, HID)]
    with pytest.raises(pkg.W8A8Error, match="invalid weight file configuration"):
        pkg.write_weight_file(tmp_path / "a.w8a8", 100, NQKV, HID, layers)
    # fewer layers than declared: the file is left without a valid header
    w = pkg.lib().b200_w8a8_weight_file_create(str(tmp_path / "b.w8a8").encode(), D, NQKV, HID, 2)
    assert w and pkg.lib().b200_w8a8_weight_file_close(w) == 1
    with pytest.raises(pkg.W8A8Error, match="not a packed"):
        pkg.weight_file_info(tmp_path / "b.w8a8")
    # non-finite weights are refused like in the packer
    ws, gs = ref.make_layer_fp32(0, D, NQKV, HID)
    ws[3] = ws[3].clone()
    ws[3][5, 7] = float("nan")
    with pytest.raises(pkg.W8A8Error):
        pkg.write_weight_file(tmp_path / "c.w8a8", D, NQKV, HID, [(ws, gs)])
