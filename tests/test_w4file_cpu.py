"""The on-disk container for prepacked INT4 weights, on the CPU: bit-exact round trip of what the
packing oracle produces, the index, and every way a file can be wrong (magic, version, truncation,
flipped payload bit, flipped table bit)."""
import struct

import pytest
import torch

from oracle import int4
from wmma_ops_b200 import w4file


def _pair(K, N, group, seed):
    codes, scales = int4.seeded_w4(K, N, group, seed=seed)
    return int4.pack_ref(codes), scales, group


def test_round_trip_is_bit_exact(tmp_path):
    tensors = {"qkv": _pair(256, 384, 128, 1), "down.proj": _pair(512, 136, 64, 2), "tiny": _pair(64, 8, 64, 3)}
    path = tmp_path / "layer.w4"
    n = w4file.save_w4(path, tensors)
    assert n == path.stat().st_size and n % 256 == 0
    index = w4file.read_w4_index(path)
    assert list(index) == list(tensors)
    assert (index["down.proj"]["K"], index["down.proj"]["N"], index["down.proj"]["group_size"]) == (512, 136, 64)
    assert all(e["qweight_offset"] % 256 == 0 and e["scales_offset"] % 256 == 0 for e in index.values())
    back = w4file.load_w4(path, device="cpu")
    for name, (q, s, g) in tensors.items():
        q2, s2, g2 = back[name]
        assert g2 == g and q2.dtype == torch.int32 and s2.dtype == torch.float16
        assert torch.equal(q2, q) and torch.equal(s2.view(torch.int16), s.view(torch.int16))
        # and what was stored is the packed form of the codes: unpacking gives them back
        K, N = q.shape[0] * 64, s.shape[1]
        assert torch.equal(int4.pack_ref(int4.unpack_ref(q2, K, N)), q)
    only = w4file.load_w4(path, device="cpu", names=["tiny"])
    assert list(only) == ["tiny"]
    with pytest.raises(RuntimeError, match="no entry named"):
        w4file.load_w4(path, device="cpu", names=["absent"])


def test_header_layout_matches_the_c_declaration(tmp_path):
    path = tmp_path / "one.w4"
    w4file.save_w4(path, {"w": _pair(128, 128, 128, 4)})
    raw = path.read_bytes()
    magic, version, hbytes, ebytes, n = struct.unpack_from("<8sIIII", raw, 0)
    assert (magic, version, hbytes, ebytes, n) == (b"W4B200\0\0", 1, 64, 128, 1)
    name, K, N, group, zp, q_off, q_bytes, s_off, s_bytes = struct.unpack_from("<64sIIIIQQQQ", raw, 64)
    assert name.rstrip(b"\0") == b"w" and (K, N, group, zp) == (128, 128, 128, 8)
    assert q_bytes == (K // 64) * 1 * 4096 and s_bytes == (K // group) * N * 2 and q_off == 256


@pytest.mark.parametrize("damage", ["magic", "version", "truncate", "payload_bit", "table_bit", "short"])
def test_damaged_files_are_refused(tmp_path, damage):
    path = tmp_path / "bad.w4"
    w4file.save_w4(path, {"a": _pair(128, 256, 128, 5), "b": _pair(64, 128, 64, 6)})
    raw = bytearray(path.read_bytes())
    index = w4file.read_w4_index(path)
    expect = {"magic": "bad magic", "version": "version 2 is not supported", "truncate": "outside the file",
              "payload_bit": "checksum mismatch", "table_bit": "table checksum", "short": "shorter than its header"}[damage]
    if damage == "magic":
        raw[0] ^= 0xFF
    elif damage == "version":
        raw[8] = 2
    elif damage == "truncate":
        raw = raw[:index["b"]["scales_offset"] + 10]
    elif damage == "payload_bit":
        raw[index["a"]["qweight_offset"] + 17] ^= 0x04
    elif damage == "table_bit":
        raw[64 + 70] ^= 0x01
    elif damage == "short":
        raw = raw[:20]
    path.write_bytes(bytes(raw))
    with pytest.raises(RuntimeError, match=expect):
        w4file.load_w4(path, device="cpu")
    if damage == "payload_bit":
        # the flag that skips verification loads the (damaged) bytes as they are
        got = w4file.load_w4(path, device="cpu", verify=False)
        assert not torch.equal(got["a"][0], _pair(128, 256, 128, 5)[0])


def test_save_rejects_mismatched_tensors(tmp_path):
    q, s, g = _pair(256, 128, 128, 7)
    with pytest.raises(RuntimeError, match="do not match K"):
        w4file.save_w4(tmp_path / "x.w4", {"w": (q, s, 64)})
    with pytest.raises(RuntimeError, match="qweight must be int32"):
        w4file.save_w4(tmp_path / "x.w4", {"w": (q.float(), s, g)})
    with pytest.raises(RuntimeError, match="column tiles"):
        w4file.save_w4(tmp_path / "x.w4", {"w": (q, torch.cat([s, s], dim=1), g)})
    with pytest.raises(RuntimeError, match="nothing to save"):
        w4file.save_w4(tmp_path / "x.w4", {})
    assert not (tmp_path / "x.w4").exists()
