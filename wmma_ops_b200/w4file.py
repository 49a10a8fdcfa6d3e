"""On-disk container for prepacked INT4 weights ("W4-B200-v1" blocks plus their fp16 scales).

The reference tree has no INT4 code and therefore no file format; this is the storage form of what
`int4_prepack` returns, so that a model's weights are packed once and loaded straight into the
layout the kernels read (no repacking at load time). The byte layout is declared for C readers in
include/wmma_ops_b200.h (wmma_ops_w4_file_header / wmma_ops_w4_file_entry).

File layout (little endian, every payload 256-byte aligned)
  header   64 bytes   magic "W4B200\\0\\0", version (1), header_bytes (64), entry_bytes (128),
                      n_entries, table_crc32 (of the entry table), reserved
  table    n_entries x 128 bytes: name[64] (UTF-8, zero padded), K, N, group_size, zero_point,
                      qweight_offset, qweight_bytes, scales_offset, scales_bytes (u64 each),
                      qweight_crc32, scales_crc32, reserved
  payloads qweight: uint32 [K/64][ceil(N/128)][128][8] exactly as in device memory;
           scales:  fp16 [K/group_size][N]
Version rule: a reader refuses a file whose version it does not know; the packed block layout is
part of the version.
"""
from __future__ import annotations

import os
import struct
import zlib
from typing import Dict, Iterable, Optional, Tuple

import numpy as np
import torch

MAGIC = b"W4B200\0\0"
VERSION = 1
HEADER_BYTES = 64
ENTRY_BYTES = 128
ALIGN = 256
ZERO_POINT = 8

_HEADER = struct.Struct("<8sIIIII36x")          # magic, version, header_bytes, entry_bytes, n_entries, table_crc32
_ENTRY = struct.Struct("<64sIIIIQQQQII8x")      # name, K, N, group, zero_point, q_off, q_bytes, s_off, s_bytes, q_crc, s_crc
assert _HEADER.size == HEADER_BYTES and _ENTRY.size == ENTRY_BYTES


def _fail(msg: str):
    raise RuntimeError(f"w4 file: {msg}")


def _align(n: int) -> int:
    return (n + ALIGN - 1) // ALIGN * ALIGN


def _as_bytes(t: torch.Tensor) -> bytes:
    return t.detach().contiguous().cpu().numpy().tobytes()


def _check_pair(name: str, qweight: torch.Tensor, scales: torch.Tensor, group_size: int) -> Tuple[int, int]:
    if qweight.dtype != torch.int32 or qweight.dim() != 4 or qweight.size(2) != 128 or qweight.size(3) != 8:
        _fail(f"{name}: qweight must be int32 [K/64, ceil(N/128), 128, 8] as returned by int4_prepack")
    if scales.dtype != torch.float16 or scales.dim() != 2:
        _fail(f"{name}: scales must be float16 [K/group_size, N]")
    K, N = qweight.size(0) * 64, scales.size(1)
    if group_size <= 0 or K % group_size != 0 or scales.size(0) * group_size != K:
        _fail(f"{name}: scales rows ({scales.size(0)}) do not match K / group_size = {K} / {group_size}")
    if qweight.size(1) != (N + 127) // 128:
        _fail(f"{name}: qweight has {qweight.size(1)} column tiles but N = {N}")
    if len(name.encode("utf-8")) > 63:
        _fail(f"{name}: names are limited to 63 bytes")
    return K, N


def save_w4(path, tensors: Dict[str, Tuple[torch.Tensor, torch.Tensor, int]]) -> int:
    """Writes `tensors` (name -> (qweight, scales, group_size), tensors on any device) to `path`.
    Returns the number of bytes written. The file is written to a temporary name and renamed, so a
    reader never sees a partial file."""
    names = list(tensors)
    if not names:
        _fail("nothing to save")
    table_end = HEADER_BYTES + ENTRY_BYTES * len(names)
    offset = _align(table_end)
    entries, blobs = [], []
    for name in names:
        qweight, scales, group = tensors[name]
        K, N = _check_pair(name, qweight, scales, int(group))
        qb, sb = _as_bytes(qweight), _as_bytes(scales)
        q_off = offset
        s_off = _align(q_off + len(qb))
        offset = _align(s_off + len(sb))
        entries.append(_ENTRY.pack(name.encode("utf-8"), K, N, int(group), ZERO_POINT, q_off, len(qb), s_off, len(sb),
                                   zlib.crc32(qb) & 0xFFFFFFFF, zlib.crc32(sb) & 0xFFFFFFFF))
        blobs.append((q_off, qb, s_off, sb))
    table = b"".join(entries)
    header = _HEADER.pack(MAGIC, VERSION, HEADER_BYTES, ENTRY_BYTES, len(names), zlib.crc32(table) & 0xFFFFFFFF)
    tmp = f"{os.fspath(path)}.tmp{os.getpid()}"
    with open(tmp, "wb") as f:
        f.write(header)
        f.write(table)
        for q_off, qb, s_off, sb in blobs:
            f.write(b"\0" * (q_off - f.tell()))
            f.write(qb)
            f.write(b"\0" * (s_off - f.tell()))
            f.write(sb)
        f.write(b"\0" * (offset - f.tell()))
        total = f.tell()
    os.replace(tmp, path)
    return total


def read_w4_index(path) -> Dict[str, dict]:
    """The entry table of a file: name -> {K, N, group_size, zero_point, offsets, sizes, crcs}.
    Validates magic, version, table checksum and that every payload lies inside the file."""
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        raw = f.read(HEADER_BYTES)
        if len(raw) < HEADER_BYTES:
            _fail("file is shorter than its header")
        magic, version, hbytes, ebytes, n, table_crc = _HEADER.unpack(raw)
        if magic != MAGIC:
            _fail("bad magic (not a W4-B200 weight file)")
        if version != VERSION:
            _fail(f"version {version} is not supported by this reader (knows version {VERSION})")
        if hbytes != HEADER_BYTES or ebytes != ENTRY_BYTES or n < 1 or HEADER_BYTES + n * ENTRY_BYTES > size:
            _fail("corrupt header")
        table = f.read(n * ENTRY_BYTES)
    if zlib.crc32(table) & 0xFFFFFFFF != table_crc:
        _fail("entry table checksum mismatch")
    out = {}
    for i in range(n):
        (name, K, N, group, zp, q_off, q_bytes, s_off, s_bytes, q_crc, s_crc) = _ENTRY.unpack_from(table, i * ENTRY_BYTES)
        name = name.rstrip(b"\0").decode("utf-8")
        if zp != ZERO_POINT:
            _fail(f"{name}: zero point {zp} is not supported")
        if K % 64 != 0 or group <= 0 or K % group != 0 or N % 8 != 0:
            _fail(f"{name}: invalid shape K={K} N={N} group_size={group}")
        want_q = (K // 64) * ((N + 127) // 128) * 4096
        want_s = (K // group) * N * 2
        if q_bytes != want_q or s_bytes != want_s:
            _fail(f"{name}: payload sizes {q_bytes}/{s_bytes} do not match the shape ({want_q}/{want_s})")
        if q_off % ALIGN or s_off % ALIGN or q_off + q_bytes > size or s_off + s_bytes > size:
            _fail(f"{name}: payload lies outside the file (truncated?)")
        out[name] = {"K": K, "N": N, "group_size": group, "zero_point": zp, "qweight_offset": q_off,
                     "qweight_bytes": q_bytes, "scales_offset": s_off, "scales_bytes": s_bytes,
                     "qweight_crc32": q_crc, "scales_crc32": s_crc}
    return out


def load_w4(path, device=None, names: Optional[Iterable[str]] = None, verify: bool = True
            ) -> Dict[str, Tuple[torch.Tensor, torch.Tensor, int]]:
    """Loads entries of a file as name -> (qweight int32 [K/64, ceil(N/128), 128, 8], scales fp16
    [K/g, N], group_size) on `device` (default: the current CUDA device; "cpu" keeps host tensors).
    verify=True checks the CRC-32 of every payload it reads. The tensors are ready for matmul_w4a16."""
    index = read_w4_index(path)
    wanted = list(index) if names is None else list(names)
    for n in wanted:
        if n not in index:
            _fail(f"no entry named {n!r} (has: {', '.join(index)})")
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    device = torch.device(device)
    mm = np.memmap(path, dtype=np.uint8, mode="r")
    out = {}
    for n in wanted:
        e = index[n]
        qraw = mm[e["qweight_offset"]:e["qweight_offset"] + e["qweight_bytes"]]
        sraw = mm[e["scales_offset"]:e["scales_offset"] + e["scales_bytes"]]
        if verify:
            if zlib.crc32(qraw) & 0xFFFFFFFF != e["qweight_crc32"]:
                _fail(f"{n}: packed weights checksum mismatch")
            if zlib.crc32(sraw) & 0xFFFFFFFF != e["scales_crc32"]:
                _fail(f"{n}: scales checksum mismatch")
        K, N, g = e["K"], e["N"], e["group_size"]
        q = torch.from_numpy(np.array(qraw, copy=True).view(np.int32).reshape(K // 64, (N + 127) // 128, 128, 8))
        s = torch.from_numpy(np.array(sraw, copy=True).view(np.float16).reshape(K // g, N))
        if device.type == "cuda":
            q = q.pin_memory().to(device, non_blocking=True)
            s = s.pin_memory().to(device, non_blocking=True)
        out[n] = (q, s, g)
    if device.type == "cuda":
        torch.cuda.synchronize(device)
    return out
