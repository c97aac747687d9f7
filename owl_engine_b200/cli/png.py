"""Pure-CPU PNG writer (zlib + CRC32 from the standard library; no imaging or graphics dependency).

The GUI-agent workload needs deterministic screenshots whose content the model must actually look
at: solid colours, optionally with a contrasting rectangle. ``data_url_png`` returns the
``data:image/png;base64,...`` form the chat endpoint accepts.

Reference counterpart: ``apps/cli/src/workload/png.rs:1-6``.
"""
from __future__ import annotations

import base64
import struct
import zlib

RED, GREEN, BLUE, YELLOW, PURPLE = (220, 30, 30), (30, 180, 60), (40, 70, 220), (240, 220, 40), (140, 50, 190)
NAMES = {RED: "red", GREEN: "green", BLUE: "blue", YELLOW: "yellow", PURPLE: "purple"}


def _chunk(tag: bytes, data: bytes) -> bytes:
    return struct.pack(">I", len(data)) + tag + data + struct.pack(">I", zlib.crc32(tag + data) & 0xFFFFFFFF)


def encode_png(w: int, h: int, rgb: tuple, box: tuple | None = None, box_rgb: tuple = (255, 255, 255)) -> bytes:
    """8-bit RGB, filter 0 on every row. ``box`` = (x0, y0, x1, y1) painted in ``box_rgb``."""
    row_bg = bytes(rgb) * w
    rows = bytearray()
    for y in range(h):
        rows.append(0)
        if box and box[1] <= y < box[3]:
            x0, x1 = max(0, box[0]), min(w, box[2])
            rows += row_bg[:3 * x0] + bytes(box_rgb) * (x1 - x0) + row_bg[3 * x1:]
        else:
            rows += row_bg
    ihdr = struct.pack(">IIBBBBB", w, h, 8, 2, 0, 0, 0)
    return b"\x89PNG\r\n\x1a\n" + _chunk(b"IHDR", ihdr) + _chunk(b"IDAT", zlib.compress(bytes(rows), 6)) + _chunk(b"IEND", b"")


def decode_png(data: bytes):
    """Inverse for the subset ``encode_png`` writes plus filters 1-4 (used by the server's image path)."""
    import numpy as np

    assert data[:8] == b"\x89PNG\r\n\x1a\n", "not a PNG"
    pos, idat, w = 8, b"", 0
    while pos < len(data):
        n, tag = struct.unpack(">I4s", data[pos:pos + 8])
        body = data[pos + 8:pos + 8 + n]
        if tag == b"IHDR":
            w, h, depth, ctype, _, _, interlace = struct.unpack(">IIBBBBB", body)
            assert depth == 8 and ctype in (2, 6) and interlace == 0, "only 8-bit RGB/RGBA non-interlaced PNGs"
            bpp = 3 if ctype == 2 else 4
        elif tag == b"IDAT":
            idat += body
        pos += 12 + n
    raw = zlib.decompress(idat)
    stride = w * bpp
    out = np.zeros((h, stride), dtype=np.uint8)
    prev = np.zeros(stride, dtype=np.int32)
    for y in range(h):
        f = raw[y * (stride + 1)]
        line = np.frombuffer(raw, dtype=np.uint8, count=stride, offset=y * (stride + 1) + 1).astype(np.int32)
        if f == 0:
            cur = line
        elif f == 2:
            cur = (line + prev) & 255
        else:
            cur = np.zeros(stride, dtype=np.int32)
            for i in range(stride):
                a = cur[i - bpp] if i >= bpp else 0
                b, c = prev[i], (prev[i - bpp] if i >= bpp else 0)
                if f == 1:
                    p = a
                elif f == 3:
                    p = (a + b) // 2
                else:
                    pa, pb, pc = abs(b - c), abs(a - c), abs(a + b - 2 * c)
                    p = a if pa <= pb and pa <= pc else (b if pb <= pc else c)
                cur[i] = (line[i] + p) & 255
        out[y] = cur
        prev = cur
    return out.reshape(h, w, bpp)[:, :, :3]


def data_url_png(w: int, h: int, rgb: tuple, **kw) -> str:
    return "data:image/png;base64," + base64.b64encode(encode_png(w, h, rgb, **kw)).decode()
