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


MAX_PNG_SIDE = 16384          # images come from clients: the header's claims are checked before anything is allocated
MAX_PNG_PIXELS = 64 << 20     # 64 Mpixel (an 8k x 8k screenshot): about 200 MB decoded


def decode_png(data: bytes):
    """Inverse for the subset ``encode_png`` writes plus filters 1-4 (used by the server's image path). The bytes come from
    a client: every structural claim (signature, chunk lengths, header fields, the size of the decompressed data) is
    checked, and anything else than a well-formed 8-bit RGB / RGBA non-interlaced PNG raises ``ValueError``."""
    import numpy as np

    if data[:8] != b"\x89PNG\r\n\x1a\n":
        raise ValueError("not a PNG (bad signature)")
    pos, idat, hdr = 8, [], None
    while pos + 8 <= len(data):
        n, tag = struct.unpack(">I4s", data[pos:pos + 8])
        if pos + 12 + n > len(data):
            raise ValueError(f"PNG chunk {tag!r} of {n} bytes runs past the end of the data")
        body = data[pos + 8:pos + 8 + n]
        if tag == b"IHDR":
            if n != 13:
                raise ValueError("PNG header chunk has the wrong length")
            hdr = struct.unpack(">IIBBBBB", body)
        elif tag == b"IDAT":
            idat.append(body)
        elif tag == b"IEND":
            break
        pos += 12 + n
    if hdr is None:
        raise ValueError("PNG without a header chunk")
    w, h, depth, ctype, comp, filt, interlace = hdr
    if depth != 8 or ctype not in (2, 6) or interlace != 0 or comp != 0 or filt != 0:
        raise ValueError("only 8-bit RGB / RGBA non-interlaced PNGs are accepted")
    if not (0 < w <= MAX_PNG_SIDE and 0 < h <= MAX_PNG_SIDE) or w * h > MAX_PNG_PIXELS:
        raise ValueError(f"PNG of {w} x {h} pixels (sides must be 1..{MAX_PNG_SIDE}, at most {MAX_PNG_PIXELS >> 20} Mpixel)")
    bpp = 3 if ctype == 2 else 4
    stride = w * bpp
    want = h * (stride + 1)
    z = zlib.decompressobj()
    try:
        raw = z.decompress(b"".join(idat), want + 1)            # never inflate more than the header accounts for
    except zlib.error as e:
        raise ValueError(f"PNG image data does not inflate: {e}") from None
    if len(raw) != want:
        raise ValueError(f"PNG image data inflates to {len(raw)} bytes, the header accounts for {want}")
    out = np.zeros((h, stride), dtype=np.uint8)
    prev = bytes(stride)
    for y in range(h):
        o = y * (stride + 1)
        f, line = raw[o], raw[o + 1:o + 1 + stride]
        if f == 0:
            cur = line
        elif f == 2:                                            # Up: whole row at once
            cur = ((np.frombuffer(line, dtype=np.uint8).astype(np.int32) + np.frombuffer(prev, dtype=np.uint8)) & 255).astype(np.uint8).tobytes()
        elif f == 1:                                            # Sub: a running sum per channel
            px = np.frombuffer(line, dtype=np.uint8).reshape(w, bpp).astype(np.int64)
            cur = (np.cumsum(px, axis=0) & 255).astype(np.uint8).tobytes()
        elif f in (3, 4):                                       # Average / Paeth depend on the pixel just decoded: a tight byte loop
            c = bytearray(stride)
            for i in range(stride):
                a = c[i - bpp] if i >= bpp else 0
                b = prev[i]
                if f == 3:
                    p = (a + b) >> 1
                else:
                    cc = prev[i - bpp] if i >= bpp else 0
                    pa, pb, pc = abs(b - cc), abs(a - cc), abs(a + b - 2 * cc)
                    p = a if pa <= pb and pa <= pc else (b if pb <= pc else cc)
                c[i] = (line[i] + p) & 255
            cur = bytes(c)
        else:
            raise ValueError(f"PNG row {y} uses filter {f} (0..4 exist)")
        out[y] = np.frombuffer(cur, dtype=np.uint8)
        prev = cur
    return out.reshape(h, w, bpp)[:, :, :3]


def data_url_png(w: int, h: int, rgb: tuple, **kw) -> str:
    return "data:image/png;base64," + base64.b64encode(encode_png(w, h, rgb, **kw)).decode()
