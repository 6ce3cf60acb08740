"""Independent reader of the reference's v7 container, for the sync tests.

Restates the loader of turbovec/src/io_v7.rs (`load_image` :1293-1580, `parse_header_at` :1143-1222,
`delta_verified` :843-858) in numpy: superblock, the two alternating commit headers, the delta check that makes
a commit adoptable, the tail rows and the pending redo ops.  Test infrastructure only.
"""
import struct

import numpy as np

MAX_OPS = 1024
BLK = 32


def crc32c(lib, data: bytes) -> int:
    buf = np.frombuffer(data, np.uint8)
    return int(lib.tv_crc32c(buf.ctypes.data, buf.size)) & 0xFFFFFFFF


class Geo:
    def __init__(self, kind, dim, bits, n_calib):
        self.kind, self.dim, self.bits, self.n_calib = kind, dim, bits, n_calib
        self.rb = dim // (8 // bits)
        levels = 1 << bits
        self.idb = 8 if kind == 1 else 0
        self.sb_len = 23 + (levels - 1) * 4 + levels * 4 + 4 + n_calib * 8 + 4
        self.op_size = 1 + self.rb + 4 + self.idb
        self.hdr_len = 16 + 31 * (self.rb + 4 + self.idb) + 4 + MAX_OPS * (5 + self.op_size) + 4 + MAX_OPS * 4 + 12 + 4
        self.unit_len = BLK * self.rb + BLK * 4 + BLK * self.idb

    def hdr_at(self, slot):
        return self.sb_len + slot * self.hdr_len

    def unit_at(self, block):
        return self.hdr_at(2) + block * self.unit_len


def _parse_header(lib, raw, geo, slot):
    at = geo.hdr_at(slot)
    b = raw[at: at + geo.hdr_len]
    if len(b) < 16:
        return None
    gen, n = struct.unpack_from("<QQ", b, 0)
    if gen % 2 != slot or geo.unit_at(n // BLK) > len(raw):
        return None
    tail_row = geo.rb + 4 + geo.idb
    p = 16 + (n % BLK) * tail_row
    try:
        (n_groups,) = struct.unpack_from("<I", b, p)
        if n_groups > MAX_OPS:
            return None
        p += 4
        ops = []
        for _ in range(n_groups):
            blk, n_ops = struct.unpack_from("<IB", b, p)
            if blk >= n // BLK:
                return None
            p += 5
            for _ in range(n_ops):
                lane = b[p]
                if lane >= BLK:
                    return None
                ops.append((blk * BLK + lane, at + p + 1))
                p += geo.op_size
        (n_mat,) = struct.unpack_from("<I", b, p)
        if n_mat > MAX_OPS:
            return None
        p += 4
        mat = list(struct.unpack_from(f"<{n_mat}I", b, p))
        p += 4 * n_mat
        app_from, app_to, delta_crc = struct.unpack_from("<III", b, p)
        p += 12
        (stored,) = struct.unpack_from("<I", b, p)
    except struct.error:
        return None
    if crc32c(lib, bytes(b[:p])) != stored:
        return None
    return {"gen": gen, "n": n, "tail_at": at + 16, "ops": ops, "mat": mat, "app": (app_from, app_to),
            "delta_crc": delta_crc, "used": p + 4, "slot": slot}


def _delta_ok(lib, raw, geo, h):
    units = h["mat"] + list(range(h["app"][0], h["app"][1]))
    parts = [struct.pack("<Q", h["gen"])]
    for u in units:
        at = geo.unit_at(u)
        if at + geo.unit_len > len(raw):
            return False
        parts.append(struct.pack("<I", u))
        parts.append(bytes(raw[at: at + geo.unit_len]))
    return crc32c(lib, b"".join(parts)) == h["delta_crc"]


def read(lib, raw: bytes):
    """Parses a v7 image; returns a dict with the adopted commit's state, or raises ValueError."""
    if raw[:4] != b"TV7\0" or raw[4] != 2:
        raise ValueError("not a v7 revision-2 file")
    bits, kind = raw[5], raw[6]
    (dim,) = struct.unpack_from("<I", raw, 7)
    (nonce,) = struct.unpack_from("<Q", raw, 11)
    (max_ops,) = struct.unpack_from("<I", raw, 19)
    assert max_ops == MAX_OPS
    levels = 1 << bits
    off = 23 + (2 * levels - 1) * 4
    (n_calib,) = struct.unpack_from("<I", raw, off)
    off += 4
    shift = np.frombuffer(raw, "<f4", n_calib, off).copy()
    scale = np.frombuffer(raw, "<f4", n_calib, off + 4 * n_calib).copy()
    off += 8 * n_calib
    (stored,) = struct.unpack_from("<I", raw, off)
    if crc32c(lib, raw[:off]) != stored:
        raise ValueError("corrupt superblock")
    geo = Geo(kind, dim, bits, n_calib)
    cands = [h for h in (_parse_header(lib, raw, geo, 0), _parse_header(lib, raw, geo, 1)) if h]
    cands.sort(key=lambda h: -h["gen"])
    newest = cands[0]["gen"] if cands else None
    chosen = next((h for h in cands if _delta_ok(lib, raw, geo, h)), None)
    if chosen is None:
        raise ValueError("no valid commit header")
    n, rb = chosen["n"], geo.rb
    nb, total = n // BLK, -(-n // BLK)
    codes = np.zeros((total, rb, BLK), np.uint8)
    scales = np.zeros(total * BLK, np.float32)
    ids = np.zeros(total * BLK, np.uint64)
    for b in range(nb):
        at = geo.unit_at(b)
        codes[b] = np.frombuffer(raw, np.uint8, rb * BLK, at).reshape(rb, BLK)
        scales[b * BLK:(b + 1) * BLK] = np.frombuffer(raw, "<f4", BLK, at + rb * BLK)
        if kind == 1:
            ids[b * BLK:(b + 1) * BLK] = np.frombuffer(raw, "<u8", BLK, at + rb * BLK + BLK * 4)

    def place(slot, at):
        codes[slot // BLK, :, slot % BLK] = np.frombuffer(raw, np.uint8, rb, at)
        scales[slot] = np.frombuffer(raw, "<f4", 1, at + rb)[0]
        if kind == 1:
            ids[slot] = np.frombuffer(raw, "<u8", 1, at + rb + 4)[0]

    for slot, at in chosen["ops"]:
        place(slot, at)
    tail_row = rb + 4 + geo.idb
    for k in range(n % BLK):
        place(nb * BLK + k, chosen["tail_at"] + k * tail_row)
    return {"geo": geo, "nonce": nonce, "gen": chosen["gen"], "newest": newest, "n": n, "slot": chosen["slot"],
            "codes": codes, "scales": scales[:n], "ids": ids[:n] if kind == 1 else None, "shift": shift, "scale": scale,
            "pending": sorted(s for s, _ in chosen["ops"]), "mat": chosen["mat"], "app": chosen["app"],
            "used": chosen["used"]}
