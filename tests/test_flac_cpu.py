"""Native FLAC decoder against streams written by a small encoder in this file (every subframe kind, Rice partitions with
both parameter widths and an escape partition, wasted bits, the three stereo modes, several block-size codes)."""
import struct

import numpy as np
import pytest

from tensorrt_edge_llm_b200.runtime import native as rt


class Bits:
    def __init__(self):
        self.v, self.n = 0, 0

    def put(self, value, k):
        if k:
            self.v = (self.v << k) | (int(value) & ((1 << k) - 1))
            self.n += k

    def signed(self, value, k):
        self.put(int(value) & ((1 << k) - 1), k)

    def unary(self, zeros):
        self.put(1, zeros + 1)

    def pad(self):
        self.put(0, (-self.n) % 8)

    def bytes(self):
        assert self.n % 8 == 0
        return self.v.to_bytes(self.n // 8, "big") if self.n else b""


def _crc8(data):
    c = 0
    for b in data:
        c ^= b
        for _ in range(8):
            c = ((c << 1) ^ 0x07) & 0xFF if c & 0x80 else (c << 1) & 0xFF
    return c


def _residual(w, res, order, block, part_order=0, method=0, escape_first=False):
    pbits = 4 if method == 0 else 5
    w.put(method, 2)
    w.put(part_order, 4)
    parts = 1 << part_order
    i = 0
    for q in range(parts):
        count = (block >> part_order) - (order if q == 0 else 0) if part_order else block - order
        seg = res[i:i + count]
        i += count
        if escape_first and q == 0:
            w.put((1 << pbits) - 1, pbits)
            raw = max(int(np.abs(seg).max()).bit_length() + 1, 1) if len(seg) else 1
            w.put(raw, 5)
            for r in seg:
                w.signed(r, raw)
            continue
        mean = float(np.abs(seg).mean()) if len(seg) else 0.0
        k = min(max(int(np.log2(mean + 1)), 0), (1 << pbits) - 2)
        w.put(k, pbits)
        for r in seg:
            u = (int(r) << 1) ^ (int(r) >> 63)
            w.unary(u >> k)
            w.put(u & ((1 << k) - 1), k)


def _subframe(w, x, bps, kind, **kw):
    x = np.asarray(x, dtype=np.int64)
    block = len(x)
    wasted = kw.get("wasted", 0)
    if wasted:
        assert not np.any(x & ((1 << wasted) - 1))
        x = x >> wasted
        bps -= wasted
    w.put(0, 1)
    if kind == "constant":
        w.put(0, 6)
    elif kind == "verbatim":
        w.put(1, 6)
    elif kind == "fixed":
        w.put(8 + kw["order"], 6)
    else:
        w.put(31 + len(kw["coef"]), 6)
    w.put(1 if wasted else 0, 1)
    if wasted:
        w.unary(wasted - 1)
    if kind == "constant":
        w.signed(x[0], bps)
    elif kind == "verbatim":
        for v in x:
            w.signed(v, bps)
    elif kind == "fixed":
        order = kw["order"]
        for v in x[:order]:
            w.signed(v, bps)
        res = x.copy()
        for _ in range(order):
            res[1:] = res[1:] - res[:-1]              # repeated first differences = the fixed predictors' residuals
        _residual(w, res[order:], order, block, kw.get("part_order", 0), kw.get("method", 0), kw.get("escape_first", False))
    else:
        coef, shift, prec = kw["coef"], kw["shift"], kw["precision"]
        order = len(coef)
        for v in x[:order]:
            w.signed(v, bps)
        w.put(prec - 1, 4)
        w.signed(shift, 5)
        for c in coef:
            w.signed(c, prec)
        res = []
        for i in range(order, block):
            pred = sum(int(coef[j]) * int(x[i - 1 - j]) for j in range(order)) >> shift
            res.append(int(x[i]) - pred)
        _residual(w, np.asarray(res, dtype=np.int64), order, block, kw.get("part_order", 0), kw.get("method", 0))


def _frame(number, channels, bps, mode, subframes, block, bs_code=6):
    w = Bits()
    w.put(0b11111111111110, 14)
    w.put(0, 1)
    w.put(0, 1)
    w.put(bs_code, 4)
    w.put(0, 4)                                        # sample rate: from STREAMINFO
    w.put({"independent": len(channels) - 1, "left_side": 8, "side_right": 9, "mid_side": 10}[mode], 4)
    w.put(0, 3)                                        # sample size: from STREAMINFO
    w.put(0, 1)
    w.put(number, 8)                                   # frame numbers below 128 code as one byte
    if bs_code == 6:
        w.put(block - 1, 8)
    elif bs_code == 7:
        w.put(block - 1, 16)
    head = w.bytes()
    w.put(_crc8(head), 8)
    for c, (x, (kind, kw)) in enumerate(zip(channels, subframes)):
        side = (mode == "left_side" and c == 1) or (mode == "side_right" and c == 0) or (mode == "mid_side" and c == 1)
        _subframe(w, x, bps + (1 if side else 0), kind, **kw)
    w.pad()
    w.put(0, 16)                                       # frame CRC-16 (the decoder does not check it)
    return w.bytes()


def _stream(frames, rate, nch, bps, total):
    info = Bits()
    info.put(16, 16); info.put(4096, 16); info.put(0, 24); info.put(0, 24)
    info.put(rate, 20); info.put(nch - 1, 3); info.put(bps - 1, 5); info.put(total, 36)
    info.put(0, 128)
    body = info.bytes()
    padding = bytes([0x81, 0, 0, 4]) + b"\x00" * 4     # a PADDING block, flagged last
    return b"fLaC" + bytes([0x00]) + len(body).to_bytes(3, "big") + body + padding + b"".join(frames)


def test_mono_every_subframe_kind_and_rice_variant():
    rng = np.random.default_rng(0)
    t = np.arange(64)
    smooth = (3000 * np.sin(t / 5.0) + 40 * rng.standard_normal(64)).astype(np.int64)
    blocks = [
        (np.full(64, -1234), ("constant", {})),
        (rng.integers(-30000, 30000, 64), ("verbatim", {})),
        (smooth, ("fixed", {"order": 0})),
        (smooth, ("fixed", {"order": 1, "part_order": 2})),
        (smooth, ("fixed", {"order": 2, "method": 1})),
        (smooth, ("fixed", {"order": 3, "part_order": 1, "escape_first": True})),
        (smooth, ("fixed", {"order": 4, "part_order": 3})),
        (smooth, ("lpc", {"coef": [1900, -920], "shift": 10, "precision": 12})),
        (smooth, ("lpc", {"coef": [700, 300, -100, 50, -20, 10, 5, -3], "shift": 10, "precision": 15, "part_order": 2, "method": 1})),
        ((smooth >> 3) << 3, ("fixed", {"order": 2, "wasted": 3})),
    ]
    frames = [_frame(i, [x], 16, "independent", [sf], 64) for i, (x, sf) in enumerate(blocks)]
    want = np.concatenate([np.asarray(x, dtype=np.int64) for x, _ in blocks])
    clip = rt.parse_flac(_stream(frames, 16000, 1, 16, len(want)))
    got = np.asarray(clip.samples)
    assert clip.sample_rate == 16000 and got.shape == want.shape
    assert np.array_equal(np.round(got * 32768).astype(np.int64), want)
    assert np.array_equal(np.asarray(rt.parse_audio(_stream(frames, 16000, 1, 16, len(want))).samples), got)


@pytest.mark.parametrize("mode", ["independent", "left_side", "side_right", "mid_side"])
def test_stereo_decorrelation_modes_and_block_size_codes(mode):
    rng = np.random.default_rng(1)
    frames, lefts, rights = [], [], []
    for i, (block, code) in enumerate(((192, 1), (576, 2), (256, 8), (300, 7), (37, 6))):
        t = np.arange(block)
        left = (2000 * np.sin(t / 7.0 + i) + 30 * rng.standard_normal(block)).astype(np.int64)
        right = (left * 0.8 + 500 * np.cos(t / 11.0) + 20 * rng.standard_normal(block)).astype(np.int64)
        if mode == "independent":
            chans = [left, right]
        elif mode == "left_side":
            chans = [left, left - right]
        elif mode == "side_right":
            chans = [left - right, right]
        else:
            chans = [(left + right) >> 1, left - right]
        sub = [("fixed", {"order": 2}), ("fixed", {"order": 1, "method": 1})]
        frames.append(_frame(i, chans, 16, mode, sub, block, bs_code=code))
        lefts.append(left); rights.append(right)
    left, right = np.concatenate(lefts), np.concatenate(rights)
    clip = rt.parse_flac(_stream(frames, 44100, 2, 16, len(left)))
    assert clip.sample_rate == 44100
    assert np.allclose(np.asarray(clip.samples), (left + right) / 2.0 / 32768.0, atol=1e-7)


def test_malformed_streams_are_refused():
    x = np.arange(64) * 10
    good = _stream([_frame(0, [x], 16, "independent", [("fixed", {"order": 1})], 64)], 16000, 1, 16, 64)
    assert len(rt.parse_flac(good).samples) == 64
    for bad in (good[:20], b"RIFFxxxx" + good[8:], good[:60], good[:50] + b"\x12\x34" + good[52:]):
        with pytest.raises(RuntimeError):
            rt.parse_flac(bad)
    header_at = good.index(b"\xff\xf8")
    broken = bytearray(good)
    broken[header_at + 4] ^= 0x01                      # the coded frame number no longer matches the header CRC-8
    with pytest.raises(RuntimeError, match="checksum"):
        rt.parse_flac(bytes(broken))
    with pytest.raises(RuntimeError, match="MP3"):
        rt.parse_audio(b"ID3\x04" + b"\x00" * 40)
    with pytest.raises(RuntimeError, match="unknown audio"):
        rt.parse_audio(b"OggS" + b"\x00" * 40)
