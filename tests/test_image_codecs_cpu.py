"""Native PNG / JPEG / zlib decoders against Python's zlib and Pillow (used only as the oracle and to make test files)."""
import io
import zlib

import numpy as np
import pytest

from tensorrt_edge_llm_b200.runtime import native as rt

PIL = pytest.importorskip("PIL.Image")


def _img(h=37, w=53, seed=0):
    rng = np.random.default_rng(seed)
    yy, xx = np.mgrid[0:h, 0:w]
    base = np.stack([(xx * 255 // max(w - 1, 1)), (yy * 255 // max(h - 1, 1)), ((xx + yy) * 4 % 256)], -1).astype(np.int32)
    return np.clip(base + rng.integers(-20, 20, size=base.shape), 0, 255).astype(np.uint8)


def _pixels(im):
    return np.asarray(im.pixels, dtype=np.uint8).reshape(im.height, im.width, 3)


def _save(arr_or_img, fmt, **kw):
    im = arr_or_img if hasattr(arr_or_img, "save") else PIL.fromarray(arr_or_img)
    buf = io.BytesIO()
    im.save(buf, fmt, **kw)
    return buf.getvalue()


def test_inflate_matches_zlib():
    rng = np.random.default_rng(1)
    cases = [b"", b"a", b"hello hello hello hello " * 200, bytes(rng.integers(0, 256, 5000, dtype=np.uint8)),
             bytes(rng.integers(0, 4, 70000, dtype=np.uint8))]
    for data in cases:
        for level in (0, 1, 6, 9):              # stored, fixed-code and dynamic-code blocks
            assert rt.inflate_zlib(zlib.compress(data, level)) == data
    fixed = zlib.compressobj(6, zlib.DEFLATED, 15, 8, zlib.Z_FIXED)
    assert rt.inflate_zlib(fixed.compress(cases[2]) + fixed.flush()) == cases[2]
    with pytest.raises(RuntimeError):
        rt.inflate_zlib(zlib.compress(cases[2]), 100)                   # output bound
    with pytest.raises(RuntimeError):
        rt.inflate_zlib(zlib.compress(cases[2])[:-40])                  # truncated
    with pytest.raises(RuntimeError):
        rt.inflate_zlib(b"\x00\x01\x02\x03\x04\x05\x06")


def test_png_colour_types_and_depths():
    a = _img()
    for kw in ({}, {"compress_level": 0}, {"optimize": True}):
        im = rt.parse_image(_save(a, "PNG", **kw))
        assert (im.width, im.height, im.channels) == (53, 37, 3) and np.array_equal(_pixels(im), a)
    rgba = np.concatenate([a, np.full(a.shape[:2] + (1,), 200, np.uint8)], -1)
    assert np.array_equal(_pixels(rt.decode_png(_save(rgba, "PNG"))), a)               # alpha dropped
    grey = a[..., 0]
    assert np.array_equal(_pixels(rt.decode_png(_save(grey, "PNG")))[..., 1], grey)
    la = PIL.fromarray(grey).convert("LA")
    assert np.array_equal(_pixels(rt.decode_png(_save(la, "PNG")))[..., 2], grey)
    pal = PIL.fromarray(a).quantize(colors=16)                                          # 4-bit palette indices
    assert np.array_equal(_pixels(rt.decode_png(_save(pal, "PNG"))), np.asarray(pal.convert("RGB")))
    pal200 = PIL.fromarray(a).quantize(colors=200)                                      # 8-bit palette indices
    assert np.array_equal(_pixels(rt.decode_png(_save(pal200, "PNG"))), np.asarray(pal200.convert("RGB")))
    bw = PIL.fromarray(grey > 100)                                                      # 1-bit grey
    assert np.array_equal(_pixels(rt.decode_png(_save(bw, "PNG")))[..., 0], np.asarray(bw.convert("L")))
    g16 = PIL.fromarray((grey.astype(np.uint16) << 8) | 0x3c)                           # 16-bit grey keeps the high byte
    assert np.array_equal(_pixels(rt.decode_png(_save(g16, "PNG")))[..., 0], grey)


def test_png_every_row_filter(tmp_path):
    """Rows written with each of the five filter types (hand-built file: encoders pick filters adaptively)."""
    a = _img(10, 7, seed=3)
    h, w, _ = a.shape
    raw = bytearray()
    prev = np.zeros(w * 3, np.int32)
    for y in range(h):
        cur = a[y].reshape(-1).astype(np.int32)
        f = y % 5
        left = np.concatenate([np.zeros(3, np.int32), cur[:-3]])
        ul = np.concatenate([np.zeros(3, np.int32), prev[:-3]])
        if f == 0:
            enc = cur
        elif f == 1:
            enc = cur - left
        elif f == 2:
            enc = cur - prev
        elif f == 3:
            enc = cur - ((left + prev) >> 1)
        else:
            p = left + prev - ul
            pa, pb, pc = abs(p - left), abs(p - prev), abs(p - ul)
            pred = np.where((pa <= pb) & (pa <= pc), left, np.where(pb <= pc, prev, ul))
            enc = cur - pred
        raw += bytes([f]) + bytes((enc % 256).astype(np.uint8))
        prev = cur

    def chunk(t, d):
        import struct
        return struct.pack(">I", len(d)) + t + d + struct.pack(">I", zlib.crc32(t + d))
    import struct
    z = zlib.compress(bytes(raw))
    png = (b"\x89PNG\r\n\x1a\n" + chunk(b"IHDR", struct.pack(">IIBBBBB", w, h, 8, 2, 0, 0, 0)) + chunk(b"IDAT", z[:20]) + chunk(b"IDAT", z[20:])
           + chunk(b"IEND", b""))
    assert np.array_equal(np.asarray(PIL.open(io.BytesIO(png)).convert("RGB")), a)      # the file is a valid PNG
    assert np.array_equal(_pixels(rt.decode_png(png)), a)
    path = tmp_path / "x.png"
    path.write_bytes(png)
    assert np.array_equal(_pixels(rt.load_image(str(path))), a)
    with pytest.raises(RuntimeError):
        rt.decode_png(png[:60])


@pytest.mark.parametrize("shape,ctype", [((10, 7), 2), ((1, 1), 2), ((3, 9), 2), ((17, 33), 0), ((9, 5), 6), ((8, 8), 3)])
def test_png_adam7_interlaced(shape, ctype):
    """Adam7 files built by hand (seven reduced images, each filtered on its own; sizes that leave some passes empty), with
    Pillow as the oracle that the file is valid."""
    import struct
    h, w = shape
    a = _img(h, w, seed=h * w)
    if ctype == 2:
        px, depth = a, 8
    elif ctype == 6:
        px, depth = np.concatenate([a, np.full((h, w, 1), 77, np.uint8)], -1), 8
    elif ctype == 0:
        px, depth = a[..., :1], 8
    else:                                             # palette of 4 colours at 2 bits per index
        px, depth = (a[..., :1] // 64).astype(np.uint8), 2
    passes = [(0, 0, 8, 8), (4, 0, 8, 8), (0, 4, 4, 8), (2, 0, 4, 4), (0, 2, 2, 4), (1, 0, 2, 2), (0, 1, 1, 2)]
    raw = bytearray()
    for q, (x0, y0, dx, dy) in enumerate(passes):
        sub = px[y0::dy, x0::dx]
        if sub.shape[0] == 0 or sub.shape[1] == 0:
            continue
        prev = None
        for y in range(sub.shape[0]):
            if depth == 8:
                cur = sub[y].reshape(-1).astype(np.int32)
            else:                                     # pack 2-bit indices, most significant first
                idx = sub[y].reshape(-1)
                idx = np.concatenate([idx, np.zeros((-len(idx)) % 4, np.uint8)])
                cur = (idx[0::4] << 6 | idx[1::4] << 4 | idx[2::4] << 2 | idx[3::4]).astype(np.int32)
            f = 2 if (prev is not None and (y + q) % 2) else 0          # "up" filter on some rows, none on the others
            enc = cur - prev if f == 2 else cur
            raw += bytes([f]) + bytes((enc % 256).astype(np.uint8))
            prev = cur

    def chunk(t, d):
        return struct.pack(">I", len(d)) + t + d + struct.pack(">I", zlib.crc32(t + d))
    body = chunk(b"IHDR", struct.pack(">IIBBBBB", w, h, depth, ctype, 0, 0, 1))
    palette = bytes([10, 20, 30, 200, 100, 0, 0, 250, 120, 255, 255, 255])
    if ctype == 3:
        body += chunk(b"PLTE", palette)
    png = b"\x89PNG\r\n\x1a\n" + body + chunk(b"IDAT", zlib.compress(bytes(raw))) + chunk(b"IEND", b"")
    want = np.asarray(PIL.open(io.BytesIO(png)).convert("RGB"))
    if ctype == 2:
        assert np.array_equal(want, a)
    got = _pixels(rt.decode_png(png))
    assert got.shape == (h, w, 3) and np.array_equal(got, want)
    with pytest.raises(RuntimeError):
        rt.decode_png(png[:-30])                      # truncated image data


def test_jpeg_baseline_against_pillow():
    a = _img(70, 90, seed=5)
    smooth = np.asarray(PIL.fromarray(a).resize((45, 35)).resize((90, 70), PIL.BICUBIC))
    for sub, tol_mean, tol_max in ((0, 0.2, 4), (1, 0.6, 5), (2, 0.6, 5)):           # 4:4:4, 4:2:2, 4:2:0
        data = _save(smooth, "JPEG", quality=90, subsampling=sub)
        want = np.asarray(PIL.open(io.BytesIO(data)).convert("RGB")).astype(np.int32)
        got = _pixels(rt.parse_image(data)).astype(np.int32)
        assert got.shape == want.shape
        diff = np.abs(got - want)
        # differences are inverse-DCT and interpolation rounding only (chroma is interpolated with the same 3:1 triangle filter)
        assert diff.mean() < tol_mean and diff.max() <= tol_max, (sub, diff.mean(), diff.max())
    grey = _save(smooth[..., 0], "JPEG", quality=85)
    got = _pixels(rt.decode_jpeg(grey))
    want = np.asarray(PIL.open(io.BytesIO(grey)).convert("L")).astype(np.int32)
    assert np.abs(got[..., 0].astype(np.int32) - want).max() <= 2 and np.array_equal(got[..., 0], got[..., 2])
    # sizes that are not multiples of the MCU, optimised Huffman tables, restart intervals
    odd = smooth[:61, :77]
    for kw in ({"optimize": True}, {"restart_marker_blocks": 3}, {"restart_marker_rows": 1}):
        try:
            data = _save(odd, "JPEG", quality=80, subsampling=2, **kw)
        except TypeError:
            continue
        want = np.asarray(PIL.open(io.BytesIO(data)).convert("RGB")).astype(np.int32)
        got = _pixels(rt.decode_jpeg(data)).astype(np.int32)
        assert got.shape == (61, 77, 3) and np.abs(got - want).mean() < 0.8
    with pytest.raises(RuntimeError):
        rt.decode_jpeg(data[:200])
    with pytest.raises(RuntimeError, match="unsupported image container"):
        rt.parse_image(b"GIF89a" + b"\x00" * 64)


import struct as struct  # noqa: E402


def _patch_sos(data: bytes, edit) -> bytes:
    """Return ``data`` with its start-of-scan header bytes changed by ``edit(header bytearray)``."""
    b = bytearray(data)
    i = b.find(b"\xff\xda")
    n = (b[i + 2] << 8) | b[i + 3]
    hdr = b[i + 4:i + 2 + n]
    edit(hdr)
    b[i + 4:i + 2 + n] = hdr
    return bytes(b)


def test_jpeg_progressive_against_pillow():
    """Progressive frames (spectral selection and successive approximation over several scans) decode to the same
    pixels as the baseline form of the same coefficients would: compared with Pillow's decode of the same bytes."""
    rng = np.random.default_rng(11)
    yy, xx = np.mgrid[0:97, 0:131]
    smooth = np.stack([(xx * 2) % 256, (yy * 3) % 256, ((xx + yy) * 1.5) % 256], -1).astype(np.uint8)
    noisy = np.clip(smooth.astype(np.int32) + rng.integers(-40, 40, smooth.shape), 0, 255).astype(np.uint8)
    for img, sub, quality, tol_mean in ((smooth, 0, 92, 0.3), (noisy, 2, 75, 0.8), (noisy, 1, 50, 0.8), (smooth[:8, :8], 2, 90, 1.5)):
        data = _save(img, "JPEG", quality=quality, subsampling=sub, progressive=True)
        assert b"\xff\xc2" in data                                   # a progressive frame header
        want = np.asarray(PIL.open(io.BytesIO(data)).convert("RGB")).astype(np.int32)
        got = _pixels(rt.decode_jpeg(data)).astype(np.int32)
        assert got.shape == want.shape
        diff = np.abs(got - want)
        assert diff.mean() < tol_mean and diff.max() <= 6, (sub, quality, diff.mean(), diff.max())
    for kw in ({"restart_marker_blocks": 3}, {"restart_marker_rows": 1}):     # restart intervals inside every scan
        try:
            data = _save(noisy, "JPEG", quality=60, subsampling=2, progressive=True, **kw)
        except TypeError:
            continue
        want = np.asarray(PIL.open(io.BytesIO(data)).convert("RGB")).astype(np.int32)
        assert np.abs(_pixels(rt.decode_jpeg(data)).astype(np.int32) - want).mean() < 0.8
    grey = _save(noisy[..., 0], "JPEG", quality=70, progressive=True)
    got = _pixels(rt.decode_jpeg(grey))
    want = np.asarray(PIL.open(io.BytesIO(grey)).convert("L")).astype(np.int32)
    assert np.abs(got[..., 0].astype(np.int32) - want).max() <= 2
    # a cut-off progressive file and one whose scan parameters are impossible both raise
    with pytest.raises(RuntimeError):
        rt.decode_jpeg(data[:150])
    sos = data.index(b"\xff\xda")
    ns = data[sos + 4]
    broken = bytearray(data)
    broken[sos + 5 + 2 * ns] = 9                                     # spectral start > spectral end
    broken[sos + 6 + 2 * ns] = 3
    with pytest.raises(RuntimeError):
        rt.decode_jpeg(bytes(broken))


def test_jpeg_malformed_scan_headers_raise_cleanly():
    """Crafted files from untrusted requests: a scan that names one component twice (leaving another on tables that were
    never defined), a frame header with duplicate ids, a header that promises more data than the file holds, and sizes
    beyond the pixel cap all end in an exception, never in an out-of-bounds read or an endless decode."""
    a = _img(32, 48, seed=9)
    data = _save(a, "JPEG", quality=80, subsampling=0)

    def dup_component(h):          # ns=3: make the third entry name the first component again, with table ids 3/3
        h[5] = h[1]
        h[6] = 0x33
    with pytest.raises(RuntimeError, match="twice|not defined"):
        rt.decode_jpeg(_patch_sos(data, dup_component))

    def undefined_tables(h):       # second component on Huffman tables 2/2, which the file never defines
        h[4] = 0x22
    with pytest.raises(RuntimeError, match="not defined"):
        rt.decode_jpeg(_patch_sos(data, undefined_tables))
    b = bytearray(data)
    i = b.find(b"\xff\xc0")
    b[i + 13] = b[i + 10]            # SOF: second component id := first component id
    with pytest.raises(RuntimeError, match="twice"):
        rt.decode_jpeg(bytes(b))
    # a header that claims a far larger image than the scan data covers: must stop, not decode zeros for megapixels
    big = bytearray(data)
    big[i + 5:i + 9] = struct.pack(">HH", 4000, 4000)
    with pytest.raises(RuntimeError, match="ends before"):
        rt.decode_jpeg(bytes(big))
    huge = bytearray(data)
    huge[i + 5:i + 9] = struct.pack(">HH", 32000, 32000)
    with pytest.raises(RuntimeError, match="limit"):
        rt.decode_jpeg(bytes(huge))
    with pytest.raises(RuntimeError, match="limit|range"):
        rt.parse_image(b"P6\n30000 30000\n255\n" + b"\x00" * 64)
