// Huffman JPEG decoder (ITU T.81 baseline / extended sequential and progressive, 8-bit samples).
//
// Flow: markers → quantisation tables (DQT), Huffman tables (DHT), frame header (SOF0 / SOF1 / SOF2), restart interval
// (DRI) → for every MCU of the scan: per component block, a DC difference and run-length coded AC coefficients in zig-zag
// order → dequantise → 8×8 inverse DCT → planes → chroma interpolated up to the luma grid → YCbCr → RGB.
// A progressive frame spreads each block's coefficients over several scans (a band of the zig-zag order, high bits first
// and single correction bits later); its scans are merged into a coefficient store and transformed after the last one.
// Counterpart in the reference: the stb_image header behind cpp/runtime/imageUtils.cpp.
#include "media.h"

#include <algorithm>
#include <array>
#include <cmath>
#include <cstring>
#include <stdexcept>

namespace telb {
namespace {

[[noreturn]] void bad(const char* what) { throw std::runtime_error(what); }

const uint8_t kZigzag[64] = {0,  1,  8,  16, 9,  2,  3,  10, 17, 24, 32, 25, 18, 11, 4,  5,  12, 19, 26, 33, 40, 48,
                             41, 34, 27, 20, 13, 6,  7,  14, 21, 28, 35, 42, 49, 56, 57, 50, 43, 36, 29, 22, 15, 23,
                             30, 37, 44, 51, 58, 59, 52, 45, 38, 31, 39, 46, 53, 60, 61, 54, 47, 55, 62, 63};

struct JHuff {
    bool set = false;
    std::array<int, 18> mincode{}, maxcode{}, valptr{};
    std::vector<uint8_t> vals;
    JHuff() { maxcode.fill(-1); }                    // a table that was never defined matches no code
    void build(const uint8_t* counts, const uint8_t* symbols, int total) {
        vals.assign(symbols, symbols + total);
        int code = 0, k = 0;
        for (int len = 1; len <= 16; ++len) {
            valptr[len] = k;
            mincode[len] = code;
            code += counts[len - 1];
            k += counts[len - 1];
            maxcode[len] = counts[len - 1] ? code - 1 : -1;
            code <<= 1;
        }
        set = true;
    }
};

struct BitsMsb {
    const uint8_t* p;
    size_t n, at;
    uint32_t buf = 0;
    int cnt = 0;
    bool hit_marker = false;
    int pad_bytes = 0;                  // zero bytes fed after the scan's data ended
    int bit() {
        if (cnt == 0) {
            uint8_t b = 0;
            // a decoder may read a little past the last data byte (a final code completed by padding); a file whose
            // header promises far more blocks than its data holds must fail instead of decoding zeros for ever
            if ((hit_marker || at >= n) && ++pad_bytes > 16) bad("JPEG scan data ends before the image is complete");
            if (!hit_marker && at < n) {
                b = p[at];
                if (b == 0xff) {
                    if (at + 1 < n && p[at + 1] == 0x00) {
                        at += 2;                                 // stuffed zero after a data byte of 0xff
                    } else {
                        hit_marker = true;                       // a marker: the scan's data is over, feed zeros
                        b = 0;
                    }
                } else {
                    ++at;
                }
            }
            buf = b;
            cnt = 8;
        }
        --cnt;
        return (buf >> cnt) & 1;
    }
    int bits(int k) {
        int v = 0;
        for (int i = 0; i < k; ++i) v = (v << 1) | bit();
        return v;
    }
    void reset() { cnt = 0; hit_marker = false; pad_bytes = 0; }
};

int decode_symbol(BitsMsb& s, const JHuff& h) {
    int code = 0;
    for (int len = 1; len <= 16; ++len) {
        code = (code << 1) | s.bit();
        if (h.maxcode[len] >= 0 && code <= h.maxcode[len] && code >= h.mincode[len]) {
            const size_t idx = static_cast<size_t>(h.valptr[len] + code - h.mincode[len]);
            if (idx >= h.vals.size()) break;          // over-subscribed table: the code has no symbol
            return h.vals[idx];
        }
    }
    bad("invalid Huffman code in a JPEG scan");
}

inline int extend(int v, int bits) { return bits && v < (1 << (bits - 1)) ? v - (1 << bits) + 1 : v; }

struct Component {
    int id = 0, h = 1, v = 1, tq = 0, td = 0, ta = 0, pred = 0;
    int stride = 0, rows = 0;
    std::vector<uint8_t> plane;
    // progressive frames: every block's coefficients (natural order, not yet dequantised) live until the last scan
    int bw = 0, bh = 0;
    std::vector<int16_t> coef;
};

void idct8x8(const float* in, uint8_t* out, int stride) {
    // function-local static initialised by a lambda: the language guarantees one initialisation even when several
    // requests decode images at the same time
    static const std::array<std::array<float, 8>, 8> c = [] {
        std::array<std::array<float, 8>, 8> t{};
        for (int x = 0; x < 8; ++x)
            for (int u = 0; u < 8; ++u) t[x][u] = (u == 0 ? std::sqrt(0.125f) : 0.5f) * std::cos((2 * x + 1) * u * 3.14159265358979323846f / 16);
        return t;
    }();
    float tmp[64];
    for (int y = 0; y < 8; ++y)                      // rows: sum over horizontal frequency u
        for (int x = 0; x < 8; ++x) {
            float s = 0;
            for (int u = 0; u < 8; ++u) s += c[x][u] * in[y * 8 + u];
            tmp[y * 8 + x] = s;
        }
    for (int x = 0; x < 8; ++x)                      // columns: sum over vertical frequency v
        for (int y = 0; y < 8; ++y) {
            float s = 0;
            for (int v = 0; v < 8; ++v) s += c[y][v] * tmp[v * 8 + x];
            const int q = static_cast<int>(std::lround(s + 128.f));
            out[y * stride + x] = static_cast<uint8_t>(std::min(std::max(q, 0), 255));
        }
}

// One scan of a progressive frame (ITU-T T.81 annex G): spectral selection ``ss..se`` and successive approximation
// ``ah/al``.  DC scans may interleave several components; an AC scan holds one component and walks that component's own
// block grid (the blocks that cover its samples, not the MCU-padded grid).  Returns the offset of the byte after the
// scan's entropy-coded data.
size_t decode_progressive_scan(const uint8_t* p, size_t n, size_t start, const std::vector<Component*>& sc, int ss, int se, int ah,
                               int al, const std::array<JHuff, 4>& dc, const std::array<JHuff, 4>& ac, int width, int height,
                               int hmax, int vmax, int mcux, int mcuy, int restart) {
    if (ss > se || se > 63 || al > 13 || (ah != 0 && ah != al + 1)) bad("bad JPEG progressive scan parameters");
    if (ss == 0 && se != 0) bad("a JPEG progressive scan mixes DC and AC coefficients");
    if (ss > 0 && sc.size() != 1) bad("a JPEG progressive AC scan must hold one component");
    for (const Component* c : sc) {
        if (ss == 0 && ah == 0 && (c->td > 3 || !dc[c->td].set)) bad("JPEG scan uses a Huffman table that was not defined");
        if (ss > 0 && (c->ta > 3 || !ac[c->ta].set)) bad("JPEG scan uses a Huffman table that was not defined");
    }
    BitsMsb s{p, n, start};
    int eobrun = 0, until_restart = restart;
    const int p1 = 1 << al, m1 = -(1 << al);

    auto restart_if_due = [&]() {
        if (!restart) return;
        if (until_restart == 0) {
            s.reset();
            while (s.at + 1 < n && !(p[s.at] == 0xff && p[s.at + 1] >= 0xd0 && p[s.at + 1] <= 0xd7)) ++s.at;
            if (s.at + 1 >= n) bad("JPEG restart marker missing");
            s.at += 2;
            for (Component* c : sc) c->pred = 0;
            eobrun = 0;
            until_restart = restart;
        }
        --until_restart;
    };
    auto refine = [&](int16_t& v) {                       // one correction bit for a coefficient that is already non-zero
        if (s.bit() && (v & p1) == 0) v = static_cast<int16_t>(v + (v >= 0 ? p1 : m1));
    };
    auto block = [&](Component& c, int16_t* blk) {
        if (ss == 0) {
            if (ah == 0) {
                const int t = decode_symbol(s, dc[c.td]);
                if (t > 11) bad("bad JPEG DC category");
                c.pred += extend(s.bits(t), t);
                blk[0] = static_cast<int16_t>(c.pred * p1);
            } else if (s.bit()) {
                blk[0] = static_cast<int16_t>(blk[0] | p1);
            }
            return;
        }
        if (ah == 0) {                                    // first pass over this band
            if (eobrun > 0) { --eobrun; return; }
            for (int k = ss; k <= se; ++k) {
                const int rs = decode_symbol(s, ac[c.ta]);
                const int r = rs >> 4, sz = rs & 15;
                if (sz == 0) {
                    if (r < 15) {                         // end of band for this block and 2^r - 1 + extra following ones
                        eobrun = (1 << r) - 1;
                        if (r) eobrun += s.bits(r);
                        break;
                    }
                    k += 15;                              // sixteen zeros
                    continue;
                }
                k += r;
                if (k > 63) bad("JPEG AC run leaves the block");
                blk[kZigzag[k]] = static_cast<int16_t>(extend(s.bits(sz), sz) * p1);
            }
            return;
        }
        int k = ss;                                       // refinement pass
        if (eobrun == 0) {
            for (; k <= se; ++k) {
                const int rs = decode_symbol(s, ac[c.ta]);
                int r = rs >> 4, val = 0;
                if (rs & 15) {
                    if ((rs & 15) != 1) bad("bad JPEG refinement symbol");
                    val = s.bit() ? p1 : m1;              // a coefficient that becomes non-zero in this pass
                } else if (r != 15) {
                    eobrun = 1 << r;                      // counts this block too
                    if (r) eobrun += s.bits(r);
                    break;
                }
                // step over r coefficients whose history is zero, correcting the non-zero ones passed on the way
                while (k <= se) {
                    int16_t& v = blk[kZigzag[k]];
                    if (v != 0) refine(v);
                    else if (--r < 0) break;
                    ++k;
                }
                if (val) {
                    if (k > 63) bad("JPEG AC run leaves the block");
                    blk[kZigzag[k]] = static_cast<int16_t>(val);
                }
            }
        }
        if (eobrun > 0) {
            for (; k <= se; ++k) {
                int16_t& v = blk[kZigzag[k]];
                if (v != 0) refine(v);
            }
            --eobrun;
        }
    };

    for (Component* c : sc) c->pred = 0;
    if (sc.size() > 1) {
        for (int my = 0; my < mcuy; ++my)
            for (int mx = 0; mx < mcux; ++mx) {
                restart_if_due();
                for (Component* c : sc)
                    for (int by = 0; by < c->v; ++by)
                        for (int bx = 0; bx < c->h; ++bx)
                            block(*c, &c->coef[(static_cast<size_t>(my * c->v + by) * c->bw + mx * c->h + bx) * 64]);
            }
    } else {
        Component& c = *sc[0];
        const int cw = (width * c.h + hmax - 1) / hmax, ch = (height * c.v + vmax - 1) / vmax;
        const int nbx = (cw + 7) / 8, nby = (ch + 7) / 8;
        for (int by = 0; by < nby; ++by)
            for (int bx = 0; bx < nbx; ++bx) {
                restart_if_due();
                block(c, &c.coef[(static_cast<size_t>(by) * c.bw + bx) * 64]);
            }
    }
    // the next segment starts at the first marker that is neither a stuffed zero nor a restart marker
    size_t at = s.at;
    while (at + 1 < n && !(p[at] == 0xff && p[at + 1] != 0x00 && p[at + 1] != 0xff && !(p[at + 1] >= 0xd0 && p[at + 1] <= 0xd7))) ++at;
    return at;
}

}  // namespace

Image decode_jpeg(const std::string& bytes) {
    const uint8_t* p = reinterpret_cast<const uint8_t*>(bytes.data());
    const size_t n = bytes.size();
    if (n < 4 || p[0] != 0xff || p[1] != 0xd8) bad("not a JPEG file");
    std::array<std::array<uint16_t, 64>, 4> qt{};
    std::array<JHuff, 4> dc, ac;
    std::vector<Component> comps;
    int width = 0, height = 0, restart = 0, adobe_transform = -1;
    size_t at = 2;
    bool decoded = false, progressive = false, any_scan = false;
    while (at + 4 <= n && !decoded) {
        if (p[at] != 0xff) { ++at; continue; }
        const int marker = p[at + 1];
        if (marker == 0xff) { ++at; continue; }       // fill bytes
        at += 2;
        if (marker == 0xd8 || marker == 0x01 || (marker >= 0xd0 && marker <= 0xd7)) continue;
        if (marker == 0xd9) break;
        if (at + 2 > n) bad("truncated JPEG segment");
        const size_t len = (p[at] << 8) | p[at + 1];
        if (len < 2 || at + len > n) bad("truncated JPEG segment");
        const uint8_t* d = p + at + 2;
        const size_t dn = len - 2;
        if (marker == 0xdb) {                                           // DQT
            size_t i = 0;
            while (i < dn) {
                const int pq = d[i] >> 4, tq = d[i] & 15;
                ++i;
                if (tq > 3 || i + (pq ? 128 : 64) > dn) bad("bad JPEG quantisation table");
                for (int k = 0; k < 64; ++k) {
                    qt[tq][kZigzag[k]] = pq ? static_cast<uint16_t>((d[i] << 8) | d[i + 1]) : d[i];
                    i += pq ? 2 : 1;
                }
            }
        } else if (marker == 0xc4) {                                    // DHT
            size_t i = 0;
            while (i + 17 <= dn) {
                const int tc = d[i] >> 4, th = d[i] & 15;
                int total = 0;
                for (int k = 0; k < 16; ++k) total += d[i + 1 + k];
                if (tc > 1 || th > 3 || total > 256 || i + 17 + total > dn) bad("bad JPEG Huffman table");
                (tc ? ac : dc)[th].build(d + i + 1, d + i + 17, total);
                i += 17 + total;
            }
        } else if (marker == 0xc0 || marker == 0xc1 || marker == 0xc2) { // SOF0 / SOF1 / SOF2 (progressive)
            if (!comps.empty()) bad("JPEG file with more than one frame header");
            progressive = marker == 0xc2;
            if (dn < 6 || d[0] != 8) bad("only 8-bit JPEG images are read");
            height = (d[1] << 8) | d[2];
            width = (d[3] << 8) | d[4];
            const int nc = d[5];
            if ((nc != 1 && nc != 3) || dn < 6 + 3 * static_cast<size_t>(nc)) bad("JPEG images with one or three components are read");
            if (width <= 0 || height <= 0 || width > (1 << 15) || height > (1 << 15)) bad("JPEG size out of range");
            if (static_cast<uint64_t>(width) * static_cast<uint64_t>(height) > max_image_pixels()) bad("JPEG image has more pixels than the decoder's limit");
            comps.assign(nc, Component());
            for (int k = 0; k < nc; ++k) {
                comps[k].id = d[6 + 3 * k];
                comps[k].h = d[7 + 3 * k] >> 4;
                comps[k].v = d[7 + 3 * k] & 15;
                comps[k].tq = d[8 + 3 * k];
                if (comps[k].h < 1 || comps[k].h > 2 || comps[k].v < 1 || comps[k].v > 2 || comps[k].tq > 3) bad("JPEG sampling factors other than 1 and 2 are not read");
                for (int j = 0; j < k; ++j)
                    if (comps[j].id == comps[k].id) bad("JPEG frame header names a component twice");
            }
        } else if (marker >= 0xc3 && marker <= 0xcf && marker != 0xc4 && marker != 0xc8 && marker != 0xcc) {
            bad("this JPEG coding process (lossless, hierarchical or arithmetic) is not read");
        } else if (marker == 0xdd) {                                    // DRI
            if (dn < 2) bad("bad JPEG restart interval");
            restart = (d[0] << 8) | d[1];
        } else if (marker == 0xee) {                                    // APP14 "Adobe": colour transform flag
            if (dn >= 12 && !std::memcmp(d, "Adobe", 5)) adobe_transform = d[11];
        } else if (marker == 0xda && progressive) {                     // SOS of a progressive frame: one of many scans
            if (dn < 1) bad("truncated JPEG scan header");
            const int ns = d[0];
            if (ns < 1 || ns > static_cast<int>(comps.size()) || dn < 1 + 2 * static_cast<size_t>(ns) + 3) bad("bad JPEG scan header");
            int hmax = 1, vmax = 1;
            for (auto& c : comps) { hmax = std::max(hmax, c.h); vmax = std::max(vmax, c.v); }
            const int mcux = (width + 8 * hmax - 1) / (8 * hmax), mcuy = (height + 8 * vmax - 1) / (8 * vmax);
            if (!any_scan)
                for (auto& c : comps) {
                    c.bw = mcux * c.h;
                    c.bh = mcuy * c.v;
                    c.coef.assign(static_cast<size_t>(c.bw) * c.bh * 64, 0);
                }
            std::vector<Component*> sc;
            for (int k = 0; k < ns; ++k) {
                const int id = d[1 + 2 * k];
                auto it = std::find_if(comps.begin(), comps.end(), [&](const Component& c) { return c.id == id; });
                if (it == comps.end()) bad("JPEG scan names an unknown component");
                if (std::find(sc.begin(), sc.end(), &*it) != sc.end()) bad("JPEG scan names a component twice");
                it->td = d[2 + 2 * k] >> 4;
                it->ta = d[2 + 2 * k] & 15;
                sc.push_back(&*it);
            }
            const uint8_t* tail = d + 1 + 2 * ns;
            at = decode_progressive_scan(p, n, at + len, sc, tail[0], tail[1], tail[2] >> 4, tail[2] & 15, dc, ac, width, height, hmax,
                                         vmax, mcux, mcuy, restart);
            any_scan = true;
            continue;
        } else if (marker == 0xda) {                                    // SOS: decode the (single) scan
            if (comps.empty()) bad("JPEG scan before its frame header");
            const int ns = d[0];
            if (ns != static_cast<int>(comps.size()) || dn < 1 + 2 * static_cast<size_t>(ns) + 3) bad("JPEG scans must hold every component (non-interleaved scans are not read)");
            std::vector<uint8_t> assigned(comps.size(), 0);
            for (int k = 0; k < ns; ++k) {
                const int id = d[1 + 2 * k];
                auto it = std::find_if(comps.begin(), comps.end(), [&](const Component& c) { return c.id == id; });
                if (it == comps.end()) bad("JPEG scan names an unknown component");
                if (assigned[it - comps.begin()]) bad("JPEG scan names a component twice");
                assigned[it - comps.begin()] = 1;
                it->td = d[2 + 2 * k] >> 4;
                it->ta = d[2 + 2 * k] & 15;
            }
            for (const auto& c : comps)      // every component, not only the ones the scan header happened to name
                if (c.td > 3 || c.ta > 3 || !dc[c.td].set || !ac[c.ta].set) bad("JPEG scan uses a Huffman table that was not defined");
            int hmax = 1, vmax = 1;
            for (auto& c : comps) { hmax = std::max(hmax, c.h); vmax = std::max(vmax, c.v); }
            const int mcux = (width + 8 * hmax - 1) / (8 * hmax), mcuy = (height + 8 * vmax - 1) / (8 * vmax);
            for (auto& c : comps) {
                c.stride = mcux * c.h * 8;
                c.rows = mcuy * c.v * 8;
                c.plane.assign(static_cast<size_t>(c.stride) * c.rows, 0);
                c.pred = 0;
            }
            BitsMsb s{p, n, at + len};
            int until_restart = restart;
            float block[64];
            for (int my = 0; my < mcuy; ++my)
                for (int mx = 0; mx < mcux; ++mx) {
                    if (restart && until_restart == 0) {
                        // byte-align, step over the RSTn marker, reset the DC predictors
                        s.reset();
                        while (s.at + 1 < n && !(p[s.at] == 0xff && p[s.at + 1] >= 0xd0 && p[s.at + 1] <= 0xd7)) ++s.at;
                        if (s.at + 1 >= n) bad("JPEG restart marker missing");
                        s.at += 2;
                        for (auto& c : comps) c.pred = 0;
                        until_restart = restart;
                    }
                    for (auto& c : comps)
                        for (int by = 0; by < c.v; ++by)
                            for (int bx = 0; bx < c.h; ++bx) {
                                std::fill(block, block + 64, 0.f);
                                const int t = decode_symbol(s, dc[c.td]);
                                if (t > 11) bad("bad JPEG DC category");
                                c.pred += extend(s.bits(t), t);
                                block[0] = static_cast<float>(c.pred) * qt[c.tq][0];
                                for (int k = 1; k < 64;) {
                                    const int rs = decode_symbol(s, ac[c.ta]);
                                    const int r = rs >> 4, sz = rs & 15;
                                    if (sz == 0) {
                                        if (r == 15) { k += 16; continue; }
                                        break;                         // end of block
                                    }
                                    k += r;
                                    if (k > 63) bad("JPEG AC run leaves the block");
                                    const int z = kZigzag[k];
                                    block[z] = static_cast<float>(extend(s.bits(sz), sz)) * qt[c.tq][z];
                                    ++k;
                                }
                                const int x0 = (mx * c.h + bx) * 8, y0 = (my * c.v + by) * 8;
                                idct8x8(block, &c.plane[static_cast<size_t>(y0) * c.stride + x0], c.stride);
                            }
                    if (restart) --until_restart;
                }
            decoded = true;
        }
        at += len;
    }
    if (progressive && any_scan) {
        // every scan has been merged into the coefficient store: dequantise and transform each block once
        float block[64];
        for (auto& c : comps) {
            c.stride = c.bw * 8;
            c.rows = c.bh * 8;
            c.plane.assign(static_cast<size_t>(c.stride) * c.rows, 0);
            for (int by = 0; by < c.bh; ++by)
                for (int bx = 0; bx < c.bw; ++bx) {
                    const int16_t* blk = &c.coef[(static_cast<size_t>(by) * c.bw + bx) * 64];
                    for (int z = 0; z < 64; ++z) block[z] = static_cast<float>(blk[z]) * qt[c.tq][z];
                    idct8x8(block, &c.plane[static_cast<size_t>(by) * 8 * c.stride + bx * 8], c.stride);
                }
            c.coef.clear();
            c.coef.shrink_to_fit();
        }
        decoded = true;
    }
    if (!decoded) bad("JPEG file without image data");
    int hmax = 1, vmax = 1;
    for (auto& c : comps) { hmax = std::max(hmax, c.h); vmax = std::max(vmax, c.v); }
    Image im;
    im.width = width;
    im.height = height;
    im.channels = 3;
    im.pixels.resize(static_cast<size_t>(width) * height * 3);
    const bool ycc = comps.size() == 3 && adobe_transform != 0;
    for (int y = 0; y < height; ++y)
        for (int x = 0; x < width; ++x) {
            int v[3] = {0, 128, 128};
            for (size_t k = 0; k < comps.size(); ++k) {
                const Component& c = comps[k];
                if (c.h == hmax && c.v == vmax) {
                    v[k] = c.plane[static_cast<size_t>(y) * c.stride + x];
                    continue;
                }
                // subsampled plane: triangle filter between the two nearest samples per axis (weights 3/4 and 1/4, the
                // "fancy upsampling" of the common decoders), edges replicated
                const int cw = (width * c.h + hmax - 1) / hmax, ch = (height * c.v + vmax - 1) / vmax;
                int x0 = x, x1 = x, y0 = y, y1 = y;
                if (c.h != hmax) {
                    x0 = x >> 1;
                    x1 = std::min(std::max((x & 1) ? x0 + 1 : x0 - 1, 0), cw - 1);
                }
                if (c.v != vmax) {
                    y0 = y >> 1;
                    y1 = std::min(std::max((y & 1) ? y0 + 1 : y0 - 1, 0), ch - 1);
                }
                auto at_ = [&](int yy, int xx) { return static_cast<int>(c.plane[static_cast<size_t>(yy) * c.stride + xx]); };
                const int wx1 = c.h != hmax ? 1 : 0, wy1 = c.v != vmax ? 1 : 0;       // weights in quarters: far sample, near sample
                const int wx_near = 4 - wx1, wy_near = 4 - wy1;
                const int sum = wy_near * (wx_near * at_(y0, x0) + wx1 * at_(y0, x1)) + wy1 * (wx_near * at_(y1, x0) + wx1 * at_(y1, x1));
                v[k] = (sum + 8) >> 4;
            }
            uint8_t* px = &im.pixels[(static_cast<size_t>(y) * width + x) * 3];
            if (comps.size() == 1) {
                px[0] = px[1] = px[2] = static_cast<uint8_t>(v[0]);
            } else if (ycc) {
                const float Y = static_cast<float>(v[0]), cb = v[1] - 128.f, cr = v[2] - 128.f;
                auto clamp8 = [](float f) { return static_cast<uint8_t>(std::min(std::max(static_cast<int>(std::lround(f)), 0), 255)); };
                px[0] = clamp8(Y + 1.402f * cr);
                px[1] = clamp8(Y - 0.344136f * cb - 0.714136f * cr);
                px[2] = clamp8(Y + 1.772f * cb);
            } else {
                px[0] = static_cast<uint8_t>(v[0]);
                px[1] = static_cast<uint8_t>(v[1]);
                px[2] = static_cast<uint8_t>(v[2]);
            }
        }
    return im;
}

}  // namespace telb
