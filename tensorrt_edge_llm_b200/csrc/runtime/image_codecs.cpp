// PNG and baseline JPEG decoding for the vision front end, written against the format specifications (RFC 1950 / 1951
// for the zlib stream and DEFLATE, the PNG specification's filter definitions, ITU T.81 for JPEG) so that image
// parts of chat requests (data: URIs are almost always PNG or JPEG) need no third-party decoder.
//
// Counterpart in the reference: cpp/runtime/imageUtils.cpp, which hands these formats to the stb_image header.
// Covered: PNG non-interlaced and Adam7-interlaced, colour types 0 / 2 / 3 / 4 / 6, bit depths 1 / 2 / 4 / 8 / 16 (alpha is dropped, 16-bit
// samples keep their high byte); JPEG sequential Huffman (SOF0 / SOF1), 8-bit, one or three components, sampling
// factors 1 or 2, restart intervals.  Not covered (a clear error is raised): progressive,
// arithmetic-coded, lossless and four-component JPEG.
#include "media.h"

#include <algorithm>
#include <array>
#include <cmath>
#include <cstring>
#include <stdexcept>

namespace telb {
namespace {

[[noreturn]] void bad(const char* what) { throw std::runtime_error(what); }

// ---- DEFLATE -----------------------------------------------------------------------------------------------------

struct BitsLsb {
    const uint8_t* p;
    size_t n, at = 0;
    uint32_t buf = 0;
    int cnt = 0;
    int bit() {
        if (cnt == 0) {
            if (at >= n) bad("deflate stream ends early");
            buf = p[at++];
            cnt = 8;
        }
        const int b = buf & 1;
        buf >>= 1;
        --cnt;
        return b;
    }
    uint32_t bits(int k) {
        uint32_t v = 0;
        for (int i = 0; i < k; ++i) v |= static_cast<uint32_t>(bit()) << i;
        return v;
    }
    void align() { cnt = 0; }
};

// Canonical Huffman code described by its code lengths: count[len] codes of each length, symbols in code order.
struct Huff {
    std::array<uint16_t, 16> count{};
    std::vector<uint16_t> symbol;
    void build(const uint8_t* lengths, int n) {
        count.fill(0);
        for (int i = 0; i < n; ++i) ++count[lengths[i]];
        count[0] = 0;
        std::array<uint16_t, 16> offs{};
        for (int l = 1; l < 15; ++l) offs[l + 1] = offs[l] + count[l];
        symbol.assign(n, 0);
        for (int i = 0; i < n; ++i)
            if (lengths[i]) symbol[offs[lengths[i]]++] = static_cast<uint16_t>(i);
    }
    int decode(BitsLsb& s) const {
        int code = 0, first = 0, index = 0;
        for (int len = 1; len <= 15; ++len) {
            code |= s.bit();
            const int c = count[len];
            if (code - c < first) return symbol[index + (code - first)];
            index += c;
            first = (first + c) << 1;
            code <<= 1;
        }
        bad("invalid Huffman code in a deflate stream");
    }
};

const uint16_t kLenBase[29] = {3, 4, 5, 6, 7, 8, 9, 10, 11, 13, 15, 17, 19, 23, 27, 31, 35, 43, 51, 59, 67, 83, 99, 115, 131, 163, 195, 227, 258};
const uint8_t kLenExtra[29] = {0, 0, 0, 0, 0, 0, 0, 0, 1, 1, 1, 1, 2, 2, 2, 2, 3, 3, 3, 3, 4, 4, 4, 4, 5, 5, 5, 5, 0};
const uint16_t kDistBase[30] = {1, 2, 3, 4, 5, 7, 9, 13, 17, 25, 33, 49, 65, 97, 129, 193, 257, 385, 513, 769, 1025, 1537, 2049, 3073,
                                4097, 6145, 8193, 12289, 16385, 24577};
const uint8_t kDistExtra[30] = {0, 0, 0, 0, 1, 1, 2, 2, 3, 3, 4, 4, 5, 5, 6, 6, 7, 7, 8, 8, 9, 9, 10, 10, 11, 11, 12, 12, 13, 13};

void inflate_block(BitsLsb& s, const Huff& lit, const Huff& dist, std::vector<uint8_t>& out, size_t limit) {
    for (;;) {
        const int sym = lit.decode(s);
        if (sym < 256) {
            if (out.size() >= limit) bad("deflate output exceeds the expected size");
            out.push_back(static_cast<uint8_t>(sym));
        } else if (sym == 256) {
            return;
        } else {
            if (sym > 285) bad("invalid length symbol in a deflate stream");
            const int len = kLenBase[sym - 257] + static_cast<int>(s.bits(kLenExtra[sym - 257]));
            const int ds = dist.decode(s);
            if (ds > 29) bad("invalid distance symbol in a deflate stream");
            const size_t d = kDistBase[ds] + s.bits(kDistExtra[ds]);
            if (d > out.size()) bad("deflate distance reaches before the start of the output");
            if (out.size() + len > limit) bad("deflate output exceeds the expected size");
            size_t from = out.size() - d;
            for (int i = 0; i < len; ++i) out.push_back(out[from++]);      // may overlap its own output: byte by byte
        }
    }
}

}  // namespace

std::string inflate_zlib(const std::string& z, size_t max_output) {
    if (z.size() < 6) bad("zlib stream too short");
    const uint8_t* p = reinterpret_cast<const uint8_t*>(z.data());
    if ((p[0] & 0x0f) != 8 || ((p[0] << 8) | p[1]) % 31 != 0 || (p[1] & 0x20)) bad("not a zlib stream (or one with a preset dictionary)");
    BitsLsb s{p + 2, z.size() - 2};
    std::vector<uint8_t> out;
    Huff fixed_lit, fixed_dist;
    {
        uint8_t l[288];
        for (int i = 0; i < 144; ++i) l[i] = 8;
        for (int i = 144; i < 256; ++i) l[i] = 9;
        for (int i = 256; i < 280; ++i) l[i] = 7;
        for (int i = 280; i < 288; ++i) l[i] = 8;
        fixed_lit.build(l, 288);
        uint8_t d[30];
        std::fill(d, d + 30, 5);
        fixed_dist.build(d, 30);
    }
    int last;
    do {
        last = s.bit();
        const uint32_t type = s.bits(2);
        if (type == 0) {
            s.align();
            if (s.at + 4 > s.n) bad("deflate stream ends early");
            const uint32_t len = s.p[s.at] | (s.p[s.at + 1] << 8), nlen = s.p[s.at + 2] | (s.p[s.at + 3] << 8);
            s.at += 4;
            if ((len ^ 0xffff) != nlen) bad("stored deflate block with inconsistent length");
            if (s.at + len > s.n || out.size() + len > max_output) bad("stored deflate block out of range");
            out.insert(out.end(), s.p + s.at, s.p + s.at + len);
            s.at += len;
        } else if (type == 1) {
            inflate_block(s, fixed_lit, fixed_dist, out, max_output);
        } else if (type == 2) {
            const int nlen = static_cast<int>(s.bits(5)) + 257, ndist = static_cast<int>(s.bits(5)) + 1, ncode = static_cast<int>(s.bits(4)) + 4;
            if (nlen > 286 || ndist > 30) bad("deflate block declares too many codes");
            static const uint8_t order[19] = {16, 17, 18, 0, 8, 7, 9, 6, 10, 5, 11, 4, 12, 3, 13, 2, 14, 1, 15};
            uint8_t lengths[320] = {0};
            for (int i = 0; i < ncode; ++i) lengths[order[i]] = static_cast<uint8_t>(s.bits(3));
            Huff code;
            code.build(lengths, 19);
            std::memset(lengths, 0, sizeof lengths);
            int i = 0;
            while (i < nlen + ndist) {
                const int sym = code.decode(s);
                if (sym < 16) {
                    lengths[i++] = static_cast<uint8_t>(sym);
                } else {
                    int rep;
                    uint8_t val = 0;
                    if (sym == 16) {
                        if (i == 0) bad("deflate code lengths repeat nothing");
                        val = lengths[i - 1];
                        rep = 3 + static_cast<int>(s.bits(2));
                    } else if (sym == 17) {
                        rep = 3 + static_cast<int>(s.bits(3));
                    } else {
                        rep = 11 + static_cast<int>(s.bits(7));
                    }
                    if (i + rep > nlen + ndist) bad("deflate code lengths overrun");
                    while (rep--) lengths[i++] = val;
                }
            }
            if (lengths[256] == 0) bad("deflate block without an end code");
            Huff lit, dist;
            lit.build(lengths, nlen);
            dist.build(lengths + nlen, ndist);
            inflate_block(s, lit, dist, out, max_output);
        } else {
            bad("invalid deflate block type");
        }
    } while (!last);
    return std::string(out.begin(), out.end());
}

// ---- PNG ---------------------------------------------------------------------------------------------------------

namespace {
inline uint32_t be32(const uint8_t* p) { return (uint32_t(p[0]) << 24) | (uint32_t(p[1]) << 16) | (uint32_t(p[2]) << 8) | p[3]; }
inline int paeth(int a, int b, int c) {
    const int p = a + b - c, pa = std::abs(p - a), pb = std::abs(p - b), pc = std::abs(p - c);
    return (pa <= pb && pa <= pc) ? a : (pb <= pc ? b : c);
}
}  // namespace

Image decode_png(const std::string& bytes) {
    static const uint8_t sig[8] = {0x89, 'P', 'N', 'G', 0x0d, 0x0a, 0x1a, 0x0a};
    const uint8_t* p = reinterpret_cast<const uint8_t*>(bytes.data());
    const size_t n = bytes.size();
    if (n < 8 || std::memcmp(p, sig, 8) != 0) bad("not a PNG file");
    uint32_t w = 0, h = 0;
    int depth = 0, ctype = -1, interlace = 0;
    std::vector<uint8_t> palette;
    std::string idat;
    size_t at = 8;
    bool end = false;
    while (!end && at + 12 <= n) {
        const uint32_t len = be32(p + at);
        const char* type = reinterpret_cast<const char*>(p + at + 4);
        if (at + 12 + static_cast<size_t>(len) > n) bad("truncated PNG chunk");
        const uint8_t* d = p + at + 8;
        if (!std::memcmp(type, "IHDR", 4)) {
            if (len < 13) bad("short PNG header");
            w = be32(d);
            h = be32(d + 4);
            depth = d[8];
            ctype = d[9];
            interlace = d[12];
            if (d[10] != 0 || d[11] != 0) bad("unknown PNG compression or filter method");
        } else if (!std::memcmp(type, "PLTE", 4)) {
            palette.assign(d, d + len);
        } else if (!std::memcmp(type, "IDAT", 4)) {
            idat.append(reinterpret_cast<const char*>(d), len);
        } else if (!std::memcmp(type, "IEND", 4)) {
            end = true;
        }
        at += 12 + static_cast<size_t>(len);
    }
    if (ctype < 0 || w == 0 || h == 0 || w > (1u << 15) || h > (1u << 15)) bad("PNG without a usable header");
    if (static_cast<uint64_t>(w) * h > max_image_pixels()) bad("PNG image has more pixels than the decoder's limit");
    if (interlace != 0 && interlace != 1) bad("unknown PNG interlace method");
    int samples;
    switch (ctype) {
        case 0: samples = 1; break;
        case 2: samples = 3; break;
        case 3: samples = 1; break;
        case 4: samples = 2; break;
        case 6: samples = 4; break;
        default: bad("unknown PNG colour type");
    }
    const bool depth_ok = depth == 8 || ((ctype == 0 || ctype == 3) && (depth == 1 || depth == 2 || depth == 4)) || (ctype != 3 && depth == 16);
    if (!depth_ok) bad("PNG bit depth does not fit its colour type");
    if (ctype == 3 && palette.size() < 3) bad("palette PNG without a palette");
    const int bpp = std::max(1, samples * depth / 8);
    // A non-interlaced image is one pass over every pixel; Adam7 stores seven reduced images (pixel (x0 + i dx, y0 + j dy) of pass
    // p), each filtered on its own with a fresh "previous row".
    struct Pass { uint32_t x0, y0, dx, dy; };
    static const Pass kAdam7[7] = {{0, 0, 8, 8}, {4, 0, 8, 8}, {0, 4, 4, 8}, {2, 0, 4, 4}, {0, 2, 2, 4}, {1, 0, 2, 2}, {0, 1, 1, 2}};
    static const Pass kWhole[1] = {{0, 0, 1, 1}};
    const Pass* passes = interlace ? kAdam7 : kWhole;
    const int n_pass = interlace ? 7 : 1;
    auto pass_dims = [&](const Pass& ps, uint32_t& pw, uint32_t& ph) {
        pw = w > ps.x0 ? (w - ps.x0 + ps.dx - 1) / ps.dx : 0;
        ph = h > ps.y0 ? (h - ps.y0 + ps.dy - 1) / ps.dy : 0;
    };
    size_t raw_need = 0;
    for (int q = 0; q < n_pass; ++q) {
        uint32_t pw, ph;
        pass_dims(passes[q], pw, ph);
        if (pw && ph) raw_need += ((static_cast<size_t>(pw) * samples * depth + 7) / 8 + 1) * ph;
    }
    const std::string raw = inflate_zlib(idat, raw_need);
    if (raw.size() < raw_need) bad("PNG image data is shorter than its header says");
    Image im;
    im.width = static_cast<int>(w);
    im.height = static_cast<int>(h);
    im.channels = 3;
    im.pixels.resize(static_cast<size_t>(w) * h * 3);
    const uint8_t* src = reinterpret_cast<const uint8_t*>(raw.data());
    for (int q = 0; q < n_pass; ++q) {
        const Pass& ps = passes[q];
        uint32_t pw, ph;
        pass_dims(ps, pw, ph);
        if (!pw || !ph) continue;
        const size_t row_bytes = (static_cast<size_t>(pw) * samples * depth + 7) / 8;
        std::vector<uint8_t> prev(row_bytes, 0), cur(row_bytes);
        for (uint32_t y = 0; y < ph; ++y) {
            const int filter = src[0];
            ++src;
            for (size_t i = 0; i < row_bytes; ++i) {
                const int a = i >= static_cast<size_t>(bpp) ? cur[i - bpp] : 0, b = prev[i], c = i >= static_cast<size_t>(bpp) ? prev[i - bpp] : 0;
                int v = src[i];
                switch (filter) {
                    case 0: break;
                    case 1: v += a; break;
                    case 2: v += b; break;
                    case 3: v += (a + b) >> 1; break;
                    case 4: v += paeth(a, b, c); break;
                    default: bad("unknown PNG row filter");
                }
                cur[i] = static_cast<uint8_t>(v);
            }
            src += row_bytes;
            uint8_t* row = &im.pixels[static_cast<size_t>(ps.y0 + y * ps.dy) * w * 3];
            for (uint32_t x = 0; x < pw; ++x) {
                uint8_t* dst = row + static_cast<size_t>(ps.x0 + x * ps.dx) * 3;
                auto sample = [&](int k) -> int {           // k-th sample of pixel x of this pass, scaled to 8 bits
                    if (depth == 8) return cur[static_cast<size_t>(x) * samples + k];
                    if (depth == 16) return cur[(static_cast<size_t>(x) * samples + k) * 2];
                    const size_t bit = static_cast<size_t>(x) * depth;
                    const int v = (cur[bit >> 3] >> (8 - depth - static_cast<int>(bit & 7))) & ((1 << depth) - 1);
                    return ctype == 3 ? v : v * 255 / ((1 << depth) - 1);
                };
                if (ctype == 3) {
                    const size_t idx = static_cast<size_t>(sample(0)) * 3;
                    if (idx + 3 > palette.size()) bad("PNG palette index out of range");
                    dst[0] = palette[idx];
                    dst[1] = palette[idx + 1];
                    dst[2] = palette[idx + 2];
                } else if (ctype == 0 || ctype == 4) {
                    dst[0] = dst[1] = dst[2] = static_cast<uint8_t>(sample(0));
                } else {
                    dst[0] = static_cast<uint8_t>(sample(0));
                    dst[1] = static_cast<uint8_t>(sample(1));
                    dst[2] = static_cast<uint8_t>(sample(2));
                }
            }
            prev.swap(cur);
        }
    }
    return im;
}

}  // namespace telb
