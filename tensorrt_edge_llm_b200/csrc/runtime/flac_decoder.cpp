// FLAC decoding for audio parts of requests, written against the format specification (RFC 9639): STREAMINFO, frame
// headers with their CRC-8, the four subframe kinds (constant, verbatim, fixed predictors of order 0-4, linear prediction
// of order 1-32), Rice-coded residuals with 4- and 5-bit parameters, partitions and escape codes, wasted bits, and the
// three stereo decorrelation modes.  Channels are averaged to mono and scaled to [-1, 1], as the WAV reader does.
//
// Counterpart in the reference: cpp/runtime/audioLoader.cpp, which hands FLAC (and MP3) to the miniaudio header.
// Not covered: MP3; Ogg-encapsulated FLAC; the frame footer CRC-16 is not verified (the header CRC-8 is).
#include <algorithm>
#include <cstring>
#include <fstream>
#include <sstream>
#include <stdexcept>

#include "media.h"

namespace telb {

namespace {

[[noreturn]] void bad(const char* what) { throw std::runtime_error(std::string("FLAC: ") + what); }

struct BitReader {
    const uint8_t* p;
    size_t n, byte = 0;
    int bit = 0;                    // bits of p[byte] already consumed
    BitReader(const uint8_t* data, size_t size) : p(data), n(size) {}
    uint32_t bits(int k) {          // k <= 32, most significant first
        uint32_t v = 0;
        while (k > 0) {
            if (byte >= n) bad("stream ends inside a frame");
            const int take = std::min(k, 8 - bit);
            v = (v << take) | ((p[byte] >> (8 - bit - take)) & ((1u << take) - 1));
            bit += take;
            k -= take;
            if (bit == 8) {
                bit = 0;
                ++byte;
            }
        }
        return v;
    }
    int64_t sbits(int k) {          // two's complement, k <= 33
        if (k == 0) return 0;
        uint64_t v = k > 32 ? (static_cast<uint64_t>(bits(k - 32)) << 32) | bits(32) : bits(k);
        const uint64_t sign = 1ull << (k - 1);
        return static_cast<int64_t>((v ^ sign)) - static_cast<int64_t>(sign);
    }
    uint32_t unary() {              // zeros before the next one bit
        uint32_t z = 0;
        for (;;) {
            if (byte >= n) bad("stream ends inside a residual");
            const int left = 8 - bit;
            const uint32_t cur = p[byte] & ((1u << left) - 1);
            if (cur == 0) {
                z += left;
                bit = 0;
                ++byte;
                continue;
            }
            int lead = 0;
            while (!(cur & (1u << (left - 1 - lead)))) ++lead;
            z += lead;
            bit += lead + 1;
            if (bit == 8) {
                bit = 0;
                ++byte;
            }
            return z;
        }
    }
    void align() {
        if (bit) {
            bit = 0;
            ++byte;
        }
    }
};

uint8_t crc8(const uint8_t* p, size_t n) {
    uint8_t c = 0;
    for (size_t i = 0; i < n; ++i) {
        c ^= p[i];
        for (int b = 0; b < 8; ++b) c = (c & 0x80) ? static_cast<uint8_t>((c << 1) ^ 0x07) : static_cast<uint8_t>(c << 1);
    }
    return c;
}

void read_residual(BitReader& br, int order, int block, std::vector<int64_t>& out) {
    const int method = br.bits(2);
    if (method > 1) bad("reserved residual coding method");
    const int pbits = method == 0 ? 4 : 5;
    const uint32_t escape = method == 0 ? 15 : 31;
    const int part_order = br.bits(4);
    const int parts = 1 << part_order;
    if ((block >> part_order) << part_order != block && part_order > 0) bad("block size is not a multiple of the partition count");
    int i = order;
    for (int q = 0; q < parts; ++q) {
        int count = (block >> part_order) - (q == 0 ? order : 0);
        if (part_order == 0) count = block - order;
        if (count < 0) bad("partition smaller than the predictor order");
        const uint32_t k = br.bits(pbits);
        if (k == escape) {
            const int raw = br.bits(5);
            for (int j = 0; j < count; ++j) out[i++] = br.sbits(raw);
        } else {
            for (int j = 0; j < count; ++j) {
                const uint32_t msb = br.unary();
                const uint32_t lsb = k ? br.bits(static_cast<int>(k)) : 0;
                const uint64_t u = (static_cast<uint64_t>(msb) << k) | lsb;
                out[i++] = static_cast<int64_t>(u >> 1) ^ -static_cast<int64_t>(u & 1);       // zig-zag
            }
        }
    }
}

void read_subframe(BitReader& br, int block, int bps, std::vector<int64_t>& out) {
    if (br.bits(1)) bad("subframe padding bit is set");
    const int type = br.bits(6);
    int wasted = 0;
    if (br.bits(1)) wasted = static_cast<int>(br.unary()) + 1;
    bps -= wasted;
    if (bps <= 0) bad("more wasted bits than sample bits");
    out.assign(block, 0);
    if (type == 0) {                                    // constant
        const int64_t v = br.sbits(bps);
        for (int i = 0; i < block; ++i) out[i] = v;
    } else if (type == 1) {                             // verbatim
        for (int i = 0; i < block; ++i) out[i] = br.sbits(bps);
    } else if (type >= 8 && type <= 12) {               // fixed predictor
        const int order = type - 8;
        if (order > block) bad("fixed predictor order exceeds the block size");
        for (int i = 0; i < order; ++i) out[i] = br.sbits(bps);
        read_residual(br, order, block, out);
        for (int i = order; i < block; ++i) {
            int64_t pred = 0;
            switch (order) {
                case 1: pred = out[i - 1]; break;
                case 2: pred = 2 * out[i - 1] - out[i - 2]; break;
                case 3: pred = 3 * out[i - 1] - 3 * out[i - 2] + out[i - 3]; break;
                case 4: pred = 4 * out[i - 1] - 6 * out[i - 2] + 4 * out[i - 3] - out[i - 4]; break;
                default: break;
            }
            out[i] += pred;
        }
    } else if (type >= 32) {                            // linear prediction
        const int order = type - 31;
        if (order > block) bad("LPC order exceeds the block size");
        for (int i = 0; i < order; ++i) out[i] = br.sbits(bps);
        const int precision = br.bits(4) + 1;
        if (precision == 16) bad("reserved LPC coefficient precision");
        const int shift = static_cast<int>(br.sbits(5));
        if (shift < 0) bad("negative LPC shift");
        int64_t coef[32];
        for (int j = 0; j < order; ++j) coef[j] = br.sbits(precision);
        read_residual(br, order, block, out);
        for (int i = order; i < block; ++i) {
            int64_t acc = 0;
            for (int j = 0; j < order; ++j) acc += coef[j] * out[i - 1 - j];
            out[i] += acc >> shift;
        }
    } else {
        bad("reserved subframe type");
    }
    if (wasted)
        for (int i = 0; i < block; ++i) out[i] *= (1ll << wasted);
}

}  // namespace

AudioClip parse_flac(const std::string& bytes) {
    const uint8_t* d = reinterpret_cast<const uint8_t*>(bytes.data());
    const size_t n = bytes.size();
    if (n < 42 || std::memcmp(d, "fLaC", 4) != 0) bad("not a FLAC stream");
    size_t at = 4;
    int rate = 0, channels = 0, bps = 0;
    uint64_t total = 0;
    bool last = false, have_info = false;
    while (!last) {
        if (at + 4 > n) bad("truncated metadata");
        last = (d[at] & 0x80) != 0;
        const int kind = d[at] & 0x7f;
        const size_t len = (static_cast<size_t>(d[at + 1]) << 16) | (static_cast<size_t>(d[at + 2]) << 8) | d[at + 3];
        at += 4;
        if (at + len > n) bad("truncated metadata block");
        if (kind == 0) {
            if (len < 34) bad("short STREAMINFO");
            const uint8_t* s = d + at;
            rate = (s[10] << 12) | (s[11] << 4) | (s[12] >> 4);
            channels = ((s[12] >> 1) & 7) + 1;
            bps = (((s[12] & 1) << 4) | (s[13] >> 4)) + 1;
            total = (static_cast<uint64_t>(s[13] & 0x0f) << 32) | (static_cast<uint64_t>(s[14]) << 24) | (s[15] << 16) | (s[16] << 8) | s[17];
            have_info = true;
        }
        at += len;
    }
    if (!have_info || rate <= 0 || channels < 1 || channels > 8 || bps < 4 || bps > 32) bad("missing or invalid STREAMINFO");
    if (total > (1ull << 31)) bad("stream longer than the decoder's limit");
    AudioClip clip;
    clip.sample_rate = rate;
    if (total) clip.samples.reserve(static_cast<size_t>(total));
    const float scale = 1.0f / static_cast<float>(1ull << (bps - 1));
    std::vector<std::vector<int64_t>> ch(channels);
    while (at + 2 <= n) {
        if (d[at] != 0xff || (d[at + 1] & 0xfe) != 0xf8) {     // not a frame sync: trailing bytes (ID3 tags, padding) end the stream
            bool rest_zero = true;
            for (size_t i = at; i < n && rest_zero; ++i) rest_zero = d[i] == 0;
            if (rest_zero || clip.samples.size() >= total) break;
            bad("lost frame synchronisation");
        }
        BitReader br(d + at, n - at);
        br.bits(15);                                            // sync + reserved
        br.bits(1);                                             // blocking strategy (only the coded number's meaning changes)
        const int bs_code = br.bits(4), sr_code = br.bits(4), ch_code = br.bits(4), ss_code = br.bits(3);
        if (br.bits(1)) bad("reserved frame header bit is set");
        // UTF-8 style coded frame / sample number
        const uint32_t first = br.bits(8);
        int extra = 0;
        if (first >= 0xfe) extra = 6;
        else if (first >= 0xfc) extra = 5;
        else if (first >= 0xf8) extra = 4;
        else if (first >= 0xf0) extra = 3;
        else if (first >= 0xe0) extra = 2;
        else if (first >= 0xc0) extra = 1;
        else if (first >= 0x80) bad("invalid coded frame number");
        for (int i = 0; i < extra; ++i)
            if ((br.bits(8) & 0xc0) != 0x80) bad("invalid coded frame number");
        int block = 0;
        if (bs_code == 0) bad("reserved block size");
        else if (bs_code == 1) block = 192;
        else if (bs_code <= 5) block = 576 << (bs_code - 2);
        else if (bs_code == 6) block = br.bits(8) + 1;
        else if (bs_code == 7) block = br.bits(16) + 1;
        else block = 256 << (bs_code - 8);
        if (sr_code == 12) br.bits(8);
        else if (sr_code == 13 || sr_code == 14) br.bits(16);
        else if (sr_code == 15) bad("invalid sample rate code");
        int frame_bps = bps;
        static const int kBits[8] = {0, 8, 12, 0, 16, 20, 24, 32};
        if (ss_code == 3) bad("reserved sample size");
        if (ss_code != 0) frame_bps = kBits[ss_code];
        const size_t header_len = br.byte;
        const uint8_t want_crc = static_cast<uint8_t>(br.bits(8));
        if (crc8(d + at, header_len) != want_crc) bad("frame header checksum mismatch");
        int nch;
        int mode = 0;                                           // 0 independent, 1 left/side, 2 side/right, 3 mid/side
        if (ch_code < 8) nch = ch_code + 1;
        else if (ch_code <= 10) {
            nch = 2;
            mode = ch_code - 7;
        } else bad("reserved channel assignment");
        if (nch != channels) bad("frame channel count differs from STREAMINFO");
        for (int c = 0; c < nch; ++c) {
            const bool side = (mode == 1 && c == 1) || (mode == 2 && c == 0) || (mode == 3 && c == 1);
            read_subframe(br, block, frame_bps + (side ? 1 : 0), ch[c]);
        }
        br.align();
        br.bits(16);                                            // frame CRC-16 (not verified)
        if (mode == 1) {
            for (int i = 0; i < block; ++i) ch[1][i] = ch[0][i] - ch[1][i];
        } else if (mode == 2) {
            for (int i = 0; i < block; ++i) ch[0][i] = ch[1][i] + ch[0][i];
        } else if (mode == 3) {
            for (int i = 0; i < block; ++i) {
                const int64_t side = ch[1][i];
                const int64_t mid = (ch[0][i] << 1) | (side & 1);
                ch[0][i] = (mid + side) >> 1;
                ch[1][i] = (mid - side) >> 1;
            }
        }
        const float fs = (frame_bps == bps ? scale : 1.0f / static_cast<float>(1ull << (frame_bps - 1))) / static_cast<float>(nch);
        for (int i = 0; i < block; ++i) {
            int64_t sum = 0;
            for (int c = 0; c < nch; ++c) sum += ch[c][i];
            clip.samples.push_back(static_cast<float>(sum) * fs);
        }
        at += br.byte;
    }
    if (total && clip.samples.size() > total) clip.samples.resize(static_cast<size_t>(total));
    if (clip.samples.empty()) bad("no audio frames");
    return clip;
}

AudioClip parse_audio(const std::string& bytes) {
    if (bytes.size() >= 4 && std::memcmp(bytes.data(), "fLaC", 4) == 0) return parse_flac(bytes);
    if (bytes.size() >= 4 && std::memcmp(bytes.data(), "RIFF", 4) == 0) return parse_wav(bytes);
    if (bytes.size() >= 3 && (std::memcmp(bytes.data(), "ID3", 3) == 0 || (static_cast<uint8_t>(bytes[0]) == 0xff && (bytes[1] & 0xe0) == 0xe0)))
        throw std::runtime_error("MP3 audio is not decoded here: send WAV or FLAC");
    throw std::runtime_error("unknown audio container: WAV (RIFF) and FLAC are read");
}

AudioClip load_audio(const std::string& path) {
    std::ifstream f(path, std::ios::binary);
    if (!f) throw std::runtime_error("cannot open " + path);
    std::ostringstream ss;
    ss << f.rdbuf();
    return parse_audio(ss.str());
}

}  // namespace telb
