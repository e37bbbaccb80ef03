#include "media.h"

#include <cstdlib>
#include <climits>

#include <algorithm>
#include <cmath>
#include <complex>
#include <cstring>
#include <fstream>
#include <sstream>
#include <stdexcept>

namespace telb {

namespace {

std::string read_file(const std::string& path) {
    std::ifstream f(path, std::ios::binary);
    if (!f) throw std::runtime_error("cannot open " + path);
    std::ostringstream ss;
    ss << f.rdbuf();
    return ss.str();
}

template <typename T>
T rd(const std::string& b, size_t at) {
    if (at + sizeof(T) > b.size()) throw std::runtime_error("truncated file");
    T v;
    std::memcpy(&v, b.data() + at, sizeof(T));
    return v;
}

}  // namespace

// ---- audio -----------------------------------------------------------------------------------------------------------

AudioClip parse_wav(const std::string& b) {
    if (b.size() < 12 || b.compare(0, 4, "RIFF") != 0 || b.compare(8, 4, "WAVE") != 0) throw std::runtime_error("not a RIFF/WAVE file");
    int fmt = 0, channels = 0, rate = 0, bits = 0;
    size_t data_at = 0, data_len = 0;
    for (size_t at = 12; at + 8 <= b.size();) {
        const std::string id = b.substr(at, 4);
        const uint32_t len = rd<uint32_t>(b, at + 4);
        if (id == "fmt ") {
            fmt = rd<uint16_t>(b, at + 8);
            channels = rd<uint16_t>(b, at + 10);
            rate = static_cast<int>(rd<uint32_t>(b, at + 12));
            bits = rd<uint16_t>(b, at + 22);
            if (fmt == 0xFFFE && len >= 26) fmt = rd<uint16_t>(b, at + 8 + 24);      // WAVE_FORMAT_EXTENSIBLE: sub-format tag
        } else if (id == "data") {
            data_at = at + 8;
            data_len = std::min<size_t>(len, b.size() - data_at);
            break;
        }
        at += 8 + len + (len & 1);
    }
    if (!channels || !rate || !data_at) throw std::runtime_error("WAVE file without fmt / data chunks");
    if (!((fmt == 1 && (bits == 16 || bits == 24 || bits == 32)) || (fmt == 3 && bits == 32)))
        throw std::runtime_error("unsupported WAVE encoding (PCM 16/24/32 and float32 are read)");
    const int bytes = bits / 8;
    const size_t frames = data_len / (static_cast<size_t>(bytes) * channels);
    AudioClip clip;
    clip.sample_rate = rate;
    clip.samples.resize(frames);
    for (size_t i = 0; i < frames; ++i) {
        float acc = 0.f;
        for (int c = 0; c < channels; ++c) {
            const size_t at = data_at + (i * channels + c) * bytes;
            float v;
            if (fmt == 3) v = rd<float>(b, at);
            else if (bits == 16) v = rd<int16_t>(b, at) / 32768.f;
            else if (bits == 32) v = rd<int32_t>(b, at) / 2147483648.f;
            else {
                int32_t x = static_cast<uint8_t>(b[at]) | (static_cast<uint8_t>(b[at + 1]) << 8) | (static_cast<int8_t>(b[at + 2]) << 16);
                v = x / 8388608.f;
            }
            acc += v;
        }
        clip.samples[i] = acc / channels;
    }
    return clip;
}

AudioClip load_wav(const std::string& path) { return parse_wav(read_file(path)); }

std::vector<float> resample_linear(const std::vector<float>& x, int from_rate, int to_rate) {
    if (from_rate == to_rate || x.empty()) return x;
    const size_t n = static_cast<size_t>(std::llround(static_cast<double>(x.size()) * to_rate / from_rate));
    std::vector<float> y(n);
    const double step = static_cast<double>(from_rate) / to_rate;
    for (size_t i = 0; i < n; ++i) {
        const double pos = i * step;
        const size_t i0 = std::min(static_cast<size_t>(pos), x.size() - 1), i1 = std::min(i0 + 1, x.size() - 1);
        const double f = pos - i0;
        y[i] = static_cast<float>(x[i0] * (1.0 - f) + x[i1] * f);
    }
    return y;
}

namespace {
double hz_to_mel(double f) {          // Slaney: linear below 1 kHz, logarithmic above
    const double f_sp = 200.0 / 3.0, min_log_hz = 1000.0, min_log_mel = min_log_hz / f_sp, logstep = std::log(6.4) / 27.0;
    return f >= min_log_hz ? min_log_mel + std::log(f / min_log_hz) / logstep : f / f_sp;
}
double mel_to_hz(double m) {
    const double f_sp = 200.0 / 3.0, min_log_hz = 1000.0, min_log_mel = min_log_hz / f_sp, logstep = std::log(6.4) / 27.0;
    return m >= min_log_mel ? min_log_hz * std::exp(logstep * (m - min_log_mel)) : f_sp * m;
}
}  // namespace

std::vector<float> mel_filterbank(const MelConfig& c) {
    const int bins = c.n_fft / 2 + 1;
    std::vector<double> pts(c.n_mels + 2);
    const double m0 = hz_to_mel(c.f_min), m1 = hz_to_mel(c.f_max);
    for (int i = 0; i < c.n_mels + 2; ++i) pts[i] = mel_to_hz(m0 + (m1 - m0) * i / (c.n_mels + 1));
    std::vector<float> fb(static_cast<size_t>(c.n_mels) * bins, 0.f);
    for (int m = 0; m < c.n_mels; ++m) {
        const double lo = pts[m], ce = pts[m + 1], hi = pts[m + 2], norm = 2.0 / (hi - lo);
        for (int k = 0; k < bins; ++k) {
            const double f = static_cast<double>(k) * c.sample_rate / c.n_fft;
            const double w = std::max(0.0, std::min((f - lo) / (ce - lo), (hi - f) / (hi - ce)));
            fb[static_cast<size_t>(m) * bins + k] = static_cast<float>(w * norm);
        }
    }
    return fb;
}

std::vector<float> log_mel_spectrogram(const std::vector<float>& in, const MelConfig& c, int* frames_out) {
    std::vector<float> x = in;
    if (c.pad_to_samples > 0) x.resize(c.pad_to_samples, 0.f);
    const int n = static_cast<int>(x.size()), pad = c.n_fft / 2, bins = c.n_fft / 2 + 1;
    if (n <= pad) throw std::runtime_error("clip shorter than half a window");
    std::vector<float> padded(n + 2 * pad);
    for (int i = 0; i < n + 2 * pad; ++i) {
        int j = i - pad;
        if (j < 0) j = -j;
        if (j >= n) j = 2 * (n - 1) - j;
        padded[i] = x[j];
    }
    const int total = 1 + n / c.hop, frames = std::max(total - 1, 1);
    std::vector<double> window(c.n_fft);
    for (int i = 0; i < c.n_fft; ++i) window[i] = 0.5 - 0.5 * std::cos(2.0 * M_PI * i / c.n_fft);       // periodic Hann
    // twiddles of the direct transform; n_fft is a few hundred, so the O(n_fft · bins) DFT per frame is cheap next to the model
    std::vector<double> cs(c.n_fft), sn(c.n_fft);
    for (int i = 0; i < c.n_fft; ++i) {
        cs[i] = std::cos(2.0 * M_PI * i / c.n_fft);
        sn[i] = std::sin(2.0 * M_PI * i / c.n_fft);
    }
    const std::vector<float> fb = mel_filterbank(c);
    std::vector<float> out(static_cast<size_t>(c.n_mels) * frames);
    std::vector<double> seg(c.n_fft), power(bins);
    float gmax = -1e30f;
    for (int t = 0; t < frames; ++t) {
        for (int i = 0; i < c.n_fft; ++i) seg[i] = padded[static_cast<size_t>(t) * c.hop + i] * window[i];
        for (int k = 0; k < bins; ++k) {
            double re = 0.0, im = 0.0;
            int idx = 0;
            for (int i = 0; i < c.n_fft; ++i) {
                re += seg[i] * cs[idx];
                im -= seg[i] * sn[idx];
                idx += k;
                if (idx >= c.n_fft) idx -= c.n_fft;
            }
            power[k] = re * re + im * im;
        }
        for (int m = 0; m < c.n_mels; ++m) {
            double acc = 0.0;
            const float* w = fb.data() + static_cast<size_t>(m) * bins;
            for (int k = 0; k < bins; ++k) acc += w[k] * power[k];
            const float v = c.whisper_norm ? static_cast<float>(std::log10(std::max(acc, 1e-10))) : static_cast<float>(std::log(std::max(acc, 1e-10)));
            out[static_cast<size_t>(m) * frames + t] = v;
            gmax = std::max(gmax, v);
        }
    }
    if (c.whisper_norm)
        for (auto& v : out) v = (std::max(v, gmax - 8.f) + 4.f) / 4.f;
    if (frames_out) *frames_out = frames;
    return out;
}

// ---- images ----------------------------------------------------------------------------------------------------------

namespace {
int next_int(const std::string& b, size_t& at) {
    for (;;) {
        while (at < b.size() && std::isspace(static_cast<unsigned char>(b[at]))) ++at;
        if (at < b.size() && b[at] == '#') {
            while (at < b.size() && b[at] != '\n') ++at;
            continue;
        }
        break;
    }
    int v = 0;
    bool any = false;
    while (at < b.size() && std::isdigit(static_cast<unsigned char>(b[at]))) {
        v = v * 10 + (b[at++] - '0');
        any = true;
    }
    if (!any) throw std::runtime_error("malformed PNM header");
    return v;
}
}  // namespace

uint64_t max_image_pixels() {
    static const uint64_t limit = [] {
        const char* e = std::getenv("TELB_MAX_IMAGE_PIXELS");
        if (e && *e) {
            char* end = nullptr;
            const unsigned long long v = std::strtoull(e, &end, 10);
            if (end != e && v > 0) return static_cast<uint64_t>(v);
        }
        return static_cast<uint64_t>(64) << 20;
    }();
    return limit;
}

Image parse_image(const std::string& b) {
    Image im;
    if (b.size() >= 8 && static_cast<uint8_t>(b[0]) == 0x89 && b[1] == 'P' && b[2] == 'N' && b[3] == 'G') return decode_png(b);
    if (b.size() >= 3 && static_cast<uint8_t>(b[0]) == 0xff && static_cast<uint8_t>(b[1]) == 0xd8) return decode_jpeg(b);
    if (b.size() >= 2 && b[0] == 'P' && (b[1] == '6' || b[1] == '5')) {
        size_t at = 2;
        im.channels = b[1] == '6' ? 3 : 1;
        im.width = next_int(b, at);
        im.height = next_int(b, at);
        const int maxv = next_int(b, at);
        if (maxv != 255) throw std::runtime_error("only 8-bit PNM images are read");
        if (im.width <= 0 || im.height <= 0 || static_cast<uint64_t>(im.width) * static_cast<uint64_t>(im.height) > max_image_pixels())
            throw std::runtime_error("PNM image size out of range");
        ++at;
        const size_t need = static_cast<size_t>(im.width) * im.height * im.channels;
        if (at + need > b.size()) throw std::runtime_error("truncated PNM image");
        im.pixels.assign(b.begin() + at, b.begin() + at + need);
        if (im.channels == 1) {                       // grey → RGB so the encoders see three channels
            std::vector<uint8_t> rgb(need * 3);
            for (size_t i = 0; i < need; ++i) rgb[3 * i] = rgb[3 * i + 1] = rgb[3 * i + 2] = im.pixels[i];
            im.pixels.swap(rgb);
            im.channels = 3;
        }
        return im;
    }
    if (b.size() >= 54 && b[0] == 'B' && b[1] == 'M') {
        const uint32_t off = rd<uint32_t>(b, 10);
        const int32_t w = rd<int32_t>(b, 18), h = rd<int32_t>(b, 22);
        const uint16_t bpp = rd<uint16_t>(b, 28);
        const uint32_t comp = rd<uint32_t>(b, 30);
        if ((bpp != 24 && bpp != 32) || (comp != 0 && comp != 3)) throw std::runtime_error("only uncompressed 24 / 32 bit BMP images are read");
        if (w <= 0 || h == 0 || h == INT32_MIN || static_cast<uint64_t>(w) * static_cast<uint64_t>(std::abs(h)) > max_image_pixels())
            throw std::runtime_error("BMP image size out of range");
        im.width = w;
        im.height = std::abs(h);
        im.channels = 3;
        const int bytes = bpp / 8;
        const size_t stride = (static_cast<size_t>(w) * bytes + 3) & ~size_t(3);
        if (off + stride * im.height > b.size()) throw std::runtime_error("truncated BMP image");
        im.pixels.resize(static_cast<size_t>(w) * im.height * 3);
        for (int y = 0; y < im.height; ++y) {
            const int src_y = h > 0 ? im.height - 1 - y : y;          // bottom-up unless the height is negative
            const uint8_t* row = reinterpret_cast<const uint8_t*>(b.data()) + off + stride * src_y;
            for (int x = 0; x < w; ++x) {
                uint8_t* px = &im.pixels[(static_cast<size_t>(y) * w + x) * 3];
                px[0] = row[x * bytes + 2];
                px[1] = row[x * bytes + 1];
                px[2] = row[x * bytes + 0];
            }
        }
        return im;
    }
    throw std::runtime_error("unsupported image container (PNG, baseline JPEG, binary PPM / PGM and uncompressed BMP are read)");
}

Image load_image(const std::string& path) { return parse_image(read_file(path)); }

Image resize_bilinear(const Image& im, int ow, int oh) {
    Image out;
    out.width = ow;
    out.height = oh;
    out.channels = im.channels;
    out.pixels.resize(static_cast<size_t>(ow) * oh * im.channels);
    const double sx = static_cast<double>(im.width) / ow, sy = static_cast<double>(im.height) / oh;
    for (int y = 0; y < oh; ++y) {
        const double fy = std::max((y + 0.5) * sy - 0.5, 0.0);
        const int y0 = std::min(static_cast<int>(fy), im.height - 1), y1 = std::min(y0 + 1, im.height - 1);
        const double wy = fy - y0;
        for (int x = 0; x < ow; ++x) {
            const double fx = std::max((x + 0.5) * sx - 0.5, 0.0);
            const int x0 = std::min(static_cast<int>(fx), im.width - 1), x1 = std::min(x0 + 1, im.width - 1);
            const double wx = fx - x0;
            for (int c = 0; c < im.channels; ++c) {
                auto px = [&](int yy, int xx) { return static_cast<double>(im.pixels[(static_cast<size_t>(yy) * im.width + xx) * im.channels + c]); };
                const double v = (px(y0, x0) * (1 - wx) + px(y0, x1) * wx) * (1 - wy) + (px(y1, x0) * (1 - wx) + px(y1, x1) * wx) * wy;
                out.pixels[(static_cast<size_t>(y) * ow + x) * im.channels + c] = static_cast<uint8_t>(std::lround(std::min(std::max(v, 0.0), 255.0)));
            }
        }
    }
    return out;
}

namespace {
inline double cubic(double t) {        // Keys kernel, a = -0.75 (the coefficient the common image libraries use)
    const double a = -0.75;
    t = std::fabs(t);
    if (t <= 1) return ((a + 2) * t - (a + 3)) * t * t + 1;
    if (t < 2) return ((a * t - 5 * a) * t + 8 * a) * t - 4 * a;
    return 0;
}
}  // namespace

Image resize_bicubic(const Image& im, int ow, int oh) {
    Image out;
    out.width = ow;
    out.height = oh;
    out.channels = im.channels;
    out.pixels.resize(static_cast<size_t>(ow) * oh * im.channels);
    const double sx = static_cast<double>(im.width) / ow, sy = static_cast<double>(im.height) / oh;
    for (int y = 0; y < oh; ++y) {
        const double fy = (y + 0.5) * sy - 0.5;
        const int y0 = static_cast<int>(std::floor(fy));
        for (int x = 0; x < ow; ++x) {
            const double fx = (x + 0.5) * sx - 0.5;
            const int x0 = static_cast<int>(std::floor(fx));
            for (int c = 0; c < im.channels; ++c) {
                double acc = 0;
                for (int j = -1; j <= 2; ++j) {
                    const int yy = std::min(std::max(y0 + j, 0), im.height - 1);
                    const double wy = cubic(fy - (y0 + j));
                    for (int i = -1; i <= 2; ++i) {
                        const int xx = std::min(std::max(x0 + i, 0), im.width - 1);
                        acc += wy * cubic(fx - (x0 + i)) * im.pixels[(static_cast<size_t>(yy) * im.width + xx) * im.channels + c];
                    }
                }
                out.pixels[(static_cast<size_t>(y) * ow + x) * im.channels + c] = static_cast<uint8_t>(std::lround(std::min(std::max(acc, 0.0), 255.0)));
            }
        }
    }
    return out;
}

std::vector<float> normalize_chw(const Image& im, const std::vector<float>& mean, const std::vector<float>& stddev) {
    if (static_cast<int>(mean.size()) != im.channels || static_cast<int>(stddev.size()) != im.channels)
        throw std::runtime_error("mean / std need one entry per channel");
    const size_t plane = static_cast<size_t>(im.width) * im.height;
    std::vector<float> out(plane * im.channels);
    for (size_t i = 0; i < plane; ++i)
        for (int c = 0; c < im.channels; ++c) out[c * plane + i] = (im.pixels[i * im.channels + c] / 255.f - mean[c]) / stddev[c];
    return out;
}

void smart_resize(int height, int width, int factor, long long min_pixels, long long max_pixels, int* out_h, int* out_w) {
    if (height <= 0 || width <= 0 || factor <= 0) throw std::runtime_error("smart_resize needs positive sizes");
    auto round_to = [&](double v) { return std::max<long long>(factor, static_cast<long long>(std::llround(v / factor)) * factor); };
    long long h = round_to(height), w = round_to(width);
    if (h * w > max_pixels) {
        const double beta = std::sqrt(static_cast<double>(height) * width / max_pixels);
        h = std::max<long long>(factor, static_cast<long long>(std::floor(height / beta / factor)) * factor);
        w = std::max<long long>(factor, static_cast<long long>(std::floor(width / beta / factor)) * factor);
    } else if (h * w < min_pixels) {
        const double beta = std::sqrt(static_cast<double>(min_pixels) / (static_cast<double>(height) * width));
        h = static_cast<long long>(std::ceil(height * beta / factor)) * factor;
        w = static_cast<long long>(std::ceil(width * beta / factor)) * factor;
    }
    *out_h = static_cast<int>(h);
    *out_w = static_cast<int>(w);
}

}  // namespace telb
