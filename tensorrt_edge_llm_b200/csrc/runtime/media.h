// Host-side media utilities: WAV / PCM loading and resampling, log-mel spectrogram, simple image decoding and
// resizing / normalisation for the vision and audio encoders.
//
// Counterparts in the reference: cpp/runtime/{audioLoader,audioUtils,melSpectrogram,imageUtils}.cpp (which lean on
// the third-party miniaudio and stb single-header libraries; here the formats that need no entropy decoder are
// parsed directly: RIFF/WAVE PCM16 / PCM24 / PCM32 / float32, binary PPM / PGM and uncompressed BMP; PNG, sequential
// JPEG and FLAC have decoders of their own in image_codecs.cpp / jpeg_decoder.cpp / flac_decoder.cpp).
#pragma once

#include <cstdint>
#include <string>
#include <vector>

namespace telb {

struct AudioClip {
    std::vector<float> samples;      // mono, [-1, 1]
    int sample_rate = 0;
};

AudioClip parse_wav(const std::string& bytes);                       // multi-channel input is averaged to mono
AudioClip load_wav(const std::string& path);
AudioClip parse_flac(const std::string& bytes);                      // native FLAC streams (flac_decoder.cpp); channels averaged to mono
AudioClip parse_audio(const std::string& bytes);                     // by magic: RIFF/WAVE or FLAC
AudioClip load_audio(const std::string& path);
std::vector<float> resample_linear(const std::vector<float>& x, int from_rate, int to_rate);

struct MelConfig {
    int sample_rate = 16000;
    int n_fft = 400;
    int hop = 160;
    int n_mels = 128;
    float f_min = 0.f;
    float f_max = 8000.f;
    bool whisper_norm = true;        // log10, clamp to (max - 8), (x + 4) / 4
    int pad_to_samples = 0;          // zero-pad / cut the clip to this many samples first (0 = as is)
};

// Slaney-scale triangular filters, area-normalised: [n_mels, n_fft/2 + 1] row-major.
std::vector<float> mel_filterbank(const MelConfig& c);
// Hann window, reflect padding of n_fft/2 at both ends, power spectrum, mel projection, log; the last frame is
// dropped (as the Whisper feature extractor does).  Returns [n_mels, frames] row-major and sets `frames`.
std::vector<float> log_mel_spectrogram(const std::vector<float>& samples, const MelConfig& c, int* frames);

struct Image {
    int width = 0, height = 0, channels = 3;
    std::vector<uint8_t> pixels;     // HWC
};

// Upper bound on width x height that the decoders accept before they allocate anything (headers come from untrusted
// requests).  64 Mpixel by default; `TELB_MAX_IMAGE_PIXELS` overrides it for the process.
uint64_t max_image_pixels();
Image parse_image(const std::string& bytes);                         // by magic: PNG, JPEG, PPM (P6), PGM (P5), BMP 24 / 32 bit
Image decode_png(const std::string& bytes);                          // non-interlaced; always returns RGB
Image decode_jpeg(const std::string& bytes);                         // sequential or progressive Huffman; always returns RGB
// RFC 1950 zlib stream → bytes; throws when the output would exceed `max_output`.
std::string inflate_zlib(const std::string& stream, size_t max_output);
Image load_image(const std::string& path);
Image resize_bilinear(const Image& im, int out_w, int out_h);
Image resize_bicubic(const Image& im, int out_w, int out_h);
// HWC uint8 → CHW float, (x / 255 - mean[c]) / std[c]
std::vector<float> normalize_chw(const Image& im, const std::vector<float>& mean, const std::vector<float>& stddev);
// Largest (h, w) with h, w multiples of `factor`, min_pixels ≤ h·w ≤ max_pixels and close to the input aspect ratio
// (the "smart resize" rule of the Qwen-VL image processors).
void smart_resize(int height, int width, int factor, long long min_pixels, long long max_pixels, int* out_h, int* out_w);

}  // namespace telb
