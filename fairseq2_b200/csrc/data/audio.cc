// WAV decoding, Kaldi-style filter bank features and PNG decoding for the
// native data pipeline (no external codec libraries are required).
#include <zlib.h>

#include <cmath>
#include <cstring>

#include "extras.h"

namespace fs2d {

namespace {

uint32_t le32(const uint8_t* p) { return p[0] | (p[1] << 8) | (p[2] << 16) | (static_cast<uint32_t>(p[3]) << 24); }
uint16_t le16(const uint8_t* p) { return static_cast<uint16_t>(p[0] | (p[1] << 8)); }
uint32_t be32(const uint8_t* p) { return (static_cast<uint32_t>(p[0]) << 24) | (p[1] << 16) | (p[2] << 8) | p[3]; }

}  // namespace

// =================================================================== AudioDecoder
Data AudioDecoder::operator()(Data&& d) const {
    if (!d.is_memory_block()) throw std::invalid_argument("The input data must be of type `MemoryBlock`.");
    const MemoryBlock& mb = d.as_memory_block();
    const uint8_t* b = mb.data();
    const size_t n = mb.size();
    if (n < 44 || std::memcmp(b, "RIFF", 4) != 0 || std::memcmp(b + 8, "WAVE", 4) != 0)
        throw std::invalid_argument("The input audio is not a RIFF/WAVE file (only WAV is supported by this build).");
    size_t p = 12;
    uint16_t fmt = 0, channels = 0, bits = 0;
    uint32_t rate = 0;
    const uint8_t* data = nullptr;
    size_t data_len = 0;
    while (p + 8 <= n) {
        const uint32_t len = le32(b + p + 4);
        if (std::memcmp(b + p, "fmt ", 4) == 0 && p + 8 + 16 <= n) {
            fmt = le16(b + p + 8);
            channels = le16(b + p + 10);
            rate = le32(b + p + 12);
            bits = le16(b + p + 22);
            if (fmt == 0xFFFE && len >= 26) fmt = le16(b + p + 8 + 24);  // WAVE_FORMAT_EXTENSIBLE sub-format
        } else if (std::memcmp(b + p, "data", 4) == 0) {
            data = b + p + 8;
            data_len = std::min<size_t>(len, n - (p + 8));
            break;
        }
        p += 8 + len + (len & 1);
    }
    if (data == nullptr || channels == 0 || bits == 0) throw std::invalid_argument("The WAV file has no fmt/data chunk.");
    const size_t bytes = bits / 8;
    const int64_t frames = static_cast<int64_t>(data_len / (bytes * channels));
    at::ScalarType out_dtype = dtype_.value_or(fmt == 3 ? at::kFloat : (bits <= 16 ? at::kShort : at::kInt));
    at::Tensor wav = at::empty({frames, channels}, at::kFloat);
    float* w = wav.data_ptr<float>();
    const bool to_float = at::isFloatingType(out_dtype);
    for (int64_t i = 0; i < frames * channels; ++i) {
        const uint8_t* s = data + i * bytes;
        float v;
        if (fmt == 3 && bits == 32) {
            std::memcpy(&v, s, 4);
        } else if (fmt == 1 && bits == 16) {
            v = static_cast<int16_t>(le16(s));
            if (to_float) v /= 32768.f;
        } else if (fmt == 1 && bits == 8) {
            v = static_cast<float>(s[0]) - 128.f;
            if (to_float) v /= 128.f;
        } else if (fmt == 1 && bits == 24) {
            int32_t x = (s[0] | (s[1] << 8) | (s[2] << 16));
            if (x & 0x800000) x |= ~0xFFFFFF;
            v = static_cast<float>(x);
            if (to_float) v /= 8388608.f;
        } else if (fmt == 1 && bits == 32) {
            v = static_cast<float>(static_cast<int32_t>(le32(s)));
            if (to_float) v /= 2147483648.f;
        } else {
            throw std::invalid_argument("The WAV sample format is not supported.");
        }
        w[i] = v;
    }
    at::Tensor out = wav.to(out_dtype);
    if (!keepdim_ && channels == 1) out = out.squeeze(-1);
    std::string format = std::string("WAV/") + (fmt == 3 ? "FLOAT" : "PCM_") + (fmt == 3 ? "" : std::to_string(bits));
    DataDict res{{"waveform", Data(out)}, {"sample_rate", Data(static_cast<double>(rate))}, {"format", Data(format)}};
    return Data(std::move(res));
}

// ======================================================= WaveformToFbankConverter
Data WaveformToFbankConverter::operator()(Data&& d) const {
    if (!d.is_dict()) throw std::invalid_argument("The input data must be a dict with 'waveform' and 'sample_rate'.");
    const Data* wv = d.find("waveform");
    const Data* sr = d.find("sample_rate");
    if (wv == nullptr || !wv->is_tensor() || sr == nullptr || !(sr->is_float() || sr->is_int()))
        throw std::invalid_argument("The input dict must have a 'waveform' tensor and a numeric 'sample_rate'.");
    const double rate = sr->is_float() ? sr->as_float() : static_cast<double>(sr->as_int());
    at::Tensor wav = wv->as_tensor().to(at::kFloat);
    if (wav.dim() == 1) wav = wav.unsqueeze(channel_last_ ? 1 : 0);
    if (wav.dim() != 2) throw std::invalid_argument("The waveform must be one or two dimensional.");
    at::Tensor mono = (channel_last_ ? wav.select(1, 0) : wav.select(0, 0)).contiguous() * scale_;

    const int64_t win = static_cast<int64_t>(rate * 0.025), shift = static_cast<int64_t>(rate * 0.010);
    const int64_t num_samples = mono.size(0);
    if (num_samples < win) throw std::invalid_argument("The waveform is shorter than one analysis window.");
    const int64_t num_frames = 1 + (num_samples - win) / shift;
    int64_t nfft = 1;
    while (nfft < win) nfft <<= 1;

    at::Tensor frames = mono.unfold(0, win, shift).clone();               // [F, win]
    frames = frames - frames.mean(1, true);                               // remove DC offset
    at::Tensor first = frames.narrow(1, 0, 1);
    at::Tensor shifted = at::cat({first, frames.narrow(1, 0, win - 1)}, 1);
    frames = frames - 0.97 * shifted;                                     // pre-emphasis
    at::Tensor k = at::arange(win, at::kFloat);
    at::Tensor povey = at::pow(0.5 - 0.5 * at::cos(2.0 * M_PI * k / (win - 1)), 0.85);
    frames = frames * povey;
    at::Tensor padded = at::zeros({num_frames, nfft}, at::kFloat);
    padded.narrow(1, 0, win).copy_(frames);
    at::Tensor spec = at::abs(at::fft_rfft(padded, nfft, 1)).pow(2);      // power spectrum [F, nfft/2+1]

    // mel filter bank (Kaldi: 20 Hz .. Nyquist, triangular filters on the mel scale)
    const double low = 20.0, high = rate / 2.0;
    auto mel = [](double f) { return 1127.0 * std::log(1.0 + f / 700.0); };
    const double mlow = mel(low), mhigh = mel(high);
    const int64_t bins = nfft / 2 + 1;
    at::Tensor fb = at::zeros({num_mel_bins_, bins}, at::kFloat);
    float* fbp = fb.data_ptr<float>();
    const double delta = (mhigh - mlow) / (num_mel_bins_ + 1);
    for (int m = 0; m < num_mel_bins_; ++m) {
        const double left = mlow + m * delta, center = left + delta, right = center + delta;
        for (int64_t i = 0; i < nfft / 2; ++i) {
            const double mf = mel(rate * i / nfft);
            if (mf > left && mf < right)
                fbp[m * bins + i] = static_cast<float>(mf <= center ? (mf - left) / (center - left)
                                                                     : (right - mf) / (right - center));
        }
    }
    at::Tensor feats = at::log(at::clamp_min(at::matmul(spec, fb.t()), 1.1920929e-7));  // [F, mel]
    if (standardize_) {
        at::Tensor mu = feats.mean(0, true), sd = feats.std(0, true, true);
        feats = (feats - mu) / (sd + 1e-8);
    }
    if (dtype_) feats = feats.to(*dtype_);
    DataDict out;
    for (const auto& kv : d.as_dict()) {
        if (kv.first == "waveform" && !keep_waveform_) continue;
        out.push_back(kv);
    }
    out.emplace_back("fbank", Data(feats));
    return Data(std::move(out));
}

// ================================================================== ImageDecoder
Data ImageDecoder::operator()(Data&& d) const {
    if (!d.is_memory_block()) throw std::invalid_argument("The input data must be of type `MemoryBlock`.");
    const MemoryBlock& mb = d.as_memory_block();
    const uint8_t* b = mb.data();
    const size_t n = mb.size();
    static const uint8_t sig[8] = {0x89, 'P', 'N', 'G', 0x0D, 0x0A, 0x1A, 0x0A};
    if (n < 8 || std::memcmp(b, sig, 8) != 0)
        throw std::invalid_argument("The input image is not a PNG file (JPEG decoding is not available in this build).");
    size_t p = 8;
    uint32_t width = 0, height = 0;
    int depth = 0, color = 0, interlace = 0;
    std::vector<uint8_t> idat, palette;
    while (p + 12 <= n) {
        const uint32_t len = be32(b + p);
        const uint8_t* type = b + p + 4;
        const uint8_t* body = b + p + 8;
        if (p + 12 + len > n) throw std::invalid_argument("The PNG file is truncated.");
        if (std::memcmp(type, "IHDR", 4) == 0) {
            width = be32(body);
            height = be32(body + 4);
            depth = body[8];
            color = body[9];
            interlace = body[12];
        } else if (std::memcmp(type, "PLTE", 4) == 0) {
            palette.assign(body, body + len);
        } else if (std::memcmp(type, "IDAT", 4) == 0) {
            idat.insert(idat.end(), body, body + len);
        } else if (std::memcmp(type, "IEND", 4) == 0) {
            break;
        }
        p += 12 + len;
    }
    if (width == 0 || height == 0) throw std::invalid_argument("The PNG file has no IHDR chunk.");
    if (interlace != 0) throw std::invalid_argument("Interlaced PNG files are not supported.");
    int channels = color == 0 ? 1 : color == 2 ? 3 : color == 3 ? 1 : color == 4 ? 2 : 4;
    if (depth != 8 && depth != 16) throw std::invalid_argument("Only 8- and 16-bit PNG files are supported.");
    const size_t bpp = static_cast<size_t>(channels) * depth / 8;
    const size_t stride = width * bpp;
    std::vector<uint8_t> raw((stride + 1) * height);
    uLongf out_len = raw.size();
    if (uncompress(raw.data(), &out_len, idat.data(), idat.size()) != Z_OK || out_len != raw.size())
        throw std::invalid_argument("The PNG image data cannot be inflated.");
    std::vector<uint8_t> img(stride * height);
    for (uint32_t y = 0; y < height; ++y) {
        const uint8_t ft = raw[y * (stride + 1)];
        const uint8_t* src = raw.data() + y * (stride + 1) + 1;
        uint8_t* dst = img.data() + y * stride;
        const uint8_t* up = y > 0 ? dst - stride : nullptr;
        for (size_t x = 0; x < stride; ++x) {
            const int a = x >= bpp ? dst[x - bpp] : 0;
            const int bb = up ? up[x] : 0;
            const int c = (up && x >= bpp) ? up[x - bpp] : 0;
            int pred = 0;
            switch (ft) {
                case 0: pred = 0; break;
                case 1: pred = a; break;
                case 2: pred = bb; break;
                case 3: pred = (a + bb) / 2; break;
                case 4: {
                    const int pp = a + bb - c, pa = std::abs(pp - a), pb = std::abs(pp - bb), pc = std::abs(pp - c);
                    pred = (pa <= pb && pa <= pc) ? a : (pb <= pc ? bb : c);
                    break;
                }
                default: throw std::invalid_argument("The PNG file uses an unknown filter type.");
            }
            dst[x] = static_cast<uint8_t>(src[x] + pred);
        }
    }
    at::Tensor out;
    if (color == 3) {
        out = at::empty({static_cast<int64_t>(height), static_cast<int64_t>(width), 3}, at::kByte);
        uint8_t* o = out.data_ptr<uint8_t>();
        for (size_t i = 0; i < static_cast<size_t>(width) * height; ++i) {
            const size_t idx = static_cast<size_t>(img[i]) * 3;
            if (idx + 2 >= palette.size())
                throw std::invalid_argument("The PNG palette index is out of range.");
            o[3 * i] = palette[idx];
            o[3 * i + 1] = palette[idx + 1];
            o[3 * i + 2] = palette[idx + 2];
        }
        channels = 3;
    } else if (depth == 8) {
        out = at::empty({static_cast<int64_t>(height), static_cast<int64_t>(width), channels}, at::kByte);
        std::memcpy(out.data_ptr<uint8_t>(), img.data(), img.size());
    } else {
        out = at::empty({static_cast<int64_t>(height), static_cast<int64_t>(width), channels}, at::kShort);
        int16_t* o = out.data_ptr<int16_t>();
        for (size_t i = 0; i < img.size() / 2; ++i) o[i] = static_cast<int16_t>((img[2 * i] << 8) | img[2 * i + 1]);
    }
    DataDict res{{"bit_depth", Data(static_cast<double>(depth))}, {"format", Data(static_cast<double>(channels))},
                 {"image", Data(out)}};
    return Data(std::move(res));
}

}  // namespace fs2d
