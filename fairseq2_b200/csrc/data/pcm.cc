// Uncompressed audio containers of the data pipeline: RIFF/WAVE (also RF64 sizes and WAVE_FORMAT_EXTENSIBLE),
// AIFF / AIFF-C and Sun/NeXT AU. Sample encodings: signed/unsigned integer PCM of 8 to 32 bits in either byte
// order, IEEE float 32/64, and the G.711 companded forms (mu-law, A-law). Integer samples are decoded exactly
// (no float intermediate), so 32-bit PCM survives a round trip.
#include <cmath>
#include <cstring>

#include "extras.h"

namespace fs2d {

namespace {

uint32_t le32(const uint8_t* p) { return p[0] | (p[1] << 8) | (p[2] << 16) | (static_cast<uint32_t>(p[3]) << 24); }
uint16_t le16(const uint8_t* p) { return static_cast<uint16_t>(p[0] | (p[1] << 8)); }
uint32_t be32(const uint8_t* p) { return (static_cast<uint32_t>(p[0]) << 24) | (p[1] << 16) | (p[2] << 8) | p[3]; }
uint16_t be16(const uint8_t* p) { return static_cast<uint16_t>((p[0] << 8) | p[1]); }

enum class Enc { Int, UInt8, Float, ULaw, ALaw };

struct PcmSpec {
    const char* container = "";
    Enc enc = Enc::Int;
    bool big_endian = false;
    int bits = 0;          // stored bits per sample (8, 16, 24, 32, 64)
    int channels = 0;
    double rate = 0.0;
    const uint8_t* data = nullptr;
    size_t len = 0;
};

int16_t ulaw_to_linear(uint8_t u) {
    u = static_cast<uint8_t>(~u);
    int t = (((u & 0x0f) << 3) + 0x84) << ((u >> 4) & 7);
    t -= 0x84;
    return static_cast<int16_t>((u & 0x80) ? -t : t);
}

int16_t alaw_to_linear(uint8_t a) {
    a ^= 0x55;
    int exponent = (a >> 4) & 7, mantissa = a & 0x0f;
    int t = exponent == 0 ? (mantissa << 4) + 8 : ((mantissa << 4) + 0x108) << (exponent - 1);
    return static_cast<int16_t>((a & 0x80) ? t : -t);
}

// 80-bit IEEE 754 extended (the sample rate field of AIFF)
double extended_to_double(const uint8_t* p) {
    const int exponent = ((p[0] & 0x7f) << 8) | p[1];
    uint64_t mantissa = 0;
    for (int i = 0; i < 8; ++i) mantissa = (mantissa << 8) | p[2 + i];
    if (exponent == 0 && mantissa == 0) return 0.0;
    double v = std::ldexp(static_cast<double>(mantissa), exponent - 16383 - 63);
    return (p[0] & 0x80) ? -v : v;
}

bool parse_wav(const uint8_t* b, size_t n, PcmSpec& s) {
    if (n < 12 || (std::memcmp(b, "RIFF", 4) != 0 && std::memcmp(b, "RF64", 4) != 0) || std::memcmp(b + 8, "WAVE", 4) != 0)
        return false;
    s.container = "WAV";
    size_t p = 12;
    uint16_t fmt = 0;
    bool have_fmt = false;
    while (p + 8 <= n) {
        const uint32_t len = le32(b + p + 4);
        if (std::memcmp(b + p, "fmt ", 4) == 0 && p + 8 + 16 <= n) {
            fmt = le16(b + p + 8);
            s.channels = le16(b + p + 10);
            s.rate = le32(b + p + 12);
            s.bits = le16(b + p + 22);
            if (fmt == 0xFFFE && len >= 26 && p + 8 + 26 <= n) fmt = le16(b + p + 8 + 24);   // sub-format
            have_fmt = true;
        } else if (std::memcmp(b + p, "data", 4) == 0) {
            s.data = b + p + 8;
            // 0xFFFFFFFF: the real size is in an RF64 ds64 chunk or unknown (streamed): use what is there
            s.len = len == 0xFFFFFFFFu ? n - (p + 8) : std::min<size_t>(len, n - (p + 8));
            break;
        }
        p += 8 + static_cast<size_t>(len) + (len & 1);
    }
    if (!have_fmt || s.data == nullptr) throw std::invalid_argument("The WAV file has no fmt/data chunk.");
    switch (fmt) {
        case 1: s.enc = s.bits == 8 ? Enc::UInt8 : Enc::Int; break;
        case 3: s.enc = Enc::Float; break;
        case 6: s.enc = Enc::ALaw; break;
        case 7: s.enc = Enc::ULaw; break;
        default: throw std::invalid_argument("The WAV sample format (tag " + std::to_string(fmt) + ") is not supported.");
    }
    return true;
}

bool parse_aiff(const uint8_t* b, size_t n, PcmSpec& s) {
    if (n < 12 || std::memcmp(b, "FORM", 4) != 0) return false;
    const bool aifc = std::memcmp(b + 8, "AIFC", 4) == 0;
    if (!aifc && std::memcmp(b + 8, "AIFF", 4) != 0) return false;
    s.container = "AIFF";
    s.big_endian = true;
    size_t p = 12;
    bool have_comm = false;
    uint32_t frames = 0;
    while (p + 8 <= n) {
        const uint32_t len = be32(b + p + 4);
        const uint8_t* c = b + p + 8;
        if (std::memcmp(b + p, "COMM", 4) == 0 && p + 8 + 18 <= n) {
            s.channels = be16(c);
            frames = be32(c + 2);
            s.bits = be16(c + 6);
            s.rate = extended_to_double(c + 8);
            s.enc = Enc::Int;
            if (aifc && len >= 22 && p + 8 + 22 <= n) {
                const char* t = reinterpret_cast<const char*>(c + 18);
                if (std::memcmp(t, "NONE", 4) == 0 || std::memcmp(t, "twos", 4) == 0) {
                } else if (std::memcmp(t, "sowt", 4) == 0) {
                    s.big_endian = false;
                } else if (std::memcmp(t, "fl32", 4) == 0 || std::memcmp(t, "FL32", 4) == 0) {
                    s.enc = Enc::Float;
                    s.bits = 32;
                } else if (std::memcmp(t, "fl64", 4) == 0 || std::memcmp(t, "FL64", 4) == 0) {
                    s.enc = Enc::Float;
                    s.bits = 64;
                } else if (std::memcmp(t, "ulaw", 4) == 0 || std::memcmp(t, "ULAW", 4) == 0) {
                    s.enc = Enc::ULaw;
                    s.bits = 8;
                } else if (std::memcmp(t, "alaw", 4) == 0 || std::memcmp(t, "ALAW", 4) == 0) {
                    s.enc = Enc::ALaw;
                    s.bits = 8;
                } else {
                    throw std::invalid_argument("The AIFF-C compression type '" + std::string(t, 4) + "' is not supported.");
                }
            }
            have_comm = true;
        } else if (std::memcmp(b + p, "SSND", 4) == 0 && p + 16 <= n) {
            const uint32_t offset = be32(c);
            if (8 + static_cast<size_t>(offset) <= len) {
                s.data = c + 8 + offset;
                s.len = std::min<size_t>(len - 8 - offset, n - (p + 16 + offset));
            }
        }
        p += 8 + static_cast<size_t>(len) + (len & 1);
    }
    if (!have_comm) throw std::invalid_argument("The AIFF file has no COMM chunk.");
    if (s.data == nullptr) {
        if (frames != 0) throw std::invalid_argument("The AIFF file has no SSND chunk.");
        s.data = b;
        s.len = 0;
    }
    // sample sizes that are not a multiple of 8 are stored left-justified in the next whole number of bytes
    s.bits = (s.bits + 7) / 8 * 8;
    const size_t frame_bytes = static_cast<size_t>(s.bits / 8) * static_cast<size_t>(std::max(s.channels, 1));
    s.len = std::min(s.len, static_cast<size_t>(frames) * frame_bytes);
    return true;
}

bool parse_au(const uint8_t* b, size_t n, PcmSpec& s) {
    if (n < 24 || std::memcmp(b, ".snd", 4) != 0) return false;
    s.container = "AU";
    s.big_endian = true;
    const uint32_t offset = be32(b + 4), size = be32(b + 8), encoding = be32(b + 12);
    s.rate = be32(b + 16);
    s.channels = static_cast<int>(be32(b + 20));
    if (offset < 24 || offset > n) throw std::invalid_argument("The AU header has an invalid data offset.");
    s.data = b + offset;
    s.len = size == 0xFFFFFFFFu ? n - offset : std::min<size_t>(size, n - offset);
    switch (encoding) {
        case 1: s.enc = Enc::ULaw; s.bits = 8; break;
        case 2: s.enc = Enc::Int; s.bits = 8; break;
        case 3: s.enc = Enc::Int; s.bits = 16; break;
        case 4: s.enc = Enc::Int; s.bits = 24; break;
        case 5: s.enc = Enc::Int; s.bits = 32; break;
        case 6: s.enc = Enc::Float; s.bits = 32; break;
        case 7: s.enc = Enc::Float; s.bits = 64; break;
        case 27: s.enc = Enc::ALaw; s.bits = 8; break;
        default: throw std::invalid_argument("The AU encoding " + std::to_string(encoding) + " is not supported.");
    }
    return true;
}

}  // namespace

bool is_pcm_container(const uint8_t* b, size_t n) {
    if (n < 12) return false;
    return std::memcmp(b, "RIFF", 4) == 0 || std::memcmp(b, "RF64", 4) == 0 || std::memcmp(b, "FORM", 4) == 0 ||
           std::memcmp(b, ".snd", 4) == 0;
}

at::Tensor decode_pcm_container(const uint8_t* b, size_t n, std::optional<at::ScalarType> dtype, double& rate,
                                std::string& format) {
    PcmSpec s;
    if (!parse_wav(b, n, s) && !parse_aiff(b, n, s) && !parse_au(b, n, s))
        throw std::invalid_argument("The input audio is not a WAV, AIFF, AU or FLAC stream.");
    if (s.channels <= 0 || s.channels > 1024) throw std::invalid_argument("The audio header gives an invalid channel count.");
    const bool companded = s.enc == Enc::ULaw || s.enc == Enc::ALaw;
    if (companded && s.bits != 8) throw std::invalid_argument("Companded audio must have 8 bits per sample.");
    if (s.enc == Enc::Float && s.bits != 32 && s.bits != 64)
        throw std::invalid_argument("Floating-point audio must have 32 or 64 bits per sample.");
    if ((s.enc == Enc::Int || s.enc == Enc::UInt8) && s.bits != 8 && s.bits != 16 && s.bits != 24 && s.bits != 32)
        throw std::invalid_argument("Integer audio of " + std::to_string(s.bits) + " bits per sample is not supported.");
    const size_t bytes = static_cast<size_t>(s.bits / 8);
    const int64_t frames = static_cast<int64_t>(s.len / (bytes * static_cast<size_t>(s.channels)));
    const int64_t count = frames * s.channels;
    rate = s.rate;

    at::Tensor out;
    if (s.enc == Enc::Float) {
        at::Tensor raw = at::empty({frames, s.channels}, s.bits == 32 ? at::kFloat : at::kDouble);
        uint8_t* dst = static_cast<uint8_t*>(raw.data_ptr());
        if (!s.big_endian) {
            std::memcpy(dst, s.data, static_cast<size_t>(count) * bytes);
        } else {
            for (int64_t i = 0; i < count; ++i)
                for (size_t k = 0; k < bytes; ++k) dst[i * bytes + k] = s.data[i * bytes + (bytes - 1 - k)];
        }
        out = raw.to(dtype.value_or(at::kFloat));
        format = std::string(s.container) + (s.bits == 32 ? "/FLOAT" : "/DOUBLE");
    } else {
        at::Tensor raw = at::empty({frames, s.channels}, at::kInt);
        int32_t* w = raw.data_ptr<int32_t>();
        int value_bits = s.bits;
        if (companded) {
            value_bits = 16;
            for (int64_t i = 0; i < count; ++i)
                w[i] = s.enc == Enc::ULaw ? ulaw_to_linear(s.data[i]) : alaw_to_linear(s.data[i]);
        } else if (s.enc == Enc::UInt8) {
            for (int64_t i = 0; i < count; ++i) w[i] = static_cast<int32_t>(s.data[i]) - 128;
        } else {
            for (int64_t i = 0; i < count; ++i) {
                const uint8_t* p = s.data + static_cast<size_t>(i) * bytes;
                uint32_t v = 0;
                if (s.big_endian)
                    for (size_t k = 0; k < bytes; ++k) v = (v << 8) | p[k];
                else
                    for (size_t k = bytes; k-- > 0;) v = (v << 8) | p[k];
                const int shift = 32 - s.bits;                       // sign-extend from `bits`
                w[i] = static_cast<int32_t>(v << shift) >> shift;
            }
        }
        const at::ScalarType out_dtype = dtype.value_or(value_bits <= 16 ? at::kShort : at::kInt);
        if (at::isFloatingType(out_dtype))
            out = (raw.to(at::kDouble) / static_cast<double>(int64_t{1} << (value_bits - 1))).to(out_dtype);
        else
            out = raw.to(out_dtype);
        format = std::string(s.container) + "/" +
                 (s.enc == Enc::ULaw ? "ULAW" : s.enc == Enc::ALaw ? "ALAW" : "PCM_" + std::to_string(s.bits));
    }
    return out;
}

}  // namespace fs2d
