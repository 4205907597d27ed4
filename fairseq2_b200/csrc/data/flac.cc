// FLAC (free lossless audio codec) stream decoder for the audio pipeline operator: STREAMINFO, fixed and variable
// block-size frames, constant / verbatim / fixed-predictor / LPC subframes, Rice and escaped residual partitions,
// wasted bits, all four channel assignments, CRC-8 of every frame header and CRC-16 of every frame. Written from
// the format specification (RFC 9639); fairseq2n gets the same capability from libsndfile
// (data/audio/detail/sndfile.cc).
#include <cstring>
#include <stdexcept>
#include <string>

#include "extras.h"

namespace fs2d {

namespace {

struct FlacError : std::invalid_argument {
    explicit FlacError(const std::string& m) : std::invalid_argument("The FLAC stream is invalid: " + m) {}
};

class BitReader {
public:
    BitReader(const uint8_t* p, size_t n) : p_(p), n_(n) {}

    uint32_t bits(int count) {          // count <= 32
        uint32_t v = 0;
        while (count > 0) {
            if (byte_ >= n_) throw FlacError("the stream ends inside a frame.");
            const int avail = 8 - bit_;
            const int take = count < avail ? count : avail;
            const uint32_t chunk = (p_[byte_] >> (avail - take)) & ((1u << take) - 1u);
            v = take == 32 ? chunk : ((v << take) | chunk);
            bit_ += take;
            if (bit_ == 8) {
                bit_ = 0;
                ++byte_;
            }
            count -= take;
        }
        return v;
    }
    int64_t sbits(int count) {          // two's complement, count <= 33 (side channel of 32-bit audio)
        if (count == 0) return 0;
        uint64_t v = count > 32 ? (static_cast<uint64_t>(bits(count - 32)) << 32) | bits(32) : bits(count);
        const uint64_t sign = 1ull << (count - 1);
        return static_cast<int64_t>((v ^ sign)) - static_cast<int64_t>(sign);
    }
    uint32_t unary() {                  // number of zero bits before the next one bit
        uint32_t zeros = 0;
        while (true) {
            if (byte_ >= n_) throw FlacError("the stream ends inside a residual.");
            const uint8_t rest = static_cast<uint8_t>(p_[byte_] << bit_);
            if (rest == 0) {
                zeros += static_cast<uint32_t>(8 - bit_);
                bit_ = 0;
                ++byte_;
                continue;
            }
            const int lead = __builtin_clz(static_cast<uint32_t>(rest)) - 24;
            zeros += static_cast<uint32_t>(lead);
            bit_ += lead + 1;
            if (bit_ >= 8) {
                bit_ -= 8;
                ++byte_;
            }
            return zeros;
        }
    }
    void align() {
        if (bit_ != 0) {
            bit_ = 0;
            ++byte_;
        }
    }
    size_t byte_pos() const { return byte_; }
    bool aligned() const { return bit_ == 0; }

private:
    const uint8_t* p_;
    size_t n_;
    size_t byte_ = 0;
    int bit_ = 0;
};

uint8_t crc8(const uint8_t* p, size_t n) {
    uint8_t c = 0;
    for (size_t i = 0; i < n; ++i) {
        c ^= p[i];
        for (int k = 0; k < 8; ++k) c = static_cast<uint8_t>((c & 0x80) ? (c << 1) ^ 0x07 : (c << 1));
    }
    return c;
}

uint16_t crc16(const uint8_t* p, size_t n) {
    uint16_t c = 0;
    for (size_t i = 0; i < n; ++i) {
        c = static_cast<uint16_t>(c ^ (p[i] << 8));
        for (int k = 0; k < 8; ++k) c = static_cast<uint16_t>((c & 0x8000) ? (c << 1) ^ 0x8005 : (c << 1));
    }
    return c;
}

void read_residual(BitReader& br, int order, int block, int64_t* out) {
    const uint32_t method = br.bits(2);
    if (method > 1) throw FlacError("reserved residual coding method.");
    const int param_bits = method == 0 ? 4 : 5;
    const uint32_t escape = method == 0 ? 15u : 31u;
    const int porder = static_cast<int>(br.bits(4));
    const int parts = 1 << porder;
    if ((block % parts) != 0 || (block >> porder) < order) throw FlacError("bad residual partition order.");
    int i = order;
    for (int part = 0; part < parts; ++part) {
        const int count = (block >> porder) - (part == 0 ? order : 0);
        const uint32_t param = br.bits(param_bits);
        if (param == escape) {
            const int raw = static_cast<int>(br.bits(5));
            for (int k = 0; k < count; ++k) out[i++] = br.sbits(raw);
        } else {
            for (int k = 0; k < count; ++k) {
                const uint64_t q = br.unary();
                const uint64_t u = (q << param) | (param ? br.bits(static_cast<int>(param)) : 0u);
                out[i++] = static_cast<int64_t>(u >> 1) ^ -static_cast<int64_t>(u & 1);
            }
        }
    }
}

void read_subframe(BitReader& br, int bps, int block, int64_t* s) {
    if (br.bits(1) != 0) throw FlacError("non-zero subframe padding bit.");
    const uint32_t type = br.bits(6);
    int wasted = 0;
    if (br.bits(1)) wasted = static_cast<int>(br.unary()) + 1;
    if (wasted >= bps) throw FlacError("more wasted bits than sample bits.");
    bps -= wasted;
    if (type == 0) {
        const int64_t v = br.sbits(bps);
        for (int i = 0; i < block; ++i) s[i] = v;
    } else if (type == 1) {
        for (int i = 0; i < block; ++i) s[i] = br.sbits(bps);
    } else if (type >= 8 && type <= 12) {
        const int order = static_cast<int>(type) - 8;
        if (order > block) throw FlacError("fixed predictor order exceeds the block size.");
        for (int i = 0; i < order; ++i) s[i] = br.sbits(bps);
        read_residual(br, order, block, s);
        for (int i = order; i < block; ++i) {
            int64_t pred = 0;
            switch (order) {
                case 1: pred = s[i - 1]; break;
                case 2: pred = 2 * s[i - 1] - s[i - 2]; break;
                case 3: pred = 3 * s[i - 1] - 3 * s[i - 2] + s[i - 3]; break;
                case 4: pred = 4 * s[i - 1] - 6 * s[i - 2] + 4 * s[i - 3] - s[i - 4]; break;
                default: break;
            }
            s[i] += pred;
        }
    } else if (type >= 32) {
        const int order = static_cast<int>(type) - 31;
        if (order > block) throw FlacError("LPC order exceeds the block size.");
        for (int i = 0; i < order; ++i) s[i] = br.sbits(bps);
        const int precision = static_cast<int>(br.bits(4)) + 1;
        if (precision == 16) throw FlacError("reserved LPC precision.");
        const int64_t shift = br.sbits(5);
        if (shift < 0) throw FlacError("negative LPC shift.");
        int64_t coef[32];
        for (int j = 0; j < order; ++j) coef[j] = br.sbits(precision);
        read_residual(br, order, block, s);
        for (int i = order; i < block; ++i) {
            int64_t acc = 0;
            for (int j = 0; j < order; ++j) acc += coef[j] * s[i - 1 - j];
            s[i] += acc >> shift;
        }
    } else {
        throw FlacError("reserved subframe type.");
    }
    if (wasted)
        for (int i = 0; i < block; ++i) s[i] *= (int64_t{1} << wasted);
}

}  // namespace

bool is_flac(const uint8_t* b, size_t n) { return n >= 4 && std::memcmp(b, "fLaC", 4) == 0; }

// Decodes a whole stream into interleaved samples [frames, channels] (int32; 32-bit audio fits, the side channel's
// extra bit is gone after decorrelation).
at::Tensor decode_flac(const uint8_t* b, size_t n, int& sample_rate, int& bits_per_sample) {
    if (!is_flac(b, n)) throw FlacError("missing 'fLaC' marker.");
    size_t p = 4;
    bool have_info = false, last = false;
    int channels = 0, bps = 0, rate = 0, max_block = 0;
    uint64_t total = 0;
    while (!last) {
        if (p + 4 > n) throw FlacError("truncated metadata.");
        last = (b[p] & 0x80) != 0;
        const int type = b[p] & 0x7f;
        const size_t len = (static_cast<size_t>(b[p + 1]) << 16) | (b[p + 2] << 8) | b[p + 3];
        p += 4;
        if (p + len > n) throw FlacError("truncated metadata block.");
        if (type == 0) {
            if (len < 34) throw FlacError("short STREAMINFO block.");
            const uint8_t* s = b + p;
            max_block = (s[2] << 8) | s[3];
            rate = (s[10] << 12) | (s[11] << 4) | (s[12] >> 4);
            channels = ((s[12] >> 1) & 7) + 1;
            bps = (((s[12] & 1) << 4) | (s[13] >> 4)) + 1;
            total = (static_cast<uint64_t>(s[13] & 15) << 32) | (static_cast<uint64_t>(s[14]) << 24) | (s[15] << 16) |
                    (s[16] << 8) | s[17];
            have_info = true;
        } else if (type == 127) {
            throw FlacError("forbidden metadata block type.");
        }
        p += len;
    }
    if (!have_info || rate == 0 || bps < 4 || bps > 32 || max_block < 16) throw FlacError("missing or bad STREAMINFO.");
    sample_rate = rate;
    bits_per_sample = bps;

    std::vector<int32_t> pcm;
    if (total) pcm.reserve(static_cast<size_t>(total) * channels);
    std::vector<int64_t> chan(static_cast<size_t>(8) * 65536);
    while (p + 2 <= n) {
        // frame header
        if (b[p] != 0xff || (b[p + 1] & 0xfe) != 0xf8) throw FlacError("lost frame synchronisation.");
        BitReader br(b + p, n - p);
        br.bits(15);
        br.bits(1);                                                 // blocking strategy: only affects the number below
        const uint32_t bs_code = br.bits(4), sr_code = br.bits(4), ch_code = br.bits(4), ss_code = br.bits(3);
        if (br.bits(1)) throw FlacError("reserved header bit set.");
        // UTF-8-like coded frame or sample number (up to 36 bits): only its length matters here
        const uint32_t first = br.bits(8);
        int extra = 0;
        if (first >= 0xfe) extra = 6;
        else if (first >= 0xfc) extra = 5;
        else if (first >= 0xf8) extra = 4;
        else if (first >= 0xf0) extra = 3;
        else if (first >= 0xe0) extra = 2;
        else if (first >= 0xc0) extra = 1;
        else if (first >= 0x80) throw FlacError("bad coded frame number.");
        for (int i = 0; i < extra; ++i)
            if ((br.bits(8) & 0xc0) != 0x80) throw FlacError("bad coded frame number.");
        int block;
        if (bs_code == 0) throw FlacError("reserved block size.");
        else if (bs_code == 1) block = 192;
        else if (bs_code <= 5) block = 576 << (bs_code - 2);
        else if (bs_code == 6) block = static_cast<int>(br.bits(8)) + 1;
        else if (bs_code == 7) block = static_cast<int>(br.bits(16)) + 1;
        else block = 256 << (bs_code - 8);
        if (sr_code == 12) br.bits(8);
        else if (sr_code == 13 || sr_code == 14) br.bits(16);
        else if (sr_code == 15) throw FlacError("invalid sample rate code.");
        static const int kSizes[8] = {0, 8, 12, -1, 16, 20, 24, 32};
        const int fbps = ss_code == 0 ? bps : kSizes[ss_code];
        if (fbps != bps) throw FlacError("a frame changes the sample size.");
        const size_t hdr_len = br.byte_pos();
        if (br.bits(8) != crc8(b + p, hdr_len)) throw FlacError("frame header CRC mismatch.");
        int nch;
        if (ch_code < 8) nch = static_cast<int>(ch_code) + 1;
        else if (ch_code <= 10) nch = 2;
        else throw FlacError("reserved channel assignment.");
        if (nch != channels) throw FlacError("a frame changes the channel count.");
        if (block > 65535 + 1) throw FlacError("block too large.");
        // subframes
        for (int c = 0; c < nch; ++c) {
            const bool side = (ch_code == 8 && c == 1) || (ch_code == 9 && c == 0) || (ch_code == 10 && c == 1);
            read_subframe(br, bps + (side ? 1 : 0), block, chan.data() + static_cast<size_t>(c) * 65536);
        }
        br.align();
        const size_t body = br.byte_pos();
        if (p + body + 2 > n) throw FlacError("truncated frame.");
        const uint16_t want = static_cast<uint16_t>((b[p + body] << 8) | b[p + body + 1]);
        if (want != crc16(b + p, body)) throw FlacError("frame CRC mismatch.");
        p += body + 2;
        // inter-channel decorrelation
        int64_t* c0 = chan.data();
        int64_t* c1 = chan.data() + 65536;
        if (ch_code == 8) {
            for (int i = 0; i < block; ++i) c1[i] = c0[i] - c1[i];
        } else if (ch_code == 9) {
            for (int i = 0; i < block; ++i) c0[i] = c1[i] + c0[i];
        } else if (ch_code == 10) {
            for (int i = 0; i < block; ++i) {
                const int64_t side = c1[i];
                const int64_t mid = c0[i] * 2 + (side & 1);
                c0[i] = (mid + side) >> 1;
                c1[i] = (mid - side) >> 1;
            }
        }
        const size_t at = pcm.size();
        pcm.resize(at + static_cast<size_t>(block) * nch);
        for (int i = 0; i < block; ++i)
            for (int c = 0; c < nch; ++c)
                pcm[at + static_cast<size_t>(i) * nch + c] = static_cast<int32_t>(chan[static_cast<size_t>(c) * 65536 + i]);
    }
    if (p != n) throw FlacError("trailing bytes after the last frame.");
    int64_t frames = static_cast<int64_t>(pcm.size() / channels);
    if (total && static_cast<uint64_t>(frames) > total) frames = static_cast<int64_t>(total);
    at::Tensor out = at::empty({frames, channels}, at::kInt);
    std::memcpy(out.data_ptr<int32_t>(), pcm.data(), static_cast<size_t>(frames) * channels * 4);
    return out;
}

}  // namespace fs2d
