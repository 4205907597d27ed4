// Audio decoding front (FLAC in flac.cc, WAV / AIFF / AU in pcm.cc), Kaldi-style filter bank features and PNG /
// JPEG decoding for the native data pipeline (no external codec libraries are required).
#include <cmath>
#include <cstring>

#include "extras.h"

namespace fs2d {

namespace {

uint32_t be32(const uint8_t* p) { return (static_cast<uint32_t>(p[0]) << 24) | (p[1] << 16) | (p[2] << 8) | p[3]; }

}  // namespace

// =================================================================== AudioDecoder
Data AudioDecoder::operator()(Data&& d) const {
    if (!d.is_memory_block()) throw std::invalid_argument("The input data must be of type `MemoryBlock`.");
    const MemoryBlock& mb = d.as_memory_block();
    const uint8_t* b = mb.data();
    const size_t n = mb.size();
    if (is_flac(b, n)) {
        int rate = 0, bps = 0;
        at::Tensor pcm = decode_flac(b, n, rate, bps);                                  // int32 [frames, channels]
        const at::ScalarType out_dtype = dtype_.value_or(bps <= 16 ? at::kShort : at::kInt);
        at::Tensor out = at::isFloatingType(out_dtype)
                             ? (pcm.to(at::kDouble) / static_cast<double>(int64_t{1} << (bps - 1))).to(out_dtype)
                             : pcm.to(out_dtype);
        if (!keepdim_ && out.size(1) == 1) out = out.squeeze(-1);
        DataDict res{{"waveform", Data(out)}, {"sample_rate", Data(static_cast<double>(rate))},
                     {"format", Data("FLAC/PCM_" + std::to_string(bps))}};
        return Data(std::move(res));
    }
    if (n >= 4 && std::memcmp(b, "OggS", 4) == 0)
        throw std::invalid_argument("Ogg containers (Vorbis/Opus) are lossy codecs that this build does not decode; "
                                    "convert the audio to FLAC or WAV.");
    double rate = 0.0;
    std::string format;
    at::Tensor out = decode_pcm_container(b, n, dtype_, rate, format);               // [frames, channels]
    if (!keepdim_ && out.size(1) == 1) out = out.squeeze(-1);
    DataDict res{{"waveform", Data(out)}, {"sample_rate", Data(rate)}, {"format", Data(format)}};
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

// ------------------------------------------------------------------------ JPEG
// DCT JPEG with Huffman coding, sequential (baseline / extended) and progressive (spectral selection + successive
// approximation), interleaved and non-interleaved scans: 8-bit samples, 1 or 3 components, sampling factors up to
// 2x2 (4:4:4, 4:2:2, 4:2:0), restart intervals. Scans fill per-component coefficient arrays; dequantisation, the
// inverse DCT, chroma upsampling and colour conversion run once after the last scan. Arithmetic-coded, lossless
// and hierarchical files are rejected.
namespace {

struct JpegHuff {
    uint8_t bits[17] = {0};
    uint8_t vals[256] = {0};
    int mincode[17] = {0}, maxcode[18] = {0}, valptr[17] = {0};
    bool present = false;
    void build() {
        int code = 0, k = 0;
        for (int l = 1; l <= 16; ++l) {
            valptr[l] = k;
            mincode[l] = code;
            code += bits[l];
            k += bits[l];
            maxcode[l] = bits[l] ? code - 1 : -1;
            code <<= 1;
        }
        maxcode[17] = 0x7fffffff;
        present = true;
    }
};

struct JpegBits {
    const uint8_t* p;
    const uint8_t* end;
    uint32_t acc = 0;
    int cnt = 0;
    int get_bit() {
        if (cnt == 0) {
            uint8_t b = p < end ? *p++ : 0;
            if (b == 0xFF) {
                const uint8_t b2 = p < end ? *p : 0;
                if (b2 == 0) ++p;                 // stuffed zero
                else { --p; b = 0; }              // a marker: feed zeros, the caller resynchronises
            }
            acc = b;
            cnt = 8;
        }
        --cnt;
        return (acc >> cnt) & 1;
    }
    int get_bits(int n) {
        int v = 0;
        for (int i = 0; i < n; ++i) v = (v << 1) | get_bit();
        return v;
    }
    void reset() { cnt = 0; }
};

int jpeg_decode_symbol(JpegBits& br, const JpegHuff& h) {
    int code = 0;
    for (int l = 1; l <= 16; ++l) {
        code = (code << 1) | br.get_bit();
        if (h.maxcode[l] >= 0 && code <= h.maxcode[l] && code >= h.mincode[l])
            return h.vals[h.valptr[l] + code - h.mincode[l]];
    }
    throw std::invalid_argument("The JPEG entropy-coded data is corrupt.");
}

int jpeg_extend(int v, int t) { return t == 0 ? 0 : (v < (1 << (t - 1)) ? v - (1 << t) + 1 : v); }

const int kZigzag[64] = {0,  1,  8,  16, 9,  2,  3,  10, 17, 24, 32, 25, 18, 11, 4,  5,  12, 19, 26, 33, 40, 48,
                         41, 34, 27, 20, 13, 6,  7,  14, 21, 28, 35, 42, 49, 56, 57, 50, 43, 36, 29, 22, 15, 23,
                         30, 37, 44, 51, 58, 59, 52, 45, 38, 31, 39, 46, 53, 60, 61, 54, 47, 55, 62, 63};

void jpeg_idct8x8(const float* in, uint8_t* out, int out_stride) {
    static float c[8][8];
    static bool init = false;
    if (!init) {
        for (int x = 0; x < 8; ++x)
            for (int u = 0; u < 8; ++u)
                c[x][u] = (u == 0 ? 0.35355339059f : 0.5f) * std::cos((2 * x + 1) * u * 3.14159265358979323846 / 16.0);
        init = true;
    }
    float tmp[64];
    for (int y = 0; y < 8; ++y)          // rows
        for (int x = 0; x < 8; ++x) {
            float s = 0.f;
            for (int u = 0; u < 8; ++u) s += c[x][u] * in[y * 8 + u];
            tmp[y * 8 + x] = s;
        }
    for (int x = 0; x < 8; ++x)          // columns
        for (int y = 0; y < 8; ++y) {
            float s = 0.f;
            for (int v = 0; v < 8; ++v) s += c[y][v] * tmp[v * 8 + x];
            const int val = static_cast<int>(std::lround(s + 128.f));
            out[y * out_stride + x] = static_cast<uint8_t>(val < 0 ? 0 : (val > 255 ? 255 : val));
        }
}

struct JpegComp {
    int id = 0, h = 1, v = 1, tq = 0, td = 0, ta = 0, pred = 0;
    int bw = 0, bh = 0;                  // plane size in pixels (multiple of 8 * sampling)
    int blocks_w = 0, blocks_h = 0;      // coefficient storage in blocks (padded to whole MCUs)
    int own_bw = 0, own_bh = 0;          // blocks a non-interleaved scan of this component visits
    std::vector<int16_t> coef;           // [blocks_h][blocks_w][64] in natural (row-major) order, not dequantised
    std::vector<uint8_t> plane;
};

// One scan of a progressive frame for one block: spectral band [ss, se], successive-approximation bits ah/al.
struct JpegScan {
    int ss = 0, se = 63, ah = 0, al = 0;
    int eobrun = 0;
};

void jpeg_refine_nonzero(JpegBits& br, int16_t* c, int p1, int m1) {
    if (br.get_bit() && (*c & p1) == 0) *c = static_cast<int16_t>(*c >= 0 ? *c + p1 : *c + m1);
}

void jpeg_decode_block(JpegBits& br, JpegComp& c, const JpegHuff* dc, const JpegHuff* ac, JpegScan& sc, int16_t* blk,
                       bool progressive) {
    const auto corrupt = [] { return std::invalid_argument("The JPEG entropy-coded data is corrupt."); };
    if (!progressive) {
        const int t = jpeg_decode_symbol(br, dc[c.td]);
        if (t > 11) throw corrupt();
        c.pred += jpeg_extend(br.get_bits(t), t);
        blk[0] = static_cast<int16_t>(c.pred);
        for (int k = 1; k < 64;) {
            const int rs = jpeg_decode_symbol(br, ac[c.ta]);
            const int r = rs >> 4, sz = rs & 15;
            if (sz == 0) {
                if (r == 15) { k += 16; continue; }
                break;
            }
            k += r;
            if (k > 63) throw corrupt();
            blk[kZigzag[k]] = static_cast<int16_t>(jpeg_extend(br.get_bits(sz), sz));
            ++k;
        }
        return;
    }
    if (sc.ss == 0) {                                               // DC scan
        if (sc.ah == 0) {
            const int t = jpeg_decode_symbol(br, dc[c.td]);
            if (t > 11) throw corrupt();
            c.pred += jpeg_extend(br.get_bits(t), t);
            blk[0] = static_cast<int16_t>(c.pred * (1 << sc.al));
        } else if (br.get_bit()) {
            blk[0] = static_cast<int16_t>(blk[0] | (1 << sc.al));
        }
        return;
    }
    if (sc.ah == 0) {                                               // AC band, first pass
        if (sc.eobrun > 0) {
            --sc.eobrun;
            return;
        }
        for (int k = sc.ss; k <= sc.se;) {
            const int rs = jpeg_decode_symbol(br, ac[c.ta]);
            const int r = rs >> 4, sz = rs & 15;
            if (sz == 0) {
                if (r < 15) {
                    sc.eobrun = (1 << r) - 1;
                    if (r) sc.eobrun += br.get_bits(r);
                    break;
                }
                k += 16;
                continue;
            }
            k += r;
            if (k > sc.se) throw corrupt();
            blk[kZigzag[k]] = static_cast<int16_t>(jpeg_extend(br.get_bits(sz), sz) * (1 << sc.al));
            ++k;
        }
        return;
    }
    // AC band, refinement pass: every coefficient that is already non-zero reads one correction bit; new
    // coefficients (magnitude 1 << al) are placed after `r` still-zero positions
    const int p1 = 1 << sc.al, m1 = -(1 << sc.al);
    int k = sc.ss;
    if (sc.eobrun == 0) {
        for (; k <= sc.se; ++k) {
            const int rs = jpeg_decode_symbol(br, ac[c.ta]);
            int r = rs >> 4, value = 0;
            const int sz = rs & 15;
            if (sz) {
                if (sz != 1) throw corrupt();
                value = br.get_bit() ? p1 : m1;
            } else if (r != 15) {
                sc.eobrun = 1 << r;
                if (r) sc.eobrun += br.get_bits(r);
                break;
            }
            do {
                int16_t* cf = blk + kZigzag[k];
                if (*cf != 0) {
                    jpeg_refine_nonzero(br, cf, p1, m1);
                } else if (--r < 0) {
                    break;
                }
                ++k;
            } while (k <= sc.se);
            if (value) {
                if (k > sc.se) throw corrupt();
                blk[kZigzag[k]] = static_cast<int16_t>(value);
            }
        }
    }
    if (sc.eobrun > 0) {
        for (; k <= sc.se; ++k) {
            int16_t* cf = blk + kZigzag[k];
            if (*cf != 0) jpeg_refine_nonzero(br, cf, p1, m1);
        }
        --sc.eobrun;
    }
}

at::Tensor decode_jpeg(const uint8_t* b, size_t n) {
    auto be16 = [&](size_t p) { return (static_cast<int>(b[p]) << 8) | b[p + 1]; };
    float qt[4][64] = {};
    bool qt_present[4] = {false, false, false, false};
    JpegHuff dc[4], ac[4];
    std::vector<JpegComp> comps;
    int width = 0, height = 0, restart = 0, hmax = 1, vmax = 1;
    int mcus_x = 0, mcus_y = 0;
    size_t p = 2;
    bool got_frame = false, progressive = false, got_scan = false;
    bool saw_jfif = false, saw_adobe = false;
    int adobe_transform = 0;
    while (p + 4 <= n) {
        if (b[p] != 0xFF) throw std::invalid_argument("The JPEG marker stream is corrupt.");
        while (p < n && b[p] == 0xFF) ++p;
        const uint8_t m = b[p++];
        if (m == 0xD8 || (m >= 0xD0 && m <= 0xD7) || m == 0x01) continue;
        if (m == 0xD9) break;
        if (p + 2 > n) break;
        const size_t len = static_cast<size_t>(be16(p));
        if (len < 2 || p + len > n) throw std::invalid_argument("The JPEG file is truncated.");
        const size_t seg = p + 2, seg_end = p + len;
        if (m == 0xE0 && len >= 7 && std::memcmp(b + seg, "JFIF\0", 5) == 0) {
            saw_jfif = true;
        } else if (m == 0xEE && len >= 14 && std::memcmp(b + seg, "Adobe", 5) == 0) {
            saw_adobe = true;
            adobe_transform = b[seg + 11];                           // 0: as stored, 1: YCbCr, 2: YCCK
        } else if (m == 0xDB) {                                     // DQT
            size_t q = seg;
            while (q < seg_end) {
                const int pq = b[q] >> 4, tq = b[q] & 15;
                ++q;
                if (tq > 3) throw std::invalid_argument("The JPEG quantization table index is invalid.");
                for (int i = 0; i < 64; ++i) {
                    qt[tq][kZigzag[i]] = pq ? static_cast<float>(be16(q)) : static_cast<float>(b[q]);
                    q += pq ? 2 : 1;
                }
                qt_present[tq] = true;
            }
        } else if (m == 0xC4) {                                     // DHT
            size_t q = seg;
            while (q < seg_end) {
                const int tc = b[q] >> 4, th = b[q] & 15;
                ++q;
                if (th > 3 || tc > 1) throw std::invalid_argument("The JPEG Huffman table index is invalid.");
                JpegHuff& h = tc ? ac[th] : dc[th];
                int total = 0;
                for (int l = 1; l <= 16; ++l) {
                    h.bits[l] = b[q++];
                    total += h.bits[l];
                }
                if (total > 256 || q + total > seg_end) throw std::invalid_argument("The JPEG Huffman table is corrupt.");
                for (int i = 0; i < total; ++i) h.vals[i] = b[q++];
                h.build();
            }
        } else if (m == 0xC0 || m == 0xC1 || m == 0xC2) {           // SOF0 / SOF1 (sequential), SOF2 (progressive)
            if (got_frame) throw std::invalid_argument("The JPEG file has more than one frame header.");
            if (b[seg] != 8) throw std::invalid_argument("Only 8-bit JPEG files are supported.");
            progressive = m == 0xC2;
            height = be16(seg + 1);
            width = be16(seg + 3);
            const int nc = b[seg + 5];
            if ((nc != 1 && nc != 3 && nc != 4) || width <= 0 || height <= 0 ||
                seg + 6 + 3 * static_cast<size_t>(nc) > seg_end)
                throw std::invalid_argument("Only JPEG files with one, three or four components are supported.");
            comps.resize(nc);
            for (int i = 0; i < nc; ++i) {
                comps[i].id = b[seg + 6 + 3 * i];
                comps[i].h = b[seg + 7 + 3 * i] >> 4;
                comps[i].v = b[seg + 7 + 3 * i] & 15;
                comps[i].tq = b[seg + 8 + 3 * i];
                if (comps[i].h < 1 || comps[i].h > 2 || comps[i].v < 1 || comps[i].v > 2 || comps[i].tq > 3)
                    throw std::invalid_argument("The JPEG sampling factors are not supported.");
                hmax = std::max(hmax, comps[i].h);
                vmax = std::max(vmax, comps[i].v);
            }
            if (nc == 1) comps[0].h = comps[0].v = hmax = vmax = 1;  // a single component is never interleaved
            mcus_x = (width + 8 * hmax - 1) / (8 * hmax);
            mcus_y = (height + 8 * vmax - 1) / (8 * vmax);
            for (auto& c : comps) {
                c.blocks_w = mcus_x * c.h;
                c.blocks_h = mcus_y * c.v;
                c.bw = c.blocks_w * 8;
                c.bh = c.blocks_h * 8;
                c.own_bw = ((width * c.h + hmax - 1) / hmax + 7) / 8;
                c.own_bh = ((height * c.v + vmax - 1) / vmax + 7) / 8;
                c.coef.assign(static_cast<size_t>(c.blocks_w) * c.blocks_h * 64, 0);
            }
            got_frame = true;
        } else if (m >= 0xC3 && m <= 0xCF && m != 0xC8 && m != 0xCC) {
            throw std::invalid_argument("Lossless, hierarchical and arithmetic-coded JPEG files are not supported.");
        } else if (m == 0xDD) {                                     // DRI
            restart = be16(seg);
        } else if (m == 0xDA) {                                     // SOS: an entropy-coded scan follows
            if (!got_frame) throw std::invalid_argument("The JPEG file has no frame header before its scan.");
            const int ns = b[seg];
            if (ns < 1 || ns > static_cast<int>(comps.size()) || seg + 1 + 2 * static_cast<size_t>(ns) + 3 > seg_end)
                throw std::invalid_argument("The JPEG scan header is corrupt.");
            std::vector<JpegComp*> in_scan;
            for (int i = 0; i < ns; ++i) {
                const int cid = b[seg + 1 + 2 * i];
                JpegComp* found = nullptr;
                for (auto& c : comps)
                    if (c.id == cid) found = &c;
                if (found == nullptr) throw std::invalid_argument("The JPEG scan names an unknown component.");
                found->td = b[seg + 2 + 2 * i] >> 4;
                found->ta = b[seg + 2 + 2 * i] & 15;
                if (found->td > 3 || found->ta > 3) throw std::invalid_argument("The JPEG Huffman table index is invalid.");
                in_scan.push_back(found);
            }
            JpegScan sc;
            sc.ss = b[seg + 1 + 2 * ns];
            sc.se = b[seg + 2 + 2 * ns];
            sc.ah = b[seg + 3 + 2 * ns] >> 4;
            sc.al = b[seg + 3 + 2 * ns] & 15;
            if (!progressive) {
                sc = JpegScan{};
            } else if (sc.ss > sc.se || sc.se > 63 || sc.al > 13 || (sc.ss == 0 && sc.se != 0) ||
                       (sc.ss > 0 && ns != 1)) {
                throw std::invalid_argument("The JPEG progressive scan parameters are invalid.");
            }
            for (JpegComp* c : in_scan) {
                const bool need_dc = !progressive || (sc.ss == 0 && sc.ah == 0);
                const bool need_ac = !progressive || sc.ss > 0;
                if (!qt_present[c->tq] || (need_dc && !dc[c->td].present) || (need_ac && !ac[c->ta].present))
                    throw std::invalid_argument("The JPEG scan refers to a table that was not defined.");
                c->pred = 0;
            }
            JpegBits br{b + seg_end, b + n};
            int until_restart = restart;
            const auto maybe_restart = [&] {
                if (restart && until_restart == 0) {
                    br.reset();
                    while (br.p + 1 < br.end && !(br.p[0] == 0xFF && br.p[1] >= 0xD0 && br.p[1] <= 0xD7)) ++br.p;
                    br.p += 2;
                    for (JpegComp* c : in_scan) c->pred = 0;
                    sc.eobrun = 0;
                    until_restart = restart;
                }
            };
            if (ns == 1) {
                // non-interleaved: the component's own blocks in raster order, one block per "MCU"
                JpegComp& c = *in_scan[0];
                for (int by = 0; by < c.own_bh; ++by)
                    for (int bx = 0; bx < c.own_bw; ++bx) {
                        maybe_restart();
                        jpeg_decode_block(br, c, dc, ac, sc,
                                          c.coef.data() + (static_cast<size_t>(by) * c.blocks_w + bx) * 64, progressive);
                        if (restart) --until_restart;
                    }
            } else {
                for (int my = 0; my < mcus_y; ++my)
                    for (int mx = 0; mx < mcus_x; ++mx) {
                        maybe_restart();
                        for (JpegComp* c : in_scan)
                            for (int by = 0; by < c->v; ++by)
                                for (int bx = 0; bx < c->h; ++bx)
                                    jpeg_decode_block(br, *c, dc, ac, sc,
                                                      c->coef.data() + (static_cast<size_t>(my * c->v + by) * c->blocks_w +
                                                                        mx * c->h + bx) * 64,
                                                      progressive);
                        if (restart) --until_restart;
                    }
            }
            got_scan = true;
            // the next marker sits after the entropy-coded bytes: skip stuffed 0xFF00 pairs and restart markers
            size_t q = static_cast<size_t>(br.p - b);
            if (q > seg_end && br.cnt == 0 && b[q - 1] == 0xFF) --q;   // the reader stopped on a marker's 0xFF
            while (q + 1 < n && !(b[q] == 0xFF && b[q + 1] != 0 && !(b[q + 1] >= 0xD0 && b[q + 1] <= 0xD7))) ++q;
            p = q;
            continue;
        }
        p = seg_end;
    }
    if (!got_frame || !got_scan) throw std::invalid_argument("The JPEG file has no image scan.");
    {
        {
            // dequantisation and inverse DCT of every block
            for (auto& c : comps) {
                c.plane.assign(static_cast<size_t>(c.bw) * c.bh, 0);
                for (int by = 0; by < c.blocks_h; ++by)
                    for (int bx = 0; bx < c.blocks_w; ++bx) {
                        const int16_t* src = c.coef.data() + (static_cast<size_t>(by) * c.blocks_w + bx) * 64;
                        float blk[64];
                        for (int i = 0; i < 64; ++i) blk[i] = static_cast<float>(src[i]) * qt[c.tq][i];
                        jpeg_idct8x8(blk, c.plane.data() + static_cast<size_t>(by) * 8 * c.bw + bx * 8, c.bw);
                    }
            }
            // chroma upsampling with the triangle filter ("3/4 near + 1/4 far", separable) on the valid part of each
            // plane, then colour conversion
            const int nc = static_cast<int>(comps.size());
            at::Tensor out = at::empty({height, width, nc}, at::kByte);
            uint8_t* o = out.data_ptr<uint8_t>();
            std::vector<std::vector<uint8_t>> full(nc);
            for (int ci = 0; ci < nc; ++ci) {
                const JpegComp& c = comps[ci];
                const int fx = hmax / c.h, fy = vmax / c.v;
                const int cw = (width * c.h + hmax - 1) / hmax, ch = (height * c.v + vmax - 1) / vmax;
                std::vector<uint8_t>& f = full[ci];
                f.resize(static_cast<size_t>(width) * height);
                auto at_ = [&](int x, int y) {
                    x = x < 0 ? 0 : (x >= cw ? cw - 1 : x);
                    y = y < 0 ? 0 : (y >= ch ? ch - 1 : y);
                    return static_cast<int>(c.plane[static_cast<size_t>(y) * c.bw + x]);
                };
                for (int y = 0; y < height; ++y)
                    for (int x = 0; x < width; ++x) {
                        int val;
                        if (fx == 1 && fy == 1) {
                            val = at_(x, y);
                        } else if (fx == 2 && fy == 1) {
                            const int i = x >> 1;
                            val = (x & 1) ? (3 * at_(i, y) + at_(i + 1, y) + 2) >> 2 : (3 * at_(i, y) + at_(i - 1, y) + 1) >> 2;
                        } else if (fx == 1 && fy == 2) {
                            const int j = y >> 1;
                            val = (y & 1) ? (3 * at_(x, j) + at_(x, j + 1) + 2) >> 2 : (3 * at_(x, j) + at_(x, j - 1) + 1) >> 2;
                        } else {
                            const int i = x >> 1, j = y >> 1, jf = (y & 1) ? j + 1 : j - 1;
                            auto colsum = [&](int xi) { return 3 * at_(xi, j) + at_(xi, jf); };
                            val = (x & 1) ? (3 * colsum(i) + colsum(i + 1) + 7) >> 4 : (3 * colsum(i) + colsum(i - 1) + 8) >> 4;
                        }
                        f[static_cast<size_t>(y) * width + x] = static_cast<uint8_t>(val);
                    }
            }
            auto sample = [&](int ci, int x, int y) { return static_cast<int>(full[ci][static_cast<size_t>(y) * width + x]); };
            auto clamp8 = [](float v) { const int i = static_cast<int>(std::lround(v)); return static_cast<uint8_t>(i < 0 ? 0 : (i > 255 ? 255 : i)); };
            // What the stored components mean (the rules of the JFIF / Adobe conventions): three components are
            // YCbCr unless an Adobe marker says "no transform" or, without any marker, the component ids spell
            // "RGB"; four components are CMYK as stored unless the Adobe marker says YCCK. Output: gray, RGB, or
            // CMYK with the file's polarity (Adobe files store inverted ink values; they are passed on unchanged).
            bool ycc = false;
            if (nc == 3) {
                if (saw_jfif) ycc = true;
                else if (saw_adobe) ycc = adobe_transform != 0;
                else ycc = !(comps[0].id == 'R' && comps[1].id == 'G' && comps[2].id == 'B');
            } else if (nc == 4) {
                ycc = saw_adobe && adobe_transform == 2;
            }
            for (int y = 0; y < height; ++y)
                for (int x = 0; x < width; ++x) {
                    uint8_t* px = o + (static_cast<size_t>(y) * width + x) * nc;
                    if (nc == 1) {
                        px[0] = static_cast<uint8_t>(sample(0, x, y));
                        continue;
                    }
                    if (!ycc) {
                        for (int ci = 0; ci < nc; ++ci) px[ci] = static_cast<uint8_t>(sample(ci, x, y));
                        continue;
                    }
                    const float Y = static_cast<float>(sample(0, x, y));
                    const float cb = static_cast<float>(sample(1, x, y)) - 128.f;
                    const float cr = static_cast<float>(sample(2, x, y)) - 128.f;
                    const uint8_t r = clamp8(Y + 1.402f * cr);
                    const uint8_t g = clamp8(Y - 0.344136f * cb - 0.714136f * cr);
                    const uint8_t bl = clamp8(Y + 1.772f * cb);
                    if (nc == 3) {
                        px[0] = r, px[1] = g, px[2] = bl;
                    } else {   // YCCK -> CMYK: the first three planes are the YCbCr form of (255 - C, 255 - M, 255 - Y)
                        px[0] = static_cast<uint8_t>(255 - r), px[1] = static_cast<uint8_t>(255 - g);
                        px[2] = static_cast<uint8_t>(255 - bl), px[3] = static_cast<uint8_t>(sample(3, x, y));
                    }
                }
            return out;
        }
    }
}

}  // namespace

// ================================================================== ImageDecoder
Data ImageDecoder::operator()(Data&& d) const {
    if (!d.is_memory_block()) throw std::invalid_argument("The input data must be of type `MemoryBlock`.");
    const MemoryBlock& mb = d.as_memory_block();
    const uint8_t* b = mb.data();
    const size_t n = mb.size();
    if (n >= 4 && b[0] == 0xFF && b[1] == 0xD8) {
        at::Tensor img = decode_jpeg(b, n);
        if (pin_memory_) img = img.pin_memory();
        const double channels = static_cast<double>(img.size(2));
        DataDict res{{"channels", Data(channels)}, {"height", Data(static_cast<double>(img.size(0)))},
                     {"width", Data(static_cast<double>(img.size(1)))}, {"bit_depth", Data(8.0)},
                     {"format", Data(channels)}};
        if (device_.has_value() && !device_->is_cpu()) img = img.to(*device_, /*non_blocking=*/pin_memory_);
        res.emplace_back("image", Data(img));
        return Data(std::move(res));
    }
    if (!is_png(b, n)) throw std::invalid_argument("The input image is neither a PNG nor a JPEG file.");
    int depth = 0, color = 0;
    at::Tensor out = decode_png(b, n, pin_memory_, depth, color);
    const double channels = static_cast<double>(out.size(2));
    DataDict res{{"bit_depth", Data(static_cast<double>(depth))}, {"color_type", Data(static_cast<double>(color))},
                 {"channels", Data(channels)}, {"height", Data(static_cast<double>(out.size(0)))},
                 {"width", Data(static_cast<double>(out.size(1)))}, {"format", Data(channels)}};
    if (device_.has_value() && !device_->is_cpu()) out = out.to(*device_, /*non_blocking=*/pin_memory_);
    res.emplace_back("image", Data(out));
    return Data(std::move(res));
}

}  // namespace fs2d
