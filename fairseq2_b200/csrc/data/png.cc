// PNG decoder of the data pipeline (zlib is the only dependency): every colour type (gray, RGB, palette,
// gray + alpha, RGBA) at every legal bit depth (1, 2, 4, 8, 16), Adam7 interlacing, palette transparency, chunk
// checksums. Samples of fewer than 8 bits are scaled to the full 8-bit range; a palette image comes out as RGB
// (RGBA when it has a transparency chunk); 16-bit samples come out as int16 holding the unsigned bit pattern.
#include <zlib.h>

#include <cstring>

#include "extras.h"

namespace fs2d {

namespace {

uint32_t be32(const uint8_t* p) { return (static_cast<uint32_t>(p[0]) << 24) | (p[1] << 16) | (p[2] << 8) | p[3]; }

struct Pass { uint32_t x0, y0, dx, dy; };
constexpr Pass kAdam7[7] = {{0, 0, 8, 8}, {4, 0, 8, 8}, {0, 4, 4, 8}, {2, 0, 4, 4}, {0, 2, 2, 4}, {1, 0, 2, 2}, {0, 1, 1, 2}};
constexpr Pass kWhole = {0, 0, 1, 1};

void unfilter_row(uint8_t type, uint8_t* row, const uint8_t* up, size_t len, size_t bpp) {
    switch (type) {
        case 0: break;
        case 1:
            for (size_t x = bpp; x < len; ++x) row[x] = static_cast<uint8_t>(row[x] + row[x - bpp]);
            break;
        case 2:
            if (up != nullptr)
                for (size_t x = 0; x < len; ++x) row[x] = static_cast<uint8_t>(row[x] + up[x]);
            break;
        case 3:
            for (size_t x = 0; x < len; ++x) {
                const int a = x >= bpp ? row[x - bpp] : 0, b = up != nullptr ? up[x] : 0;
                row[x] = static_cast<uint8_t>(row[x] + ((a + b) >> 1));
            }
            break;
        case 4:
            for (size_t x = 0; x < len; ++x) {
                const int a = x >= bpp ? row[x - bpp] : 0, b = up != nullptr ? up[x] : 0;
                const int c = (up != nullptr && x >= bpp) ? up[x - bpp] : 0;
                const int p = a + b - c, pa = std::abs(p - a), pb = std::abs(p - b), pc = std::abs(p - c);
                row[x] = static_cast<uint8_t>(row[x] + ((pa <= pb && pa <= pc) ? a : (pb <= pc ? b : c)));
            }
            break;
        default: throw std::invalid_argument("The PNG file uses an unknown filter type.");
    }
}

}  // namespace

bool is_png(const uint8_t* b, size_t n) {
    static const uint8_t sig[8] = {0x89, 'P', 'N', 'G', 0x0D, 0x0A, 0x1A, 0x0A};
    return n >= 8 && std::memcmp(b, sig, 8) == 0;
}

at::Tensor decode_png(const uint8_t* b, size_t n, bool pin_memory, int& bit_depth, int& color_type) {
    if (!is_png(b, n)) throw std::invalid_argument("The input is not a PNG file.");
    size_t p = 8;
    uint32_t width = 0, height = 0;
    int depth = 0, color = -1, interlace = 0;
    bool have_header = false, ended = false;
    std::vector<uint8_t> idat, palette, alpha;
    while (p + 12 <= n) {
        const uint32_t len = be32(b + p);
        const uint8_t* type = b + p + 4;
        const uint8_t* body = b + p + 8;
        if (len > n || p + 12 + len > n) throw std::invalid_argument("The PNG file is truncated.");
        if (static_cast<uint32_t>(crc32(crc32(0L, Z_NULL, 0), type, 4 + len)) != be32(body + len))
            throw std::invalid_argument("A chunk of the PNG file fails its checksum.");
        if (std::memcmp(type, "IHDR", 4) == 0) {
            if (len != 13) throw std::invalid_argument("The PNG header chunk has the wrong size.");
            width = be32(body);
            height = be32(body + 4);
            depth = body[8];
            color = body[9];
            if (body[10] != 0 || body[11] != 0) throw std::invalid_argument("The PNG file uses an unknown compression or filter method.");
            interlace = body[12];
            have_header = true;
        } else if (std::memcmp(type, "PLTE", 4) == 0) {
            palette.assign(body, body + len);
        } else if (std::memcmp(type, "tRNS", 4) == 0) {
            alpha.assign(body, body + len);
        } else if (std::memcmp(type, "IDAT", 4) == 0) {
            idat.insert(idat.end(), body, body + len);
        } else if (std::memcmp(type, "IEND", 4) == 0) {
            ended = true;
            break;
        }
        p += 12 + static_cast<size_t>(len);
    }
    if (!have_header || width == 0 || height == 0) throw std::invalid_argument("The PNG file has no valid IHDR chunk.");
    if (!ended) throw std::invalid_argument("The PNG file is truncated.");
    if (static_cast<uint64_t>(width) * height > (uint64_t{1} << 31)) throw std::invalid_argument("The PNG image is too large.");
    if (interlace != 0 && interlace != 1) throw std::invalid_argument("The PNG file uses an unknown interlace method.");
    int in_channels;
    switch (color) {
        case 0: in_channels = 1; break;
        case 2: in_channels = 3; break;
        case 3: in_channels = 1; break;
        case 4: in_channels = 2; break;
        case 6: in_channels = 4; break;
        default: throw std::invalid_argument("The PNG file has an unknown colour type.");
    }
    const bool depth_ok = (color == 0 && (depth == 1 || depth == 2 || depth == 4 || depth == 8 || depth == 16)) ||
                          (color == 3 && (depth == 1 || depth == 2 || depth == 4 || depth == 8)) ||
                          ((color == 2 || color == 4 || color == 6) && (depth == 8 || depth == 16));
    if (!depth_ok) throw std::invalid_argument("The PNG bit depth does not go with its colour type.");
    if (color == 3 && (palette.empty() || palette.size() % 3 != 0)) throw std::invalid_argument("The PNG file has no valid palette.");
    bit_depth = depth;
    color_type = color;

    const size_t pixel_bits = static_cast<size_t>(in_channels) * static_cast<size_t>(depth);
    const size_t bpp = std::max<size_t>(1, pixel_bits / 8);
    const Pass* passes = interlace ? kAdam7 : &kWhole;
    const int num_passes = interlace ? 7 : 1;
    size_t total = 0;
    for (int k = 0; k < num_passes; ++k) {
        const Pass& ps = passes[k];
        if (width <= ps.x0 || height <= ps.y0) continue;
        const size_t pw = (width - ps.x0 + ps.dx - 1) / ps.dx, ph = (height - ps.y0 + ps.dy - 1) / ps.dy;
        total += ph * (1 + (pw * pixel_bits + 7) / 8);
    }
    std::vector<uint8_t> raw(total);
    {
        z_stream zs;
        std::memset(&zs, 0, sizeof zs);
        if (inflateInit(&zs) != Z_OK) throw std::runtime_error("zlib cannot be initialised.");
        zs.next_in = idat.data();
        zs.avail_in = static_cast<uInt>(idat.size());
        zs.next_out = raw.data();
        zs.avail_out = static_cast<uInt>(raw.size());
        const int rc = inflate(&zs, Z_FINISH);
        const size_t produced = raw.size() - zs.avail_out;
        inflateEnd(&zs);
        // Z_BUF_ERROR with a full output buffer: trailing data after the image, which decoders ignore
        if ((rc != Z_STREAM_END && !(rc == Z_BUF_ERROR && produced == raw.size())) || produced != raw.size())
            throw std::invalid_argument("The PNG image data cannot be inflated.");
    }

    const bool is_palette = color == 3;
    const int out_channels = is_palette ? (alpha.empty() ? 3 : 4) : in_channels;
    const bool wide = depth == 16;
    const auto H = static_cast<int64_t>(height), W = static_cast<int64_t>(width);
    at::Tensor out = at::empty({H, W, out_channels},
                               at::TensorOptions().dtype(wide ? at::kShort : at::kByte).pinned_memory(pin_memory));
    uint8_t* o8 = wide ? nullptr : out.data_ptr<uint8_t>();
    int16_t* o16 = wide ? out.data_ptr<int16_t>() : nullptr;
    const unsigned max_sample = (1u << depth) - 1;
    const size_t palette_size = palette.size() / 3;

    size_t offset = 0;
    for (int k = 0; k < num_passes; ++k) {
        const Pass& ps = passes[k];
        if (width <= ps.x0 || height <= ps.y0) continue;
        const size_t pw = (width - ps.x0 + ps.dx - 1) / ps.dx, ph = (height - ps.y0 + ps.dy - 1) / ps.dy;
        const size_t row_bytes = (pw * pixel_bits + 7) / 8;
        const uint8_t* prev = nullptr;
        for (size_t r = 0; r < ph; ++r) {
            uint8_t* line = raw.data() + offset;
            offset += 1 + row_bytes;
            uint8_t* row = line + 1;
            unfilter_row(line[0], row, prev, row_bytes, bpp);
            prev = row;
            const size_t y = ps.y0 + r * ps.dy;
            if (!interlace && !is_palette && depth == 8) {
                std::memcpy(o8 + y * static_cast<size_t>(W) * out_channels, row, row_bytes);
                continue;
            }
            for (size_t i = 0; i < pw; ++i) {
                const size_t x = ps.x0 + i * ps.dx;
                const size_t dst = (y * static_cast<size_t>(W) + x) * out_channels;
                if (wide) {
                    for (int c = 0; c < in_channels; ++c) {
                        const uint8_t* s = row + (i * in_channels + c) * 2;
                        o16[dst + c] = static_cast<int16_t>(static_cast<uint16_t>((s[0] << 8) | s[1]));
                    }
                } else if (depth == 8) {
                    if (is_palette) {
                        const size_t idx = row[i];
                        if (idx >= palette_size) throw std::invalid_argument("The PNG palette index is out of range.");
                        o8[dst] = palette[3 * idx], o8[dst + 1] = palette[3 * idx + 1], o8[dst + 2] = palette[3 * idx + 2];
                        if (out_channels == 4) o8[dst + 3] = idx < alpha.size() ? alpha[idx] : 255;
                    } else {
                        for (int c = 0; c < in_channels; ++c) o8[dst + c] = row[i * in_channels + c];
                    }
                } else {   // 1, 2 or 4 bits: one channel, packed from the high bits down
                    const size_t bit = i * depth;
                    const unsigned v = (row[bit >> 3] >> (8 - depth - (bit & 7))) & max_sample;
                    if (is_palette) {
                        if (v >= palette_size) throw std::invalid_argument("The PNG palette index is out of range.");
                        o8[dst] = palette[3 * v], o8[dst + 1] = palette[3 * v + 1], o8[dst + 2] = palette[3 * v + 2];
                        if (out_channels == 4) o8[dst + 3] = v < alpha.size() ? alpha[v] : 255;
                    } else {
                        o8[dst] = static_cast<uint8_t>(v * 255 / max_sample);
                    }
                }
            }
        }
    }
    return out;
}

}  // namespace fs2d
