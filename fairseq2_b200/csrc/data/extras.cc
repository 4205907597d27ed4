// Element selectors, collater, file/text/zip sources, file mapper and text
// converters of the native data pipeline runtime.
#include <iconv.h>

#include <cerrno>
#include <dirent.h>
#include <fnmatch.h>
#include <sys/stat.h>
#include <zlib.h>

#include <algorithm>
#include <limits>
#include <cctype>
#include <cstring>
#include <fstream>
#include <list>
#include <map>
#include <mutex>

#include "extras.h"

namespace fs2d {

// ============================================================ element selector
// Path mini-language: "a.b[0]", "[*].audio.data", several paths separated by ','.
namespace {

struct PathStep {
    enum Kind { Key, Index, Wildcard } kind;
    std::string key;
    size_t index = 0;
};

// One element path: keys separated by dots, list positions in brackets after a key or another position
// ("a.b[0]", "[*].c"). No empty keys, no blanks, a dot only between a key or position and a following key.
bool parse_path(const std::string& s, std::vector<PathStep>& out) {
    size_t i = 0;
    if (s.empty()) return false;
    bool need_key = false;              // the previous character was a dot
    while (i < s.size()) {
        if (s[i] == '[') {
            if (need_key) return false;                              // "foo.[0]"
            size_t j = s.find(']', i);
            if (j == std::string::npos) return false;
            std::string inner = s.substr(i + 1, j - i - 1);
            if (inner == "*") {
                out.push_back({PathStep::Wildcard, "", 0});
            } else {
                if (inner.empty() || inner.size() > 18 || !std::all_of(inner.begin(), inner.end(), ::isdigit)) return false;
                out.push_back({PathStep::Index, "", static_cast<size_t>(std::stoull(inner))});
            }
            i = j + 1;
        } else {
            size_t j = i;
            while (j < s.size() && s[j] != '.' && s[j] != '[') {
                if (s[j] == ' ' || s[j] == ']' || s[j] == ',') return false;
                ++j;
            }
            if (j == i) return false;
            out.push_back({PathStep::Key, s.substr(i, j - i), 0});
            i = j;
            need_key = false;
        }
        if (i < s.size() && s[i] == '.') {
            ++i;
            need_key = true;
            if (i >= s.size()) return false;                         // "foo."
        } else if (i < s.size() && s[i] != '[') {
            return false;
        }
    }
    return !need_key;
}

std::vector<std::vector<PathStep>> parse_selector(const std::string& s) {
    auto fail = [&]() {
        throw std::invalid_argument("`selector` must contain one or more well-formatted element paths, but is '" + s +
                                    "' instead.");
    };
    std::vector<std::vector<PathStep>> out;
    size_t start = 0;
    while (true) {
        size_t c = s.find(',', start);
        std::string part = s.substr(start, c == std::string::npos ? std::string::npos : c - start);
        size_t a = part.find_first_not_of(' ');
        size_t b = part.find_last_not_of(' ');
        if (a == std::string::npos) fail();
        std::vector<PathStep> path;
        if (!parse_path(part.substr(a, b - a + 1), path)) fail();
        out.push_back(std::move(path));
        if (c == std::string::npos) break;
        start = c + 1;
    }
    return out;
}

// The path as it reads for one concrete element: wildcards up to `upto` replaced by the positions in `taken`.
std::string concrete_path(const std::vector<PathStep>& path, const std::vector<size_t>& taken) {
    std::string out;
    size_t w = 0;
    for (const PathStep& st : path) {
        if (st.kind == PathStep::Key) {
            if (!out.empty()) out += ".";
            out += st.key;
        } else if (st.kind == PathStep::Index) {
            out += "[" + std::to_string(st.index) + "]";
        } else {
            out += w < taken.size() ? "[" + std::to_string(taken[w]) + "]" : "[*]";
            ++w;
        }
    }
    return out;
}

void visit_path_at(Data& d, const std::vector<PathStep>& path, size_t pos, const std::function<void(Data&)>& fn,
                   std::vector<size_t>& taken) {
    if (pos == path.size()) {
        fn(d);
        return;
    }
    const PathStep& st = path[pos];
    auto missing = [&]() {
        throw std::invalid_argument("The input data does not have an element at path '" + concrete_path(path, taken) +
                                    "'.");
    };
    if (st.kind == PathStep::Key) {
        Data* e = d.find(st.key);
        if (e == nullptr) missing();
        visit_path_at(*e, path, pos + 1, fn, taken);
    } else if (st.kind == PathStep::Index) {
        if (!d.is_list() || st.index >= d.as_list().size()) missing();
        visit_path_at(d.as_list()[st.index], path, pos + 1, fn, taken);
    } else {
        if (!d.is_list()) missing();
        DataList& items = d.as_list();
        for (size_t i = 0; i < items.size(); ++i) {
            taken.push_back(i);
            visit_path_at(items[i], path, pos + 1, fn, taken);
            taken.pop_back();
        }
    }
}

void visit_path(Data& d, const std::vector<PathStep>& path, size_t pos, const std::function<void(Data&)>& fn,
                const std::string&) {
    std::vector<size_t> taken;
    visit_path_at(d, path, pos, fn, taken);
}

}  // namespace

void validate_selector(const std::string& selector) { parse_selector(selector); }

Data apply_selected(Data&& d, const std::optional<std::string>& selector, const MapFn& fn) {
    if (!selector) return fn(std::move(d));
    Data copy = d.deep_copy();  // containers are shared; never mutate the caller's view
    for (const auto& path : parse_selector(*selector))
        visit_path(copy, path, 0, [&](Data& e) { e = fn(std::move(e)); }, *selector);
    return copy;
}

const Data& select_single(const Data& d, const std::optional<std::string>& selector) {
    if (!selector) return d;
    const Data* found = nullptr;
    auto paths = parse_selector(*selector);
    visit_path(const_cast<Data&>(d), paths[0], 0, [&](Data& e) { found = &e; }, *selector);
    if (found == nullptr) throw std::invalid_argument("The input data does not have an element at path '" + *selector + "'.");
    return *found;
}

// ==================================================================== collater
namespace {

Data collate_tensors(const std::vector<at::Tensor>& ts, const std::optional<int64_t>& pad_value, int64_t pad_to_multiple,
                     const std::string& path) {
    if (!pad_value) {
        for (const auto& t : ts)
            if (t.sizes() != ts[0].sizes())
                throw std::invalid_argument("The tensors at path '" + path +
                                            "' in the bucket must all have the same shape when no padding value is set.");
        return Data(at::stack(ts));
    }
    int64_t max_len = 0;
    for (const auto& t : ts) {
        if (t.dim() == 0) throw std::invalid_argument("Zero-dimensional tensors at path '" + path + "' cannot be padded.");
        max_len = std::max<int64_t>(max_len, t.size(0));
    }
    if (pad_to_multiple > 1) max_len = ((max_len + pad_to_multiple - 1) / pad_to_multiple) * pad_to_multiple;
    std::vector<int64_t> shape = ts[0].sizes().vec();
    shape[0] = max_len;
    shape.insert(shape.begin(), static_cast<int64_t>(ts.size()));
    at::Tensor out = at::full(shape, *pad_value, ts[0].options());
    std::vector<int64_t> lens;
    bool ragged = false;
    for (size_t i = 0; i < ts.size(); ++i) {
        const int64_t n = ts[i].size(0);
        lens.push_back(n);
        if (n != max_len) ragged = true;
        out[static_cast<int64_t>(i)].narrow(0, 0, n).copy_(ts[i]);
    }
    DataList lens_l;
    lens_l.reserve(lens.size());
    for (int64_t n : lens) lens_l.emplace_back(n);
    DataDict d{{"is_ragged", Data(ragged)}, {"seqs", Data(out)}, {"seq_lens", Data(std::move(lens_l))}};
    return Data(std::move(d));
}

}  // namespace

Collater::Collater(std::optional<int64_t> pad_value, int64_t pad_to_multiple, std::vector<CollateOverride> overrides)
    : pad_value_(pad_value), pad_to_multiple_(pad_to_multiple), overrides_(std::move(overrides)) {
    if (pad_to_multiple_ > 1 && !pad_value_)
        throw std::invalid_argument("`pad_value` must be set when `pad_to_multiple` is greater than 1.");
    for (const auto& ov : overrides_)
        if (ov.pad_to_multiple > 1 && !ov.pad_value)
            throw std::invalid_argument("`pad_value` of the selector '" + ov.selector +
                                        "' must be set when `pad_to_multiple` is greater than 1.");
}

namespace {

const char* collate_type_name(const Data& d) {
    if (d.is_none()) return "none";
    if (d.is_bool()) return "bool";
    if (d.is_int()) return "int";
    if (d.is_float()) return "float";
    if (d.is_string()) return "string";
    if (d.is_tensor()) return "torch.Tensor";
    if (d.is_memory_block()) return "memory_block";
    if (d.is_list()) return "list";
    if (d.is_dict()) return "dict";
    return "pyobj";
}

// "The bucket item 1 ..." at the root, "The element at path 'a[0]' in the bucket item 1 ..." below it.
std::string item_ref(const char* what, const std::string& path, size_t item) {
    if (path.empty()) return "The bucket item " + std::to_string(item);
    return std::string("The ") + what + " at path '" + path + "' in the bucket item " + std::to_string(item);
}

// An override selector matches a path segment by segment; `[*]` stands for any list index.
bool selector_matches(const std::string& selector, const std::string& path) {
    size_t i = 0, j = 0;
    while (i < selector.size() && j < path.size()) {
        if (selector.compare(i, 3, "[*]") == 0 && path[j] == '[') {
            const size_t close = path.find(']', j);
            if (close == std::string::npos) return false;
            i += 3;
            j = close + 1;
        } else if (selector[i] == path[j]) {
            ++i;
            ++j;
        } else {
            return false;
        }
    }
    return i == selector.size() && j == path.size();
}

}  // namespace

Data Collater::operator()(Data&& bucket) const {
    if (!bucket.is_list()) {
        // a single example is a bucket of one
        DataList one;
        one.push_back(std::move(bucket));
        return collate(one, "");
    }
    DataList& items = bucket.as_list();
    if (items.empty()) throw std::invalid_argument("The bucket must contain at least one element, but is empty instead.");
    return collate(items, "");
}

Data Collater::collate(DataList& items, const std::string& path) const {
    const Data& first = items[0];
    for (size_t i = 1; i < items.size(); ++i)
        if (items[i].index() != first.index())
            throw std::invalid_argument(item_ref("element", path, i) + " must be of type `" + collate_type_name(first) +
                                        "`, but is of type `" + collate_type_name(items[i]) + "` instead.");
    if (first.is_dict()) {
        const size_t n = first.as_dict().size();
        for (size_t i = 1; i < items.size(); ++i)
            if (items[i].as_dict().size() != n)
                throw std::invalid_argument(item_ref("`dict`", path, i) + " must have a length of " + std::to_string(n) +
                                            ", but has a length of " + std::to_string(items[i].as_dict().size()) +
                                            " instead.");
        DataDict out;
        for (const auto& kv : first.as_dict()) {
            const std::string sub = path.empty() ? kv.first : path + "." + kv.first;
            DataList column;
            column.reserve(items.size());
            for (size_t i = 0; i < items.size(); ++i) {
                const Data* e = items[i].find(kv.first);
                if (e == nullptr)
                    throw std::invalid_argument("The bucket item " + std::to_string(i) +
                                                " does not have an element at path '" + sub + "'.");
                column.push_back(*e);
            }
            out.emplace_back(kv.first, collate(column, sub));
        }
        return Data(std::move(out));
    }
    if (first.is_list()) {
        const size_t n = first.as_list().size();
        for (size_t i = 1; i < items.size(); ++i)
            if (items[i].as_list().size() != n)
                throw std::invalid_argument(item_ref("`list`", path, i) + " must have a length of " + std::to_string(n) +
                                            ", but has a length of " + std::to_string(items[i].as_list().size()) +
                                            " instead.");
        DataList out;
        for (size_t k = 0; k < n; ++k) {
            DataList column;
            column.reserve(items.size());
            for (auto& it : items) column.push_back(it.as_list()[k]);
            out.push_back(collate(column, path + "[" + std::to_string(k) + "]"));
        }
        return Data(std::move(out));
    }
    if (first.is_tensor()) {
        std::vector<at::Tensor> ts;
        ts.reserve(items.size());
        for (auto& it : items) ts.push_back(it.as_tensor());
        std::optional<int64_t> pad = pad_value_;
        int64_t mult = pad_to_multiple_;
        for (const auto& ov : overrides_)
            if (selector_matches(ov.selector, path)) {
                pad = ov.pad_value;
                mult = ov.pad_to_multiple;
            }
        if (!pad) {
            try {
                return Data(at::stack(ts));
            } catch (const c10::Error& ex) {
                std::throw_with_nested(std::invalid_argument(
                    (path.empty() ? std::string("The tensors in the bucket")
                                  : "The tensors at path '" + path + "' in the bucket") +
                    " cannot be stacked. See nested exception for details."));
            }
        }
        return collate_tensors(ts, pad, mult, path);
    }
    return Data(DataList(items));  // other leaves stay a list
}

// ================================================================= list_files
namespace {

// natural order: digit runs compare numerically
bool natural_less(const std::string& a, const std::string& b) {
    size_t i = 0, j = 0;
    while (i < a.size() && j < b.size()) {
        if (std::isdigit(static_cast<unsigned char>(a[i])) && std::isdigit(static_cast<unsigned char>(b[j]))) {
            size_t ie = i, je = j;
            while (ie < a.size() && std::isdigit(static_cast<unsigned char>(a[ie]))) ++ie;
            while (je < b.size() && std::isdigit(static_cast<unsigned char>(b[je]))) ++je;
            std::string na = a.substr(i, ie - i), nb = b.substr(j, je - j);
            na.erase(0, std::min(na.find_first_not_of('0'), na.size() - 1));
            nb.erase(0, std::min(nb.find_first_not_of('0'), nb.size() - 1));
            if (na.size() != nb.size()) return na.size() < nb.size();
            if (na != nb) return na < nb;
            i = ie;
            j = je;
        } else {
            if (a[i] != b[j]) return a[i] < b[j];
            ++i;
            ++j;
        }
    }
    return a.size() - i < b.size() - j;
}

void walk(const std::string& dir, const std::optional<std::string>& pattern, std::vector<std::string>& out) {
    DIR* d = ::opendir(dir.c_str());
    if (d == nullptr) throw ByteStreamError("The directory '" + dir + "' cannot be opened.");
    std::vector<std::string> names;
    while (dirent* e = ::readdir(d)) {
        std::string n = e->d_name;
        if (n != "." && n != "..") names.push_back(n);
    }
    ::closedir(d);
    std::sort(names.begin(), names.end(), natural_less);
    for (const auto& n : names) {
        std::string full = dir + "/" + n;
        struct stat st {};
        if (::stat(full.c_str(), &st) != 0) continue;
        if (S_ISDIR(st.st_mode)) walk(full, pattern, out);
        else if (S_ISREG(st.st_mode) && (!pattern || ::fnmatch(pattern->c_str(), full.c_str(), 0) == 0))
            out.push_back(full);
    }
}

}  // namespace

DataPipelineBuilder list_files(const std::string& path, std::optional<std::string> pattern) {
    std::vector<std::string> files;
    struct stat st {};
    if (::stat(path.c_str(), &st) != 0) throw ByteStreamError("'" + path + "' does not exist.");
    if (S_ISDIR(st.st_mode)) walk(path, pattern, files);
    else files.push_back(path);
    DataList items;
    for (auto& f : files) items.emplace_back(std::move(f));
    return read_list(std::move(items));
}

// ================================================================== read_text
namespace {

bool is_utf8_name(const std::string& name) {
    std::string e;
    for (char c : name)
        if (c != '-' && c != '_') e += static_cast<char>(std::tolower(static_cast<unsigned char>(c)));
    return e.empty() || e == "utf8" || e == "ascii" || e == "usascii";
}

// Converts a whole text file from `encoding` to UTF-8 with iconv; positions recorded by the reader refer to the
// converted bytes, which are a pure function of the file. An invalid or truncated multi-byte sequence is an error.
MemoryBlock reencode_to_utf8(const MemoryBlock& in, const std::string& encoding, const std::string& path) {
    iconv_t cd = iconv_open("UTF-8", encoding.c_str());
    if (cd == reinterpret_cast<iconv_t>(-1))
        throw std::invalid_argument("The text encoding '" + encoding + "' is not known to iconv.");
    std::vector<char> out(in.size() + in.size() / 2 + 16);
    char* src = const_cast<char*>(reinterpret_cast<const char*>(in.data()));
    size_t src_left = in.size();
    size_t used = 0;
    while (true) {
        char* dst = out.data() + used;
        size_t dst_left = out.size() - used;
        const size_t rc = src_left > 0 ? iconv(cd, &src, &src_left, &dst, &dst_left)
                                       : iconv(cd, nullptr, nullptr, &dst, &dst_left);   // flush the shift state
        used = out.size() - dst_left;
        if (rc != static_cast<size_t>(-1)) {
            if (src_left == 0) {
                char* d2 = out.data() + used;
                size_t l2 = out.size() - used;
                iconv(cd, nullptr, nullptr, &d2, &l2);
                used = out.size() - l2;
                break;
            }
            continue;
        }
        if (errno == E2BIG) {
            out.resize(out.size() * 2);
            continue;
        }
        const size_t at = in.size() - src_left;
        iconv_close(cd);
        throw ByteStreamError("'" + path + "' is not valid " + encoding + " text (byte offset " + std::to_string(at) +
                              (errno == EINVAL ? ", truncated sequence)." : ", invalid sequence)."));
    }
    iconv_close(cd);
    return MemoryBlock::copy_of(out.data(), used);
}

class TextSource final : public DataSource {
public:
    TextSource(std::string path, std::optional<std::string> key, std::string ending, bool ltrim, bool rtrim,
               bool skip_empty, bool memory_map, const std::optional<std::string>& encoding)
        : path_(std::move(path)), key_(std::move(key)), ending_(std::move(ending)), ltrim_(ltrim), rtrim_(rtrim),
          skip_empty_(skip_empty) {
        block_ = memory_map ? MemoryBlock::map_file(path_) : MemoryBlock::read_file(path_);
        if (encoding && !is_utf8_name(*encoding)) block_ = reencode_to_utf8(block_, *encoding, path_);
    }
    std::optional<Data> next() override {
        const char* base = reinterpret_cast<const char*>(block_.data());
        const size_t n = block_.size();
        while (pos_ < n) {
            size_t e = pos_;
            while (e < n && base[e] != '\n') ++e;
            size_t line_end = e;
            if (line_end > pos_ && base[line_end - 1] == '\r' && ending_ != "lf") --line_end;
            size_t a = pos_, b = line_end;
            if (ltrim_) while (a < b && std::isspace(static_cast<unsigned char>(base[a]))) ++a;
            if (rtrim_) while (b > a && std::isspace(static_cast<unsigned char>(base[b - 1]))) --b;
            pos_ = e < n ? e + 1 : n;
            ++line_nr_;
            if (a == b && skip_empty_) continue;
            std::string line(base + a, b - a);
            if (key_) return Data(DataDict{{*key_, Data(std::move(line))}});
            return Data(std::move(line));
        }
        return std::nullopt;
    }
    void reset(bool) override {
        pos_ = 0;
        line_nr_ = 0;
    }
    void record_position(Tape& t, bool) const override {
        t.record_int(static_cast<int64_t>(pos_));
        t.record_int(static_cast<int64_t>(line_nr_));
    }
    void reload_position(Tape& t, bool) override {
        pos_ = static_cast<size_t>(t.read_int());
        line_nr_ = static_cast<size_t>(t.read_int());
    }
    Finitude finitude() const override { return Finitude::Finite; }

private:
    std::string path_;
    std::optional<std::string> key_;
    std::string ending_;
    bool ltrim_, rtrim_, skip_empty_;
    MemoryBlock block_;
    size_t pos_ = 0, line_nr_ = 0;
};

}  // namespace

DataPipelineBuilder read_text(const std::string& path, std::optional<std::string> key, const std::string& line_ending,
                              bool ltrim, bool rtrim, bool skip_empty, bool memory_map, size_t,
                              std::optional<std::string> encoding) {
    if (line_ending != "infer" && line_ending != "lf" && line_ending != "crlf")
        throw std::invalid_argument("`line_ending` must be 'infer', 'lf' or 'crlf'.");
    return DataPipelineBuilder([=]() -> std::unique_ptr<DataSource> {
        return std::make_unique<TextSource>(path, key, line_ending, ltrim, rtrim, skip_empty, memory_map, encoding);
    });
}

// ====================================================== read_zipped_records
// Minimal ZIP reader (central directory, methods 0 = stored and 8 = deflate).
namespace {

uint32_t rd32(const uint8_t* p) { return p[0] | (p[1] << 8) | (p[2] << 16) | (static_cast<uint32_t>(p[3]) << 24); }
uint16_t rd16(const uint8_t* p) { return static_cast<uint16_t>(p[0] | (p[1] << 8)); }

struct ZipEntry {
    std::string name;
    uint32_t method, comp_size, size, local_off;
};

class ZipSource final : public DataSource {
public:
    explicit ZipSource(const std::string& path) : path_(path) {
        block_ = MemoryBlock::map_file(path);
        const uint8_t* b = block_.data();
        const size_t n = block_.size();
        if (n < 22) throw RecordError("'" + path + "' is not a valid zip archive.");
        size_t eocd = std::string::npos;
        for (size_t i = n - 22;; --i) {
            if (rd32(b + i) == 0x06054b50) {
                eocd = i;
                break;
            }
            if (i == 0 || n - i > 65557) break;
        }
        if (eocd == std::string::npos) throw RecordError("'" + path + "' is not a valid zip archive.");
        const uint16_t count = rd16(b + eocd + 10);
        size_t p = rd32(b + eocd + 16);
        for (uint16_t i = 0; i < count; ++i) {
            if (p + 46 > n || rd32(b + p) != 0x02014b50) throw RecordError("'" + path + "' has a corrupt central directory.");
            ZipEntry e;
            e.method = rd16(b + p + 10);
            e.comp_size = rd32(b + p + 20);
            e.size = rd32(b + p + 24);
            const uint16_t nl = rd16(b + p + 28), xl = rd16(b + p + 30), cl = rd16(b + p + 32);
            e.local_off = rd32(b + p + 42);
            e.name.assign(reinterpret_cast<const char*>(b + p + 46), nl);
            p += 46 + nl + xl + cl;
            if (!e.name.empty() && e.name.back() != '/') entries_.push_back(std::move(e));
        }
    }
    std::optional<Data> next() override {
        if (pos_ >= entries_.size()) return std::nullopt;
        const ZipEntry& e = entries_[pos_++];
        const uint8_t* b = block_.data();
        const size_t lo = e.local_off;
        if (lo + 30 > block_.size() || rd32(b + lo) != 0x04034b50)
            throw RecordError("The zip record '" + e.name + "' in '" + path_ + "' is corrupt.");
        const size_t data_off = lo + 30 + rd16(b + lo + 26) + rd16(b + lo + 28);
        if (data_off + e.comp_size > block_.size())
            throw RecordError("The zip record '" + e.name + "' in '" + path_ + "' is truncated.");
        if (e.method == 0) return Data(block_.slice(data_off, e.size));
        if (e.method != 8) throw RecordError("The zip record '" + e.name + "' uses an unsupported compression method.");
        std::vector<uint8_t> out(e.size);
        z_stream zs{};
        if (inflateInit2(&zs, -MAX_WBITS) != Z_OK) throw RecordError("zlib cannot be initialised.");
        zs.next_in = const_cast<Bytef*>(b + data_off);
        zs.avail_in = e.comp_size;
        zs.next_out = out.data();
        zs.avail_out = e.size;
        const int rc = inflate(&zs, Z_FINISH);
        inflateEnd(&zs);
        if (rc != Z_STREAM_END) throw RecordError("The zip record '" + e.name + "' in '" + path_ + "' cannot be inflated.");
        return Data(MemoryBlock::copy_of(out.data(), out.size()));
    }
    void reset(bool) override { pos_ = 0; }
    void record_position(Tape& t, bool) const override { t.record_int(static_cast<int64_t>(pos_)); }
    void reload_position(Tape& t, bool) override { pos_ = static_cast<size_t>(t.read_int()); }
    Finitude finitude() const override { return Finitude::Finite; }

private:
    std::string path_;
    MemoryBlock block_;
    std::vector<ZipEntry> entries_;
    size_t pos_ = 0;
};

}  // namespace

DataPipelineBuilder read_zipped_records(const std::string& path) {
    return DataPipelineBuilder([path]() -> std::unique_ptr<DataSource> { return std::make_unique<ZipSource>(path); });
}

// ================================================================= FileMapper
struct FileMapper::Cache {
    std::mutex m;
    std::list<std::pair<std::string, MemoryBlock>> lru;
    std::map<std::string, std::list<std::pair<std::string, MemoryBlock>>::iterator> index;
};

FileMapper::FileMapper(std::optional<std::string> root_dir, size_t cached_fd_count)
    : root_(std::move(root_dir)), capacity_(cached_fd_count == 0 ? 100 : cached_fd_count),
      cache_(std::make_shared<Cache>()) {}

namespace {

std::string trimmed(const std::string& s) {
    size_t b = 0, e = s.size();
    while (b < e && std::isspace(static_cast<unsigned char>(s[b]))) ++b;
    while (e > b && std::isspace(static_cast<unsigned char>(s[e - 1]))) --e;
    return s.substr(b, e - b);
}

// 1234567 -> "1,234,567"
std::string with_thousands(size_t v) {
    std::string digits = std::to_string(v), out;
    for (size_t i = 0; i < digits.size(); ++i) {
        if (i != 0 && (digits.size() - i) % 3 == 0) out.push_back(',');
        out.push_back(digits[i]);
    }
    return out;
}

// The offset or size specifier of "path:offset:size": decimal digits only, and it has to fit a size_t.
size_t parse_specifier(const char* what, const std::string& spec, const std::string& text) {
    if (text.empty() || !std::all_of(text.begin(), text.end(), [](unsigned char c) { return std::isdigit(c) != 0; }))
        throw std::invalid_argument(std::string("The ") + what + " specifier of '" + spec + "' must be an integer, but is '" +
                                    text + "' instead.");
    size_t v = 0;
    for (const char c : text) {
        const size_t digit = static_cast<size_t>(c - '0');
        if (v > (std::numeric_limits<size_t>::max() - digit) / 10)
            throw std::invalid_argument(std::string("The ") + what + " specifier of '" + spec +
                                        "' must be a machine-representable integer, but is '" + text +
                                        "' instead, which is out of range.");
        v = v * 10 + digit;
    }
    return v;
}

}  // namespace

Data FileMapper::operator()(Data&& d) const {
    if (!d.is_string()) {
        const char* tn = d.is_none() ? "pyobj" : collate_type_name(d);
        throw std::invalid_argument(std::string("The input data must be of type `string`, but is of type `") + tn + "` instead.");
    }
    std::string spec = d.as_string();
    // "path[:offset[:size]]": one to three fields between colons, none of them blank
    std::vector<std::string> fields;
    for (size_t pos = 0;;) {
        const size_t c = spec.find(':', pos);
        fields.push_back(trimmed(spec.substr(pos, c == std::string::npos ? std::string::npos : c - pos)));
        if (c == std::string::npos) break;
        pos = c + 1;
    }
    if (fields.size() > 3 || std::any_of(fields.begin(), fields.end(), [](const std::string& f) { return f.empty(); }))
        throw std::invalid_argument("The input string must be a pathname with optional offset and size specifiers, but is '" +
                                    spec + "' instead.");
    const std::string& path = fields[0];
    std::optional<size_t> off, len;
    if (fields.size() >= 2) off = parse_specifier("offset", spec, fields[1]);
    if (fields.size() == 3) len = parse_specifier("size", spec, fields[2]);
    std::string full = (root_ && !path.empty() && path[0] != '/') ? *root_ + "/" + path : path;
    MemoryBlock block;
    {
        std::lock_guard<std::mutex> lk(cache_->m);
        auto it = cache_->index.find(full);
        if (it != cache_->index.end()) {
            cache_->lru.splice(cache_->lru.begin(), cache_->lru, it->second);
            block = it->second->second;
        }
    }
    if (block.data() == nullptr && block.size() == 0) {
        block = MemoryBlock::map_file(full);
        std::lock_guard<std::mutex> lk(cache_->m);
        cache_->lru.emplace_front(full, block);
        cache_->index[full] = cache_->lru.begin();
        while (cache_->lru.size() > capacity_) {
            cache_->index.erase(cache_->lru.back().first);
            cache_->lru.pop_back();
        }
    }
    if (off) {
        if (*off > block.size())
            throw std::invalid_argument("The specified offset within '" + spec + "' must be less than or equal to the file size (" +
                                        with_thousands(block.size()) + " bytes), but is " + with_thousands(*off) + " instead.");
        const size_t l = len ? *len : block.size() - *off;
        if (l > block.size() - *off)
            throw std::invalid_argument("The end of the specified region within '" + spec +
                                        "' must be less than or equal to the file size (" + with_thousands(block.size()) +
                                        " bytes), but is " + with_thousands(*off + l) + " instead.");
        block = block.slice(*off, l);
    }
    DataDict out{{"path", Data(spec)}, {"data", Data(block)}};
    return Data(std::move(out));
}

// ============================================================= text converters
namespace {

[[noreturn]] void refuse_non_string(const Data& d) {
    const char* tn = d.is_none() ? "pyobj" : collate_type_name(d);
    throw std::invalid_argument(std::string("The input data must be of type `string`, but is of type `") + tn + "` instead.");
}

struct IntegralType {
    const char* name;
    int64_t lo, hi;
};

IntegralType integral_type(at::ScalarType t) {
    switch (t) {
        case at::kByte: return {"torch.uint8", 0, 255};
        case at::kChar: return {"torch.int8", -128, 127};
        case at::kShort: return {"torch.int16", -32768, 32767};
        case at::kInt: return {"torch.int32", std::numeric_limits<int32_t>::min(), std::numeric_limits<int32_t>::max()};
        default: return {"torch.int64", std::numeric_limits<int64_t>::min(), std::numeric_limits<int64_t>::max()};
    }
}

}  // namespace

StrSplitter::StrSplitter(char sep, std::optional<std::vector<std::string>> names, std::vector<size_t> indices,
                         bool exclude, bool single_index)
    : sep_(sep), names_(std::move(names)), indices_(std::move(indices)), exclude_(exclude),
      single_index_(single_index && !exclude) {
    // with kept (not excluded) indices every kept field gets one name
    if (names_ && !indices_.empty() && !exclude_ && names_->size() != indices_.size())
        throw std::invalid_argument("`names` and `indices` must have the same length, but have the lengths " +
                                    std::to_string(names_->size()) + " and " + std::to_string(indices_.size()) + " instead.");
    std::sort(indices_.begin(), indices_.end());
}

Data StrSplitter::operator()(Data&& d) const {
    if (!d.is_string()) refuse_non_string(d);
    const std::string& s = d.as_string();
    std::vector<std::string> fields;
    size_t start = 0;
    while (true) {
        size_t p = s.find(sep_, start);
        fields.push_back(s.substr(start, p == std::string::npos ? std::string::npos : p - start));
        if (p == std::string::npos) break;
        start = p + 1;
    }
    if (!indices_.empty()) {
        // kept or excluded, the highest index has to exist in the line
        if (indices_.back() >= fields.size())
            throw std::invalid_argument("The input string must have at least " + std::to_string(indices_.back()) +
                                        " field(s), but has " + std::to_string(fields.size()) + " instead.");
        std::vector<std::string> kept;
        if (exclude_) {
            for (size_t i = 0; i < fields.size(); ++i)
                if (!std::binary_search(indices_.begin(), indices_.end(), i)) kept.push_back(fields[i]);
        } else {
            for (size_t i : indices_) kept.push_back(fields[i]);
        }
        fields = std::move(kept);
    }
    if (names_) {
        if (names_->size() != fields.size())
            throw std::invalid_argument("The number of fields must match the number of names (" +
                                        std::to_string(names_->size()) + "), but is " + std::to_string(fields.size()) +
                                        " instead.");
        DataDict out;
        for (size_t i = 0; i < fields.size(); ++i) out.emplace_back((*names_)[i], Data(std::move(fields[i])));
        return Data(std::move(out));
    }
    // one kept index given as an int yields the field itself rather than a list of one
    if (single_index_ && fields.size() == 1) return Data(std::move(fields[0]));
    DataList out;
    for (auto& f : fields) out.emplace_back(std::move(f));
    return Data(std::move(out));
}

Data StrToIntConverter::operator()(Data&& d) const {
    if (!d.is_string()) refuse_non_string(d);
    const std::string& s = d.as_string();
    const std::string head = "The input string must represent a 64-bit integer, but is '" + s + "' instead";
    try {
        size_t idx = 0;
        long long v = std::stoll(s, &idx, base_);
        if (idx != s.size()) throw std::invalid_argument("trailing characters");
        return Data(static_cast<int64_t>(v));
    } catch (const std::out_of_range&) {
        throw std::invalid_argument(head + ", which is out of range.");
    } catch (const std::exception&) {
        throw std::invalid_argument(head + ".");
    }
}

Data StrToTensorConverter::operator()(Data&& d) const {
    if (!d.is_string()) refuse_non_string(d);
    const std::string& s = d.as_string();
    const IntegralType type = integral_type(dtype_);
    const std::string head = std::string("The input string must be a space-separated list representing values of type `") +
                             type.name + "`, but contains an element with value '";
    std::vector<int64_t> vals;
    size_t i = 0;
    while (i < s.size()) {
        while (i < s.size() && std::isspace(static_cast<unsigned char>(s[i]))) ++i;
        if (i >= s.size()) break;
        size_t j = i;
        while (j < s.size() && !std::isspace(static_cast<unsigned char>(s[j]))) ++j;
        const std::string tok = s.substr(i, j - i);
        bool parsed = false, in_range = true;
        long long v = 0;
        try {
            size_t idx = 0;
            v = std::stoll(tok, &idx);
            parsed = idx == tok.size();
        } catch (const std::out_of_range&) {
            parsed = true;
            in_range = false;
        } catch (const std::exception&) {
        }
        if (!parsed) throw std::invalid_argument(head + tok + "' that cannot be parsed as `" + type.name + "`.");
        if (!in_range || v < type.lo || v > type.hi)
            throw std::invalid_argument(head + tok + "' that is out of range for `" + type.name + "`.");
        vals.push_back(v);
        i = j;
    }
    at::Tensor t = at::tensor(vals, at::kLong).to(dtype_);
    if (size_) t = t.view(*size_);                   // a -1 extent is inferred; a mismatch raises torch's shape error
    return Data(t);
}

}  // namespace fs2d
