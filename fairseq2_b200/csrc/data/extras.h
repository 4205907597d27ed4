// Declarations of the pipeline helpers implemented in extras.cc / audio.cc.
#pragma once

#include <mutex>
#include <random>
#include <string_view>

#include "data.h"

namespace fs2d {

// Throws std::invalid_argument unless `selector` is a comma-separated list of well-formed element paths.
void validate_selector(const std::string& selector);
Data apply_selected(Data&& d, const std::optional<std::string>& selector, const MapFn& fn);
const Data& select_single(const Data& d, const std::optional<std::string>& selector);

struct CollateOverride {
    std::string selector;
    std::optional<int64_t> pad_value;
    int64_t pad_to_multiple = 1;
};

// Recursive collation of a bucket (list of examples) into stacked / padded tensors.
class Collater {
public:
    Collater(std::optional<int64_t> pad_value, int64_t pad_to_multiple, std::vector<CollateOverride> overrides);
    Data operator()(Data&& bucket) const;

private:
    Data collate(DataList& items, const std::string& path) const;
    std::optional<int64_t> pad_value_;
    int64_t pad_to_multiple_;
    std::vector<CollateOverride> overrides_;
};

// "path[:offset[:length]]" -> {"path": str, "data": MemoryBlock} with an LRU of mapped files.
class FileMapper {
public:
    FileMapper(std::optional<std::string> root_dir, size_t cached_fd_count);
    Data operator()(Data&& d) const;

private:
    struct Cache;
    std::optional<std::string> root_;
    size_t capacity_;
    std::shared_ptr<Cache> cache_;
};

class StrSplitter {
public:
    StrSplitter(char sep, std::optional<std::vector<std::string>> names, std::vector<size_t> indices, bool exclude, bool single_index = false);
    Data operator()(Data&& d) const;

private:
    char sep_;
    std::optional<std::vector<std::string>> names_;
    std::vector<size_t> indices_;
    bool exclude_;
    bool single_index_;  // `indices` was one int, not a list: the field itself is returned
};

class StrToIntConverter {
public:
    explicit StrToIntConverter(int base) : base_(base) {}
    Data operator()(Data&& d) const;

private:
    int base_;
};

class StrToTensorConverter {
public:
    StrToTensorConverter(std::optional<std::vector<int64_t>> size, at::ScalarType dtype)
        : size_(std::move(size)), dtype_(dtype) {
        if (!at::isIntegralType(dtype, /*includeBool=*/false))
            throw std::invalid_argument("Only integral types are supported.");
    }
    Data operator()(Data&& d) const;

private:
    std::optional<std::vector<int64_t>> size_;
    at::ScalarType dtype_;
};

// flac.cc
bool is_flac(const uint8_t* b, size_t n);
at::Tensor decode_flac(const uint8_t* b, size_t n, int& sample_rate, int& bits_per_sample);

// pcm.cc: WAV / AIFF / AIFF-C / AU with integer, float, mu-law and A-law samples -> [frames, channels]
bool is_pcm_container(const uint8_t* b, size_t n);
at::Tensor decode_pcm_container(const uint8_t* b, size_t n, std::optional<at::ScalarType> dtype, double& rate,
                                std::string& format);

// WAV, AIFF, AU and FLAC decoder -> {"waveform", "sample_rate", "format"}.
class AudioDecoder {
public:
    AudioDecoder(bool keepdim, std::optional<at::ScalarType> dtype) : keepdim_(keepdim), dtype_(dtype) {}
    Data operator()(Data&& d) const;

private:
    bool keepdim_;
    std::optional<at::ScalarType> dtype_;
};

// Kaldi-compatible log-mel filter bank features (povey window, pre-emphasis 0.97, 25 ms / 10 ms frames).
class WaveformToFbankConverter {
public:
    WaveformToFbankConverter(int num_mel_bins, float waveform_scale, bool channel_last, bool standardize,
                             bool keep_waveform, std::optional<at::ScalarType> dtype)
        : num_mel_bins_(num_mel_bins), scale_(waveform_scale), channel_last_(channel_last),
          standardize_(standardize), keep_waveform_(keep_waveform), dtype_(dtype) {}
    Data operator()(Data&& d) const;

private:
    int num_mel_bins_;
    float scale_;
    bool channel_last_, standardize_, keep_waveform_;
    std::optional<at::ScalarType> dtype_;
};

// png.cc: every colour type and bit depth, Adam7 interlacing, palette transparency, chunk checksums
bool is_png(const uint8_t* b, size_t n);
at::Tensor decode_png(const uint8_t* b, size_t n, bool pin_memory, int& bit_depth, int& color_type);

// PNG and JPEG (sequential and progressive) decoder ->
// {"image" [H, W, C], "channels", "height", "width", "bit_depth", "format" (= channels)}; PNG adds "color_type".
class ImageDecoder {
public:
    ImageDecoder() = default;
    ImageDecoder(std::optional<at::Device> device, bool pin_memory) : device_(device), pin_memory_(pin_memory) {}
    Data operator()(Data&& d) const;

private:
    std::optional<at::Device> device_;
    bool pin_memory_ = false;
};

// sentencepiece.cc: a SentencePiece runtime (model reader, normalizer, unigram / BPE / char / word segmentation).
struct SamplingOptions {
    int nbest_size = -1;   // < 0: sample from the whole lattice; > 1: sample among the n best; else the best path
    float alpha = 0.1f;    // unigram: inverse temperature; BPE: merge dropout probability
};

class SentencePieceModel {
public:
    // `control_symbols`: appended as control pieces unless the model holds them; "<sym>@0" is inserted at index 0.
    SentencePieceModel(std::string_view serialized, const std::vector<std::string>& control_symbols);
    static SentencePieceModel from_file(const std::string& path, const std::vector<std::string>& control_symbols);

    size_t size() const;
    int unk_id() const;
    int bos_id() const;   // -1 where the model has no such control piece
    int eos_id() const;
    int pad_id() const;
    int piece_to_id(std::string_view piece) const;   // the unknown id for a piece that is not in the vocabulary
    const std::string& id_to_piece(int id) const;
    bool is_control(int id) const;

    std::string normalize(std::string_view text) const;
    std::vector<int64_t> encode(std::string_view text, const SamplingOptions* sampling = nullptr,
                                std::mt19937_64* rng = nullptr) const;
    std::vector<std::pair<std::string, int>> encode_as_pieces(std::string_view text,
                                                              const SamplingOptions* sampling = nullptr,
                                                              std::mt19937_64* rng = nullptr) const;
    std::vector<std::pair<std::vector<std::pair<std::string, int>>, float>> nbest_encode(std::string_view text,
                                                                                         size_t nbest) const;
    std::string decode(const std::vector<int64_t>& ids) const;
    std::string decode_tokens(const std::vector<std::string>& tokens) const;

private:
    std::string decode_pieces(const std::vector<std::pair<std::string, int>>& pieces) const;
    struct Impl;
    std::shared_ptr<Impl> impl_;
};

// str -> int64 tensor: prefix tokens + pieces (optionally reversed, optionally sampled) + suffix tokens.
class SentencePieceEncoder {
public:
    SentencePieceEncoder(SentencePieceModel model, std::vector<std::string> prefix_tokens,
                         std::vector<std::string> suffix_tokens, bool reverse, bool enable_sampling, int nbest_size,
                         float alpha, std::optional<at::Device> device, bool pin_memory, uint64_t seed);
    at::Tensor encode(std::string_view text) const;
    std::vector<std::string> encode_as_tokens(std::string_view text) const;
    Data operator()(Data&& d) const;

private:
    SentencePieceModel model_;
    std::vector<int64_t> prefix_, suffix_;
    bool reverse_, sampling_;
    SamplingOptions options_;
    std::optional<at::Device> device_;
    bool pin_;
    std::shared_ptr<std::pair<std::mutex, std::mt19937_64>> rng_;
};

class SentencePieceDecoder {
public:
    SentencePieceDecoder(SentencePieceModel model, bool reverse) : model_(std::move(model)), reverse_(reverse) {}
    std::string decode(const at::Tensor& indices) const;
    Data operator()(Data&& d) const;

private:
    SentencePieceModel model_;
    bool reverse_;
};

}  // namespace fs2d
