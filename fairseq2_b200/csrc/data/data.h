// Core types of the native data pipeline runtime: the `Data` value that flows
// through pipelines, the `Tape` used to record/replay positions, and the
// `DataSource` pull-iterator interface every source and operator implements.
//
// Behavioural contract follows fairseq2n (data/data.h, data/tape.h,
// data/data_source.h); the implementation is independent.
#pragma once

#include <pybind11/pybind11.h>
#include <torch/extension.h>

#include <atomic>
#include <cstdint>
#include <functional>
#include <memory>
#include <optional>
#include <stdexcept>
#include <string>
#include <utility>
#include <variant>
#include <vector>

namespace fs2d {

namespace py = pybind11;

// ---------------------------------------------------------------- errors
class DataPipelineError : public std::runtime_error {
public:
    explicit DataPipelineError(const std::string& msg, bool recoverable = false)
        : std::runtime_error(msg), recoverable_(recoverable) {}
    bool recoverable() const noexcept { return recoverable_; }

private:
    bool recoverable_;
};

class ByteStreamError : public std::runtime_error {
public:
    using std::runtime_error::runtime_error;
};

class RecordError : public std::runtime_error {
public:
    using std::runtime_error::runtime_error;
};

// ---------------------------------------------------------- memory block
// Reference-counted, read-only byte range (heap buffer or mmap'ed file).
class MemoryBlock {
public:
    MemoryBlock() = default;
    MemoryBlock(std::shared_ptr<const void> owner, const uint8_t* data, size_t size)
        : owner_(std::move(owner)), data_(data), size_(size) {}

    static MemoryBlock copy_of(const void* src, size_t n);
    static MemoryBlock map_file(const std::string& path);
    static MemoryBlock read_file(const std::string& path);

    const uint8_t* data() const noexcept { return data_; }
    size_t size() const noexcept { return size_; }
    bool empty() const noexcept { return size_ == 0; }
    MemoryBlock slice(size_t offset, size_t length) const {
        if (offset > size_ || length > size_ - offset) throw std::out_of_range("MemoryBlock slice out of range");
        return MemoryBlock(owner_, data_ + offset, length);
    }

private:
    std::shared_ptr<const void> owner_;
    const uint8_t* data_ = nullptr;
    size_t size_ = 0;
};

// --------------------------------------------------------------- py object
// Holds an arbitrary Python object; reference counting takes the GIL.
class PyObjectHolder {
public:
    PyObjectHolder() = default;
    explicit PyObjectHolder(py::object o) : obj_(std::make_shared<Guard>(std::move(o))) {}
    py::object get() const { return obj_ ? obj_->o : py::none(); }

private:
    struct Guard {
        explicit Guard(py::object x) : o(std::move(x)) {}
        ~Guard() {
            py::gil_scoped_acquire gil;
            o = py::object();
        }
        py::object o;
    };
    std::shared_ptr<Guard> obj_;
};

// -------------------------------------------------------------------- Data
class Data;
using DataList = std::vector<Data>;
using DataDict = std::vector<std::pair<std::string, Data>>;  // insertion ordered

class Data {
public:
    using Variant = std::variant<std::monostate, bool, int64_t, double, std::string, at::Tensor, MemoryBlock,
                                 std::shared_ptr<DataList>, std::shared_ptr<DataDict>, PyObjectHolder>;

    Data() = default;
    Data(bool v) : v_(v) {}
    Data(int64_t v) : v_(v) {}
    Data(int v) : v_(static_cast<int64_t>(v)) {}
    Data(double v) : v_(v) {}
    Data(std::string v) : v_(std::move(v)) {}
    Data(const char* v) : v_(std::string(v)) {}
    Data(at::Tensor v) : v_(std::move(v)) {}
    Data(MemoryBlock v) : v_(std::move(v)) {}
    Data(DataList v) : v_(std::make_shared<DataList>(std::move(v))) {}
    Data(DataDict v) : v_(std::make_shared<DataDict>(std::move(v))) {}
    Data(PyObjectHolder v) : v_(std::move(v)) {}

    size_t index() const { return v_.index(); }   // which alternative is held: equal for values of one type
    bool is_none() const { return std::holds_alternative<std::monostate>(v_); }
    bool is_bool() const { return std::holds_alternative<bool>(v_); }
    bool is_int() const { return std::holds_alternative<int64_t>(v_); }
    bool is_float() const { return std::holds_alternative<double>(v_); }
    bool is_string() const { return std::holds_alternative<std::string>(v_); }
    bool is_tensor() const { return std::holds_alternative<at::Tensor>(v_); }
    bool is_memory_block() const { return std::holds_alternative<MemoryBlock>(v_); }
    bool is_list() const { return std::holds_alternative<std::shared_ptr<DataList>>(v_); }
    bool is_dict() const { return std::holds_alternative<std::shared_ptr<DataDict>>(v_); }
    bool is_py() const { return std::holds_alternative<PyObjectHolder>(v_); }

    bool as_bool() const { return std::get<bool>(v_); }
    int64_t as_int() const { return std::get<int64_t>(v_); }
    double as_float() const { return std::get<double>(v_); }
    const std::string& as_string() const { return std::get<std::string>(v_); }
    const at::Tensor& as_tensor() const { return std::get<at::Tensor>(v_); }
    const MemoryBlock& as_memory_block() const { return std::get<MemoryBlock>(v_); }
    DataList& as_list() { return *std::get<std::shared_ptr<DataList>>(v_); }
    const DataList& as_list() const { return *std::get<std::shared_ptr<DataList>>(v_); }
    DataDict& as_dict() { return *std::get<std::shared_ptr<DataDict>>(v_); }
    const DataDict& as_dict() const { return *std::get<std::shared_ptr<DataDict>>(v_); }
    const PyObjectHolder& as_py() const { return std::get<PyObjectHolder>(v_); }

    // Lists and dicts are held by shared_ptr: copying a Data is cheap; call
    // `deep_copy` before mutating a value that other holders may observe.
    Data deep_copy() const;

    const Data* find(const std::string& key) const {
        if (!is_dict()) return nullptr;
        for (const auto& kv : as_dict())
            if (kv.first == key) return &kv.second;
        return nullptr;
    }
    Data* find(const std::string& key) {
        if (!is_dict()) return nullptr;
        for (auto& kv : as_dict())
            if (kv.first == key) return &kv.second;
        return nullptr;
    }

    const char* type_name() const;

private:
    Variant v_;
};

// conversions (must hold the GIL)
Data data_from_py(py::handle h);
py::object data_to_py(const Data& d);

// -------------------------------------------------------------------- Tape
// Linear log of Data values. Sources append their state with `record` in a
// fixed order and read it back with `read` in the same order.
class Tape {
public:
    Tape() = default;
    explicit Tape(DataList storage) : storage_(std::move(storage)) {}

    void record(Data d) { storage_.push_back(std::move(d)); }
    void record_int(int64_t v) { record(Data(v)); }
    void record_bool(bool v) { record(Data(v)); }

    Data read() {
        if (pos_ >= storage_.size()) throw std::invalid_argument("The tape is corrupt (read past its end).");
        return storage_[pos_++];
    }
    int64_t read_int() {
        Data d = read();
        if (!d.is_int()) throw std::invalid_argument("The tape is corrupt (expected an integer).");
        return d.as_int();
    }
    bool read_bool() {
        Data d = read();
        if (!d.is_bool()) throw std::invalid_argument("The tape is corrupt (expected a boolean).");
        return d.as_bool();
    }
    void rewind() { pos_ = 0; }
    bool at_end() const { return pos_ == storage_.size(); }
    const DataList& storage() const { return storage_; }

private:
    DataList storage_;
    size_t pos_ = 0;
};

// -------------------------------------------------------------- DataSource
enum class Finitude { Finite = 0, PseudoInfinite = 1, Infinite = 2 };

inline Finitude max_finitude(Finitude a, Finitude b) { return static_cast<int>(a) > static_cast<int>(b) ? a : b; }

class DataSource {
public:
    virtual ~DataSource() = default;
    virtual std::optional<Data> next() = 0;
    virtual void reset(bool reset_rng) = 0;
    virtual void record_position(Tape& t, bool strict) const = 0;
    virtual void reload_position(Tape& t, bool strict) = 0;
    virtual Finitude finitude() const = 0;
};

using DataSourceFactory = std::function<std::unique_ptr<DataSource>()>;

// ------------------------------------------------------------ DataPipeline
// A DataPipeline is a cheap-to-copy handle: copies refer to the same underlying
// source and position (like the Python object they are exposed as).
class DataPipeline {
public:
    DataPipeline() : s_(std::make_shared<State>()) {}
    explicit DataPipeline(DataSourceFactory f) : s_(std::make_shared<State>()) { s_->factory = std::move(f); }

    std::optional<Data> next();
    void reset(bool reset_rng = false);
    void record_position(Tape& t, bool strict = true) const;
    void reload_position(Tape& t, bool strict = true);
    bool is_broken() const noexcept { return s_->broken; }
    Finitude finitude() const;
    void set_max_num_warnings(size_t n) { s_->max_num_warnings = n; }

    // static factories
    static class DataPipelineBuilder constant(Data example, std::optional<std::string> key);
    static class DataPipelineBuilder count(int64_t start, int64_t step, std::optional<std::string> key);
    static class DataPipelineBuilder concat(std::vector<DataPipeline> pipelines);
    static class DataPipelineBuilder round_robin(std::vector<DataPipeline> pipelines, bool stop_at_shortest,
                                                 bool allow_repeats);
    static class DataPipelineBuilder sample(std::vector<DataPipeline> pipelines, std::optional<std::vector<float>> weights,
                                            uint64_t seed, bool allow_repeats);
    static class DataPipelineBuilder zip(std::vector<DataPipeline> pipelines, std::vector<std::string> names,
                                         bool zip_to_shortest, bool flatten, bool disable_parallelism);

    void ensure_initialized() const;

private:
    struct State {
        DataSourceFactory factory;
        std::unique_ptr<DataSource> source;
        bool broken = false;
        size_t max_num_warnings = 0;
        size_t warning_count = 0;
    };
    void check_broken() const {
        if (s_->broken) throw DataPipelineError("The data pipeline is broken by a previous operation and cannot be used.");
    }
    std::shared_ptr<State> s_;
};

// Python callables wrapped for use from worker threads.
using MapFn = std::function<Data(Data&&)>;
using PredicateFn = std::function<bool(const Data&)>;
using YieldFn = std::function<DataPipeline(const Data&)>;
using CostFn = std::function<double(const Data&)>;
using BucketCreationFn = std::function<std::optional<std::pair<DataList, DataList>>(DataList&&)>;

class DataPipelineBuilder {
public:
    explicit DataPipelineBuilder(DataSourceFactory f) : factory_(std::move(f)) {}

    DataPipelineBuilder bucket(size_t bucket_size, bool drop_remainder) &&;
    DataPipelineBuilder bucket_by_length(std::vector<std::pair<size_t, size_t>> bucket_sizes,
                                         std::optional<std::string> selector, size_t min_data_len,
                                         bool skip_below_min, bool skip_above_max, bool drop_remainder) &&;
    DataPipelineBuilder dynamic_bucket(double threshold, CostFn cost_fn, std::optional<BucketCreationFn> creation_fn,
                                       std::optional<size_t> min_num_examples, std::optional<size_t> max_num_examples,
                                       bool drop_remainder) &&;
    DataPipelineBuilder filter(PredicateFn fn) &&;
    DataPipelineBuilder map(std::vector<MapFn> fns, std::optional<std::string> selector, size_t num_parallel_calls,
                            bool deterministic) &&;
    DataPipelineBuilder pack(int64_t num_elements, int64_t max_seq_len, int64_t pad_value, bool truncate,
                             bool drop_remainder, bool pinned_memory) &&;
    DataPipelineBuilder prefetch(size_t num_examples) &&;
    DataPipelineBuilder repeat(std::optional<size_t> num_repeats, bool reset_rng) &&;
    DataPipelineBuilder shard(size_t shard_idx, size_t num_shards, bool allow_uneven) &&;
    DataPipelineBuilder shuffle(size_t window, uint64_t seed) &&;
    DataPipelineBuilder skip(size_t n) &&;
    DataPipelineBuilder take(size_t n) &&;
    DataPipelineBuilder yield_from(YieldFn fn) &&;
    DataPipeline and_return(size_t max_num_warnings = 0) &&;

    DataSourceFactory take_factory() { return std::move(factory_); }

private:
    DataSourceFactory factory_;
};

// free-standing sources
DataPipelineBuilder read_list(DataList items);
DataPipelineBuilder list_files(const std::string& path, std::optional<std::string> pattern);
DataPipelineBuilder read_zipped_records(const std::string& path);
DataPipelineBuilder read_text(const std::string& path, std::optional<std::string> key, const std::string& line_ending,
                              bool ltrim, bool rtrim, bool skip_empty, bool memory_map, size_t block_size,
                              std::optional<std::string> encoding = std::nullopt);
DataPipelineBuilder read_py_iterator(py::object iterator, py::object reset_fn, bool infinite);

// length of an example for bucketing/packing: tensor -> size(0), list -> size, int -> itself
size_t data_length(const Data& d);

}  // namespace fs2d
