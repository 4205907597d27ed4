// DataPipeline, its builder and every source/operator.
//
// Semantics follow fairseq2n's data pipeline (native/src/fairseq2n/data/*):
// lazy instantiation, broken-state tracking, recoverable errors up to
// `max_num_warnings`, and position record/reload through a Tape so that a
// pipeline can be checkpointed and resumed mid-epoch.
#include <algorithm>
#include <condition_variable>
#include <deque>
#include <mutex>
#include <numeric>
#include <random>
#include <thread>

#include "extras.h"

namespace fs2d {

// ===================================================================== pipeline
void DataPipeline::ensure_initialized() const {
    if (s_->source == nullptr) {
        if (!s_->factory) return;  // an empty pipeline yields nothing
        try {
            s_->source = s_->factory();
        } catch (const ByteStreamError& ex) {
            s_->broken = true;
            throw DataPipelineError(ex.what());
        } catch (...) {
            s_->broken = true;
            throw;
        }
    }
}

std::optional<Data> DataPipeline::next() {
    check_broken();
    ensure_initialized();
    if (s_->source == nullptr) return std::nullopt;
    while (true) {
        try {
            return s_->source->next();
        } catch (const DataPipelineError& ex) {
            if (ex.recoverable() && s_->warning_count < s_->max_num_warnings) {
                ++s_->warning_count;
                continue;  // skip the faulty example
            }
            // only an error that cannot be recovered from makes every later read fail
            if (!ex.recoverable()) s_->broken = true;
            throw;
        } catch (const ByteStreamError& ex) {
            s_->broken = true;
            throw DataPipelineError(ex.what());
        } catch (const RecordError& ex) {
            s_->broken = true;
            throw DataPipelineError(ex.what());
        } catch (...) {
            s_->broken = true;
            throw;
        }
    }
}

void DataPipeline::reset(bool reset_rng) {
    check_broken();
    if (s_->source == nullptr) return;
    try {
        s_->source->reset(reset_rng);
    } catch (...) {
        s_->broken = true;
        throw;
    }
}

void DataPipeline::record_position(Tape& t, bool strict) const {
    check_broken();
    if (s_->source == nullptr) {
        t.record_bool(false);
        return;
    }
    t.record_bool(true);
    t.record_bool(strict);
    try {
        s_->source->record_position(t, strict);
    } catch (...) {
        s_->broken = true;
        throw;
    }
}

void DataPipeline::reload_position(Tape& t, bool) {
    check_broken();
    const bool initialized = t.read_bool();
    if (!initialized) {
        if (s_->source != nullptr) s_->source->reset(true);
        return;
    }
    const bool strict = t.read_bool();
    ensure_initialized();
    if (s_->source == nullptr) return;
    try {
        s_->source->reload_position(t, strict);
    } catch (...) {
        s_->broken = true;
        throw;
    }
}

Finitude DataPipeline::finitude() const {
    ensure_initialized();
    return s_->source ? s_->source->finitude() : Finitude::Finite;
}

DataPipeline DataPipelineBuilder::and_return(size_t max_num_warnings) && {
    DataPipeline p(std::move(factory_));
    p.set_max_num_warnings(max_num_warnings);
    return p;
}

namespace {

// Small counter-based generator (splitmix64): its whole state is one integer,
// which makes recording it on a tape trivial and exact.
struct Rng {
    using result_type = uint64_t;
    uint64_t state;
    explicit Rng(uint64_t seed) : state(seed) {}
    void seed(uint64_t s) { state = s; }
    static constexpr result_type min() { return 0; }
    static constexpr result_type max() { return UINT64_MAX; }
    result_type operator()() {
        uint64_t z = (state += 0x9E3779B97F4A7C15ull);
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        return z ^ (z >> 31);
    }
    double uniform() { return static_cast<double>((*this)() >> 11) * (1.0 / 9007199254740992.0); }
    size_t below(size_t n) { return static_cast<size_t>((*this)() % n); }
};

// ======================================================================= sources
class ListSource final : public DataSource {
public:
    explicit ListSource(DataList items) : items_(std::move(items)) {}
    std::optional<Data> next() override {
        if (pos_ >= items_.size()) return std::nullopt;
        return items_[pos_++];
    }
    void reset(bool) override { pos_ = 0; }
    void record_position(Tape& t, bool) const override { t.record_int(static_cast<int64_t>(pos_)); }
    void reload_position(Tape& t, bool) override { pos_ = static_cast<size_t>(t.read_int()); }
    Finitude finitude() const override { return Finitude::Finite; }

private:
    DataList items_;
    size_t pos_ = 0;
};

class ConstantSource final : public DataSource {
public:
    ConstantSource(Data ex, std::optional<std::string> key) : ex_(std::move(ex)), key_(std::move(key)) {}
    std::optional<Data> next() override {
        if (key_) return Data(DataDict{{*key_, ex_}});
        return ex_;
    }
    void reset(bool) override {}
    void record_position(Tape&, bool) const override {}
    void reload_position(Tape&, bool) override {}
    Finitude finitude() const override { return Finitude::PseudoInfinite; }

private:
    Data ex_;
    std::optional<std::string> key_;
};

class CountSource final : public DataSource {
public:
    CountSource(int64_t start, int64_t step, std::optional<std::string> key)
        : start_(start), step_(step), cur_(start), key_(std::move(key)) {}
    std::optional<Data> next() override {
        const int64_t v = cur_;
        cur_ += step_;
        if (key_) return Data(DataDict{{*key_, Data(v)}});
        return Data(v);
    }
    void reset(bool) override { cur_ = start_; }
    void record_position(Tape& t, bool) const override { t.record_int(cur_); }
    void reload_position(Tape& t, bool) override { cur_ = t.read_int(); }
    Finitude finitude() const override { return Finitude::PseudoInfinite; }

private:
    int64_t start_, step_, cur_;
    std::optional<std::string> key_;
};

Finitude max_finitude_of(const std::vector<DataPipeline>& ps) {
    Finitude f = Finitude::Finite;
    for (const auto& p : ps) f = max_finitude(f, p.finitude());
    return f;
}

class ConcatSource final : public DataSource {
public:
    explicit ConcatSource(std::vector<DataPipeline> ps) : ps_(std::move(ps)) { fin_ = max_finitude_of(ps_); }
    std::optional<Data> next() override {
        for (auto& p : ps_) {
            auto d = p.next();
            if (d) return d;
        }
        return std::nullopt;
    }
    void reset(bool r) override {
        for (auto& p : ps_) p.reset(r);
    }
    void record_position(Tape& t, bool s) const override {
        for (const auto& p : ps_) p.record_position(t, s);
    }
    void reload_position(Tape& t, bool s) override {
        for (auto& p : ps_) p.reload_position(t, s);
    }
    Finitude finitude() const override { return fin_; }

private:
    std::vector<DataPipeline> ps_;
    Finitude fin_;
};

// One buffered example per pipeline; cycles through them. An exhausted
// pipeline is marked "epoch done" and (if allow_repeats) restarted. Ends when
// all (or, with stop_at_shortest, any) pipelines completed an epoch; the check
// happens only when the cursor is back at pipeline 0.
class RoundRobinSource final : public DataSource {
public:
    RoundRobinSource(std::vector<DataPipeline> ps, bool stop_at_shortest, bool allow_repeats)
        : ps_(std::move(ps)), stop_at_shortest_(stop_at_shortest), allow_repeats_(allow_repeats) {
        fin_ = max_finitude_of(ps_);
        buffer_.resize(ps_.size());
        mark_endless_done();
    }
    std::optional<Data> next() override {
        if (ps_.empty() || eod_) return std::nullopt;
        if (!filled_) {
            for (size_t i = 0; i < ps_.size(); ++i) {
                buffer_[i] = ps_[i].next();
                if (!buffer_[i]) done_[i] = true;  // empty pipeline
            }
            filled_ = true;
        }
        for (size_t tries = 0; tries <= ps_.size(); ++tries) {
            if (idx_ == 0 && finished()) {
                eod_ = true;
                return std::nullopt;
            }
            const size_t i = idx_;
            idx_ = (idx_ + 1) % ps_.size();
            if (!buffer_[i]) continue;  // pipeline that never yields (or is not repeated)
            Data out = *buffer_[i];
            buffer_[i] = ps_[i].next();
            if (!buffer_[i]) {
                done_[i] = true;
                if (allow_repeats_) {
                    ps_[i].reset(false);
                    buffer_[i] = ps_[i].next();
                }
            } else if (ps_[i].finitude() == Finitude::PseudoInfinite) {
                done_[i] = true;
            }
            return out;
        }
        eod_ = true;
        return std::nullopt;
    }
    void reset(bool r) override {
        for (auto& p : ps_) p.reset(r);
        std::fill(buffer_.begin(), buffer_.end(), std::nullopt);
        mark_endless_done();
        idx_ = 0;
        filled_ = false;
        eod_ = false;
    }
    void record_position(Tape& t, bool s) const override {
        t.record_bool(filled_);
        t.record_bool(eod_);
        t.record_int(static_cast<int64_t>(idx_));
        for (size_t i = 0; i < ps_.size(); ++i) {
            t.record_bool(done_[i]);
            t.record_bool(buffer_[i].has_value());
            if (buffer_[i]) t.record(*buffer_[i]);
        }
        for (const auto& p : ps_) p.record_position(t, s);
    }
    void reload_position(Tape& t, bool s) override {
        filled_ = t.read_bool();
        eod_ = t.read_bool();
        idx_ = static_cast<size_t>(t.read_int());
        for (size_t i = 0; i < ps_.size(); ++i) {
            done_[i] = t.read_bool();
            if (t.read_bool()) buffer_[i] = t.read();
            else buffer_[i] = std::nullopt;
        }
        for (auto& p : ps_) p.reload_position(t, s);
    }
    Finitude finitude() const override { return fin_; }

private:
    // A pipeline that never ends by construction (`constant`, `count`) has no epoch to finish: it counts as
    // through once it has been read, so the round ends when the pipelines that do end have all been through once.
    // (A pipeline made endless with `repeat()` keeps the whole round going for ever.)
    void mark_endless_done() { done_.assign(ps_.size(), false); }
    bool finished() const {
        if (stop_at_shortest_) {
            for (size_t i = 0; i < ps_.size(); ++i)
                if (done_[i] && ps_[i].finitude() != Finitude::PseudoInfinite) return true;
            return false;
        }
        return std::all_of(done_.begin(), done_.end(), [](bool b) { return b; });
    }
    std::vector<DataPipeline> ps_;
    bool stop_at_shortest_, allow_repeats_;
    Finitude fin_;
    std::vector<std::optional<Data>> buffer_;
    std::vector<bool> done_;
    size_t idx_ = 0;
    bool filled_ = false, eod_ = false;
};

// Weighted sampling among pipelines with a seeded generator.
class SampleSource final : public DataSource {
public:
    SampleSource(std::vector<DataPipeline> ps, std::vector<float> w, uint64_t seed, bool allow_repeats)
        : ps_(std::move(ps)), weights_(std::move(w)), seed_(seed), allow_repeats_(allow_repeats), gen_(seed) {
        fin_ = max_finitude_of(ps_);
        buffer_.resize(ps_.size());
        mark_endless_done();
        blocked_.assign(ps_.size(), false);
    }
    std::optional<Data> next() override {
        if (ps_.empty() || eod_) return std::nullopt;
        if (!filled_) {
            for (size_t i = 0; i < ps_.size(); ++i) {
                buffer_[i] = ps_[i].next();
                if (!buffer_[i])
                    throw DataPipelineError("The pipeline at index " + std::to_string(i) +
                                            " is empty and cannot be sampled.");
            }
            filled_ = true;
        }
        while (true) {
            if (all_done()) {
                eod_ = true;
                return std::nullopt;
            }
            double total = 0;
            for (size_t i = 0; i < ps_.size(); ++i)
                if (!blocked_[i]) total += weights_[i];
            if (total <= 0) {
                eod_ = true;
                return std::nullopt;
            }
            const double u = gen_.uniform() * total;
            double acc = 0;
            size_t pick = ps_.size();
            for (size_t i = 0; i < ps_.size(); ++i) {
                if (blocked_[i]) continue;
                acc += weights_[i];
                pick = i;
                if (u < acc) break;
            }
            Data out = *buffer_[pick];
            buffer_[pick] = ps_[pick].next();
            if (!buffer_[pick]) {
                done_[pick] = true;
                if (allow_repeats_) {
                    ps_[pick].reset(false);
                    buffer_[pick] = ps_[pick].next();
                } else {
                    blocked_[pick] = true;
                }
            } else if (ps_[pick].finitude() == Finitude::PseudoInfinite) {
                done_[pick] = true;
            }
            return out;
        }
    }
    void reset(bool r) override {
        for (auto& p : ps_) p.reset(r);
        std::fill(buffer_.begin(), buffer_.end(), std::nullopt);
        mark_endless_done();
        std::fill(blocked_.begin(), blocked_.end(), false);
        filled_ = eod_ = false;
        if (r) gen_.seed(seed_);
    }
    void record_position(Tape& t, bool s) const override {
        t.record_bool(filled_);
        t.record_bool(eod_);
        t.record_int(static_cast<int64_t>(gen_.state));
        for (size_t i = 0; i < ps_.size(); ++i) {
            t.record_bool(done_[i]);
            t.record_bool(blocked_[i]);
            t.record_bool(buffer_[i].has_value());
            if (buffer_[i]) t.record(*buffer_[i]);
        }
        for (const auto& p : ps_) p.record_position(t, s);
    }
    void reload_position(Tape& t, bool s) override {
        filled_ = t.read_bool();
        eod_ = t.read_bool();
        gen_.state = static_cast<uint64_t>(t.read_int());
        for (size_t i = 0; i < ps_.size(); ++i) {
            done_[i] = t.read_bool();
            blocked_[i] = t.read_bool();
            if (t.read_bool()) buffer_[i] = t.read();
            else buffer_[i] = std::nullopt;
        }
        for (auto& p : ps_) p.reload_position(t, s);
    }
    Finitude finitude() const override { return fin_; }

private:
    // `constant` / `count` pipelines have no epoch to finish: they count as through once they have been drawn from,
    // so sampling ends when every pipeline has been through once
    void mark_endless_done() { done_.assign(ps_.size(), false); }
    bool all_done() const {
        return std::all_of(done_.begin(), done_.end(), [](bool b) { return b; });
    }
    std::vector<DataPipeline> ps_;
    std::vector<float> weights_;
    uint64_t seed_;
    bool allow_repeats_;
    Rng gen_;
    Finitude fin_;
    std::vector<std::optional<Data>> buffer_;
    std::vector<bool> done_, blocked_;
    bool filled_ = false, eod_ = false;
};

class ZipSource final : public DataSource {
public:
    ZipSource(std::vector<DataPipeline> ps, std::vector<std::string> names, bool to_shortest, bool flatten)
        : ps_(std::move(ps)), names_(std::move(names)), to_shortest_(to_shortest), flatten_(flatten) {
        fin_ = max_finitude_of(ps_);
    }
    std::optional<Data> next() override {
        if (ps_.empty()) return std::nullopt;
        DataList items;
        items.reserve(ps_.size());
        // Pipelines that are endless by construction (`constant`, `count`) ride along: the zip ends with the others.
        bool only_endless = true;
        for (auto& p : ps_)
            if (p.finitude() != Finitude::PseudoInfinite) only_endless = false;
        if (only_endless) throw DataPipelineError("Cannot zip only pseudo-infinite pipelines.");
        std::vector<size_t> ended, going;
        for (size_t i = 0; i < ps_.size(); ++i) {
            auto d = ps_[i].next();
            if (!d) {
                ended.push_back(i);
                items.emplace_back();
            } else {
                if (ps_[i].finitude() != Finitude::PseudoInfinite) going.push_back(i);
                items.push_back(std::move(*d));
            }
        }
        if (!ended.empty()) {
            if (to_shortest_ || going.empty()) return std::nullopt;
            std::string idx;
            for (size_t i : going) idx += (idx.empty() ? "" : ", ") + std::to_string(i);
            throw DataPipelineError("The zipped data pipelines must all have the same number of examples, but the data "
                                    "pipelines at the indices [" + idx + "] have more examples than the others.");
        }
        if (flatten_) {
            if (items[0].is_dict()) {
                DataDict out;
                for (auto& it : items) {
                    if (!it.is_dict())
                        throw DataPipelineError("The zipped data pipelines must all return only dicts or only non-dicts when `flatten` is set.");
                    for (auto& kv : it.as_dict()) {
                        for (const auto& e : out)
                            if (e.first == kv.first)
                                throw DataPipelineError("The zipped data pipelines must all return unique keys when `flatten` is set, but the key '" + kv.first + "' is not unique.");
                        out.push_back(kv);
                    }
                }
                return Data(std::move(out));
            }
            DataList out;
            for (auto& it : items) {
                if (it.is_dict())
                    throw DataPipelineError("The zipped data pipelines must all return only dicts or only non-dicts when `flatten` is set.");
                if (it.is_list())
                    for (auto& e : it.as_list()) out.push_back(e);
                else
                    out.push_back(it);
            }
            return Data(std::move(out));
        }
        if (!names_.empty()) {
            DataDict out;
            for (size_t i = 0; i < items.size(); ++i) out.emplace_back(names_[i], std::move(items[i]));
            return Data(std::move(out));
        }
        return Data(std::move(items));
    }
    void reset(bool r) override {
        for (auto& p : ps_) p.reset(r);
    }
    void record_position(Tape& t, bool s) const override {
        for (const auto& p : ps_) p.record_position(t, s);
    }
    void reload_position(Tape& t, bool s) override {
        for (auto& p : ps_) p.reload_position(t, s);
    }
    Finitude finitude() const override { return fin_; }

private:
    std::vector<DataPipeline> ps_;
    std::vector<std::string> names_;
    bool to_shortest_, flatten_;
    Finitude fin_;
};

// Wraps a Python iterator; its state is the pickled iterator itself.
class PyIteratorSource final : public DataSource {
public:
    // The iterator is handed to `reset_fn` before its first element is read, here and after every reset: a source
    // built anew over an iterator that an earlier pass used up (a `yield_from` callback after a reset of the outer
    // pipeline) starts from the beginning like any other source.
    PyIteratorSource(py::object it, py::object reset_fn, bool infinite)
        : it_(std::move(it)), reset_fn_(std::move(reset_fn)), infinite_(infinite) {}
    ~PyIteratorSource() override {
        py::gil_scoped_acquire gil;
        it_ = py::object();
        reset_fn_ = py::object();
    }
    std::optional<Data> next() override {
        py::gil_scoped_acquire gil;
        if (pending_reset_) {
            pending_reset_ = false;
            it_ = reset_fn_(it_);
        }
        PyObject* item = PyIter_Next(it_.ptr());
        if (item == nullptr) {
            if (PyErr_Occurred()) throw py::error_already_set();
            return std::nullopt;
        }
        return data_from_py(py::reinterpret_steal<py::object>(item));
    }
    void reset(bool) override { pending_reset_ = true; }
    void record_position(Tape& t, bool) const override {
        py::gil_scoped_acquire gil;
        py::object dumps = py::module_::import("pickle").attr("dumps");
        t.record(Data(PyObjectHolder(dumps(it_))));
        t.record(Data(pending_reset_));
    }
    void reload_position(Tape& t, bool) override {
        py::gil_scoped_acquire gil;
        Data d = t.read();
        py::object loads = py::module_::import("pickle").attr("loads");
        it_ = loads(data_to_py(d));
        pending_reset_ = t.read_bool();
    }
    Finitude finitude() const override { return infinite_ ? Finitude::Infinite : Finitude::Finite; }

private:
    py::object it_, reset_fn_;
    bool infinite_;
    bool pending_reset_ = true;
};

// ===================================================================== operators
class BucketSource final : public DataSource {
public:
    BucketSource(std::unique_ptr<DataSource> in, size_t n, bool drop) : in_(std::move(in)), n_(n), drop_(drop) {}
    std::optional<Data> next() override {
        DataList out;
        out.reserve(n_);
        while (out.size() < n_) {
            auto d = in_->next();
            if (!d) break;
            out.push_back(std::move(*d));
        }
        if (out.empty()) return std::nullopt;
        if (drop_ && out.size() < n_) return std::nullopt;
        return Data(std::move(out));
    }
    void reset(bool r) override { in_->reset(r); }
    void record_position(Tape& t, bool s) const override { in_->record_position(t, s); }
    void reload_position(Tape& t, bool s) override { in_->reload_position(t, s); }
    Finitude finitude() const override { return in_->finitude(); }

private:
    std::unique_ptr<DataSource> in_;
    size_t n_;
    bool drop_;
};

class BucketByLengthSource final : public DataSource {
public:
    BucketByLengthSource(std::unique_ptr<DataSource> in, std::vector<std::pair<size_t, size_t>> sizes,
                         std::optional<std::string> selector, size_t min_len, bool skip_below, bool skip_above,
                         bool drop)
        : in_(std::move(in)), sizes_(std::move(sizes)), selector_(std::move(selector)), min_len_(min_len),
          skip_below_(skip_below), skip_above_(skip_above), drop_(drop) {
        std::sort(sizes_.begin(), sizes_.end(),
                  [](const auto& a, const auto& b) { return a.second < b.second; });
        max_len_ = sizes_.empty() ? 0 : sizes_.back().second;
        buckets_.resize(sizes_.size());
    }
    std::optional<Data> next() override {
        while (auto d = in_->next()) {
            const size_t len = data_length(select_single(*d, selector_));
            if (len < min_len_) {
                if (skip_below_) continue;
                throw DataPipelineError("The length of the input data must be at least " + std::to_string(min_len_) +
                                        ", but is " + std::to_string(len) + " instead.");
            }
            if (len > max_len_) {
                if (skip_above_) continue;
                throw DataPipelineError("The length of the input data must be at most " + std::to_string(max_len_) +
                                        ", but is " + std::to_string(len) + " instead.");
            }
            size_t b = 0;
            while (sizes_[b].second < len) ++b;
            buckets_[b].push_back(std::move(*d));
            if (buckets_[b].size() >= sizes_[b].first) {
                DataList out = std::move(buckets_[b]);
                buckets_[b].clear();
                return Data(std::move(out));
            }
        }
        if (drop_) {
            for (auto& b : buckets_) b.clear();
            return std::nullopt;
        }
        // end of data: emit the largest non-empty bucket, topped up from smaller buckets
        for (size_t i = buckets_.size(); i-- > 0;) {
            if (buckets_[i].empty()) continue;
            DataList out = std::move(buckets_[i]);
            buckets_[i].clear();
            for (size_t j = i; j-- > 0 && out.size() < sizes_[i].first;) {
                while (!buckets_[j].empty() && out.size() < sizes_[i].first) {
                    out.push_back(std::move(buckets_[j].back()));
                    buckets_[j].pop_back();
                }
            }
            return Data(std::move(out));
        }
        return std::nullopt;
    }
    void reset(bool r) override {
        for (auto& b : buckets_) b.clear();
        in_->reset(r);
    }
    void record_position(Tape& t, bool s) const override {
        for (const auto& b : buckets_) t.record(Data(DataList(b)));
        in_->record_position(t, s);
    }
    void reload_position(Tape& t, bool s) override {
        for (auto& b : buckets_) b = t.read().as_list();
        in_->reload_position(t, s);
    }
    Finitude finitude() const override { return in_->finitude(); }

private:
    std::unique_ptr<DataSource> in_;
    std::vector<std::pair<size_t, size_t>> sizes_;
    std::optional<std::string> selector_;
    size_t min_len_, max_len_ = 0;
    bool skip_below_, skip_above_, drop_;
    std::vector<DataList> buckets_;
};

class DynamicBucketSource final : public DataSource {
public:
    DynamicBucketSource(std::unique_ptr<DataSource> in, double threshold, CostFn cost,
                        std::optional<BucketCreationFn> creation, std::optional<size_t> min_n,
                        std::optional<size_t> max_n, bool drop)
        : in_(std::move(in)), threshold_(threshold), cost_(std::move(cost)), creation_(std::move(creation)),
          min_n_(min_n), max_n_(max_n), drop_(drop) {}
    std::optional<Data> next() override {
        if (!ready_.empty()) {
            Data out(std::move(ready_.front()));
            ready_.pop_front();
            return out;
        }
        // the cost runs over the examples added since the last bucket was cut: what a creation function hands back
        // as the remainder starts the next bucket at cost zero (fairseq2n's dynamic_bucket_data_source.cc does so)
        double& cost = acc_cost_;
        auto full = [&]() {
            const bool cost_ok = cost >= threshold_;
            const bool min_ok = !min_n_ || buffer_.size() >= *min_n_;
            const bool max_hit = max_n_ && buffer_.size() >= *max_n_;
            return (cost_ok && min_ok) || max_hit;
        };
        while (true) {
            if (!buffer_.empty() && full()) {
                if (creation_) {
                    auto res = (*creation_)(DataList(buffer_));
                    if (res) {
                        for (auto& b : res->first) ready_.push_back(b.is_list() ? b.as_list() : DataList{b});
                        buffer_ = std::move(res->second);
                        cost = 0;
                        if (!ready_.empty()) {
                            Data out(std::move(ready_.front()));
                            ready_.pop_front();
                            return out;
                        }
                    }
                } else {
                    DataList out = std::move(buffer_);
                    buffer_.clear();
                    cost = 0;
                    return Data(std::move(out));
                }
            }
            auto d = in_->next();
            if (!d) break;
            cost += cost_(*d);
            buffer_.push_back(std::move(*d));
        }
        cost = 0;
        if (buffer_.empty() || drop_) {
            buffer_.clear();
            return std::nullopt;
        }
        DataList out = std::move(buffer_);
        buffer_.clear();
        return Data(std::move(out));
    }
    void reset(bool r) override {
        buffer_.clear();
        ready_.clear();
        acc_cost_ = 0;
        in_->reset(r);
    }
    void record_position(Tape& t, bool s) const override {
        t.record(Data(acc_cost_));
        t.record(Data(DataList(buffer_)));
        DataList rd;
        for (const auto& b : ready_) rd.emplace_back(DataList(b));
        t.record(Data(std::move(rd)));
        in_->record_position(t, s);
    }
    void reload_position(Tape& t, bool s) override {
        acc_cost_ = t.read().as_float();
        buffer_ = t.read().as_list();
        ready_.clear();
        for (auto& b : t.read().as_list()) ready_.push_back(b.as_list());
        in_->reload_position(t, s);
    }
    Finitude finitude() const override { return in_->finitude(); }

private:
    double acc_cost_ = 0;
    std::unique_ptr<DataSource> in_;
    double threshold_;
    CostFn cost_;
    std::optional<BucketCreationFn> creation_;
    std::optional<size_t> min_n_, max_n_;
    bool drop_;
    DataList buffer_;
    std::deque<DataList> ready_;
};

class FilterSource final : public DataSource {
public:
    FilterSource(std::unique_ptr<DataSource> in, PredicateFn fn) : in_(std::move(in)), fn_(std::move(fn)) {}
    std::optional<Data> next() override {
        while (auto d = in_->next())
            if (fn_(*d)) return d;
        return std::nullopt;
    }
    void reset(bool r) override { in_->reset(r); }
    void record_position(Tape& t, bool s) const override { in_->record_position(t, s); }
    void reload_position(Tape& t, bool s) override { in_->reload_position(t, s); }
    Finitude finitude() const override { return in_->finitude(); }

private:
    std::unique_ptr<DataSource> in_;
    PredicateFn fn_;
};

// ---------------------------------------------------------------- thread pool
class WorkerPool {
public:
    explicit WorkerPool(size_t n) {
        for (size_t i = 0; i < n; ++i) threads_.emplace_back([this] { run(); });
    }
    ~WorkerPool() {
        {
            std::lock_guard<std::mutex> lk(m_);
            stop_ = true;
        }
        cv_.notify_all();
        for (auto& t : threads_) t.join();
    }
    void submit(std::function<void()> fn) {
        {
            std::lock_guard<std::mutex> lk(m_);
            q_.push_back(std::move(fn));
        }
        cv_.notify_one();
    }

private:
    void run() {
        while (true) {
            std::function<void()> fn;
            {
                std::unique_lock<std::mutex> lk(m_);
                cv_.wait(lk, [this] { return stop_ || !q_.empty(); });
                if (stop_ && q_.empty()) return;
                fn = std::move(q_.front());
                q_.pop_front();
            }
            fn();
        }
    }
    std::vector<std::thread> threads_;
    std::deque<std::function<void()>> q_;
    std::mutex m_;
    std::condition_variable cv_;
    bool stop_ = false;
};

// map: sequential, or `num_parallel_calls` workers. In parallel mode a buffer
// of N examples is filled, mapped concurrently and drained in order
// (deterministic) -- output order always equals input order.
class MapSource final : public DataSource {
public:
    MapSource(std::unique_ptr<DataSource> in, std::vector<MapFn> fns, std::optional<std::string> selector,
              size_t num_parallel)
        : in_(std::move(in)), fns_(std::move(fns)), selector_(std::move(selector)), n_(num_parallel), window_(num_parallel) {
        if (n_ > 1) pool_ = std::make_unique<WorkerPool>(n_);
    }
    std::optional<Data> next() override {
        if (n_ <= 1) {
            auto d = in_->next();
            if (!d) return std::nullopt;
            return invoke(std::move(*d));
        }
        if (out_pos_ >= out_.size()) {
            if (!fill()) return std::nullopt;
        }
        auto& slot = out_[out_pos_++];
        if (slot.error) std::rethrow_exception(slot.error);
        return std::move(slot.value);
    }
    void reset(bool r) override {
        out_.clear();
        out_pos_ = 0;
        window_ = n_;
        in_->reset(r);
    }
    void record_position(Tape& t, bool s) const override {
        // remaining mapped-but-unread outputs are part of the position (left out of a state that is not strict)
        DataList rest;
        if (s)
            for (size_t i = out_pos_; i < out_.size(); ++i)
                if (!out_[i].error) rest.push_back(out_[i].value);
        t.record(Data(std::move(rest)));
        in_->record_position(t, s);
    }
    void reload_position(Tape& t, bool s) override {
        out_.clear();
        out_pos_ = 0;
        for (auto& e : t.read().as_list()) out_.push_back(Slot{e, nullptr});
        in_->reload_position(t, s);
    }
    Finitude finitude() const override { return in_->finitude(); }

private:
    struct Slot {
        Data value;
        std::exception_ptr error;
    };
    Data invoke(Data&& d) {
        Data cur = std::move(d);
        for (const auto& fn : fns_) cur = apply_selected(std::move(cur), selector_, fn);
        return cur;
    }
    // Reads a window of inputs and maps it on the workers, one contiguous slice per worker (output order = input
    // order). The window starts at `num_parallel_calls` items, so a short or interactive pipeline reads no further
    // ahead than it asks for, and doubles on every refill up to kMaxItemsPerWorker per worker, so that the cost of
    // handing work over is spread over many items when the function is cheap.
    static constexpr size_t kMaxItemsPerWorker = 32;
    bool fill() {
        out_.clear();
        out_pos_ = 0;
        DataList in;
        while (in.size() < window_) {
            auto d = in_->next();
            if (!d) break;
            in.push_back(std::move(*d));
        }
        if (in.empty()) return false;
        if (in.size() == window_) window_ = std::min(window_ * 2, n_ * kMaxItemsPerWorker);
        out_.resize(in.size());
        const size_t tasks = std::min(n_, in.size());
        const size_t per_task = (in.size() + tasks - 1) / tasks;
        std::mutex m;
        std::condition_variable cv;
        size_t pending = tasks;
        for (size_t k = 0; k < tasks; ++k) {
            pool_->submit([&, k] {
                const size_t lo = k * per_task, hi = std::min(in.size(), lo + per_task);
                for (size_t i = lo; i < hi; ++i) {
                    try {
                        out_[i].value = invoke(std::move(in[i]));
                    } catch (...) {
                        out_[i].error = std::current_exception();
                    }
                }
                std::lock_guard<std::mutex> lk(m);
                if (--pending == 0) cv.notify_one();
            });
        }
        {
            MaybeRelease rel;  // the GIL must not be held while waiting for workers that may need it
            std::unique_lock<std::mutex> lk(m);
            cv.wait(lk, [&] { return pending == 0; });
        }
        return true;
    }
    struct MaybeRelease {
        PyThreadState* st = nullptr;
        MaybeRelease() {
            if (PyGILState_Check()) st = PyEval_SaveThread();
        }
        ~MaybeRelease() {
            if (st) PyEval_RestoreThread(st);
        }
    };

    std::unique_ptr<DataSource> in_;
    std::vector<MapFn> fns_;
    std::optional<std::string> selector_;
    size_t n_;
    std::unique_ptr<WorkerPool> pool_;
    size_t window_ = 0;
    std::vector<Slot> out_;
    size_t out_pos_ = 0;
};

// map with `deterministic=False`: up to 2 x `num_parallel_calls` elements are in flight on the workers at any
// time and results are handed out in the order in which they finish, so one slow element never holds back the
// others and the workers never wait for a window to drain. The position of such a stage is the set of finished,
// not yet returned results plus the position of its input (recording it waits for the elements in flight).
class AsyncMapSource final : public DataSource {
public:
    AsyncMapSource(std::unique_ptr<DataSource> in, std::vector<MapFn> fns, std::optional<std::string> selector,
                   size_t num_parallel)
        : in_(std::move(in)), fns_(std::move(fns)), selector_(std::move(selector)), n_(num_parallel),
          st_(std::make_shared<Shared>()), pool_(std::make_unique<WorkerPool>(num_parallel)) {}
    ~AsyncMapSource() override {
        pool_.reset();   // joins the workers: no task outlives the state it writes to
    }
    std::optional<Data> next() override {
        while (true) {
            top_up();
            MaybeRelease rel;   // workers running Python callables need the interpreter lock
            std::unique_lock<std::mutex> lk(st_->m);
            st_->cv.wait(lk, [&] { return !st_->done.empty() || st_->in_flight == 0; });
            if (!st_->done.empty()) {
                Slot slot = std::move(st_->done.front());
                st_->done.pop_front();
                lk.unlock();
                if (slot.error) std::rethrow_exception(slot.error);
                return std::move(slot.value);
            }
            if (eod_) return std::nullopt;
            // nothing finished, nothing in flight and the input still has elements: read more
        }
    }
    void reset(bool r) override {
        drain();
        st_->done.clear();
        eod_ = false;
        in_->reset(r);
    }
    void record_position(Tape& t, bool s) const override {
        const_cast<AsyncMapSource*>(this)->drain();
        DataList rest;
        if (s)
            for (const Slot& slot : st_->done)
                if (!slot.error) rest.push_back(slot.value);
        t.record(Data(std::move(rest)));
        in_->record_position(t, s);
    }
    void reload_position(Tape& t, bool s) override {
        drain();
        st_->done.clear();
        eod_ = false;
        for (auto& e : t.read().as_list()) st_->done.push_back(Slot{e, nullptr});
        in_->reload_position(t, s);
    }
    Finitude finitude() const override { return in_->finitude(); }

private:
    struct Slot {
        Data value;
        std::exception_ptr error;
    };
    struct Shared {
        std::mutex m;
        std::condition_variable cv;
        std::deque<Slot> done;
        size_t in_flight = 0;
    };
    struct MaybeRelease {
        PyThreadState* st = nullptr;
        MaybeRelease() {
            if (PyGILState_Check()) st = PyEval_SaveThread();
        }
        ~MaybeRelease() {
            if (st) PyEval_RestoreThread(st);
        }
    };
    void top_up() {
        while (!eod_) {
            {
                std::lock_guard<std::mutex> lk(st_->m);
                if (st_->in_flight + st_->done.size() >= 2 * n_) return;
            }
            auto d = in_->next();
            if (!d) {
                eod_ = true;
                return;
            }
            {
                std::lock_guard<std::mutex> lk(st_->m);
                ++st_->in_flight;
            }
            auto st = st_;
            auto item = std::make_shared<Data>(std::move(*d));
            pool_->submit([this, st, item] {
                Slot slot;
                try {
                    Data cur = std::move(*item);
                    for (const auto& fn : fns_) cur = apply_selected(std::move(cur), selector_, fn);
                    slot.value = std::move(cur);
                } catch (...) {
                    slot.error = std::current_exception();
                }
                std::lock_guard<std::mutex> lk(st->m);
                st->done.push_back(std::move(slot));
                --st->in_flight;
                st->cv.notify_all();
            });
        }
    }
    void drain() {
        MaybeRelease rel;
        std::unique_lock<std::mutex> lk(st_->m);
        st_->cv.wait(lk, [&] { return st_->in_flight == 0; });
    }

    std::unique_ptr<DataSource> in_;
    std::vector<MapFn> fns_;
    std::optional<std::string> selector_;
    size_t n_;
    bool eod_ = false;
    std::shared_ptr<Shared> st_;
    std::unique_ptr<WorkerPool> pool_;
};

// Packs 1-D tensors into fixed-size buffers of `num_elements` elements.
class PackSource final : public DataSource {
public:
    PackSource(std::unique_ptr<DataSource> in, int64_t num_elements, int64_t max_seq_len, int64_t pad_value,
               bool truncate, bool drop_remainder, bool pinned)
        : in_(std::move(in)), capacity_(num_elements), max_seq_len_(max_seq_len), pad_(pad_value),
          truncate_(truncate), drop_(drop_remainder), pinned_(pinned) {}
    // Rules (those of fairseq2n's packed_data_source.cc:19-122):
    //  * a piece of a sequence is at most `max_seq_len` long and never crosses the end of the buffer;
    //  * `truncate`: a sequence that is longer than the room it gets is cut. Cut at the end of the buffer, the next
    //    buffer starts again with the last token that went in (so that no next-token target is lost); cut by
    //    `max_seq_len` inside a buffer, the rest follows as its own piece;
    //  * without `truncate` a sequence that does not fit (or is longer than `max_seq_len`) closes the buffer and
    //    opens the next one; alone in an empty buffer it is an error;
    //  * a last, partly filled buffer is dropped only with `truncate` and `drop_remainder`.
    std::optional<Data> next() override {
        at::Tensor buf;
        DataList lens;
        int64_t fill = 0;
        bool filled = false;
        while (true) {
            at::Tensor seq;
            std::optional<Data> example;
            if (remainder_.defined()) {
                seq = remainder_;
                remainder_ = at::Tensor();
            } else {
                example = in_->next();
                if (!example) break;
                if (!example->is_tensor())
                    throw DataPipelineError("The pack operation can only be used with tensor inputs.", /*recoverable=*/true);
                seq = example->as_tensor();
                if (seq.dim() != 1)
                    throw DataPipelineError("The input tensors to the pack operation must be one-dimensional.",
                                            /*recoverable=*/true);
            }
            if (!buf.defined()) {
                buf = at::full({capacity_}, pad_, seq.options().pinned_memory(pinned_));
            } else {
                seq = seq.to(buf.device());
            }
            const int64_t numel = seq.numel();
            if (numel == 0) continue;
            const int64_t piece = std::min(numel, std::min(capacity_ - fill, max_seq_len_));
            if (numel > piece) {
                if (truncate_) {
                    const bool at_buffer_end = fill + piece == capacity_;
                    remainder_ = seq.slice(0, at_buffer_end ? piece - 1 : piece);
                    seq = seq.slice(0, 0, piece);
                } else {
                    if (fill == 0)
                        throw DataPipelineError("The input tensor is too long to pack.", /*recoverable=*/true);
                    remainder_ = seq;
                    break;
                }
            }
            buf.slice(0, fill, fill + piece).copy_(seq);
            lens.emplace_back(piece);
            fill += piece;
            if (fill == capacity_) {
                filled = true;
                break;
            }
        }
        if (truncate_ && !filled && drop_) return std::nullopt;
        if (!buf.defined()) return std::nullopt;
        DataDict out{{"seqs", Data(buf)}, {"seq_lens", Data(std::move(lens))}};
        return Data(std::move(out));
    }
    void reset(bool r) override {
        remainder_ = at::Tensor();
        eod_ = false;
        in_->reset(r);
    }
    void record_position(Tape& t, bool s) const override {
        t.record_bool(eod_);
        t.record_bool(remainder_.defined());
        if (remainder_.defined()) t.record(Data(remainder_));
        in_->record_position(t, s);
    }
    void reload_position(Tape& t, bool s) override {
        eod_ = t.read_bool();
        if (t.read_bool()) remainder_ = t.read().as_tensor();
        else remainder_ = at::Tensor();
        in_->reload_position(t, s);
    }
    Finitude finitude() const override { return in_->finitude(); }

private:
    std::unique_ptr<DataSource> in_;
    int64_t capacity_, max_seq_len_, pad_;
    bool truncate_, drop_, pinned_;
    at::Tensor remainder_;
    bool eod_ = false;
};

// Background thread that keeps up to `n` examples ready.
class PrefetchSource final : public DataSource {
public:
    PrefetchSource(std::unique_ptr<DataSource> in, size_t n) : in_(std::move(in)), n_(n) {}
    ~PrefetchSource() override { stop_thread(); }
    std::optional<Data> next() override {
        if (n_ == 0) return in_->next();
        ensure_thread();
        MaybeRelease rel;  // the producer may need the GIL (Python map functions)
        std::unique_lock<std::mutex> lk(m_);
        cv_out_.wait(lk, [this] { return !q_.empty() || state_ != State::Running; });
        if (!q_.empty()) {
            Data d = std::move(q_.front());
            q_.pop_front();
            cv_in_.notify_one();
            return d;
        }
        if (state_ == State::Faulted) {
            std::exception_ptr e = error_;
            state_ = State::Eod;
            lk.unlock();
            std::rethrow_exception(e);
        }
        return std::nullopt;
    }
    void reset(bool r) override {
        stop_thread();
        q_.clear();
        state_ = State::NotRunning;
        in_->reset(r);
    }
    void record_position(Tape& t, bool s) const override {
        auto* self = const_cast<PrefetchSource*>(this);
        self->stop_thread();  // quiesce: the queue and the inner position are then consistent
        {
            std::lock_guard<std::mutex> lk(m_);
            t.record(Data(s ? DataList(q_.begin(), q_.end()) : DataList{}));   // not strict: without the queue
            t.record_bool(state_ == State::Eod);
        }
        in_->record_position(t, s);
        if (self->state_ != State::Eod) self->state_ = State::NotRunning;
    }
    void reload_position(Tape& t, bool s) override {
        stop_thread();
        q_.clear();
        for (auto& e : t.read().as_list()) q_.push_back(e);
        state_ = t.read_bool() ? State::Eod : State::NotRunning;
        in_->reload_position(t, s);
    }
    Finitude finitude() const override { return in_->finitude(); }

private:
    enum class State { NotRunning, Running, Eod, Faulted };
    struct MaybeRelease {
        PyThreadState* st = nullptr;
        MaybeRelease() {
            if (PyGILState_Check()) st = PyEval_SaveThread();
        }
        ~MaybeRelease() {
            if (st) PyEval_RestoreThread(st);
        }
    };
    void ensure_thread() {
        std::lock_guard<std::mutex> lk(m_);
        if (state_ != State::NotRunning) return;
        state_ = State::Running;
        stop_ = false;
        thread_ = std::thread([this] { produce(); });
    }
    void produce() {
        while (true) {
            {
                std::unique_lock<std::mutex> lk(m_);
                cv_in_.wait(lk, [this] { return stop_ || q_.size() < n_; });
                if (stop_) return;
            }
            std::optional<Data> d;
            try {
                d = in_->next();
            } catch (...) {
                std::lock_guard<std::mutex> lk(m_);
                error_ = std::current_exception();
                state_ = State::Faulted;
                cv_out_.notify_all();
                return;
            }
            std::lock_guard<std::mutex> lk(m_);
            if (!d) {
                state_ = State::Eod;
                cv_out_.notify_all();
                return;
            }
            q_.push_back(std::move(*d));
            cv_out_.notify_one();
        }
    }
    void stop_thread() {
        {
            std::lock_guard<std::mutex> lk(m_);
            stop_ = true;
        }
        cv_in_.notify_all();
        if (thread_.joinable()) {
            MaybeRelease rel;
            thread_.join();
        }
        std::lock_guard<std::mutex> lk(m_);
        if (state_ == State::Running) state_ = State::NotRunning;
    }

    std::unique_ptr<DataSource> in_;
    size_t n_;
    mutable std::mutex m_;
    std::condition_variable cv_in_, cv_out_;
    std::deque<Data> q_;
    std::thread thread_;
    State state_ = State::NotRunning;
    bool stop_ = false;
    std::exception_ptr error_;
};

class RepeatSource final : public DataSource {
public:
    RepeatSource(std::unique_ptr<DataSource> in, std::optional<size_t> n, bool reset_rng)
        : in_(std::move(in)), n_(n), reset_rng_(reset_rng) {}
    std::optional<Data> next() override {
        if (n_ && *n_ == 0) return std::nullopt;
        while (true) {
            auto d = in_->next();
            if (d) {
                has_data_ = true;
                return d;
            }
            if (!has_data_) return std::nullopt;  // inner never produced anything
            ++repeat_nr_;
            if (n_ && repeat_nr_ >= *n_) return std::nullopt;
            in_->reset(reset_rng_);
            has_data_ = false;
        }
    }
    void reset(bool r) override {
        repeat_nr_ = 0;
        has_data_ = false;
        in_->reset(r);
    }
    void record_position(Tape& t, bool s) const override {
        t.record_int(static_cast<int64_t>(repeat_nr_));
        t.record_bool(has_data_);
        in_->record_position(t, s);
    }
    void reload_position(Tape& t, bool s) override {
        repeat_nr_ = static_cast<size_t>(t.read_int());
        has_data_ = t.read_bool();
        in_->reload_position(t, s);
    }
    Finitude finitude() const override {
        return n_ ? in_->finitude() : Finitude::Infinite;   // repeated without a count: endless for good
    }

private:
    std::unique_ptr<DataSource> in_;
    std::optional<size_t> n_;
    bool reset_rng_;
    size_t repeat_nr_ = 0;
    bool has_data_ = false;
};

class ShardSource final : public DataSource {
public:
    ShardSource(std::unique_ptr<DataSource> in, size_t idx, size_t n, bool uneven)
        : in_(std::move(in)), idx_(idx), n_(n), uneven_(uneven) {}
    std::optional<Data> next() override {
        std::optional<Data> mine;
        for (size_t i = 0; i < n_; ++i) {
            auto d = in_->next();
            if (!d) {
                // incomplete final group
                if (uneven_ && mine) return mine;
                return std::nullopt;
            }
            if (i == idx_) mine = std::move(d);
        }
        return mine;
    }
    void reset(bool r) override { in_->reset(r); }
    void record_position(Tape& t, bool s) const override { in_->record_position(t, s); }
    void reload_position(Tape& t, bool s) override { in_->reload_position(t, s); }
    Finitude finitude() const override { return in_->finitude(); }

private:
    std::unique_ptr<DataSource> in_;
    size_t idx_, n_;
    bool uneven_;
};

// Window shuffle: fill a window, Fisher-Yates it, then replace-one-read-one.
class ShuffleSource final : public DataSource {
public:
    ShuffleSource(std::unique_ptr<DataSource> in, size_t window, uint64_t seed)
        : in_(std::move(in)), window_(window == 0 ? SIZE_MAX : window), seed_(seed), gen_(seed) {}
    std::optional<Data> next() override {
        if (window_ == 1) return in_->next();
        if (!filled_) {
            while (buf_.size() < window_) {
                auto d = in_->next();
                if (!d) {
                    inner_done_ = true;
                    break;
                }
                buf_.push_back(std::move(*d));
            }
            for (size_t k = buf_.size(); k > 1; --k) std::swap(buf_[k - 1], buf_[gen_.below(k)]);  // Fisher-Yates
            filled_ = true;
        }
        if (buf_.empty()) return std::nullopt;
        if (inner_done_) {
            Data out = std::move(buf_.back());
            buf_.pop_back();
            return out;
        }
        // pick a random slot, emit it, refill the slot from the input
        const size_t i = gen_.below(buf_.size());
        Data out = std::move(buf_[i]);
        auto d = in_->next();
        if (d) {
            buf_[i] = std::move(*d);
        } else {
            inner_done_ = true;
            buf_[i] = std::move(buf_.back());
            buf_.pop_back();
        }
        return out;
    }
    void reset(bool r) override {
        buf_.clear();
        filled_ = inner_done_ = false;
        if (r) gen_.seed(seed_);
        in_->reset(r);
    }
    void record_position(Tape& t, bool s) const override {
        // not strict: the buffered examples are left out of the state (smaller, and the run goes on with what the
        // input still holds); the buffer is filled again from there
        t.record(Data(s ? DataList(buf_) : DataList{}));
        t.record_bool(s ? filled_ : false);
        t.record_bool(inner_done_);
        t.record_int(static_cast<int64_t>(gen_.state));
        in_->record_position(t, s);
    }
    void reload_position(Tape& t, bool s) override {
        buf_ = t.read().as_list();
        filled_ = t.read_bool();
        inner_done_ = t.read_bool();
        gen_.state = static_cast<uint64_t>(t.read_int());
        in_->reload_position(t, s);
    }
    Finitude finitude() const override { return in_->finitude(); }

private:
    std::unique_ptr<DataSource> in_;
    size_t window_;
    uint64_t seed_;
    Rng gen_;
    DataList buf_;
    bool filled_ = false, inner_done_ = false;
};

class SkipSource final : public DataSource {
public:
    SkipSource(std::unique_ptr<DataSource> in, size_t n) : in_(std::move(in)), n_(n) {}
    std::optional<Data> next() override {
        while (skipped_ < n_) {
            if (!in_->next()) return std::nullopt;
            ++skipped_;
        }
        return in_->next();
    }
    void reset(bool r) override {
        skipped_ = 0;
        in_->reset(r);
    }
    void record_position(Tape& t, bool s) const override {
        t.record_int(static_cast<int64_t>(skipped_));
        in_->record_position(t, s);
    }
    void reload_position(Tape& t, bool s) override {
        skipped_ = static_cast<size_t>(t.read_int());
        in_->reload_position(t, s);
    }
    Finitude finitude() const override { return in_->finitude(); }

private:
    std::unique_ptr<DataSource> in_;
    size_t n_, skipped_ = 0;
};

class TakeSource final : public DataSource {
public:
    TakeSource(std::unique_ptr<DataSource> in, size_t n) : in_(std::move(in)), n_(n) {}
    std::optional<Data> next() override {
        if (taken_ >= n_) return std::nullopt;
        auto d = in_->next();
        if (d) ++taken_;
        return d;
    }
    void reset(bool r) override {
        taken_ = 0;
        in_->reset(r);
    }
    void record_position(Tape& t, bool s) const override {
        t.record_int(static_cast<int64_t>(taken_));
        in_->record_position(t, s);
    }
    void reload_position(Tape& t, bool s) override {
        taken_ = static_cast<size_t>(t.read_int());
        in_->reload_position(t, s);
    }
    Finitude finitude() const override { return Finitude::Finite; }

private:
    std::unique_ptr<DataSource> in_;
    size_t n_, taken_ = 0;
};

class YieldFromSource final : public DataSource {
public:
    YieldFromSource(std::unique_ptr<DataSource> in, YieldFn fn) : in_(std::move(in)), fn_(std::move(fn)) {}
    std::optional<Data> next() override {
        while (true) {
            if (sub_) {
                auto d = sub_->next();
                if (d) return d;
                sub_.reset();
                example_.reset();
            }
            auto ex = in_->next();
            if (!ex) return std::nullopt;
            example_ = *ex;
            sub_ = std::make_unique<DataPipeline>(fn_(*ex));
            if (sub_->finitude() != Finitude::Finite)
                throw DataPipelineError("The data pipeline to yield from cannot be infinite.");
        }
    }
    void reset(bool r) override {
        sub_.reset();
        example_.reset();
        in_->reset(r);
    }
    void record_position(Tape& t, bool s) const override {
        t.record_bool(example_.has_value());
        if (example_) {
            t.record(*example_);
            sub_->record_position(t, s);
        }
        in_->record_position(t, s);
    }
    void reload_position(Tape& t, bool s) override {
        if (t.read_bool()) {
            example_ = t.read();
            sub_ = std::make_unique<DataPipeline>(fn_(*example_));
            sub_->reload_position(t, s);
        } else {
            example_.reset();
            sub_.reset();
        }
        in_->reload_position(t, s);
    }
    Finitude finitude() const override { return in_->finitude(); }

private:
    std::unique_ptr<DataSource> in_;
    YieldFn fn_;
    std::optional<Data> example_;
    std::unique_ptr<DataPipeline> sub_;
};

template <typename T, typename... Args>
DataSourceFactory chain(DataSourceFactory inner, Args... args) {
    return [inner = std::move(inner), args...]() mutable -> std::unique_ptr<DataSource> {
        return std::make_unique<T>(inner(), args...);
    };
}

}  // namespace

// ============================================================== builder methods
DataPipelineBuilder DataPipelineBuilder::bucket(size_t bucket_size, bool drop_remainder) && {
    if (bucket_size == 0) throw std::invalid_argument("`bucket_size` must be greater than zero.");
    return DataPipelineBuilder(chain<BucketSource>(std::move(factory_), bucket_size, drop_remainder));
}

DataPipelineBuilder DataPipelineBuilder::bucket_by_length(std::vector<std::pair<size_t, size_t>> bucket_sizes,
                                                           std::optional<std::string> selector, size_t min_data_len,
                                                           bool skip_below_min, bool skip_above_max,
                                                           bool drop_remainder) && {
    if (bucket_sizes.empty()) throw std::invalid_argument("`bucket_sizes` must contain at least one element.");
    return DataPipelineBuilder(chain<BucketByLengthSource>(std::move(factory_), bucket_sizes, selector, min_data_len,
                                                           skip_below_min, skip_above_max, drop_remainder));
}

DataPipelineBuilder DataPipelineBuilder::dynamic_bucket(double threshold, CostFn cost_fn,
                                                         std::optional<BucketCreationFn> creation_fn,
                                                         std::optional<size_t> min_num_examples,
                                                         std::optional<size_t> max_num_examples,
                                                         bool drop_remainder) && {
    if (threshold <= 0) throw std::invalid_argument("`threshold` must be greater than zero.");
    if (max_num_examples && *max_num_examples == 0)
        throw std::invalid_argument("`max_num_examples` must be greater than zero.");
    if (min_num_examples && max_num_examples && *min_num_examples > *max_num_examples)
        throw std::invalid_argument("`max_num_examples` must be greater than or equal to `min_num_examples`.");
    return DataPipelineBuilder(chain<DynamicBucketSource>(std::move(factory_), threshold, cost_fn, creation_fn,
                                                          min_num_examples, max_num_examples, drop_remainder));
}

DataPipelineBuilder DataPipelineBuilder::filter(PredicateFn fn) && {
    return DataPipelineBuilder(chain<FilterSource>(std::move(factory_), fn));
}

DataPipelineBuilder DataPipelineBuilder::map(std::vector<MapFn> fns, std::optional<std::string> selector,
                                              size_t num_parallel_calls, bool deterministic) && {
    if (num_parallel_calls == 0) throw std::invalid_argument("`num_parallel_calls` must be greater than zero.");
    if (selector) validate_selector(*selector);
    if (!deterministic && num_parallel_calls > 1)
        return DataPipelineBuilder(chain<AsyncMapSource>(std::move(factory_), fns, selector, num_parallel_calls));
    return DataPipelineBuilder(chain<MapSource>(std::move(factory_), fns, selector, num_parallel_calls));
}

DataPipelineBuilder DataPipelineBuilder::pack(int64_t num_elements, int64_t max_seq_len, int64_t pad_value,
                                               bool truncate, bool drop_remainder, bool pinned_memory) && {
    if (num_elements <= 0) throw std::invalid_argument("`num_elements` must be greater than zero.");
    if (max_seq_len <= 0) throw std::invalid_argument("`max_seq_len` must be greater than zero.");
    return DataPipelineBuilder(chain<PackSource>(std::move(factory_), num_elements, max_seq_len, pad_value, truncate,
                                                 drop_remainder, pinned_memory));
}

DataPipelineBuilder DataPipelineBuilder::prefetch(size_t num_examples) && {
    return DataPipelineBuilder(chain<PrefetchSource>(std::move(factory_), num_examples));
}

DataPipelineBuilder DataPipelineBuilder::repeat(std::optional<size_t> num_repeats, bool reset_rng) && {
    return DataPipelineBuilder(chain<RepeatSource>(std::move(factory_), num_repeats, reset_rng));
}

DataPipelineBuilder DataPipelineBuilder::shard(size_t shard_idx, size_t num_shards, bool allow_uneven) && {
    if (shard_idx >= num_shards)
        throw std::invalid_argument("`shard_idx` must be less than `num_shards` (" + std::to_string(num_shards) +
                                    "), but is " + std::to_string(shard_idx) + " instead.");
    return DataPipelineBuilder(chain<ShardSource>(std::move(factory_), shard_idx, num_shards, allow_uneven));
}

DataPipelineBuilder DataPipelineBuilder::shuffle(size_t window, uint64_t seed) && {
    return DataPipelineBuilder(chain<ShuffleSource>(std::move(factory_), window, seed));
}

DataPipelineBuilder DataPipelineBuilder::skip(size_t n) && {
    return DataPipelineBuilder(chain<SkipSource>(std::move(factory_), n));
}

DataPipelineBuilder DataPipelineBuilder::take(size_t n) && {
    return DataPipelineBuilder(chain<TakeSource>(std::move(factory_), n));
}

DataPipelineBuilder DataPipelineBuilder::yield_from(YieldFn fn) && {
    return DataPipelineBuilder(chain<YieldFromSource>(std::move(factory_), fn));
}

// ================================================================ static sources
DataPipelineBuilder read_list(DataList items) {
    auto shared = std::make_shared<DataList>(std::move(items));
    return DataPipelineBuilder([shared]() -> std::unique_ptr<DataSource> { return std::make_unique<ListSource>(*shared); });
}

DataPipelineBuilder DataPipeline::constant(Data example, std::optional<std::string> key) {
    return DataPipelineBuilder([example, key]() -> std::unique_ptr<DataSource> {
        return std::make_unique<ConstantSource>(example, key);
    });
}

DataPipelineBuilder DataPipeline::count(int64_t start, int64_t step, std::optional<std::string> key) {
    return DataPipelineBuilder([start, step, key]() -> std::unique_ptr<DataSource> {
        return std::make_unique<CountSource>(start, step, key);
    });
}

namespace {
std::shared_ptr<std::vector<DataPipeline>> share(std::vector<DataPipeline> ps) {
    for (const auto& p : ps)
        if (p.is_broken()) throw std::invalid_argument("At least one of the specified data pipelines is broken.");
    return std::make_shared<std::vector<DataPipeline>>(std::move(ps));
}
}  // namespace

namespace {

void refuse_broken(const std::vector<DataPipeline>& pipelines, const char* what) {
    for (const auto& p : pipelines)
        if (p.is_broken())
            throw std::invalid_argument(std::string("At least one of the specified data pipelines is broken and cannot be ") +
                                        what + ".");
}

}  // namespace

DataPipelineBuilder DataPipeline::concat(std::vector<DataPipeline> pipelines) {
    refuse_broken(pipelines, "concatenated");
    auto sp = share(std::move(pipelines));
    return DataPipelineBuilder([sp]() -> std::unique_ptr<DataSource> {
        return std::make_unique<ConcatSource>(std::move(*sp));
    });
}

DataPipelineBuilder DataPipeline::round_robin(std::vector<DataPipeline> pipelines, bool stop_at_shortest,
                                              bool allow_repeats) {
    refuse_broken(pipelines, "used in round robin");
    auto sp = share(std::move(pipelines));
    return DataPipelineBuilder([sp, stop_at_shortest, allow_repeats]() -> std::unique_ptr<DataSource> {
        return std::make_unique<RoundRobinSource>(std::move(*sp), stop_at_shortest, allow_repeats);
    });
}

DataPipelineBuilder DataPipeline::sample(std::vector<DataPipeline> pipelines, std::optional<std::vector<float>> weights,
                                         uint64_t seed, bool allow_repeats) {
    refuse_broken(pipelines, "sampled");
    std::vector<float> w = weights ? *weights : std::vector<float>(pipelines.size(), 1.0f);
    if (w.size() != pipelines.size())
        throw std::invalid_argument("The number of `pipelines` and `weights` must be equal.");
    for (float x : w)
        if (!(x > 0) || !std::isfinite(x)) throw std::invalid_argument("All `weights` must be positive and finite.");
    auto sp = share(std::move(pipelines));
    return DataPipelineBuilder([sp, w, seed, allow_repeats]() -> std::unique_ptr<DataSource> {
        return std::make_unique<SampleSource>(std::move(*sp), w, seed, allow_repeats);
    });
}

DataPipelineBuilder DataPipeline::zip(std::vector<DataPipeline> pipelines, std::vector<std::string> names,
                                      bool zip_to_shortest, bool flatten, bool) {
    refuse_broken(pipelines, "zipped");
    if (!names.empty() && flatten)
        throw std::invalid_argument("`names` and `flatten` are mutually exclusive and cannot be specified at the same time.");
    if (!names.empty() && names.size() != pipelines.size())
        throw std::invalid_argument("The number of `pipelines` and the number of `names` must be equal, but are " +
                                    std::to_string(pipelines.size()) + " and " + std::to_string(names.size()) +
                                    " instead.");
    bool any_inf = false, any_fin = false;
    for (const auto& p : pipelines) {
        if (p.finitude() == Finitude::Infinite) any_inf = true;
        else if (p.finitude() == Finitude::Finite) any_fin = true;
    }
    if (any_inf && any_fin && !zip_to_shortest) throw DataPipelineError("Cannot mix finite and infinite pipelines in zip.");
    auto sp = share(std::move(pipelines));
    return DataPipelineBuilder([sp, names, zip_to_shortest, flatten]() -> std::unique_ptr<DataSource> {
        return std::make_unique<ZipSource>(std::move(*sp), names, zip_to_shortest, flatten);
    });
}

DataPipelineBuilder read_py_iterator(py::object iterator, py::object reset_fn, bool infinite) {
    // The factory may be destroyed on any thread and without the interpreter lock (a pipeline built inside a
    // `yield_from` callback dies in the middle of a `next()` that runs unlocked): the references are dropped under
    // the lock, whoever drops them.
    auto release = [](py::object* o) {
        py::gil_scoped_acquire gil;
        delete o;
    };
    std::shared_ptr<py::object> it(new py::object(std::move(iterator)), release);
    std::shared_ptr<py::object> rf(new py::object(std::move(reset_fn)), release);
    return DataPipelineBuilder([it, rf, infinite]() -> std::unique_ptr<DataSource> {
        py::gil_scoped_acquire gil;
        return std::make_unique<PyIteratorSource>(*it, *rf, infinite);
    });
}

}  // namespace fs2d
