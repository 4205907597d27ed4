// Unit tests of the native data runtime, written against the C++ API (no Python callables involved): the tape, the
// memory block, the value type, the LRU file mapper, the collater and the pipeline operators with their
// record/reload and reset contracts. A tiny registry stands in for a test framework: `TEST(name) { ... }` registers a
// case, `CHECK`/`CHECK_THROWS` record failures, and `run_all()` (bound to Python) returns one row per case so that the
// Python test suite can assert on them. Counterpart in spirit of fairseq2n's `native/tests/*.cc`.
#include <unistd.h>

#include <cstdio>
#include <fstream>
#include <random>
#include <sstream>
#include <thread>

#include "../data.h"
#include "../extras.h"

namespace {

using namespace fs2d;

struct Case {
    const char* name;
    void (*fn)();
};

std::vector<Case>& registry() {
    static std::vector<Case> r;
    return r;
}

struct Failure : std::runtime_error {
    using std::runtime_error::runtime_error;
};

struct Registrar {
    Registrar(const char* n, void (*f)()) { registry().push_back({n, f}); }
};

#define TEST(name)                                   \
    static void test_##name();                       \
    static Registrar registrar_##name(#name, test_##name); \
    static void test_##name()

#define CHECK(cond)                                                                                   \
    do {                                                                                              \
        if (!(cond)) {                                                                                \
            std::ostringstream os;                                                                    \
            os << __FILE__ << ":" << __LINE__ << ": CHECK(" #cond ") failed";                         \
            throw Failure(os.str());                                                                  \
        }                                                                                             \
    } while (0)

#define CHECK_THROWS(expr, ExType)                                                                    \
    do {                                                                                              \
        bool thrown_ = false;                                                                         \
        try {                                                                                         \
            (void)(expr);                                                                             \
        } catch (const ExType&) {                                                                     \
            thrown_ = true;                                                                           \
        }                                                                                             \
        if (!thrown_) {                                                                               \
            std::ostringstream os;                                                                    \
            os << __FILE__ << ":" << __LINE__ << ": " #expr " did not throw " #ExType;                \
            throw Failure(os.str());                                                                  \
        }                                                                                             \
    } while (0)

DataList ints(int64_t n, int64_t start = 0) {
    DataList l;
    for (int64_t i = 0; i < n; ++i) l.emplace_back(start + i);
    return l;
}

std::vector<int64_t> drain(DataPipeline& p) {
    std::vector<int64_t> out;
    while (auto d = p.next()) out.push_back(d->as_int());
    return out;
}

std::vector<int64_t> iota(int64_t n, int64_t start = 0) {
    std::vector<int64_t> v;
    for (int64_t i = 0; i < n; ++i) v.push_back(start + i);
    return v;
}

struct TempFile {
    std::string path;
    TempFile(const std::string& tag, const std::string& content) {
        char buf[] = "/tmp/fs2d_test_XXXXXX";
        int fd = mkstemp(buf);
        if (fd < 0) throw Failure("mkstemp failed");
        path = buf;
        ssize_t n = write(fd, content.data(), content.size());
        close(fd);
        if (n != static_cast<ssize_t>(content.size())) throw Failure("short write to " + tag);
    }
    ~TempFile() { std::remove(path.c_str()); }
};

// Runs `make()` to the end; then, for every split point k, takes k examples, records the position, takes two more
// (so that internal buffers move on), reloads the position and checks that the tail equals the uninterrupted run;
// finally checks that reset() replays from the start.
template <typename Make>
void check_round_trip(Make make, bool check_reset = true) {
    DataPipeline full = make();
    const std::vector<int64_t> want = drain(full);
    for (size_t k = 0; k <= want.size(); ++k) {
        DataPipeline p = make();
        for (size_t i = 0; i < k; ++i) CHECK(p.next().has_value());
        Tape t;
        p.record_position(t);
        p.next();
        p.next();
        t.rewind();
        p.reload_position(t);
        std::vector<int64_t> tail = drain(p);
        CHECK(tail == std::vector<int64_t>(want.begin() + static_cast<long>(k), want.end()));
        // a position recorded in one pipeline restores a freshly built one
        DataPipeline q = make();
        t.rewind();
        q.reload_position(t);
        CHECK(drain(q) == tail);
    }
    if (check_reset) {
        DataPipeline p = make();
        p.next();
        p.next();
        p.reset(true);
        CHECK(drain(p) == want);
    }
}

// ------------------------------------------------------------------- tape
TEST(tape_replays_in_order) {
    Tape t;
    t.record_int(7);
    t.record_bool(true);
    t.record(Data(std::string("x")));
    CHECK(!t.at_end());
    t.rewind();
    CHECK(t.read_int() == 7);
    CHECK(t.read_bool());
    CHECK(t.read().as_string() == "x");
    CHECK(t.at_end());
    t.rewind();
    CHECK(t.read_int() == 7);
}

TEST(tape_rejects_overrun_and_type_mismatch) {
    Tape t;
    t.record_int(1);
    t.rewind();
    CHECK_THROWS(t.read_bool(), std::invalid_argument);
    CHECK_THROWS(t.read(), std::invalid_argument);
    Tape u(DataList{Data(true)});
    CHECK_THROWS(u.read_int(), std::invalid_argument);
}

TEST(tape_storage_round_trip) {
    Tape t;
    t.record(Data(DataList{Data(1), Data(2.5)}));
    Tape u(t.storage());
    Data d = u.read();
    CHECK(d.is_list() && d.as_list().size() == 2 && d.as_list()[1].as_float() == 2.5);
}

// ----------------------------------------------------------- memory block
TEST(memory_block_copy_and_slice) {
    const char src[] = "0123456789";
    MemoryBlock b = MemoryBlock::copy_of(src, 10);
    CHECK(b.size() == 10 && !b.empty() && b.data()[3] == '3');
    MemoryBlock s = b.slice(2, 5);
    CHECK(s.size() == 5 && s.data()[0] == '2' && s.data()[4] == '6');
    CHECK(b.slice(10, 0).empty());
    CHECK_THROWS(b.slice(11, 0), std::out_of_range);
    CHECK_THROWS(b.slice(4, 7), std::out_of_range);
    CHECK(MemoryBlock().empty());
}

TEST(memory_block_slice_outlives_parent) {
    MemoryBlock s;
    {
        std::string big(1 << 16, 'a');
        big[40000] = 'z';
        MemoryBlock b = MemoryBlock::copy_of(big.data(), big.size());
        s = b.slice(40000, 8);
    }
    CHECK(s.size() == 8 && s.data()[0] == 'z' && s.data()[1] == 'a');
}

TEST(memory_block_files) {
    std::string content;
    for (int i = 0; i < 5000; ++i) content += static_cast<char>('a' + i % 26);
    TempFile f("content", content);
    MemoryBlock m = MemoryBlock::map_file(f.path);
    MemoryBlock r = MemoryBlock::read_file(f.path);
    CHECK(m.size() == content.size() && r.size() == content.size());
    CHECK(std::equal(m.data(), m.data() + m.size(), r.data()));
    CHECK(m.data()[27] == 'b');
    TempFile e("empty", "");
    CHECK(MemoryBlock::map_file(e.path).empty());
    CHECK_THROWS(MemoryBlock::map_file("/nonexistent/fs2d"), ByteStreamError);
    CHECK_THROWS(MemoryBlock::read_file("/nonexistent/fs2d"), ByteStreamError);
}

// ------------------------------------------------------------------- data
TEST(data_variants_and_deep_copy) {
    Data d(DataDict{{"a", Data(1)}, {"b", Data(DataList{Data(2), Data(std::string("s"))})}});
    CHECK(d.is_dict() && d.find("a") && d.find("a")->as_int() == 1 && d.find("zz") == nullptr);
    Data shallow = d;
    Data deep = d.deep_copy();
    d.find("b")->as_list()[0] = Data(99);
    CHECK(shallow.find("b")->as_list()[0].as_int() == 99);     // shared storage
    CHECK(deep.find("b")->as_list()[0].as_int() == 2);         // independent storage
    CHECK(std::string(Data().type_name()) != std::string(Data(1).type_name()));
    CHECK(data_length(Data(DataList{Data(1), Data(2), Data(3)})) == 3);
    CHECK(data_length(Data(at::zeros({5, 2}))) == 5);
}

// ------------------------------------------------------------ file mapper
TEST(file_mapper_lru_and_ranges) {
    TempFile a("a", "AAAAAAAAAA"), b("b", "BBBBBBBBBB"), c("c", "0123456789");
    FileMapper fm(std::nullopt, 2);                               // room for two mappings: the third evicts the first
    for (int round = 0; round < 3; ++round)
        for (const std::string* p : {&a.path, &b.path, &c.path}) {
            Data out = fm(Data(*p));
            CHECK(out.find("path")->as_string() == *p);
            CHECK(out.find("data")->as_memory_block().size() == 10);
        }
    Data r = fm(Data(c.path + ":3:4"));
    const MemoryBlock& blk = r.find("data")->as_memory_block();
    CHECK(blk.size() == 4 && blk.data()[0] == '3' && blk.data()[3] == '6');
    Data tail = fm(Data(c.path + ":8"));
    CHECK(tail.find("data")->as_memory_block().size() == 2);
    CHECK_THROWS(fm(Data(c.path + ":8:5")), std::exception);
    CHECK_THROWS(fm(Data(int64_t{3})), std::invalid_argument);
    CHECK_THROWS(fm(Data(std::string("/nonexistent/fs2d"))), std::exception);
    // a block handed out earlier stays valid after its file left the cache
    Data first = fm(Data(a.path));
    fm(Data(b.path));
    fm(Data(c.path));
    CHECK(first.find("data")->as_memory_block().data()[9] == 'A');
}

TEST(file_mapper_root_dir_and_threads) {
    TempFile a("a", "hello world");
    const size_t slash = a.path.rfind('/');
    FileMapper fm(a.path.substr(0, slash), 1);
    const std::string rel = a.path.substr(slash + 1);
    std::vector<std::thread> ts;
    std::atomic<int> good{0};
    for (int i = 0; i < 8; ++i)
        ts.emplace_back([&] {
            for (int k = 0; k < 50; ++k) {
                Data out = fm(Data(rel + ":6:5"));
                const MemoryBlock& m = out.find("data")->as_memory_block();
                if (m.size() == 5 && m.data()[0] == 'w') ++good;
            }
        });
    for (auto& t : ts) t.join();
    CHECK(good == 400);
}

// --------------------------------------------------------------- collater
TEST(collater_pads_and_stacks) {
    Collater pad(0, 4, {});
    DataList bucket{Data(at::ones({3}, at::kLong)), Data(at::ones({5}, at::kLong))};
    Data out = pad(Data(bucket));
    CHECK(out.is_dict());
    const at::Tensor& seqs = out.find("seqs")->as_tensor();
    CHECK(seqs.size(0) == 2 && seqs.size(1) == 8);               // padded to a multiple of 4
    CHECK(seqs[0][3].item<int64_t>() == 0 && seqs[1][4].item<int64_t>() == 1);
    const DataList& lens = out.find("seq_lens")->as_list();                // plain integers, as the batch types expect
    CHECK(lens.size() == 2 && lens[0].as_int() == 3 && lens[1].as_int() == 5);
    Collater stack(std::nullopt, 1, {});
    Data st = stack(Data(DataList{Data(at::zeros({2, 2})), Data(at::ones({2, 2}))}));
    CHECK(st.is_tensor() && st.as_tensor().size(0) == 2 && st.as_tensor()[1][0][0].item<float>() == 1.f);
    CHECK_THROWS(stack(Data(DataList{Data(at::zeros({2})), Data(at::zeros({3}))})), std::exception);
}

// ------------------------------------------------------------- converters
TEST(string_converters) {
    StrSplitter split('\t', std::nullopt, {}, false);
    Data parts = split(Data(std::string("a\tb\tc")));
    CHECK(parts.is_list() && parts.as_list().size() == 3 && parts.as_list()[2].as_string() == "c");
    StrSplitter named(',', std::vector<std::string>{"x", "y"}, {}, false);
    Data kv = named(Data(std::string("1,2")));
    CHECK(kv.is_dict() && kv.find("y")->as_string() == "2");
    CHECK_THROWS(named(Data(std::string("1,2,3"))), std::exception);
    StrToIntConverter hex(16);
    CHECK(hex(Data(std::string("ff"))).as_int() == 255);
    CHECK_THROWS(hex(Data(std::string("zz"))), std::exception);
    StrToTensorConverter tt(std::nullopt, at::kLong);
    Data t = tt(Data(std::string("4 5 6")));
    CHECK(t.as_tensor().numel() == 3 && t.as_tensor()[2].item<int64_t>() == 6);
}

// -------------------------------------------------------------- pipelines
TEST(pipeline_read_list_round_trip) {
    check_round_trip([] { return read_list(ints(7)).and_return(); });
}

TEST(pipeline_bucket) {
    DataPipeline p = read_list(ints(7)).bucket(3, false).and_return();
    std::vector<size_t> sizes;
    while (auto d = p.next()) sizes.push_back(d->as_list().size());
    CHECK((sizes == std::vector<size_t>{3, 3, 1}));
    DataPipeline q = read_list(ints(7)).bucket(3, true).and_return();
    size_t n = 0;
    while (q.next()) ++n;
    CHECK(n == 2);
}

TEST(pipeline_map_parallel_keeps_order) {
    auto make = [] {
        MapFn sq = [](Data&& d) {
            std::this_thread::sleep_for(std::chrono::microseconds(200 * (d.as_int() % 3)));
            return Data(d.as_int() * d.as_int());
        };
        return read_list(ints(40)).map({sq}, std::nullopt, 4, true).and_return();
    };
    DataPipeline p = make();
    std::vector<int64_t> got = drain(p);
    CHECK(got.size() == 40);
    for (int64_t i = 0; i < 40; ++i) CHECK(got[static_cast<size_t>(i)] == i * i);
    check_round_trip(make);
}

TEST(pipeline_map_error_breaks_pipeline) {
    MapFn bad = [](Data&& d) -> Data {
        if (d.as_int() == 2) throw std::runtime_error("boom");
        return std::move(d);
    };
    DataPipeline p = read_list(ints(5)).map({bad}, std::nullopt, 1, true).and_return();
    CHECK(p.next()->as_int() == 0);
    CHECK(p.next()->as_int() == 1);
    CHECK_THROWS(p.next(), std::exception);
}

TEST(pipeline_filter_skip_take) {
    check_round_trip([] {
        PredicateFn even = [](const Data& d) { return d.as_int() % 2 == 0; };
        return read_list(ints(20)).filter(even).skip(2).take(5).and_return();
    });
    PredicateFn even = [](const Data& d) { return d.as_int() % 2 == 0; };
    DataPipeline p = read_list(ints(20)).filter(even).skip(2).take(5).and_return();
    CHECK((drain(p) == std::vector<int64_t>{4, 6, 8, 10, 12}));
}

TEST(pipeline_shard) {
    for (size_t r = 0; r < 3; ++r) {
        DataPipeline p = read_list(ints(10)).shard(r, 3, false).and_return();
        std::vector<int64_t> got = drain(p);
        CHECK(got.size() == 3);                                   // even shards: the 10th example is dropped
        for (size_t i = 0; i < got.size(); ++i) CHECK(got[i] == static_cast<int64_t>(3 * i + r));
    }
    DataPipeline u = read_list(ints(10)).shard(0, 3, true).and_return();
    CHECK(drain(u).size() == 4);
    check_round_trip([] { return read_list(ints(10)).shard(1, 3, false).and_return(); });
    CHECK_THROWS(read_list(ints(3)).shard(3, 3, false).and_return().next(), std::exception);
}

TEST(pipeline_shuffle_is_seeded_permutation) {
    auto make = [] { return read_list(ints(50)).shuffle(16, 7).and_return(); };
    DataPipeline a = make(), b = make();
    std::vector<int64_t> x = drain(a), y = drain(b);
    CHECK(x == y);
    CHECK(x != iota(50));
    std::vector<int64_t> sorted = x;
    std::sort(sorted.begin(), sorted.end());
    CHECK(sorted == iota(50));
    DataPipeline c = read_list(ints(50)).shuffle(16, 8).and_return();
    CHECK(drain(c) != x);
    check_round_trip(make, /*check_reset=*/false);
    // reset(false) keeps the generator state: the second epoch is another permutation
    DataPipeline d = make();
    std::vector<int64_t> e1 = drain(d);
    d.reset(false);
    std::vector<int64_t> e2 = drain(d);
    CHECK(e1 != e2);
    d.reset(true);
    CHECK(drain(d) == e1);
}

TEST(pipeline_repeat) {
    DataPipeline p = read_list(ints(3)).repeat(2, true).and_return();
    CHECK((drain(p) == std::vector<int64_t>{0, 1, 2, 0, 1, 2}));
    check_round_trip([] { return read_list(ints(3)).repeat(3, true).and_return(); });
    DataPipeline inf = read_list(ints(2)).repeat(std::nullopt, true).and_return();
    CHECK(inf.finitude() != Finitude::Finite);
    for (int i = 0; i < 9; ++i) CHECK(inf.next()->as_int() == i % 2);
}

TEST(pipeline_concat_and_count) {
    auto make = [] {
        return DataPipeline::concat({read_list(ints(3)).and_return(), read_list(ints(2, 10)).and_return()}).and_return();
    };
    DataPipeline p = make();
    CHECK((drain(p) == std::vector<int64_t>{0, 1, 2, 10, 11}));
    check_round_trip(make);
    DataPipeline c = DataPipeline::count(5, 3, std::nullopt).take(4).and_return();
    CHECK((drain(c) == std::vector<int64_t>{5, 8, 11, 14}));
    check_round_trip([] { return DataPipeline::count(5, 3, std::nullopt).take(6).and_return(); });
}

TEST(pipeline_round_robin) {
    auto make = [] {
        return DataPipeline::round_robin({read_list(ints(4)).and_return(), read_list(ints(2, 100)).and_return()}, false,
                                         true)
            .and_return();
    };
    DataPipeline p = make();
    // the shorter pipeline restarts until the longest is exhausted
    CHECK((drain(p) == std::vector<int64_t>{0, 100, 1, 101, 2, 100, 3, 101}));
    check_round_trip(make);
    DataPipeline s = DataPipeline::round_robin({read_list(ints(4)).and_return(), read_list(ints(2, 100)).and_return()},
                                               true, true)
                         .and_return();
    CHECK((drain(s) == std::vector<int64_t>{0, 100, 1, 101}));
}

TEST(pipeline_sample_follows_weights) {
    auto make = [] {
        // repeated without a count: endless for good (a bare `constant` counts as through after one draw)
        return DataPipeline::sample({read_list(DataList{Data(0)}).repeat(std::nullopt, false).and_return(),
                                     read_list(DataList{Data(1)}).repeat(std::nullopt, false).and_return()},
                                    std::vector<float>{0.8f, 0.2f}, 3, true)
            .take(2000)
            .and_return();
    };
    DataPipeline p = make();
    std::vector<int64_t> got = drain(p);
    const double ones = static_cast<double>(std::count(got.begin(), got.end(), 1));
    CHECK(ones / 2000.0 > 0.15 && ones / 2000.0 < 0.25);
    DataPipeline q = make();
    CHECK(drain(q) == got);                                        // seeded
    DataPipeline r = make();
    for (int i = 0; i < 100; ++i) r.next();
    Tape t;
    r.record_position(t);
    std::vector<int64_t> tail = drain(r);
    DataPipeline r2 = make();
    t.rewind();
    r2.reload_position(t);
    CHECK(drain(r2) == tail);
}

TEST(pipeline_zip) {
    DataPipeline z = DataPipeline::zip({read_list(ints(3)).and_return(), read_list(ints(3, 10)).and_return()}, {}, false,
                                       false, true)
                         .and_return();
    int64_t i = 0;
    while (auto d = z.next()) {
        CHECK(d->is_list() && d->as_list()[0].as_int() == i && d->as_list()[1].as_int() == 10 + i);
        ++i;
    }
    CHECK(i == 3);
    DataPipeline named = DataPipeline::zip({read_list(ints(2)).and_return(), read_list(ints(2, 5)).and_return()},
                                           {"a", "b"}, false, false, true)
                             .and_return();
    auto d = named.next();
    CHECK(d->is_dict() && d->find("b")->as_int() == 5);
    DataPipeline uneven = DataPipeline::zip({read_list(ints(2)).and_return(), read_list(ints(3)).and_return()}, {},
                                            false, false, true)
                              .and_return();
    uneven.next();
    uneven.next();
    CHECK_THROWS(uneven.next(), std::exception);
    DataPipeline shortest = DataPipeline::zip({read_list(ints(2)).and_return(), read_list(ints(3)).and_return()}, {},
                                              true, false, true)
                                .and_return();
    size_t n = 0;
    while (shortest.next()) ++n;
    CHECK(n == 2);
}

TEST(pipeline_prefetch_round_trip) {
    check_round_trip([] { return read_list(ints(30)).prefetch(4).and_return(); });
}

TEST(pipeline_yield_from) {
    auto make = [] {
        YieldFn f = [](const Data& d) { return read_list(ints(d.as_int(), d.as_int() * 10)).and_return(); };
        return read_list(ints(4)).yield_from(f).and_return();
    };
    DataPipeline p = make();
    CHECK((drain(p) == std::vector<int64_t>{10, 20, 21, 30, 31, 32}));
    check_round_trip(make);
}

TEST(pipeline_bucket_by_length) {
    DataList items;
    for (int64_t n : {1, 4, 2, 3, 1, 4, 2, 9}) items.emplace_back(at::zeros({n}));
    DataPipeline p = read_list(items).bucket_by_length({{2, 2}, {1, 4}}, std::nullopt, 1, false, true, false).and_return();
    size_t total = 0, buckets = 0;
    while (auto d = p.next()) {
        size_t longest = 0;
        for (const Data& e : d->as_list()) longest = std::max(longest, data_length(e));
        CHECK(longest <= 2 ? d->as_list().size() <= 2 : d->as_list().size() == 1);
        total += d->as_list().size();
        ++buckets;
    }
    CHECK(total == 7 && buckets >= 5);                             // the 9-element example is skipped
    DataPipeline strict = read_list(items).bucket_by_length({{2, 2}, {1, 4}}, std::nullopt, 1, false, false, false)
                              .and_return();
    bool threw = false;
    try {
        while (strict.next()) {
        }
    } catch (const std::exception&) {
        threw = true;
    }
    CHECK(threw);
}

TEST(pipeline_text_reader) {
    TempFile f("text", "  first \n\nsecond\nthird");
    auto make = [&] { return read_text(f.path, std::nullopt, "lf", true, true, true, false, 0).and_return(); };
    DataPipeline p = make();
    std::vector<std::string> lines;
    while (auto d = p.next()) lines.push_back(d->as_string());
    CHECK((lines == std::vector<std::string>{"first", "second", "third"}));
    DataPipeline q = make();
    q.next();
    Tape t;
    q.record_position(t);
    q.next();
    t.rewind();
    q.reload_position(t);
    CHECK(q.next()->as_string() == "second");
    DataPipeline mm = read_text(f.path, std::nullopt, "infer", false, false, false, true, 0).and_return();
    size_t n = 0;
    while (mm.next()) ++n;
    CHECK(n == 4);
}

TEST(pipeline_text_reader_reencodes) {
    // "café" + LF + "naïve" in ISO-8859-1
    TempFile latin("latin1", std::string("caf\xe9\nna\xefve"));
    DataPipeline p = read_text(latin.path, std::nullopt, "infer", false, false, false, false, 0, "ISO-8859-1").and_return();
    CHECK(p.next()->as_string() == "caf\xc3\xa9");
    CHECK(p.next()->as_string() == "na\xc3\xafve");
    CHECK(!p.next().has_value());
    // UTF-16LE with a BOM-less "hi" + LF + U+20AC
    TempFile wide("utf16", std::string("h\0i\0\n\0\xac\x20", 8));
    DataPipeline w = read_text(wide.path, std::nullopt, "infer", false, false, false, true, 0, "UTF-16LE").and_return();
    CHECK(w.next()->as_string() == "hi");
    CHECK(w.next()->as_string() == "\xe2\x82\xac");
    TempFile odd("utf16-truncated", std::string("h\0i", 3));
    // a stream error reaches the caller of the pipeline as a pipeline error, and the pipeline stays broken
    CHECK_THROWS(read_text(odd.path, std::nullopt, "infer", false, false, false, false, 0, "UTF-16LE").and_return().next(),
                 DataPipelineError);
    CHECK_THROWS(read_text(latin.path, std::nullopt, "infer", false, false, false, false, 0, "no-such-charset")
                     .and_return()
                     .next(),
                 std::invalid_argument);
    // UTF-8 spellings bypass the converter
    DataPipeline u = read_text(latin.path, std::nullopt, "infer", false, false, false, false, 0, "utf_8").and_return();
    CHECK(u.next()->as_string() == "caf\xe9");
}

// A serialized SentencePiece model written field by field (protobuf wire format).
struct ProtoWriter {
    std::string out;
    void varint(uint64_t v) {
        while (v >= 0x80) {
            out.push_back(static_cast<char>((v & 0x7f) | 0x80));
            v >>= 7;
        }
        out.push_back(static_cast<char>(v));
    }
    void bytes(int field, const std::string& b) {
        varint(static_cast<uint64_t>(field) << 3 | 2);
        varint(b.size());
        out += b;
    }
    void integer(int field, uint64_t v) {
        varint(static_cast<uint64_t>(field) << 3);
        varint(v);
    }
    void f32(int field, float f) {
        varint(static_cast<uint64_t>(field) << 3 | 5);
        out.append(reinterpret_cast<const char*>(&f), 4);
    }
};

std::string tiny_sentencepiece_model(int model_type, bool byte_fallback) {
    const std::string sp = "\xe2\x96\x81";
    ProtoWriter m;
    auto piece = [&](const std::string& text, float score, int type) {
        ProtoWriter p;
        p.bytes(1, text);
        p.f32(2, score);
        p.integer(3, static_cast<uint64_t>(type));
        m.bytes(1, p.out);
    };
    piece("<unk>", 0.f, 2);
    piece("<s>", 0.f, 3);
    piece("</s>", 0.f, 3);
    piece(sp + "a", -1.0f, 1);
    piece(sp + "b", -1.5f, 1);
    piece("a", -2.0f, 1);
    piece("b", -2.5f, 1);
    piece(sp + "ab", -1.2f, 1);
    piece(sp, -3.0f, 1);
    piece("ab", -2.2f, 1);
    if (byte_fallback)
        for (int b = 0; b < 256; ++b) {
            char name[8];
            std::snprintf(name, sizeof name, "<0x%02X>", b);
            piece(name, 0.f, 6);
        }
    ProtoWriter t;
    t.integer(3, static_cast<uint64_t>(model_type));
    t.integer(35, byte_fallback ? 1 : 0);
    m.bytes(2, t.out);
    ProtoWriter n;
    n.bytes(1, "identity");
    m.bytes(3, n.out);
    return m.out;
}

TEST(sentencepiece_unigram_viterbi_and_decode) {
    SentencePieceModel m(tiny_sentencepiece_model(1, false), {});
    CHECK(m.size() == 10 && m.unk_id() == 0 && m.bos_id() == 1 && m.eos_id() == 2 && m.pad_id() == -1);
    CHECK(m.normalize("  ab   a ") == "\xe2\x96\x81" "ab" "\xe2\x96\x81" "a");
    // "_ab" (-1.2) beats "_a" + "b" (-3.5); the second word is one piece
    CHECK(m.encode("ab a") == (std::vector<int64_t>{7, 3}));
    CHECK(m.decode({1, 7, 3, 2}) == "ab a");
    // an unknown run merges into one unknown token and decodes to the unknown surface
    auto pieces = m.encode_as_pieces("a xyz");
    CHECK(pieces.size() == 3 && pieces[2].second == 0 && pieces[2].first == "xyz");
    CHECK(m.decode({3, 8, 0}) == "a  \xe2\x81\x87 ");
    auto best = m.nbest_encode("ab", 3);
    CHECK(best.size() == 3 && best[0].second >= best[1].second && best[1].second >= best[2].second);
    CHECK(best[0].first.size() == 1 && best[0].first[0].second == 7);
    CHECK_THROWS(m.id_to_piece(99), std::invalid_argument);
    CHECK_THROWS(SentencePieceModel(std::string("\x0a\x05zz"), {}), std::invalid_argument);
}

TEST(sentencepiece_bpe_byte_fallback_and_control_symbols) {
    SentencePieceModel m(tiny_sentencepiece_model(2, true), {"<pad>@0", "<lang>"});
    CHECK(m.size() == 10 + 256 + 2 && m.pad_id() == 0 && m.unk_id() == 1 && m.piece_to_id("<lang>") == 267);
    // merges by score: (_ a) -1.0 first, then (_a b) -1.2
    CHECK(m.encode("ab") == (std::vector<int64_t>{8}));
    // 'z' is unknown: one byte piece; the euro sign: three
    auto ids = m.encode("a z\xe2\x82\xac");
    CHECK(ids.size() == 1 + 1 + 4 && ids[0] == 4 && ids[1] == 9);
    CHECK(m.id_to_piece(static_cast<int>(ids[2])) == "<0x7A>" && m.id_to_piece(static_cast<int>(ids[3])) == "<0xE2>");
    CHECK(m.decode(ids) == "a z\xe2\x82\xac");
    CHECK(m.decode({0, 4, 267}) == "a");
    // a torn multi-byte character decodes to the replacement character
    CHECK(m.decode({ids[3]}) == "\xef\xbf\xbd");
    std::mt19937_64 rng(1);
    SamplingOptions drop;
    drop.alpha = 1.0f;   // every merge dropped: characters only
    CHECK(m.encode("ab", &drop, &rng) == (std::vector<int64_t>{9, 6, 7}));
}

TEST(sentencepiece_encoder_tensor_layout) {
    SentencePieceModel m(tiny_sentencepiece_model(1, false), {});
    SentencePieceEncoder enc(m, {"<s>"}, {"</s>"}, /*reverse=*/true, false, -1, 0.1f, std::nullopt, false, 0);
    at::Tensor t = enc.encode("ab a");
    CHECK(t.scalar_type() == at::kLong && t.numel() == 4);
    // reversed as a whole: </s>, the pieces back to front, <s>
    CHECK(t[0].item<int64_t>() == 2 && t[1].item<int64_t>() == 3 && t[2].item<int64_t>() == 7 && t[3].item<int64_t>() == 1);
    SentencePieceDecoder dec(m, /*reverse=*/true);
    CHECK(dec.decode(t) == "ab a");
    CHECK_THROWS(SentencePieceEncoder(m, {"<nope>"}, {}, false, false, -1, 0.1f, std::nullopt, false, 0),
                 std::invalid_argument);
    Data out = enc(Data(std::string("a")));
    CHECK(out.is_tensor() && out.as_tensor().numel() == 3);
}

TEST(pipeline_broken_after_error_and_reset_recovers_nothing) {
    PredicateFn bad = [](const Data& d) -> bool {
        if (d.as_int() == 1) throw std::runtime_error("boom");
        return true;
    };
    DataPipeline p = read_list(ints(3)).filter(bad).and_return();
    p.next();
    CHECK_THROWS(p.next(), std::exception);
    CHECK(p.is_broken());
    CHECK_THROWS(p.next(), DataPipelineError);
}

}  // namespace

// (name, passed, message) per case
static std::vector<std::tuple<std::string, bool, std::string>> run_all() {
    std::vector<std::tuple<std::string, bool, std::string>> rows;
    for (const Case& c : registry()) {
        try {
            c.fn();
            rows.emplace_back(c.name, true, "");
        } catch (const std::exception& ex) {
            rows.emplace_back(c.name, false, ex.what());
        }
    }
    return rows;
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "C++ unit tests of the fairseq2_b200 native data runtime";
    m.def("run_all", &run_all, pybind11::call_guard<pybind11::gil_scoped_release>());
}
