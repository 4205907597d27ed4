// Python surface of the native data pipeline runtime (module fairseq2_b200._data).
#include <pybind11/functional.h>
#include <pybind11/stl.h>

#include "extras.h"

namespace py = pybind11;
using namespace fs2d;

namespace pybind11::detail {
// Data <-> Python object
template <>
struct type_caster<Data> {
    PYBIND11_TYPE_CASTER(Data, const_name("Any"));
    bool load(handle src, bool) {
        value = data_from_py(src);
        return true;
    }
    static handle cast(const Data& d, return_value_policy, handle) { return data_to_py(d).release(); }
};
}  // namespace pybind11::detail

namespace {

// Wraps a Python callable so that it can be invoked from any thread.
struct PyCallable {
    std::shared_ptr<py::object> fn;
    explicit PyCallable(py::object f) : fn(new py::object(std::move(f)), [](py::object* p) {
        py::gil_scoped_acquire gil;
        delete p;
    }) {}
};

MapFn as_map_fn(py::object o) {
    // native callables (Collater, FileMapper, converters...) run without the GIL
    if (py::isinstance<Collater>(o)) {
        auto c = o.cast<Collater>();
        return [c](Data&& d) { return c(std::move(d)); };
    }
    if (py::isinstance<FileMapper>(o)) {
        auto c = o.cast<FileMapper>();
        return [c](Data&& d) { return c(std::move(d)); };
    }
    if (py::isinstance<StrSplitter>(o)) {
        auto c = o.cast<StrSplitter>();
        return [c](Data&& d) { return c(std::move(d)); };
    }
    if (py::isinstance<StrToIntConverter>(o)) {
        auto c = o.cast<StrToIntConverter>();
        return [c](Data&& d) { return c(std::move(d)); };
    }
    if (py::isinstance<StrToTensorConverter>(o)) {
        auto c = o.cast<StrToTensorConverter>();
        return [c](Data&& d) { return c(std::move(d)); };
    }
    if (py::isinstance<AudioDecoder>(o)) {
        auto c = o.cast<AudioDecoder>();
        return [c](Data&& d) { return c(std::move(d)); };
    }
    if (py::isinstance<WaveformToFbankConverter>(o)) {
        auto c = o.cast<WaveformToFbankConverter>();
        return [c](Data&& d) { return c(std::move(d)); };
    }
    if (py::isinstance<ImageDecoder>(o)) {
        auto c = o.cast<ImageDecoder>();
        return [c](Data&& d) { return c(std::move(d)); };
    }
    if (py::isinstance<SentencePieceEncoder>(o)) {
        auto c = o.cast<SentencePieceEncoder>();
        return [c](Data&& d) { return c(std::move(d)); };
    }
    if (py::isinstance<SentencePieceDecoder>(o)) {
        auto c = o.cast<SentencePieceDecoder>();
        return [c](Data&& d) { return c(std::move(d)); };
    }
    PyCallable pc(std::move(o));
    return [pc](Data&& d) {
        py::gil_scoped_acquire gil;
        return data_from_py((*pc.fn)(data_to_py(d)));
    };
}

at::ScalarType dtype_from_py(const py::object& o) {
    return torch::python::detail::py_object_to_dtype(o);
}

struct PipelineIterator {
    DataPipeline* p;
};

py::dict state_dict(const DataPipeline& p, bool strict) {
    Tape t;
    {
        py::gil_scoped_release nogil;
        p.record_position(t, strict);
    }
    py::list pos;
    for (const auto& d : t.storage()) pos.append(data_to_py(d));
    py::dict out;
    out["position"] = pos;
    return out;
}

void load_state_dict(DataPipeline& p, const py::dict& sd) {
    if (!sd.contains("position")) throw std::invalid_argument("`state_dict` must contain a 'position' key.");
    py::object pos = sd["position"];
    if (!py::isinstance<py::list>(pos))
        throw std::invalid_argument("`state_dict['position']` must be a list.");
    DataList items;
    for (auto h : pos.cast<py::list>()) items.push_back(data_from_py(h));
    Tape t(std::move(items));
    {
        py::gil_scoped_release nogil;
        p.reload_position(t, true);
    }
    if (!t.at_end()) throw std::invalid_argument("`state_dict` does not belong to this data pipeline (trailing entries).");
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "fairseq2_b200 native data pipeline";

    py::register_exception<DataPipelineError>(m, "DataPipelineError", PyExc_RuntimeError);
    py::register_exception<ByteStreamError>(m, "ByteStreamError", PyExc_RuntimeError);
    py::register_exception<RecordError>(m, "RecordError", PyExc_RuntimeError);

    py::class_<MemoryBlock>(m, "MemoryBlock", py::buffer_protocol())
        .def(py::init<>())
        .def(py::init([](py::buffer b, bool copy) {
            // Shares the exporter's bytes unless a copy is asked for: the buffer view stays held, which
            // keeps the exporter alive and unresizable, and is released under the GIL with the last reference.
            auto info = std::make_unique<py::buffer_info>(b.request());
            const size_t n = static_cast<size_t>(info->size * info->itemsize);
            if (info->view() != nullptr && PyBuffer_IsContiguous(info->view(), 'C') == 0)
                throw std::invalid_argument("`buffer` must be contiguous in memory.");
            if (copy) return MemoryBlock::copy_of(info->ptr, n);
            const auto* data = static_cast<const uint8_t*>(info->ptr);
            std::shared_ptr<const void> owner(info.release(), [](const void* held) {
                py::gil_scoped_acquire gil;
                delete static_cast<const py::buffer_info*>(held);
            });
            return MemoryBlock(std::move(owner), data, n);
        }), py::arg("buffer"), py::arg("copy") = false)
        .def("__reduce_ex__", [](py::object self, int protocol) {
            // protocol 5 hands the bytes over as a PickleBuffer (out-of-band capable), older ones as bytes
            py::object cls = self.attr("__class__");
            if (protocol >= 5)
                return py::make_tuple(cls, py::make_tuple(py::module_::import("pickle").attr("PickleBuffer")(self)));
            return py::make_tuple(cls, py::make_tuple(py::bytes(self)));
        })
        .def("__len__", &MemoryBlock::size)
        .def("__bytes__", [](const MemoryBlock& b) {
            return py::bytes(reinterpret_cast<const char*>(b.data()), b.size());
        })
        .def_buffer([](MemoryBlock& b) {
            return py::buffer_info(const_cast<uint8_t*>(b.data()), 1, py::format_descriptor<uint8_t>::format(), 1,
                                   {b.size()}, {1}, /*readonly=*/true);
        });

    py::class_<DataPipeline>(m, "DataPipeline")
        .def(py::init<>())
        .def("__iter__", [](DataPipeline& p) { return PipelineIterator{&p}; }, py::keep_alive<0, 1>())
        .def("reset", [](DataPipeline& p, bool reset_rng) {
            py::gil_scoped_release nogil;
            p.reset(reset_rng);
        }, py::arg("reset_rng") = false)
        .def_property_readonly("is_broken", &DataPipeline::is_broken)
        .def("is_infinite", [](const DataPipeline& p) { return p.finitude() != Finitude::Finite; })
        .def("state_dict", &state_dict, py::arg("strict") = true)
        .def("load_state_dict", &load_state_dict)
        .def_static("constant", [](Data example, std::optional<std::string> key) {
            return DataPipeline::constant(std::move(example), std::move(key));
        }, py::arg("example"), py::arg("key") = py::none())
        .def_static("count", &DataPipeline::count, py::arg("start") = 0, py::arg("step") = 1, py::arg("key") = py::none())
        .def_static("concat", &DataPipeline::concat, py::arg("pipelines"))
        .def_static("round_robin", &DataPipeline::round_robin, py::arg("pipelines"), py::arg("stop_at_shortest") = false,
                    py::arg("allow_repeats") = true)
        .def_static("sample", &DataPipeline::sample, py::arg("pipelines"), py::arg("weights") = py::none(),
                    py::arg("seed") = py::none().is_none() ? 0 : 0, py::arg("allow_repeats") = true)
        .def_static("zip", &DataPipeline::zip, py::arg("pipelines"), py::arg("names") = std::vector<std::string>{},
                    py::arg("zip_to_shortest") = false, py::arg("flatten") = false,
                    py::arg("disable_parallelism") = false);

    py::class_<PipelineIterator>(m, "_DataPipelineIterator")
        .def("__iter__", [](PipelineIterator& it) { return it; })
        .def("__next__", [](PipelineIterator& it) {
            std::optional<Data> d;
            {
                py::gil_scoped_release nogil;
                d = it.p->next();
            }
            if (!d) throw py::stop_iteration();
            return std::move(*d);
        });

    py::class_<DataPipelineBuilder>(m, "DataPipelineBuilder")
        .def("bucket", [](DataPipelineBuilder& b, size_t n, bool drop) -> DataPipelineBuilder& {
            b = std::move(b).bucket(n, drop);
            return b;
        }, py::arg("bucket_size"), py::arg("drop_remainder") = false, py::return_value_policy::reference_internal)
        .def("bucket_by_length", [](DataPipelineBuilder& b, std::vector<std::pair<size_t, size_t>> sizes,
                                    std::optional<std::string> selector, size_t min_len, bool skip_below,
                                    bool skip_above, bool drop) -> DataPipelineBuilder& {
            b = std::move(b).bucket_by_length(std::move(sizes), std::move(selector), min_len, skip_below, skip_above, drop);
            return b;
        }, py::arg("bucket_sizes"), py::arg("selector") = py::none(), py::arg("min_data_len") = 1,
           py::arg("skip_below_min_examples") = false, py::arg("skip_above_max_examples") = false,
           py::arg("drop_remainder") = false, py::return_value_policy::reference_internal)
        .def("collate", [](DataPipelineBuilder& b, std::optional<int64_t> pad_value, int64_t pad_to_multiple,
                           std::optional<std::vector<CollateOverride>> overrides, size_t npc) -> DataPipelineBuilder& {
            Collater c(pad_value, pad_to_multiple, overrides.value_or(std::vector<CollateOverride>{}));
            b = std::move(b).map({[c](Data&& d) { return c(std::move(d)); }}, std::nullopt, npc, true);
            return b;
        }, py::arg("pad_value") = py::none(), py::arg("pad_to_multiple") = 1, py::arg("overrides") = py::none(),
           py::arg("num_parallel_calls") = 1, py::return_value_policy::reference_internal)
        .def("dynamic_bucket", [](DataPipelineBuilder& b, double threshold, py::object cost_fn,
                                  std::optional<py::object> creation_fn, std::optional<size_t> min_n,
                                  std::optional<size_t> max_n, bool drop) -> DataPipelineBuilder& {
            PyCallable cost(std::move(cost_fn));
            CostFn cf = [cost](const Data& d) {
                py::gil_scoped_acquire gil;
                return (*cost.fn)(data_to_py(d)).cast<double>();
            };
            std::optional<BucketCreationFn> bf;
            if (creation_fn && !creation_fn->is_none()) {
                PyCallable cr(std::move(*creation_fn));
                bf = [cr](DataList&& items) -> std::optional<std::pair<DataList, DataList>> {
                    py::gil_scoped_acquire gil;
                    py::object res = (*cr.fn)(data_to_py(Data(std::move(items))));
                    auto tup = res.cast<py::tuple>();
                    Data a = data_from_py(tup[0]), r = data_from_py(tup[1]);
                    return std::make_pair(a.as_list(), r.as_list());
                };
            }
            b = std::move(b).dynamic_bucket(threshold, std::move(cf), std::move(bf), min_n, max_n, drop);
            return b;
        }, py::arg("threshold"), py::arg("cost_fn"), py::arg("bucket_creation_fn") = py::none(),
           py::arg("min_num_examples") = py::none(), py::arg("max_num_examples") = py::none(),
           py::arg("drop_remainder") = false, py::return_value_policy::reference_internal)
        .def("filter", [](DataPipelineBuilder& b, py::object fn) -> DataPipelineBuilder& {
            PyCallable pc(std::move(fn));
            b = std::move(b).filter([pc](const Data& d) {
                py::gil_scoped_acquire gil;
                return (*pc.fn)(data_to_py(d)).cast<bool>();
            });
            return b;
        }, py::arg("predicate"), py::return_value_policy::reference_internal)
        .def("map", [](DataPipelineBuilder& b, py::object fn, std::optional<std::string> selector, size_t npc,
                       bool deterministic) -> DataPipelineBuilder& {
            std::vector<MapFn> fns;
            if (py::isinstance<py::list>(fn) || py::isinstance<py::tuple>(fn)) {
                for (auto f : fn) fns.push_back(as_map_fn(py::reinterpret_borrow<py::object>(f)));
            } else {
                fns.push_back(as_map_fn(std::move(fn)));
            }
            b = std::move(b).map(std::move(fns), std::move(selector), npc, deterministic);
            return b;
        }, py::arg("fn"), py::arg("selector") = py::none(), py::arg("num_parallel_calls") = 1,
           py::arg("deterministic") = true, py::return_value_policy::reference_internal)
        .def("pack", [](DataPipelineBuilder& b, int64_t num_elements, int64_t max_seq_len, int64_t pad_value,
                        bool truncate, bool drop, bool pinned) -> DataPipelineBuilder& {
            b = std::move(b).pack(num_elements, max_seq_len, pad_value, truncate, drop, pinned);
            return b;
        }, py::arg("num_elements"), py::arg("max_seq_len"), py::arg("pad_value") = 0, py::arg("truncate") = true,
           py::arg("drop_remainder") = true, py::arg("pinned_memory") = false,
           py::return_value_policy::reference_internal)
        .def("prefetch", [](DataPipelineBuilder& b, size_t n) -> DataPipelineBuilder& {
            b = std::move(b).prefetch(n);
            return b;
        }, py::arg("num_examples"), py::return_value_policy::reference_internal)
        .def("repeat", [](DataPipelineBuilder& b, std::optional<size_t> n, bool reset_rng) -> DataPipelineBuilder& {
            b = std::move(b).repeat(n, reset_rng);
            return b;
        }, py::arg("num_repeats") = py::none(), py::arg("reset_rng") = false,
           py::return_value_policy::reference_internal)
        .def("shard", [](DataPipelineBuilder& b, size_t idx, size_t n, bool uneven) -> DataPipelineBuilder& {
            b = std::move(b).shard(idx, n, uneven);
            return b;
        }, py::arg("shard_idx"), py::arg("num_shards"), py::arg("allow_uneven") = false,
           py::return_value_policy::reference_internal)
        .def("shuffle", [](DataPipelineBuilder& b, size_t window, uint64_t seed) -> DataPipelineBuilder& {
            b = std::move(b).shuffle(window, seed);
            return b;
        }, py::arg("shuffle_window"), py::arg("seed") = 0, py::return_value_policy::reference_internal)
        .def("skip", [](DataPipelineBuilder& b, size_t n) -> DataPipelineBuilder& {
            b = std::move(b).skip(n);
            return b;
        }, py::arg("num_examples"), py::return_value_policy::reference_internal)
        .def("take", [](DataPipelineBuilder& b, size_t n) -> DataPipelineBuilder& {
            b = std::move(b).take(n);
            return b;
        }, py::arg("num_examples"), py::return_value_policy::reference_internal)
        .def("yield_from", [](DataPipelineBuilder& b, py::object fn) -> DataPipelineBuilder& {
            PyCallable pc(std::move(fn));
            b = std::move(b).yield_from([pc](const Data& d) {
                py::gil_scoped_acquire gil;
                return (*pc.fn)(data_to_py(d)).cast<DataPipeline>();
            });
            return b;
        }, py::arg("fn"), py::return_value_policy::reference_internal)
        .def("and_return", [](DataPipelineBuilder& b, size_t max_num_warnings) {
            return std::move(b).and_return(max_num_warnings);
        }, py::arg("max_num_warnings") = 0);

    py::class_<CollateOverride>(m, "CollateOptionsOverride")
        .def(py::init([](std::string selector, std::optional<int64_t> pad_value, int64_t pad_to_multiple) {
            return CollateOverride{std::move(selector), pad_value, pad_to_multiple};
        }), py::arg("selector"), py::arg("pad_value") = py::none(), py::arg("pad_to_multiple") = 1)
        .def_readonly("selector", &CollateOverride::selector)
        .def_readonly("pad_value", &CollateOverride::pad_value)
        .def_readonly("pad_to_multiple", &CollateOverride::pad_to_multiple);

    py::class_<Collater>(m, "Collater")
        .def(py::init([](std::optional<int64_t> pad_value, int64_t pad_to_multiple,
                         std::optional<std::vector<CollateOverride>> overrides) {
            return Collater(pad_value, pad_to_multiple, overrides.value_or(std::vector<CollateOverride>{}));
        }), py::arg("pad_value") = py::none(), py::arg("pad_to_multiple") = 1, py::arg("overrides") = py::none())
        .def("__call__", [](const Collater& c, Data d) { return c(std::move(d)); });

    py::class_<FileMapper>(m, "FileMapper")
        .def(py::init([](std::optional<py::object> root, std::optional<size_t> n) {
            std::optional<std::string> r;
            if (root && !root->is_none()) r = py::str(*root).cast<std::string>();
            return FileMapper(r, n.value_or(0));
        }), py::arg("root_dir") = py::none(), py::arg("cached_fd_count") = py::none())
        .def("__call__", [](const FileMapper& f, Data d) { return f(std::move(d)); });

    py::class_<StrSplitter>(m, "StrSplitter")
        .def(py::init([](const std::string& sep, std::optional<std::vector<std::string>> names,
                         std::optional<py::object> indices, bool exclude) {
            if (sep.size() != 1) throw std::invalid_argument("`sep` must be of length 1.");
            std::vector<size_t> idx;
            bool single = false;
            if (indices && !indices->is_none()) {
                single = py::isinstance<py::int_>(*indices);
                if (single) idx.push_back(indices->cast<size_t>());
                else idx = indices->cast<std::vector<size_t>>();
            }
            return StrSplitter(sep[0], std::move(names), std::move(idx), exclude, single);
        }), py::arg("sep") = "\t", py::arg("names") = py::none(), py::arg("indices") = py::none(),
           py::arg("exclude") = false)
        .def("__call__", [](const StrSplitter& s, Data d) { return s(std::move(d)); });

    py::class_<StrToIntConverter>(m, "StrToIntConverter")
        .def(py::init<int>(), py::arg("base") = 10)
        .def("__call__", [](const StrToIntConverter& s, Data d) { return s(std::move(d)); });

    py::class_<StrToTensorConverter>(m, "StrToTensorConverter")
        .def(py::init([](std::optional<std::vector<int64_t>> size, std::optional<py::object> dtype) {
            at::ScalarType dt = at::kInt;
            if (dtype && !dtype->is_none()) dt = dtype_from_py(*dtype);
            return StrToTensorConverter(std::move(size), dt);
        }), py::arg("size") = py::none(), py::arg("dtype") = py::none())
        .def("__call__", [](const StrToTensorConverter& s, Data d) { return s(std::move(d)); });

    py::class_<AudioDecoder>(m, "AudioDecoder")
        .def(py::init([](bool keepdim, std::optional<py::object> dtype) {
            std::optional<at::ScalarType> dt;
            if (dtype && !dtype->is_none()) dt = dtype_from_py(*dtype);
            return AudioDecoder(keepdim, dt);
        }), py::arg("keepdim") = false, py::arg("dtype") = py::none())
        .def("__call__", [](const AudioDecoder& a, Data d) { return a(std::move(d)); });

    py::class_<WaveformToFbankConverter>(m, "WaveformToFbankConverter")
        .def(py::init([](int bins, float scale, bool channel_last, bool standardize, bool keep_waveform,
                         std::optional<py::object> dtype) {
            std::optional<at::ScalarType> dt;
            if (dtype && !dtype->is_none()) dt = dtype_from_py(*dtype);
            return WaveformToFbankConverter(bins, scale, channel_last, standardize, keep_waveform, dt);
        }), py::arg("num_mel_bins") = 80, py::arg("waveform_scale") = 1.0f, py::arg("channel_last") = false,
           py::arg("standardize") = false, py::arg("keep_waveform") = false, py::arg("dtype") = py::none())
        .def("__call__", [](const WaveformToFbankConverter& a, Data d) { return a(std::move(d)); });

    py::class_<ImageDecoder>(m, "ImageDecoder")
        .def(py::init([](std::optional<std::string> device, bool pin_memory) {
            std::optional<at::Device> dev;
            if (device) dev = at::Device(*device);
            return ImageDecoder(dev, pin_memory);
        }), py::arg("device") = py::none(), py::arg("pin_memory") = false)
        .def("__call__", [](const ImageDecoder& a, Data d) { return a(std::move(d)); });

    py::class_<SentencePieceModel>(m, "SentencePieceModel")
        .def(py::init([](py::object path, std::vector<std::string> control_symbols) {
            return SentencePieceModel::from_file(py::str(path).cast<std::string>(), control_symbols);
        }), py::arg("path"), py::arg("control_symbols") = std::vector<std::string>{})
        .def_static("from_serialized", [](py::bytes blob, std::vector<std::string> control_symbols) {
            std::string s = blob;
            return SentencePieceModel(s, control_symbols);
        }, py::arg("serialized"), py::arg("control_symbols") = std::vector<std::string>{})
        .def_property_readonly("vocabulary_size", &SentencePieceModel::size)
        .def_property_readonly("unk_idx", &SentencePieceModel::unk_id)
        .def_property_readonly("bos_idx", [](const SentencePieceModel& s) -> std::optional<int> {
            return s.bos_id() < 0 ? std::nullopt : std::optional<int>(s.bos_id());
        })
        .def_property_readonly("eos_idx", [](const SentencePieceModel& s) -> std::optional<int> {
            return s.eos_id() < 0 ? std::nullopt : std::optional<int>(s.eos_id());
        })
        .def_property_readonly("pad_idx", [](const SentencePieceModel& s) -> std::optional<int> {
            return s.pad_id() < 0 ? std::nullopt : std::optional<int>(s.pad_id());
        })
        .def("token_to_index", [](const SentencePieceModel& s, const std::string& t) { return s.piece_to_id(t); })
        .def("index_to_token", [](const SentencePieceModel& s, int i) { return s.id_to_piece(i); })
        .def("is_control", &SentencePieceModel::is_control)
        .def("normalize", [](const SentencePieceModel& s, const std::string& t) { return s.normalize(t); })
        .def("encode", [](const SentencePieceModel& s, const std::string& t) { return s.encode(t); })
        .def("encode_as_tokens", [](const SentencePieceModel& s, const std::string& t) {
            std::vector<std::string> out;
            for (auto& p : s.encode_as_pieces(t)) out.push_back(std::move(p.first));
            return out;
        })
        .def("nbest_encode", [](const SentencePieceModel& s, const std::string& t, size_t n) {
            std::vector<std::pair<std::vector<int>, float>> out;
            for (auto& r : s.nbest_encode(t, n)) {
                std::vector<int> ids;
                for (auto& p : r.first) ids.push_back(p.second);
                out.emplace_back(std::move(ids), r.second);
            }
            return out;
        })
        .def("decode", [](const SentencePieceModel& s, const std::vector<int64_t>& ids) { return s.decode(ids); })
        .def("decode_from_tokens", [](const SentencePieceModel& s, const std::vector<std::string>& toks) {
            return s.decode_tokens(toks);
        });

    py::class_<SentencePieceEncoder>(m, "SentencePieceEncoder")
        .def(py::init([](SentencePieceModel model, std::vector<std::string> prefix, std::vector<std::string> suffix,
                         bool reverse, bool enable_sampling, int nbest_size, float alpha,
                         std::optional<std::string> device, bool pin_memory, uint64_t seed) {
            std::optional<at::Device> dev;
            if (device) dev = at::Device(*device);
            return SentencePieceEncoder(std::move(model), std::move(prefix), std::move(suffix), reverse,
                                        enable_sampling, nbest_size, alpha, dev, pin_memory, seed);
        }), py::arg("model"), py::arg("prefix_tokens") = std::vector<std::string>{},
           py::arg("suffix_tokens") = std::vector<std::string>{}, py::arg("reverse") = false,
           py::arg("enable_sampling") = false, py::arg("nbest_size") = -1, py::arg("alpha") = 0.1f,
           py::arg("device") = py::none(), py::arg("pin_memory") = false, py::arg("seed") = 0)
        .def("__call__", [](const SentencePieceEncoder& e, const std::string& text) { return e.encode(text); })
        .def("encode_as_tokens", [](const SentencePieceEncoder& e, const std::string& text) {
            return e.encode_as_tokens(text);
        });

    py::class_<SentencePieceDecoder>(m, "SentencePieceDecoder")
        .def(py::init<SentencePieceModel, bool>(), py::arg("model"), py::arg("reverse") = false)
        .def("__call__", [](const SentencePieceDecoder& d, const at::Tensor& t) { return d.decode(t); });

    m.def("read_sequence", [](py::sequence seq) {
        DataList items;
        for (auto h : seq) items.push_back(data_from_py(h));
        return read_list(std::move(items));
    }, py::arg("seq"));
    m.def("list_files", [](py::object path, std::optional<std::string> pattern) {
        return list_files(py::str(path).cast<std::string>(), std::move(pattern));
    }, py::arg("path"), py::arg("pattern") = py::none());
    m.def("read_zipped_records", [](py::object path) {
        return read_zipped_records(py::str(path).cast<std::string>());
    }, py::arg("path"));
    m.def("read_text", [](py::object path, std::optional<std::string> key, std::optional<std::string> encoding,
                          const std::string& line_ending, bool ltrim, bool rtrim, bool skip_empty, bool memory_map,
                          std::optional<size_t> block_size) {
        return read_text(py::str(path).cast<std::string>(), std::move(key), line_ending, ltrim, rtrim, skip_empty,
                         memory_map, block_size.value_or(0), std::move(encoding));
    }, py::arg("path"), py::arg("key") = py::none(), py::arg("encoding") = py::none(),
       py::arg("line_ending") = "infer", py::arg("ltrim") = false, py::arg("rtrim") = false,
       py::arg("skip_empty") = false, py::arg("memory_map") = false, py::arg("block_size") = py::none());
    m.def("read_iterator", [](py::object iterator, py::object reset_fn, bool infinite, bool skip_pickling_check) {
        if (!skip_pickling_check) {
            try {
                py::module_::import("pickle").attr("dumps")(iterator);
            } catch (py::error_already_set&) {
                throw py::type_error(
                    "`iterator` is not pickleable; set `skip_pickling_check` to True to bypass (see `read_iterator` documentation for details).");
            }
        }
        return read_py_iterator(std::move(iterator), std::move(reset_fn), infinite);
    }, py::arg("iterator"), py::arg("reset_fn"), py::arg("infinite"), py::arg("skip_pickling_check") = false);
}
