// Data value type, memory blocks and Python conversions.
#include "data.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstring>
#include <fstream>

namespace fs2d {

// ---------------------------------------------------------------- MemoryBlock
MemoryBlock MemoryBlock::copy_of(const void* src, size_t n) {
    auto buf = std::shared_ptr<uint8_t>(new uint8_t[n > 0 ? n : 1], std::default_delete<uint8_t[]>());
    if (n > 0) std::memcpy(buf.get(), src, n);
    const uint8_t* p = buf.get();
    return MemoryBlock(std::shared_ptr<const void>(buf, p), p, n);
}

namespace {
struct Mapping {
    void* addr;
    size_t len;
    ~Mapping() {
        if (addr != nullptr && addr != MAP_FAILED) ::munmap(addr, len);
    }
};
}  // namespace

MemoryBlock MemoryBlock::map_file(const std::string& path) {
    int fd = ::open(path.c_str(), O_RDONLY | O_CLOEXEC);
    if (fd < 0) throw ByteStreamError("The file '" + path + "' cannot be opened: " + std::strerror(errno));
    struct stat st {};
    if (::fstat(fd, &st) != 0) {
        ::close(fd);
        throw ByteStreamError("The size of '" + path + "' cannot be determined.");
    }
    const size_t n = static_cast<size_t>(st.st_size);
    if (n == 0) {
        ::close(fd);
        return MemoryBlock();
    }
    void* addr = ::mmap(nullptr, n, PROT_READ, MAP_PRIVATE, fd, 0);
    ::close(fd);
    if (addr == MAP_FAILED) throw ByteStreamError("The file '" + path + "' cannot be memory mapped.");
    std::shared_ptr<Mapping> m(new Mapping{addr, n});  // built in place: a temporary would unmap on destruction
    return MemoryBlock(std::shared_ptr<const void>(m, addr), static_cast<const uint8_t*>(addr), n);
}

MemoryBlock MemoryBlock::read_file(const std::string& path) {
    std::ifstream fp(path, std::ios::binary | std::ios::ate);
    if (!fp) throw ByteStreamError("The file '" + path + "' cannot be opened.");
    const std::streamsize n = fp.tellg();
    fp.seekg(0);
    auto buf = std::shared_ptr<uint8_t>(new uint8_t[n > 0 ? n : 1], std::default_delete<uint8_t[]>());
    if (n > 0 && !fp.read(reinterpret_cast<char*>(buf.get()), n))
        throw ByteStreamError("The file '" + path + "' cannot be read.");
    const uint8_t* p = buf.get();
    return MemoryBlock(std::shared_ptr<const void>(buf, p), p, static_cast<size_t>(n));
}

// ----------------------------------------------------------------------- Data
Data Data::deep_copy() const {
    if (is_list()) {
        DataList out;
        out.reserve(as_list().size());
        for (const auto& e : as_list()) out.push_back(e.deep_copy());
        return Data(std::move(out));
    }
    if (is_dict()) {
        DataDict out;
        out.reserve(as_dict().size());
        for (const auto& kv : as_dict()) out.emplace_back(kv.first, kv.second.deep_copy());
        return Data(std::move(out));
    }
    return *this;
}

const char* Data::type_name() const {
    switch (v_.index()) {
        case 0: return "None";
        case 1: return "bool";
        case 2: return "int";
        case 3: return "float";
        case 4: return "str";
        case 5: return "Tensor";
        case 6: return "MemoryBlock";
        case 7: return "list";
        case 8: return "dict";
        default: return "object";
    }
}

size_t data_length(const Data& d) {
    if (d.is_tensor()) {
        const at::Tensor& t = d.as_tensor();
        if (t.dim() == 0) throw std::invalid_argument("The length of a zero-dimensional tensor is undefined.");
        return static_cast<size_t>(t.size(0));
    }
    if (d.is_list()) return d.as_list().size();
    if (d.is_int()) return static_cast<size_t>(d.as_int());
    if (d.is_string()) return d.as_string().size();
    throw std::invalid_argument(std::string("The length of a value of type `") + d.type_name() + "` is undefined.");
}

// ------------------------------------------------------------- py conversions
Data data_from_py(py::handle h) {
    if (h.is_none()) return Data();
    if (py::isinstance<py::bool_>(h)) return Data(h.cast<bool>());
    if (py::isinstance<py::int_>(h)) return Data(h.cast<int64_t>());
    if (py::isinstance<py::float_>(h)) return Data(h.cast<double>());
    if (py::isinstance<py::str>(h)) return Data(h.cast<std::string>());
    if (THPVariable_Check(h.ptr())) return Data(THPVariable_Unpack(h.ptr()));
    if (py::isinstance<MemoryBlock>(h)) return Data(h.cast<MemoryBlock>());
    if (py::isinstance<py::list>(h) || py::isinstance<py::tuple>(h)) {
        // tuples are converted like lists so that native ops can index into them
        DataList out;
        auto seq = py::reinterpret_borrow<py::sequence>(h);
        out.reserve(py::len(seq));
        for (auto item : seq) out.push_back(data_from_py(item));
        return Data(std::move(out));
    }
    if (py::isinstance<py::dict>(h)) {
        auto d = py::reinterpret_borrow<py::dict>(h);
        bool str_keys = true;
        for (auto kv : d)
            if (!py::isinstance<py::str>(kv.first)) {
                str_keys = false;
                break;
            }
        if (str_keys) {
            DataDict out;
            out.reserve(py::len(d));
            for (auto kv : d) out.emplace_back(kv.first.cast<std::string>(), data_from_py(kv.second));
            return Data(std::move(out));
        }
    }
    return Data(PyObjectHolder(py::reinterpret_borrow<py::object>(h)));
}

py::object data_to_py(const Data& d) {
    if (d.is_none()) return py::none();
    if (d.is_bool()) return py::bool_(d.as_bool());
    if (d.is_int()) return py::int_(d.as_int());
    if (d.is_float()) return py::float_(d.as_float());
    if (d.is_string()) return py::str(d.as_string());
    if (d.is_tensor()) return py::reinterpret_steal<py::object>(THPVariable_Wrap(d.as_tensor()));
    if (d.is_memory_block()) return py::cast(d.as_memory_block());
    if (d.is_list()) {
        py::list out;
        for (const auto& e : d.as_list()) out.append(data_to_py(e));
        return std::move(out);
    }
    if (d.is_dict()) {
        py::dict out;
        for (const auto& kv : d.as_dict()) out[py::str(kv.first)] = data_to_py(kv.second);
        return std::move(out);
    }
    return d.as_py().get();
}

}  // namespace fs2d
