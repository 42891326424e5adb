// Memory-mapped safetensors reader: multi-file index by tensor name with dtype/shape checks,
// plus mlock / touch / prefetch of the mapping (role of the reference's src/core/safetensors.cpp).
#pragma once
#include <dirent.h>
#include <algorithm>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <map>
#include <memory>
#include <vector>

#include "json.hpp"

namespace qwh {

struct MappedFile {
    std::string path;
    const uint8_t *data = nullptr;
    size_t size = 0;
    explicit MappedFile(const std::string &p) : path(p) {
        int fd = ::open(p.c_str(), O_RDONLY);
        if (fd < 0) fail("cannot open " + p);
        struct stat st{};
        if (fstat(fd, &st) != 0) { ::close(fd); fail("cannot stat " + p); }
        size = size_t(st.st_size);
        void *m = size ? mmap(nullptr, size, PROT_READ, MAP_SHARED, fd, 0) : nullptr;
        ::close(fd);
        if (size && m == MAP_FAILED) fail("cannot mmap " + p);
        data = static_cast<const uint8_t *>(m);
    }
    ~MappedFile() { if (data) munmap(const_cast<uint8_t *>(data), size); }
    MappedFile(const MappedFile &) = delete;
    bool lock() const { return size == 0 || mlock(data, size) == 0; }
    void prefetch() const { if (size) madvise(const_cast<uint8_t *>(data), size, MADV_WILLNEED); }
    uint64_t touch() const {            // read one byte per page so the file is in the page cache
        uint64_t s = 0;
        for (size_t i = 0; i < size; i += 4096) s += data[i];
        return s;
    }
};

enum class DType { F32, F16, BF16, I32, I64, U8, I8, F8E4M3, Other };
inline size_t dtype_size(DType d) {
    switch (d) { case DType::F32: case DType::I32: return 4; case DType::F16: case DType::BF16: return 2;
                 case DType::I64: return 8; default: return 1; }
}
inline DType dtype_of(const std::string &s) {
    if (s == "F32") return DType::F32; if (s == "F16") return DType::F16; if (s == "BF16") return DType::BF16;
    if (s == "I32") return DType::I32; if (s == "I64") return DType::I64; if (s == "U8") return DType::U8;
    if (s == "I8") return DType::I8; if (s == "F8_E4M3") return DType::F8E4M3;
    return DType::Other;
}

struct TensorView {
    std::string name;
    DType dtype = DType::Other;
    std::vector<int64_t> shape;
    const uint8_t *data = nullptr;
    size_t nbytes = 0;
    int64_t numel() const { int64_t n = 1; for (auto d : shape) n *= d; return n; }
    int64_t dim(size_t i) const { QWH_CHECK(i < shape.size(), name + ": dim"); return shape[i]; }
};

class SafeTensors {
public:
    void add_file(const std::string &path) {
        auto f = std::make_shared<MappedFile>(path);
        QWH_CHECK(f->size >= 8, path + ": too short");
        uint64_t hlen;
        std::memcpy(&hlen, f->data, 8);
        QWH_CHECK(8 + hlen <= f->size, path + ": bad header length");
        Json h = Json::parse(std::string(reinterpret_cast<const char *>(f->data + 8), size_t(hlen)));
        const uint8_t *base = f->data + 8 + hlen;
        for (auto &kv : h.obj) {
            if (kv.first == "__metadata__") continue;
            TensorView t;
            t.name = kv.first;
            t.dtype = dtype_of(kv.second["dtype"].as_str());
            for (auto &d : kv.second["shape"].arr) t.shape.push_back(d.as_int());
            const int64_t b = kv.second["data_offsets"][0].as_int(), e = kv.second["data_offsets"][1].as_int();
            QWH_CHECK(b >= 0 && e >= b && size_t(8 + hlen + e) <= f->size, path + ": " + t.name + " out of range");
            t.data = base + b;
            t.nbytes = size_t(e - b);
            QWH_CHECK(t.dtype == DType::Other || t.nbytes == size_t(t.numel()) * dtype_size(t.dtype), t.name + ": size/shape mismatch");
            tensors_[t.name] = t;
        }
        files_.push_back(f);
    }
    bool has(const std::string &n) const { return tensors_.count(n) != 0; }
    // every *.safetensors file of a directory, in name order
    void add_dir(const std::string &dir) {
        std::vector<std::string> files;
        if (DIR *d = opendir(dir.c_str())) {
            while (dirent *e = readdir(d)) {
                const std::string n = e->d_name;
                if (n.size() > 12 && n.compare(n.size() - 12, 12, ".safetensors") == 0) files.push_back(dir + "/" + n);
            }
            closedir(d);
        }
        QWH_CHECK(!files.empty(), dir + ": no .safetensors files");
        std::sort(files.begin(), files.end());
        for (auto &f : files) add_file(f);
    }

    const TensorView &get(const std::string &n) const {
        auto it = tensors_.find(n);
        if (it == tensors_.end()) fail("tensor not found: " + n);
        return it->second;
    }
    const TensorView &get(const std::string &n, DType d, const std::vector<int64_t> &shape) const {
        const TensorView &t = get(n);
        QWH_CHECK(t.dtype == d, n + ": unexpected dtype");
        QWH_CHECK(t.shape == shape, n + ": unexpected shape");
        return t;
    }
    const std::vector<std::shared_ptr<MappedFile>> &files() const { return files_; }
    size_t count() const { return tensors_.size(); }
    std::vector<std::string> names() const { std::vector<std::string> v; for (auto &kv : tensors_) v.push_back(kv.first); return v; }

private:
    std::map<std::string, TensorView> tensors_;
    std::vector<std::shared_ptr<MappedFile>> files_;
};

}  // namespace qwh
