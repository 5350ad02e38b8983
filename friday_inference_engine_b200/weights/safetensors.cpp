// The safetensors container (reader, writer), sharded checkpoints, and the comparison of
// a model's declared tensors with a source's (weights.h).
#include <errno.h>
#include <fcntl.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <fstream>
#include <set>
#include <sstream>

#include "friday/ops.h"
#include "friday/weights.h"
#include "weights/upload.h"

namespace friday {

size_t stored_dtype_size(const std::string& d) {
    if (d == "F64" || d == "I64") return 8;
    if (d == "F32" || d == "I32") return 4;
    if (d == "BF16" || d == "F16" || d == "I16") return 2;
    if (d == "I8" || d == "U8" || d == "BOOL") return 1;
    return 0;
}
bool stored_dtype_is_float(const std::string& d) { return d == "F64" || d == "F32" || d == "BF16" || d == "F16"; }
bool stored_dtype_is_32bit_float(const std::string& d) { return d == "F64" || d == "F32"; }

// ------------------------------------------------------------------ one file
SafetensorsFile::SafetensorsFile(const std::string& path) : path_(path) {
    int fd = open(path.c_str(), O_RDONLY);
    if (fd < 0) throw WeightsError(path + ": cannot open: " + strerror(errno));
    struct stat st;
    fstat(fd, &st);
    size_ = (size_t)st.st_size;
    if (size_ < 8) {
        close(fd);
        throw WeightsError(path + ": too short to be a safetensors file");
    }
    map_ = mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (map_ == MAP_FAILED) {
        map_ = nullptr;
        throw WeightsError(path + ": cannot map the file: " + strerror(errno));
    }
    uint64_t n = 0;
    memcpy(&n, map_, 8);
    if (n == 0 || 8 + n > size_)
        throw WeightsError(format("%s: header length %llu does not fit the file (%zu bytes)", path.c_str(),
                                  (unsigned long long)n, size_));
    base_ = 8 + (size_t)n;
    Json header;
    try {
        header = Json::parse(std::string((const char*)map_ + 8, (size_t)n));
    } catch (const std::invalid_argument& e) {
        throw WeightsError(path + ": header is not JSON: " + e.what());
    }
    if (!header.is_object()) throw WeightsError(path + ": header is not a JSON object");
    for (const auto& m : header.members()) {
        if (m.first == "__metadata__") {
            metadata_ = m.second;
            continue;
        }
        const Json& info = m.second;
        Entry e;
        try {
            e.t.dtype = info.at("dtype").as_string();
            for (const Json& s : info.at("shape").items()) e.t.shape.push_back(s.as_int());
            e.lo = (size_t)info.at("data_offsets")[0].as_int();
            e.hi = (size_t)info.at("data_offsets")[1].as_int();
        } catch (const std::exception&) {
            throw WeightsError(path + ": tensor '" + m.first + "' has a malformed header entry");
        }
        const size_t es = stored_dtype_size(e.t.dtype);
        if (es == 0) throw WeightsError(path + ": tensor '" + m.first + "' has dtype " + e.t.dtype + ", which is not supported");
        if (e.hi < e.lo || e.hi - e.lo != (size_t)e.t.numel() * es || base_ + e.hi > size_)
            throw WeightsError(path + ": tensor '" + m.first + "' has a byte range that does not match its shape");
        entries_[m.first] = e;
        order_.push_back(m.first);
    }
}

SafetensorsFile::~SafetensorsFile() {
    if (map_) munmap(map_, size_);
}

bool SafetensorsFile::info(const std::string& name, StoredTensor* out) const {
    auto it = entries_.find(name);
    if (it == entries_.end()) return false;
    if (out) *out = it->second.t;
    return true;
}

const void* SafetensorsFile::bytes(const std::string& name, size_t* n) const {
    auto it = entries_.find(name);
    if (it == entries_.end()) return nullptr;
    if (n) *n = it->second.hi - it->second.lo;
    return (const char*)map_ + base_ + it->second.lo;
}

// ------------------------------------------------------------------ conversions on the host
namespace {

class SafetensorsSource : public WeightSource {
public:
    // single file
    explicit SafetensorsSource(const std::string& path) : where_(path) {
        files_.emplace_back(new SafetensorsFile(path));
        for (const auto& n : files_[0]->names()) {
            file_of_[n] = 0;
            order_.push_back(n);
        }
    }
    // an index and its shards
    SafetensorsSource(const std::string& dir, const std::string& index_path) : where_(index_path) {
        std::ifstream f(index_path);
        std::stringstream ss;
        ss << f.rdbuf();
        Json index;
        try {
            index = Json::parse(ss.str());
        } catch (const std::invalid_argument& e) {
            throw WeightsError(index_path + ": not JSON: " + e.what());
        }
        const Json* map = index.is_object() ? index.find("weight_map") : nullptr;
        if (!map || !map->is_object()) throw WeightsError(index_path + ": no 'weight_map' object");
        std::map<std::string, int> shard_no;
        for (const auto& m : map->members()) {
            if (!m.second.is_string()) throw WeightsError(index_path + ": weight_map['" + m.first + "'] is not a file name");
            const std::string& file = m.second.as_string();
            auto it = shard_no.find(file);
            if (it == shard_no.end()) {
                const std::string path = dir + "/" + file;
                struct stat st;
                if (stat(path.c_str(), &st) != 0)
                    throw WeightsError(index_path + " names the shard " + file + ", which is not in the folder");
                files_.emplace_back(new SafetensorsFile(path));
                it = shard_no.emplace(file, (int)files_.size() - 1).first;
            }
            file_of_[m.first] = it->second;
            order_.push_back(m.first);
        }
    }
    std::string where() const override { return where_; }
    std::vector<std::string> names() const override { return order_; }
    bool info(const std::string& name, StoredTensor* out) const override {
        auto it = file_of_.find(name);
        return it != file_of_.end() && files_[it->second]->info(name, out);
    }
    std::string shard_of(const std::string& name) const {
        auto it = file_of_.find(name);
        return it == file_of_.end() ? "" : files_[it->second]->path();
    }
    void load(const std::string& name, const Tensor& dst, cudaStream_t stream) override {
        auto it = file_of_.find(name);
        StoredTensor t;
        size_t n = 0;
        const void* src = it == file_of_.end() ? nullptr : files_[it->second]->bytes(name, &n);
        if (!src && !(it != file_of_.end() && files_[it->second]->info(name, &t) && t.numel() == 0))
            throw WeightsError(where_ + ": tensor '" + name + "' is not there");
        files_[it->second]->info(name, &t);
        if (!uploader_ || uploader_stream_ != stream) {
            uploader_.reset(new Uploader(stream));
            uploader_stream_ = stream;
        }
        uploader_->upload(t.dtype, src, t, dst, name);
    }

private:
    std::string where_;
    std::vector<std::unique_ptr<SafetensorsFile>> files_;
    std::map<std::string, int> file_of_;
    std::vector<std::string> order_;
    std::unique_ptr<Uploader> uploader_;
    cudaStream_t uploader_stream_ = nullptr;
};

bool file_exists(const std::string& p) {
    struct stat st;
    return stat(p.c_str(), &st) == 0;
}

}  // namespace

std::unique_ptr<WeightSource> open_safetensors(const std::string& path) {
    return std::unique_ptr<WeightSource>(new SafetensorsSource(path));
}

std::unique_ptr<WeightSource> open_model_weights(const std::string& dir) {
    const std::string single = dir + "/model.safetensors", index = dir + "/model.safetensors.index.json";
    if (file_exists(single)) return std::unique_ptr<WeightSource>(new SafetensorsSource(single));
    if (file_exists(index)) return std::unique_ptr<WeightSource>(new SafetensorsSource(dir, index));
    throw WeightsError(dir + ": neither model.safetensors nor model.safetensors.index.json (with its shards) is in the "
                       "model folder");
}

// ------------------------------------------------------------------ the one error
void check_names(const std::vector<Part::Named>& expected, const WeightSource& source,
                 const std::vector<std::string>& ignorable) {
    const std::vector<std::string> have = source.names();
    const std::set<std::string> have_set(have.begin(), have.end());
    std::set<std::string> want_set;
    WeightsError err("");
    std::vector<std::string> notes;
    for (const auto& e : expected) {
        if (!want_set.insert(e.name).second) continue;
        StoredTensor t;
        if (!have_set.count(e.name)) {
            err.missing.push_back(e.name);
        } else if (!source.info(e.name, &t)) {
            err.missing.push_back(e.name);
            notes.push_back(e.name);
        } else if (t.shape != e.decl.shape) {
            err.wrong_shape.push_back(ShapeMismatch{e.name, t.shape, e.decl.shape});
        }
    }
    for (const auto& n : have)
        if (!want_set.count(n) && std::find(ignorable.begin(), ignorable.end(), n) == ignorable.end())
            err.unexpected.push_back(n);
    if (err.missing.empty() && err.unexpected.empty() && err.wrong_shape.empty()) return;
    auto join = [](const std::vector<std::string>& v) {
        std::string s;
        for (const auto& x : v) s += (s.empty() ? "" : ", ") + x;
        return s;
    };
    auto dims = [](const std::vector<int64_t>& v) {
        std::string s = "[";
        for (size_t i = 0; i < v.size(); ++i) s += (i ? ", " : "") + std::to_string(v[i]);
        return s + "]";
    };
    std::string text = source.where() + " do not fit the model:";
    if (!err.missing.empty()) text += format("\n  missing (%zu): ", err.missing.size()) + join(err.missing);
    if (!notes.empty())
        text += format("\n    of these, listed in the index but absent from their shard (%zu): ", notes.size()) + join(notes);
    if (!err.unexpected.empty()) text += format("\n  unexpected (%zu): ", err.unexpected.size()) + join(err.unexpected);
    if (!err.wrong_shape.empty()) {
        text += format("\n  wrong shape (%zu): ", err.wrong_shape.size());
        for (size_t i = 0; i < err.wrong_shape.size(); ++i)
            text += (i ? "; " : "") + err.wrong_shape[i].name + " is " + dims(err.wrong_shape[i].got) + ", the model needs " +
                    dims(err.wrong_shape[i].want);
    }
    WeightsError out(text);
    out.missing = err.missing;
    out.unexpected = err.unexpected;
    out.wrong_shape = err.wrong_shape;
    throw out;
}

// ------------------------------------------------------------------ writer
void write_safetensors(const std::string& path, const std::vector<HostTensor>& tensors, const Json& metadata) {
    Json header = Json::object();
    if (metadata.is_object() && metadata.size()) {
        Json md = Json::object();
        for (const auto& m : metadata.members())
            md.set(m.first, m.second.is_string() ? m.second : Json(m.second.dump()));
        header.set("__metadata__", md);
    }
    size_t offset = 0;
    for (const auto& t : tensors) {
        Json e = Json::object();
        e.set("dtype", Json(t.dtype));
        Json shape = Json::array();
        for (int64_t s : t.shape) shape.push(Json(s));
        e.set("shape", shape);
        Json range = Json::array();
        range.push(Json((int64_t)offset));
        range.push(Json((int64_t)(offset + t.bytes.size())));
        e.set("data_offsets", range);
        header.set(t.name, e);
        offset += t.bytes.size();
    }
    std::string text = header.dump();
    while (text.size() % 8) text += ' ';
    const std::string tmp = path + ".tmp";
    FILE* f = fopen(tmp.c_str(), "wb");
    if (!f) throw WeightsError(path + ": cannot write: " + strerror(errno));
    const uint64_t n = text.size();
    bool ok = fwrite(&n, 8, 1, f) == 1 && fwrite(text.data(), 1, text.size(), f) == text.size();
    for (const auto& t : tensors)
        if (ok && !t.bytes.empty()) ok = fwrite(t.bytes.data(), 1, t.bytes.size(), f) == t.bytes.size();
    ok = (fclose(f) == 0) && ok;
    if (!ok || rename(tmp.c_str(), path.c_str()) != 0) throw WeightsError(path + ": write failed: " + strerror(errno));
}

}  // namespace friday
