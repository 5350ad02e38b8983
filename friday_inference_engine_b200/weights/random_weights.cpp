// The random-weights mode: a source of seeded numbers for the loader, and the writer of
// model folders (config.json + model.safetensors, optionally in shards).
#include <errno.h>
#include <string.h>
#include <sys/stat.h>

#include <fstream>

#include "csrc/philox.h"
#include "friday/config.h"
#include "friday/model.h"
#include "friday/weights.h"
#include "ops/kernels.h"
#include "weights/upload.h"

namespace friday {

static const float kStd = 0.02f;

uint64_t random_stream_key(uint64_t seed, const std::string& name) {
    // FNV-1a over the seed's bytes, a zero byte and the name, then a 64-bit finalizer: a stream per (seed, tensor)
    uint64_t h = 1469598103934665603ull;
    auto eat = [&](uint8_t b) { h = (h ^ b) * 1099511628211ull; };
    for (int i = 0; i < 8; ++i) eat((uint8_t)(seed >> (8 * i)));
    eat(0);
    for (unsigned char c : name) eat(c);
    h ^= h >> 30;
    h *= 0xbf58476d1ce4e5b9ull;
    h ^= h >> 27;
    h *= 0x94d049bb133111ebull;
    h ^= h >> 31;
    return h;
}

void random_tensor_host(uint64_t seed, const std::string& name, bool one, int64_t count, float* out) {
    const uint64_t key = random_stream_key(seed, name);
    const float mean = one ? 1.0f : 0.0f;
    for (int64_t i = 0; i < count; ++i) {
        volatile float scaled = (float)fr_normal_at(key, (uint64_t)i) * kStd;      // rounded before the sum, as the kernel does
        out[i] = scaled + mean;
    }
}

namespace {

class RandomSource : public WeightSource {
public:
    RandomSource(const std::vector<Part::Named>& expected, uint64_t seed, const std::string& dtype, bool on_device)
        : seed_(seed), dtype_(dtype), on_device_(on_device) {
        for (const auto& e : expected)
            if (!decl_.count(e.name)) {
                decl_[e.name] = e.decl;
                order_.push_back(e.name);
            }
    }
    std::string where() const override { return format("random weights (seed %llu)", (unsigned long long)seed_); }
    std::vector<std::string> names() const override { return order_; }
    bool info(const std::string& name, StoredTensor* out) const override {
        auto it = decl_.find(name);
        if (it == decl_.end()) return false;
        if (out) {
            out->dtype = it->second.integer ? "I32" : dtype_;
            out->shape = it->second.shape;
        }
        return true;
    }
    void load(const std::string& name, const Tensor& dst, cudaStream_t stream) override {
        const ParamDecl& d = decl_.at(name);
        StoredTensor t;
        info(name, &t);
        const int64_t n = t.numel();
        if (n == 0) return;
        const int64_t cols = t.shape.size() >= 2 ? t.shape.back() : 1, rows = n / cols;
        const size_t es = dtype_size(dst.dtype);
        if (d.integer) {
            cuda_check(cudaMemset2DAsync(dst.data, (size_t)dst.ld * es, 0, (size_t)cols * es, (size_t)rows, stream), "cudaMemset2DAsync");
            return;
        }
        if (on_device_) {
            const auto& k = kernels::rowwise();
            const uint64_t key = random_stream_key(seed_, name);
            const float mean = d.one ? 1.0f : 0.0f;
            // numbers are rounded to the stored dtype first (what a written folder would hold), then to the model's
            const bool direct = (int64_t)dst.ld == cols && ((dtype_ == "BF16") == (dst.dtype == DType::BF16));
            if (direct) {
                if (k.random_normal(dst.data, n, (int)dst.dtype, key, mean, kStd, stream) != 0) throw KernelError(k.last_error());
                return;
            }
            const DType stored = dtype_ == "BF16" ? DType::BF16 : DType::F32;
            DeviceBuffer tmp((size_t)n * dtype_size(stored));
            if (k.random_normal(tmp.get(), n, (int)stored, key, mean, kStd, stream) != 0) throw KernelError(k.last_error());
            if (stored == dst.dtype) {
                cuda_check(cudaMemcpy2DAsync(dst.data, (size_t)dst.ld * es, tmp.get(), (size_t)cols * es, (size_t)cols * es,
                                             (size_t)rows, cudaMemcpyDeviceToDevice, stream), "cudaMemcpy2DAsync");
                cuda_check(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
                return;
            }
            // bf16 numbers into a 32-bit model (or the reverse): through the host
            std::vector<uint8_t> host((size_t)n * dtype_size(stored));
            cuda_check(cudaMemcpyAsync(host.data(), tmp.get(), host.size(), cudaMemcpyDeviceToHost, stream), "cudaMemcpyAsync");
            cuda_check(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
            Uploader up(stream);
            up.upload(stored == DType::BF16 ? "BF16" : "F32", host.data(), t, dst, name);
            return;
        }
        std::vector<float> f((size_t)n);
        random_tensor_host(seed_, name, d.one, n, f.data());
        Uploader up(stream);
        if (dtype_ == "BF16") {
            std::vector<uint16_t> b((size_t)n);
            for (int64_t i = 0; i < n; ++i) b[i] = float_to_bf16(f[i]);
            up.upload("BF16", b.data(), t, dst, name);
        } else {
            up.upload("F32", f.data(), t, dst, name);
        }
    }

private:
    uint64_t seed_;
    std::string dtype_;
    bool on_device_;
    std::map<std::string, ParamDecl> decl_;
    std::vector<std::string> order_;
};

}  // namespace

std::unique_ptr<WeightSource> random_weights(const std::vector<Part::Named>& expected, uint64_t seed,
                                             const std::string& dtype, bool on_device) {
    if (dtype != "BF16" && dtype != "F32") throw WeightsError("random weights are stored as BF16 or F32, not " + dtype);
    return std::unique_ptr<WeightSource>(new RandomSource(expected, seed, dtype, on_device));
}

void write_random_model(const std::string& dir, const Json& config_json, uint64_t seed, const std::string& dtype, int shards) {
    if (dtype != "BF16" && dtype != "F32") throw WeightsError("model folders are written as BF16 or F32, not " + dtype);
    const Architecture arch = architecture(architecture_name_of(config_json));
    const Json typed = arch.read_config(config_json);
    DecoderModel model(arch.build_spec(typed), DType::BF16);
    if (mkdir(dir.c_str(), 0777) != 0 && errno != EEXIST) throw WeightsError(dir + ": cannot create: " + strerror(errno));
    {
        std::ofstream f(dir + "/config.json");
        f << typed.dump(1) << "\n";
        if (!f) throw WeightsError(dir + "/config.json: cannot write");
    }
    std::vector<HostTensor> tensors;
    std::map<std::string, bool> seen;
    for (const auto& e : model.named_params()) {
        if (seen[e.name]) continue;
        seen[e.name] = true;
        HostTensor t;
        t.name = e.name;
        t.shape = e.decl.shape;
        int64_t n = 1;
        for (int64_t s : t.shape) n *= s;
        if (e.decl.integer) {
            t.dtype = "I32";
            t.bytes.assign((size_t)n * 4, 0);
        } else {
            std::vector<float> f((size_t)n);
            random_tensor_host(seed, e.name, e.decl.one, n, f.data());
            t.dtype = dtype;
            if (dtype == "BF16") {
                t.bytes.resize((size_t)n * 2);
                uint16_t* b = (uint16_t*)t.bytes.data();
                for (int64_t i = 0; i < n; ++i) b[i] = float_to_bf16(f[i]);
            } else {
                t.bytes.resize((size_t)n * 4);
                memcpy(t.bytes.data(), f.data(), (size_t)n * 4);
            }
        }
        tensors.push_back(std::move(t));
    }
    Json md = Json::object();
    md.set("format", Json("pt"));
    md.set("seed", Json(std::to_string(seed)));
    if (shards <= 1) {
        write_safetensors(dir + "/model.safetensors", tensors, md);
        return;
    }
    Json map = Json::object();
    const size_t per = (tensors.size() + shards - 1) / shards;
    for (int s = 0; s < shards; ++s) {
        std::vector<HostTensor> part;
        const std::string file = format("model-%05d-of-%05d.safetensors", s + 1, shards);
        for (size_t i = s * per; i < std::min(tensors.size(), (s + 1) * per); ++i) {
            map.set(tensors[i].name, Json(file));
            part.push_back(std::move(tensors[i]));
        }
        write_safetensors(dir + "/" + file, part, md);
    }
    Json index = Json::object();
    index.set("metadata", Json::object());
    index.set("weight_map", map);
    std::ofstream f(dir + "/model.safetensors.index.json");
    f << index.dump(1) << "\n";
    if (!f) throw WeightsError(dir + "/model.safetensors.index.json: cannot write");
}

}  // namespace friday
