// Weights by tensor name: sources (a safetensors file, a sharded checkpoint, seeded random
// numbers), the loader's one error, and the writer of model folders.
//
// A source offers names, and for each name its stored dtype and shape and its bytes.  The
// loader (model.h) compares what the model declares with what the source offers before a
// byte is copied and reports every difference in ONE WeightsError: tensors the model needs
// and the source lacks, tensors the source has and the model does not know, tensors whose
// shape is wrong.  The reference reports these one at a time, some as a bare
// std::out_of_range (model_layout.cpp:66, transformer.cpp:527, 1000-1005).
//
// Storage rule: floating tensors are kept in the activation dtype (bfloat16 or float32);
// in bfloat16 mode a tensor that the file stores in 32 bits stays in 32 bits; integer
// tables become int32.
#pragma once
#include <cuda_runtime.h>

#include <map>
#include <memory>
#include <string>
#include <vector>

#include "friday/base.h"
#include "friday/json.h"
#include "friday/parts.h"

namespace friday {

struct StoredTensor {
    std::string dtype;                 // safetensors names: "BF16", "F16", "F32", "F64", "I64", "I32", "I16", "I8", "U8", "BOOL"
    std::vector<int64_t> shape;
    int64_t numel() const {
        int64_t n = 1;
        for (int64_t s : shape) n *= s;
        return n;
    }
};
size_t stored_dtype_size(const std::string& dtype);     // 0 if unknown
bool stored_dtype_is_float(const std::string& dtype);
bool stored_dtype_is_32bit_float(const std::string& dtype);      // F32 or F64

class WeightSource {
public:
    virtual ~WeightSource() {}
    virtual std::string where() const = 0;                              // for messages
    virtual std::vector<std::string> names() const = 0;
    virtual bool info(const std::string& name, StoredTensor* out) const = 0;
    // Puts tensor `name`, converted to dst.dtype, into device memory: element (r, c) of the tensor seen as
    // [rows, cols] (cols = the last dimension; a vector is one column) goes to dst.data + (r * dst.ld + c).
    virtual void load(const std::string& name, const Tensor& dst, cudaStream_t stream) = 0;
};

// One safetensors file: an 8-byte little-endian header length, a JSON header (name -> dtype, shape, byte
// range), then the raw bytes; memory-mapped read-only.  The reference reads GGUF through the same kind of
// table (gguf_file.h:53-91, model_layout.h:17-23).
class SafetensorsFile {
public:
    explicit SafetensorsFile(const std::string& path);
    ~SafetensorsFile();
    const std::string& path() const { return path_; }
    const std::vector<std::string>& names() const { return order_; }
    bool info(const std::string& name, StoredTensor* out) const;
    const void* bytes(const std::string& name, size_t* n) const;        // nullptr if absent
    const Json& metadata() const { return metadata_; }

private:
    struct Entry { StoredTensor t; size_t lo, hi; };
    std::string path_;
    std::map<std::string, Entry> entries_;
    std::vector<std::string> order_;
    Json metadata_;
    void* map_ = nullptr;
    size_t size_ = 0, base_ = 0;
};

// A model folder's weights: model.safetensors, or model.safetensors.index.json with the shards it names.
std::unique_ptr<WeightSource> open_model_weights(const std::string& model_dir);
std::unique_ptr<WeightSource> open_safetensors(const std::string& path);

// Seeded random numbers for the tensors `expected` names: matrices, tables and biases N(0, 0.02), norm weights
// 1 + N(0, 0.02); every tensor has a stream of its own derived from (seed, name), so any tensor can be made
// alone, in any order.  on_device draws with a kernel (billions of parameters in seconds); otherwise on the
// host, which is what written model folders hold.  The reference has no such mode (its tests draw N(0,1) fp16
// tensors per kernel: tests/kernels/test_decode_attention.cu:45-50).
std::unique_ptr<WeightSource> random_weights(const std::vector<Part::Named>& expected, uint64_t seed,
                                             const std::string& dtype, bool on_device);
uint64_t random_stream_key(uint64_t seed, const std::string& name);
// The host's numbers for one tensor, as float32 (before the rounding to the storage dtype).
void random_tensor_host(uint64_t seed, const std::string& name, bool one, int64_t count, float* out);

// Writes name -> (dtype, shape, host bytes) in the order given.
struct HostTensor {
    std::string name, dtype;
    std::vector<int64_t> shape;
    std::vector<uint8_t> bytes;
};
void write_safetensors(const std::string& path, const std::vector<HostTensor>& tensors, const Json& metadata = Json());

// config.json and model.safetensors for a typed configuration and a seed (dtype "BF16" or "F32").  With
// shards > 1 the tensors are spread over model-0000i-of-0000n.safetensors with a model.safetensors.index.json.
void write_random_model(const std::string& dir, const Json& config_json, uint64_t seed, const std::string& dtype = "BF16",
                        int shards = 1);

// Raises one WeightsError that lists every mismatch between `expected` and what `source` offers.
void check_names(const std::vector<Part::Named>& expected, const WeightSource& source,
                 const std::vector<std::string>& ignorable);

}  // namespace friday
