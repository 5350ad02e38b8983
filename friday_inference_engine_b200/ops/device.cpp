// Device memory (DeviceBuffer, Arena) and the small helpers of base.h.
#include <stdarg.h>
#include <stdio.h>

#include "friday/ops.h"

namespace friday {

std::string format(const char* fmt, ...) {
    char buf[2048];
    va_list ap;
    va_start(ap, fmt);
    int n = vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (n < (int)sizeof buf) return std::string(buf, n < 0 ? 0 : n);
    std::string big((size_t)n + 1, '\0');
    va_start(ap, fmt);
    vsnprintf(&big[0], big.size(), fmt, ap);
    va_end(ap);
    big.resize((size_t)n);
    return big;
}

const char* dtype_name(DType d) {
    return d == DType::F32 ? "float32" : d == DType::BF16 ? "bfloat16" : "int32";
}

DType parse_dtype(const std::string& name) {
    if (name == "bfloat16" || name == "bf16") return DType::BF16;
    if (name == "float32" || name == "fp32" || name == "f32") return DType::F32;
    throw Error(ErrorKind::Other, "dtype must be bfloat16 or float32, got '" + name + "'");
}

void cuda_check(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw KernelError(format("%s: %s", what, cudaGetErrorString(e)));
}

DeviceBuffer::DeviceBuffer(size_t bytes, bool zero) : n_(bytes) {
    if (bytes == 0) return;
    cudaError_t e = cudaMalloc(&p_, bytes);
    if (e != cudaSuccess) {
        p_ = nullptr;
        throw KernelError(format("cannot allocate %.3f GB of device memory: %s", bytes / 1e9, cudaGetErrorString(e)));
    }
    if (zero) {      // finished before anyone can use the buffer on another stream
        cuda_check(cudaMemset(p_, 0, bytes), "cudaMemset");
        cuda_check(cudaStreamSynchronize(nullptr), "cudaStreamSynchronize");
    }
}

DeviceBuffer::~DeviceBuffer() {
    if (p_) cudaFree(p_);
}

DeviceBuffer& DeviceBuffer::operator=(DeviceBuffer&& o) noexcept {
    if (this != &o) {
        if (p_) cudaFree(p_);
        p_ = o.p_;
        n_ = o.n_;
        o.p_ = nullptr;
        o.n_ = 0;
    }
    return *this;
}

Arena::~Arena() {
    for (auto& b : blocks_) cudaFree(b.p);
}

size_t Arena::capacity() const {
    size_t t = 0;
    for (const auto& b : blocks_) t += b.size;
    return t;
}

void* Arena::alloc(size_t bytes) {
    bytes = (bytes + 255) & ~(size_t)255;
    if (bytes == 0) bytes = 256;
    if (blocks_.empty() || offset_ + bytes > blocks_.back().size) {
        if (frozen)
            throw KernelError("a pass needed more working memory while its launches were being captured in a graph");
        size_t want = capacity();
        if (want < first_) want = first_;
        if (want < bytes) want = bytes;
        BlockMem b{nullptr, want};
        cudaError_t e = cudaMalloc(&b.p, want);
        if (e != cudaSuccess)
            throw KernelError(format("cannot allocate %.3f GB of working memory: %s", want / 1e9, cudaGetErrorString(e)));
        blocks_.push_back(b);
        offset_ = 0;
        ++generation_;
    }
    void* p = (char*)blocks_.back().p + offset_;
    offset_ += bytes;
    return p;
}

void Arena::reset() {
    if (blocks_.size() > 1) {
        // join the blocks: everything handed out is dead, but kernels that read it may still run
        cuda_check(cudaStreamSynchronize(stream_), "cudaStreamSynchronize");
        size_t total = capacity();
        for (auto& b : blocks_) cudaFree(b.p);
        blocks_.clear();
        BlockMem b{nullptr, total};
        cudaError_t e = cudaMalloc(&b.p, total);
        if (e != cudaSuccess)
            throw KernelError(format("cannot allocate %.3f GB of working memory: %s", total / 1e9, cudaGetErrorString(e)));
        blocks_.push_back(b);
        ++generation_;
    }
    offset_ = 0;
}

}  // namespace friday
