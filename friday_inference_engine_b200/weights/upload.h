// Host tensors to device memory, converted on the way (internal to the weight sources).
#pragma once
#include <algorithm>
#include <string>

#include "weights/convert.h"
#include "friday/ops.h"
#include "friday/weights.h"

namespace friday {

inline float half_to_float(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu, u;
    if (exp == 0) {
        if (man == 0) u = sign;
        else {
            int shift = 0;
            while (!(man & 0x400u)) { man <<= 1; ++shift; }
            man &= 0x3FFu;
            u = sign | ((uint32_t)(127 - 15 - shift + 1) << 23) | (man << 13);
        }
    } else if (exp == 31) u = sign | 0x7F800000u | (man << 13);
    else u = sign | ((exp - 15 + 127) << 23) | (man << 13);
    float f;
    memcpy(&f, &u, 4);
    return f;
}

// count elements from `src` (stored dtype) to `dst` (DType)
inline void convert(const std::string& from, const void* src, DType to, void* dst, size_t count, const std::string& name) {
    if (to == DType::I32) {
        int32_t* o = (int32_t*)dst;
        if (from == "I32") memcpy(o, src, count * 4);
        else if (from == "I64") for (size_t i = 0; i < count; ++i) o[i] = (int32_t)((const int64_t*)src)[i];
        else if (from == "I16") for (size_t i = 0; i < count; ++i) o[i] = ((const int16_t*)src)[i];
        else if (from == "I8") for (size_t i = 0; i < count; ++i) o[i] = ((const int8_t*)src)[i];
        else if (from == "U8" || from == "BOOL") for (size_t i = 0; i < count; ++i) o[i] = ((const uint8_t*)src)[i];
        else throw WeightsError("tensor '" + name + "': a floating tensor (" + from + ") where an integer table is needed");
        return;
    }
    if (!stored_dtype_is_float(from))
        throw WeightsError("tensor '" + name + "': an integer tensor (" + from + ") where a floating one is needed");
    if (to == DType::F32) {
        float* o = (float*)dst;
        if (from == "F32") memcpy(o, src, count * 4);
        else if (from == "BF16") for (size_t i = 0; i < count; ++i) o[i] = bf16_to_float(((const uint16_t*)src)[i]);
        else if (from == "F16") for (size_t i = 0; i < count; ++i) o[i] = half_to_float(((const uint16_t*)src)[i]);
        else for (size_t i = 0; i < count; ++i) o[i] = (float)((const double*)src)[i];
    } else {
        uint16_t* o = (uint16_t*)dst;
        if (from == "BF16") memcpy(o, src, count * 2);
        else if (from == "F32") for (size_t i = 0; i < count; ++i) o[i] = float_to_bf16(((const float*)src)[i]);
        else if (from == "F16") for (size_t i = 0; i < count; ++i) o[i] = float_to_bf16(half_to_float(((const uint16_t*)src)[i]));
        else for (size_t i = 0; i < count; ++i) o[i] = float_to_bf16((float)((const double*)src)[i]);
    }
}

// Host rows to device rows with a pitch, converting on the way, through two pinned buffers.
class Uploader {
public:
    explicit Uploader(cudaStream_t s) : stream_(s) {}
    ~Uploader() {
        for (int i = 0; i < 2; ++i) {
            if (ev_[i]) cudaEventDestroy(ev_[i]);
            if (buf_[i]) cudaFreeHost(buf_[i]);
        }
    }
    void upload(const std::string& from, const void* src, const StoredTensor& t, const Tensor& dst, const std::string& name) {
        const int64_t cols = t.shape.size() >= 2 ? t.shape.back() : 1;
        const int64_t rows = cols ? t.numel() / cols : 0;
        if (rows == 0 || cols == 0) return;
        const size_t ses = stored_dtype_size(from), des = dtype_size(dst.dtype);
        const bool same = (from == "BF16" && dst.dtype == DType::BF16) || (from == "F32" && dst.dtype == DType::F32) ||
                          (from == "I32" && dst.dtype == DType::I32);
        if ((int64_t)dst.ld == cols && same) {        // one contiguous piece, straight from the mapped file
            cuda_check(cudaMemcpyAsync(dst.data, src, (size_t)rows * cols * ses, cudaMemcpyHostToDevice, stream_), "cudaMemcpyAsync");
            cuda_check(cudaStreamSynchronize(stream_), "cudaStreamSynchronize");
            return;
        }
        if (same) {        // rows with a pitch, straight from the mapped file
            cuda_check(cudaMemcpy2DAsync(dst.data, (size_t)dst.ld * des, src, (size_t)cols * ses, (size_t)cols * ses,
                                         (size_t)rows, cudaMemcpyHostToDevice, stream_), "cudaMemcpy2DAsync");
            cuda_check(cudaStreamSynchronize(stream_), "cudaStreamSynchronize");
            return;
        }
        const size_t row_bytes = (size_t)cols * des;
        int64_t per = (int64_t)(kChunk / (row_bytes ? row_bytes : 1));
        if (per < 1) per = 1;
        for (int64_t r0 = 0; r0 < rows; r0 += per) {
            const int64_t n = std::min(per, rows - r0);
            const int b = next_++ & 1;
            ensure(b, (size_t)n * row_bytes);
            if (ev_[b]) cuda_check(cudaEventSynchronize(ev_[b]), "cudaEventSynchronize");
            convert(from, (const char*)src + (size_t)r0 * cols * ses, dst.dtype, buf_[b], (size_t)n * cols, name);
            cuda_check(cudaMemcpy2DAsync((char*)dst.data + (size_t)r0 * dst.ld * des, (size_t)dst.ld * des, buf_[b],
                                         row_bytes, row_bytes, (size_t)n, cudaMemcpyHostToDevice, stream_),
                       "cudaMemcpy2DAsync");
            if (!ev_[b]) cuda_check(cudaEventCreateWithFlags(&ev_[b], cudaEventDisableTiming), "cudaEventCreate");
            cuda_check(cudaEventRecord(ev_[b], stream_), "cudaEventRecord");
        }
        cuda_check(cudaStreamSynchronize(stream_), "cudaStreamSynchronize");
    }

private:
    static constexpr size_t kChunk = (size_t)32 << 20;
    void ensure(int b, size_t bytes) {
        if (cap_[b] >= bytes) return;
        if (buf_[b]) {
            if (ev_[b]) cudaEventSynchronize(ev_[b]);
            cudaFreeHost(buf_[b]);
        }
        cap_[b] = std::max(bytes, kChunk);
        cuda_check(cudaMallocHost(&buf_[b], cap_[b]), "cudaMallocHost");
    }
    cudaStream_t stream_;
    void* buf_[2] = {nullptr, nullptr};
    size_t cap_[2] = {0, 0};
    cudaEvent_t ev_[2] = {nullptr, nullptr};
    int next_ = 0;
};


}  // namespace friday
