// C++ host-side mirror of the reference host runtime's W8A8 operator methods, over the C ABI.
//
// The reference host is Rust (crates/inferrous-qwen3/src/gpu.rs); no Rust toolchain is available
// to this build, so the host layer above include/w8a8.h is written in C++ with the reference's
// names, argument order and error behaviour:
//   gpu::Matrix                       src/gpu.rs:43-49      -> w8a8::Matrix
//   gpu::Workspace (hot-path fields)  src/gpu.rs:76-143     -> w8a8::Workspace
//   GpuModel::norm_quantize           src/gpu.rs:340-363    -> GpuLinear::norm_quantize
//   GpuModel::linear_residual         src/gpu.rs:364-423    -> GpuLinear::linear_residual
//   GpuModel::quantize                src/gpu.rs:424-449    -> GpuLinear::quantize
//   GpuModel::linear_quantized        src/gpu.rs:450-509    -> GpuLinear::linear_quantized
//   GpuModel::residual                src/gpu.rs:510-517    -> GpuLinear::residual
//   direct launches in forward()      src/gpu.rs:571-590, 730-745, 770-777
//                                                           -> linear_triple, linear_swiglu, swiglu
// Like the reference, every method takes caller-owned output buffers, queues work on the one
// stream the object was built with, and reports failure as an error value (Rust `Result` there,
// a thrown w8a8::Error here); nothing allocates in a launch path and nothing falls back to the CPU.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/w8a8.h"

namespace w8a8 {

struct Error : std::runtime_error {
    int status;
    Error(int st, const std::string &where)
        : std::runtime_error(where + ": " + w8a8_status_string(st) + (st == W8A8_ERR_CUDA ? std::string(" (") + w8a8_last_cuda_error() + ")" : "")),
          status(st) {}
};
inline void ensure(int status, const char *where) {
    if (status != W8A8_OK) throw Error(status, where);
}
inline void cuda_ensure(cudaError_t e, const char *where) {
    if (e != cudaSuccess) throw std::runtime_error(std::string(where) + ": " + cudaGetErrorString(e));
}

// Owning device buffer (the role of cuda_core::DeviceBuffer<T> in the reference host).
template <class T> class DeviceBuffer {
   public:
    DeviceBuffer() = default;
    explicit DeviceBuffer(size_t n) : n_(n) { cuda_ensure(cudaMalloc(&p_, n * sizeof(T)), "cudaMalloc"); }
    static DeviceBuffer from_host(const std::vector<T> &h) {
        DeviceBuffer b(h.size());
        cuda_ensure(cudaMemcpy(b.p_, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice), "cudaMemcpy H2D");
        return b;
    }
    static DeviceBuffer zeroed(size_t n) {
        DeviceBuffer b(n);
        cuda_ensure(cudaMemset(b.p_, 0, n * sizeof(T)), "cudaMemset");
        return b;
    }
    DeviceBuffer(DeviceBuffer &&o) noexcept : p_(o.p_), n_(o.n_) { o.p_ = nullptr; o.n_ = 0; }
    DeviceBuffer &operator=(DeviceBuffer &&o) noexcept {
        if (this != &o) { release(); p_ = o.p_; n_ = o.n_; o.p_ = nullptr; o.n_ = 0; }
        return *this;
    }
    DeviceBuffer(const DeviceBuffer &) = delete;
    DeviceBuffer &operator=(const DeviceBuffer &) = delete;
    ~DeviceBuffer() { release(); }
    T *ptr() { return p_; }
    const T *ptr() const { return p_; }
    size_t len() const { return n_; }
    std::vector<T> to_host_vec(cudaStream_t s) const {
        std::vector<T> h(n_);
        cuda_ensure(cudaStreamSynchronize(s), "cudaStreamSynchronize");
        cuda_ensure(cudaMemcpy(h.data(), p_, n_ * sizeof(T), cudaMemcpyDeviceToHost), "cudaMemcpy D2H");
        return h;
    }
    void copy_from_host(const std::vector<T> &h) {
        cuda_ensure(cudaMemcpy(p_, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice), "cudaMemcpy H2D");
    }

   private:
    void release() {
        if (p_) cudaFree(p_);
        p_ = nullptr;
    }
    T *p_ = nullptr;
    size_t n_ = 0;
};

// The reference stores activations as f32 buffers that hold bf16-representable values.
using Buffer = DeviceBuffer<float>;

// gpu::Matrix {w, map, scale, k, n}: the TMA descriptor lives inside the C handle.
struct Matrix {
    DeviceBuffer<int8_t> w;
    Buffer scale;
    int k = 0, n = 0;
    w8a8_weight_t handle = nullptr;
    Matrix(const std::vector<int8_t> &weights, const std::vector<float> &scales, int n_, int k_)
        : w(DeviceBuffer<int8_t>::from_host(weights)), scale(Buffer::from_host(scales)), k(k_), n(n_) {
        ensure(w8a8_weight_create(w.ptr(), scale.ptr(), n, k, &handle), "w8a8_weight_create");
    }
    Matrix(Matrix &&) = delete;
    ~Matrix() {
        if (handle) w8a8_weight_destroy(handle);
    }
};

// The hot path's share of gpu::Workspace: int8 scratch for the two activation widths, scales, maxima.
struct Workspace {
    DeviceBuffer<int8_t> quant4, quant12;
    Buffer scales;
    DeviceBuffer<uint32_t> maxima;
    Workspace(int rows, int hidden = 4096, int intermediate = 12288)
        : quant4((size_t)rows * hidden), quant12((size_t)rows * intermediate), scales(rows), maxima(rows) {}
};

class GpuLinear {
   public:
    // `device::load(&ctx)` + the single stream of GpuModel::new (src/gpu.rs:247-250).
    explicit GpuLinear(int device = 0) {
        ensure(w8a8_init(device), "w8a8_init");
        cuda_ensure(cudaStreamCreate(&stream_), "cudaStreamCreate");
    }
    ~GpuLinear() {
        if (stream_) {
            cudaStreamSynchronize(stream_);
            cudaStreamDestroy(stream_);
        }
    }
    cudaStream_t stream() const { return stream_; }

    void norm_quantize(const Buffer &x, const Buffer &gain, Buffer *out, DeviceBuffer<int8_t> &q, Buffer &scale,
                       DeviceBuffer<uint32_t> *maxima) {
        const int K = (int)gain.len(), M = (int)(x.len() / gain.len());
        ensure(w8a8_rmsnorm_quantize(x.ptr(), gain.ptr(), W8A8_F32, 1e-6f, M, K, K, q.ptr(), scale.ptr(),
                                     out ? out->ptr() : nullptr, maxima ? maxima->ptr() : nullptr, stream_),
               "norm_quantize");
    }
    void quantize(const Buffer &x, int width, DeviceBuffer<int8_t> &q, Buffer &scale) {
        ensure(w8a8_quantize(x.ptr(), W8A8_F32, (int)(x.len() / width), width, width, q.ptr(), scale.ptr(), stream_), "quantize");
    }
    void quantize_with_max(const Buffer &x, int width, const DeviceBuffer<uint32_t> &maxima, DeviceBuffer<int8_t> &q, Buffer &scale) {
        ensure(w8a8_quantize_with_max(x.ptr(), W8A8_F32, maxima.ptr(), (int)(x.len() / width), width, width, q.ptr(), scale.ptr(), stream_),
               "quantize_with_max");
    }
    // The row count is scale.len(), as in the reference (`let nr = scale.len()`, src/gpu.rs:458).
    void linear_quantized(const DeviceBuffer<int8_t> &q, const Buffer &scale, const Matrix &w, Buffer &out, int rows) {
        ensure(w8a8_linear(q.ptr(), scale.ptr(), w.handle, rows, nullptr, out.ptr(), nullptr, W8A8_F32, stream_), "linear_quantized");
    }
    // Quantizes x (with the producer's maximum when the decode path has one, src/gpu.rs:377-390), projects,
    // and writes both the projection and bf16(residual + projection).
    void linear_residual(const Buffer &x, const Matrix &w, DeviceBuffer<int8_t> &q, Buffer &scale, Buffer &out,
                         const DeviceBuffer<uint32_t> *maxima, const Buffer &residual, Buffer &combined, int rows) {
        if (rows == 1 && w.k == 12288 && maxima)
            quantize_with_max(x, w.k, *maxima, q, scale);
        else
            quantize(x, w.k, q, scale);
        ensure(w8a8_linear(q.ptr(), scale.ptr(), w.handle, rows, residual.ptr(), out.ptr(), combined.ptr(), W8A8_F32, stream_),
               "linear_residual");
    }
    void residual(const Buffer &a, const Buffer &b, Buffer &out) {
        ensure(w8a8_residual(a.ptr(), b.ptr(), W8A8_F32, out.len(), out.ptr(), stream_), "residual");
    }
    void linear_triple(const DeviceBuffer<int8_t> &q, const Buffer &scale, const Matrix &w0, Buffer &out0, const Matrix &w1,
                       Buffer &out1, const Matrix &w2, Buffer &out2, int rows) {
        const w8a8_weight_t ws[3] = {w0.handle, w1.handle, w2.handle};
        void *outs[3] = {out0.ptr(), out1.ptr(), out2.ptr()};
        ensure(w8a8_linear_grouped(q.ptr(), scale.ptr(), ws, 3, rows, outs, W8A8_F32, stream_), "linear_triple");
    }
    void linear_pair(const DeviceBuffer<int8_t> &q, const Buffer &scale, const Matrix &w0, Buffer &out0, const Matrix &w1,
                     Buffer &out1, int rows) {
        const w8a8_weight_t ws[2] = {w0.handle, w1.handle};
        void *outs[2] = {out0.ptr(), out1.ptr()};
        ensure(w8a8_linear_grouped(q.ptr(), scale.ptr(), ws, 2, rows, outs, W8A8_F32, stream_), "linear_pair");
    }
    void linear_swiglu(const DeviceBuffer<int8_t> &q, const Buffer &scale, const Matrix &w0, Buffer &gate, const Matrix &w1,
                       Buffer &up, Buffer &out, DeviceBuffer<uint32_t> &maxima, int rows) {
        ensure(w8a8_linear_gate_up_swiglu(q.ptr(), scale.ptr(), w0.handle, w1.handle, rows, gate.ptr(), up.ptr(), out.ptr(),
                                          maxima.ptr(), W8A8_F32, stream_),
               "linear_swiglu");
    }
    void swiglu(const Buffer &gate, const Buffer &up, Buffer &out, DeviceBuffer<uint32_t> *maxima, int rows) {
        const int I = (int)(gate.len() / rows);
        ensure(w8a8_swiglu(gate.ptr(), up.ptr(), W8A8_F32, rows, I, I, out.ptr(), maxima ? maxima->ptr() : nullptr, stream_), "swiglu");
    }
    void rounding_probe(const Buffer &input, DeviceBuffer<int8_t> &out) {
        ensure(w8a8_rounding_probe(input.ptr(), out.ptr(), input.len(), stream_), "rounding_probe");
    }

   private:
    cudaStream_t stream_ = nullptr;
};

}  // namespace w8a8
