// shrewq.hpp — C++ host-side mirror of Shrew's `quantize` module over the libshrewq C ABI.
//
// The reference's boundary for this path is Rust (crates/shrew/src/quantize.rs; names
// re-exported at crates/shrew/src/lib.rs:120-124).  This header keeps those names, argument
// meanings and error behaviour for a C++ host: QuantBits / QuantMode / QuantGranularity /
// QuantConfig (quantize.rs:35-140), QuantizedTensor (:150-185), quantize_tensor (:194-205),
// dequantize_tensor (:210-225), QuantizedLinear with from_linear / create / forward /
// parameters (:384-482), quantize_named_parameters and quantization_stats (:500-586).
// Tensors live on the GPU; every computation is a libshrewq kernel; errors are thrown as
// shrew::Error carrying the library's message (the Rust API returns Result<_, Error>).
// Header-only; link with libshrewq.so and the CUDA runtime.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "shrewq.h"

namespace shrew {

struct Error : std::runtime_error {
    int code;
    Error(int c, const std::string &m) : std::runtime_error(m), code(c) {}
};

enum class DType { F32 = SHREWQ_F32, BF16 = SHREWQ_BF16 };
inline size_t dtype_size(DType d) { return d == DType::F32 ? 4 : 2; }

// ---- device (the role of B::Device) -------------------------------------------------
class Device {
  public:
    Device() = default;  // empty handle; a usable device is Device(index)
    explicit Device(int index, cudaStream_t stream = nullptr) {
        shrewq_ctx *c = nullptr;
        int rc = shrewq_ctx_create(index, stream, &c);
        if (rc != SHREWQ_OK) throw Error(rc, shrewq_last_error(nullptr));
        ctx_.reset(c, shrewq_ctx_destroy);
        index_ = index;
    }
    shrewq_ctx *ctx() const { return ctx_.get(); }
    int index() const { return index_; }
    void check(int rc) const {
        if (rc != SHREWQ_OK) throw Error(rc, ctx_ ? shrewq_last_error(ctx_.get()) : "device handle is empty");
    }
    void synchronize() const { check(shrewq_ctx_synchronize(ctx_.get())); }

  private:
    std::shared_ptr<shrewq_ctx> ctx_;
    int index_ = 0;
};

// ---- a minimal device tensor (what the path needs of Tensor<B>) ------------------------
class Tensor {
  public:
    Tensor() = default;
    Tensor(std::vector<size_t> shape, DType dtype, const Device &dev) : shape_(std::move(shape)), dtype_(dtype), dev_(dev) {
        void *p = nullptr;
        size_t bytes = elem_count() * dtype_size(dtype);
        cudaSetDevice(dev.index());
        if (cudaMalloc(&p, bytes ? bytes : 1) != cudaSuccess) throw Error(SHREWQ_ERR_ALLOC, "cudaMalloc failed");
        buf_.reset(p, cudaFree);
    }
    // Tensor::from_f64_slice(data, shape, DType::F32, &dev)
    static Tensor from_f64_slice(const std::vector<double> &data, std::vector<size_t> shape, DType dtype, const Device &dev) {
        if (dtype != DType::F32) throw Error(SHREWQ_ERR_UNSUPPORTED, "from_f64_slice: F32 only in this mirror");
        Tensor t(std::move(shape), dtype, dev);
        if (data.size() != t.elem_count()) throw Error(SHREWQ_ERR_INVALID_ARG, "from_f64_slice: size mismatch");
        std::vector<float> f(data.begin(), data.end());
        cudaMemcpy(t.data(), f.data(), f.size() * 4, cudaMemcpyHostToDevice);
        return t;
    }
    static Tensor zeros(std::vector<size_t> shape, DType dtype, const Device &dev) {
        Tensor t(std::move(shape), dtype, dev);
        cudaMemset(t.data(), 0, t.elem_count() * dtype_size(dtype));
        return t;
    }
    std::vector<double> to_f64_vec() const {
        if (dtype_ != DType::F32) throw Error(SHREWQ_ERR_UNSUPPORTED, "to_f64_vec: F32 only in this mirror");
        std::vector<float> f(elem_count());
        cudaMemcpy(f.data(), data(), f.size() * 4, cudaMemcpyDeviceToHost);
        return std::vector<double>(f.begin(), f.end());
    }
    const std::vector<size_t> &dims() const { return shape_; }
    size_t rank() const { return shape_.size(); }
    size_t elem_count() const {
        size_t n = 1;
        for (size_t s : shape_) n *= s;
        return n;
    }
    DType dtype() const { return dtype_; }
    const Device &device() const { return dev_; }
    void *data() const { return buf_.get(); }

  private:
    std::vector<size_t> shape_;
    DType dtype_ = DType::F32;
    Device dev_{};
    std::shared_ptr<void> buf_;
};

// ---- configuration — quantize.rs:35-140 --------------------------------------------------
enum class QuantBits { Int8, Int4 };
enum class QuantMode { Symmetric, Asymmetric };
enum class QuantGranularity { PerTensor = SHREWQ_PER_TENSOR, PerChannel = SHREWQ_PER_CHANNEL };

struct QuantConfig {
    QuantBits bits = QuantBits::Int8;
    QuantMode mode = QuantMode::Symmetric;
    QuantGranularity granularity = QuantGranularity::PerTensor;
    static QuantConfig int8() { return {}; }
    static QuantConfig int8_per_channel() { return {QuantBits::Int8, QuantMode::Symmetric, QuantGranularity::PerChannel}; }
    static QuantConfig int4() { return {QuantBits::Int4, QuantMode::Symmetric, QuantGranularity::PerTensor}; }
    static QuantConfig int4_per_channel() { return {QuantBits::Int4, QuantMode::Symmetric, QuantGranularity::PerChannel}; }
    QuantConfig asymmetric() const { return {bits, QuantMode::Asymmetric, granularity}; }
    double qmax() const { return bits == QuantBits::Int8 ? 127.0 : 7.0; }
    double qmin() const {
        if (bits == QuantBits::Int8) return mode == QuantMode::Symmetric ? -127.0 : -128.0;
        return mode == QuantMode::Symmetric ? -7.0 : -8.0;
    }
    void require_int8_symmetric() const {
        if (bits != QuantBits::Int8 || mode != QuantMode::Symmetric)
            throw Error(SHREWQ_ERR_UNSUPPORTED, "only INT8 symmetric quantization has device kernels");
    }
};

// ---- QuantizedTensor — quantize.rs:150-185 -------------------------------------------------
struct QuantizedTensor {
    std::shared_ptr<int8_t> data;    // device, flat, source order
    std::shared_ptr<double> scales;  // device, 1 or shape[0] values
    size_t n_scales = 0;
    std::vector<size_t> shape;
    DType original_dtype = DType::F32;
    QuantConfig config;
    Device device;

    std::vector<double> zero_points() const { return std::vector<double>(n_scales, 0.0); }  // symmetric: all 0.0
    std::vector<double> scales_host() const {
        std::vector<double> s(n_scales);
        cudaMemcpy(s.data(), scales.get(), n_scales * 8, cudaMemcpyDeviceToHost);
        return s;
    }
    std::vector<int8_t> data_host() const {
        std::vector<int8_t> q(numel());
        cudaMemcpy(q.data(), data.get(), q.size(), cudaMemcpyDeviceToHost);
        return q;
    }
    size_t numel() const {
        size_t n = 1;
        for (size_t s : shape) n *= s;
        return n;
    }
    size_t size_bytes() const { return config.bits == QuantBits::Int8 ? numel() : (numel() + 1) / 2; }
    double compression_ratio() const { return double(numel() * 4) / double(size_bytes()); }
};

inline std::pair<size_t, size_t> rows_cols(const std::vector<size_t> &shape) {
    if (shape.empty()) return {1, 1};  // rank 0: one per-tensor element (quantize.rs:276-278)
    size_t cols = 1;
    for (size_t i = 1; i < shape.size(); ++i) cols *= shape[i];
    return {shape[0], cols};  // channel_size = product(shape[1..]) (quantize.rs:280-281)
}

// quantize_tensor — quantize.rs:194-205
inline QuantizedTensor quantize_tensor(const Tensor &tensor, const QuantConfig &config) {
    config.require_int8_symmetric();
    if (tensor.dtype() != DType::F32) throw Error(SHREWQ_ERR_UNSUPPORTED, "quantize_tensor: F32 tensors only");
    const Device &dev = tensor.device();
    auto [rows, cols] = rows_cols(tensor.dims());
    QuantGranularity g = tensor.rank() == 0 ? QuantGranularity::PerTensor : config.granularity;
    QuantizedTensor qt;
    qt.n_scales = g == QuantGranularity::PerChannel ? rows : 1;
    qt.shape = tensor.dims();
    qt.original_dtype = tensor.dtype();
    qt.config = config;
    qt.device = dev;
    void *q = nullptr, *s = nullptr;
    cudaSetDevice(dev.index());
    if (cudaMalloc(&q, rows * cols ? rows * cols : 1) != cudaSuccess || cudaMalloc(&s, (qt.n_scales ? qt.n_scales : 1) * 8) != cudaSuccess)
        throw Error(SHREWQ_ERR_ALLOC, "cudaMalloc failed");
    qt.data.reset(static_cast<int8_t *>(q), cudaFree);
    qt.scales.reset(static_cast<double *>(s), cudaFree);
    dev.check(shrewq_quantize_f32(dev.ctx(), static_cast<const float *>(tensor.data()), rows, cols, int(g), qt.data.get(),
                                  qt.scales.get()));
    return qt;
}

// dequantize_tensor — quantize.rs:210-225
inline Tensor dequantize_tensor(const QuantizedTensor &qt, const Device &dev) {
    Tensor out(qt.shape, qt.original_dtype, dev);
    auto [rows, cols] = rows_cols(qt.shape);
    QuantGranularity g = qt.shape.empty() ? QuantGranularity::PerTensor : qt.config.granularity;
    dev.check(shrewq_dequantize(dev.ctx(), qt.data.get(), qt.scales.get(), rows, cols, int(g), int(qt.original_dtype), out.data()));
    return out;
}

// what QuantizedLinear::from_linear reads of shrew_nn::Linear: weight [out,in], bias [1,out]
struct Linear {
    Tensor weight;
    Tensor bias;  // empty (rank 0, no buffer) when absent
    bool has_bias = false;
    std::vector<Tensor> parameters() const { return has_bias ? std::vector<Tensor>{weight, bias} : std::vector<Tensor>{weight}; }
    std::vector<std::pair<std::string, Tensor>> named_parameters() const {
        std::vector<std::pair<std::string, Tensor>> v{{"weight", weight}};
        if (has_bias) v.push_back({"bias", bias});
        return v;
    }
};

// ---- QuantizedLinear — quantize.rs:384-482 ---------------------------------------------------
class QuantizedLinear {
  public:
    size_t in_features = 0, out_features = 0;

    // QuantizedLinear::new — quantize.rs:437-447
    static QuantizedLinear create(QuantizedTensor weight_q, const Tensor *bias, const Device &device) {
        weight_q.config.require_int8_symmetric();
        if (weight_q.shape.size() != 2) throw Error(SHREWQ_ERR_INVALID_ARG, "QuantizedLinear needs a rank-2 weight");
        QuantizedLinear l;
        l.weight_q_ = std::move(weight_q);
        l.device_ = device;
        l.in_features = l.weight_q_.shape[1];
        l.out_features = l.weight_q_.shape[0];
        if (bias) l.bias_ = *bias, l.has_bias_ = true;
        shrewq_linear *h = nullptr;
        device.check(shrewq_linear_create(device.ctx(), l.weight_q_.data.get(), l.weight_q_.scales.get(),
                                          bias ? static_cast<const float *>(bias->data()) : nullptr, l.out_features,
                                          l.in_features, int(l.weight_q_.config.granularity), &h));
        l.h_.reset(h, shrewq_linear_destroy);
        return l;
    }
    // QuantizedLinear::from_linear — quantize.rs:413-434
    static QuantizedLinear from_linear(const Linear &linear, const QuantConfig &config) {
        auto params = linear.parameters();
        QuantizedTensor wq = quantize_tensor(params[0], config);
        return create(std::move(wq), params.size() > 1 ? &params[1] : nullptr, params[0].device());
    }
    const QuantizedTensor &weight_quantized() const { return weight_q_; }
    size_t memory_savings_bytes() const { return shrewq_linear_memory_savings_bytes(h_.get()); }
    // Module::forward — quantize.rs:463-476.  x is [M, in_features]; the result has x's dtype.
    Tensor forward(const Tensor &x, int epilogue = SHREWQ_EPILOGUE_NONE) const {
        if (x.rank() != 2 || x.dims()[1] != in_features) throw Error(SHREWQ_ERR_INVALID_ARG, "forward: x must be [M, in_features]");
        Tensor y({x.dims()[0], out_features}, x.dtype(), device_);
        device_.check(shrewq_linear_forward(h_.get(), x.data(), int(x.dtype()), x.dims()[0], y.data(), int(x.dtype()),
                                            out_features, epilogue));
        return y;
    }
    // inference only — quantize.rs:478-481
    std::vector<Tensor> parameters() const { return {}; }
    // the rest of the Module surface (trait defaults in the reference; quantize.rs:462-482 overrides only forward
    // and parameters): nothing to name or count, the mode flag is kept as set and the forward ignores it
    std::vector<std::pair<std::string, Tensor>> named_parameters() const { return {}; }
    size_t num_parameters() const { return 0; }
    size_t trainable_params_count() const { return 0; }
    void set_training(bool training) { training_ = training; }
    bool is_training() const { return training_; }

  private:
    QuantizedTensor weight_q_;
    Tensor bias_;
    bool has_bias_ = false;
    bool training_ = true;
    Device device_;
    std::shared_ptr<shrewq_linear> h_;
};

// ---- model-level helpers — quantize.rs:500-586 -------------------------------------------------
template <class Module>
std::vector<std::pair<std::string, QuantizedTensor>> quantize_named_parameters(const Module &module, const QuantConfig &config) {
    std::vector<std::pair<std::string, QuantizedTensor>> out;
    for (auto &nt : module.named_parameters())
        if (nt.second.rank() >= 2) out.push_back({nt.first, quantize_tensor(nt.second, config)});  // a [1,out] bias counts
    return out;
}

struct QuantStats {
    size_t num_quantized = 0, num_fp32 = 0, fp32_bytes = 0, quantized_bytes = 0;
    double compression_ratio = 1.0;
};

template <class Module>
QuantStats quantization_stats(const Module &module, const QuantConfig &config) {
    QuantStats st;
    for (auto &nt : module.named_parameters()) {
        const Tensor &t = nt.second;
        size_t numel = t.elem_count();
        st.fp32_bytes += numel * 4;
        if (t.rank() >= 2) {
            st.num_quantized += 1;
            size_t q = config.bits == QuantBits::Int8 ? numel : (numel + 1) / 2;
            size_t meta = config.granularity == QuantGranularity::PerTensor ? 16 : (t.dims().empty() ? 16 : t.dims()[0] * 16);
            st.quantized_bytes += q + meta;
        } else {
            st.num_fp32 += 1;
            st.quantized_bytes += numel * 4;
        }
    }
    st.compression_ratio = st.quantized_bytes ? double(st.fp32_bytes) / double(st.quantized_bytes) : 1.0;
    return st;
}

}  // namespace shrew
