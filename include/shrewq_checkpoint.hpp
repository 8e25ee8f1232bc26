// shrewq_checkpoint.hpp — QuantizedTensors of the C++ mirror (shrewq.hpp) to and from the on-disk record
// (shrewq_safetensors.hpp).  The reference has no such step: a quantized model is re-quantized from its
// float checkpoint at every start (crates/shrew/src/quantize.rs:413-434 is the only constructor path from
// weights; safetensors.rs:61-75 has no 8-bit signed type).  With this, a host quantizes once, saves, and a
// serving process loads codes and scales straight into QuantizedLinear::create (quantize.rs:437-447).
// INT8 symmetric records only, like the rest of the C++ mirror.  Header-only.
#pragma once

#include <string>
#include <utility>
#include <vector>

#include "shrewq.hpp"
#include "shrewq_safetensors.hpp"

namespace shrew {

inline void save_quantized(const std::string &path, const std::vector<std::pair<std::string, QuantizedTensor>> &named) {
    namespace st = shrewq::st;
    struct Host {
        std::vector<int8_t> codes;
        std::vector<double> scales, zps;
    };
    std::vector<Host> host(named.size());  // sized once: the records below point into it
    std::vector<std::pair<std::string, st::Tensor>> tensors;
    std::vector<st::Description> desc;
    for (size_t i = 0; i < named.size(); ++i) {
        const QuantizedTensor &t = named[i].second;
        t.config.require_int8_symmetric();
        host[i].codes = t.data_host();
        host[i].scales = t.scales_host();
        host[i].zps = t.zero_points();
        st::Quantized q;
        q.name = named[i].first;
        q.bits = 8;
        q.mode = "symmetric";
        q.granularity = (t.config.granularity == QuantGranularity::PerChannel && !t.shape.empty()) ? "per_channel" : "per_tensor";
        q.original_dtype = t.original_dtype == DType::F32 ? "F32" : "BF16";
        q.shape.assign(t.shape.begin(), t.shape.end());
        q.codes = host[i].codes.data();
        q.scales = reinterpret_cast<const uint8_t *>(host[i].scales.data());
        q.zero_points = reinterpret_cast<const uint8_t *>(host[i].zps.data());
        q.n_scales = t.n_scales;
        st::append_quantized(tensors, desc, q);
    }
    st::write_file(path, tensors, st::quantized_metadata(desc));
}

// Every quantized record of the file as a device-resident QuantizedTensor, in the description's order.
inline std::vector<std::pair<std::string, QuantizedTensor>> load_quantized(const std::string &path, const Device &dev) {
    namespace st = shrewq::st;
    const st::File file = st::File::open(path);
    std::vector<std::pair<std::string, QuantizedTensor>> out;
    for (const st::Quantized &q : file.quantized()) {
        if (q.bits != 8 || q.mode != "symmetric")
            throw Error(SHREWQ_ERR_UNSUPPORTED, "load_quantized: '" + q.name + "' is not an INT8 symmetric record");
        QuantizedTensor t;
        t.shape.assign(q.shape.begin(), q.shape.end());
        t.n_scales = q.n_scales;
        t.original_dtype = q.original_dtype == "BF16" ? DType::BF16 : DType::F32;
        t.config = q.granularity == "per_channel" ? QuantConfig::int8_per_channel() : QuantConfig::int8();
        t.device = dev;
        void *codes = nullptr, *scales = nullptr;
        const size_t n = t.numel();
        cudaSetDevice(dev.index());
        if (cudaMalloc(&codes, n ? n : 1) != cudaSuccess || cudaMalloc(&scales, (q.n_scales ? q.n_scales : 1) * 8) != cudaSuccess)
            throw Error(SHREWQ_ERR_ALLOC, "cudaMalloc failed");
        t.data.reset(static_cast<int8_t *>(codes), cudaFree);
        t.scales.reset(static_cast<double *>(scales), cudaFree);
        if (n) cudaMemcpy(codes, q.codes, n, cudaMemcpyHostToDevice);
        if (q.n_scales) cudaMemcpy(scales, q.scales, q.n_scales * 8, cudaMemcpyHostToDevice);  // raw little-endian f64
        out.emplace_back(q.name, std::move(t));
    }
    return out;
}

}  // namespace shrew
