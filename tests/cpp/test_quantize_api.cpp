// The reference's own quantization unit tests (crates/shrew/src/quantize.rs:601-789),
// restated against the C++ mirror of its API and run on the GPU through libshrewq.
// Each function names the Rust test it follows.  Exit code 0 = all passed.
#include <cmath>
#include <cstdio>
#include <cstdlib>

#include "shrewq.hpp"
#include "shrewq_checkpoint.hpp"

using namespace shrew;

#define CHECK(cond)                                                           \
    do {                                                                      \
        if (!(cond)) {                                                        \
            std::fprintf(stderr, "%s:%d: CHECK failed: %s\n", __FILE__, __LINE__, #cond); \
            std::exit(1);                                                     \
        }                                                                     \
    } while (0)

static Device DEV;

// quantize.rs:601-625
static void test_int8_symmetric_per_tensor() {
    std::vector<double> data{1.0, -0.5, 0.25, -1.0, 0.0, 0.75};
    Tensor tensor = Tensor::from_f64_slice(data, {2, 3}, DType::F32, DEV);
    QuantizedTensor qt = quantize_tensor(tensor, QuantConfig::int8());
    CHECK((qt.shape == std::vector<size_t>{2, 3}));
    CHECK(qt.n_scales == 1);
    CHECK(qt.zero_points() == std::vector<double>{0.0});
    std::vector<double> rec = dequantize_tensor(qt, DEV).to_f64_vec();
    for (size_t i = 0; i < data.size(); ++i) CHECK(std::fabs(data[i] - rec[i]) < 0.02);
    // the exact codes (golden vector: 1/(1/127) is slightly above 127, so -0.5 -> -64)
    std::vector<int8_t> q = qt.data_host();
    const int expect[6] = {127, -64, 32, -127, 0, 95};
    for (int i = 0; i < 6; ++i) CHECK(q[i] == expect[i]);
}

// quantize.rs:651-673
static void test_int8_per_channel() {
    std::vector<double> data(12);
    for (int i = 0; i < 12; ++i) data[i] = (i - 6.0) * 0.1;
    Tensor tensor = Tensor::from_f64_slice(data, {3, 4}, DType::F32, DEV);
    QuantizedTensor qt = quantize_tensor(tensor, QuantConfig::int8_per_channel());
    CHECK(qt.n_scales == 3);
    std::vector<double> rec = dequantize_tensor(qt, DEV).to_f64_vec();
    for (size_t i = 0; i < data.size(); ++i) CHECK(std::fabs(data[i] - rec[i]) < 0.01);
}

// quantize.rs:701-710 (INT8 half; INT4 has no device kernel and must be an error, not a fallback)
static void test_compression_ratio() {
    Tensor tensor = Tensor::zeros({256, 128}, DType::F32, DEV);
    QuantizedTensor qt8 = quantize_tensor(tensor, QuantConfig::int8());
    CHECK(std::fabs(qt8.compression_ratio() - 4.0) < 0.01);
    bool threw = false;
    try {
        quantize_tensor(tensor, QuantConfig::int4());
    } catch (const Error &e) {
        threw = e.code == SHREWQ_ERR_UNSUPPORTED;
    }
    CHECK(threw);
}

// quantize.rs:714-739
static void test_quantized_linear_forward() {
    std::vector<double> w{0.3, -0.2, 0.5, 0.1, -0.4, 0.25, 0.05, -0.6, 0.15, 0.45, -0.35, 0.2};
    std::vector<double> b{0.1, -0.1, 0.05};
    std::vector<double> x{0.5, -1.0, 0.25, 2.0, -0.75, 0.3, 1.5, -0.2};
    Linear linear{Tensor::from_f64_slice(w, {3, 4}, DType::F32, DEV), Tensor::from_f64_slice(b, {1, 3}, DType::F32, DEV), true};
    Tensor input = Tensor::from_f64_slice(x, {2, 4}, DType::F32, DEV);
    QuantizedLinear ql = QuantizedLinear::from_linear(linear, QuantConfig::int8());
    std::vector<double> y = ql.forward(input).to_f64_vec();
    CHECK(y.size() == 6);
    for (int m = 0; m < 2; ++m)
        for (int n = 0; n < 3; ++n) {
            double ref = b[n];
            for (int k = 0; k < 4; ++k) ref += x[m * 4 + k] * w[n * 4 + k];
            CHECK(std::fabs(ref - y[m * 3 + n]) < 0.5);   // the reference's own bound
            CHECK(std::fabs(ref - y[m * 3 + n]) < 0.02);  // and what INT8 actually achieves here
        }
}

// quantize.rs:741-746
static void test_quantized_linear_no_trainable_params() {
    Linear linear{Tensor::zeros({2, 4}, DType::F32, DEV), Tensor::zeros({1, 2}, DType::F32, DEV), true};
    QuantizedLinear ql = QuantizedLinear::from_linear(linear, QuantConfig::int8());
    CHECK(ql.parameters().empty());
    // (beyond the reference's assertion: the rest of the Module surface follows from that)
    CHECK(ql.named_parameters().empty() && ql.num_parameters() == 0 && ql.trainable_params_count() == 0);
    ql.set_training(false);
    CHECK(!ql.is_training());
}

// quantize.rs:748-755
static void test_quantized_linear_memory_savings() {
    Linear linear{Tensor::zeros({128, 256}, DType::F32, DEV), Tensor::zeros({1, 128}, DType::F32, DEV), true};
    QuantizedLinear ql = QuantizedLinear::from_linear(linear, QuantConfig::int8());
    CHECK(ql.memory_savings_bytes() == 98304);
    CHECK(ql.in_features == 256 && ql.out_features == 128);
}

// quantize.rs:759-766
static void test_quantize_named_parameters() {
    Linear linear{Tensor::zeros({4, 8}, DType::F32, DEV), Tensor::zeros({1, 4}, DType::F32, DEV), true};
    auto quantized = quantize_named_parameters(linear, QuantConfig::int8());
    CHECK(quantized.size() == 2);  // weight [4,8] and bias [1,4] are both rank 2
}

// quantize.rs:768-776
static void test_quantization_stats() {
    Linear linear{Tensor::zeros({32, 64}, DType::F32, DEV), Tensor::zeros({1, 32}, DType::F32, DEV), true};
    QuantStats stats = quantization_stats(linear, QuantConfig::int8());
    CHECK(stats.num_quantized == 2);
    CHECK(stats.num_fp32 == 0);
    CHECK(stats.compression_ratio > 3.0);
}

// quantize.rs:780-789
static void test_quantize_zero_tensor() {
    Tensor tensor = Tensor::zeros({2, 3}, DType::F32, DEV);
    QuantizedTensor qt = quantize_tensor(tensor, QuantConfig::int8());
    CHECK(qt.scales_host()[0] == 1.0);
    for (double v : dequantize_tensor(qt, DEV).to_f64_vec()) CHECK(v == 0.0);
}

// not a reference test: the reference cannot store a QuantizedTensor.  Quantize, save, load, and the
// loaded layer gives the same output bits.
static void test_checkpoint_round_trip(const char *path) {
    std::vector<double> w(24 * 16), b(24), x(5 * 16);
    for (size_t i = 0; i < w.size(); ++i) w[i] = std::sin(0.37 * double(i)) * 0.4;
    for (size_t i = 0; i < b.size(); ++i) b[i] = 0.01 * double(i) - 0.1;
    for (size_t i = 0; i < x.size(); ++i) x[i] = std::cos(0.11 * double(i));
    Linear linear{Tensor::from_f64_slice(w, {24, 16}, DType::F32, DEV), Tensor::from_f64_slice(b, {1, 24}, DType::F32, DEV), true};
    QuantizedLinear ql = QuantizedLinear::from_linear(linear, QuantConfig::int8_per_channel());
    QuantizedTensor pt = quantize_tensor(linear.weight, QuantConfig::int8());
    save_quantized(path, {{"fc.weight", ql.weight_quantized()}, {"fc_pt.weight", pt}});
    auto loaded = load_quantized(path, DEV);   // (the file stays for the caller to inspect)
    CHECK(loaded.size() == 2 && loaded[0].first == "fc.weight" && loaded[1].first == "fc_pt.weight");
    CHECK(loaded[0].second.data_host() == ql.weight_quantized().data_host());
    CHECK(loaded[0].second.scales_host() == ql.weight_quantized().scales_host());
    CHECK(loaded[0].second.shape == std::vector<size_t>({24, 16}) && loaded[0].second.n_scales == 24);
    CHECK(loaded[1].second.n_scales == 1 && loaded[1].second.scales_host() == pt.scales_host());
    QuantizedLinear ql2 = QuantizedLinear::create(loaded[0].second, &linear.bias, DEV);
    Tensor xt = Tensor::from_f64_slice(x, {5, 16}, DType::F32, DEV);
    CHECK(ql.forward(xt).to_f64_vec() == ql2.forward(xt).to_f64_vec());
}

// usage: test_quantize_api [file to write the checkpoint round trip to]
int main(int argc, char **argv) {
    try {
        DEV = Device(0);
        test_int8_symmetric_per_tensor();
        test_int8_per_channel();
        test_compression_ratio();
        test_quantized_linear_forward();
        test_quantized_linear_no_trainable_params();
        test_quantized_linear_memory_savings();
        test_quantize_named_parameters();
        test_quantization_stats();
        test_quantize_zero_tensor();
        if (argc > 1) test_checkpoint_round_trip(argv[1]);
        DEV.synchronize();
    } catch (const Error &e) {
        std::fprintf(stderr, "shrew::Error %d: %s\n", e.code, e.what());
        return 2;
    }
    std::puts("9 reference tests passed");
    if (argc > 1) std::puts("checkpoint round trip passed");
    return 0;
}
