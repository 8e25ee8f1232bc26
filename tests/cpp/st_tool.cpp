// Test driver for include/shrewq_safetensors.hpp (host only, no GPU):
//   st_tool dump <file>        one line per metadata entry, tensor and quantized record (FNV-1a of the bytes)
//   st_tool copy <in> <out>    reads <in> and writes its contents again with the C++ writer
// Exit code 0, or 2 with "error: <message>" on stdout when the file is refused.
#include <cinttypes>
#include <cstdio>
#include <set>

#include "shrewq_safetensors.hpp"

using namespace shrewq::st;

static uint64_t fnv(const void *p, size_t n) {
    uint64_t h = 1469598103934665603ull;
    const uint8_t *b = static_cast<const uint8_t *>(p);
    for (size_t i = 0; i < n; ++i) h = (h ^ b[i]) * 1099511628211ull;
    return h;
}

static std::string shape_text(const std::vector<uint64_t> &s) {
    std::string o = "[";
    for (size_t k = 0; k < s.size(); ++k) o += (k ? "," : "") + std::to_string(s[k]);
    return o + "]";
}

int main(int argc, char **argv) {
    if (argc < 3) return 1;
    const std::string cmd = argv[1];
    try {
        const File f = File::open(argv[2]);
        const std::vector<Quantized> qs = f.quantized();
        if (cmd == "dump") {
            for (const auto &kv : f.metadata()) printf("meta %s %s\n", kv.first.c_str(), kv.second.c_str());
            for (const std::string &n : f.names()) {
                const Tensor &t = f.at(n);
                printf("tensor %s %s %s %zu %016" PRIx64 "\n", n.c_str(), t.dtype.c_str(), shape_text(t.shape).c_str(), t.nbytes,
                       fnv(t.data, t.nbytes));
            }
            for (const Quantized &q : qs) {
                uint64_t count = 1;
                for (uint64_t d : q.shape) count *= d;
                printf("quant %s %d %s %s %s %s %zu %016" PRIx64 " %016" PRIx64 " %016" PRIx64 "\n", q.name.c_str(), q.bits,
                       q.mode.c_str(), q.granularity.c_str(), q.original_dtype.c_str(), shape_text(q.shape).c_str(), q.n_scales,
                       fnv(q.codes, count), fnv(q.scales, q.n_scales * 8), fnv(q.zero_points, q.n_scales * 8));
            }
            return 0;
        }
        if (cmd == "copy" && argc >= 4) {
            std::vector<std::pair<std::string, Tensor>> out;
            std::vector<Description> desc;
            std::set<std::string> used;
            for (const Quantized &q : qs) {
                append_quantized(out, desc, q);
                used.insert(q.name + ".qweight");
                used.insert(q.name + ".scales");
                used.insert(q.name + ".zero_points");
            }
            for (const std::string &n : f.names())
                if (!used.count(n)) out.emplace_back(n, f.at(n));
            std::map<std::string, std::string> md = quantized_metadata(desc);
            for (const auto &kv : f.metadata())
                if (kv.first != kQuantizedKey) md[kv.first] = kv.second;
            write_file(argv[3], out, md);
            return 0;
        }
        return 1;
    } catch (const FormatError &e) {
        printf("error: %s\n", e.what());
        return 2;
    }
}
