// shrewq_safetensors.hpp — C++ reader / writer of the on-disk record for quantized tensors.
//
// Container: safetensors, as the reference writes it for float tensors
// (crates/shrew/src/safetensors.rs:1-28,336-377): an 8-byte little-endian header length, a JSON
// header (name -> {dtype, shape, data_offsets}, plus "__metadata__" with string values), then the raw
// little-endian tensor bytes, offsets relative to their start.  The reference has no record for
// QuantizedTensor (crates/shrew/src/quantize.rs:150-185); this format stores its fields as ordinary
// entries
//
//     <name>.qweight       I8    the tensor's shape      codes, source order
//     <name>.scales        F64   [1] or [shape[0]]
//     <name>.zero_points   F64   same length             all 0.0 in symmetric mode
//
// and describes every record in the metadata entry "shrew.quantized", a JSON object
// name -> {bits, mode, granularity, original_dtype}.  The Python side of the same format is
// shrew_b200/qsafetensors.py; files written by either are read by the other and by any safetensors
// reader.  The checks of File::open are the reference reader's (header size limit, UTF-8 / JSON
// object, known dtype, byte count per entry: safetensors.rs:132-140,383-403) plus: offsets inside the
// file, no overlap, no hole, nothing trailing.
//
// Host side only: the arrays are views into a read-only mapping of the file, ready for one
// cudaMemcpy each into the buffers shrewq_linear_create takes (entries sit back to back, so a view
// is only as aligned as the bytes before it make it).  Header-only, C++17, POSIX (mmap); no
// dependency on the CUDA library.  Errors are thrown as shrewq::st::FormatError.
#pragma once

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace shrewq {
namespace st {

struct FormatError : std::runtime_error {
    explicit FormatError(const std::string &m) : std::runtime_error(m) {}
};

// ---- a small JSON reader / writer: all the header needs --------------------------------------------
namespace json {

struct Value;
using Member = std::pair<std::string, Value>;

struct Value {
    enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
    bool b = false;
    double num = 0.0;
    bool is_int = false;      // the number was written without fraction or exponent and fits int64
    int64_t i = 0;
    std::string str;
    std::vector<Value> arr;
    std::vector<Member> obj;  // members in file order, duplicates kept (the caller decides)

    const Value *get(const std::string &key) const {
        for (const Member &m : obj)
            if (m.first == key) return &m.second;
        return nullptr;
    }
};

class Parser {
  public:
    Parser(const char *p, size_t n) : p_(p), end_(p + n) {}
    Value parse_document() {
        Value v = value(0);
        ws();
        if (p_ != end_) fail("trailing characters after the JSON value");
        return v;
    }

  private:
    const char *p_, *end_;
    [[noreturn]] void fail(const std::string &m) const { throw FormatError("invalid header: " + m); }
    void ws() {
        while (p_ < end_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\r' || *p_ == '\t')) ++p_;
    }
    bool lit(const char *s) {
        const size_t n = strlen(s);
        if ((size_t)(end_ - p_) >= n && memcmp(p_, s, n) == 0) { p_ += n; return true; }
        return false;
    }
    static void put_utf8(std::string &o, uint32_t c) {
        if (c < 0x80) o += (char)c;
        else if (c < 0x800) { o += (char)(0xC0 | (c >> 6)); o += (char)(0x80 | (c & 0x3F)); }
        else if (c < 0x10000) { o += (char)(0xE0 | (c >> 12)); o += (char)(0x80 | ((c >> 6) & 0x3F)); o += (char)(0x80 | (c & 0x3F)); }
        else { o += (char)(0xF0 | (c >> 18)); o += (char)(0x80 | ((c >> 12) & 0x3F)); o += (char)(0x80 | ((c >> 6) & 0x3F)); o += (char)(0x80 | (c & 0x3F)); }
    }
    uint32_t hex4() {
        if (end_ - p_ < 4) fail("truncated \\u escape");
        uint32_t v = 0;
        for (int k = 0; k < 4; ++k) {
            const char c = *p_++;
            v <<= 4;
            if (c >= '0' && c <= '9') v |= (uint32_t)(c - '0');
            else if (c >= 'a' && c <= 'f') v |= (uint32_t)(c - 'a' + 10);
            else if (c >= 'A' && c <= 'F') v |= (uint32_t)(c - 'A' + 10);
            else fail("bad \\u escape");
        }
        return v;
    }
    std::string string() {
        if (p_ >= end_ || *p_ != '"') fail("expected a string");
        ++p_;
        std::string o;
        while (true) {
            if (p_ >= end_) fail("unterminated string");
            const unsigned char c = (unsigned char)*p_++;
            if (c == '"') break;
            if (c < 0x20) fail("control character in a string");
            if (c != '\\') { o += (char)c; continue; }
            if (p_ >= end_) fail("unterminated escape");
            const char e = *p_++;
            switch (e) {
                case '"': o += '"'; break;
                case '\\': o += '\\'; break;
                case '/': o += '/'; break;
                case 'b': o += '\b'; break;
                case 'f': o += '\f'; break;
                case 'n': o += '\n'; break;
                case 'r': o += '\r'; break;
                case 't': o += '\t'; break;
                case 'u': {
                    uint32_t c1 = hex4();
                    if (c1 >= 0xD800 && c1 < 0xDC00) {
                        if (!lit("\\u")) fail("lone surrogate");
                        const uint32_t c2 = hex4();
                        if (c2 < 0xDC00 || c2 >= 0xE000) fail("bad surrogate pair");
                        c1 = 0x10000 + ((c1 - 0xD800) << 10) + (c2 - 0xDC00);
                    } else if (c1 >= 0xDC00 && c1 < 0xE000) {
                        fail("lone surrogate");
                    }
                    put_utf8(o, c1);
                    break;
                }
                default: fail("unknown escape");
            }
        }
        return o;
    }
    Value number() {
        const char *s = p_;
        if (p_ < end_ && *p_ == '-') ++p_;
        if (p_ >= end_ || *p_ < '0' || *p_ > '9') fail("bad number");
        if (*p_ == '0') ++p_;
        else while (p_ < end_ && *p_ >= '0' && *p_ <= '9') ++p_;
        bool integral = true;
        if (p_ < end_ && *p_ == '.') {
            integral = false;
            ++p_;
            if (p_ >= end_ || *p_ < '0' || *p_ > '9') fail("bad number");
            while (p_ < end_ && *p_ >= '0' && *p_ <= '9') ++p_;
        }
        if (p_ < end_ && (*p_ == 'e' || *p_ == 'E')) {
            integral = false;
            ++p_;
            if (p_ < end_ && (*p_ == '+' || *p_ == '-')) ++p_;
            if (p_ >= end_ || *p_ < '0' || *p_ > '9') fail("bad number");
            while (p_ < end_ && *p_ >= '0' && *p_ <= '9') ++p_;
        }
        Value v;
        v.kind = Value::Number;
        const std::string text(s, p_);
        v.num = strtod(text.c_str(), nullptr);
        if (integral && text.size() <= 19) {  // at most 18 digits and a sign: no overflow
            v.is_int = true;
            v.i = strtoll(text.c_str(), nullptr, 10);
        }
        return v;
    }
    Value value(int depth) {
        if (depth > 64) fail("nesting too deep");
        ws();
        if (p_ >= end_) fail("unexpected end");
        Value v;
        const char c = *p_;
        if (c == '{') {
            ++p_;
            v.kind = Value::Object;
            ws();
            if (p_ < end_ && *p_ == '}') { ++p_; return v; }
            while (true) {
                ws();
                std::string k = string();
                ws();
                if (p_ >= end_ || *p_ != ':') fail("expected ':'");
                ++p_;
                v.obj.emplace_back(std::move(k), value(depth + 1));
                ws();
                if (p_ < end_ && *p_ == ',') { ++p_; continue; }
                if (p_ < end_ && *p_ == '}') { ++p_; break; }
                fail("expected ',' or '}'");
            }
        } else if (c == '[') {
            ++p_;
            v.kind = Value::Array;
            ws();
            if (p_ < end_ && *p_ == ']') { ++p_; return v; }
            while (true) {
                v.arr.push_back(value(depth + 1));
                ws();
                if (p_ < end_ && *p_ == ',') { ++p_; continue; }
                if (p_ < end_ && *p_ == ']') { ++p_; break; }
                fail("expected ',' or ']'");
            }
        } else if (c == '"') {
            v.kind = Value::String;
            v.str = string();
        } else if (lit("true")) {
            v.kind = Value::Bool;
            v.b = true;
        } else if (lit("false")) {
            v.kind = Value::Bool;
        } else if (lit("null")) {
            v.kind = Value::Null;
        } else {
            v = number();
        }
        return v;
    }
};

inline bool valid_utf8(const char *s, size_t n) {
    const unsigned char *p = (const unsigned char *)s, *e = p + n;
    while (p < e) {
        const unsigned char c = *p++;
        int more;
        uint32_t cp;
        if (c < 0x80) continue;
        else if ((c & 0xE0) == 0xC0) { more = 1; cp = c & 0x1F; }
        else if ((c & 0xF0) == 0xE0) { more = 2; cp = c & 0x0F; }
        else if ((c & 0xF8) == 0xF0) { more = 3; cp = c & 0x07; }
        else return false;
        if (e - p < more) return false;
        for (int k = 0; k < more; ++k) {
            if ((*p & 0xC0) != 0x80) return false;
            cp = (cp << 6) | (*p++ & 0x3F);
        }
        if ((more == 1 && cp < 0x80) || (more == 2 && cp < 0x800) || (more == 3 && (cp < 0x10000 || cp > 0x10FFFF)) ||
            (cp >= 0xD800 && cp < 0xE000))
            return false;
    }
    return true;
}

inline void quote(std::string &o, const std::string &s) {
    o += '"';
    for (const unsigned char c : s) {
        switch (c) {
            case '"': o += "\\\""; break;
            case '\\': o += "\\\\"; break;
            case '\n': o += "\\n"; break;
            case '\r': o += "\\r"; break;
            case '\t': o += "\\t"; break;
            default:
                if (c < 0x20) {
                    char buf[8];
                    snprintf(buf, sizeof buf, "\\u%04x", c);
                    o += buf;
                } else {
                    o += (char)c;  // UTF-8 passes through
                }
        }
    }
    o += '"';
}

}  // namespace json

// safetensors dtype string -> bytes per element (0: not a dtype of the format)
inline size_t dtype_size(const std::string &d) {
    static const std::pair<const char *, size_t> table[] = {
        {"F64", 8}, {"F32", 4}, {"F16", 2}, {"BF16", 2}, {"I64", 8}, {"I32", 4}, {"I16", 2}, {"I8", 1},
        {"U8", 1},  {"U16", 2}, {"U32", 4}, {"U64", 8},  {"BOOL", 1}};
    for (const auto &t : table)
        if (d == t.first) return t.second;
    return 0;
}

struct Tensor {
    std::string dtype;
    std::vector<uint64_t> shape;
    const uint8_t *data = nullptr;  // into the file's mapping (File) or the caller's memory (write_file)
    size_t nbytes = 0;
    uint64_t elements() const {
        uint64_t n = 1;
        for (uint64_t d : shape) n *= d;
        return n;
    }
};

// The fields of QuantizedTensor (quantize.rs:150-185) as host views.
struct Quantized {
    std::string name;
    int bits = 8;                     // 8 or 4 (one code per byte either way)
    std::string mode;                 // "symmetric" | "asymmetric"
    std::string granularity;          // "per_tensor" | "per_channel"
    std::string original_dtype;       // safetensors dtype string of the source tensor
    std::vector<uint64_t> shape;
    const int8_t *codes = nullptr;    // shape's element count
    // n_scales little-endian f64 values each, as raw bytes: entries sit back to back in the file, so
    // these need not be 8-byte aligned.  Copy them (cudaMemcpy, memcpy) or read them through scale() /
    // zero_point(); do not cast the pointers to double *.
    const uint8_t *scales = nullptr;
    const uint8_t *zero_points = nullptr;
    size_t n_scales = 0;

    double scale(size_t i) const { return f64_at(scales, i); }
    double zero_point(size_t i) const { return f64_at(zero_points, i); }
    static double f64_at(const uint8_t *p, size_t i) {
        uint64_t bits = 0;
        for (int k = 7; k >= 0; --k) bits = (bits << 8) | p[8 * i + k];
        double d;
        memcpy(&d, &bits, 8);
        return d;
    }
};

constexpr uint64_t kMaxHeaderBytes = 100000000;  // the reference's sanity limit (safetensors.rs:383-388)
constexpr const char *kQuantizedKey = "shrew.quantized";

class File {
  public:
    static File open(const std::string &path) {
        File f;
        f.map_ = std::make_shared<Mapping>(path);
        f.parse();
        return f;
    }
    const std::map<std::string, std::string> &metadata() const { return metadata_; }
    const std::vector<std::string> &names() const { return order_; }  // header order
    const Tensor *find(const std::string &name) const {
        auto it = tensors_.find(name);
        return it == tensors_.end() ? nullptr : &it->second;
    }
    const Tensor &at(const std::string &name) const {
        const Tensor *t = find(name);
        if (!t) throw FormatError("no tensor named '" + name + "'");
        return *t;
    }

    // The quantized records the metadata describes, reassembled and checked, in the description's order.
    std::vector<Quantized> quantized() const {
        std::vector<Quantized> out;
        auto it = metadata_.find(kQuantizedKey);
        if (it == metadata_.end()) return out;
        json::Value desc;
        try {
            desc = json::Parser(it->second.data(), it->second.size()).parse_document();
        } catch (const FormatError &e) {
            throw FormatError(std::string("metadata '") + kQuantizedKey + "' is not JSON: " + e.what());
        }
        if (desc.kind != json::Value::Object) throw FormatError(std::string("metadata '") + kQuantizedKey + "' is not an object");
        for (const json::Member &m : desc.obj) {
            const std::string &name = m.first;
            const json::Value &d = m.second;
            Quantized q;
            q.name = name;
            const Tensor *part[3];
            static const char *suffix[3] = {".qweight", ".scales", ".zero_points"};
            static const char *want_dtype[3] = {"I8", "F64", "F64"};
            for (int k = 0; k < 3; ++k) {
                part[k] = find(name + suffix[k]);
                if (!part[k]) throw FormatError("quantized record '" + name + "': entry '" + name + suffix[k] + "' is missing");
                if (part[k]->dtype != want_dtype[k])
                    throw FormatError("quantized record '" + name + "': '" + name + suffix[k] + "' has dtype " + part[k]->dtype +
                                      ", expected " + want_dtype[k]);
            }
            const json::Value *bits = d.kind == json::Value::Object ? d.get("bits") : nullptr;
            const json::Value *mode = bits ? d.get("mode") : nullptr;
            const json::Value *gran = bits ? d.get("granularity") : nullptr;
            const json::Value *orig = bits ? d.get("original_dtype") : nullptr;
            const bool ok = bits && mode && gran && orig && bits->kind == json::Value::Number && bits->is_int &&
                            (bits->i == 4 || bits->i == 8) && mode->kind == json::Value::String &&
                            (mode->str == "symmetric" || mode->str == "asymmetric") && gran->kind == json::Value::String &&
                            (gran->str == "per_tensor" || gran->str == "per_channel") && orig->kind == json::Value::String &&
                            dtype_size(orig->str) != 0;
            if (!ok) throw FormatError("quantized record '" + name + "': bad description");
            q.bits = (int)bits->i;
            q.mode = mode->str;
            q.granularity = gran->str;
            q.original_dtype = orig->str;
            q.shape = part[0]->shape;
            const uint64_t rows = q.shape.empty() ? 1 : q.shape[0];
            const uint64_t want = (q.granularity == "per_channel" && !q.shape.empty()) ? rows : 1;
            for (int k = 1; k < 3; ++k)
                if (part[k]->shape.size() != 1 || part[k]->shape[0] != want)
                    throw FormatError("quantized record '" + name + "': wrong number of scales for granularity " + q.granularity);
            q.codes = reinterpret_cast<const int8_t *>(part[0]->data);
            q.scales = part[1]->data;
            q.zero_points = part[2]->data;
            q.n_scales = (size_t)want;
            out.push_back(std::move(q));
        }
        return out;
    }

  private:
    struct Mapping {
        const uint8_t *base = nullptr;
        size_t size = 0;
        explicit Mapping(const std::string &path) {
            const int fd = ::open(path.c_str(), O_RDONLY);
            if (fd < 0) throw FormatError("cannot open '" + path + "'");
            struct stat sb;
            if (fstat(fd, &sb) != 0) { ::close(fd); throw FormatError("cannot stat '" + path + "'"); }
            size = (size_t)sb.st_size;
            if (size > 0) {
                void *p = mmap(nullptr, size, PROT_READ, MAP_PRIVATE, fd, 0);
                if (p == MAP_FAILED) { ::close(fd); throw FormatError("cannot map '" + path + "'"); }
                base = static_cast<const uint8_t *>(p);
            }
            ::close(fd);
        }
        ~Mapping() {
            if (base) munmap(const_cast<uint8_t *>(base), size);
        }
        Mapping(const Mapping &) = delete;
        Mapping &operator=(const Mapping &) = delete;
    };

    std::shared_ptr<Mapping> map_;  // views stay valid while any copy of the File lives
    std::map<std::string, std::string> metadata_;
    std::map<std::string, Tensor> tensors_;
    std::vector<std::string> order_;

    void parse() {
        const uint8_t *base = map_->base;
        const size_t size = map_->size;
        if (size < 8) throw FormatError("file shorter than the 8-byte header length");
        uint64_t hlen = 0;
        for (int k = 7; k >= 0; --k) hlen = (hlen << 8) | base[k];
        if (hlen > kMaxHeaderBytes) throw FormatError("header size " + std::to_string(hlen) + " bytes is unreasonably large");
        if (8 + hlen > size) throw FormatError("header runs past the end of the file");
        const char *htext = reinterpret_cast<const char *>(base + 8);
        if (!json::valid_utf8(htext, (size_t)hlen)) throw FormatError("invalid header: not UTF-8");
        const json::Value root = json::Parser(htext, (size_t)hlen).parse_document();
        if (root.kind != json::Value::Object) throw FormatError("header is not a JSON object");
        const uint64_t data_len = size - 8 - hlen;
        const uint8_t *data = base + 8 + hlen;
        struct Span { uint64_t start, end; const std::string *name; };
        std::vector<Span> spans;
        for (const json::Member &m : root.obj) {
            const std::string &key = m.first;
            const json::Value &val = m.second;
            if (key == "__metadata__") {
                if (val.kind != json::Value::Object) throw FormatError("__metadata__ is not an object");
                for (const json::Member &kv : val.obj) {
                    if (kv.second.kind != json::Value::String) throw FormatError("__metadata__ values must be strings");
                    metadata_[kv.first] = kv.second.str;
                }
                continue;
            }
            if (tensors_.count(key)) throw FormatError("duplicate tensor name '" + key + "'");
            if (val.kind != json::Value::Object) throw FormatError("entry '" + key + "' is not an object");
            const json::Value *dt = val.get("dtype"), *sh = val.get("shape"), *off = val.get("data_offsets");
            Tensor t;
            if (!dt || dt->kind != json::Value::String || dtype_size(dt->str) == 0)
                throw FormatError("'" + key + "': unsupported dtype");
            t.dtype = dt->str;
            if (!sh || sh->kind != json::Value::Array) throw FormatError("'" + key + "': bad shape");
            uint64_t count = 1;
            for (const json::Value &d : sh->arr) {
                if (d.kind != json::Value::Number || !d.is_int || d.i < 0) throw FormatError("'" + key + "': bad shape");
                t.shape.push_back((uint64_t)d.i);
                if (d.i != 0 && count > UINT64_MAX / (uint64_t)d.i / 16) throw FormatError("'" + key + "': bad shape (too large)");
                count *= (uint64_t)d.i;
            }
            if (!off || off->kind != json::Value::Array || off->arr.size() != 2 || off->arr[0].kind != json::Value::Number ||
                off->arr[1].kind != json::Value::Number || !off->arr[0].is_int || !off->arr[1].is_int || off->arr[0].i < 0 ||
                off->arr[1].i < 0)
                throw FormatError("'" + key + "': data_offsets must be two non-negative integers");
            const uint64_t start = (uint64_t)off->arr[0].i, end = (uint64_t)off->arr[1].i;
            if (end < start || end > data_len)
                throw FormatError("'" + key + "': data_offsets [" + std::to_string(start) + "," + std::to_string(end) +
                                  "] outside the " + std::to_string(data_len) + "-byte data section");
            const uint64_t expect = count * dtype_size(t.dtype);
            if (end - start != expect)
                throw FormatError("'" + key + "': expected " + std::to_string(expect) + " bytes for its shape of " + t.dtype +
                                  ", got " + std::to_string(end - start));
            t.data = data + start;
            t.nbytes = (size_t)expect;
            auto ins = tensors_.emplace(key, std::move(t));
            order_.push_back(key);
            spans.push_back(Span{start, end, &ins.first->first});
        }
        std::sort(spans.begin(), spans.end(), [](const Span &a, const Span &b) {
            return a.start != b.start ? a.start < b.start : a.end < b.end;
        });
        uint64_t pos = 0;
        for (const Span &s : spans) {
            if (s.start != pos)
                throw FormatError("'" + *s.name + "': data section has a hole or an overlap at byte " + std::to_string(pos));
            pos = s.end;
        }
        if (pos != data_len) throw FormatError(std::to_string(data_len - pos) + " trailing bytes not covered by any entry");
    }
};

// Writes the tensors in the given order, back to back; "format": "shrew" is added to the metadata like the
// reference's writer does (safetensors.rs:360-361); the header is padded with spaces to a multiple of 8
// bytes.  The file appears under its name only when complete (written beside it, then renamed).
inline void write_file(const std::string &path, const std::vector<std::pair<std::string, Tensor>> &tensors,
                       const std::map<std::string, std::string> &metadata = {}) {
    std::string h = "{\"__metadata__\":{";
    std::map<std::string, std::string> md = metadata;
    if (!md.count("format")) md["format"] = "shrew";
    bool first = true;
    // "format" first, the rest in key order (any order is valid; this one is reproducible)
    auto put_kv = [&](const std::string &k, const std::string &v) {
        if (!first) h += ',';
        first = false;
        json::quote(h, k);
        h += ':';
        json::quote(h, v);
    };
    put_kv("format", md["format"]);
    for (const auto &kv : md)
        if (kv.first != "format") put_kv(kv.first, kv.second);
    h += '}';
    uint64_t off = 0;
    std::map<std::string, int> seen;
    for (const auto &nt : tensors) {
        const Tensor &t = nt.second;
        if (nt.first == "__metadata__" || seen[nt.first]++) throw FormatError("duplicate tensor name '" + nt.first + "'");
        const size_t es = dtype_size(t.dtype);
        if (es == 0) throw FormatError("unsupported dtype '" + t.dtype + "' for '" + nt.first + "'");
        if (t.elements() * es != t.nbytes)
            throw FormatError("'" + nt.first + "': " + std::to_string(t.nbytes) + " bytes of data for its shape of " + t.dtype);
        h += ',';
        json::quote(h, nt.first);
        h += ":{\"dtype\":\"" + t.dtype + "\",\"shape\":[";
        for (size_t k = 0; k < t.shape.size(); ++k) h += (k ? "," : "") + std::to_string(t.shape[k]);
        h += "],\"data_offsets\":[" + std::to_string(off) + "," + std::to_string(off + t.nbytes) + "]}";
        off += t.nbytes;
    }
    h += '}';
    while (h.size() % 8) h += ' ';
    const std::string tmp = path + ".tmp." + std::to_string((long)getpid());
    FILE *f = fopen(tmp.c_str(), "wb");
    if (!f) throw FormatError("cannot create '" + tmp + "'");
    uint8_t len[8];
    for (int k = 0; k < 8; ++k) len[k] = (uint8_t)((uint64_t)h.size() >> (8 * k));
    bool ok = fwrite(len, 1, 8, f) == 8 && fwrite(h.data(), 1, h.size(), f) == h.size();
    for (const auto &nt : tensors)
        if (ok && nt.second.nbytes) ok = fwrite(nt.second.data, 1, nt.second.nbytes, f) == nt.second.nbytes;
    ok = (fclose(f) == 0) && ok;
    if (!ok || rename(tmp.c_str(), path.c_str()) != 0) {
        remove(tmp.c_str());
        throw FormatError("cannot write '" + path + "'");
    }
}

// The three entries and the description of one quantized record, appended to `tensors` / `desc`;
// pass `desc` through quantized_metadata() to get the metadata map for write_file.
struct Description {
    std::string name;
    int bits;
    std::string mode, granularity, original_dtype;
};

inline void append_quantized(std::vector<std::pair<std::string, Tensor>> &tensors, std::vector<Description> &desc,
                             const Quantized &q) {
    uint64_t count = 1;
    for (uint64_t d : q.shape) count *= d;
    const uint64_t rows = q.shape.empty() ? 1 : q.shape[0];
    const uint64_t want = (q.granularity == "per_channel" && !q.shape.empty()) ? rows : 1;
    if (q.n_scales != want)
        throw FormatError("'" + q.name + "': " + std::to_string(q.n_scales) + " scales for granularity " + q.granularity);
    if (q.bits != 4 && q.bits != 8) throw FormatError("'" + q.name + "': records hold 8-bit or 4-bit codes (one per byte)");
    if ((q.mode != "symmetric" && q.mode != "asymmetric") || (q.granularity != "per_tensor" && q.granularity != "per_channel") ||
        dtype_size(q.original_dtype) == 0)
        throw FormatError("'" + q.name + "': bad description");
    Tensor c{"I8", q.shape, reinterpret_cast<const uint8_t *>(q.codes), (size_t)count};
    Tensor s{"F64", {want}, q.scales, (size_t)want * 8};
    Tensor z{"F64", {want}, q.zero_points, (size_t)want * 8};
    tensors.emplace_back(q.name + ".qweight", std::move(c));
    tensors.emplace_back(q.name + ".scales", std::move(s));
    tensors.emplace_back(q.name + ".zero_points", std::move(z));
    desc.push_back(Description{q.name, q.bits, q.mode, q.granularity, q.original_dtype});
}

inline std::map<std::string, std::string> quantized_metadata(const std::vector<Description> &desc) {
    std::vector<const Description *> sorted;
    for (const Description &d : desc) sorted.push_back(&d);
    std::sort(sorted.begin(), sorted.end(), [](const Description *a, const Description *b) { return a->name < b->name; });
    std::string j = "{";
    for (size_t k = 0; k < sorted.size(); ++k) {
        const Description &d = *sorted[k];
        if (k) j += ',';
        json::quote(j, d.name);
        j += ":{\"bits\":" + std::to_string(d.bits) + ",\"granularity\":";
        json::quote(j, d.granularity);
        j += ",\"mode\":";
        json::quote(j, d.mode);
        j += ",\"original_dtype\":";
        json::quote(j, d.original_dtype);
        j += '}';
    }
    j += '}';
    return {{kQuantizedKey, j}};
}

}  // namespace st
}  // namespace shrewq
