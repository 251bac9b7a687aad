// C++17 mirror of rusty-loader's WeightsContext for the quantised-linear path
// (rusty-loader/src/lib.rs:97-218): memory-mapped safetensors files, a name -> file map, tensor views, and the two
// ways a quantised tensor reaches the device:
//
//   upload_quantized(name, ctx, engine)  what the reference does: three uploads and the affine_dequantize kernel into
//                                        a full f32 tensor (lib.rs:155-218);
//   upload_qlinear(name, ctx, ...)       the weight stays at one byte per element and comes back as the fused linear's
//                                        QWeight; with (rank, world) only this rank's output rows and groups are uploaded.
//
// On-disk contract (lib.rs:161-187, rusty-graph/src/model_builder.rs:68-72): `name.weight` bytes with the shape taken
// verbatim, `name.scales` and `name.biases` f32, one pair per 64 consecutive flat elements; quantised iff `name.scales`
// exists.  The container: 8-byte little-endian header length, a JSON object {name: {dtype, shape, data_offsets}}, then
// the byte buffer.  Only that flat header shape is parsed here (strings, integers, arrays of integers, one level of
// objects, and a `__metadata__` object of strings that is skipped).
//
// Header-only; needs rusty_host.hpp and the C ABI.  Errors are LoaderError (Io / Safetensors / Json / MissingWeight,
// the variants of lib.rs:15-25).
#pragma once

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <cstdint>
#include <cstring>
#include <algorithm>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "rusty_host.hpp"

namespace rusty {

struct LoaderError : std::runtime_error {
    std::string kind;
    LoaderError(std::string k, const std::string& msg) : std::runtime_error(k + ": " + msg), kind(std::move(k)) {}
};

struct TensorInfo {
    std::string dtype;           // "U8", "I8", "F32", ...
    std::vector<size_t> shape;
    size_t begin = 0, end = 0;   // byte range inside the file's data buffer
};

namespace detail {

inline size_t dtype_size(const std::string& d) {
    if (d == "U8" || d == "I8" || d == "BOOL") return 1;
    if (d == "I16" || d == "U16" || d == "F16" || d == "BF16") return 2;
    if (d == "I32" || d == "U32" || d == "F32") return 4;
    if (d == "I64" || d == "U64" || d == "F64") return 8;
    return 0;
}

// Minimal parser for the safetensors header.
class HeaderParser {
public:
    HeaderParser(const char* p, size_t n, std::string file) : p_(p), end_(p + n), file_(std::move(file)) {}
    std::map<std::string, TensorInfo> parse() {
        std::map<std::string, TensorInfo> out;
        ws();
        expect('{');
        ws();
        if (peek() == '}') return out;
        for (;;) {
            ws();
            std::string key = string();
            ws();
            expect(':');
            ws();
            if (key == "__metadata__") {
                skip_value();
            } else {
                out[key] = entry(key);
            }
            ws();
            if (peek() == ',') {
                ++p_;
                continue;
            }
            expect('}');
            break;
        }
        return out;
    }

private:
    [[noreturn]] void bad(const std::string& what) const { throw LoaderError("Json", file_ + ": " + what); }
    char peek() const { return p_ < end_ ? *p_ : '\0'; }
    void ws() {
        while (p_ < end_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\t' || *p_ == '\r')) ++p_;
    }
    void expect(char c) {
        if (peek() != c) bad(std::string("expected '") + c + "'");
        ++p_;
    }
    std::string string() {
        expect('"');
        std::string s;
        while (p_ < end_ && *p_ != '"') {
            if (*p_ == '\\') {
                ++p_;
                if (p_ >= end_) bad("unterminated escape");
                switch (*p_) {
                    case 'n': s += '\n'; break;
                    case 't': s += '\t'; break;
                    case 'u':  // tensor names are ASCII in practice; keep the escape verbatim
                        s += "\\u";
                        break;
                    default: s += *p_;
                }
                ++p_;
            } else {
                s += *p_++;
            }
        }
        expect('"');
        return s;
    }
    size_t integer() {
        if (peek() < '0' || peek() > '9') bad("expected a non-negative integer");
        size_t v = 0;
        while (peek() >= '0' && peek() <= '9') {
            const size_t d = (size_t)(*p_++ - '0');
            if (v > (SIZE_MAX - d) / 10) bad("integer overflow");
            v = v * 10 + d;
        }
        return v;
    }
    std::vector<size_t> int_array() {
        std::vector<size_t> v;
        expect('[');
        ws();
        if (peek() == ']') {
            ++p_;
            return v;
        }
        for (;;) {
            ws();
            v.push_back(integer());
            ws();
            if (peek() == ',') {
                ++p_;
                continue;
            }
            expect(']');
            break;
        }
        return v;
    }
    void skip_value() {  // strings, numbers, literals, nested arrays / objects
        ws();
        const char c = peek();
        if (c == '"') {
            string();
        } else if (c == '{' || c == '[') {
            const char close = c == '{' ? '}' : ']';
            ++p_;
            ws();
            if (peek() == close) {
                ++p_;
                return;
            }
            for (;;) {
                ws();
                if (c == '{') {
                    string();
                    ws();
                    expect(':');
                }
                skip_value();
                ws();
                if (peek() == ',') {
                    ++p_;
                    continue;
                }
                expect(close);
                break;
            }
        } else {
            while (p_ < end_ && *p_ != ',' && *p_ != '}' && *p_ != ']') ++p_;
        }
    }
    TensorInfo entry(const std::string& name) {
        TensorInfo t;
        bool have_d = false, have_s = false, have_o = false;
        expect('{');
        for (;;) {
            ws();
            const std::string k = string();
            ws();
            expect(':');
            ws();
            if (k == "dtype") {
                t.dtype = string();
                have_d = true;
            } else if (k == "shape") {
                t.shape = int_array();
                have_s = true;
            } else if (k == "data_offsets") {
                const std::vector<size_t> o = int_array();
                if (o.size() != 2) throw LoaderError("Safetensors", file_ + ": " + name + ": data_offsets needs two entries");
                t.begin = o[0];
                t.end = o[1];
                have_o = true;
            } else {
                skip_value();
            }
            ws();
            if (peek() == ',') {
                ++p_;
                continue;
            }
            expect('}');
            break;
        }
        if (!have_d || !have_s || !have_o) throw LoaderError("Safetensors", file_ + ": malformed entry " + name);
        return t;
    }
    const char* p_;
    const char* end_;
    std::string file_;
};

class MappedFile {
public:
    explicit MappedFile(const std::string& path) : path_(path) {
        const int fd = ::open(path.c_str(), O_RDONLY);
        if (fd < 0) throw LoaderError("Io", path + ": " + std::strerror(errno));
        struct stat st;
        if (::fstat(fd, &st) != 0) {
            ::close(fd);
            throw LoaderError("Io", path + ": " + std::strerror(errno));
        }
        size_ = (size_t)st.st_size;
        if (size_ > 0) {
            void* m = ::mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd, 0);
            if (m == MAP_FAILED) {
                ::close(fd);
                throw LoaderError("Io", path + ": mmap: " + std::strerror(errno));
            }
            base_ = static_cast<const unsigned char*>(m);
        }
        ::close(fd);
        if (size_ < 8) throw LoaderError("Safetensors", path + ": shorter than the 8-byte header length");
        uint64_t n = 0;
        for (int i = 7; i >= 0; --i) n = (n << 8) | base_[i];
        if (n > size_ - 8 || n > (100ull << 20)) throw LoaderError("Safetensors", path + ": header length does not fit the file");
        data_ = base_ + 8 + n;
        data_len_ = size_ - 8 - (size_t)n;
        entries_ = HeaderParser(reinterpret_cast<const char*>(base_ + 8), (size_t)n, path).parse();
        for (const auto& kv : entries_) {
            const TensorInfo& t = kv.second;
            const size_t es = dtype_size(t.dtype);
            if (es == 0) throw LoaderError("Safetensors", path + ": " + kv.first + ": unknown dtype " + t.dtype);
            // checked products: a crafted shape such as [2^32, 2^32] must not wrap to a small element count
            size_t count = 1, nbytes = 0;
            bool overflow = false;
            for (size_t d : t.shape) overflow = overflow || __builtin_mul_overflow(count, d, &count);
            overflow = overflow || __builtin_mul_overflow(count, es, &nbytes);
            if (overflow) throw LoaderError("Safetensors", path + ": " + kv.first + ": shape overflows the address space");
            if (t.begin > t.end || t.end > data_len_ || t.end - t.begin != nbytes)
                throw LoaderError("Safetensors", path + ": " + kv.first + ": data_offsets do not match shape and dtype");
        }
        // no two tensors may share bytes (the reference's safetensors crate validates the same)
        std::vector<std::pair<size_t, size_t>> ranges;
        for (const auto& kv : entries_)
            if (kv.second.end > kv.second.begin) ranges.emplace_back(kv.second.begin, kv.second.end);
        std::sort(ranges.begin(), ranges.end());
        for (size_t i = 1; i < ranges.size(); ++i)
            if (ranges[i].first < ranges[i - 1].second) throw LoaderError("Safetensors", path + ": tensor byte ranges overlap");
    }
    ~MappedFile() {
        if (base_) ::munmap(const_cast<unsigned char*>(base_), size_);
    }
    MappedFile(const MappedFile&) = delete;
    MappedFile& operator=(const MappedFile&) = delete;
    const std::map<std::string, TensorInfo>& entries() const { return entries_; }
    const unsigned char* data(const TensorInfo& t) const { return data_ + t.begin; }

private:
    std::string path_;
    const unsigned char* base_ = nullptr;
    const unsigned char* data_ = nullptr;
    size_t size_ = 0, data_len_ = 0;
    std::map<std::string, TensorInfo> entries_;
};

}  // namespace detail

class WeightsContext {
public:
    static constexpr size_t GROUP = 64;  // elements per (scale, bias) pair (kernels.wgsl:395)

    void load_file(const std::string& path) {
        auto f = std::make_shared<detail::MappedFile>(path);
        const std::string key = path.substr(path.find_last_of('/') == std::string::npos ? 0 : path.find_last_of('/') + 1);
        files_[key] = f;
        for (const auto& kv : f->entries()) weight_map_[kv.first] = key;
    }
    bool contains(const std::string& name) const { return weight_map_.count(name) != 0; }
    // (shape, dtype) or nullptr
    const TensorInfo* get_tensor_info(const std::string& name) const {
        auto it = weight_map_.find(name);
        if (it == weight_map_.end()) return nullptr;
        return &files_.at(it->second)->entries().at(name);
    }
    // the tensor's bytes (a view of the mapping) and its info
    std::pair<const unsigned char*, const TensorInfo*> read_bytes(const std::string& name) const {
        auto it = weight_map_.find(name);
        if (it == weight_map_.end()) throw LoaderError("MissingWeight", name);
        const auto& f = files_.at(it->second);
        const TensorInfo& t = f->entries().at(name);
        return {f->data(t), &t};
    }
    bool is_quantized(const std::string& name) const { return contains(name + ".scales"); }

    struct QuantizedShard {
        const unsigned char* q;  // rows x cols bytes
        const float* scales;
        const float* biases;
        size_t rows, cols, groups;
        // column shards of [in,out] storage are gathered copies (a column block is not contiguous in the file)
        std::shared_ptr<std::vector<unsigned char>> own_q;
        std::shared_ptr<std::vector<float>> own_s, own_b;
    };
    // Host views of the part of `name` that `rank` of `world` keeps: a block of output features made of whole groups --
    // rows of an [out,in] matrix whose input width is a multiple of 64, or columns of an [in,out] matrix whose output
    // width is a multiple of 64 * world.
    QuantizedShard quantized_shard(const std::string& name, int layout = RUSTY_CUDA_LAYOUT_KN, int rank = 0, int world = 1) const {
        const std::string wn = name + ".weight";
        if (!contains(wn)) throw LoaderError("MissingWeight", wn);
        auto w = read_bytes(wn);
        auto s = read_bytes(name + ".scales");
        auto b = read_bytes(name + ".biases");
        if (w.second->shape.size() != 2) throw LoaderError("Safetensors", wn + ": a linear weight has two dimensions");
        const size_t rows = w.second->shape[0], cols = w.second->shape[1], total = rows * cols;
        if (w.second->end - w.second->begin != total) throw LoaderError("Safetensors", wn + ": not one byte per element");
        const size_t groups = (total + GROUP - 1) / GROUP;
        if ((s.second->end - s.second->begin) / 4 < groups || (b.second->end - b.second->begin) / 4 < groups)
            throw LoaderError("Safetensors", name + ": too few (scale, bias) pairs");
        QuantizedShard out{w.first, reinterpret_cast<const float*>(s.first), reinterpret_cast<const float*>(b.first), rows, cols, groups, {}, {}, {}};
        if (world > 1 && layout == RUSTY_CUDA_LAYOUT_KN) {
            // [in,out]: rows = input features, cols = output features; the groups of 64 run along the columns
            if (cols % ((size_t)world * GROUP) != 0) throw LoaderError("Safetensors", name + ": cannot be cut into column shards of whole groups");
            const size_t nl = cols / (size_t)world, gpr = cols / GROUP, gl = nl / GROUP;
            out.own_q = std::make_shared<std::vector<unsigned char>>(rows * nl);
            out.own_s = std::make_shared<std::vector<float>>(rows * gl);
            out.own_b = std::make_shared<std::vector<float>>(rows * gl);
            for (size_t r = 0; r < rows; ++r) {
                std::memcpy(out.own_q->data() + r * nl, out.q + r * cols + (size_t)rank * nl, nl);
                std::memcpy(out.own_s->data() + r * gl, out.scales + r * gpr + (size_t)rank * gl, gl * sizeof(float));
                std::memcpy(out.own_b->data() + r * gl, out.biases + r * gpr + (size_t)rank * gl, gl * sizeof(float));
            }
            out.q = out.own_q->data();
            out.scales = out.own_s->data();
            out.biases = out.own_b->data();
            out.cols = nl;
            out.groups = rows * gl;
        } else if (world > 1) {
            if (rows % (size_t)world != 0 || cols % GROUP != 0)
                throw LoaderError("Safetensors", name + ": cannot be cut into row shards of whole groups");
            const size_t nl = rows / (size_t)world, gpr = cols / GROUP;
            out.q += (size_t)rank * nl * cols;
            out.scales += (size_t)rank * nl * gpr;
            out.biases += (size_t)rank * nl * gpr;
            out.rows = nl;
            out.groups = nl * gpr;
        }
        return out;
    }

    // The reference's load path: an f32 copy made by the dequantize kernel (lib.rs:155-218).
    UnifiedTensor upload_quantized(const std::string& name, const CudaContext& ctx, const ComputeEngine& engine) const {
        const QuantizedShard p = quantized_shard(name);
        UnifiedTensor q = UnifiedTensor::from_bytes(ctx, p.q, p.rows * p.cols, {p.rows * p.cols}, DType::U8);
        UnifiedTensor s = UnifiedTensor::make(ctx, p.scales, {p.groups});
        UnifiedTensor b = UnifiedTensor::make(ctx, p.biases, {p.groups});
        UnifiedTensor out = UnifiedTensor::empty(ctx, {p.rows, p.cols});
        engine.affine_dequantize(ctx, q, s, b, out);
        return out;
    }
    // The fused path: the weight stays one byte per element.
    std::shared_ptr<QWeight> upload_qlinear(const std::string& name, const CudaContext& ctx, int layout = RUSTY_CUDA_LAYOUT_KN, int rank = 0,
                                            int world = 1) const {
        const QuantizedShard p = quantized_shard(name, layout, rank, world);
        UnifiedTensor q = UnifiedTensor::from_bytes(ctx, p.q, p.rows * p.cols, {p.rows, p.cols}, DType::U8);
        UnifiedTensor s = UnifiedTensor::make(ctx, p.scales, {p.groups});
        UnifiedTensor b = UnifiedTensor::make(ctx, p.biases, {p.groups});
        const uint32_t n = (uint32_t)(layout == RUSTY_CUDA_LAYOUT_NK ? p.rows : p.cols), k = (uint32_t)(layout == RUSTY_CUDA_LAYOUT_NK ? p.cols : p.rows);
        return std::make_shared<QWeight>(ctx, q, s, &b, n, k, layout, RUSTY_CUDA_QMODE_AFFINE_G64);
    }

private:
    std::map<std::string, std::shared_ptr<detail::MappedFile>> files_;
    std::map<std::string, std::string> weight_map_;
};

}  // namespace rusty
