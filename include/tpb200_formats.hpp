// tpb200_formats.hpp -- read-only checkpoint containers for the quantized-linear path,
// header-only C++: safetensors with the reference's ConvRot weight resolution, and GGUF.
//
// Mirrors src/core/safetensors.zig, src/core/gguf.zig:1-60 / :200-295 and the Loader of
// src/models/dit.zig:690-722 (int4 is told from int8 by the halved column count; every
// ConvRot weight has a per-row `<name>_scale`).  Files are memory-mapped; tensor bytes are
// views into the mapping and stay valid while the reader object lives.  Failures throw
// tpbfmt::Error whose `name` is the reference's error tag (MissingTensor, ShapeMismatch,
// InvalidHeader, ...).  The Python twin is tensorpencil_b200/formats.py.
#ifndef TPB200_FORMATS_HPP
#define TPB200_FORMATS_HPP

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdint>
#include <cstring>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

namespace tpbfmt {

struct Error : std::runtime_error {
    std::string name;
    Error(const std::string &n, const std::string &detail = "") : std::runtime_error(detail.empty() ? n : n + ": " + detail), name(n) {}
};

struct TensorView {
    std::string name, dtype;        // the container's tag: "I8", "U8", "F32", "BF16", "Q4_K", ...
    std::vector<int64_t> shape;     // row-major
    const uint8_t *data = nullptr;
    size_t bytes = 0;
    int64_t elemCount() const {
        int64_t n = 1;
        for (int64_t s : shape) n *= s;
        return n;
    }
    // toF32Alloc: f32 / f16 / bf16 tensors as float
    std::vector<float> toF32() const {
        std::vector<float> out((size_t)elemCount());
        if (dtype == "F32") {
            std::memcpy(out.data(), data, out.size() * 4);
        } else if (dtype == "BF16") {
            for (size_t i = 0; i < out.size(); i++) {
                uint16_t h;
                std::memcpy(&h, data + 2 * i, 2);
                const uint32_t u = (uint32_t)h << 16;
                std::memcpy(&out[i], &u, 4);
            }
        } else if (dtype == "F16") {
            for (size_t i = 0; i < out.size(); i++) {
                uint16_t h;
                std::memcpy(&h, data + 2 * i, 2);
                const uint32_t sign = (uint32_t)(h & 0x8000) << 16, exp = (h >> 10) & 31, man = h & 1023;
                uint32_t u;
                if (exp == 0) {
                    if (man == 0) {
                        u = sign;
                    } else {  // subnormal
                        int e = -1;
                        uint32_t m = man;
                        while (!(m & 1024)) { m <<= 1; e++; }
                        u = sign | (uint32_t)(127 - 15 - e) << 23 | (m & 1023) << 13;
                    }
                } else if (exp == 31) {
                    u = sign | 0x7f800000u | man << 13;
                } else {
                    u = sign | (exp + 112) << 23 | man << 13;
                }
                std::memcpy(&out[i], &u, 4);
            }
        } else {
            throw Error("UnsupportedDType", name + ": " + dtype + " has no f32 view");
        }
        return out;
    }
};

class Mapping {
  public:
    explicit Mapping(const std::string &path) {
        fd_ = ::open(path.c_str(), O_RDONLY);
        if (fd_ < 0) throw Error("FileNotFound", path);
        struct stat st;
        if (fstat(fd_, &st) != 0 || st.st_size <= 0) {
            ::close(fd_);
            throw Error("FileTooSmall", path);
        }
        size_ = (size_t)st.st_size;
        p_ = static_cast<const uint8_t *>(mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0));
        if (p_ == MAP_FAILED) {
            ::close(fd_);
            throw Error("MapFailed", path);
        }
    }
    ~Mapping() {
        if (p_ && p_ != MAP_FAILED) munmap(const_cast<uint8_t *>(p_), size_);
        if (fd_ >= 0) ::close(fd_);
    }
    Mapping(const Mapping &) = delete;
    Mapping &operator=(const Mapping &) = delete;
    const uint8_t *data() const { return p_; }
    size_t size() const { return size_; }

  private:
    int fd_ = -1;
    const uint8_t *p_ = nullptr;
    size_t size_ = 0;
};

// ---- safetensors ----------------------------------------------------------------------

namespace detail {
// The subset of JSON a safetensors header uses: objects, arrays, strings, integers.
struct Json {
    const char *p, *end;
    void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) p++; }
    bool eat(char c) { ws(); if (p < end && *p == c) { p++; return true; } return false; }
    void need(char c) { if (!eat(c)) throw Error("InvalidHeader", std::string("expected '") + c + "'"); }
    std::string str() {
        ws();
        if (p >= end || *p != '"') throw Error("InvalidHeader", "expected a string");
        p++;
        std::string s;
        while (p < end && *p != '"') {
            if (*p == '\\' && p + 1 < end) {
                p++;
                switch (*p) {
                    case 'n': s += '\n'; break;
                    case 't': s += '\t'; break;
                    case 'u': s += '?'; p += 4; break;  // names in this path are ASCII
                    default: s += *p;
                }
                p++;
            } else {
                s += *p++;
            }
        }
        if (p >= end) throw Error("InvalidHeader", "unterminated string");
        p++;
        return s;
    }
    int64_t integer() {
        ws();
        bool neg = false;
        if (p < end && *p == '-') { neg = true; p++; }
        if (p >= end || *p < '0' || *p > '9') throw Error("InvalidHeader", "expected a number");
        int64_t v = 0;
        while (p < end && *p >= '0' && *p <= '9') v = v * 10 + (*p++ - '0');
        return neg ? -v : v;
    }
    void skipValue() {
        ws();
        if (p >= end) throw Error("InvalidHeader", "truncated");
        if (*p == '"') { str(); return; }
        if (*p == '{') { p++; if (eat('}')) return; do { str(); need(':'); skipValue(); } while (eat(',')); need('}'); return; }
        if (*p == '[') { p++; if (eat(']')) return; do { skipValue(); } while (eat(',')); need(']'); return; }
        while (p < end && *p != ',' && *p != '}' && *p != ']') p++;  // number, true, false, null
    }
};
inline size_t dtypeBytes(const std::string &dt) {
    if (dt == "F32" || dt == "I32") return 4;
    if (dt == "F16" || dt == "BF16") return 2;
    if (dt == "I8" || dt == "U8" || dt == "F8_E4M3") return 1;
    if (dt == "I64") return 8;
    return 0;
}
}  // namespace detail

class SafeTensors {
  public:
    explicit SafeTensors(const std::string &path) : map_(path) {
        if (map_.size() < 8) throw Error("FileTooSmall");
        uint64_t hlen;
        std::memcpy(&hlen, map_.data(), 8);
        if (hlen > map_.size() - 8) throw Error("InvalidHeader", "header length exceeds the file");
        const uint8_t *payload = map_.data() + 8 + hlen;
        const size_t payload_size = map_.size() - 8 - (size_t)hlen;
        detail::Json j{reinterpret_cast<const char *>(map_.data() + 8), reinterpret_cast<const char *>(map_.data() + 8 + hlen)};
        j.need('{');
        if (!j.eat('}')) {
            do {
                const std::string name = j.str();
                j.need(':');
                if (name == "__metadata__") { j.skipValue(); continue; }
                TensorView v;
                v.name = name;
                int64_t lo = 0, hi = 0;
                j.need('{');
                do {
                    const std::string key = j.str();
                    j.need(':');
                    if (key == "dtype") {
                        v.dtype = j.str();
                    } else if (key == "shape") {
                        j.need('[');
                        if (!j.eat(']')) { do { v.shape.push_back(j.integer()); } while (j.eat(',')); j.need(']'); }
                    } else if (key == "data_offsets") {
                        j.need('['); lo = j.integer(); j.need(','); hi = j.integer(); j.need(']');
                    } else {
                        j.skipValue();
                    }
                } while (j.eat(','));
                j.need('}');
                const size_t eb = detail::dtypeBytes(v.dtype);
                if (eb == 0) throw Error("UnsupportedDType", name + ": " + v.dtype);
                for (int64_t s : v.shape) if (s < 0) throw Error("InvalidShape", name);
                if (lo < 0 || hi < lo || (size_t)hi > payload_size || (size_t)(hi - lo) != (size_t)v.elemCount() * eb)
                    throw Error("InvalidOffsets", name);
                v.data = payload + lo;
                v.bytes = (size_t)(hi - lo);
                tensors_[name] = v;
            } while (j.eat(','));
            j.need('}');
        }
    }
    const TensorView *get(const std::string &name) const {
        auto it = tensors_.find(name);
        return it == tensors_.end() ? nullptr : &it->second;
    }
    const std::map<std::string, TensorView> &tensors() const { return tensors_; }

  private:
    Mapping map_;
    std::map<std::string, TensorView> tensors_;
};

struct ConvRotWeight {
    const uint8_t *w = nullptr;     // int8 [rows][cols] (bits 8) or packed nibbles [rows][cols/2] (bits 4)
    size_t w_bytes = 0;
    std::vector<float> row_scale;   // [rows]
    int bits = 0;
    int64_t rows = 0, cols = 0;
};

constexpr int64_t kConvRotGroup = 256;  // src/ops/convrot.zig

// Loader.mat for an int8/int4 ConvRot weight (src/models/dit.zig:690-722).
inline ConvRotWeight loadConvRotWeight(const SafeTensors &st, const std::string &name, int64_t rows, int64_t cols) {
    const TensorView *v = st.get(name);
    if (!v) throw Error("MissingTensor", name);
    const bool halved = v->shape.size() == 2 && v->shape[0] == rows && cols % 2 == 0 && v->shape[1] == cols / 2;
    const bool is_i4 = v->dtype == "U8" || (v->dtype == "I8" && halved);
    if (!is_i4 && v->dtype != "I8") throw Error("UnsupportedCheckpoint", name + ": " + v->dtype + " is not a ConvRot weight");
    const int64_t stored_cols = is_i4 ? cols / 2 : cols;
    if (is_i4 && cols % 2 != 0) throw Error("ShapeMismatch", name);
    if (v->shape.size() != 2 || v->shape[0] != rows || v->shape[1] != stored_cols) throw Error("ShapeMismatch", name);
    const TensorView *sv = st.get(name + "_scale");
    if (!sv) throw Error("MissingTensor", name + "_scale");
    if (sv->elemCount() != rows) throw Error("ShapeMismatch", name + "_scale");
    if (cols % kConvRotGroup != 0) throw Error("ShapeMismatch", name + ": cols is not a multiple of the rotation group");
    ConvRotWeight w;
    w.w = v->data;
    w.w_bytes = v->bytes;
    w.row_scale = sv->toF32();
    w.bits = is_i4 ? 4 : 8;
    w.rows = rows;
    w.cols = cols;
    return w;
}

// ---- GGUF -----------------------------------------------------------------------------

struct GgmlType { const char *tag; int block_elems, block_bytes; };
// ggml type id -> tag and block geometry (src/core/gguf.zig:40-56)
inline const GgmlType *ggmlType(uint32_t id) {
    static const std::map<uint32_t, GgmlType> t = {
        {0, {"F32", 1, 4}},      {1, {"F16", 1, 2}},      {2, {"Q4_0", 32, 18}},    {8, {"Q8_0", 32, 34}},
        {12, {"Q4_K", 256, 144}}, {13, {"Q5_K", 256, 176}}, {14, {"Q6_K", 256, 210}}, {16, {"I8", 1, 1}},
        {20, {"IQ4_NL", 32, 18}}, {26, {"I32", 1, 4}},      {30, {"BF16", 1, 2}}};
    auto it = t.find(id);
    return it == t.end() ? nullptr : &it->second;
}

// llama.cpp tensor names -> the HF-style names the model loaders ask for (src/core/gguf.zig:396-480):
// "blk.<n>.<suffix>" -> "layers.<n>.<HF suffix>" (a suffix without an entry keeps its spelling), the three
// top-level names, everything else unchanged.  Gemma's "sandwich" norms rename three entries (ffn_norm is
// the norm before the feed-forward block there); Gemma 4 adds a per-layer output scale.
inline std::string canonicalName(const std::string &raw, const std::string &arch) {
    static const std::map<std::string, std::string> top = {
        {"token_embd.weight", "embed_tokens.weight"}, {"output_norm.weight", "norm.weight"}, {"output.weight", "lm_head.weight"}};
    static const std::map<std::string, std::string> base = {
        {"attn_norm.weight", "input_layernorm.weight"},
        {"post_attention_norm.weight", "post_attention_layernorm.weight"},
        {"ffn_norm.weight", "post_attention_layernorm.weight"},
        {"attn_q.weight", "self_attn.q_proj.weight"},
        {"attn_k.weight", "self_attn.k_proj.weight"},
        {"attn_v.weight", "self_attn.v_proj.weight"},
        {"attn_output.weight", "self_attn.o_proj.weight"},
        {"attn_q_norm.weight", "self_attn.q_norm.weight"},
        {"attn_k_norm.weight", "self_attn.k_norm.weight"},
        {"ffn_gate.weight", "mlp.gate_proj.weight"},
        {"ffn_up.weight", "mlp.up_proj.weight"},
        {"ffn_down.weight", "mlp.down_proj.weight"}};
    const auto t = top.find(raw);
    if (t != top.end()) return t->second;
    if (raw.compare(0, 4, "blk.") != 0) return raw;
    const size_t dot = raw.find('.', 4);
    if (dot == std::string::npos || dot == 4) return raw;
    const std::string layer = raw.substr(4, dot - 4), suffix = raw.substr(dot + 1);
    for (char c : layer)
        if (c < '0' || c > '9') return raw;
    const bool gemma = arch == "gemma3" || arch == "gemma4";
    std::string mapped = suffix;
    if (gemma && suffix == "ffn_norm.weight") mapped = "pre_feedforward_layernorm.weight";
    else if (gemma && suffix == "post_ffw_norm.weight") mapped = "post_feedforward_layernorm.weight";
    else if (arch == "gemma4" && suffix == "layer_output_scale.weight") mapped = "out_scale.weight";
    else {
        const auto b = base.find(suffix);
        if (b != base.end()) mapped = b->second;
    }
    return "layers." + layer + "." + mapped;
}

class Gguf {
  public:
    explicit Gguf(const std::string &path) : map_(path) {
        if (map_.size() < 24) throw Error("FileTooSmall");
        if (std::memcmp(map_.data(), "GGUF", 4) != 0) throw Error("InvalidMagic");
        pos_ = 4;
        version = take<uint32_t>();
        if (version != 2 && version != 3) throw Error("UnsupportedVersion", std::to_string(version));
        const uint64_t n_tensors = take<uint64_t>(), n_kv = take<uint64_t>();
        for (uint64_t i = 0; i < n_kv; i++) {
            const std::string key = str();
            const uint32_t t = take<uint32_t>();
            value(key, t);
        }
        struct Info { std::string name; std::vector<int64_t> shape; uint32_t tid; uint64_t off; };
        std::vector<Info> infos;
        for (uint64_t i = 0; i < n_tensors; i++) {
            Info in;
            in.name = str();
            const uint32_t nd = take<uint32_t>();
            if (nd > 8) throw Error("InvalidShape", in.name);
            std::vector<int64_t> dims(nd);
            for (auto &d : dims) d = (int64_t)take<uint64_t>();
            in.shape.assign(dims.rbegin(), dims.rend());  // stored fastest-first: reversed to row-major
            in.tid = take<uint32_t>();
            in.off = take<uint64_t>();
            if (!ggmlType(in.tid)) throw Error("UnsupportedTensorType", in.name);
            if (in.off % alignment != 0) throw Error("InvalidOffsets", in.name);
            infos.push_back(in);
        }
        const size_t data_start = (pos_ + alignment - 1) / alignment * alignment;
        for (const Info &in : infos) {
            const GgmlType *gt = ggmlType(in.tid);
            if (tensors_.count(in.name)) throw Error("DuplicateTensor", in.name);
            TensorView v;
            v.name = in.name;
            v.dtype = gt->tag;
            v.shape = in.shape;
            if (!v.shape.empty() && v.shape.back() % gt->block_elems != 0) throw Error("InvalidShape", in.name);
            v.bytes = (size_t)(v.elemCount() / gt->block_elems) * gt->block_bytes;
            if (data_start + in.off + v.bytes > map_.size()) throw Error("InvalidOffsets", in.name);
            v.data = map_.data() + data_start + in.off;
            tensors_[in.name] = v;
        }
    }
    // By the name in the file or by the canonical HF-style name (the reference's reader stores the
    // latter, gguf.zig:256) for the file's general.architecture.
    const TensorView *get(const std::string &name) const {
        auto it = tensors_.find(name);
        if (it != tensors_.end()) return &it->second;
        const auto a = strings.find("general.architecture");
        const std::string arch = a == strings.end() ? "" : a->second;
        for (const auto &kv : tensors_)
            if (canonicalName(kv.first, arch) == name) return &kv.second;
        return nullptr;
    }
    const std::map<std::string, TensorView> &tensors() const { return tensors_; }
    uint32_t version = 0;
    size_t alignment = 32;
    std::map<std::string, std::string> strings;   // string-valued metadata
    std::map<std::string, int64_t> integers;      // integer- and bool-valued metadata

  private:
    template <typename T>
    T take() {
        if (map_.size() - pos_ < sizeof(T)) throw Error("InvalidHeader", "truncated");
        T v;
        std::memcpy(&v, map_.data() + pos_, sizeof(T));
        pos_ += sizeof(T);
        return v;
    }
    std::string str() {
        const uint64_t n = take<uint64_t>();
        if (n > map_.size() - pos_) throw Error("InvalidHeader", "string runs past the file");
        std::string s(reinterpret_cast<const char *>(map_.data() + pos_), (size_t)n);
        pos_ += (size_t)n;
        return s;
    }
    void value(const std::string &key, uint32_t t, bool in_array = false) {
        int64_t iv = 0;
        bool is_int = true;
        switch (t) {
            case 0: iv = take<uint8_t>(); break;
            case 1: iv = take<int8_t>(); break;
            case 2: iv = take<uint16_t>(); break;
            case 3: iv = take<int16_t>(); break;
            case 4: iv = take<uint32_t>(); break;
            case 5: iv = take<int32_t>(); break;
            case 6: (void)take<float>(); is_int = false; break;
            case 7: iv = take<uint8_t>() != 0; break;
            case 8: { const std::string s = str(); if (!in_array) strings[key] = s; is_int = false; break; }
            case 9: {
                const uint32_t et = take<uint32_t>();
                const uint64_t n = take<uint64_t>();
                if (et == 9) throw Error("InvalidHeader", "nested arrays");
                for (uint64_t i = 0; i < n; i++) value(key, et, true);
                is_int = false;
                break;
            }
            case 10: iv = (int64_t)take<uint64_t>(); break;
            case 11: iv = take<int64_t>(); break;
            case 12: (void)take<double>(); is_int = false; break;
            default: throw Error("InvalidHeader", "kv type " + std::to_string(t));
        }
        if (is_int && !in_array) {
            integers[key] = iv;
            if (key == "general.alignment" && iv > 0) alignment = (size_t)iv;
        }
    }
    Mapping map_;
    size_t pos_ = 0;
    std::map<std::string, TensorView> tensors_;
};

}  // namespace tpbfmt

#endif  // TPB200_FORMATS_HPP
