#include "gguf.hpp"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cmath>
#include <cstring>

namespace tuckmill {

namespace {

[[noreturn]] void invalid(const std::string &what) {
    throw TuckmillError(ErrorCode::InvalidArtifact, "GGUF: " + what,
                        "Re-import the artifact; its header could not be parsed.");
}

struct Cursor {
    const unsigned char *p;
    uint64_t size, pos = 0;
    template <class T>
    T take() {
        if (pos + sizeof(T) > size) invalid("truncated header");
        T v;
        memcpy(&v, p + pos, sizeof(T));
        pos += sizeof(T);
        return v;
    }
    std::string str() {
        const uint64_t n = take<uint64_t>();
        if (n > size - pos) invalid("string runs past the end of the file");
        std::string s((const char *)p + pos, (size_t)n);
        pos += n;
        return s;
    }
};

GgufValue read_value(Cursor &c, uint32_t ty, int depth = 0) {
    GgufValue v;
    switch (ty) {
        case 0: v.kind = GgufValue::UInt; v.u = c.take<uint8_t>(); break;
        case 1: v.kind = GgufValue::Int; v.i = c.take<int8_t>(); break;
        case 2: v.kind = GgufValue::UInt; v.u = c.take<uint16_t>(); break;
        case 3: v.kind = GgufValue::Int; v.i = c.take<int16_t>(); break;
        case 4: v.kind = GgufValue::UInt; v.u = c.take<uint32_t>(); break;
        case 5: v.kind = GgufValue::Int; v.i = c.take<int32_t>(); break;
        case 6: v.kind = GgufValue::Float; v.f = c.take<float>(); break;
        case 7: v.kind = GgufValue::Bool; v.u = c.take<uint8_t>(); break;
        case 8: v.kind = GgufValue::String; v.s = c.str(); break;
        case 9: {
            if (depth > 2) invalid("metadata arrays nested too deeply");
            const uint32_t et = c.take<uint32_t>();
            const uint64_t n = c.take<uint64_t>();
            v.kind = GgufValue::Array;
            v.array_len = n;
            for (uint64_t i = 0; i < n; ++i) read_value(c, et, depth + 1);  // skipped, bounds-checked
            break;
        }
        case 10: v.kind = GgufValue::UInt; v.u = c.take<uint64_t>(); break;
        case 11: v.kind = GgufValue::Int; v.i = c.take<int64_t>(); break;
        case 12: v.kind = GgufValue::Float; v.f = c.take<double>(); break;
        default: invalid("unknown metadata value type " + std::to_string(ty));
    }
    return v;
}

}  // namespace

bool ggml_block(uint32_t type_id, uint64_t *block_elems, uint64_t *block_bytes) {
    switch (type_id) {
        case 0: *block_elems = 1; *block_bytes = 4; return true;
        case 1: *block_elems = 1; *block_bytes = 2; return true;
        case 8: *block_elems = 32; *block_bytes = 34; return true;
        default: return false;
    }
}

GgufInspection GgufInspection::open(const std::string &path) {
    GgufInspection g;
    g.fd_ = ::open(path.c_str(), O_RDONLY);
    if (g.fd_ < 0) throw TuckmillError(ErrorCode::InvalidArtifact, "cannot open artifact " + path);
    struct stat st;
    if (fstat(g.fd_, &st) != 0 || st.st_size < 24) invalid("file is too small");
    g.file_size = (uint64_t)st.st_size;
    void *m = mmap(nullptr, g.file_size, PROT_READ, MAP_PRIVATE, g.fd_, 0);
    if (m == MAP_FAILED) throw TuckmillError(ErrorCode::Internal, "cannot map artifact " + path);
    g.data = (const unsigned char *)m;
    Cursor c{g.data, g.file_size};
    if (c.take<uint32_t>() != 0x46554747u) invalid("bad magic");
    g.version = c.take<uint32_t>();
    if (g.version != 2 && g.version != 3) invalid("unsupported version " + std::to_string(g.version));
    const uint64_t n_tensors = c.take<uint64_t>(), n_kv = c.take<uint64_t>();
    if (n_tensors > (1u << 20) || n_kv > (1u << 20)) invalid("implausible tensor or metadata count");
    for (uint64_t i = 0; i < n_kv; ++i) {
        std::string key = c.str();
        const uint32_t ty = c.take<uint32_t>();
        g.metadata[key] = read_value(c, ty);
    }
    for (uint64_t i = 0; i < n_tensors; ++i) {
        GgufTensor t;
        t.name = c.str();
        const uint32_t nd = c.take<uint32_t>();
        if (nd == 0 || nd > 4) invalid("tensor " + t.name + " has " + std::to_string(nd) + " dims");
        uint64_t elems = 1;
        for (uint32_t d = 0; d < nd; ++d) {
            t.dims.push_back(c.take<uint64_t>());
            if (t.dims.back() == 0 || elems > UINT64_MAX / t.dims.back()) invalid("tensor " + t.name + " overflows");
            elems *= t.dims.back();
        }
        t.type_id = c.take<uint32_t>();
        t.offset = c.take<uint64_t>();
        uint64_t be = 0, bb = 0;
        if (ggml_block(t.type_id, &be, &bb)) {
            if (t.dims[0] % be != 0) invalid("tensor " + t.name + " rows are not block aligned");
            t.byte_size = elems / be * bb;
        }
        g.tensors.push_back(std::move(t));
    }
    uint64_t align = 32;
    g.get_u64("general.alignment", &align);
    if (align == 0 || (align & (align - 1)) != 0) invalid("alignment is not a power of two");
    const uint64_t start = (c.pos + align - 1) / align * align;
    for (GgufTensor &t : g.tensors) {
        t.offset += start;
        if (t.byte_size && (t.offset > g.file_size || t.byte_size > g.file_size - t.offset))
            invalid("tensor " + t.name + " lies outside the file");
    }
    return g;
}

GgufInspection::~GgufInspection() {
    if (data) munmap((void *)data, file_size);
    if (fd_ >= 0) close(fd_);
}

GgufInspection::GgufInspection(GgufInspection &&o) noexcept
    : tensors(std::move(o.tensors)), metadata(std::move(o.metadata)), version(o.version),
      file_size(o.file_size), data(o.data), fd_(o.fd_) {
    o.data = nullptr;
    o.fd_ = -1;
}

const GgufValue *GgufInspection::get(const std::string &key) const {
    auto it = metadata.find(key);
    return it == metadata.end() ? nullptr : &it->second;
}

bool GgufInspection::get_u64(const std::string &key, uint64_t *out) const {
    const GgufValue *v = get(key);
    if (!v) return false;
    if (v->kind == GgufValue::UInt) { *out = v->u; return true; }
    if (v->kind == GgufValue::Int && v->i >= 0) { *out = (uint64_t)v->i; return true; }
    return false;
}

bool GgufInspection::get_f32(const std::string &key, float *out) const {
    const GgufValue *v = get(key);
    if (!v || v->kind != GgufValue::Float) return false;
    *out = (float)v->f;
    return true;
}

std::string GgufInspection::arch_id() const {
    const GgufValue *v = get("general.architecture");
    return v && v->kind == GgufValue::String ? v->s : "";
}

long GgufInspection::find(const std::string &name) const {
    for (size_t i = 0; i < tensors.size(); ++i)
        if (tensors[i].name == name) return (long)i;
    return -1;
}

const GgufTensor &GgufWeights::meta(size_t index) const {
    if (index >= insp_.tensors.size())
        throw TuckmillError(ErrorCode::Internal,
                            "tensor index " + std::to_string(index) + " is outside the inspected range");
    return insp_.tensors[index];
}

uint32_t GgufWeights::tensor_type_id(size_t index) const { return meta(index).type_id; }

std::pair<uint64_t, uint64_t> GgufWeights::tensor_dims(size_t index) const {
    const GgufTensor &t = meta(index);
    uint64_t out = 1;
    for (size_t d = 1; d < t.dims.size(); ++d) out *= t.dims[d];
    return {t.dims[0], t.dims.size() > 1 ? out : 1};
}

uint64_t GgufWeights::tensor_bytes(size_t index) const { return meta(index).byte_size; }

void GgufWeights::read_tensor_into(size_t index, uint64_t offset, void *dst, size_t len) const {
    const GgufTensor &t = meta(index);
    if (offset > t.byte_size || len > t.byte_size - offset)
        throw TuckmillError(ErrorCode::Internal, "tensor " + std::to_string(index) + " read past its " +
                                                     std::to_string(t.byte_size) + " bytes");
    memcpy(dst, insp_.data + t.offset + offset, len);
}

// A whole small vector dequantised to f32 (crates/tuckcore/src/tensor.rs:52-104).
std::vector<float> GgufWeights::read_vector(size_t index) const {
    const GgufTensor &t = meta(index);
    const unsigned char *p = insp_.data + t.offset;
    std::vector<float> out;
    if (t.type_id == 0) {
        out.resize(t.byte_size / 4);
        memcpy(out.data(), p, t.byte_size);
    } else if (t.type_id == 1) {
        out.resize(t.byte_size / 2);
        for (size_t i = 0; i < out.size(); ++i) {
            const uint16_t b = (uint16_t)(p[2 * i] | (p[2 * i + 1] << 8));
            const uint32_t sign = b >> 15, ex = (b >> 10) & 0x1f, mant = b & 0x3ff;
            float v = ex == 0 ? (float)mant * std::ldexp(1.0f, -24)
                      : ex == 31 ? (mant ? NAN : INFINITY)
                                 : (1.0f + (float)mant / 1024.0f) * std::ldexp(1.0f, (int)ex - 15);
            out[i] = sign ? -v : v;
        }
    } else {
        throw TuckmillError(ErrorCode::UnsupportedQuantization,
                            "vector tensor " + t.name + " has type " + std::to_string(t.type_id) +
                                "; vectors must be F32 or F16");
    }
    return out;
}

}  // namespace tuckmill
