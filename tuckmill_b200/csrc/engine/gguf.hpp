// GGUF v2/v3 inspection and tensor reads (the part of crates/manifest/src/gguf.rs
// the executor needs: metadata lookups, tensor name/dims/type/offset) and the
// engine's weight access trait (crates/tuckcore/src/engine/mod.rs:22-121).
#pragma once
#include <cstdint>
#include <map>
#include <string>
#include <vector>

#include "error.hpp"

namespace tuckmill {

struct GgufValue {
    enum Kind { None, UInt, Int, Float, Bool, String, Array } kind = None;
    uint64_t u = 0;
    int64_t i = 0;
    double f = 0.0;
    std::string s;
    uint64_t array_len = 0;
};

struct GgufTensor {
    std::string name;
    std::vector<uint64_t> dims;  // innermost first: [in_dim, out_dim]
    uint32_t type_id = 0;
    uint64_t offset = 0;  // absolute file offset
    uint64_t byte_size = 0;
};

// GGML type table rows this path executes (crates/manifest/src/ggml.rs:40-77):
// F32 (0): 1 elem / 4 B, F16 (1): 1 / 2 B, Q8_0 (8): 32 elems / 34 B.
bool ggml_block(uint32_t type_id, uint64_t *block_elems, uint64_t *block_bytes);

class GgufInspection {
public:
    static GgufInspection open(const std::string &path);
    ~GgufInspection();
    GgufInspection(GgufInspection &&o) noexcept;
    GgufInspection(const GgufInspection &) = delete;

    const GgufValue *get(const std::string &key) const;
    bool get_u64(const std::string &key, uint64_t *out) const;
    bool get_f32(const std::string &key, float *out) const;
    std::string arch_id() const;  // general.architecture, "" when absent
    long find(const std::string &name) const;  // tensor index or -1

    std::vector<GgufTensor> tensors;
    std::map<std::string, GgufValue> metadata;
    uint32_t version = 0;
    uint64_t file_size = 0;
    const unsigned char *data = nullptr;  // read-only mapping of the whole file

private:
    GgufInspection() = default;
    int fd_ = -1;
};

// Read access to an artifact's tensors by inspection index.
class WeightSource {
public:
    virtual ~WeightSource() = default;
    virtual uint32_t tensor_type_id(size_t index) const = 0;
    virtual std::pair<uint64_t, uint64_t> tensor_dims(size_t index) const = 0;  // (in_dim, out_dim)
    virtual uint64_t tensor_bytes(size_t index) const = 0;
    virtual void read_tensor_into(size_t index, uint64_t offset, void *dst, size_t len) const = 0;
    virtual std::vector<float> read_vector(size_t index) const = 0;
};

class GgufWeights : public WeightSource {
public:
    explicit GgufWeights(const GgufInspection &insp) : insp_(insp) {}
    uint32_t tensor_type_id(size_t index) const override;
    std::pair<uint64_t, uint64_t> tensor_dims(size_t index) const override;
    uint64_t tensor_bytes(size_t index) const override;
    void read_tensor_into(size_t index, uint64_t offset, void *dst, size_t len) const override;
    std::vector<float> read_vector(size_t index) const override;

private:
    const GgufTensor &meta(size_t index) const;
    const GgufInspection &insp_;
};

}  // namespace tuckmill
