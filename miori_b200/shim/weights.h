// Operand descriptors with the reference's interface (reference src/weights.h:10-41):
// every tensor is a byte range [begin, end) of one device-visible buffer.  The safetensors
// loader is not part of the quantized-matmul path; tensors are registered from memory.
#pragma once
#include <Metal/Metal.hpp>

#include <cstdint>
#include <map>
#include <string>
#include <vector>

namespace miori {

struct Metal;

struct Tensor {
    std::string name;
    std::string dtype;
    std::vector<int64_t> shape;
    uint64_t begin = 0;
    uint64_t end = 0;
    const uint8_t* ptr = nullptr;

    int64_t rows() const { return shape.empty() ? 0 : shape[0]; }
    int64_t cols() const { return shape.size() < 2 ? 0 : shape[1]; }
    size_t bytes() const { return (size_t)(end - begin); }
};

class Weights {
public:
    ~Weights();
    // Reserve one shared buffer of `bytes` (offsets handed out by add() are 256-byte aligned,
    // the alignment the reference planned for, docs/MILESTONES.md:52).
    bool reserve(Metal& m, size_t bytes, std::string& err);
    // Copy `bytes` of host data into the buffer and register it under `name`.
    const Tensor& add(const std::string& name, const std::string& dtype,
                      const std::vector<int64_t>& shape, const void* data, size_t bytes);
    // Throws std::runtime_error for an unknown name (src/weights.cpp:70).
    const Tensor& get(const std::string& name) const;
    const Tensor* find(const std::string& name) const;
    bool has(const std::string& name) const { return find(name) != nullptr; }
    MTL::Buffer* buffer() const { return buf_; }
    const uint8_t* data() const { return data_; }
    size_t data_size() const { return used_; }
    size_t tensor_count() const { return tensors_.size(); }
    const std::map<std::string, Tensor>& tensors() const { return tensors_; }

private:
    MTL::Buffer* buf_ = nullptr;
    uint8_t* data_ = nullptr;
    size_t cap_ = 0, used_ = 0;
    std::map<std::string, Tensor> tensors_;
};

}  // namespace miori
