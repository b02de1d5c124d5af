// CUDA-backed stand-ins for the handful of metal-cpp types that Miori's operator API names
// (reference src/ops.h, src/metal.h, src/weights.h).  Callers keep writing
//   MTL::Buffer* b = m.new_buffer(n);  memcpy(b->contents(), ...);  b->length();
//   auto* e = cb->computeCommandEncoder();  ...;  e->endEncoding();
// and get CUDA managed memory and a CUDA stream underneath, through the C ABI in
// include/miori_b200.h.
#pragma once
#include <cstddef>

extern "C" {
struct miori_device;
struct miori_buffer;
}

namespace MTL {

class Device;  // opaque; the reference only passes it to Weights::load

// MTL::Buffer: host-visible when created shared (the reference's default), device-only
// otherwise (contents() is then nullptr, as for MTLResourceStorageModePrivate).
class Buffer {
public:
    void* contents() const;
    std::size_t length() const;
    void release();  // frees the storage and this object
    // device address used by the operator wrappers
    void* gpu() const;

    explicit Buffer(miori_buffer* h) : h_(h) {}

private:
    ~Buffer() = default;
    miori_buffer* h_;
};

// One encoder per command buffer; dispatches run in program order on the device's stream.
class ComputeCommandEncoder {
public:
    explicit ComputeCommandEncoder(void* stream) : stream_(stream) {}
    void endEncoding() { ended_ = true; }
    void* stream() const { return stream_; }
    bool ended() const { return ended_; }

private:
    void* stream_;
    bool ended_ = false;
};

class CommandBuffer {
public:
    explicit CommandBuffer(miori_device* dev, void* stream) : dev_(dev), enc_(stream) {}
    ComputeCommandEncoder* computeCommandEncoder() { return &enc_; }
    miori_device* device() const { return dev_; }

private:
    miori_device* dev_;
    ComputeCommandEncoder enc_;
};

}  // namespace MTL
