// Device runtime with the reference's interface (reference src/metal.h:10-22), backed by
// the C ABI of libmiori_b200.so.  `Metal` keeps its name so that engine code compiles
// unchanged; there is no shader library to load, so init()'s path argument is ignored.
#pragma once
#include <Metal/Metal.hpp>

#include <cstddef>
#include <string>

namespace miori {

struct Metal {
    miori_device* dev = nullptr;

    // Opens GPU 0 (or the ordinal in MIORI_DEVICE).  Returns false and fills err on failure,
    // like the reference (src/metal.cpp:10-24).
    bool init(const std::string& metallib_path, std::string& err);
    // Throws std::runtime_error on allocation failure (src/metal.cpp:42-48).
    MTL::Buffer* new_buffer(size_t bytes, bool shared = true);
    // Throws std::runtime_error if no command scope can be opened (src/metal.cpp:50-54).
    MTL::CommandBuffer* begin();
    // Closes the scope; wait=true blocks until the device has finished (src/metal.cpp:56-59)
    // and throws std::runtime_error if a launch failed asynchronously.
    void submit(MTL::CommandBuffer* cb, bool wait = true);
    void print_info() const;
    ~Metal();
};

}  // namespace miori
