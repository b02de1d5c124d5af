// Stand-in for Apple's <Metal/Metal.hpp> so that the reference's src/weights.h and
// src/cpu_ref.h compile unmodified on Linux.  Only the two class names that
// weights.h mentions by pointer are needed.
#pragma once
namespace MTL {
class Buffer;
class Device;
}  // namespace MTL
