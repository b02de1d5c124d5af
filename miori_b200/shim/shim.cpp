// Bodies of the CUDA-backed runtime, weights registry and hot-path operators declared in
// metal.h / weights.h / ops.h, all on top of the C ABI (include/miori_b200.h).
#include "fused_ops.h"
#include "ops.h"

#include "miori_b200.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <stdexcept>

// ---------------------------------------------------------------- MTL stand-ins
void* MTL::Buffer::contents() const { return miori_buffer_contents(h_); }
std::size_t MTL::Buffer::length() const { return miori_buffer_length(h_); }
void* MTL::Buffer::gpu() const { return miori_buffer_device_ptr(h_); }
void MTL::Buffer::release() {
    miori_buffer_free(h_);
    delete this;
}

namespace miori {

namespace {
[[noreturn]] void raise(const char* what) {
    throw std::runtime_error(std::string(what) + ": " + miori_last_error());
}
inline void check(int rc, const char* what) {
    if (rc != MIORI_OK) raise(what);
}
inline const uint8_t* at(MTL::Buffer* b, uint64_t off) {
    return static_cast<const uint8_t*>(b->gpu()) + off;
}
inline uint8_t* at_mut(MTL::Buffer* b, uint64_t off) { return static_cast<uint8_t*>(b->gpu()) + off; }
}  // namespace

// ---------------------------------------------------------------- Metal (device runtime)
bool Metal::init(const std::string&, std::string& err) {
    int ordinal = 0;
    if (const char* env = std::getenv("MIORI_DEVICE")) ordinal = std::atoi(env);
    if (miori_device_open(ordinal, &dev) != MIORI_OK) {
        err = miori_last_error();
        dev = nullptr;
        return false;
    }
    return true;
}

Metal::~Metal() {
    if (dev) miori_device_close(dev);
}

MTL::Buffer* Metal::new_buffer(size_t bytes, bool shared) {
    miori_buffer* h = nullptr;
    if (miori_buffer_alloc(dev, bytes, shared ? 1 : 0, &h) != MIORI_OK)
        throw std::runtime_error(std::string("buffer allocation failed: ") + miori_last_error());
    return new MTL::Buffer(h);
}

MTL::CommandBuffer* Metal::begin() {
    if (!dev || miori_begin(dev) != MIORI_OK)
        throw std::runtime_error(std::string("command buffer: ") + miori_last_error());
    return new MTL::CommandBuffer(dev, miori_device_stream(dev));
}

void Metal::submit(MTL::CommandBuffer* cb, bool wait) {
    const int rc = miori_submit(dev, wait ? 1 : 0);
    delete cb;
    if (rc != MIORI_OK) raise("submit");
    if (wait && miori_device_error_poll() != 0) raise("kernel error");
}

void Metal::print_info() const {
    std::printf("device: CUDA ordinal %d (%s)\n", miori_device_ordinal(dev), miori_version());
}

// ---------------------------------------------------------------- Weights
Weights::~Weights() {
    if (buf_) buf_->release();
}

bool Weights::reserve(Metal& m, size_t bytes, std::string& err) {
    try {
        buf_ = m.new_buffer(bytes, true);
    } catch (const std::exception& e) {
        err = e.what();
        return false;
    }
    data_ = static_cast<uint8_t*>(buf_->contents());
    cap_ = bytes;
    used_ = 0;
    return true;
}

const Tensor& Weights::add(const std::string& name, const std::string& dtype,
                           const std::vector<int64_t>& shape, const void* data, size_t bytes) {
    const size_t off = (used_ + 255) & ~size_t(255);
    if (!buf_ || off + bytes > cap_) throw std::runtime_error("weights buffer too small for " + name);
    std::memcpy(data_ + off, data, bytes);
    Tensor t;
    t.name = name;
    t.dtype = dtype;
    t.shape = shape;
    t.begin = off;
    t.end = off + bytes;
    t.ptr = data_ + off;
    used_ = off + bytes;
    return tensors_[name] = t;
}

const Tensor* Weights::find(const std::string& name) const {
    auto it = tensors_.find(name);
    return it == tensors_.end() ? nullptr : &it->second;
}

const Tensor& Weights::get(const std::string& name) const {
    if (const Tensor* t = find(name)) return *t;
    throw std::runtime_error("missing tensor: " + name);
}

// ---------------------------------------------------------------- operators
void gemv4_b(Metal&, MTL::ComputeCommandEncoder* e, const Weights& w, const Tensor& q,
             const Tensor& s, const Tensor& b, MTL::Buffer* x, MTL::Buffer* y, uint32_t N, uint32_t K,
             uint32_t B) {
    check(miori_gemv4(at(w.buffer(), q.begin), at(w.buffer(), s.begin), at(w.buffer(), b.begin),
                      x->gpu(), y->gpu(), N, K, B, kGroup, MIORI_OUT_F32, e->stream()),
          "gemv4");
}

void gemv8_b_off(Metal&, MTL::ComputeCommandEncoder* e, const Weights& w, const Tensor& q,
                 const Tensor& s, const Tensor& b, MTL::Buffer* x, MTL::Buffer* y, uint32_t N,
                 uint32_t K, uint32_t B, uint32_t xoff, uint32_t yoff) {
    check(miori_gemv8(at(w.buffer(), q.begin), at(w.buffer(), s.begin), at(w.buffer(), b.begin),
                      at(x, xoff), at_mut(y, yoff), N, K, B, kGroup, MIORI_OUT_F32, e->stream()),
          "gemv8");
}

void gemv4(Metal& m, MTL::ComputeCommandEncoder* e, const Weights& w, const Tensor& q,
           const Tensor& s, const Tensor& b, MTL::Buffer* x, MTL::Buffer* y, uint32_t N, uint32_t K) {
    gemv4_b(m, e, w, q, s, b, x, y, N, K, 1);
}

// The reference's x4 / x2 variants differ only in how rows map to SIMD groups; one kernel
// family serves all three entry points here.
void gemv4x4(Metal& m, MTL::ComputeCommandEncoder* e, const Weights& w, const Tensor& q,
             const Tensor& s, const Tensor& b, MTL::Buffer* x, MTL::Buffer* y, uint32_t N, uint32_t K) {
    gemv4_b(m, e, w, q, s, b, x, y, N, K, 1);
}
void gemv4x2(Metal& m, MTL::ComputeCommandEncoder* e, const Weights& w, const Tensor& q,
             const Tensor& s, const Tensor& b, MTL::Buffer* x, MTL::Buffer* y, uint32_t N, uint32_t K) {
    gemv4_b(m, e, w, q, s, b, x, y, N, K, 1);
}

void gemv4_raw(Metal&, MTL::ComputeCommandEncoder* e, MTL::Buffer* q, MTL::Buffer* s, MTL::Buffer* b,
               MTL::Buffer* x, MTL::Buffer* y, uint32_t N, uint32_t K) {
    check(miori_gemv4(q->gpu(), s->gpu(), b->gpu(), x->gpu(), y->gpu(), N, K, 1, kGroup, MIORI_OUT_F32,
                      e->stream()),
          "gemv4_raw");
}

void gemv8_b(Metal& m, MTL::ComputeCommandEncoder* e, const Weights& w, const Tensor& q,
             const Tensor& s, const Tensor& b, MTL::Buffer* x, MTL::Buffer* y, uint32_t N, uint32_t K,
             uint32_t B) {
    gemv8_b_off(m, e, w, q, s, b, x, y, N, K, B, 0, 0);
}

void gemv8(Metal& m, MTL::ComputeCommandEncoder* e, const Weights& w, const Tensor& q,
           const Tensor& s, const Tensor& b, MTL::Buffer* x, MTL::Buffer* y, uint32_t N, uint32_t K) {
    gemv8_b_off(m, e, w, q, s, b, x, y, N, K, 1, 0, 0);
}

void gemv8_off(Metal&, MTL::ComputeCommandEncoder* e, MTL::Buffer* wbuf, uint32_t qoff, uint32_t soff,
               uint32_t boff, MTL::Buffer* x, MTL::Buffer* y, uint32_t N, uint32_t K, uint32_t xoff,
               uint32_t yoff) {
    check(miori_gemv8(at(wbuf, qoff), at(wbuf, soff), at(wbuf, boff), at(x, xoff), at_mut(y, yoff), N, K,
                      1, kGroup, MIORI_OUT_F32, e->stream()),
          "gemv8_off");
}

void dequant4(Metal&, MTL::ComputeCommandEncoder* e, const Weights& w, const Tensor& q,
              const Tensor& s, const Tensor& b, MTL::Buffer* out, uint32_t N, uint32_t K,
              uint32_t boff) {
    check(miori_dequant4_rowmajor(at(w.buffer(), q.begin), at(w.buffer(), s.begin),
                                  at(w.buffer(), b.begin), at_mut(out, boff), N, K, kGroup,
                                  e->stream()),
          "dequant4");
}

void dequant8(Metal&, MTL::ComputeCommandEncoder* e, const Weights& w, const Tensor& q,
              const Tensor& s, const Tensor& b, MTL::Buffer* out, uint32_t N, uint32_t K) {
    check(miori_dequant8_rowmajor(at(w.buffer(), q.begin), at(w.buffer(), s.begin),
                                  at(w.buffer(), b.begin), out->gpu(), N, K, kGroup, e->stream()),
          "dequant8");
}

void dequant_tile(Metal&, MTL::ComputeCommandEncoder* e, const Weights& w, const Tensor& q,
                  const Tensor& s, const Tensor& b, MTL::Buffer* out, uint32_t N, uint32_t K,
                  uint32_t boff) {
    check(miori_dequant4_cache(at(w.buffer(), q.begin), at(w.buffer(), s.begin),
                               at(w.buffer(), b.begin), at_mut(out, boff), N, K, kGroup, e->stream()),
          "dequant_tile");
}

void gemm_mpp_off(Metal&, MTL::ComputeCommandEncoder* e, MTL::Buffer* A, MTL::Buffer* B,
                  MTL::Buffer* C, uint32_t M, uint32_t N, uint32_t K, uint32_t aoff, uint32_t boff,
                  uint32_t coff) {
    check(miori_gemm_bf16_cache(at(A, aoff), at(B, boff), at_mut(C, coff), M, N, K, MIORI_OUT_F32,
                                e->stream()),
          "gemm_mpp");
}

void gemm_mpp(Metal& m, MTL::ComputeCommandEncoder* e, MTL::Buffer* A, MTL::Buffer* B,
              MTL::Buffer* C, uint32_t M, uint32_t N, uint32_t K, uint32_t boff) {
    gemm_mpp_off(m, e, A, B, C, M, N, K, 0, boff, 0);
}

void gemm_naive(Metal&, MTL::ComputeCommandEncoder* e, MTL::Buffer* A, MTL::Buffer* B,
                MTL::Buffer* C, uint32_t M, uint32_t N, uint32_t K, uint32_t lda, uint32_t ldb,
                uint32_t ldc, uint32_t aoff, uint32_t boff, uint32_t coff) {
    check(miori_gemm_bf16_strided(at(A, aoff), lda, at(B, boff), ldb, at_mut(C, coff), ldc, M, N, K,
                                  MIORI_OUT_F32, e->stream()),
          "gemm_naive");
}

void rmsnorm(Metal&, MTL::ComputeCommandEncoder* e, MTL::Buffer* x, const Weights& w, const Tensor& gamma,
             MTL::Buffer* y, uint32_t rows, uint32_t n, float eps) {
    check(miori_rmsnorm(at(x, 0), at(w.buffer(), gamma.begin), at_mut(y, 0), rows, n, eps, 0, e->stream()),
          "rmsnorm");
}

void silu_mul(Metal&, MTL::ComputeCommandEncoder* e, MTL::Buffer* gate, MTL::Buffer* up, MTL::Buffer* out,
              uint32_t n) {
    check(miori_silu_mul(at(gate, 0), at(up, 0), at_mut(out, 0), n, 0, e->stream()), "silu_mul");
}

void postnorm_add(Metal&, MTL::ComputeCommandEncoder* e, MTL::Buffer* x, MTL::Buffer* src, const Weights& w,
                  const Tensor& gamma, MTL::Buffer* out, uint32_t rows, uint32_t n, float eps) {
    check(miori_post_norm_add(at(x, 0), at(src, 0), at(w.buffer(), gamma.begin), at_mut(out, 0), rows, n, eps, 0,
                              e->stream()),
          "postnorm_add");
}

void gemv4_silu(Metal&, MTL::ComputeCommandEncoder* e, const Weights& w, const Tensor& q, const Tensor& s,
                const Tensor& b, MTL::Buffer* x, MTL::Buffer* y, uint32_t N, uint32_t K, uint32_t B) {
    check(miori_gemv4_silu(at(w.buffer(), q.begin), at(w.buffer(), s.begin), at(w.buffer(), b.begin), x->gpu(),
                           y->gpu(), N, K, B, kGroup, 0, e->stream()),
          "gemv4_silu");
}

void gemv4_rmsnorm(Metal&, MTL::ComputeCommandEncoder* e, const Weights& w, const Tensor& q, const Tensor& s,
                   const Tensor& b, MTL::Buffer* x, const Tensor& gamma, float eps, MTL::Buffer* y, uint32_t N,
                   uint32_t K, uint32_t B) {
    check(miori_gemv4_rmsnorm(at(w.buffer(), q.begin), at(w.buffer(), s.begin), at(w.buffer(), b.begin), x->gpu(),
                              at(w.buffer(), gamma.begin), eps, y->gpu(), N, K, B, kGroup, MIORI_OUT_F32,
                              e->stream()),
          "gemv4_rmsnorm");
}

void gemv4_rmsnorm_silu(Metal&, MTL::ComputeCommandEncoder* e, const Weights& w, const Tensor& q, const Tensor& s,
                        const Tensor& b, MTL::Buffer* x, const Tensor& gamma, float eps, MTL::Buffer* y,
                        uint32_t N, uint32_t K, uint32_t B) {
    check(miori_gemv4_rmsnorm_silu(at(w.buffer(), q.begin), at(w.buffer(), s.begin), at(w.buffer(), b.begin),
                                   x->gpu(), at(w.buffer(), gamma.begin), eps, y->gpu(), N, K, B, kGroup, 0,
                                   e->stream()),
          "gemv4_rmsnorm_silu");
}

void embed8(Metal&, MTL::ComputeCommandEncoder* e, const Weights& w, const Tensor& q, const Tensor& s,
            const Tensor& b, MTL::Buffer* tokens, MTL::Buffer* out, uint32_t T, uint32_t K) {
    check(miori_embed8(at(w.buffer(), q.begin), at(w.buffer(), s.begin), at(w.buffer(), b.begin),
                       at(tokens, 0), at_mut(out, 0), T, (uint32_t)q.rows(), K, kGroup, 0, e->stream()),
          "embed8");
}

void gemm_mpp32(Metal& m, MTL::ComputeCommandEncoder* e, MTL::Buffer* A, MTL::Buffer* B,
                MTL::Buffer* C, uint32_t M, uint32_t N, uint32_t K, uint32_t boff) {
    gemm_mpp_off(m, e, A, B, C, M, N, K, 0, boff, 0);
}

}  // namespace miori
