// Host test of the operator shim's error behaviour against the fake C ABI: what the reference
// reports by return value stays a return value (Metal::init), what it throws stays a
// std::runtime_error (new_buffer, begin, submit), a failed launch throws from the operator, and
// an error that a kernel recorded on the device surfaces at the waiting submit.
#include "ops.h"

#include <cstdio>
#include <cstring>
#include <functional>
#include <stdexcept>
#include <string>

extern "C" {
void fake_fail(int which, int rc);
void fake_device_errors(int n);
int fake_polls(void);
int fake_launches(void);
int fake_open_devices(void);
}
enum { F_OPEN, F_BEGIN, F_SUBMIT, F_ALLOC, F_LAUNCH };

static int failures = 0;
static void expect(bool ok, const char* what) {
    std::printf("%s: %s\n", what, ok ? "ok" : "FAILED");
    if (!ok) ++failures;
}
// true if fn throws a std::runtime_error whose text contains every needle
static bool throws(const std::function<void()>& fn, const char* n1, const char* n2 = "") {
    try {
        fn();
    } catch (const std::runtime_error& e) {
        const std::string s = e.what();
        return s.find(n1) != std::string::npos && s.find(n2) != std::string::npos;
    } catch (...) {
        return false;
    }
    return false;
}

int main() {
    using namespace miori;
    std::string err;
    {
        Metal m;
        fake_fail(F_OPEN, -3);
        expect(!m.init("ignored.metallib", err) && err.find("miori_device_open") != std::string::npos && !m.dev,
               "init reports a device that cannot be opened by return value");
        fake_fail(F_OPEN, 0);
        expect(throws([&] { m.begin(); }, "command buffer"), "begin without a device throws");
    }
    {
        Metal m;
        expect(m.init("", err), "init");
        fake_fail(F_ALLOC, -2);
        expect(throws([&] { m.new_buffer(64); }, "buffer allocation failed", "miori_buffer_alloc"),
               "new_buffer failure throws");
        fake_fail(F_ALLOC, 0);
        fake_fail(F_BEGIN, -1);
        expect(throws([&] { m.begin(); }, "command buffer", "miori_begin"), "begin failure throws");
        fake_fail(F_BEGIN, 0);

        MTL::Buffer* a = m.new_buffer(256);
        expect(a->length() == 256 && a->contents() != nullptr, "buffer length and contents");
        Weights w;
        expect(w.reserve(m, 4096, err), "weights reserve");
        const uint8_t zeros[256] = {0};
        const Tensor& tq = w.add("q", "U32", {8, 4}, zeros, 128);
        const Tensor& ts = w.add("s", "BF16", {8, 1}, zeros, 16);
        const Tensor& tb = w.add("b", "BF16", {8, 1}, zeros, 16);

        // a clean scope: one launch, one poll at the waiting submit, none without waiting
        auto* cb = m.begin();
        gemv4(m, cb->computeCommandEncoder(), w, tq, ts, tb, a, a, 8, 32);
        const int p0 = fake_polls();
        m.submit(cb, false);
        expect(fake_polls() == p0, "submit(wait=false) does not read the device error record");
        cb = m.begin();
        m.submit(cb, true);
        expect(fake_polls() == p0 + 1 && fake_launches() == 1, "submit(wait=true) polls once");

        // a launch the library refuses throws from the operator, naming it
        cb = m.begin();
        fake_fail(F_LAUNCH, -1);
        expect(throws([&] { gemv8(m, cb->computeCommandEncoder(), w, tq, ts, tb, a, a, 8, 32); }, "gemv8",
                      "miori_gemv8"),
               "refused launch throws from the operator");
        fake_fail(F_LAUNCH, 0);
        // the submit itself fails (e.g. an asynchronous launch failure seen by the synchronize)
        fake_fail(F_SUBMIT, -4);
        expect(throws([&] { m.submit(cb, true); }, "submit", "miori_submit"), "failed submit throws");
        fake_fail(F_SUBMIT, 0);
        // a kernel recorded an error (a bounded wait that expired): the waiting submit throws
        cb = m.begin();
        fake_device_errors(2);
        expect(throws([&] { m.submit(cb, true); }, "kernel error", "2 internal error"),
               "device error record turns into runtime_error at submit");
        cb = m.begin();
        bool clean = true;
        try {
            m.submit(cb, true);
        } catch (...) {
            clean = false;
        }
        expect(clean, "the record is cleared: the next submit succeeds");
        a->release();
    }
    expect(fake_open_devices() == 0, "every opened device was closed");
    std::printf(failures ? "shim_errors: %d failures\n" : "shim_errors: ok\n", failures);
    return failures ? 1 : 0;
}
