/* A stand-in for libmiori_b200.so's C ABI that runs without a GPU, for host tests of the C++
 * operator shim: buffers are host memory, launches do nothing, and any entry can be told to fail
 * (fake_fail) or the device-error record to be non-empty (fake_device_errors).  Entries take
 * unspecified arguments on purpose: only the names and return codes matter to the callers. */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

enum { F_OPEN, F_BEGIN, F_SUBMIT, F_ALLOC, F_LAUNCH, F_COUNT };
static int g_fail[F_COUNT];
static int g_device_errors;
static int g_polls, g_launches, g_open;
static char g_msg[128] = "";

void fake_fail(int which, int rc) { g_fail[which] = rc; }
void fake_device_errors(int n) { g_device_errors = n; }
int fake_polls(void) { return g_polls; }
int fake_launches(void) { return g_launches; }
int fake_open_devices(void) { return g_open; }

static int result(int which, const char* who) {
    if (g_fail[which]) snprintf(g_msg, sizeof g_msg, "%s: scripted failure %d", who, g_fail[which]);
    return g_fail[which];
}

const char* miori_last_error(void) { return g_msg; }
const char* miori_version(void) { return "fake"; }

struct dev { int ordinal; };
struct buf { void* p; size_t n; };

int miori_device_open(int ordinal, struct dev** out) {
    int rc = result(F_OPEN, "miori_device_open");
    if (rc) return rc;
    *out = malloc(sizeof **out);
    (*out)->ordinal = ordinal;
    ++g_open;
    return 0;
}
int miori_device_close(struct dev* d) { free(d); --g_open; return 0; }
void* miori_device_stream(struct dev* d) { return d; }
int miori_device_ordinal(struct dev* d) { return d->ordinal; }
int miori_buffer_alloc(struct dev* d, size_t bytes, int shared, struct buf** out) {
    (void)d; (void)shared;
    int rc = result(F_ALLOC, "miori_buffer_alloc");
    if (rc) return rc;
    *out = malloc(sizeof **out);
    (*out)->p = calloc(1, bytes ? bytes : 1);
    (*out)->n = bytes;
    return 0;
}
int miori_buffer_free(struct buf* b) { if (b) { free(b->p); free(b); } return 0; }
void* miori_buffer_contents(struct buf* b) { return b->p; }
void* miori_buffer_device_ptr(struct buf* b) { return b->p; }
size_t miori_buffer_length(struct buf* b) { return b->n; }
int miori_begin(struct dev* d) { (void)d; return result(F_BEGIN, "miori_begin"); }
int miori_submit(struct dev* d, int wait) { (void)d; (void)wait; return result(F_SUBMIT, "miori_submit"); }
int miori_device_error_poll(void) {
    ++g_polls;
    if (g_device_errors) snprintf(g_msg, sizeof g_msg, "kernel reported %d internal error(s)", g_device_errors);
    int n = g_device_errors;
    g_device_errors = 0;
    return n;
}

#define LAUNCH(name) int name() { ++g_launches; return result(F_LAUNCH, #name); }
LAUNCH(miori_gemv4)
LAUNCH(miori_gemv8)
LAUNCH(miori_dequant4_cache)
LAUNCH(miori_dequant4_rowmajor)
LAUNCH(miori_dequant8_rowmajor)
LAUNCH(miori_gemm_bf16_cache)
LAUNCH(miori_gemm_bf16_strided)
LAUNCH(miori_rmsnorm)
LAUNCH(miori_silu_mul)
LAUNCH(miori_embed8)
LAUNCH(miori_post_norm_add)
LAUNCH(miori_gemv4_silu)
LAUNCH(miori_gemv4_rmsnorm)
LAUNCH(miori_gemv4_rmsnorm_silu)
