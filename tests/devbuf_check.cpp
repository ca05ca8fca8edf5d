// Host-only check of the device-buffer invariant (p == nullptr <=> bytes == 0) with an allocator that fails on demand.
// Compiled and run by tests/test_devbuf.py; no CUDA involved.
#include <cstdio>
#include <cstdlib>
#include <string>

static bool g_fail_next = false;
static int g_live = 0;
static int fake_malloc(void** pp, size_t n) {
    if (g_fail_next) { *pp = nullptr; return 2; }
    *pp = std::malloc(n);
    ++g_live;
    return 0;
}
static void fake_free(void* p) { std::free(p); --g_live; }
#define THRML_DEV_MALLOC(pp, n) fake_malloc((pp), (n))
#define THRML_DEV_FREE(p) fake_free((p))
#define THRML_DEV_OK 0
#define THRML_DEV_IS_OOM(e) ((e) == 2)
#define THRML_DEV_ERRSTR(e) "out of memory (fake)"
#include "devbuf.h"

namespace thrml {
int32_t fail(int32_t code, const std::string&) { return code; }
}  // namespace thrml

#define CHECK(c) do { if (!(c)) { std::printf("FAILED: %s (line %d)\n", #c, __LINE__); return 1; } } while (0)

int main() {
    DevBuf b;
    CHECK(b.p == nullptr && b.bytes == 0 && !b.holds(1));
    CHECK(b.alloc(100) == THRML_OK && b.p && b.bytes == 100 && b.holds(100) && !b.holds(101));
    g_fail_next = true;
    CHECK(b.alloc(1000) == THRML_ERR_OOM);
    CHECK(b.p == nullptr && b.bytes == 0);  // a failed allocation leaves the buffer empty ...
    CHECK(!b.holds(1) && !b.holds(1000));   // ... so every growth guard allocates again
    CHECK(b.reserve(1000) == THRML_ERR_OOM && b.p == nullptr && b.bytes == 0);
    g_fail_next = false;
    CHECK(b.reserve(1000) == THRML_OK && b.holds(1000));
    void* before = b.p;
    CHECK(b.reserve(10) == THRML_OK && b.p == before);  // large enough: untouched
    CHECK(b.alloc(0) == THRML_OK && b.p == nullptr && b.bytes == 0);
    DevBuf c;
    CHECK(c.alloc(8) == THRML_OK);
    DevBuf d(std::move(c));
    CHECK(c.p == nullptr && c.bytes == 0 && d.holds(8));
    d.release();
    CHECK(g_live == 0);
    std::printf("ok\n");
    return 0;
}
