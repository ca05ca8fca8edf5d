// Owning handle of one device allocation, shared by the translation units of the library.
//
// Invariant (every growth guard in the library relies on it): p == nullptr  <=>  bytes == 0.  A failed allocation
// leaves the buffer empty, so a later `holds(need)` is false and the caller allocates again (or fails again) instead of
// handing a null pointer to a kernel.
//
// THRML_DEV_MALLOC / THRML_DEV_FREE name the allocator; the library leaves them at cudaMalloc / cudaFree, the host-only
// unit test of the invariant substitutes an allocator that fails on demand.
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>

#include "tables.h"

#ifndef THRML_DEV_MALLOC
#include <cuda_runtime.h>
#define THRML_DEV_MALLOC(pp, n) cudaMalloc((pp), (n))
#define THRML_DEV_FREE(p) cudaFree((p))
#define THRML_DEV_OK cudaSuccess
#define THRML_DEV_IS_OOM(e) ((e) == cudaErrorMemoryAllocation)
#define THRML_DEV_ERRSTR(e) cudaGetErrorString((e))
#endif

struct DevBuf {
    void* p = nullptr;
    size_t bytes = 0;
    DevBuf() = default;
    DevBuf(const DevBuf&) = delete;
    DevBuf& operator=(const DevBuf&) = delete;
    DevBuf(DevBuf&& o) noexcept : p(o.p), bytes(o.bytes) { o.p = nullptr; o.bytes = 0; }
    ~DevBuf() { release(); }
    void release() {
        if (p) THRML_DEV_FREE(p);
        p = nullptr;
        bytes = 0;
    }
    // Replaces the allocation with one of exactly n bytes (n == 0 leaves the buffer empty).
    int32_t alloc(size_t n) {
        release();
        if (n == 0) return THRML_OK;
        void* q = nullptr;
        auto e = THRML_DEV_MALLOC(&q, n);
        if (e != THRML_DEV_OK || !q)
            return thrml::fail(THRML_DEV_IS_OOM(e) ? THRML_ERR_OOM : THRML_ERR_CUDA, std::string("cudaMalloc: ") + THRML_DEV_ERRSTR(e));
        p = q;
        bytes = n;
        return THRML_OK;
    }
    // True when the buffer can serve `need` bytes as it stands.
    bool holds(size_t need) const { return p != nullptr && bytes >= need; }
    // Grows to at least `need` bytes (contents are not kept); no-op when already large enough.
    int32_t reserve(size_t need) { return holds(need) || need == 0 ? THRML_OK : alloc(need); }
    template <class T> T* as() const { return static_cast<T*>(p); }
};
