// Bounds-checking build of the fused kernels (-DEMA_BOUNDS_CHECK; build.py --checked).
//
// Before every launch the host writes the address range of every buffer of the call (tensors from their shapes and
// strides, scratch from its byte count) into a small table in device memory.  In the checked build every plain
// global-memory access of the fused kernels goes through EMA_AT(): an address that lies inside none of the call's
// buffers is recorded (first violation only: 0x400 | site in the table's status word) and the access is redirected to
// a 64-byte sink inside the table, so that nothing outside the call's buffers is ever touched and nothing traps.
// The host reads and clears the word with ema_b200_bounds_status().  TMA accesses need no such check: the tensor map
// carries the extents and the copy engine clips to them.
//
// In the normal build EMA_AT(p, ptr, site) is `ptr` and the table pointer in the kernel parameters is null.
//
// The check catches an access outside ALL buffers of the call; a write that strays from one buffer of the call into
// another is what the guard-zone test (sentinel margins around every buffer) is for.
#pragma once

#include <stdint.h>

namespace ema {

constexpr int kBoundsMaxRanges = 24;
struct BoundsTable {
    unsigned status;   // 0, or 0x400 | site of the first rejected access
    int n;
    unsigned long long lo[kBoundsMaxRanges], hi[kBoundsMaxRanges];   // [lo, hi) byte addresses
    uint4 sink[4];     // where rejected accesses go
};

#ifdef EMA_BOUNDS_CHECK
template <typename T>
__device__ __forceinline__ T *bounds_at(BoundsTable *tb, T *ptr, unsigned site, unsigned bytes) {
    if (!tb) return ptr;   // a launch outside the checked entry points
    const unsigned long long a = reinterpret_cast<unsigned long long>(ptr);
    for (int i = 0; i < tb->n; ++i)
        if (a >= tb->lo[i] && a + bytes <= tb->hi[i]) return ptr;
    atomicCAS(&tb->status, 0u, 0x400u | (site & 0x3ffu));
    return reinterpret_cast<T *>(tb->sink);
}
// ptr checked for an access of sizeof(*ptr) bytes / of `bytes` bytes (vector accesses through a narrower pointer type)
#define EMA_AT(p, ptr, site) ::ema::bounds_at((p).bounds, (ptr), (site), static_cast<unsigned>(sizeof(*(ptr))))
#define EMA_ATN(p, ptr, site, bytes) ::ema::bounds_at((p).bounds, (ptr), (site), static_cast<unsigned>(bytes))
#else
#define EMA_AT(p, ptr, site) (ptr)
#define EMA_ATN(p, ptr, site, bytes) (ptr)
#endif

// Pointer parameters of the stage kernels.  Normal build: a plain restrict-qualified pointer.  Checking build: a pointer
// that carries the table and checks every dereference (p[i], *p) - derived pointers (p + n) keep the table; chk(p) gives
// the raw pointer after checking sizeof(*p) bytes, chk_bytes(p, n) after checking n bytes (vector accesses).
#ifdef EMA_BOUNDS_CHECK
template <typename T>
struct CheckedPtr {
    T *p;
    BoundsTable *tb;
    unsigned site;
    template <typename I>
    __device__ __forceinline__ CheckedPtr operator+(I off) const { return CheckedPtr{p + off, tb, site}; }
    template <typename I>
    __device__ __forceinline__ T &operator[](I i) const { return *bounds_at(tb, p + i, site, static_cast<unsigned>(sizeof(T))); }
    __device__ __forceinline__ T &operator*() const { return *bounds_at(tb, p, site, static_cast<unsigned>(sizeof(T))); }
};
template <typename T> using Ptr = CheckedPtr<T>;
template <typename T>
__device__ __forceinline__ T *chk(CheckedPtr<T> q) { return bounds_at(q.tb, q.p, q.site, static_cast<unsigned>(sizeof(T))); }
template <typename T>
__device__ __forceinline__ T *chk_bytes(CheckedPtr<T> q, unsigned bytes) { return bounds_at(q.tb, q.p, q.site, bytes); }
template <typename T>
inline Ptr<T> make_ptr(T *p, BoundsTable *tb, unsigned site) { return CheckedPtr<T>{p, tb, site}; }
#else
template <typename T> using Ptr = T *__restrict__;
template <typename T>
__device__ __forceinline__ T *chk(T *q) { return q; }
template <typename T>
__device__ __forceinline__ T *chk_bytes(T *q, unsigned) { return q; }
template <typename T>
inline T *make_ptr(T *p, BoundsTable *, unsigned) { return p; }
#endif

// host side (ema_api.cu): one (pointer, bytes) pair per buffer of the call
struct BoundsRange {
    const void *ptr;
    size_t bytes;
};
// Writes the ranges into this device's table on `stream` and returns the table (checked build); null otherwise.
BoundsTable *bounds_prepare(const BoundsRange *ranges, int n, cudaStream_t stream);
int bounds_read_status(int clear);

}  // namespace ema
