// The page allocator of the cache manager: page ids 0..n-1 of one cache group, a free list used as a
// stack (so that a fresh pool hands out 0, 1, 2, ... and a page given back is the next one handed out),
// and a reference count per page. Host code only: it is built with the host compiler into a library of
// its own and called through a C interface, so it needs neither a GPU nor the CUDA toolkit.
//
// The reference keeps the same books in cpp/src/paged.cpp:17-61 (BlockPool: allocate throws when the
// list is empty, free below a count of one throws). Here every call returns a status instead of
// throwing across the C boundary; the Python wrapper turns the status into its exception.
#include <cstdint>
#include <new>
#include <vector>

#if defined(_WIN32)
#define NIBH_API extern "C" __declspec(dllexport)
#else
#define NIBH_API extern "C" __attribute__((visibility("default")))
#endif

namespace {

enum Status : int32_t {
    OK = 0,
    EMPTY = -1,        // fewer free pages than asked for; nothing was taken
    BAD_PAGE = -2,     // page id outside 0..n-1
    NOT_HELD = -3,     // free or incref of a page whose count is zero
    BAD_ARG = -4,
};

struct PagePool {
    std::vector<int32_t> free_stack;   // back() is handed out next
    std::vector<int32_t> ref;

    explicit PagePool(int32_t n) : ref(static_cast<size_t>(n), 0) {
        free_stack.reserve(static_cast<size_t>(n));
        for (int32_t p = n - 1; p >= 0; --p) free_stack.push_back(p);
    }
    bool valid(int32_t page) const { return page >= 0 && static_cast<size_t>(page) < ref.size(); }
};

}  // namespace

NIBH_API int32_t nibh_abi_version() { return 1; }

NIBH_API void* nibh_pool_create(int32_t num_pages) {
    if (num_pages <= 0) return nullptr;
    return new (std::nothrow) PagePool(num_pages);
}

NIBH_API void nibh_pool_destroy(void* pool) { delete static_cast<PagePool*>(pool); }

NIBH_API int32_t nibh_pool_num_pages(const void* pool) {
    return static_cast<int32_t>(static_cast<const PagePool*>(pool)->ref.size());
}

NIBH_API int32_t nibh_pool_num_free(const void* pool) {
    return static_cast<int32_t>(static_cast<const PagePool*>(pool)->free_stack.size());
}

// Takes n pages, all of them or none; their ids go to out[0..n) in the order they were taken.
NIBH_API int32_t nibh_pool_allocate(void* pool, int32_t n, int32_t* out) {
    PagePool* p = static_cast<PagePool*>(pool);
    if (n < 0 || (n > 0 && out == nullptr)) return BAD_ARG;
    if (static_cast<size_t>(n) > p->free_stack.size()) return EMPTY;
    for (int32_t i = 0; i < n; ++i) {
        const int32_t page = p->free_stack.back();
        p->free_stack.pop_back();
        p->ref[static_cast<size_t>(page)] = 1;
        out[i] = page;
    }
    return OK;
}

NIBH_API int32_t nibh_pool_incref(void* pool, int32_t page) {
    PagePool* p = static_cast<PagePool*>(pool);
    if (!p->valid(page)) return BAD_PAGE;
    if (p->ref[static_cast<size_t>(page)] <= 0) return NOT_HELD;
    ++p->ref[static_cast<size_t>(page)];
    return OK;
}

// Drops one reference of each page in pages[0..n); a page whose count reaches zero goes back on the
// stack. Entries below zero (a block table's "no page" mark) are skipped. Stops at the first error and
// returns its status with the number of entries already handled in *done (if given).
NIBH_API int32_t nibh_pool_free(void* pool, const int32_t* pages, int32_t n, int32_t* done) {
    PagePool* p = static_cast<PagePool*>(pool);
    if (n < 0 || (n > 0 && pages == nullptr)) return BAD_ARG;
    int32_t status = OK;
    int32_t i = 0;
    for (; i < n; ++i) {
        const int32_t page = pages[i];
        if (page < 0) continue;
        if (!p->valid(page)) { status = BAD_PAGE; break; }
        int32_t& r = p->ref[static_cast<size_t>(page)];
        if (r <= 0) { status = NOT_HELD; break; }
        if (--r == 0) p->free_stack.push_back(page);
    }
    if (done != nullptr) *done = i;
    return status;
}

// The count of a page, or BAD_PAGE.
NIBH_API int32_t nibh_pool_refcount(const void* pool, int32_t page) {
    const PagePool* p = static_cast<const PagePool*>(pool);
    if (!p->valid(page)) return BAD_PAGE;
    return p->ref[static_cast<size_t>(page)];
}

// Copies the free stack (bottom first) to out[0..cap); returns its size.
NIBH_API int32_t nibh_pool_free_list(const void* pool, int32_t* out, int32_t cap) {
    const PagePool* p = static_cast<const PagePool*>(pool);
    const int32_t n = static_cast<int32_t>(p->free_stack.size());
    for (int32_t i = 0; i < n && i < cap; ++i) out[i] = p->free_stack[static_cast<size_t>(i)];
    return n;
}
