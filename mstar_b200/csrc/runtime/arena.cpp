// Shared-memory tensor arena: a /dev/shm segment with a first-fit, coalescing free-list allocator (256-byte
// granularity). A producer reserves a block, writes the tensor bytes and ships (segment, offset) in the tensor
// descriptor; a consumer in another process maps the segment and reads in place. Segments are added on demand
// ("<base>.seg<i>"). The allocator state lives in the process that owns the arena (the producer); consumers only
// map. Optional canary words around every block are checked on free.
//
// Reference counterparts: Rust `Allocator` / `ShmArena` / `SegmentedShmArena` (rust/src/shm.rs:49-374) and the
// Python arena transport (mstar/communication/arena.py:153-809).
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include <dlfcn.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#define MSTAR_RT_API extern "C" __attribute__((visibility("default")))

namespace {

constexpr uint64_t ALIGN = 256;
constexpr uint64_t CANARY = 0xC0FFEE5AFEC0DE11ull;

inline uint64_t align_up(uint64_t n) { return (n + ALIGN - 1) & ~(ALIGN - 1); }

struct Segment {
    std::string path;
    uint8_t* base = nullptr;
    uint64_t bytes = 0;
    std::map<uint64_t, uint64_t> free_blocks;   // offset -> size, coalesced
    std::map<uint64_t, uint64_t> used;          // offset -> size
    bool owner = false;
    bool pinned = false;                        // registered with the CUDA runtime (page-locked, DMA-able)
};

struct Arena {
    std::string base_name;
    uint64_t segment_bytes;
    int max_segments;
    bool canaries;
    std::vector<Segment> segs;
    std::mutex mu;
    uint64_t bytes_in_use = 0;
    uint64_t pin_budget = 0;                    // bytes that may be page-locked; 0 = pinning off
    uint64_t pinned_bytes = 0;
};

// ---- CUDA host registration -------------------------------------------------------------------------------
// A mapped /dev/shm segment is ordinary pageable memory: a copy between it and a GPU goes through the driver's
// staging buffer and blocks the calling thread. Registered with cudaHostRegister the segment is page-locked, copies
// from and to it are true asynchronous DMA, and a consumer can upload an arriving tensor straight from the producer's
// block. This library is built without CUDA: the two runtime entry points are looked up in an already loaded (or
// loadable) libcudart at run time, and a process without a GPU simply gets "unavailable". Tests install their own
// hooks instead.
typedef int (*HostRegisterFn)(void*, size_t, unsigned int);
typedef int (*HostUnregisterFn)(void*);
HostRegisterFn g_register = nullptr;
HostUnregisterFn g_unregister = nullptr;
bool g_hooks_set = false;
std::mutex g_pin_mu;

bool resolve_cuda() {
    std::lock_guard<std::mutex> lk(g_pin_mu);
    if (g_hooks_set) return g_register != nullptr;
    g_hooks_set = true;
    const char* names[] = {"libcudart.so.12", "libcudart.so.13", "libcudart.so"};
    void* lib = nullptr;
    for (const char* n : names) {
        lib = dlopen(n, RTLD_NOW | RTLD_NOLOAD);        // the copy the process already uses, if any
        if (lib) break;
    }
    for (const char* n : names) {
        if (lib) break;
        lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
    }
    if (!lib) return false;
    g_register = reinterpret_cast<HostRegisterFn>(dlsym(lib, "cudaHostRegister"));
    g_unregister = reinterpret_cast<HostUnregisterFn>(dlsym(lib, "cudaHostUnregister"));
    if (!g_register || !g_unregister) g_register = nullptr;
    return g_register != nullptr;
}

// Page-lock one mapped segment if the budget allows. Returns true when the segment is pinned afterwards.
bool pin_segment(Segment& s, uint64_t* budget_left) {
    if (s.pinned) return true;
    if (!resolve_cuda() || (budget_left && *budget_left < s.bytes)) return false;
    const unsigned int kPortable = 1;       // cudaHostRegisterPortable: valid in every CUDA context of the process
    if (g_register(s.base, (size_t)s.bytes, kPortable) != 0) return false;
    s.pinned = true;
    if (budget_left) *budget_left -= s.bytes;
    return true;
}

void unpin_segment(Segment& s) {
    if (s.pinned && g_unregister) g_unregister(s.base);
    s.pinned = false;
}

bool open_segment(Segment* s, const std::string& path, uint64_t bytes, bool create) {
    int fd = create ? ::open(path.c_str(), O_RDWR | O_CREAT | O_TRUNC, 0600) : ::open(path.c_str(), O_RDWR);
    if (fd < 0) return false;
    if (create && ftruncate(fd, (off_t)bytes) != 0) { ::close(fd); return false; }
    struct stat st;
    if (fstat(fd, &st) != 0) { ::close(fd); return false; }
    void* p = mmap(nullptr, (size_t)st.st_size, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    ::close(fd);
    if (p == MAP_FAILED) return false;
    s->path = path;
    s->base = static_cast<uint8_t*>(p);
    s->bytes = (uint64_t)st.st_size;
    s->owner = create;
    if (create) s->free_blocks[0] = s->bytes;
    return true;
}

bool seg_alloc(Segment& s, uint64_t need, uint64_t* off) {
    for (auto it = s.free_blocks.begin(); it != s.free_blocks.end(); ++it) {
        if (it->second >= need) {
            *off = it->first;
            const uint64_t rest = it->second - need;
            const uint64_t start = it->first;
            s.free_blocks.erase(it);
            if (rest) s.free_blocks[start + need] = rest;
            s.used[start] = need;
            return true;
        }
    }
    return false;
}

void seg_free(Segment& s, uint64_t off) {
    auto u = s.used.find(off);
    if (u == s.used.end()) return;
    uint64_t size = u->second;
    s.used.erase(u);
    auto next = s.free_blocks.lower_bound(off);
    if (next != s.free_blocks.end() && off + size == next->first) {
        size += next->second;
        next = s.free_blocks.erase(next);
    }
    if (next != s.free_blocks.begin()) {
        auto prev = std::prev(next);
        if (prev->first + prev->second == off) {
            prev->second += size;
            return;
        }
    }
    s.free_blocks[off] = size;
}

}  // namespace

MSTAR_RT_API void* mstar_arena_create(const char* base_name, unsigned long long segment_bytes, int max_segments,
                                      int canaries) {
    Arena* a = new Arena();
    a->base_name = base_name;
    a->segment_bytes = align_up(segment_bytes);
    a->max_segments = max_segments < 1 ? 1 : max_segments;
    a->canaries = canaries != 0;
    Segment s;
    if (!open_segment(&s, "/dev/shm/" + a->base_name + ".seg0", a->segment_bytes, true)) {
        delete a;
        return nullptr;
    }
    a->segs.push_back(std::move(s));
    return a;
}

// Reserve `bytes`; writes the segment index and the payload offset. Returns 0, or -1 when out of space.
MSTAR_RT_API int mstar_arena_reserve(void* h, unsigned long long bytes, int* seg_out, unsigned long long* off_out) {
    Arena* a = static_cast<Arena*>(h);
    if (!a) return -1;
    std::lock_guard<std::mutex> lk(a->mu);
    const uint64_t guard = a->canaries ? ALIGN : 0;
    const uint64_t need = align_up(bytes ? bytes : 1) + 2 * guard;
    for (;;) {
        for (size_t i = 0; i < a->segs.size(); ++i) {
            uint64_t off;
            if (seg_alloc(a->segs[i], need, &off)) {
                if (a->canaries) {
                    memcpy(a->segs[i].base + off, &CANARY, 8);
                    memcpy(a->segs[i].base + off + need - guard, &CANARY, 8);
                }
                *seg_out = (int)i;
                *off_out = off + guard;
                a->bytes_in_use += need;
                return 0;
            }
        }
        if ((int)a->segs.size() >= a->max_segments) return -1;
        Segment s;
        const std::string path = "/dev/shm/" + a->base_name + ".seg" + std::to_string(a->segs.size());
        // a block larger than the regular segment size (a decoded video) gets a segment of its own size
        if (!open_segment(&s, path, need > a->segment_bytes ? need : a->segment_bytes, true)) return -1;
        if (a->pin_budget > a->pinned_bytes) {          // a grown arena keeps its segments page-locked while the
            uint64_t left = a->pin_budget - a->pinned_bytes;     // budget lasts; later segments stay pageable
            if (pin_segment(s, &left)) a->pinned_bytes = a->pin_budget - left;
        }
        a->segs.push_back(std::move(s));
    }
}

// Page-lock the arena's segments for CUDA (cudaHostRegister), at most `budget_bytes` in total; segments added
// later are registered too while the budget lasts. Returns the number of pinned segments, or -1 when no CUDA
// runtime can be found in this process (the arena keeps working with pageable memory).
MSTAR_RT_API int mstar_arena_pin(void* h, unsigned long long budget_bytes) {
    Arena* a = static_cast<Arena*>(h);
    if (!a) return -1;
    if (!resolve_cuda()) return -1;
    std::lock_guard<std::mutex> lk(a->mu);
    a->pin_budget = budget_bytes;
    int n = 0;
    for (auto& s : a->segs) {
        if (!s.pinned && a->pin_budget > a->pinned_bytes) {
            uint64_t left = a->pin_budget - a->pinned_bytes;
            if (pin_segment(s, &left)) a->pinned_bytes = a->pin_budget - left;
        }
        n += s.pinned ? 1 : 0;
    }
    return n;
}

MSTAR_RT_API unsigned long long mstar_arena_pinned_bytes(void* h) {
    Arena* a = static_cast<Arena*>(h);
    return a ? a->pinned_bytes : 0;
}

// Consumer side: page-lock a mapped producer segment so that uploads from it are asynchronous. 1 = pinned.
MSTAR_RT_API int mstar_arena_pin_segment(void* seg_handle) {
    Segment* s = static_cast<Segment*>(seg_handle);
    return (s && pin_segment(*s, nullptr)) ? 1 : 0;
}

// Replace the CUDA entry points (tests without a GPU install counting fakes; nullptr restores the run-time lookup).
MSTAR_RT_API void mstar_arena_set_pin_hooks(HostRegisterFn reg, HostUnregisterFn unreg) {
    std::lock_guard<std::mutex> lk(g_pin_mu);
    g_register = reg;
    g_unregister = unreg;
    g_hooks_set = reg != nullptr;
}

// Returns 0, 1 when a canary around the block was overwritten (the block is freed anyway), -1 on a bad handle.
MSTAR_RT_API int mstar_arena_free(void* h, int seg, unsigned long long payload_off) {
    Arena* a = static_cast<Arena*>(h);
    if (!a || seg < 0 || seg >= (int)a->segs.size()) return -1;
    std::lock_guard<std::mutex> lk(a->mu);
    Segment& s = a->segs[seg];
    const uint64_t guard = a->canaries ? ALIGN : 0;
    const uint64_t off = payload_off - guard;
    auto u = s.used.find(off);
    if (u == s.used.end()) return -1;
    int rc = 0;
    if (a->canaries) {
        uint64_t c0, c1;
        memcpy(&c0, s.base + off, 8);
        memcpy(&c1, s.base + off + u->second - guard, 8);
        if (c0 != CANARY || c1 != CANARY) rc = 1;
    }
    a->bytes_in_use -= u->second;
    seg_free(s, off);
    return rc;
}

MSTAR_RT_API void* mstar_arena_ptr(void* h, int seg, unsigned long long payload_off) {
    Arena* a = static_cast<Arena*>(h);
    if (!a || seg < 0 || seg >= (int)a->segs.size()) return nullptr;
    return a->segs[seg].base + payload_off;
}

MSTAR_RT_API unsigned long long mstar_arena_bytes_in_use(void* h) {
    Arena* a = static_cast<Arena*>(h);
    return a ? a->bytes_in_use : 0;
}
MSTAR_RT_API int mstar_arena_num_segments(void* h) {
    Arena* a = static_cast<Arena*>(h);
    return a ? (int)a->segs.size() : 0;
}
MSTAR_RT_API unsigned long long mstar_arena_largest_free(void* h, int seg) {
    Arena* a = static_cast<Arena*>(h);
    if (!a || seg < 0 || seg >= (int)a->segs.size()) return 0;
    uint64_t best = 0;
    for (auto& kv : a->segs[seg].free_blocks) best = kv.second > best ? kv.second : best;
    return best;
}

// Consumer side: map a producer's segment read/write. Returns a handle usable with mstar_arena_view_ptr.
MSTAR_RT_API void* mstar_arena_open_segment(const char* base_name, int seg) {
    Segment* s = new Segment();
    if (!open_segment(s, std::string("/dev/shm/") + base_name + ".seg" + std::to_string(seg), 0, false)) {
        delete s;
        return nullptr;
    }
    return s;
}
MSTAR_RT_API void* mstar_arena_view_ptr(void* seg_handle, unsigned long long off) {
    Segment* s = static_cast<Segment*>(seg_handle);
    return (s && off < s->bytes) ? s->base + off : nullptr;
}
MSTAR_RT_API void mstar_arena_close_segment(void* seg_handle) {
    Segment* s = static_cast<Segment*>(seg_handle);
    if (!s) return;
    unpin_segment(*s);
    munmap(s->base, s->bytes);
    delete s;
}

MSTAR_RT_API void mstar_arena_destroy(void* h, int unlink_files) {
    Arena* a = static_cast<Arena*>(h);
    if (!a) return;
    for (auto& s : a->segs) {
        unpin_segment(s);
        munmap(s.base, s.bytes);
        if (unlink_files) ::unlink(s.path.c_str());
    }
    delete a;
}
