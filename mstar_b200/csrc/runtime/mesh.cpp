// Control mesh over shared memory: every entity owns ONE mailbox, a multi-producer / single-consumer byte ring in
// /dev/shm/<prefix>.<entity>.mbox. Senders (any process) reserve space with a CAS on the tail, copy the frame and
// publish it by storing its length word; the consumer reads frames in order. A futex word lets the consumer
// sleep in recv until a sender (or wake()) bumps it, so an idle worker costs no CPU.
//
// Frame: [u32 len | payload | pad to 8]. len == 0: not yet published; len == 0xFFFFFFFF: wrap marker.
//
// Reference counterpart: the Rust ZMQ PUSH/PULL mailbox with eventfd wake-up (rust/src/communicator.rs:99-305).
// On one box a shared-memory ring removes the socket hop and the per-peer socket mutex.
#include <atomic>
#include <cerrno>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <string>

#include <fcntl.h>
#include <linux/futex.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <sys/syscall.h>
#include <time.h>
#include <unistd.h>

#define MSTAR_RT_API extern "C" __attribute__((visibility("default")))

namespace {

constexpr uint32_t MAGIC = 0x4d535452;  // "MSTR"
constexpr uint32_t WRAP = 0xFFFFFFFFu;

struct RingHeader {
    uint32_t magic;
    uint32_t ready;                    // set last by the creator
    uint64_t capacity;                 // bytes of the data area (power of two not required)
    std::atomic<uint64_t> tail;        // next byte to reserve (monotonic)
    std::atomic<uint64_t> head;        // next byte to consume (monotonic)
    std::atomic<uint32_t> futex_word;  // bumped on every publish / wake
    uint32_t pad;
};

struct Ring {
    RingHeader* hdr = nullptr;
    uint8_t* data = nullptr;
    size_t map_bytes = 0;
    std::string path;
};

long futex(std::atomic<uint32_t>* addr, int op, uint32_t val, const timespec* ts) {
    return syscall(SYS_futex, reinterpret_cast<uint32_t*>(addr), op, val, ts, nullptr, 0);
}

std::string mbox_path(const std::string& prefix, const std::string& entity) {
    return "/dev/shm/" + prefix + "." + entity + ".mbox";
}

bool map_ring(Ring* r, const std::string& path, uint64_t create_bytes) {
    int fd;
    if (create_bytes) {
        ::unlink(path.c_str());
        fd = ::open(path.c_str(), O_RDWR | O_CREAT | O_EXCL, 0600);
        if (fd < 0) return false;
        if (ftruncate(fd, (off_t)(sizeof(RingHeader) + create_bytes)) != 0) { ::close(fd); return false; }
    } else {
        fd = ::open(path.c_str(), O_RDWR);
        if (fd < 0) return false;
    }
    struct stat st;
    if (fstat(fd, &st) != 0 || (size_t)st.st_size < sizeof(RingHeader) + 64) { ::close(fd); return false; }
    void* p = mmap(nullptr, (size_t)st.st_size, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    ::close(fd);
    if (p == MAP_FAILED) return false;
    r->hdr = static_cast<RingHeader*>(p);
    r->data = static_cast<uint8_t*>(p) + sizeof(RingHeader);
    r->map_bytes = (size_t)st.st_size;
    r->path = path;
    if (create_bytes) {
        r->hdr->capacity = create_bytes;
        r->hdr->tail.store(0);
        r->hdr->head.store(0);
        r->hdr->futex_word.store(0);
        r->hdr->magic = MAGIC;
        std::atomic_thread_fence(std::memory_order_release);
        r->hdr->ready = 1;
    } else if (r->hdr->magic != MAGIC || !r->hdr->ready) {
        munmap(p, r->map_bytes);
        r->hdr = nullptr;
        return false;
    }
    return true;
}

struct Mesh {
    std::string prefix, entity;
    Ring own;
    std::map<std::string, Ring> peers;
    std::mutex mu;
};

inline uint64_t pad8(uint64_t n) { return (n + 7) & ~uint64_t(7); }

// Reserve `need` contiguous bytes; returns the ring offset or UINT64_MAX when the ring is full.
uint64_t reserve(Ring& r, uint64_t need, bool* wrapped, uint64_t* wrap_at) {
    RingHeader* h = r.hdr;
    const uint64_t cap = h->capacity;
    for (;;) {
        uint64_t tail = h->tail.load(std::memory_order_relaxed);
        const uint64_t head = h->head.load(std::memory_order_acquire);
        const uint64_t off = tail % cap;
        uint64_t total = need;
        bool wr = false;
        if (off + need > cap) {     // does not fit before the end: skip to the start
            total = (cap - off) + need;
            wr = true;
        }
        if (tail + total - head > cap) return UINT64_MAX;
        if (h->tail.compare_exchange_weak(tail, tail + total, std::memory_order_acq_rel)) {
            *wrapped = wr;
            *wrap_at = off;
            return wr ? 0 : off;
        }
    }
}

}  // namespace

MSTAR_RT_API void* mstar_mesh_create(const char* prefix, const char* entity, unsigned long long ring_bytes) {
    Mesh* m = new Mesh();
    m->prefix = prefix;
    m->entity = entity;
    ring_bytes = pad8(ring_bytes < 4096 ? 4096 : ring_bytes);
    if (!map_ring(&m->own, mbox_path(m->prefix, m->entity), ring_bytes)) {
        delete m;
        return nullptr;
    }
    return m;
}

// 0 ok; -1 hard error; -2 transient (peer mailbox missing or ring full) — the caller may retry.
MSTAR_RT_API int mstar_mesh_send(void* handle, const char* dst, const char* payload, unsigned long long len) {
    Mesh* m = static_cast<Mesh*>(handle);
    if (!m || len == 0 || len >= 0x7fffffffull) return -1;
    Ring* r;
    {
        std::lock_guard<std::mutex> lk(m->mu);
        auto it = m->peers.find(dst);
        if (it == m->peers.end()) {
            Ring pr;
            if (!map_ring(&pr, mbox_path(m->prefix, dst), 0)) return -2;
            it = m->peers.emplace(dst, pr).first;
        }
        r = &it->second;
    }
    const uint64_t need = pad8(4 + len);
    if (need + 8 > r->hdr->capacity) return -1;
    bool wrapped = false;
    uint64_t wrap_at = 0;
    const uint64_t off = reserve(*r, need, &wrapped, &wrap_at);
    if (off == UINT64_MAX) return -2;
    if (wrapped) {
        // tell the consumer to jump to offset 0 (only if a length word still fits there)
        if (wrap_at + 4 <= r->hdr->capacity) {
            reinterpret_cast<std::atomic<uint32_t>*>(r->data + wrap_at)->store(WRAP, std::memory_order_release);
        }
    }
    memcpy(r->data + off + 4, payload, len);
    reinterpret_cast<std::atomic<uint32_t>*>(r->data + off)->store((uint32_t)len, std::memory_order_release);
    r->hdr->futex_word.fetch_add(1, std::memory_order_release);
    futex(&r->hdr->futex_word, FUTEX_WAKE, 1, nullptr);
    return 0;
}

static long long try_pop(Mesh* m, char* out, unsigned long long cap_out, bool peek_only) {
    Ring& r = m->own;
    RingHeader* h = r.hdr;
    const uint64_t cap = h->capacity;
    for (;;) {
        const uint64_t head = h->head.load(std::memory_order_relaxed);
        if (head == h->tail.load(std::memory_order_acquire)) return 0;
        uint64_t off = head % cap;
        if (off + 4 > cap) {   // no room for a length word: implicit wrap
            h->head.store(head + (cap - off), std::memory_order_release);
            continue;
        }
        std::atomic<uint32_t>* lw = reinterpret_cast<std::atomic<uint32_t>*>(r.data + off);
        const uint32_t len = lw->load(std::memory_order_acquire);
        if (len == 0) return 0;    // reserved but not yet published
        if (len == WRAP) {
            lw->store(0, std::memory_order_relaxed);
            h->head.store(head + (cap - off), std::memory_order_release);
            continue;
        }
        if (peek_only) return (long long)len;
        if (len > cap_out) return -3;
        memcpy(out, r.data + off + 4, len);
        const uint64_t used = pad8(4 + (uint64_t)len);
        memset(r.data + off, 0, used);     // length words must read 0 before the space is reused
        h->head.store(head + used, std::memory_order_release);
        return (long long)len;
    }
}

// Returns the payload length, 0 when nothing arrived within timeout_us microseconds (0 = poll), -3 when `cap` is
// too small. Sub-millisecond waits matter: a worker whose batches are on the GPU sleeps here in slices of a few
// hundred microseconds, and a wait rounded down to zero would turn that into a spin.
MSTAR_RT_API long long mstar_mesh_recv_us(void* handle, char* out, unsigned long long cap, long long timeout_us) {
    Mesh* m = static_cast<Mesh*>(handle);
    if (!m) return -1;
    long long n = try_pop(m, out, cap, false);
    if (n != 0 || timeout_us <= 0) return n;
    const uint32_t seen = m->own.hdr->futex_word.load(std::memory_order_acquire);
    n = try_pop(m, out, cap, false);
    if (n != 0) return n;
    timespec ts;
    ts.tv_sec = (time_t)(timeout_us / 1000000);
    ts.tv_nsec = (long)(timeout_us % 1000000) * 1000L;
    futex(&m->own.hdr->futex_word, FUTEX_WAIT, seen, &ts);
    return try_pop(m, out, cap, false);
}

MSTAR_RT_API long long mstar_mesh_recv(void* handle, char* out, unsigned long long cap, int timeout_ms) {
    return mstar_mesh_recv_us(handle, out, cap, (long long)timeout_ms * 1000);
}

MSTAR_RT_API long long mstar_mesh_peek_size(void* handle) {
    Mesh* m = static_cast<Mesh*>(handle);
    return m ? try_pop(m, nullptr, 0, true) : -1;
}

MSTAR_RT_API void mstar_mesh_wake(void* handle) {
    Mesh* m = static_cast<Mesh*>(handle);
    if (!m) return;
    m->own.hdr->futex_word.fetch_add(1, std::memory_order_release);
    futex(&m->own.hdr->futex_word, FUTEX_WAKE, 64, nullptr);
}

MSTAR_RT_API void mstar_mesh_destroy(void* handle, int unlink_own) {
    Mesh* m = static_cast<Mesh*>(handle);
    if (!m) return;
    for (auto& kv : m->peers) munmap(kv.second.hdr, kv.second.map_bytes);
    if (m->own.hdr) munmap(m->own.hdr, m->own.map_bytes);
    if (unlink_own) ::unlink(m->own.path.c_str());
    delete m;
}
