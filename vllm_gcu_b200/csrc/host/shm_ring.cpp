// Broadcast ring in shared memory: one writer, R readers, every reader sees every message.
//
// The front-end process of the multi-process executor sends each command (new request,
// abort, stop) to all worker processes.  The reference does this through vLLM's
// shared-memory message queue and patches in a reader with a timeout, a cancel event and an
// asyncio form (vllm_gcu/patch/patch_0_9_2/shm_broadcast.py:16-101).  This file is the
// native part of this package's own queue: the memory layout and every access that needs
// atomics or ordering.  The region itself is created by the Python side
// (multiprocessing.shared_memory) and handed in as a raw pointer, so that its lifetime
// follows the Python objects.
//
// Layout (all offsets from the base pointer, which is page aligned):
//   Header      64 bytes      magic, slot count, slot payload bytes, reader count, write cursor
//   Cursor[R]   64 bytes each one read cursor per reader, each on its own cache line
//   Slot[S]     64-byte header (sequence, payload length, "more chunks follow" flag)
//               + payload bytes rounded up to 64
//
// Protocol: cursors count slots since start-up.  The writer may fill slot (w % S) when every
// reader's cursor is > w - S; it copies the payload, then publishes sequence = w + 1 with
// release order.  Reader r takes slot (c % S) once its sequence reads c + 1 (acquire), copies
// the payload out and then advances its cursor with release order, which hands the slot back.
// A message longer than one slot travels as consecutive chunks with the "more" flag set on
// all but the last; the caller reassembles them.  Nothing here blocks forever: every wait
// takes a deadline and returns kTimeout when it passes.
#include <atomic>
#include <cstdint>
#include <cstring>
#include <ctime>
#include <new>
#include <sched.h>

namespace {

constexpr uint64_t kMagic = 0x42323030524e4731ull;   // "B200RNG1"
constexpr int kOk = 0, kTimeout = -1, kBadArg = -2, kTooSmall = -3, kNotReady = -4;

struct alignas(64) Header {
    uint64_t magic;
    uint32_t slots;
    uint32_t slot_bytes;
    uint32_t readers;
    uint32_t reserved;
    std::atomic<uint64_t> write_cursor;
};

struct alignas(64) Cursor {
    std::atomic<uint64_t> value;
};

struct alignas(64) SlotHeader {
    std::atomic<uint64_t> sequence;
    uint32_t length;
    uint32_t more;
};

static_assert(sizeof(Header) == 64 && sizeof(Cursor) == 64 && sizeof(SlotHeader) == 64, "layout");

inline uint64_t round64(uint64_t v) { return (v + 63) & ~uint64_t(63); }

struct View {
    Header* h;
    Cursor* cursors;
    unsigned char* slots;
    uint64_t stride;

    SlotHeader* slot(uint64_t index) const {
        return reinterpret_cast<SlotHeader*>(slots + (index % h->slots) * stride);
    }
    unsigned char* payload(uint64_t index) const {
        return reinterpret_cast<unsigned char*>(slot(index)) + sizeof(SlotHeader);
    }
};

inline bool view_of(void* base, View& v) {
    if (base == nullptr) return false;
    v.h = static_cast<Header*>(base);
    if (v.h->magic != kMagic || v.h->slots == 0 || v.h->readers == 0) return false;
    v.cursors = reinterpret_cast<Cursor*>(static_cast<unsigned char*>(base) + sizeof(Header));
    v.slots = reinterpret_cast<unsigned char*>(v.cursors + v.h->readers);
    v.stride = sizeof(SlotHeader) + round64(v.h->slot_bytes);
    return true;
}

inline int64_t now_ns() {
    timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return int64_t(ts.tv_sec) * 1000000000ll + ts.tv_nsec;
}

// Spin briefly, then yield, then sleep in growing steps up to 200 us: a waiting process costs
// next to nothing while idle and still reacts within a fraction of a millisecond.
struct Backoff {
    int round = 0;
    void pause() {
        if (round < 64) {
#if defined(__x86_64__)
            __builtin_ia32_pause();
#endif
        } else if (round < 128) {
            sched_yield();
        } else {
            long ns = 5000L * (round - 127);
            if (ns > 200000L) ns = 200000L;
            timespec ts{0, ns};
            nanosleep(&ts, nullptr);
        }
        ++round;
    }
};

uint64_t slowest_reader(const View& v) {
    uint64_t lo = ~uint64_t(0);
    for (uint32_t r = 0; r < v.h->readers; ++r) {
        uint64_t c = v.cursors[r].value.load(std::memory_order_acquire);
        if (c < lo) lo = c;
    }
    return lo;
}

}  // namespace

extern "C" {

// Bytes the region must have for this geometry.
__attribute__((visibility("default")))
uint64_t b200_ring_bytes(uint32_t slots, uint32_t slot_bytes, uint32_t readers) {
    return sizeof(Header) + uint64_t(readers) * sizeof(Cursor) +
           uint64_t(slots) * (sizeof(SlotHeader) + round64(slot_bytes));
}

// Formats a zero-filled region.  Called once by the creator before any other process maps it.
__attribute__((visibility("default")))
int b200_ring_init(void* base, uint64_t bytes, uint32_t slots, uint32_t slot_bytes,
                   uint32_t readers) {
    if (base == nullptr || slots == 0 || slot_bytes == 0 || readers == 0) return kBadArg;
    if (bytes < b200_ring_bytes(slots, slot_bytes, readers)) return kTooSmall;
    if (reinterpret_cast<uintptr_t>(base) % 64 != 0) return kBadArg;
    Header* h = new (base) Header;
    h->slots = slots;
    h->slot_bytes = slot_bytes;
    h->readers = readers;
    h->reserved = 0;
    h->write_cursor.store(0, std::memory_order_relaxed);
    h->magic = kMagic;
    View v;
    if (!view_of(base, v)) return kBadArg;
    for (uint32_t r = 0; r < readers; ++r) new (&v.cursors[r]) Cursor{};
    for (uint32_t s = 0; s < slots; ++s) {
        SlotHeader* sh = new (v.slot(s)) SlotHeader;
        sh->sequence.store(0, std::memory_order_relaxed);
        sh->length = 0;
        sh->more = 0;
    }
    std::atomic_thread_fence(std::memory_order_seq_cst);
    return kOk;
}

// Writes one message (split into chunks when longer than a slot).  Waits for slow readers
// until the deadline; chunks already published stay published, so after kTimeout the ring must
// be considered broken by the caller (the executor marks itself dead).
__attribute__((visibility("default")))
int b200_ring_write(void* base, const void* data, uint64_t length, int64_t timeout_ns) {
    View v;
    if (!view_of(base, v) || (data == nullptr && length != 0)) return kBadArg;
    const unsigned char* src = static_cast<const unsigned char*>(data);
    const int64_t deadline = timeout_ns < 0 ? INT64_MAX : now_ns() + timeout_ns;
    uint64_t left = length;
    do {
        uint64_t w = v.h->write_cursor.load(std::memory_order_relaxed);
        Backoff b;
        while (slowest_reader(v) + v.h->slots <= w) {
            if (now_ns() > deadline) return kTimeout;
            b.pause();
        }
        uint32_t n = left > v.h->slot_bytes ? v.h->slot_bytes : uint32_t(left);
        SlotHeader* sh = v.slot(w);
        std::memcpy(v.payload(w), src, n);
        sh->length = n;
        sh->more = left > n ? 1u : 0u;
        sh->sequence.store(w + 1, std::memory_order_release);
        v.h->write_cursor.store(w + 1, std::memory_order_release);
        src += n;
        left -= n;
    } while (left > 0);
    return kOk;
}

// Takes the next chunk for `reader` if one is there.  Returns its length (>= 0) and sets
// *more when further chunks of the same message follow; kNotReady when the ring is empty for
// this reader; kTooSmall (and *needed) when `capacity` cannot hold the chunk.
__attribute__((visibility("default")))
int64_t b200_ring_try_read(void* base, uint32_t reader, void* out, uint64_t capacity,
                           uint32_t* more, uint64_t* needed) {
    View v;
    if (!view_of(base, v) || reader >= v.h->readers || out == nullptr) return kBadArg;
    uint64_t c = v.cursors[reader].value.load(std::memory_order_relaxed);
    SlotHeader* sh = v.slot(c);
    if (sh->sequence.load(std::memory_order_acquire) != c + 1) return kNotReady;
    uint32_t n = sh->length;
    if (n > capacity) {
        if (needed) *needed = n;
        return kTooSmall;
    }
    std::memcpy(out, v.payload(c), n);
    if (more) *more = sh->more;
    v.cursors[reader].value.store(c + 1, std::memory_order_release);
    return int64_t(n);
}

// As b200_ring_try_read, but waits up to timeout_ns for a chunk (kTimeout when none came).
// Callers that need a cancel flag or an unbounded wait call this in short slices.
__attribute__((visibility("default")))
int64_t b200_ring_read(void* base, uint32_t reader, void* out, uint64_t capacity,
                       uint32_t* more, uint64_t* needed, int64_t timeout_ns) {
    const int64_t deadline = now_ns() + (timeout_ns < 0 ? 0 : timeout_ns);
    Backoff b;
    for (;;) {
        int64_t r = b200_ring_try_read(base, reader, out, capacity, more, needed);
        if (r != kNotReady) return r;
        if (now_ns() > deadline) return kTimeout;
        b.pause();
    }
}

// Messages written so far, and how many reader `reader` has yet to take (in slots).
__attribute__((visibility("default")))
int64_t b200_ring_backlog(void* base, uint32_t reader) {
    View v;
    if (!view_of(base, v) || reader >= v.h->readers) return kBadArg;
    uint64_t w = v.h->write_cursor.load(std::memory_order_acquire);
    uint64_t c = v.cursors[reader].value.load(std::memory_order_acquire);
    return int64_t(w - c);
}

}  // extern "C"
