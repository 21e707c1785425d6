// Shared-memory collectives for CPU ranks of one host (no counterpart in the reference, whose only transport is NCCL).
//
// All ranks of a group map one POSIX shared-memory segment:
//
//     [ header | slot 0 | slot 1 | ... | slot W-1 ]
//
// A collective moves the payload through the slots in pieces of at most `slot_bytes`: every rank copies its piece into
// its own slot, a barrier makes the slots visible, every rank reads what it needs from the slots, a second barrier frees
// them for the next piece.  The barrier is a sense-reversing counter in the header; waiting is bounded (a rank that never
// arrives makes the others return an error after `timeout_s` instead of spinning forever).
#include <fcntl.h>
#include <sched.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstring>
#include <new>

namespace {

struct Header {
    std::atomic<uint32_t> arrived;
    std::atomic<uint32_t> sense;
    std::atomic<uint32_t> attached;
    uint32_t world;
    uint64_t slot_bytes;
    char pad[40];
};
static_assert(sizeof(Header) == 64, "header is one cache line");

struct Group {
    Header* hdr;
    char* slots;
    size_t map_bytes;
    int world, rank;
    uint64_t slot_bytes;
    uint32_t local_sense;
    double timeout_s;
    char name[128];
};

enum { OP_SUM = 0, OP_MAX = 1, OP_MIN = 2, OP_PROD = 3 };
enum { DT_F32 = 0, DT_F64 = 1, DT_I32 = 2, DT_I64 = 3, DT_U8 = 4 };

inline size_t dtype_size(int dt) { return dt == DT_F32 || dt == DT_I32 ? 4 : dt == DT_U8 ? 1 : 8; }

// 0 when every rank arrived, -2 after timeout_s.
int barrier(Group* g) {
    const uint32_t want = g->local_sense ^ 1u;
    g->local_sense = want;
    if (g->hdr->arrived.fetch_add(1, std::memory_order_acq_rel) + 1 == (uint32_t)g->world) {
        g->hdr->arrived.store(0, std::memory_order_relaxed);
        g->hdr->sense.store(want, std::memory_order_release);
        return 0;
    }
    const auto t0 = std::chrono::steady_clock::now();
    for (uint32_t spins = 0; g->hdr->sense.load(std::memory_order_acquire) != want; ++spins) {
        if ((spins & 63u) == 63u) {
            sched_yield();
            if (std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > g->timeout_s) return -2;
        } else {
            __builtin_ia32_pause();
        }
    }
    return 0;
}

template <typename T>
inline T combine(T a, T b, int op) {
    switch (op) {
        case OP_SUM: return a + b;
        case OP_MAX: return a > b ? a : b;
        case OP_MIN: return a < b ? a : b;
        default: return a * b;
    }
}

// dst[i] = op over ranks of slot_r[offset + i], ranks combined in rank order (every rank gets the same rounding).
template <typename T>
void reduce_slots(Group* g, T* dst, size_t elem_offset, size_t n, int op) {
    for (size_t i = 0; i < n; ++i) {
        T acc = ((const T*)(g->slots))[elem_offset + i];
        for (int r = 1; r < g->world; ++r) acc = combine(acc, ((const T*)(g->slots + (size_t)r * g->slot_bytes))[elem_offset + i], op);
        dst[i] = acc;
    }
}

void reduce_dispatch(Group* g, void* dst, size_t elem_offset, size_t n, int dt, int op) {
    switch (dt) {
        case DT_F32: reduce_slots<float>(g, (float*)dst, elem_offset, n, op); break;
        case DT_F64: reduce_slots<double>(g, (double*)dst, elem_offset, n, op); break;
        case DT_I32: reduce_slots<int32_t>(g, (int32_t*)dst, elem_offset, n, op); break;
        case DT_I64: reduce_slots<int64_t>(g, (int64_t*)dst, elem_offset, n, op); break;
        default: reduce_slots<uint8_t>(g, (uint8_t*)dst, elem_offset, n, op); break;
    }
}

}  // namespace

extern "C" {

// Maps (rank 0: creates) the segment `name` for a group of `world` ranks with `slot_bytes` per rank and waits (bounded) until
// every rank has attached.  Returns NULL on failure.
void* bmt_shm_open(const char* name, int world, int rank, uint64_t slot_bytes, double timeout_s) {
    if (world < 1 || rank < 0 || rank >= world || slot_bytes < 64 || strlen(name) >= sizeof(((Group*)0)->name)) return nullptr;
    slot_bytes = (slot_bytes + 63) & ~(uint64_t)63;
    const size_t bytes = sizeof(Header) + (size_t)world * slot_bytes;
    int fd = -1;
    const auto t0 = std::chrono::steady_clock::now();
    if (rank == 0) {
        shm_unlink(name);
        fd = shm_open(name, O_CREAT | O_EXCL | O_RDWR, 0600);
        if (fd < 0 || ftruncate(fd, (off_t)bytes) != 0) { if (fd >= 0) close(fd); return nullptr; }
    } else {
        // the creator may not have got there yet: retry until the segment exists with its full size
        for (;;) {
            fd = shm_open(name, O_RDWR, 0600);
            if (fd >= 0) {
                struct stat st;
                if (fstat(fd, &st) == 0 && (size_t)st.st_size >= bytes) break;
                close(fd);
                fd = -1;
            }
            if (std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > timeout_s) return nullptr;
            usleep(1000);
        }
    }
    void* p = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    close(fd);
    if (p == MAP_FAILED) return nullptr;
    Group* g = new (std::nothrow) Group();
    if (!g) { munmap(p, bytes); return nullptr; }
    g->hdr = (Header*)p;
    g->slots = (char*)p + sizeof(Header);
    g->map_bytes = bytes; g->world = world; g->rank = rank; g->slot_bytes = slot_bytes; g->local_sense = 0; g->timeout_s = timeout_s;
    strcpy(g->name, name);
    if (rank == 0) {
        // a fresh segment is zero-filled: counters start at 0; publish the geometry last
        g->hdr->slot_bytes = slot_bytes;
        g->hdr->world = (uint32_t)world;
    }
    g->hdr->attached.fetch_add(1, std::memory_order_acq_rel);
    while (g->hdr->attached.load(std::memory_order_acquire) < (uint32_t)world) {
        if (std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > timeout_s) {
            munmap(p, bytes);
            delete g;
            return nullptr;
        }
        usleep(200);
    }
    if (rank == 0) shm_unlink(name);  // everybody has it mapped: the name can go, the memory lives until the last unmap
    return g;
}

void bmt_shm_close(void* handle) {
    Group* g = (Group*)handle;
    if (!g) return;
    munmap((void*)g->hdr, g->map_bytes);
    delete g;
}

int bmt_shm_barrier(void* handle) { return barrier((Group*)handle); }

// In-place all-reduce of n elements.  Returns 0, -1 (bad argument) or -2 (a rank did not arrive in time).
int bmt_shm_all_reduce(void* handle, void* data, int64_t n, int dt, int op) {
    Group* g = (Group*)handle;
    if (!g || n < 0 || dt < 0 || dt > DT_U8 || op < 0 || op > OP_PROD) return -1;
    const size_t es = dtype_size(dt);
    const size_t per_piece = (size_t)(g->slot_bytes / es) / (size_t)g->world * (size_t)g->world;  // divisible by the world size
    if (per_piece == 0) return -1;
    char* mine = g->slots + (size_t)g->rank * g->slot_bytes;
    for (size_t done = 0; done < (size_t)n; done += per_piece) {
        const size_t cnt = (size_t)n - done < per_piece ? (size_t)n - done : per_piece;
        memcpy(mine, (char*)data + done * es, cnt * es);
        if (barrier(g)) return -2;
        // this rank reduces its share of the piece and leaves the result in its own slot, behind a second barrier so that
        // nobody overwrites a slot that is still being read
        const size_t share = (cnt + g->world - 1) / g->world;
        const size_t lo = share * g->rank < cnt ? share * g->rank : cnt;
        const size_t hi = lo + share < cnt ? lo + share : cnt;
        char tmp_stack[4096];
        char* tmp = (hi - lo) * es <= sizeof(tmp_stack) ? tmp_stack : new char[(hi - lo) * es];
        reduce_dispatch(g, tmp, lo, hi - lo, dt, op);
        if (barrier(g)) { if (tmp != tmp_stack) delete[] tmp; return -2; }
        memcpy(mine + lo * es, tmp, (hi - lo) * es);
        if (tmp != tmp_stack) delete[] tmp;
        if (barrier(g)) return -2;
        for (int r = 0; r < g->world; ++r) {
            const size_t rlo = share * r < cnt ? share * r : cnt;
            const size_t rhi = rlo + share < cnt ? rlo + share : cnt;
            memcpy((char*)data + (done + rlo) * es, g->slots + (size_t)r * g->slot_bytes + rlo * es, (rhi - rlo) * es);
        }
        if (barrier(g)) return -2;
    }
    return 0;
}

// dst (world * nbytes) = concatenation of every rank's src (nbytes) in rank order.
int bmt_shm_all_gather(void* handle, void* dst, const void* src, int64_t nbytes) {
    Group* g = (Group*)handle;
    if (!g || nbytes < 0) return -1;
    char* mine = g->slots + (size_t)g->rank * g->slot_bytes;
    for (size_t done = 0; done < (size_t)nbytes; done += g->slot_bytes) {
        const size_t cnt = (size_t)nbytes - done < g->slot_bytes ? (size_t)nbytes - done : (size_t)g->slot_bytes;
        memcpy(mine, (const char*)src + done, cnt);
        if (barrier(g)) return -2;
        for (int r = 0; r < g->world; ++r) memcpy((char*)dst + (size_t)r * nbytes + done, g->slots + (size_t)r * g->slot_bytes, cnt);
        if (barrier(g)) return -2;
    }
    return 0;
}

// dst (n elements) = op over ranks of src[rank * n .. (rank + 1) * n); src has world * n elements on every rank.
int bmt_shm_reduce_scatter(void* handle, void* dst, const void* src, int64_t n, int dt, int op) {
    Group* g = (Group*)handle;
    if (!g || n < 0 || dt < 0 || dt > DT_U8 || op < 0 || op > OP_PROD) return -1;
    const size_t es = dtype_size(dt);
    const size_t per_piece = (size_t)(g->slot_bytes / es) / (size_t)g->world;  // elements of one destination per piece
    if (per_piece == 0) return -1;
    char* mine = g->slots + (size_t)g->rank * g->slot_bytes;
    for (size_t done = 0; done < (size_t)n; done += per_piece) {
        const size_t cnt = (size_t)n - done < per_piece ? (size_t)n - done : per_piece;
        // slot layout of a piece: [to rank 0 | to rank 1 | ...], cnt elements each
        for (int r = 0; r < g->world; ++r) memcpy(mine + (size_t)r * cnt * es, (const char*)src + ((size_t)r * n + done) * es, cnt * es);
        if (barrier(g)) return -2;
        reduce_dispatch(g, (char*)dst + done * es, (size_t)g->rank * cnt, cnt, dt, op);
        if (barrier(g)) return -2;
    }
    return 0;
}

// data (nbytes) of rank `root` is copied to every rank.
int bmt_shm_broadcast(void* handle, void* data, int64_t nbytes, int root) {
    Group* g = (Group*)handle;
    if (!g || nbytes < 0 || root < 0 || root >= g->world) return -1;
    char* slot = g->slots + (size_t)root * g->slot_bytes;
    for (size_t done = 0; done < (size_t)nbytes; done += g->slot_bytes) {
        const size_t cnt = (size_t)nbytes - done < g->slot_bytes ? (size_t)nbytes - done : (size_t)g->slot_bytes;
        if (g->rank == root) memcpy(slot, (const char*)data + done, cnt);
        if (barrier(g)) return -2;
        if (g->rank != root) memcpy((char*)data + done, slot, cnt);
        if (barrier(g)) return -2;
    }
    return 0;
}

}  // extern "C"
