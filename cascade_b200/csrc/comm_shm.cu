// A caller-side collective for the ranks of ONE box: an all-gather of small host buffers through POSIX shared memory.
// The sharded build synchronises its ranks a dozen times per build with tiny payloads (partition sizes, counts, IPC
// handles); through a general-purpose collective each of those costs a few hundred microseconds, through shared memory a
// few microseconds. Waits are bounded: a rank that never arrives makes the others return an error, not hang.
//
// The object is made by rank 0 alone, exclusively: a leftover object of the same name (a crashed job, a reused process id)
// is marked dead and unlinked first, and the other ranks attach only to an object that is marked live, has this job's
// world size and whose round counters are those of a job that has not finished its first all-gather.
#include "common.cuh"

#include <atomic>
#include <cerrno>
#include <cstdlib>
#include <chrono>
#include <fcntl.h>
#include <new>
#include <sys/mman.h>
#include <sys/stat.h>
#include <thread>
#include <unistd.h>

namespace
{

constexpr size_t SHM_PAYLOAD = 48 * 1024;          // most bytes per rank and all-gather
constexpr double SHM_TIMEOUT_S = 120.0;             // default limit of every wait
constexpr uint64_t SHM_LIVE = 0x4353415f4c495645ull, SHM_DEAD = 0x4353415f44454144ull;

struct Shm_Header
{
    std::atomic<uint64_t> magic;                    // SHM_LIVE once rank 0 has made the object, SHM_DEAD when a later job replaces it
    uint64_t world;
    unsigned char pad[48];
};

struct Shm_Slot
{
    std::atomic<uint64_t> seq;                      // number of all-gathers this rank has published
    unsigned char pad[56];
    unsigned char data[2][SHM_PAYLOAD];             // payloads of even and odd rounds
};

struct Shm_Comm
{
    Shm_Header* header = nullptr;
    Shm_Slot* slots = nullptr;
    size_t bytes = 0;
    uint32_t rank = 0, world = 0;
    uint64_t round = 0;
    double timeout_s = SHM_TIMEOUT_S;
    std::string name;
};

double seconds_since(const std::chrono::steady_clock::time_point& t0)
{
    return std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
}

int shm_allgather(void* user, const void* send, void* recv, uint64_t bytes)
{
    Shm_Comm* c = static_cast<Shm_Comm*>(user);
    if(!c || bytes > SHM_PAYLOAD) return 1;
    const uint64_t r = ++c->round;                  // rounds count from 1
    Shm_Slot& mine = c->slots[c->rank];
    std::memcpy(mine.data[r & 1], send, bytes);
    mine.seq.store(r, std::memory_order_release);
    const auto t0 = std::chrono::steady_clock::now();
    for(uint32_t g = 0; g < c->world; ++g)
    {
        Shm_Slot& s = c->slots[g];
        uint32_t spins = 0;
        while(s.seq.load(std::memory_order_acquire) < r)
        {
            if(++spins > 2000)
            {
                std::this_thread::yield();
                if((spins & 255) == 0)
                {
                    if(c->header->magic.load(std::memory_order_acquire) != SHM_LIVE) return 3;     // the object was replaced by another job
                    if(seconds_since(t0) > c->timeout_s) return 2;                                  // a rank is missing
                }
            }
        }
        std::memcpy(static_cast<unsigned char*>(recv) + size_t(g) * bytes, s.data[r & 1], bytes);
    }
    return 0;
}

void* map_object(int fd, size_t bytes)
{
    void* p = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    return p == MAP_FAILED ? nullptr : p;
}

// Rank 0: replaces whatever carries the name by a fresh, zeroed object.
void* create_object(const char* name, size_t bytes, uint32_t world)
{
    for(int attempt = 0; attempt < 4; ++attempt)
    {
        const int old = shm_open(name, O_RDWR, 0600);
        if(old >= 0)
        {
            // a leftover: tell whoever is still attached to it, then drop the name
            struct stat sb;
            if(fstat(old, &sb) == 0 && size_t(sb.st_size) >= sizeof(Shm_Header))
                if(void* p = map_object(old, sizeof(Shm_Header)))
                {
                    static_cast<Shm_Header*>(p)->magic.store(SHM_DEAD, std::memory_order_release);
                    munmap(p, sizeof(Shm_Header));
                }
            close(old);
            shm_unlink(name);
        }
        const int fd = shm_open(name, O_CREAT | O_EXCL | O_RDWR, 0600);
        if(fd < 0) { if(errno == EEXIST) continue; return nullptr; }
        if(ftruncate(fd, off_t(bytes)) != 0) { close(fd); shm_unlink(name); return nullptr; }
        void* p = map_object(fd, bytes);
        close(fd);
        if(!p) { shm_unlink(name); return nullptr; }
        Shm_Header* h = static_cast<Shm_Header*>(p);
        h->world = world;
        h->magic.store(SHM_LIVE, std::memory_order_release);
        return p;
    }
    return nullptr;
}

// Other ranks: attach to the live object of this job, waiting for rank 0 to make it.
void* attach_object(const char* name, size_t bytes, uint32_t rank, uint32_t world, double timeout_s)
{
    const auto t0 = std::chrono::steady_clock::now();
    while(seconds_since(t0) <= timeout_s)
    {
        const int fd = shm_open(name, O_RDWR, 0600);
        if(fd >= 0)
        {
            struct stat sb;
            void* p = (fstat(fd, &sb) == 0 && size_t(sb.st_size) == bytes) ? map_object(fd, bytes) : nullptr;
            close(fd);
            if(p)
            {
                Shm_Header* h = static_cast<Shm_Header*>(p);
                Shm_Slot* slots = reinterpret_cast<Shm_Slot*>(h + 1);
                // A job that has not finished its first all-gather: nobody is past the first exchange and this rank has not published.
                bool fresh = h->magic.load(std::memory_order_acquire) == SHM_LIVE && h->world == world && slots[rank].seq.load(std::memory_order_acquire) == 0;
                for(uint32_t g = 0; fresh && g < world; ++g) fresh = slots[g].seq.load(std::memory_order_acquire) <= 1;
                if(fresh) return p;
                munmap(p, bytes);
            }
        }
        std::this_thread::sleep_for(std::chrono::milliseconds(1));
    }
    return nullptr;
}

}   // namespace

extern "C" int csa_comm_open_shm(const char* name, uint32_t rank, uint32_t world, uint32_t policy, csa_comm* out)
{
    if(!name || !out || world == 0 || world > CSA_MAX_GPUS || rank >= world) return CSA_E_INVALID;
    Shm_Comm* c = new(std::nothrow) Shm_Comm();
    if(!c) return CSA_E_NOMEM;
    c->rank = rank; c->world = world; c->name = name; c->bytes = sizeof(Shm_Header) + sizeof(Shm_Slot) * world;
    if(const char* t = std::getenv("CASCADE_COMM_TIMEOUT_S")) { const double v = std::atof(t); if(v > 0) c->timeout_s = v; }
    void* p = rank == 0 ? create_object(name, c->bytes, world) : attach_object(name, c->bytes, rank, world, c->timeout_s);
    if(!p) { delete c; return CSA_E_COMM; }
    c->header = static_cast<Shm_Header*>(p);
    c->slots = reinterpret_cast<Shm_Slot*>(c->header + 1);
    out->rank = rank; out->world = world; out->policy = policy; out->allgather = shm_allgather; out->user = c;
    return CSA_OK;
}

extern "C" int csa_comm_shm_set_timeout(csa_comm* comm, double seconds)
{
    if(!comm || !comm->user || comm->allgather != shm_allgather || !(seconds > 0)) return CSA_E_INVALID;
    static_cast<Shm_Comm*>(comm->user)->timeout_s = seconds;
    return CSA_OK;
}

extern "C" void csa_comm_close_shm(csa_comm* comm, int unlink_name)
{
    if(!comm || !comm->user) return;
    Shm_Comm* c = static_cast<Shm_Comm*>(comm->user);
    if(c->header) munmap(c->header, c->bytes);
    if(unlink_name) shm_unlink(c->name.c_str());
    delete c;
    comm->user = nullptr;
    comm->allgather = nullptr;
}
