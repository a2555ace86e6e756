// A caller-side collective for the ranks of ONE box: an all-gather of small host buffers through POSIX shared memory.
// The sharded build synchronises its ranks a dozen times per build with tiny payloads (partition sizes, counts, IPC
// handles); through a general-purpose collective each of those costs a few hundred microseconds, through shared memory a
// few microseconds. Waits are bounded: a rank that never arrives makes the others return an error, not hang.
#include "common.cuh"

#include <atomic>
#include <chrono>
#include <fcntl.h>
#include <new>
#include <sys/mman.h>
#include <thread>
#include <unistd.h>

namespace
{

constexpr size_t SHM_PAYLOAD = 48 * 1024;          // most bytes per rank and all-gather
constexpr double SHM_TIMEOUT_S = 120.0;

struct Shm_Slot
{
    std::atomic<uint64_t> seq;                      // number of all-gathers this rank has published
    unsigned char pad[56];
    unsigned char data[2][SHM_PAYLOAD];             // payloads of even and odd rounds
};

struct Shm_Comm
{
    Shm_Slot* slots = nullptr;
    size_t bytes = 0;
    uint32_t rank = 0, world = 0;
    uint64_t round = 0;
    std::string name;
};

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
                if((spins & 1023) == 0 && std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > SHM_TIMEOUT_S) return 2;
            }
        }
        std::memcpy(static_cast<unsigned char*>(recv) + size_t(g) * bytes, s.data[r & 1], bytes);
    }
    return 0;
}

}   // namespace

extern "C" int csa_comm_open_shm(const char* name, uint32_t rank, uint32_t world, uint32_t policy, csa_comm* out)
{
    if(!name || !out || world == 0 || world > CSA_MAX_GPUS || rank >= world) return CSA_E_INVALID;
    Shm_Comm* c = new(std::nothrow) Shm_Comm();
    if(!c) return CSA_E_NOMEM;
    c->rank = rank; c->world = world; c->name = name; c->bytes = sizeof(Shm_Slot) * world;
    // Every rank opens (and, if first, creates) the object; a fresh object is all zeros, which is the initial state.
    const int fd = shm_open(name, O_CREAT | O_RDWR, 0600);
    if(fd < 0) { delete c; return CSA_E_COMM; }
    if(ftruncate(fd, off_t(c->bytes)) != 0) { close(fd); delete c; return CSA_E_COMM; }
    void* p = mmap(nullptr, c->bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    close(fd);
    if(p == MAP_FAILED) { delete c; return CSA_E_COMM; }
    c->slots = static_cast<Shm_Slot*>(p);
    out->rank = rank; out->world = world; out->policy = policy; out->allgather = shm_allgather; out->user = c;
    return CSA_OK;
}

extern "C" void csa_comm_close_shm(csa_comm* comm, int unlink_name)
{
    if(!comm || !comm->user) return;
    Shm_Comm* c = static_cast<Shm_Comm*>(comm->user);
    if(c->slots) munmap(c->slots, c->bytes);
    if(unlink_name) shm_unlink(c->name.c_str());
    delete c;
    comm->user = nullptr;
    comm->allgather = nullptr;
}
