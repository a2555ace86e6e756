// `cascade <text-file> <suffix-array-file>`: the builder's command line, as the reference's (src/main.cu:12-46): reads a
// text of little-endian u16 symbols, builds its suffix array on the GPU, writes 5-byte entries. An empty output path
// builds without writing (include/GPU_SACA.hpp:301-304).
//
// Environment, names as in the reference where they apply:
//   GPU_SACA_P_TARGET     partitions to form (default 64; src/GPU_SACA.cu:413)
//   GPU_SACA_RAM_BUDGET   bytes of host memory the build may take (src/GPU_SACA.cu:50); default: 90 % of what is available.
//                         A build that needs more is refused before it starts, as the reference refuses (Host_Budget_Refusal)
//   GPU_SACA_FORCE_SPILL  if set and not 0: the suffix lists leave the device even where they would fit, i.e. the build runs
//                         part by part with its lists in host memory (the reference forces its lower tier the same way,
//                         src/Residency_Plan.cpp:44-45). Without it that build is chosen when the resident one does not fit the device
//   GPU_SACA_CHUNK_CAP    most suffixes of a part of that build (the reference's test knob for small slabs, src/GPU_SACA.cu:660)
//   GPU_SACA_SCRATCH      colon-separated scratch directories (src/GPU_SACA.cu:718-731): when the part-by-part build's lists
//                         do not fit GPU_SACA_RAM_BUDGET, the parts beyond it keep their lists in files there, striped over the
//                         directories; without it such a build is refused
//   CASCADE_DEVICE        CUDA device (default 0)
//   CASCADE_GPUS          GPUs to shard the build over (default 1): one host thread per GPU, devices CASCADE_DEVICE + i modulo
//                         the number of devices present
//   CASCADE_INDEX_DIR     if set, an index.meta for `query` is written there (what `sa_convert --meta-only` does)
//   CASCADE_VALIDATE      if set, spot-checks the order of 100000 random neighbours of the result on the host
#include "../../../include/cascade_b200.h"
#include "formats.hpp"

#include <cuda_runtime.h>

#include <atomic>
#include <chrono>
#include <cstdlib>
#include <random>
#include <thread>
#include <unistd.h>
#include <vector>

using namespace cascade_host;

static int cmp_suffixes(const uint16_t* T, uint64_t n, uint64_t i, uint64_t j, uint64_t max_cmp)
{
    const uint64_t li = n - i, lj = n - j, len = li < lj ? li : lj, lim = len < max_cmp ? len : max_cmp;
    for(uint64_t k = 0; k < lim; ++k) if(T[i + k] != T[j + k]) return T[i + k] < T[j + k] ? -1 : 1;
    if(lim == max_cmp && len > max_cmp) return 0;
    return li < lj ? -1 : 1;
}

// MemAvailable of /proc/meminfo in bytes (0 if it cannot be read).
static uint64_t available_host_bytes()
{
    std::ifstream is("/proc/meminfo");
    for(std::string key; is >> key; )
    {
        uint64_t kb = 0;
        if(key == "MemAvailable:" && (is >> kb)) return kb * 1024;
        is.ignore(4096, '\n');
    }
    return 0;
}

int main(int argc, char** argv)
{
    if(argc != 3)
    {
        std::fprintf(stderr, "Usage: cascade <text-file> <suffix-array-file>\n");
        return EXIT_FAILURE;
    }
    const std::string text_path = argv[1], sa_path = argv[2];
    const auto env_u64 = [](const char* k, uint64_t d) { const char* v = std::getenv(k); return v && *v ? std::strtoull(v, nullptr, 10) : d; };
    const int device = int(env_u64("CASCADE_DEVICE", 0));
    const uint32_t p = uint32_t(env_u64("GPU_SACA_P_TARGET", 64));

    uint64_t bytes = 0;
    if(!file_size(text_path, bytes) || bytes == 0 || bytes % 2 != 0)
    {
        std::fprintf(stderr, "error: cannot use %s as a text of 2-byte symbols\n", text_path.c_str());
        return EXIT_FAILURE;
    }
    const uint64_t n = bytes / 2;
    const auto t0 = std::chrono::steady_clock::now();
    const auto since = [&] { return std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count(); };

    if(cudaSetDevice(device) != cudaSuccess) { std::fprintf(stderr, "error: no CUDA device %d\n", device); return EXIT_FAILURE; }
    uint16_t* T = nullptr; uint8_t* SA = nullptr;
    if(cudaMallocHost(&T, (n + CSA_TEXT_PAD) * 2) != cudaSuccess || cudaMallocHost(&SA, 5 * n + CSA_SA_PAD_BYTES) != cudaSuccess)
    {
        std::fprintf(stderr, "error: cannot pin %.1f GB of host memory\n", double(7 * n) / 1e9);
        return EXIT_FAILURE;
    }
    std::string err;
    if(!read_file(text_path, T, bytes, err)) { std::fprintf(stderr, "error: %s\n", err.c_str()); return EXIT_FAILURE; }
    std::memset(T + n, 0, CSA_TEXT_PAD * 2);
    std::fprintf(stderr, "Loaded the text of %llu symbols. Time taken: %.3f s.\n", (unsigned long long)n, since());

    const uint32_t gpus = uint32_t(env_u64("CASCADE_GPUS", 1));
    // Which build: the resident one keeps every list on the device; the part-by-part one keeps them in host memory.
    size_t dev_free = 0, dev_total = 0;
    cudaMemGetInfo(&dev_free, &dev_total);
    const uint64_t resident_need = csa_build_device_bytes(n, p) + (n + CSA_TEXT_PAD) * 2 + 5 * n + CSA_SA_PAD_BYTES;
    const bool forced = env_u64("GPU_SACA_FORCE_SPILL", 0) != 0;
    const bool by_parts = gpus <= 1 && (forced || resident_need > dev_free || n >= (1ull << 32) - (1ull << 26));
    csa_tier_options tiers{};
    tiers.part_suffixes = env_u64("GPU_SACA_CHUNK_CAP", 0);
    tiers.host_list_bytes = ~uint64_t(0);
    if(by_parts)
    {
        // Host memory of that build beyond the text and the output, which are held already: 4 bytes per suffix of ranks (the
        // lanes live in the output array). Past the budget, the parts beyond it keep their lists in files if there is a
        // scratch directory; the build is refused if there is none, as the reference refuses (Host_Budget_Refusal).
        uint64_t budget = env_u64("GPU_SACA_RAM_BUDGET", 0);
        if(budget == 0) budget = uint64_t(0.9 * double(available_host_bytes()));
        const uint64_t need = 4 * n;
        if(budget != 0 && need > budget)
        {
            tiers.scratch_dir = std::getenv("GPU_SACA_SCRATCH");
            if(!tiers.scratch_dir)
            {
                std::fprintf(stderr, "error: the build would take %.1f GB more of host memory, past the budget of %.1f GB (GPU_SACA_RAM_BUDGET), "
                             "and GPU_SACA_SCRATCH names no directory for the lists\n", double(need) / 1e9, double(budget) / 1e9);
                return EXIT_FAILURE;
            }
            tiers.host_list_bytes = budget / 4 * 9;     // the bound counts 9 bytes a suffix, of which 5 are in the output array here
        }
    }
    csa_ctx* ctx = nullptr;
    const double b0 = since();
    if(gpus <= 1)
    {
        if(csa_ctx_create(device, &ctx) != CSA_OK) { std::fprintf(stderr, "error: cannot create a device context\n"); return EXIT_FAILURE; }
        csa_build_stats st{};
        const int rc = by_parts ? csa_build_sa_tiered(ctx, T, n, p, 0, SA, &tiers, &st) : csa_build_sa_host(ctx, T, n, p, 0, SA, &st);
        if(rc != CSA_OK) { std::fprintf(stderr, "error: build failed (%d): %s\n", rc, csa_last_error(ctx)); return EXIT_FAILURE; }
        if(by_parts) std::fprintf(stderr, "Built part by part (%s): the lists of %u parts in host memory, of %u parts in files (%.2f GB read, %.2f GB written).\n",
                                  forced ? "GPU_SACA_FORCE_SPILL" : "the resident build does not fit the device", st.host_parts, st.file_parts,
                                  double(st.file_bytes_read) / 1e9, double(st.file_bytes_written) / 1e9);
        std::fprintf(stderr, "Built the suffix array: %u partitions (largest %llu), %u doubling generations, %llu digit passes.\n", st.partitions,
                     (unsigned long long)st.max_partition, st.generations, (unsigned long long)st.sort_passes);
        std::fprintf(stderr, "Device time: partition %.1f ms, initial ranking %.1f ms, doubling %.1f ms, output %.1f ms.\n", st.ms_partition, st.ms_gen0,
                     st.ms_doubling, st.ms_output);
    }
    else
    {
        // One host thread per GPU; the threads meet in the library's shared-memory all-gather; every GPU gets the whole text,
        // builds its partitions' ranges and copies them to their places in the host array.
        if(gpus > CSA_MAX_GPUS) { std::fprintf(stderr, "error: CASCADE_GPUS is at most %d\n", CSA_MAX_GPUS); return EXIT_FAILURE; }
        int present = 0;
        if(cudaGetDeviceCount(&present) != cudaSuccess || present < 1) { std::fprintf(stderr, "error: no CUDA device\n"); return EXIT_FAILURE; }
        // a name of this run alone: process id and start time
        const std::string shm = "/cascade_b200_cli_" + std::to_string(getpid()) + "_" +
                                std::to_string(std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::system_clock::now().time_since_epoch()).count());
        std::vector<int> rcs(gpus, CSA_OK);
        std::vector<std::string> errs(gpus);
        std::vector<csa_build_stats> sts(gpus);
        std::vector<std::thread> pool;
        std::atomic<uint32_t> ready{0}, broken{0};      // ranks that have finished their set-up, and how many of them failed it
        for(uint32_t r = 0; r < gpus; ++r)
            pool.emplace_back([&, r]
            {
                const int dev = (device + int(r)) % present;
                csa_comm comm{};
                csa_ctx* c = nullptr;
                uint16_t* T_d = nullptr; uint8_t* out_d = nullptr;
                const uint64_t cap = n;     // room for any deal of the partitions
                bool comm_open = false;
                // Set-up first, on every rank; the ranks then meet, and nobody starts the build unless all of them can: a rank
                // that entered the build alone would wait for the others until its all-gather gave up.
                if(cudaSetDevice(dev) != cudaSuccess) { rcs[r] = CSA_E_CUDA; errs[r] = "cudaSetDevice"; }
                else if(csa_ctx_create(dev, &c) != CSA_OK) { rcs[r] = CSA_E_CUDA; errs[r] = "csa_ctx_create"; }
                else if(cudaMalloc(&T_d, (n + CSA_TEXT_PAD) * 2) != cudaSuccess || cudaMalloc(&out_d, 5 * cap + CSA_SA_PAD_BYTES) != cudaSuccess)
                { rcs[r] = CSA_E_NOMEM; errs[r] = "device memory for the text and the output"; }
                else if(cudaMemcpy(T_d, T, (n + CSA_TEXT_PAD) * 2, cudaMemcpyHostToDevice) != cudaSuccess) { rcs[r] = CSA_E_CUDA; errs[r] = "copy of the text"; }
                if(rcs[r] != CSA_OK) broken.fetch_add(1);
                ready.fetch_add(1);
                while(ready.load() < gpus) std::this_thread::yield();
                if(broken.load() == 0)
                {
                    if(csa_comm_open_shm(shm.c_str(), r, gpus, 1, &comm) != CSA_OK) { rcs[r] = CSA_E_COMM; errs[r] = "csa_comm_open_shm"; }
                    else
                    {
                        comm_open = true;
                        std::vector<uint64_t> seg_first(p), seg_count(p);
                        uint32_t seg_c = 0;
                        const int rc = csa_build_sa_multi(c, &comm, T_d, n, p, 0, out_d, cap, seg_first.data(), seg_count.data(), &seg_c, &sts[r]);
                        if(rc != CSA_OK) { rcs[r] = rc; errs[r] = csa_last_error(c); }
                        else
                        {
                            uint64_t at = 0;
                            for(uint32_t k = 0; k < seg_c; ++k)
                            {
                                cudaMemcpy(SA + 5 * seg_first[k], out_d + 5 * at, 5 * seg_count[k], cudaMemcpyDeviceToHost);
                                at += seg_count[k];
                            }
                        }
                    }
                }
                else if(rcs[r] == CSA_OK) { rcs[r] = CSA_E_COMM; errs[r] = "another rank could not be set up"; }
                cudaFree(T_d); cudaFree(out_d);
                if(c) csa_ctx_destroy(c);
                if(comm_open) csa_comm_close_shm(&comm, r == 0);
            });
        for(auto& t : pool) t.join();
        for(uint32_t r = 0; r < gpus; ++r)
            if(rcs[r] != CSA_OK) { std::fprintf(stderr, "error: build failed on GPU rank %u (%d): %s\n", r, rcs[r], errs[r].c_str()); return EXIT_FAILURE; }
        std::fprintf(stderr, "Built the suffix array on %u GPUs: %u partitions, %u doubling generations; rank 0 device time %.1f ms.\n", gpus, sts[0].partitions,
                     sts[0].generations, sts[0].ms_total);
    }
    const double build_s = since() - b0;
    std::fprintf(stderr, "Build with copies: %.3f s (%.1f M suffixes/s).\n", build_s, double(n) / build_s / 1e6);

    if(std::getenv("CASCADE_VALIDATE"))
    {
        std::mt19937_64 rng(1);
        uint64_t bad = 0;
        const auto at = [&](uint64_t r) { uint64_t v = 0; std::memcpy(&v, SA + 5 * r, 5); return v; };
        for(uint64_t k = 0; k < 100000 && n > 1; ++k)
        {
            const uint64_t r = k == 0 ? 0 : (k == 1 ? n - 2 : rng() % (n - 1));
            const uint64_t i = at(r), j = at(r + 1);
            if(i >= n || j >= n || i == j || cmp_suffixes(T, n, i, j, 1000) > 0) ++bad;
        }
        std::fprintf(stderr, "Order spot-check of 100000 neighbours: %s.\n", bad ? "FAILS" : "passes");
        if(bad) return EXIT_FAILURE;
    }
    if(!sa_path.empty())
    {
        if(!write_file(sa_path, SA, 5 * n, err)) { std::fprintf(stderr, "error: %s\n", err.c_str()); return EXIT_FAILURE; }
        std::fprintf(stderr, "Wrote %llu bytes to %s. Total time: %.3f s.\n", (unsigned long long)(5 * n), sa_path.c_str(), since());
        if(const char* dir = std::getenv("CASCADE_INDEX_DIR"))
        {
            Index_Meta m;
            m.n = n; m.text = text_path; m.sa_part = {sa_path}; m.sa_part_off = {0};
            if(!write_index_meta(dir, m, err)) { std::fprintf(stderr, "error: %s\n", err.c_str()); return EXIT_FAILURE; }
        }
    }
    if(ctx) csa_ctx_destroy(ctx);
    cudaFreeHost(T); cudaFreeHost(SA);
    return EXIT_SUCCESS;
}
