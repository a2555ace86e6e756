// TEST INFRASTRUCTURE ONLY. A thin extern "C" face over the reference's own CPU code for the
// suffix-array build and query path, so that Python tests and the CPU-baseline leg of the
// benchmark can call it through ctypes. It is compiled together with the reference's sources
// where they lie (see the Makefile beside this file); nothing of the reference is copied here.
//
// Functions of the reference that are reached:
//   test::build_sa40<uint16_t>        test/query.cpp:42-55        comparison-sort SA builder
//   test::is_correct_SA<uint16_t>     test/end-to-end.cpp:46-80   permutation + rank-order validator
//   test::brute_find<uint16_t>        test/query.cpp:82-97        suffix-array-free interval
//   ref::find_one<uint16_t>           include/CPU_Reference.hpp:42-73
//   ref::certify<uint16_t>            include/CPU_Reference.hpp:79-101
//   ref::cmp_suffixes<uint16_t>       include/CPU_Reference.hpp:107-123
//   host_search::find<uint16_t>       src/Host_Search.cpp:519-538 multi-threaded interleaved search
//   query_file::counts_hash           include/query-file.hpp:228-263

#include "CPU_Reference.hpp"
#include "Host_Search.hpp"
#include "query_tests.hpp"
#include "query-file.hpp"
#include "sa40.hpp"
#include "types.hpp"

#include <parallel/algorithm>
#include <omp.h>

#include <cstdint>
#include <cstring>
#include <vector>

namespace gpu_saca::test
{
bool is_permutation(const idx_t* SA, idx_t n);
template <typename T_sym_> bool is_correct_SA(const idx_t* SA, const T_sym_* T, idx_t n);
}

using namespace gpu_saca;

extern "C"
{

// Builds the sa40 array of `T[0, n)` with the reference's single-threaded comparison sort.
// `sa40_out` holds `5 n` bytes.
void ref_build_sa40(const uint16_t* T, uint64_t n, uint8_t* sa40_out)
{
    const std::vector<uint16_t> text(T, T + n);
    const auto SA = test::build_sa40(text);
    std::memcpy(sa40_out, SA.data(), SA_WIDTH * n);
}

// The same order through the reference's comparator `ref::cmp_suffixes`, sorted on every core:
// the form of the reference's CPU builder that a benchmark can time on all host threads.
void ref_build_sa40_parallel(const uint16_t* T, uint64_t n, uint8_t* sa40_out)
{
    std::vector<idx_t> sa(n);
    #pragma omp parallel for schedule(static)
    for(idx_t i = 0; i < n; ++i)
        sa[i] = i;

    __gnu_parallel::sort(sa.begin(), sa.end(), [&](const idx_t i, const idx_t j) { return ref::cmp_suffixes(T, n, i, j, n) < 0; });

    #pragma omp parallel for schedule(static)
    for(idx_t r = 0; r < n; ++r)
        sa40::store(sa40_out, r, sa[r]);
}

// Returns 1 iff the 5-byte suffix array is the suffix array of `T[0, n)` by the reference's validator.
int ref_is_correct_sa40(const uint16_t* T, uint64_t n, const uint8_t* sa40_in)
{
    std::vector<idx_t> sa(n);
    #pragma omp parallel for schedule(static)
    for(idx_t r = 0; r < n; ++r)
    {
        idx_t v = 0;
        std::memcpy(&v, sa40_in + SA_WIDTH * r, SA_WIDTH);
        sa[r] = v;
    }

    return test::is_correct_SA<uint16_t>(sa.data(), T, n) ? 1 : 0;
}

// `SA` must be padded as the reference pads it (`SA_PAD_BYTES`) only for device use; the host path reads 5 bytes.
void ref_find_one(const uint16_t* T, uint64_t n, const uint8_t* SA, const uint16_t* P, uint64_t m, uint64_t* lo, uint64_t* hi)
{
    const auto I = ref::find_one(T, n, SA, P, m);
    *lo = I.lo;
    *hi = I.hi;
}

void ref_brute_find(const uint16_t* T, uint64_t n, const uint16_t* P, uint64_t m, uint64_t* lo, uint64_t* hi)
{
    const auto I = test::brute_find(T, n, P, m);
    *lo = I.lo;
    *hi = I.hi;
}

int ref_certify(const uint16_t* T, uint64_t n, const uint8_t* SA, const uint16_t* P, uint64_t m, uint64_t lo, uint64_t hi)
{
    return ref::certify(T, n, SA, P, m, SA_Interval{lo, hi}) ? 1 : 0;
}

// The reference's batched host search, direct mode (no brackets). `itv_out` holds `2 q` words {lo, hi}.
// `T` and `SA` must carry the reference's tail padding (64 B and 128 B).
void ref_host_search_find(const uint16_t* T, uint64_t n, const uint8_t* SA, const uint64_t* off, const uint16_t* sym, uint64_t q,
                          uint64_t* itv_out, unsigned threads, unsigned lanes)
{
    host_search::find<uint16_t>(T, n, SA, off, sym, q, nullptr, nullptr, reinterpret_cast<SA_Interval*>(itv_out), threads, lanes);
}

uint64_t ref_counts_hash(const uint64_t* itv, uint64_t q)
{
    return query_file::counts_hash(reinterpret_cast<const SA_Interval*>(itv), q);
}

unsigned ref_thread_count(void)
{
    return host_search::thread_count(0);
}

// Sets the OpenMP team size of the calls above (a launcher may have exported OMP_NUM_THREADS=1 for its children).
void ref_set_threads(int threads)
{
    if(threads > 0)
        omp_set_num_threads(threads);
}

}
