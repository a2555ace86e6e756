// Host-side helpers of the drop-in surface that need no GPU: the query-batch generator with the semantics of the
// reference's `query gen` (src/query.cu:826-882: std::mt19937_64(seed), lengths drawn as lens[rng() % |lens|],
// substring places as rng() % (n - len + 1), random symbols as rng() % vocab) and the FNV-1a hash of the counts
// (include/query-file.hpp:228-263).
#include "common.cuh"

#include <random>
#include <vector>

extern "C" int csa_gen_queries_host(int kind, const uint16_t* text_host, uint64_t n, uint64_t q, const uint32_t* lens, uint32_t len_c, uint64_t vocab,
                                    uint64_t seed, uint64_t* off_out, uint16_t* sym_out, uint64_t sym_capacity)
{
    if(!off_out || !lens || len_c == 0 || (kind != 0 && kind != 1)) return CSA_E_INVALID;
    if(kind == 0 && (!text_host || n == 0)) return CSA_E_INVALID;
    if(kind == 1 && vocab == 0) return CSA_E_INVALID;
    std::mt19937_64 rng(seed);
    off_out[0] = 0;
    if(kind == 0)
    {
        // The places first, as the seed draws them; then the symbols.
        std::vector<uint64_t> pos(q);
        for(uint64_t i = 0; i < q; ++i)
        {
            uint64_t len = lens[rng() % len_c];
            if(len > n) len = n;
            pos[i] = rng() % (n - len + 1);
            off_out[i + 1] = off_out[i] + len;
        }
        if(off_out[q] > sym_capacity) return CSA_E_NOMEM;
        #pragma omp parallel for schedule(static)
        for(uint64_t i = 0; i < q; ++i)
            std::memcpy(sym_out + off_out[i], text_host + pos[i], (off_out[i + 1] - off_out[i]) * 2);
    }
    else
    {
        uint64_t at = 0;
        for(uint64_t i = 0; i < q; ++i)
        {
            const uint64_t len = lens[rng() % len_c];
            if(at + len > sym_capacity) return CSA_E_NOMEM;
            for(uint64_t j = 0; j < len; ++j) sym_out[at++] = static_cast<uint16_t>(rng() % vocab);
            off_out[i + 1] = at;
        }
    }
    return CSA_OK;
}

extern "C" uint64_t csa_counts_hash(const uint64_t* itv, uint64_t q)
{
    uint64_t h = 0xcbf29ce484222325ull;
    for(uint64_t i = 0; i < q; ++i)
    {
        const uint64_t c = itv[2 * i + 1] - itv[2 * i];
        for(int b = 0; b < 8; ++b) { h ^= (c >> (8 * b)) & 0xFF; h *= 0x100000001b3ull; }
    }
    return h;
}
