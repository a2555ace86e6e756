// Host-side helpers of the drop-in surface that need no GPU: the query-batch generator with the semantics of the
// reference's `query gen` (src/query.cu:826-882: std::mt19937_64(seed), lengths drawn as lens[rng() % |lens|],
// substring places as rng() % (n - len + 1), random symbols as rng() % vocab) and the FNV-1a hash of the counts
// (include/query-file.hpp:228-263).
#include "common.cuh"

#include <algorithm>
#include <random>
#include <string>
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

// ---- where an index goes: the planner of the query engine ---------------------------------------------------------------------
// The reference's planner (Query_Engine::plan and ::fit, src/Query_Engine.cu:822-1006) tries its plans in order and keeps the
// first that fits the budgets less their margins (a sixteenth of a budget, at least 1 GiB, :40-41, :941-942), choosing the
// finest table stride from 32 to 4096 that the device still holds (:38-39, :750-763). Of its four plans two search on the host
// (C: text and suffix array in pageable memory; D: suffix array mapped from its files); this engine searches on the device
// only, so its planner offers the other two: A, text and suffix array in device memory, and B, text in device memory with the
// suffix array in pinned host memory (the brackets' entries are gathered over PCIe). A request for a tier that only C or D
// would serve is answered with "nothing fits" and the reason.
namespace
{

constexpr uint64_t PLAN_STRIDE_MIN = 32, PLAN_STRIDE_MAX = 4096, PLAN_MARGIN_PARTS = 16, PLAN_MARGIN_MIN = uint64_t(1) << 30;
constexpr uint64_t PLAN_CHUNK_QUERIES = uint64_t(1) << 18, PLAN_CHUNK_SYMBOLS = uint64_t(1) << 24;     // a lane's chunk of a host batch
constexpr uint64_t PLAN_GATHER_STRIDE_MAX = 64;      // beyond it a bracket is wider than a gathered window and is searched in place across the bus
constexpr uint32_t PLAN_LANES = 3, PLAN_LOCATE = 100;

uint64_t plan_lane_device_bytes()
{
    // a lane of csa_query_host: offsets, symbols, intervals, counts, position offsets and up to PLAN_LOCATE positions per query
    return PLAN_LANES * ((PLAN_CHUNK_QUERIES + 1) * 8 + PLAN_CHUNK_SYMBOLS * 2 + PLAN_CHUNK_QUERIES * (16 + 4 + 8 + uint64_t(PLAN_LOCATE) * 8));
}

void plan_say(csa_query_placement* p, const std::string& why)
{
    std::snprintf(p->why, sizeof(p->why), "%s", why.c_str());
}

std::string plan_gb(uint64_t bytes)
{
    char b[32];
    std::snprintf(b, sizeof(b), "%.2f GB", double(bytes) / 1e9);
    return b;
}

}   // namespace

extern "C" int csa_query_plan(uint64_t n, uint64_t device_budget, uint64_t host_budget, uint64_t stride, int sa_tier, csa_query_placement* out)
{
    if(!out || n == 0 || sa_tier < 0 || sa_tier > 2) return CSA_E_INVALID;
    std::memset(out, 0, sizeof(*out));
    out->device_budget = device_budget; out->host_budget = host_budget;
    out->device_margin = std::max(PLAN_MARGIN_MIN, device_budget / PLAN_MARGIN_PARTS);
    out->host_margin = std::max(PLAN_MARGIN_MIN, host_budget / PLAN_MARGIN_PARTS);
    out->chunk_queries = PLAN_CHUNK_QUERIES; out->chunk_symbols = PLAN_CHUNK_SYMBOLS; out->key_words = 2;
    const uint64_t cap = device_budget > out->device_margin ? device_budget - out->device_margin : 0;
    const uint64_t text_bytes = (n + CSA_TEXT_PAD) * 2, sa_bytes = 5 * n + CSA_SA_PAD_BYTES;
    std::string why;
    for(int plan = 0; plan < 2; ++plan)        // A, then B
    {
        const bool sa_on_device = plan == 0;
        if((sa_tier == 1 && !sa_on_device) || (sa_tier == 2 && sa_on_device)) continue;
        const char name = sa_on_device ? 'A' : 'B';
        uint64_t dev = text_bytes + (sa_on_device ? sa_bytes : 0) + plan_lane_device_bytes();
        const uint64_t host = sa_on_device ? 0 : sa_bytes;
        if(!sa_on_device) dev += 2 * (uint64_t(1) << 20) * 352 + (uint64_t(1) << 20) * 64;       // gathered windows and brackets of a search batch
        const uint64_t room = cap > dev ? cap - dev : 0;
        uint64_t s = stride;
        if(s == 0)
        {
            const uint64_t last = sa_on_device ? PLAN_STRIDE_MAX : PLAN_GATHER_STRIDE_MAX;
            for(uint64_t t = PLAN_STRIDE_MIN; t <= last && s == 0; t *= 2) if(div_up(n, t) * 16 <= room) s = t;
            if(s == 0)
            {
                why += std::string(why.empty() ? "" : "; ") + name + " takes " + plan_gb(dev) + " of device memory without a table, which leaves " + plan_gb(room) +
                       " of the budget less its margin: too little for a table of stride " + std::to_string(PLAN_STRIDE_MIN) + " to " + std::to_string(last);
                continue;
            }
        }
        const uint64_t table = div_up(n, s) * 16;
        if(dev + table > cap)
        {
            why += std::string(why.empty() ? "" : "; ") + name + " takes " + plan_gb(dev + table) + " of device memory, past the budget of " + plan_gb(device_budget) + " less its margin";
            continue;
        }
        if(host + out->host_margin > host_budget && host > 0)
        {
            why += std::string(why.empty() ? "" : "; ") + name + " takes " + plan_gb(host) + " of pinned host memory, past the budget of " + plan_gb(host_budget) + " less its margin";
            continue;
        }
        out->plan = uint32_t(name);
        out->stride = s; out->table_bytes = table; out->device_bytes = dev + table; out->host_bytes = host;
        return CSA_OK;
    }
    if(why.empty()) why = "no plan of this engine keeps the suffix array in the tier asked for";
    plan_say(out, "no plan fits: " + why + " (plans that search on the host are not part of this engine)");
    return CSA_OK;
}
