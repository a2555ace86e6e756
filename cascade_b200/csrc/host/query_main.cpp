// `query info | plan | find | gen`: the query engine's command line with the reference's flags and key=value output
// (src/query.cu:43-112, 536-541) for the part this engine implements: search on the device, text in device memory, suffix
// array in device or pinned host memory as the planner (csa_query_plan) or --sa-res places it, a sample table of packed
// K-grams, count and (an extension) locate. The reference's host-search tiers (--text-res/--sa-res pageable, mapped) are
// refused with the reason; flags that only shape its host search are read and listed as `not_applicable=` lines.
#include "../../../include/cascade_b200.h"
#include "formats.hpp"

#include <cuda_runtime.h>

#include <algorithm>
#include <chrono>
#include <cinttypes>
#include <cstdlib>
#include <map>
#include <random>

using namespace cascade_host;

namespace
{

const char* const USAGE =
    "Usage:\n"
    "  query info --index DIR\n"
    "  query plan --index DIR [--stride S|auto] [--sa-res device|pinned|auto] [--device-budget BYTES] [--host-budget BYTES]\n"
    "  query find --index DIR --queries Q1.qry[,Q2.qry,...] [--q N] [--stride S|auto] [--sa-res device|pinned|auto] [--reps K] [--locate M]\n"
    "             [--itv-out F] [--cnt-out F] [--pos-out F] [--cnt-dir D] [--validate] [--device D] [--device-budget BYTES] [--host-budget BYTES]\n"
    "  query gen --index DIR --out Q.qry --kind substring|mutated|random|unigram [--q N --len L1[,L2,...]] [--source F] [--vocab V] [--seed S]\n";

struct Args
{
    std::string cmd;
    std::map<std::string, std::string> opt;
    bool has(const std::string& k) const { return opt.count(k) > 0; }
    std::string get(const std::string& k, const std::string& d = "") const { return has(k) ? opt.at(k) : d; }
    uint64_t u64(const std::string& k, uint64_t d) const { return has(k) ? std::strtoull(opt.at(k).c_str(), nullptr, 10) : d; }
};

bool parse(int argc, char** argv, Args& a)
{
    if(argc < 2) return false;
    a.cmd = argv[1];
    for(int i = 2; i < argc; ++i)
    {
        std::string k = argv[i];
        if(k.rfind("--", 0) != 0) return false;
        k = k.substr(2);
        if(k == "validate") { a.opt[k] = "1"; continue; }
        if(i + 1 >= argc) return false;
        a.opt[k] = argv[++i];
    }
    return true;
}

std::vector<std::string> split(const std::string& s, char c)
{
    std::vector<std::string> out;
    std::stringstream ss(s);
    for(std::string t; std::getline(ss, t, c); ) if(!t.empty()) out.push_back(t);
    return out;
}

std::string stem(const std::string& p)
{
    const auto s = p.find_last_of('/');
    std::string b = s == std::string::npos ? p : p.substr(s + 1);
    const auto d = b.find_last_of('.');
    return d == std::string::npos ? b : b.substr(0, d);
}

#define CK(call) do { const int r_ = (call); if(r_ != CSA_OK) { std::fprintf(stderr, "error: %s failed (%d): %s\n", #call, r_, csa_last_error(ctx)); return 1; } } while(0)
#define CU(call) do { const cudaError_t e_ = (call); if(e_ != cudaSuccess) { std::fprintf(stderr, "error: %s: %s\n", #call, cudaGetErrorString(e_)); return 1; } } while(0)

uint64_t available_host_bytes()
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

// The placement of the index for the options given: budgets as set or else measured, the suffix array's tier as named or
// else the planner's choice, the stride as given or else the finest that fits (`--stride auto`, the default of `plan`).
bool place(const Args& a, uint64_t n, uint64_t stride_default, csa_query_placement& pl, std::string& err)
{
    for(const char* k : {"stride", "sa-res", "text-res"})
        if(a.get(k).find(',') != std::string::npos) { err = std::string("--") + k + " takes one value here, not a list"; return false; }
    const std::string sa_res = a.get("sa-res", "auto"), text_res = a.get("text-res", "auto");
    if(text_res != "auto" && text_res != "device") { err = "--text-res " + text_res + ": this engine searches on the device and keeps the text there (device, auto)"; return false; }
    int tier = 0;
    if(sa_res == "device") tier = 1;
    else if(sa_res == "pinned") tier = 2;
    else if(sa_res != "auto") { err = "--sa-res " + sa_res + ": this engine searches on the device; the suffix array is in device or pinned memory (device, pinned, auto)"; return false; }
    uint64_t dev_budget = a.u64("device-budget", 0), host_budget = a.u64("host-budget", 0);
    if(dev_budget == 0)
    {
        size_t free_b = 0, total_b = 0;
        if(cudaMemGetInfo(&free_b, &total_b) != cudaSuccess) { cudaGetLastError(); err = "cannot measure the device's free memory; set --device-budget"; return false; }
        dev_budget = free_b;
    }
    if(host_budget == 0) host_budget = available_host_bytes();
    const std::string st = a.get("stride", stride_default ? std::to_string(stride_default) : "auto");
    const uint64_t stride = st == "auto" ? 0 : std::strtoull(st.c_str(), nullptr, 10);
    if(st != "auto" && stride == 0) { err = "--stride must be a positive number or auto"; return false; }
    if(csa_query_plan(n, dev_budget, host_budget, stride, tier, &pl) != CSA_OK) { err = "the planner refused its arguments"; return false; }
    if(pl.plan == 0) { err = pl.why; return false; }
    return true;
}

void print_placement(const csa_query_placement& pl)
{
    std::printf("plan=%c\ntext_res=device\nsa_res=%s\nstride=%" PRIu64 "\nkey_words=%u\ntable_bytes=%" PRIu64 "\ndevice_bytes=%" PRIu64 "\nhost_bytes=%" PRIu64
                "\ndevice_budget=%" PRIu64 "\nhost_budget=%" PRIu64 "\nchunk_queries=%" PRIu64 "\nchunk_symbols=%" PRIu64 "\nlanes=3\n",
                char(pl.plan), pl.plan == 'A' ? "device" : "pinned", pl.stride, pl.key_words, pl.table_bytes, pl.device_bytes, pl.host_bytes, pl.device_budget,
                pl.host_budget, pl.chunk_queries, pl.chunk_symbols);
}

int run_info(const Args& a, bool plan)
{
    Index_Meta m; std::string err;
    if(!read_index_meta(a.get("index"), m, err)) { std::fprintf(stderr, "error: %s\n", err.c_str()); return 1; }
    std::printf("n=%" PRIu64 "\nsym_bytes=%u\nsa_width=%u\nsa_order=%s\ntext=%s\nsa_part_c=%zu\nsep=%lld\n", m.n, m.sym_bytes, m.sa_width, m.sa_order.c_str(),
                m.text.c_str(), m.sa_part.size(), m.sep);
    if(!plan) return 0;
    csa_query_placement pl;
    if(!place(a, m.n, 0, pl, err)) { std::printf("plan=none\nwhy=%s\n", err.c_str()); return 1; }
    print_placement(pl);
    return 0;
}

int run_gen(const Args& a)
{
    Index_Meta m; std::string err;
    if(!read_index_meta(a.get("index"), m, err)) { std::fprintf(stderr, "error: %s\n", err.c_str()); return 1; }
    // The reference's four kinds (src/query.cu:108-111): substrings of the text, substrings with one symbol replaced by another
    // one ("mutated"), random symbols below the vocabulary, and every symbol of the vocabulary once ("unigram").
    const std::string kind = a.get("kind", "substring");
    if(kind != "substring" && kind != "random" && kind != "mutated" && kind != "unigram")
    {
        std::fprintf(stderr, "error: --kind %s is not one of substring, mutated, random, unigram\n", kind.c_str());
        return 1;
    }
    uint64_t q = a.u64("q", 1000);
    const uint64_t seed = a.u64("seed", 1), vocab = a.u64("vocab", 65536);
    if(vocab == 0 || vocab > 65536) { std::fprintf(stderr, "error: --vocab must be between 1 and 65536\n"); return 1; }
    std::vector<uint32_t> lens;
    for(const auto& t : split(a.get("len", "8"), ',')) lens.push_back(uint32_t(std::strtoul(t.c_str(), nullptr, 10)));
    const bool from_text = kind == "substring" || kind == "mutated";
    std::vector<uint16_t> T;
    uint64_t n = 0;
    if(from_text)
    {
        const std::string src = a.get("source", m.text);
        uint64_t bytes = 0;
        if(!file_size(src, bytes) || bytes == 0 || bytes % 2) { std::fprintf(stderr, "error: cannot use %s as a text of 2-byte symbols\n", src.c_str()); return 1; }
        n = bytes / 2; T.resize(n);
        if(!read_file(src, T.data(), bytes, err)) { std::fprintf(stderr, "error: %s\n", err.c_str()); return 1; }
    }
    std::vector<uint64_t> off;
    std::vector<uint16_t> sym;
    if(kind == "unigram")
    {
        q = vocab;
        off.resize(q + 1);
        sym.resize(q + 1);
        for(uint64_t c = 0; c < q; ++c) { off[c] = c; sym[c] = uint16_t(c); }
        off[q] = q;
    }
    else
    {
        const uint64_t cap = q * uint64_t(*std::max_element(lens.begin(), lens.end())) + 1;
        off.resize(q + 1);
        sym.resize(cap);
        const int rc = csa_gen_queries_host(from_text ? 0 : 1, T.data(), n, q, lens.data(), uint32_t(lens.size()), vocab, seed, off.data(), sym.data(), cap);
        if(rc != CSA_OK) { std::fprintf(stderr, "error: query generation failed (%d)\n", rc); return 1; }
        if(kind == "mutated" && vocab > 1)
        {
            std::mt19937_64 rng(seed ^ 0x6D75746174656421ull);
            for(uint64_t i = 0; i < q; ++i)
            {
                const uint64_t len = off[i + 1] - off[i];
                if(len == 0) continue;
                uint16_t& x = sym[off[i] + rng() % len];
                const uint16_t old = x;
                do x = uint16_t(rng() % vocab); while(x == old);
            }
        }
    }
    if(!write_qry(a.get("out"), off, sym.data(), seed, err)) { std::fprintf(stderr, "error: %s\n", err.c_str()); return 1; }
    std::printf("out=%s\nq=%" PRIu64 "\nsym_c=%" PRIu64 "\nkind=%s\nvocab=%" PRIu64 "\nseed=%" PRIu64 "\n", a.get("out").c_str(), q, off[q], kind.c_str(), vocab, seed);
    return 0;
}

int run_find(const Args& a)
{
    // flags of the reference that shape its host search or its own pipeline: read, named on stdout, without effect here
    for(const char* k : {"key-words", "sort", "gather", "gather-queries", "chunk-queries", "chunk-symbols", "host-threads", "host-lanes", "host-prefetch", "sa-cold",
                         "phase-times", "spot"})
        if(a.has(k)) std::printf("not_applicable=--%s\n", k);
    Index_Meta m; std::string err;
    if(!read_index_meta(a.get("index"), m, err)) { std::fprintf(stderr, "error: %s\n", err.c_str()); return 1; }
    const uint64_t n = m.n, reps = std::max<uint64_t>(1, a.u64("reps", 3));
    const uint32_t max_pos = uint32_t(a.u64("locate", 0));
    const int device = int(a.u64("device", 0));
    CU(cudaSetDevice(device));
    csa_query_placement pl;
    if(!place(a, n, 32, pl, err)) { std::fprintf(stderr, "error: %s\n", err.c_str()); return 1; }
    const uint64_t stride = pl.stride;
    const bool sa_pinned = pl.plan == 'B';
    csa_ctx* ctx = nullptr;
    if(csa_ctx_create(device, &ctx) != CSA_OK) { std::fprintf(stderr, "error: cannot create a device context\n"); return 1; }

    const auto t0 = std::chrono::steady_clock::now();
    const auto since = [&] { return std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count(); };
    std::vector<uint16_t> T(n + CSA_TEXT_PAD, 0);
    std::vector<uint8_t> SA(5 * n + CSA_SA_PAD_BYTES, 0);
    if(!read_file(m.text, T.data(), 2 * n, err)) { std::fprintf(stderr, "error: %s\n", err.c_str()); return 1; }
    // Part i holds the bytes [sa_part_off[i], sa_part_off[i + 1]) of the array's byte stream, from the start of its file.
    uint64_t at = 0;
    for(size_t i = 0; i < m.sa_part.size(); ++i)
    {
        const uint64_t begin = m.sa_part_off[i], end = (i + 1 < m.sa_part.size() ? m.sa_part_off[i + 1] : 5 * n);
        uint64_t b = 0;
        if(!file_size(m.sa_part[i], b)) { std::fprintf(stderr, "error: cannot open %s\n", m.sa_part[i].c_str()); return 1; }
        if(begin != at || end < begin || end > 5 * n || b != end - begin)
        {
            std::fprintf(stderr, "error: suffix-array part %s has %" PRIu64 " bytes; expected %" PRIu64 "\n", m.sa_part[i].c_str(), b, end - begin);
            return 1;
        }
        FILE* f = std::fopen(m.sa_part[i].c_str(), "rb");
        if(!f || std::fread(SA.data() + at, 1, b, f) != b) { std::fprintf(stderr, "error: cannot read %s\n", m.sa_part[i].c_str()); return 1; }
        std::fclose(f);
        at += b;
    }
    if(at != 5 * n) { std::fprintf(stderr, "error: the suffix-array parts hold %" PRIu64 " bytes, expected %" PRIu64 "\n", at, 5 * n); return 1; }
    uint16_t* T_d = nullptr; uint8_t* SA_d = nullptr; uint64_t* tab_d = nullptr;
    const uint64_t entries = (n + stride - 1) / stride;
    CU(cudaMalloc(&T_d, T.size() * 2)); CU(cudaMalloc(&tab_d, entries * 16));
    if(sa_pinned) CU(cudaMallocHost(&SA_d, SA.size()));        // plan B: the device reads the array across the bus
    else CU(cudaMalloc(&SA_d, SA.size()));
    CU(cudaMemcpy(T_d, T.data(), T.size() * 2, cudaMemcpyHostToDevice));
    CU(cudaMemcpy(SA_d, SA.data(), SA.size(), sa_pinned ? cudaMemcpyHostToHost : cudaMemcpyHostToDevice));
    CK(csa_table_build(ctx, T_d, n, SA_d, stride, tab_d));
    CK(csa_sync(ctx, nullptr));
    const csa_index idx{T_d, SA_d, tab_d, n, stride};
    std::printf("n=%" PRIu64 "\n", n);
    print_placement(pl);
    std::printf("load_s=%.6f\n", since());

    for(const auto& qpath : split(a.get("queries"), ','))
    {
        std::vector<uint64_t> off; std::vector<uint16_t> sym;
        if(!read_qry(qpath, a.u64("q", UINT64_MAX), off, sym, err)) { std::fprintf(stderr, "error: %s\n", err.c_str()); return 1; }
        const uint64_t q = off.size() - 1;
        std::vector<uint64_t> itv(2 * q), pos_off(q + 1), pos(max_pos ? q * uint64_t(max_pos) : 1);
        std::vector<uint32_t> cnt(q);
        uint64_t total = 0;
        // from device memory: the batch resident on the device, CUDA-event time of the search alone
        uint64_t* off_d = nullptr; uint16_t* sym_d = nullptr; uint64_t* itv_d = nullptr; uint64_t* res_d = nullptr;
        CU(cudaMalloc(&off_d, (q + 1) * 8)); CU(cudaMalloc(&sym_d, sym.size() * 2 + 16)); CU(cudaMalloc(&itv_d, 2 * q * 8 + 16)); CU(cudaMalloc(&res_d, 16));
        CU(cudaMemcpy(off_d, off.data(), (q + 1) * 8, cudaMemcpyHostToDevice));
        CU(cudaMemcpy(sym_d, sym.data(), sym.size() * 2, cudaMemcpyHostToDevice));
        std::vector<double> dev_s, e2e_s;
        cudaEvent_t e0, e1; CU(cudaEventCreate(&e0)); CU(cudaEventCreate(&e1));
        cudaStream_t st = static_cast<cudaStream_t>(csa_ctx_stream(ctx));
        for(uint64_t r = 0; r < reps; ++r)
        {
            CU(cudaEventRecord(e0, st));
            CK(csa_find(ctx, &idx, off_d, sym_d, q, itv_d));
            CU(cudaEventRecord(e1, st));
            CK(csa_sync(ctx, nullptr));
            float ms = 0; CU(cudaEventElapsedTime(&ms, e0, e1));
            dev_s.push_back(ms * 1e-3);
        }
        for(uint64_t r = 0; r < reps; ++r)
        {
            const auto b = std::chrono::steady_clock::now();
            CK(csa_query_host(ctx, &idx, off.data(), sym.data(), q, max_pos, itv.data(), cnt.data(), pos_off.data(), pos.data(), pos.size(), &total));
            e2e_s.push_back(std::chrono::duration<double>(std::chrono::steady_clock::now() - b).count());
        }
        std::sort(dev_s.begin(), dev_s.end()); std::sort(e2e_s.begin(), e2e_s.end());
        uint64_t fails = 0, first = ~0ull;
        if(a.has("validate"))
        {
            CU(cudaMemcpy(itv_d, itv.data(), 2 * q * 8, cudaMemcpyHostToDevice));
            CK(csa_certify(ctx, &idx, off_d, sym_d, q, itv_d, res_d));
            CK(csa_sync(ctx, nullptr));
            uint64_t res[2]; CU(cudaMemcpy(res, res_d, 16, cudaMemcpyDeviceToHost));
            fails = res[0]; first = res[1];
        }
        std::printf("queries=%s\nq=%" PRIu64 "\nsym_c=%" PRIu64 "\nreps=%" PRIu64 "\ndevice_search_s_min=%.6f\ndevice_search_s_median=%.6f\n"
                    "end_to_end_s_min=%.6f\nend_to_end_s_median=%.6f\nqps=%.1f\nqps_end_to_end=%.1f\ncounts_hash=%016" PRIx64 "\n",
                    qpath.c_str(), q, off[q], reps, dev_s.front(), dev_s[dev_s.size() / 2], e2e_s.front(), e2e_s[e2e_s.size() / 2], double(q) / dev_s.front(),
                    double(q) / e2e_s.front(), csa_counts_hash(itv.data(), q));
        if(max_pos) std::printf("locate_max=%u\npositions=%" PRIu64 "\n", max_pos, total);
        if(a.has("validate")) std::printf("validate=%s\nvalidate_failures=%" PRIu64 "\n", fails ? "FAIL" : "ok", fails);
        if(fails) { std::fprintf(stderr, "error: interval certificate failed for query %" PRIu64 "\n", first); return 1; }
        std::string itv_out = a.get("itv-out"), cnt_out = a.get("cnt-out"), pos_out = a.get("pos-out");
        if(a.has("cnt-dir")) cnt_out = a.get("cnt-dir") + "/" + stem(qpath) + ".cnt";
        if(!itv_out.empty() && !write_file(itv_out, itv.data(), 2 * q * 8, err)) { std::fprintf(stderr, "error: %s\n", err.c_str()); return 1; }
        if(!cnt_out.empty())
        {
            std::vector<uint64_t> c(q);
            for(uint64_t i = 0; i < q; ++i) c[i] = itv[2 * i + 1] - itv[2 * i];
            if(!write_file(cnt_out, c.data(), q * 8, err)) { std::fprintf(stderr, "error: %s\n", err.c_str()); return 1; }
        }
        if(!pos_out.empty() && max_pos)
        {
            std::vector<uint64_t> blob; blob.reserve(2 + q + 1 + total);
            blob.push_back(q); blob.push_back(total);
            blob.insert(blob.end(), pos_off.begin(), pos_off.end());
            blob.insert(blob.end(), pos.begin(), pos.begin() + total);
            if(!write_file(pos_out, blob.data(), blob.size() * 8, err)) { std::fprintf(stderr, "error: %s\n", err.c_str()); return 1; }
        }
        cudaFree(off_d); cudaFree(sym_d); cudaFree(itv_d); cudaFree(res_d);
        cudaEventDestroy(e0); cudaEventDestroy(e1);
    }
    csa_ctx_destroy(ctx);
    cudaFree(T_d); cudaFree(tab_d);
    if(sa_pinned) cudaFreeHost(SA_d); else cudaFree(SA_d);
    return 0;
}

}   // namespace

int main(int argc, char** argv)
{
    Args a;
    if(!parse(argc, argv, a) || !a.has("index")) { std::fputs(USAGE, stderr); return 1; }
    if(a.cmd == "info") return run_info(a, false);
    if(a.cmd == "plan") return run_info(a, true);
    if(a.cmd == "gen") return a.has("out") ? run_gen(a) : (std::fputs(USAGE, stderr), 1);
    if(a.cmd == "find") return a.has("queries") ? run_find(a) : (std::fputs(USAGE, stderr), 1);
    std::fputs(USAGE, stderr);
    return 1;
}
