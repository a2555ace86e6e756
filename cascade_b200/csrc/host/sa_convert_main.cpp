// sa_convert: the tool that prepares a query index from a finished suffix array, with the command line of the
// reference's tools/sa_convert.cpp:38-58:
//   sa_convert --in SA.u64 --text TEXT --sym-bytes {1,2,4} --index-dir DIR [--parts K --part-dirs D0:D1:...]
//              [--check none|range|perm] [--spot N] [--sep S] [--source STR]      64-bit entries -> 5-byte parts + index.meta
//   sa_convert --meta-only --sa SA.u40 --text TEXT --sym-bytes B --index-dir DIR [--spot N] [--sep S] [--source STR]
//   sa_convert --widen --in SA.u40 --out SA.u64
// Host code only: file formats on either side of the device path (index.meta: include/Index_Meta.hpp:207-241; part
// offsets cut at 4096-byte pages, :76-86; order spot check: include/CPU_Reference.hpp:133-168).
#include "formats.hpp"

#include <chrono>
#include <cinttypes>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <string>
#include <vector>

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

using namespace cascade_host;

namespace
{

constexpr uint64_t ENTRY = 5, PAGE = 4096, MAX_N = 1ull << 40;

enum class Mode { convert, meta_only, widen };

struct Args
{
    Mode mode = Mode::convert;
    std::string in, out, sa, text, index_dir, source, check = "perm";
    std::vector<std::string> part_dirs;
    uint32_t sym_bytes = 0;
    uint64_t parts = 1, spot = 100000;
    long long sep = -1;
};

const char* USAGE =
    "usage:\n"
    "  sa_convert --in SA.u64 --text TEXT --sym-bytes {1,2,4} --index-dir DIR\n"
    "             [--parts K --part-dirs D0:D1:...] [--check none|range|perm]\n"
    "             [--spot N] [--sep S] [--source STR]\n"
    "  sa_convert --meta-only --sa SA.u40 --text TEXT --sym-bytes B --index-dir DIR\n"
    "             [--spot N] [--sep S] [--source STR]\n"
    "  sa_convert --widen --in SA.u40 --out SA.u64\n";

std::vector<std::string> split(const std::string& v, char at)
{
    std::vector<std::string> out(1);
    for(const char c : v) { if(c == at) out.emplace_back(); else out.back().push_back(c); }
    return out;
}

// One row per option: its name, whether a value follows, and what to do with it. The flags are the reference tool's
// (tools/sa_convert.cpp:38-58); how they are read is this file's own.
struct Option
{
    const char* name;
    bool takes_value;
    void (*apply)(Args&, const std::string&);
};

const Option OPTIONS[] = {
    {"--meta-only", false, [](Args& a, const std::string&) { a.mode = Mode::meta_only; }},
    {"--widen", false, [](Args& a, const std::string&) { a.mode = Mode::widen; }},
    {"--in", true, [](Args& a, const std::string& v) { a.in = v; }},
    {"--out", true, [](Args& a, const std::string& v) { a.out = v; }},
    {"--sa", true, [](Args& a, const std::string& v) { a.sa = v; }},
    {"--text", true, [](Args& a, const std::string& v) { a.text = v; }},
    {"--index-dir", true, [](Args& a, const std::string& v) { a.index_dir = v; }},
    {"--source", true, [](Args& a, const std::string& v) { a.source = v; }},
    {"--check", true, [](Args& a, const std::string& v) { a.check = v; }},
    {"--part-dirs", true, [](Args& a, const std::string& v) { a.part_dirs = split(v, ':'); }},
    {"--sym-bytes", true, [](Args& a, const std::string& v) { a.sym_bytes = uint32_t(std::stoul(v)); }},
    {"--parts", true, [](Args& a, const std::string& v) { a.parts = std::stoull(v); }},
    {"--spot", true, [](Args& a, const std::string& v) { a.spot = std::stoull(v); }},
    {"--sep", true, [](Args& a, const std::string& v) { a.sep = std::stoll(v); }},
};

// What must hold between the options once all are read; the first rule that fails names the problem.
std::string first_broken_rule(const Args& a)
{
    if(a.mode == Mode::widen) return (a.in.empty() || a.out.empty()) ? "widening needs both --in and --out" : "";
    const bool width_ok = a.sym_bytes == 1 || a.sym_bytes == 2 || a.sym_bytes == 4;
    const bool check_ok = a.check == "none" || a.check == "range" || a.check == "perm";
    const struct { bool broken; const char* why; } rules[] = {
        {a.text.empty() || a.index_dir.empty() || a.sym_bytes == 0, "give --text, --index-dir and --sym-bytes"},
        {!width_ok, "symbols are 1, 2 or 4 bytes wide (--sym-bytes)"},
        {a.mode == Mode::convert && a.in.empty(), "a conversion reads its 64-bit entries from --in"},
        {a.mode == Mode::meta_only && a.sa.empty(), "--meta-only describes the 5-byte array given by --sa"},
        {a.parts == 0, "--parts counts from 1"},
        {a.parts > 1 && a.part_dirs.size() != a.parts, "--part-dirs must list one directory per part"},
        {a.parts > 1 && a.mode != Mode::convert, "only a conversion can cut the array into parts"},
        {!check_ok, "--check is one of none, range, perm"},
    };
    for(const auto& r : rules) if(r.broken) return r.why;
    return "";
}

bool parse(int argc, char** argv, Args& a, std::string& err)
{
    for(int i = 1; i < argc; ++i)
    {
        const std::string key = argv[i];
        if(key == "-h" || key == "--help") { err.clear(); return false; }
        const Option* opt = nullptr;
        for(const Option& o : OPTIONS) if(key == o.name) opt = &o;
        if(!opt) { err = "unknown option " + key; return false; }
        std::string value;
        if(opt->takes_value)
        {
            if(i + 1 >= argc) { err = key + " needs a value"; return false; }
            value = argv[++i];
        }
        try { opt->apply(a, value); }
        catch(const std::exception&) { err = "cannot read the value of " + key + ": " + value; return false; }
    }
    err = first_broken_rule(a);
    return err.empty();
}

std::string absolute(const std::string& p)
{
    if(!p.empty() && p[0] == '/') return p;
    char cwd[4096];
    if(!::getcwd(cwd, sizeof(cwd))) return p;
    return std::string(cwd) + "/" + p;
}

bool make_dirs(const std::string& dir)
{
    std::string cur;
    for(size_t i = 0; i <= dir.size(); ++i)
    {
        if(i == dir.size() || dir[i] == '/')
        {
            if(!cur.empty() && ::mkdir(cur.c_str(), 0777) != 0 && errno != EEXIST) return false;
        }
        if(i < dir.size()) cur.push_back(dir[i]);
    }
    return true;
}

// A whole file mapped for reading; empty files and files that cannot be opened give a null view.
class Mapping
{
    const uint8_t* base_ = nullptr;
public:
    size_t len = 0;
    Mapping() = default;
    Mapping(const Mapping&) = delete;
    Mapping& operator=(const Mapping&) = delete;
    ~Mapping() { if(base_) ::munmap(const_cast<uint8_t*>(base_), len); }
    bool map(const std::string& path)
    {
        uint64_t bytes = 0;
        if(!file_size(path, bytes) || bytes == 0) return false;
        const int fd = ::open(path.c_str(), O_RDONLY | O_CLOEXEC);
        if(fd < 0) return false;
        void* const at = ::mmap(nullptr, size_t(bytes), PROT_READ, MAP_PRIVATE, fd, 0);
        ::close(fd);
        if(at == MAP_FAILED) return false;
        base_ = static_cast<const uint8_t*>(at);
        len = size_t(bytes);
        return true;
    }
    const uint8_t* data() const { return base_; }
};

uint64_t text_length(const std::string& path, uint32_t sym_bytes, std::string& err)
{
    uint64_t bytes = 0;
    if(!file_size(path, bytes)) { err = "cannot stat text: " + path; return 0; }
    if(bytes == 0 || bytes % sym_bytes != 0) { err = "text size is not a positive multiple of the symbol width: " + path; return 0; }
    if(bytes / sym_bytes >= MAX_N) { err = "text too long for 40-bit suffix-array entries"; return 0; }
    return bytes / sym_bytes;
}

// The 5-byte array as a stream of bytes spread over mapped parts; an entry may straddle two parts.
struct Parted
{
    std::vector<const uint8_t*> part;
    std::vector<uint64_t> off;
    uint64_t bytes = 0;
    uint64_t operator()(uint64_t r) const
    {
        uint64_t v = 0;
        size_t i = 0;
        const uint64_t b = ENTRY * r;
        while(i + 1 < off.size() && off[i + 1] <= b) ++i;
        for(uint64_t k = 0; k < ENTRY; ++k)
        {
            const uint64_t x = b + k;
            while(i + 1 < off.size() && x >= off[i + 1]) ++i;
            v |= uint64_t(part[i][x - off[i]]) << (8 * k);
        }
        return v;
    }
};

template <typename S>
int compare_suffixes(const S* T, uint64_t n, uint64_t i, uint64_t j, uint64_t max_cmp)
{
    const uint64_t li = n - i, lj = n - j, len = li < lj ? li : lj, lim = len < max_cmp ? len : max_cmp;
    for(uint64_t k = 0; k < lim; ++k)
        if(T[i + k] != T[j + k]) return T[i + k] < T[j + k] ? -1 : 1;
    if(lim == max_cmp && len > max_cmp) return 0;       // undecided within the budget: counts as consistent
    return li < lj ? -1 : 1;
}

// The first, the last and `samples` random adjacent pairs must be in numeric order, shorter suffix first.
template <typename S>
bool spot_check(const S* T, uint64_t n, const Parted& sa, uint64_t samples, std::string& err)
{
    if(n < 2) return true;
    const bool all = samples >= n - 1;
    const uint64_t checks = all ? n - 1 : samples + 2;
    std::mt19937_64 rng(0x5EED);
    std::uniform_int_distribution<uint64_t> dist(0, n - 2);
    for(uint64_t k = 0; k < checks; ++k)
    {
        const uint64_t r = all ? k : (k == 0 ? 0 : (k == 1 ? n - 2 : dist(rng)));
        const uint64_t i = sa(r), j = sa(r + 1);
        if(i >= n || j >= n) { err = "suffix-array entry out of range at rank " + std::to_string(i >= n ? r : r + 1); return false; }
        if(i == j) { err = "suffix-array entry " + std::to_string(i) + " repeats at ranks " + std::to_string(r) + " and " + std::to_string(r + 1); return false; }
        if(compare_suffixes(T, n, i, j, 1000) > 0)
        {
            err = "suffix-array order violated between ranks " + std::to_string(r) + " and " + std::to_string(r + 1) + " (suffixes " + std::to_string(i) + ", "
                + std::to_string(j) + "); expected numeric order with shorter suffixes first";
            return false;
        }
    }
    return true;
}

bool spot_check(uint32_t sym_bytes, const std::string& text_path, uint64_t n, const Parted& sa, uint64_t samples, std::string& err)
{
    Mapping text;
    if(!text.map(text_path)) { err = "cannot map text: " + text_path; return false; }
    switch(sym_bytes)
    {
    case 1: return spot_check(reinterpret_cast<const uint8_t*>(text.data()), n, sa, samples, err);
    case 2: return spot_check(reinterpret_cast<const uint16_t*>(text.data()), n, sa, samples, err);
    default: return spot_check(reinterpret_cast<const uint32_t*>(text.data()), n, sa, samples, err);
    }
}

bool map_parts(const Index_Meta& m, std::vector<Mapping>& maps, Parted& sa, std::string& err)
{
    maps = std::vector<Mapping>(m.sa_part.size());
    sa.part.clear();
    for(size_t i = 0; i < m.sa_part.size(); ++i)
    {
        const uint64_t want = (i + 1 < m.sa_part.size() ? m.sa_part_off[i + 1] : ENTRY * m.n) - m.sa_part_off[i];
        uint64_t have = 0;
        if(!file_size(m.sa_part[i], have)) { err = "cannot stat suffix-array part: " + m.sa_part[i]; return false; }
        if(have != want) { err = "suffix-array part " + m.sa_part[i] + " has " + std::to_string(have) + " bytes; expected " + std::to_string(want); return false; }
        if(want == 0) { sa.part.push_back(nullptr); continue; }
        if(!maps[i].map(m.sa_part[i])) { err = "cannot map suffix-array part: " + m.sa_part[i]; return false; }
        sa.part.push_back(maps[i].data());
    }
    sa.off = m.sa_part_off;
    sa.bytes = ENTRY * m.n;
    return true;
}

double since(std::chrono::steady_clock::time_point t0) { return std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count(); }

int convert(const Args& a)
{
    std::string err;
    const auto t0 = std::chrono::steady_clock::now();
    const uint64_t n = text_length(a.text, a.sym_bytes, err);
    if(n == 0) { std::fprintf(stderr, "%s\n", err.c_str()); return 1; }
    uint64_t in_bytes = 0;
    if(!file_size(a.in, in_bytes) || in_bytes != n * 8)
    {
        std::fprintf(stderr, "input suffix array %s has %" PRIu64 " bytes; expected %" PRIu64 " (n = %" PRIu64 " uint64 entries)\n", a.in.c_str(), in_bytes, n * 8, n);
        return 1;
    }
    make_dirs(a.index_dir);
    Index_Meta m;
    m.n = n; m.sym_bytes = a.sym_bytes; m.text = absolute(a.text); m.sep = a.sep;
    m.sa_source = a.source.empty() ? ("sa_convert from " + absolute(a.in)) : a.source;
    for(uint64_t i = 0; i < a.parts; ++i)
    {
        const uint64_t cut = uint64_t((static_cast<unsigned __int128>(ENTRY * n) * i) / a.parts);
        m.sa_part_off.push_back(cut - cut % PAGE);
        const std::string dir = a.parts == 1 ? a.index_dir : a.part_dirs[i];
        make_dirs(dir);
        m.sa_part.push_back(absolute(dir + "/" + (a.parts == 1 ? std::string("sa.u40") : "sa.u40.part" + std::to_string(i))));
    }

    FILE* in = std::fopen(a.in.c_str(), "rb");
    if(!in) { std::fprintf(stderr, "cannot open %s\n", a.in.c_str()); return 1; }
    std::vector<FILE*> outs;
    for(const auto& p : m.sa_part)
    {
        FILE* f = std::fopen(p.c_str(), "wb");
        if(!f) { std::fprintf(stderr, "cannot create %s\n", p.c_str()); return 1; }
        outs.push_back(f);
    }
    std::vector<uint64_t> seen(a.check == "perm" ? (n + 63) / 64 : 0, 0);
    constexpr uint64_t CHUNK = 1u << 20;
    std::vector<uint64_t> buf(CHUNK);
    std::vector<uint8_t> packed(CHUNK * ENTRY);
    size_t part = 0;
    for(uint64_t r0 = 0; r0 < n; r0 += CHUNK)
    {
        const uint64_t e = std::min(CHUNK, n - r0);
        if(std::fread(buf.data(), 8, e, in) != e) { std::fprintf(stderr, "cannot read %s at rank %" PRIu64 "\n", a.in.c_str(), r0); return 1; }
        for(uint64_t k = 0; k < e; ++k)
        {
            const uint64_t v = buf[k];
            if(a.check != "none" && v >= n) { std::fprintf(stderr, "suffix-array entry out of range [0, n) at rank %" PRIu64 "\n", r0 + k); return 1; }
            if(a.check == "perm")
            {
                if(seen[v >> 6] & (1ull << (v & 63)))
                {
                    std::fprintf(stderr, "suffix array has a duplicate entry in ranks [%" PRIu64 ", %" PRIu64 "); it is not a permutation\n", r0, r0 + e);
                    return 1;
                }
                seen[v >> 6] |= 1ull << (v & 63);
            }
            for(uint64_t b = 0; b < ENTRY; ++b) packed[k * ENTRY + b] = uint8_t(v >> (8 * b));
        }
        // the chunk's bytes [lo, hi) of the stream go to the parts that cover them
        uint64_t lo = ENTRY * r0;
        const uint64_t hi = ENTRY * (r0 + e);
        while(lo < hi)
        {
            while(part + 1 < m.sa_part_off.size() && m.sa_part_off[part + 1] <= lo) ++part;
            const uint64_t part_end = part + 1 < m.sa_part_off.size() ? m.sa_part_off[part + 1] : ENTRY * n;
            const uint64_t upto = std::min(hi, part_end);
            if(std::fwrite(packed.data() + (lo - ENTRY * r0), 1, upto - lo, outs[part]) != upto - lo) { std::fprintf(stderr, "cannot write %s\n", m.sa_part[part].c_str()); return 1; }
            lo = upto;
        }
    }
    std::fclose(in);
    for(FILE* f : outs) if(std::fclose(f) != 0) { std::fprintf(stderr, "cannot flush the suffix-array parts\n"); return 1; }
    if(a.check == "perm") std::fprintf(stderr, "[sa_convert] permutation check passed\n");

    std::vector<Mapping> maps;
    Parted sa;
    if(!map_parts(m, maps, sa, err) || !spot_check(a.sym_bytes, m.text, n, sa, a.spot, err))
    {
        std::fprintf(stderr, "order check failed: %s\n", err.c_str());
        return 1;
    }
    std::fprintf(stderr, "[sa_convert] order spot-check passed (%" PRIu64 " pairs)\n", a.spot);
    if(!write_index_meta(a.index_dir, m, err)) { std::fprintf(stderr, "%s\n", err.c_str()); return 1; }
    std::fprintf(stderr, "[sa_convert] wrote %s/index.meta in %.1fs\n", a.index_dir.c_str(), since(t0));
    return 0;
}

int meta_only(const Args& a)
{
    std::string err;
    const uint64_t n = text_length(a.text, a.sym_bytes, err);
    if(n == 0) { std::fprintf(stderr, "%s\n", err.c_str()); return 1; }
    Index_Meta m;
    m.n = n; m.sym_bytes = a.sym_bytes; m.text = absolute(a.text); m.sep = a.sep;
    m.sa_source = a.source.empty() ? ("native 40-bit suffix array " + absolute(a.sa)) : a.source;
    m.sa_part = {absolute(a.sa)};
    m.sa_part_off = {0};
    std::vector<Mapping> maps;
    Parted sa;
    if(!map_parts(m, maps, sa, err) || !spot_check(a.sym_bytes, m.text, n, sa, a.spot, err)) { std::fprintf(stderr, "%s\n", err.c_str()); return 1; }
    make_dirs(a.index_dir);
    if(!write_index_meta(a.index_dir, m, err)) { std::fprintf(stderr, "%s\n", err.c_str()); return 1; }
    std::fprintf(stderr, "[sa_convert] order spot-check passed; wrote %s/index.meta\n", a.index_dir.c_str());
    return 0;
}

int widen(const Args& a)
{
    uint64_t in_bytes = 0;
    if(!file_size(a.in, in_bytes) || in_bytes % ENTRY != 0) { std::fprintf(stderr, "input is not a 40-bit suffix array: %s\n", a.in.c_str()); return 1; }
    FILE* in = std::fopen(a.in.c_str(), "rb");
    FILE* out = std::fopen(a.out.c_str(), "wb");
    if(!in || !out) { std::fprintf(stderr, "cannot open the input or the output\n"); return 1; }
    constexpr uint64_t CHUNK = 1u << 20;
    std::vector<uint8_t> ib(CHUNK * ENTRY);
    std::vector<uint64_t> ob(CHUNK);
    const uint64_t n = in_bytes / ENTRY;
    for(uint64_t r0 = 0; r0 < n; r0 += CHUNK)
    {
        const uint64_t e = std::min(CHUNK, n - r0);
        if(std::fread(ib.data(), ENTRY, e, in) != e) { std::fprintf(stderr, "read failed\n"); return 1; }
        for(uint64_t k = 0; k < e; ++k)
        {
            uint64_t v = 0;
            for(uint64_t b = 0; b < ENTRY; ++b) v |= uint64_t(ib[k * ENTRY + b]) << (8 * b);
            ob[k] = v;
        }
        if(std::fwrite(ob.data(), 8, e, out) != e) { std::fprintf(stderr, "write failed\n"); return 1; }
    }
    std::fclose(in);
    if(std::fclose(out) != 0) { std::fprintf(stderr, "cannot flush the output\n"); return 1; }
    return 0;
}

}   // namespace

int main(int argc, char** argv)
{
    Args a;
    std::string err;
    if(!parse(argc, argv, a, err))
    {
        if(!err.empty()) std::fprintf(stderr, "error: %s\n", err.c_str());
        std::fputs(USAGE, stderr);
        return err.empty() ? 0 : 2;
    }
    if(a.mode == Mode::widen) return widen(a);
    if(a.mode == Mode::meta_only) return meta_only(a);
    return convert(a);
}
