// On-disk formats of the drop-in surface, written from their descriptions in the reference:
//   text        n little-endian u16 symbols, no header (src/GPU_SACA.cu:51)
//   sa40        n entries of 5 little-endian bytes (include/sa40.hpp:14-24)
//   index.meta  key=value lines (include/Index_Meta.hpp:147-241)
//   .qry        64-byte header, u64 off[q+1], symbols; .itv q x {u64 lo, hi}; .cnt q x u64 (include/query-file.hpp:11-19)
//   .pos        (an extension; the reference has no locate output) u64 q, u64 total, u64 off[q+1], u64 pos[total]
#pragma once

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <cerrno>
#include <cstdlib>
#include <ctime>
#include <fstream>
#include <utility>
#include <sstream>
#include <string>
#include <sys/stat.h>
#include <vector>

namespace cascade_host
{

inline bool file_size(const std::string& path, uint64_t& bytes)
{
    struct stat st;
    if(::stat(path.c_str(), &st) != 0) return false;
    bytes = static_cast<uint64_t>(st.st_size);
    return true;
}

inline bool read_file(const std::string& path, void* dst, uint64_t bytes, std::string& err)
{
    FILE* f = std::fopen(path.c_str(), "rb");
    if(!f) { err = "cannot open " + path; return false; }
    uint64_t got = 0;
    while(got < bytes)
    {
        const size_t r = std::fread(static_cast<char*>(dst) + got, 1, size_t(std::min<uint64_t>(bytes - got, 1ull << 30)), f);
        if(r == 0) break;
        got += r;
    }
    std::fclose(f);
    if(got != bytes) { err = "short read of " + path; return false; }
    return true;
}

inline bool write_file(const std::string& path, const void* src, uint64_t bytes, std::string& err)
{
    FILE* f = std::fopen(path.c_str(), "wb");
    if(!f) { err = "cannot create " + path; return false; }
    uint64_t put = 0;
    while(put < bytes)
    {
        const size_t w = std::fwrite(static_cast<const char*>(src) + put, 1, size_t(std::min<uint64_t>(bytes - put, 1ull << 30)), f);
        if(w == 0) break;
        put += w;
    }
    const bool ok = (std::fclose(f) == 0) && put == bytes;
    if(!ok) err = "short write of " + path;
    return ok;
}

inline std::string dir_of(const std::string& p) { const auto s = p.find_last_of('/'); return s == std::string::npos ? "." : p.substr(0, s); }
inline std::string join(const std::string& dir, const std::string& p) { return (!p.empty() && p[0] == '/') ? p : dir + "/" + p; }

struct Index_Meta
{
    uint64_t n = 0;
    uint32_t sym_bytes = 2, sa_width = 5;
    std::string sa_order = "numeric_eot_smallest", text, sa_source = "cascade_b200", created_utc;
    std::vector<std::string> sa_part;
    std::vector<uint64_t> sa_part_off;
    long long sep = 65535;
};

// index.meta is a list of key=value lines (schema: include/Index_Meta.hpp:207-241 of the reference). The two helpers
// below keep the schema in ONE table of rows, used for writing and for reading.
class Meta_Lines
{
    std::vector<std::pair<std::string, std::string>> rows_;
    std::string problem_;
public:
    void put(const std::string& key, const std::string& value) { rows_.emplace_back(key, value); }
    void put(const std::string& key, unsigned long long value) { rows_.emplace_back(key, std::to_string(value)); }
    void put_signed(const std::string& key, long long value) { rows_.emplace_back(key, std::to_string(value)); }
    std::string text() const
    {
        std::string out;
        for(const auto& r : rows_) out += r.first + "=" + r.second + "\n";
        return out;
    }
    // Reads `path`; comment lines (#) and empty lines are skipped.
    bool load(const std::string& path)
    {
        std::ifstream is(path);
        if(!is) { problem_ = "cannot open index metadata: " + path; return false; }
        for(std::string line; std::getline(is, line); )
        {
            if(line.empty() || line[0] == '#') continue;
            const size_t eq = line.find('=');
            if(eq == std::string::npos) { problem_ = "index.meta: a line without `=`: " + line; return false; }
            rows_.emplace_back(line.substr(0, eq), line.substr(eq + 1));
        }
        return true;
    }
    const std::string* find(const std::string& key) const
    {
        for(auto it = rows_.rbegin(); it != rows_.rend(); ++it) if(it->first == key) return &it->second;     // a later line wins
        return nullptr;
    }
    // The accessors note the first key that is missing or unreadable and return a neutral value; `problem()` tells.
    std::string str(const std::string& key)
    {
        const std::string* v = find(key);
        if(!v && problem_.empty()) problem_ = "index.meta: no `" + key + "`";
        return v ? *v : std::string();
    }
    unsigned long long num(const std::string& key)
    {
        const std::string v = str(key);
        char* stop = nullptr;
        errno = 0;
        const unsigned long long x = v.empty() ? 0 : std::strtoull(v.c_str(), &stop, 10);
        if((v.empty() || errno != 0 || (stop && *stop)) && problem_.empty()) problem_ = "index.meta: `" + key + "` is not a number";
        return x;
    }
    const std::string& problem() const { return problem_; }
};

inline bool write_index_meta(const std::string& dir, const Index_Meta& m, std::string& err)
{
    std::string when = m.created_utc;
    if(when.empty())
    {
        char buf[32] = "";
        const std::time_t t = std::time(nullptr);
        std::strftime(buf, sizeof(buf), "%Y-%m-%dT%H:%M:%SZ", std::gmtime(&t));
        when = buf;
    }
    Meta_Lines L;
    L.put("format", "gpu_saca_query_index");
    L.put("format_version", 1ull);
    L.put("n", m.n);
    L.put("sym_bytes", m.sym_bytes);
    L.put("sa_width", m.sa_width);
    L.put("sa_order", m.sa_order);
    L.put("text", m.text);
    L.put("sa_part_c", m.sa_part.size());
    for(size_t i = 0; i < m.sa_part.size(); ++i)
    {
        L.put("sa_part_" + std::to_string(i), m.sa_part[i]);
        L.put("sa_part_off_" + std::to_string(i), m.sa_part_off[i]);
    }
    L.put_signed("sep", m.sep);
    L.put("sa_source", m.sa_source);
    L.put("created_utc", when);
    // written beside its final name and moved there, so that a reader never sees half a file
    const std::string final_path = dir + "/index.meta", draft = final_path + ".tmp";
    std::ofstream os(draft, std::ios::trunc);
    os << L.text();
    os.close();
    if(!os) { err = "cannot write " + draft; return false; }
    if(std::rename(draft.c_str(), final_path.c_str()) != 0) { err = "cannot move " + draft + " to " + final_path; return false; }
    return true;
}

inline bool read_index_meta(const std::string& dir, Index_Meta& m, std::string& err)
{
    Meta_Lines L;
    if(!L.load(dir + "/index.meta")) { err = L.problem(); return false; }
    if(L.str("format") != "gpu_saca_query_index") { err = L.problem().empty() ? "index.meta: not a query index" : L.problem(); return false; }
    if(L.num("format_version") != 1) { err = L.problem().empty() ? "index.meta: only format_version 1 is understood" : L.problem(); return false; }
    m.n = L.num("n");
    m.sym_bytes = uint32_t(L.num("sym_bytes"));
    m.sa_width = uint32_t(L.num("sa_width"));
    m.sa_order = L.str("sa_order");
    m.text = join(dir, L.str("text"));
    const unsigned long long parts = L.num("sa_part_c");
    m.sa_part.clear();
    m.sa_part_off.clear();
    for(unsigned long long i = 0; i < parts && L.problem().empty(); ++i)
    {
        m.sa_part.push_back(join(dir, L.str("sa_part_" + std::to_string(i))));
        m.sa_part_off.push_back(L.num("sa_part_off_" + std::to_string(i)));
    }
    if(!L.problem().empty()) { err = L.problem(); return false; }
    // optional keys
    const std::string* sep = L.find("sep");
    m.sep = sep ? std::atoll(sep->c_str()) : -1;
    if(const std::string* v = L.find("sa_source")) m.sa_source = *v; else m.sa_source.clear();
    if(const std::string* v = L.find("created_utc")) m.created_utc = *v; else m.created_utc.clear();
    if(m.sa_width != 5 || m.sa_order != "numeric_eot_smallest") { err = "index.meta: only 5-byte entries in numeric order are supported"; return false; }
    return true;
}

#pragma pack(push, 1)
struct Query_File_Header
{
    char magic[8]; uint32_t version, sym_bytes; uint64_t q_c, sym_c, min_len, max_len, seed, reserved;
};
#pragma pack(pop)
static_assert(sizeof(Query_File_Header) == 64, "the .qry header is 64 bytes");

inline bool read_qry(const std::string& path, uint64_t q_max, std::vector<uint64_t>& off, std::vector<uint16_t>& sym, std::string& err)
{
    FILE* f = std::fopen(path.c_str(), "rb");
    if(!f) { err = "cannot open query file: " + path; return false; }
    Query_File_Header h;
    auto fail = [&](const std::string& w) { std::fclose(f); err = w + ": " + path; return false; };
    if(std::fread(&h, sizeof(h), 1, f) != 1) return fail("truncated query-file header");
    if(std::memcmp(h.magic, "GSAQRY01", 8) != 0) return fail("not a query file (bad magic)");
    if(h.version != 1) return fail("unsupported query-file version");
    if(h.sym_bytes != 2) return fail("query-file symbol width is not 2");
    const uint64_t q = q_max < h.q_c ? q_max : h.q_c;
    off.resize(q + 1);
    if(std::fread(off.data(), 8, q + 1, f) != q + 1) return fail("truncated query offsets");
    if(off[0] != 0) return fail("query offsets must start at 0");
    for(uint64_t i = 0; i < q; ++i) if(off[i + 1] < off[i]) return fail("query offsets are not non-decreasing");
    if(off[q] > h.sym_c) return fail("query offsets exceed the symbol count");
    if(h.q_c > q && std::fseek(f, long((h.q_c - q) * 8), SEEK_CUR) != 0) return fail("cannot seek past the query offsets");
    sym.resize(off[q] + 8);
    if(off[q] && std::fread(sym.data(), 2, off[q], f) != off[q]) return fail("truncated query symbols");
    std::fclose(f);
    return true;
}

inline bool write_qry(const std::string& path, const std::vector<uint64_t>& off, const uint16_t* sym, uint64_t seed, std::string& err)
{
    Query_File_Header h{};
    std::memcpy(h.magic, "GSAQRY01", 8);
    h.version = 1; h.sym_bytes = 2; h.q_c = off.size() - 1; h.sym_c = off.back(); h.seed = seed;
    h.min_len = h.q_c ? UINT64_MAX : 0; h.max_len = 0;
    for(uint64_t i = 0; i < h.q_c; ++i) { const uint64_t l = off[i + 1] - off[i]; if(l < h.min_len) h.min_len = l; if(l > h.max_len) h.max_len = l; }
    const std::string tmp = path + ".tmp";
    FILE* f = std::fopen(tmp.c_str(), "wb");
    if(!f) { err = "cannot create query file: " + tmp; return false; }
    const bool ok = std::fwrite(&h, sizeof(h), 1, f) == 1 && std::fwrite(off.data(), 8, off.size(), f) == off.size()
                    && (h.sym_c == 0 || std::fwrite(sym, 2, h.sym_c, f) == h.sym_c);
    if(std::fclose(f) != 0 || !ok || std::rename(tmp.c_str(), path.c_str()) != 0) { err = "cannot write query file: " + path; return false; }
    return true;
}

}   // namespace cascade_host
