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
#include <ctime>
#include <fstream>
#include <map>
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

inline bool write_index_meta(const std::string& dir, const Index_Meta& m, std::string& err)
{
    std::ostringstream o;
    o << "format=gpu_saca_query_index\nformat_version=1\nn=" << m.n << "\nsym_bytes=" << m.sym_bytes << "\nsa_width=" << m.sa_width
      << "\nsa_order=" << m.sa_order << "\ntext=" << m.text << "\nsa_part_c=" << m.sa_part.size() << "\n";
    for(size_t i = 0; i < m.sa_part.size(); ++i) o << "sa_part_" << i << "=" << m.sa_part[i] << "\nsa_part_off_" << i << "=" << m.sa_part_off[i] << "\n";
    char when[32] = "";
    const std::time_t t = std::time(nullptr);
    std::strftime(when, sizeof(when), "%Y-%m-%dT%H:%M:%SZ", std::gmtime(&t));
    o << "sep=" << m.sep << "\nsa_source=" << m.sa_source << "\ncreated_utc=" << (m.created_utc.empty() ? when : m.created_utc) << "\n";
    const std::string path = dir + "/index.meta", tmp = path + ".tmp";
    { std::ofstream os(tmp); os << o.str(); if(!os) { err = "cannot write " + tmp; return false; } }
    if(std::rename(tmp.c_str(), path.c_str()) != 0) { err = "cannot rename " + tmp; return false; }
    return true;
}

inline bool read_index_meta(const std::string& dir, Index_Meta& m, std::string& err)
{
    std::ifstream is(dir + "/index.meta");
    if(!is) { err = "cannot open index metadata: " + dir + "/index.meta"; return false; }
    std::map<std::string, std::string> kv;
    for(std::string line; std::getline(is, line); )
    {
        if(line.empty() || line[0] == '#') continue;
        const auto eq = line.find('=');
        if(eq == std::string::npos) { err = "malformed line in index.meta: `" + line + "`"; return false; }
        kv[line.substr(0, eq)] = line.substr(eq + 1);
    }
    try
    {
        if(kv["format"] != "gpu_saca_query_index") { err = "not a query-index metadata file"; return false; }
        if(std::stoul(kv.at("format_version")) != 1) { err = "unsupported index-metadata version"; return false; }
        m.n = std::stoull(kv.at("n"));
        m.sym_bytes = uint32_t(std::stoul(kv.at("sym_bytes")));
        m.sa_width = uint32_t(std::stoul(kv.at("sa_width")));
        m.sa_order = kv.at("sa_order");
        m.text = join(dir, kv.at("text"));
        const uint64_t c = std::stoull(kv.at("sa_part_c"));
        m.sa_part.clear(); m.sa_part_off.clear();
        for(uint64_t i = 0; i < c; ++i)
        {
            m.sa_part.push_back(join(dir, kv.at("sa_part_" + std::to_string(i))));
            m.sa_part_off.push_back(std::stoull(kv.at("sa_part_off_" + std::to_string(i))));
        }
        m.sep = kv.count("sep") ? std::stoll(kv["sep"]) : -1;
        m.sa_source = kv["sa_source"]; m.created_utc = kv["created_utc"];
    }
    catch(const std::exception&) { err = "missing or malformed field in index.meta"; return false; }
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
