/* TEST INFRASTRUCTURE ONLY: a CPU restatement, in plain C, of the reference's algorithm for the
 * suffix-array build and the batched count/locate queries. Only the tests, the smoke check and the
 * CPU-baseline leg of the benchmark may load it; the product never does.
 *
 * Parity is pinned: tests check every function here against the reference's own compiled CPU code
 * (libcascade_ref.so, built from the reference's sources by the Makefile beside this file) and
 * against committed golden vectors produced by that code, which include the reference's
 * known-answer table (src/test_query.cu:373-392).
 *
 * Each function names the reference code that it restates (paths within the reference project).
 */
#define _GNU_SOURCE
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define SA_WIDTH 5 /* include/sa40.hpp:17 */

/* include/sa40.hpp:43-62 (host branch): the 5 little-endian bytes at rank r. */
static inline uint64_t sa40_load(const uint8_t* SA, uint64_t r)
{
    uint64_t v = 0;
    memcpy(&v, SA + SA_WIDTH * r, SA_WIDTH);
    return v;
}

/* include/sa40.hpp:66-69 */
static inline void sa40_store(uint8_t* SA, uint64_t r, uint64_t v) { memcpy(SA + SA_WIDTH * r, &v, SA_WIDTH); }

/* include/CPU_Reference.hpp:107-123 with max_cmp = n: numeric symbol order, and a suffix that is a
 * proper prefix of another one sorts first. */
int orc_cmp_suffixes(const uint16_t* T, uint64_t n, uint64_t i, uint64_t j)
{
    const uint64_t len_i = n - i, len_j = n - j;
    const uint64_t len = len_i < len_j ? len_i : len_j;
    for(uint64_t k = 0; k < len; ++k)
        if(T[i + k] != T[j + k])
            return T[i + k] < T[j + k] ? -1 : 1;
    if(i == j)
        return 0;
    return len_i < len_j ? -1 : 1;
}

/* include/CPU_Reference.hpp:26-36 */
int orc_cmp_suffix_pattern(const uint16_t* T, uint64_t n, uint64_t pos, const uint16_t* P, uint64_t m)
{
    const uint64_t len = (n - pos < m ? n - pos : m);
    for(uint64_t i = 0; i < len; ++i)
        if(T[pos + i] != P[i])
            return T[pos + i] < P[i] ? -1 : 1;
    return len < m ? -1 : 0;
}

struct cmp_ctx { const uint16_t* T; uint64_t n; };

static int cmp_idx(const void* a, const void* b, void* c)
{
    const struct cmp_ctx* x = (const struct cmp_ctx*)c;
    return orc_cmp_suffixes(x->T, x->n, *(const uint64_t*)a, *(const uint64_t*)b);
}

static void merge_runs(const struct cmp_ctx* c, const uint64_t* a, uint64_t na, const uint64_t* b, uint64_t nb, uint64_t* out)
{
    uint64_t i = 0, j = 0, k = 0;
    while(i < na && j < nb)
        out[k++] = (orc_cmp_suffixes(c->T, c->n, b[j], a[i]) < 0) ? b[j++] : a[i++];
    while(i < na) out[k++] = a[i++];
    while(j < nb) out[k++] = b[j++];
}

/* test/query.cpp:42-55 (`build_sa40`): every suffix index, comparison-sorted with `cmp_suffixes`, stored as
 * 5-byte entries. The sort is split into runs that the host's threads sort and merge; the order is total, so
 * the result does not depend on the number of threads. Returns 0, or -1 if memory runs out. */
int orc_build_sa40(const uint16_t* T, uint64_t n, uint8_t* sa40_out, int threads)
{
    if(n == 0)
        return 0;
#ifdef _OPENMP
    if(threads <= 0) threads = omp_get_max_threads();
#else
    threads = 1;
#endif
    uint64_t* sa = (uint64_t*)malloc(n * sizeof(uint64_t));
    uint64_t* tmp = (uint64_t*)malloc(n * sizeof(uint64_t));
    if(!sa || !tmp) { free(sa); free(tmp); return -1; }
    struct cmp_ctx c = {T, n};

    uint64_t runs = 1;
    while(runs < (uint64_t)threads * 4 && n / (runs * 2) >= 4096) runs *= 2;
    const uint64_t run_len = (n + runs - 1) / runs;

    #pragma omp parallel for schedule(dynamic, 1) num_threads(threads)
    for(uint64_t r = 0; r < runs; ++r)
    {
        const uint64_t b = r * run_len, e = (b + run_len < n ? b + run_len : n);
        if(b >= e) continue;
        for(uint64_t i = b; i < e; ++i) sa[i] = i;
        qsort_r(sa + b, e - b, sizeof(uint64_t), cmp_idx, &c);
    }

    uint64_t* src = sa; uint64_t* dst = tmp;
    for(uint64_t w = run_len; w < n; w *= 2)
    {
        const uint64_t pairs = (n + 2 * w - 1) / (2 * w);
        #pragma omp parallel for schedule(dynamic, 1) num_threads(threads)
        for(uint64_t p = 0; p < pairs; ++p)
        {
            const uint64_t b = p * 2 * w;
            const uint64_t mid = (b + w < n ? b + w : n), e = (b + 2 * w < n ? b + 2 * w : n);
            merge_runs(&c, src + b, mid - b, src + mid, e - mid, dst + b);
        }
        uint64_t* t = src; src = dst; dst = t;
    }

    #pragma omp parallel for schedule(static) num_threads(threads)
    for(uint64_t r = 0; r < n; ++r)
        sa40_store(sa40_out, r, src[r]);

    free(sa); free(tmp);
    return 0;
}

/* test/end-to-end.cpp:11-80 (`is_permutation` + `is_correct_SA`): SA is a permutation of [0, n), and every
 * adjacent pair x = SA[i-1], y = SA[i] has T[x] < T[y], or T[x] = T[y] and rank[x+1] < rank[y+1] with
 * rank(n) = -1. Returns 1 if correct, 0 if not, -1 if memory runs out. */
int orc_is_correct_sa40(const uint16_t* T, uint64_t n, const uint8_t* SA)
{
    if(n == 0) return 1;
    uint64_t* rank = (uint64_t*)malloc(n * sizeof(uint64_t));
    uint8_t* seen = (uint8_t*)calloc(n, 1);
    if(!rank || !seen) { free(rank); free(seen); return -1; }
    int ok = 1;
    for(uint64_t i = 0; i < n; ++i)
    {
        const uint64_t x = sa40_load(SA, i);
        if(x >= n || seen[x]) { ok = 0; break; }
        seen[x] = 1;
        rank[x] = i;
    }
    if(ok)
    {
        #pragma omp parallel for schedule(static) reduction(&& : ok)
        for(uint64_t i = 1; i < n; ++i)
        {
            const uint64_t x = sa40_load(SA, i - 1), y = sa40_load(SA, i);
            if(T[x] < T[y]) continue;
            if(T[x] > T[y]) { ok = 0; continue; }
            const int64_t nx = (x + 1 < n ? (int64_t)rank[x + 1] : -1);
            const int64_t ny = (y + 1 < n ? (int64_t)rank[y + 1] : -1);
            if(nx >= ny) ok = 0;
        }
    }
    free(rank); free(seen);
    return ok;
}

/* include/CPU_Reference.hpp:42-73 (`find_one`): lo = first rank whose truncated suffix is not smaller than P,
 * hi = first rank whose truncated suffix is greater; the empty pattern's interval is [0, n). */
void orc_find_one(const uint16_t* T, uint64_t n, const uint8_t* SA, const uint16_t* P, uint64_t m, uint64_t* lo_out, uint64_t* hi_out)
{
    if(m == 0) { *lo_out = 0; *hi_out = n; return; }
    uint64_t low = 0, high = n;
    while(low < high)
    {
        const uint64_t mid = low + (high - low) / 2;
        if(orc_cmp_suffix_pattern(T, n, sa40_load(SA, mid), P, m) < 0) low = mid + 1; else high = mid;
    }
    *lo_out = low;
    high = n;
    while(low < high)
    {
        const uint64_t mid = low + (high - low) / 2;
        if(orc_cmp_suffix_pattern(T, n, sa40_load(SA, mid), P, m) <= 0) low = mid + 1; else high = mid;
    }
    *hi_out = low;
}

/* test/query.cpp:82-97 (`brute_find`): the interval without any suffix array. */
void orc_brute_find(const uint16_t* T, uint64_t n, const uint16_t* P, uint64_t m, uint64_t* lo_out, uint64_t* hi_out)
{
    if(m == 0) { *lo_out = 0; *hi_out = n; return; }
    uint64_t less = 0, equal = 0;
    for(uint64_t i = 0; i < n; ++i)
    {
        const int c = orc_cmp_suffix_pattern(T, n, i, P, m);
        less += (c < 0);
        equal += (c == 0);
    }
    *lo_out = less; *hi_out = less + equal;
}

/* include/CPU_Reference.hpp:79-101 (`certify`) */
int orc_certify(const uint16_t* T, uint64_t n, const uint8_t* SA, const uint16_t* P, uint64_t m, uint64_t lo, uint64_t hi)
{
    if(lo > hi || hi > n) return 0;
    if(m == 0) return lo == 0 && hi == n;
    if(lo > 0 && orc_cmp_suffix_pattern(T, n, sa40_load(SA, lo - 1), P, m) >= 0) return 0;
    if(lo < hi && (orc_cmp_suffix_pattern(T, n, sa40_load(SA, lo), P, m) != 0 || orc_cmp_suffix_pattern(T, n, sa40_load(SA, hi - 1), P, m) != 0)) return 0;
    if(hi < n && orc_cmp_suffix_pattern(T, n, sa40_load(SA, hi), P, m) <= 0) return 0;
    return 1;
}

/* The batched search of src/Host_Search.cpp:519-538 in direct mode, reduced to its result: query i's interval
 * is `find_one` of sym[off[i], off[i+1]). itv_out holds {lo, hi} pairs. The host's threads share the queries. */
void orc_find_batch(const uint16_t* T, uint64_t n, const uint8_t* SA, const uint64_t* off, const uint16_t* sym, uint64_t q,
                    uint64_t* itv_out, int threads)
{
#ifdef _OPENMP
    if(threads <= 0) threads = omp_get_max_threads();
#endif
    #pragma omp parallel for schedule(dynamic, 1024) num_threads(threads)
    for(uint64_t i = 0; i < q; ++i)
        orc_find_one(T, n, SA, sym + (off[i] - off[0]), off[i + 1] - off[i], &itv_out[2 * i], &itv_out[2 * i + 1]);
}

/* Locate has no counterpart in the reference (its results are intervals and counts only, include/query-file.hpp:18-19).
 * It is defined from the interval: the positions SA[lo + k], k < min(max_pos, hi - lo), in rank order.
 * pos_out holds q * max_pos words (row i at i * max_pos), cnt_out the number of positions of each query. */
void orc_locate_batch(const uint8_t* SA, const uint64_t* itv, uint64_t q, uint32_t max_pos, uint64_t* pos_out, uint32_t* cnt_out)
{
    #pragma omp parallel for schedule(static)
    for(uint64_t i = 0; i < q; ++i)
    {
        const uint64_t lo = itv[2 * i], hi = itv[2 * i + 1];
        const uint64_t c = (hi - lo < max_pos ? hi - lo : max_pos);
        cnt_out[i] = (uint32_t)c;
        for(uint64_t k = 0; k < c; ++k)
            pos_out[i * (uint64_t)max_pos + k] = sa40_load(SA, lo + k);
    }
}

/* include/query-file.hpp:228-263: FNV-1a-64 over the little-endian bytes of the counts hi - lo. */
uint64_t orc_counts_hash(const uint64_t* itv, uint64_t q)
{
    uint64_t h = 0xcbf29ce484222325ull;
    for(uint64_t i = 0; i < q; ++i)
    {
        const uint64_t c = itv[2 * i + 1] - itv[2 * i];
        for(int b = 0; b < 8; ++b) { h ^= (c >> (8 * b)) & 0xFF; h *= 0x100000001b3ull; }
    }
    return h;
}

int orc_max_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void orc_set_threads(int threads)
{
#ifdef _OPENMP
    if(threads > 0) omp_set_num_threads(threads);
#else
    (void)threads;
#endif
}

/* The seeded synthetic corpus of the benchmark, for the CPU arms that must not load the product library. It is not
 * part of the reference (its corpora are tokenized text, dataset/tokenize-corpus.py:4-7 gives their layout: u16 ids with
 * 0xFFFF before each document); every symbol is a function of (seed, position): position 0 and every position after a
 * document's last token hold 0xFFFF, a document ends after each token with probability 1 / mean_doc, tokens are drawn by
 * inverse CDF from 64-bit thresholds. The product's generators make the same symbols (a CPU test compares them). */
static uint64_t corpus_hash64(uint64_t x)
{
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

static int corpus_ends_after(uint64_t seed, uint64_t j, uint32_t mean_doc)
{
    return corpus_hash64(seed * 0x9E3779B97F4A7C15ull + 2 * j + 1) % mean_doc == 0;
}

void orc_gen_corpus(uint16_t* text, uint64_t first, uint64_t count, uint64_t seed, uint32_t mean_doc, const uint64_t* cdf, uint32_t vocab)
{
    #pragma omp parallel for schedule(static)
    for(uint64_t k = 0; k < count; ++k)
    {
        const uint64_t i = first + k;
        int sep;
        if(i == 0) sep = 1;
        else
        {
            /* a separator follows a document's end unless that end flag belongs to a position that is a separator itself */
            uint64_t run = 0, j = i;
            while(j > 0 && corpus_ends_after(seed, j - 1, mean_doc)) { ++run; --j; }
            sep = (j == 0) ? ((i & 1) == 0) : ((run & 1) == 1);
        }
        if(sep) { text[k] = 0xFFFF; continue; }
        const uint64_t u = corpus_hash64(seed * 0xD1B54A32D192ED03ull + 2 * i);
        uint32_t a = 0, b = vocab - 1;
        while(a < b)
        {
            const uint32_t mid = (a + b) >> 1;
            if(u <= cdf[mid]) b = mid; else a = mid + 1;
        }
        text[k] = (uint16_t)a;
    }
}
