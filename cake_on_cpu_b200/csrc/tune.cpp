// Tile-shape selection with a persistent cache: the GPU counterpart of the reference's
// block-size autotuner (reference src/autotune_sa.cpp:13-82, include/autotune.h:82-86: a
// random-step search over (m_c, k_c, n_c) with a visited set and clamps) and of the override
// hook update_mr_nr (src/block_sizing.cpp:78-83).
//
// What can be chosen per shape for the large-matrix kernel: the tile width (128 or 256
// columns of C), the band height of the tile walk, and the number of K pieces each tile of the
// ragged last wave is cut into.  A search walks that small grid by random steps from the rule's
// own choice, never visiting a point twice, keeps the cheapest point seen and occasionally
// accepts a worse one as the next starting point (annealing).  Winners are kept per
// (M, N, K, schedule) and can be written to / read from a JSON file; the file named by the
// environment variable CAKE_AUTOTUNE_CACHE is loaded on first use and rewritten after every search.
//
// Host logic only: the cost of a point comes from a callback (device timing in the library,
// anything in a test).
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <set>
#include <string>
#include <tuple>
#include <vector>

#include "cake_b200.h"

namespace cakeb200 {
void set_error(const char* fmt, ...);

namespace {

struct Entry {
    int tile_n, band, k_pieces;
    float ms;
};
typedef std::tuple<int, int, int, int> ShapeKey;  // M, N, K, schedule

std::mutex g_mutex;
std::map<ShapeKey, Entry> g_cache;
bool g_env_loaded = false;

uint64_t next_random(uint64_t& state) {
    state += 0x9E3779B97F4A7C15ULL;
    uint64_t z = state;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    return z ^ (z >> 31);
}

int load_locked(const char* path) {
    FILE* f = fopen(path, "r");
    if (!f) return -1;
    std::string text;
    char buf[4096];
    size_t n;
    while ((n = fread(buf, 1, sizeof(buf), f)) > 0) text.append(buf, n);
    fclose(f);
    // one object per entry: {"M": m, "N": n, "K": k, "sched": s, "tile_n": t, "band": b, "k_pieces": p, "ms": x}
    int loaded = 0;
    size_t at = 0;
    while ((at = text.find("{\"M\":", at)) != std::string::npos) {
        int M, N, K, s, t, b, p;
        float ms;
        if (sscanf(text.c_str() + at, "{\"M\": %d, \"N\": %d, \"K\": %d, \"sched\": %d, \"tile_n\": %d, \"band\": %d, \"k_pieces\": %d, \"ms\": %f}",
                   &M, &N, &K, &s, &t, &b, &p, &ms) == 8 &&
            M > 0 && N > 0 && K > 0 && s >= 0 && s <= 2 && (t == 0 || t == 128 || t == 256) && b >= 1 && p >= 0) {
            g_cache[ShapeKey(M, N, K, s)] = {t, b, p, ms};
            loaded++;
        }
        at += 5;
    }
    return loaded;
}

int save_locked(const char* path) {
    std::string tmp = std::string(path) + ".tmp";
    FILE* f = fopen(tmp.c_str(), "w");
    if (!f) return -1;
    fprintf(f, "{\"version\": 1, \"kernel\": \"sgemm_tf32x3\", \"entries\": [\n");
    size_t i = 0;
    for (const auto& kv : g_cache) {
        fprintf(f, "  {\"M\": %d, \"N\": %d, \"K\": %d, \"sched\": %d, \"tile_n\": %d, \"band\": %d, \"k_pieces\": %d, \"ms\": %.6f}%s\n",
                std::get<0>(kv.first), std::get<1>(kv.first), std::get<2>(kv.first), std::get<3>(kv.first), kv.second.tile_n,
                kv.second.band, kv.second.k_pieces, kv.second.ms, ++i < g_cache.size() ? "," : "");
    }
    fprintf(f, "]}\n");
    fclose(f);
    return rename(tmp.c_str(), path) == 0 ? (int) g_cache.size() : -1;
}

void load_env_locked() {
    if (g_env_loaded) return;
    g_env_loaded = true;
    if (const char* path = getenv("CAKE_AUTOTUNE_CACHE")) load_locked(path);
}

}  // namespace

// The cached choice for a shape, if any (used by the kernel's host side on every launch).
bool tune_lookup(int M, int N, int K, int sched, int* tile_n, int* band, int* k_pieces) {
    std::lock_guard<std::mutex> lock(g_mutex);
    load_env_locked();
    auto it = g_cache.find(ShapeKey(M, N, K, sched));
    if (it == g_cache.end()) return false;
    *tile_n = it->second.tile_n;
    *band = it->second.band;
    *k_pieces = it->second.k_pieces;
    return true;
}

}  // namespace cakeb200

using namespace cakeb200;

extern "C" {

int cakeb200_tune_put(int M, int N, int K, int sched, int tile_n, int band, int k_pieces, float ms) {
    if (M <= 0 || N <= 0 || K <= 0 || sched < 0 || sched > 2 || (tile_n != 0 && tile_n != 128 && tile_n != 256) || band < 1 || k_pieces < 0) {
        set_error("cakeb200_tune_put: bad entry");
        return CAKEB200_ERR_ARG;
    }
    std::lock_guard<std::mutex> lock(g_mutex);
    load_env_locked();
    g_cache[ShapeKey(M, N, K, sched)] = {tile_n, band, k_pieces, ms};
    return CAKEB200_OK;
}

int cakeb200_tune_get(int M, int N, int K, int sched, int* tile_n, int* band, int* k_pieces, float* ms) {
    std::lock_guard<std::mutex> lock(g_mutex);
    load_env_locked();
    auto it = g_cache.find(ShapeKey(M, N, K, sched));
    if (it == g_cache.end()) return 0;
    if (tile_n) *tile_n = it->second.tile_n;
    if (band) *band = it->second.band;
    if (k_pieces) *k_pieces = it->second.k_pieces;
    if (ms) *ms = it->second.ms;
    return 1;
}

int cakeb200_tune_clear(void) {
    std::lock_guard<std::mutex> lock(g_mutex);
    g_env_loaded = true;  // an explicit clear is not undone by a later lazy load of the environment's file
    g_cache.clear();
    return CAKEB200_OK;
}

int cakeb200_tune_save(const char* path) {
    if (!path) return CAKEB200_ERR_ARG;
    std::lock_guard<std::mutex> lock(g_mutex);
    const int n = save_locked(path);
    if (n < 0) {
        set_error("cakeb200_tune_save: cannot write %s", path);
        return CAKEB200_ERR_ARG;
    }
    return n;
}

int cakeb200_tune_load(const char* path) {
    if (!path) return CAKEB200_ERR_ARG;
    std::lock_guard<std::mutex> lock(g_mutex);
    g_env_loaded = true;
    const int n = load_locked(path);
    if (n < 0) {
        set_error("cakeb200_tune_load: cannot read %s", path);
        return CAKEB200_ERR_ARG;
    }
    return n;
}

int cakeb200_tune_search(int M, int N, int K, int sm_count, int trials, unsigned long long seed, cakeb200_tune_cost cost,
                         void* user, int* tile_n, int* band, int* k_pieces, float* best_ms, int* evaluated) {
    if (M <= 0 || N <= 0 || K <= 0 || sm_count <= 0 || trials < 1 || !cost || !tile_n || !band || !k_pieces) {
        set_error("cakeb200_tune_search: bad argument");
        return CAKEB200_ERR_ARG;
    }
    // the grid: every axis sorted, the rule's own choice marked as the start
    std::vector<int> widths, bands, pieces;
    if (N > 128) widths = {128, 256};
    else widths = {128};
    const int rule_w = (N > 128) ? 256 : 128;
    const int tiles_m = (M + 127) / 128;
    for (int b : {2, 4, 8, 16})
        if (b <= std::max(2, tiles_m) || b == 2) bands.push_back(b);
    const int kblocks = (K + 31) / 32;
    pieces.push_back(0);  // 0 = the cost model of the library decides
    for (int s : {1, 2, 3, 4, 6, 8, 12, 16, 24, 32})
        if (s <= kblocks / 8 || s == 1) pieces.push_back(s);
    int iw = (int) (std::find(widths.begin(), widths.end(), rule_w) - widths.begin());
    int ib = (int) (std::find(bands.begin(), bands.end(), 8) - bands.begin());
    if (ib == (int) bands.size()) ib = (int) bands.size() - 1;
    int ip = 0;
    std::set<std::tuple<int, int, int>> visited;
    uint64_t rng = seed ? seed : 1;
    double best = -1, current = -1, temperature = 0.05;
    int best_w = iw, best_b = ib, best_p = ip, done = 0;
    const int points = (int) (widths.size() * bands.size() * pieces.size());
    for (int t = 0; t < trials && (int) visited.size() < points; t++) {
        int cw = iw, cb = ib, cp = ip;
        if (t > 0) {
            // random step of -1, 0 or +1 along every axis, clamped to the grid (the reference steps its three
            // block sizes by random multiples of 30 / 20 / 128 and clamps them, src/autotune_sa.cpp:36-70);
            // a point seen before is stepped on from until a new one turns up
            for (int tries = 0; tries < 64; tries++) {
                cw = std::min((int) widths.size() - 1, std::max(0, iw + (int) (next_random(rng) % 3) - 1));
                cb = std::min((int) bands.size() - 1, std::max(0, ib + (int) (next_random(rng) % 3) - 1));
                cp = std::min((int) pieces.size() - 1, std::max(0, ip + (int) (next_random(rng) % 3) - 1));
                if (!visited.count(std::make_tuple(cw, cb, cp))) break;
                iw = cw; ib = cb; ip = cp;  // walk through visited points
            }
            if (visited.count(std::make_tuple(cw, cb, cp))) {
                // cornered: take the first unvisited point of the grid
                bool found = false;
                for (int a = 0; a < (int) widths.size() && !found; a++)
                    for (int b = 0; b < (int) bands.size() && !found; b++)
                        for (int c = 0; c < (int) pieces.size() && !found; c++)
                            if (!visited.count(std::make_tuple(a, b, c))) { cw = a; cb = b; cp = c; found = true; }
            }
        }
        visited.insert(std::make_tuple(cw, cb, cp));
        const double ms = cost(widths[cw], bands[cb], pieces[cp], user);
        done++;
        if (ms <= 0) continue;  // the point is not valid for this shape
        if (best < 0 || ms < best) { best = ms; best_w = cw; best_b = cb; best_p = cp; }
        const bool accept = current < 0 || ms < current ||
                            (double) (next_random(rng) >> 11) / 9007199254740992.0 < std::exp(-(ms - current) / (current * temperature));
        if (accept) { current = ms; iw = cw; ib = cb; ip = cp; }
        temperature *= 0.9;
    }
    if (best < 0) {
        set_error("cakeb200_tune_search: no valid point");
        return CAKEB200_ERR_ARG;
    }
    *tile_n = widths[best_w];
    *band = bands[best_b];
    *k_pieces = pieces[best_p];
    if (best_ms) *best_ms = (float) best;
    if (evaluated) *evaluated = done;
    return CAKEB200_OK;
}

}  // extern "C"
