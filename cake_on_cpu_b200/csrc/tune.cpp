// Tile-shape selection with a persistent cache: the GPU counterpart of the reference's
// block-size autotuner (reference src/autotune_sa.cpp:13-82, include/autotune.h:82-86: a
// random-step search over (m_c, k_c, n_c) with a visited set and clamps) and of the override
// hook update_mr_nr (src/block_sizing.cpp:78-83).
//
// What can be chosen per shape for the large-matrix kernel: the tile width (128 or 256
// columns of C), the cluster shape (one CTA per 128-row tile, or the two CTAs of a cluster on a
// 256-row tile), the band height of the tile walk, and the number of K pieces each tile of the
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
    int tile_n, cluster, band, k_pieces;  // cluster: 0 = the rule, 1 = pairs of SMs, 2 = single SMs
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
    // one object per entry: {"M": m, "N": n, "K": k, "sched": s, "tile_n": t, "cluster": c, "band": b, "k_pieces": p, "ms": x}
    // (files written before the cluster shape could be chosen have no "cluster": the rule applies)
    int loaded = 0;
    size_t at = 0;
    while ((at = text.find("{\"M\":", at)) != std::string::npos) {
        int M, N, K, s, t, c = 0, b, p;
        float ms;
        bool got = sscanf(text.c_str() + at, "{\"M\": %d, \"N\": %d, \"K\": %d, \"sched\": %d, \"tile_n\": %d, \"cluster\": %d, \"band\": %d, \"k_pieces\": %d, \"ms\": %f}",
                          &M, &N, &K, &s, &t, &c, &b, &p, &ms) == 9;
        if (!got) {
            c = 0;
            got = sscanf(text.c_str() + at, "{\"M\": %d, \"N\": %d, \"K\": %d, \"sched\": %d, \"tile_n\": %d, \"band\": %d, \"k_pieces\": %d, \"ms\": %f}",
                         &M, &N, &K, &s, &t, &b, &p, &ms) == 8;
        }
        if (got && M > 0 && N > 0 && K > 0 && s >= 0 && s <= 2 && (t == 0 || t == 128 || t == 256) && c >= 0 && c <= 2 && b >= 1 && p >= 0) {
            g_cache[ShapeKey(M, N, K, s)] = {t, c, b, p, ms};
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
    fprintf(f, "{\"version\": 2, \"kernel\": \"sgemm_tf32x3\", \"entries\": [\n");
    size_t i = 0;
    for (const auto& kv : g_cache) {
        fprintf(f, "  {\"M\": %d, \"N\": %d, \"K\": %d, \"sched\": %d, \"tile_n\": %d, \"cluster\": %d, \"band\": %d, \"k_pieces\": %d, \"ms\": %.6f}%s\n",
                std::get<0>(kv.first), std::get<1>(kv.first), std::get<2>(kv.first), std::get<3>(kv.first), kv.second.tile_n,
                kv.second.cluster, kv.second.band, kv.second.k_pieces, kv.second.ms, ++i < g_cache.size() ? "," : "");
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
bool tune_lookup(int M, int N, int K, int sched, int* tile_n, int* band, int* k_pieces, int* cluster) {
    std::lock_guard<std::mutex> lock(g_mutex);
    load_env_locked();
    auto it = g_cache.find(ShapeKey(M, N, K, sched));
    if (it == g_cache.end()) return false;
    *tile_n = it->second.tile_n;
    *band = it->second.band;
    *k_pieces = it->second.k_pieces;
    *cluster = it->second.cluster;
    return true;
}

namespace {
// The search over a grid of four sorted axes from a starting point; `cost` gets the values of a point.
struct Axes {
    std::vector<int> v[4];
    int start[4];
};
typedef double (*PointCost)(const int* values, void* user);

int search_grid(const Axes& ax, int trials, unsigned long long seed, PointCost cost, void* user, int* best_values, float* best_ms,
                int* evaluated) {
    int at[4] = {ax.start[0], ax.start[1], ax.start[2], ax.start[3]};
    std::set<std::tuple<int, int, int, int>> visited;
    uint64_t rng = seed ? seed : 1;
    double best = -1, current = -1, temperature = 0.05;
    int best_at[4] = {at[0], at[1], at[2], at[3]}, done = 0;
    long long points = 1;
    for (int d = 0; d < 4; d++) points *= (long long) ax.v[d].size();
    auto key = [](const int* p) { return std::make_tuple(p[0], p[1], p[2], p[3]); };
    for (int t = 0; t < trials && (long long) visited.size() < points; t++) {
        int c[4] = {at[0], at[1], at[2], at[3]};
        if (t > 0) {
            // random step of -1, 0 or +1 along every axis, clamped to the grid (the reference steps its three
            // block sizes by random multiples of 30 / 20 / 128 and clamps them, src/autotune_sa.cpp:36-70);
            // a point seen before is stepped on from until a new one turns up
            for (int tries = 0; tries < 64; tries++) {
                for (int d = 0; d < 4; d++)
                    c[d] = std::min((int) ax.v[d].size() - 1, std::max(0, at[d] + (int) (next_random(rng) % 3) - 1));
                if (!visited.count(key(c))) break;
                for (int d = 0; d < 4; d++) at[d] = c[d];  // walk through visited points
            }
            if (visited.count(key(c))) {
                // cornered: take the first unvisited point of the grid
                bool found = false;
                int q[4];
                for (q[0] = 0; q[0] < (int) ax.v[0].size() && !found; q[0]++)
                    for (q[1] = 0; q[1] < (int) ax.v[1].size() && !found; q[1]++)
                        for (q[2] = 0; q[2] < (int) ax.v[2].size() && !found; q[2]++)
                            for (q[3] = 0; q[3] < (int) ax.v[3].size() && !found; q[3]++)
                                if (!visited.count(key(q))) {
                                    for (int d = 0; d < 4; d++) c[d] = q[d];
                                    found = true;
                                }
            }
        }
        visited.insert(key(c));
        const int values[4] = {ax.v[0][c[0]], ax.v[1][c[1]], ax.v[2][c[2]], ax.v[3][c[3]]};
        const double ms = cost(values, user);
        done++;
        if (ms <= 0) continue;  // the point is not valid for this shape
        if (best < 0 || ms < best) {
            best = ms;
            for (int d = 0; d < 4; d++) best_at[d] = c[d];
        }
        const bool accept = current < 0 || ms < current ||
                            (double) (next_random(rng) >> 11) / 9007199254740992.0 < std::exp(-(ms - current) / (current * temperature));
        if (accept) {
            current = ms;
            for (int d = 0; d < 4; d++) at[d] = c[d];
        }
        temperature *= 0.9;
    }
    if (best < 0) return -1;
    for (int d = 0; d < 4; d++) best_values[d] = ax.v[d][best_at[d]];
    if (best_ms) *best_ms = (float) best;
    if (evaluated) *evaluated = done;
    return 0;
}

// axes: 0 tile width, 1 cluster shape, 2 band, 3 K pieces; the rule's own choice is the start
Axes shape_axes(int M, int N, int K, bool with_clusters) {
    Axes ax;
    if (N > 128) ax.v[0] = {128, 256};
    else ax.v[0] = {128};
    const int rule_w = (N > 128) ? 256 : 128;
    if (!with_clusters) ax.v[1] = {0};
    else if (M > 128) ax.v[1] = {1, 2};
    else ax.v[1] = {2};
    const long long p256 = (M + 255) / 256 * 256LL, p128 = (M + 127) / 128 * 128LL;
    const int rule_c = !with_clusters ? 0 : ((M > 128 && p256 * 100 <= p128 * 107) ? 1 : 2);
    const int tiles_m = (M + 127) / 128;
    for (int b : {2, 4, 8, 16})
        if (b <= std::max(2, tiles_m) || b == 2) ax.v[2].push_back(b);
    const int kblocks = (K + 31) / 32;
    ax.v[3].push_back(0);  // 0 = the cost model of the library decides
    for (int s : {1, 2, 3, 4, 6, 8, 12, 16, 24, 32})
        if (s <= kblocks / 8 || s == 1) ax.v[3].push_back(s);
    ax.start[0] = (int) (std::find(ax.v[0].begin(), ax.v[0].end(), rule_w) - ax.v[0].begin());
    ax.start[1] = (int) (std::find(ax.v[1].begin(), ax.v[1].end(), rule_c) - ax.v[1].begin());
    if (ax.start[1] == (int) ax.v[1].size()) ax.start[1] = 0;
    ax.start[2] = (int) (std::find(ax.v[2].begin(), ax.v[2].end(), 8) - ax.v[2].begin());
    if (ax.start[2] == (int) ax.v[2].size()) ax.start[2] = (int) ax.v[2].size() - 1;
    ax.start[3] = 0;
    return ax;
}

struct Cost3 { cakeb200_tune_cost fn; void* user; };
double call_cost3(const int* v, void* u) { const Cost3* c = (const Cost3*) u; return c->fn(v[0], v[2], v[3], c->user); }
struct Cost4 { cakeb200_tune_cost_shape fn; void* user; };
double call_cost4(const int* v, void* u) { const Cost4* c = (const Cost4*) u; return c->fn(v[0], v[1], v[2], v[3], c->user); }
}  // namespace

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
    g_cache[ShapeKey(M, N, K, sched)] = {tile_n, 0, band, k_pieces, ms};
    return CAKEB200_OK;
}

int cakeb200_tune_put_shape(int M, int N, int K, int sched, int tile_n, int cluster, int band, int k_pieces, float ms) {
    if (cluster < 0 || cluster > 2) {
        set_error("cakeb200_tune_put_shape: cluster is 0 (rule), 1 (pairs of SMs) or 2 (single SMs)");
        return CAKEB200_ERR_ARG;
    }
    const int rc = cakeb200_tune_put(M, N, K, sched, tile_n, band, k_pieces, ms);
    if (rc) return rc;
    std::lock_guard<std::mutex> lock(g_mutex);
    g_cache[ShapeKey(M, N, K, sched)].cluster = cluster;
    return CAKEB200_OK;
}

int cakeb200_tune_get_shape(int M, int N, int K, int sched, int* tile_n, int* cluster, int* band, int* k_pieces, float* ms) {
    const int found = cakeb200_tune_get(M, N, K, sched, tile_n, band, k_pieces, ms);
    if (found && cluster) {
        std::lock_guard<std::mutex> lock(g_mutex);
        auto it = g_cache.find(ShapeKey(M, N, K, sched));
        *cluster = it == g_cache.end() ? 0 : it->second.cluster;
    }
    return found;
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
    Cost3 c = {cost, user};
    int best[4];
    if (search_grid(shape_axes(M, N, K, false), trials, seed, call_cost3, &c, best, best_ms, evaluated)) {
        set_error("cakeb200_tune_search: no valid point");
        return CAKEB200_ERR_ARG;
    }
    *tile_n = best[0]; *band = best[2]; *k_pieces = best[3];
    return CAKEB200_OK;
}

int cakeb200_tune_search_shape(int M, int N, int K, int sm_count, int trials, unsigned long long seed, cakeb200_tune_cost_shape cost,
                               void* user, int* tile_n, int* cluster, int* band, int* k_pieces, float* best_ms, int* evaluated) {
    if (M <= 0 || N <= 0 || K <= 0 || sm_count <= 0 || trials < 1 || !cost || !tile_n || !cluster || !band || !k_pieces) {
        set_error("cakeb200_tune_search_shape: bad argument");
        return CAKEB200_ERR_ARG;
    }
    Cost4 c = {cost, user};
    int best[4];
    if (search_grid(shape_axes(M, N, K, true), trials, seed, call_cost4, &c, best, best_ms, evaluated)) {
        set_error("cakeb200_tune_search_shape: no valid point");
        return CAKEB200_ERR_ARG;
    }
    *tile_n = best[0]; *cluster = best[1]; *band = best[2]; *k_pieces = best[3];
    return CAKEB200_OK;
}

}  // extern "C"
