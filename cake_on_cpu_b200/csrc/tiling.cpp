// Host-side block sizing and schedule derivation.
//
// Same arithmetic as the reference's get_cache_dims / derive_schedule /
// init_block_dims (src/block_sizing.cpp:304-595): callers that size their
// packed buffers from these numbers, or that pass a cake_cntx_t with CPU-style
// cache sizes, get identical block dimensions.  On a B200 context the three
// "cache" levels are shared memory per SM, the device L2 and HBM.
#include <cmath>
#include <cstring>

#include "cake_b200.h"

namespace {

inline int ceil_ratio(int a, int b) { return (int) std::ceil(((double) a) / b); }

inline int snap_down(int v, int q) {
    v -= v % q;
    return v ? v : q;
}

struct CacheDims {
    int m_c, k_c, n_c, sch;
};

CacheDims cache_dims(int M, int N, int K, int p, cakeb200_cntx* cx, int sch, int mcu, int kcu, int ncu) {
    const int mr = cx->mr, nr = cx->nr;
    const float elem = 4.0f;
    // L2 >= 2*(mc*kc + kc*nr) + 2*mc*nr with mc == kc  (src/block_sizing.cpp:316-321)
    const int b = 2 * nr;
    int mc_l2 = (int) ((-b + std::sqrt(b * b + 4 * (((double) cx->L2) / (2 * elem)))) / 2.0);
    mc_l2 -= mc_l2 % mr;
    // L3 >= 2*(p*mc*kc + a*p*mc*kc) + 2*p*mc*a*p*mc  (src/block_sizing.cpp:324-331)
    int mc_l3 = (int) std::sqrt((((double) cx->L3) / (2 * elem)) / (cx->ncores * (1 + 1.0 + 1.0 * cx->ncores)));
    mc_l3 -= mc_l3 % mr;
    cx->alpha_n = ((double) mc_l3) / mc_l2;

    int mc = mc_l2;
    if (M < p * mr) {
        mc = mr;
    } else if (M < p * mc_l2) {
        const int share = M / p;
        mc = share < mr ? mr : share + (mr - (share % mr));
    }

    CacheDims d;
    d.sch = (sch == CAKEB200_SCHED_NA) ? cakeb200_derive_schedule(M, N, K, p, mc, cx) : sch;
    if (mcu && ncu && kcu) {
        d.m_c = mcu; d.k_c = kcu; d.n_c = ncu;
        cx->alpha_n = 1.0;
        return d;
    }
    int nc;
    if (d.sch == CAKEB200_SCHED_NKM) {
        nc = snap_down(mc, nr);
        mc = snap_down((int) (cx->alpha_n * mc), mr);
    } else {
        nc = snap_down((int) (cx->alpha_n * p * mc), nr);
    }
    d.m_c = d.k_c = mc;
    d.n_c = nc;
    return d;
}

int m_padded(int M, int p, const cakeb200_blk_dims* x, const cakeb200_cntx* cx, int sch) {
    const int blk = (sch == CAKEB200_SCHED_MKN) ? x->m_c : p * x->m_c;
    return (M / blk) * blk + cx->mr * ceil_ratio(M % blk, cx->mr);
}

int n_padded(int N, const cakeb200_blk_dims* x, const cakeb200_cntx* cx) {
    return (N - (N % x->n_c)) + cx->nr * (int) std::ceil(((double) (N % x->n_c) / cx->nr));
}

}  // namespace

extern "C" {

int cakeb200_derive_schedule(int M, int N, int K, int p, int mc_ret, const cakeb200_cntx* cx) {
    // MEMA cut-offs (src/block_sizing.cpp:434-462); the reference stores them in float
    float m = (float) (p * mc_ret), k = m, n = m;
    const float k_cut_m = (float) ((2.0 * M) / (1.0 + (M * ((2.0 / k) - (1.0 / m)))));
    const float k_cut_n = (float) ((2.0 * N) / (1.0 + (N * ((2.0 / k) - (1.0 / n)))));
    m = n = (float) (cx->alpha_n * p * mc_ret);
    const float n_cut_m = (float) (M / (1.0 + (M * ((1.0 / n) - (1.0 / m)))));
    const float m_cut_n = (float) (N / (1.0 + (N * ((1.0 / m) - (1.0 / n)))));
    if ((float) N <= n_cut_m && (float) K <= k_cut_m) return CAKEB200_SCHED_MKN;
    if ((float) M <= m_cut_n && (float) K <= k_cut_n) return CAKEB200_SCHED_NKM;
    return CAKEB200_SCHED_KMN;
}

int cakeb200_set_schedule(int sched, int M, int N, int K) {
    if (sched != CAKEB200_SCHED_NA) return sched;
    if (M >= 2 * K && M >= N) return CAKEB200_SCHED_MKN;
    if (K >= M && K >= N) return CAKEB200_SCHED_KMN;
    if (N >= 2 * K && N >= M) return CAKEB200_SCHED_NKM;
    return CAKEB200_SCHED_KMN;
}

int cakeb200_init_block_dims(int M, int N, int K, int p, cakeb200_blk_dims* x, cakeb200_cntx* cx,
                             int sched, int mcu, int kcu, int ncu) {
    if (!x || !cx || M <= 0 || N <= 0 || K <= 0 || p <= 0 || cx->mr <= 0 || cx->nr <= 0 ||
        sched < 0 || sched > CAKEB200_SCHED_NA)
        return CAKEB200_ERR_ARG;
    std::memset(x, 0, sizeof(*x));
    const CacheDims d = cache_dims(M, N, K, p, cx, sched, mcu, kcu, ncu);
    const int mr = cx->mr, nr = cx->nr;
    x->m_c = d.m_c; x->k_c = d.k_c; x->n_c = d.n_c; x->sch = d.sch;

    // N is blocked the same way by every schedule
    x->n_pad = (N % x->n_c) ? 1 : 0;
    x->nr_rem = (int) std::ceil(((double) (N % x->n_c) / nr));
    x->n_c1 = x->nr_rem * nr;
    x->Nb = N / x->n_c + x->n_pad;
    x->N_padded = (N - (N % x->n_c)) + x->n_c1;

    if (x->sch == CAKEB200_SCHED_KMN) {
        // a CB block spans p*m_c rows; the ragged last block is spread over p_l cores
        const int span = p * x->m_c;
        x->k_pad = (K % x->k_c) ? 1 : 0;
        x->m_pad = (M % span) ? 1 : 0;
        x->mr_rem = ceil_ratio(M % span, mr);
        const int panels_per_core = ceil_ratio(x->mr_rem, p);
        x->p_l = panels_per_core ? ceil_ratio(x->mr_rem, panels_per_core) : 0;
        x->m_c1 = panels_per_core * mr;
        x->m_c1_last_core = (panels_per_core - (x->p_l * panels_per_core - x->mr_rem)) * mr;
        x->k_c1 = K % x->k_c;
        x->Mb = M / span + x->m_pad;
        x->Kb = K / x->k_c + x->k_pad;
        x->M_padded = mr * x->mr_rem + (M / span) * span;
        x->pm = p; x->pn = 1;
        return CAKEB200_OK;
    }

    // M-first and N-first give each core a k_c slice of a p*k_c deep block
    const int depth = p * x->k_c;
    x->k_pad = (K % depth) ? 1 : 0;
    x->k_rem = K % depth;
    x->k_c1 = ceil_ratio(x->k_rem, p);
    x->p_l = x->k_c1 ? ceil_ratio(x->k_rem, x->k_c1) : 0;
    x->k_c1_last_core = x->k_rem - x->k_c1 * (x->p_l - 1);
    x->Kb = K / depth + x->k_pad;
    const int span = (x->sch == CAKEB200_SCHED_MKN) ? x->m_c : p * x->m_c;
    x->m_pad = (M % span) ? 1 : 0;
    x->mr_rem = ceil_ratio(M % span, mr);
    x->m_c1 = x->mr_rem * mr;
    x->Mb = M / span + x->m_pad;
    x->M_padded = (M / span) * span + x->m_c1;
    if (x->sch == CAKEB200_SCHED_MKN) { x->pm = p; x->pn = 1; } else { x->pm = 1; x->pn = p; }
    return CAKEB200_OK;
}

size_t cakeb200_packed_A_size(int M, int K, int p, const cakeb200_blk_dims* x, const cakeb200_cntx* cx, int sched) {
    return (size_t) m_padded(M, p, x, cx, sched) * (size_t) K * sizeof(float);
}

size_t cakeb200_packed_B_size(int K, int N, int p, const cakeb200_blk_dims* x, const cakeb200_cntx* cx) {
    (void) p;
    return (size_t) K * (size_t) n_padded(N, x, cx) * sizeof(float);
}

size_t cakeb200_packed_C_size(int M, int N, int p, const cakeb200_blk_dims* x, const cakeb200_cntx* cx, int sched) {
    return (size_t) m_padded(M, p, x, cx, sched) * (size_t) n_padded(N, x, cx) * sizeof(float);
}

// Which devices a host-pointer product with p > 1 is spread over (host logic, no device needed).
int cakeb200_select_devices(const int* cc_major, int n_devices, int current, int p, int cap, int M, int* out) {
    if (!cc_major || !out || n_devices <= 0 || current < 0 || current >= n_devices) return 0;
    int limit = p < 1 ? 1 : p;
    if (cap > 0 && cap < limit) limit = cap;
    const int by_rows = M / 512 > 1 ? M / 512 : 1;  // at least 512 rows of C per device
    if (by_rows < limit) limit = by_rows;
    int got = 0;
    if (cc_major[current] == 10) out[got++] = current;
    for (int d = 0; d < n_devices && got < limit; d++)
        if (d != current && cc_major[d] == 10) out[got++] = d;
    return got;
}

}  // extern "C"
