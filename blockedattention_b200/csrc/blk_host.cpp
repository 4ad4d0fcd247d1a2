// Host side of libblkattn that needs no CUDA: error text, index helpers,
// multi-GPU partitioners and the segment scheduler that bins segments onto the
// kernels.  Everything here runs (and is tested) on a machine without a GPU.
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <map>
#include <numeric>
#include <queue>
#include <string>

#include "blk_internal.h"

static thread_local std::string g_last_error;

void blk_set_error(const std::string& msg) { g_last_error = msg; }

bool blk_env_flag(const char* name) {
    const char* v = std::getenv(name);
    return v && v[0] && std::strcmp(v, "0") != 0;
}

extern "C" const char* blk_last_error(void) { return g_last_error.c_str(); }
extern "C" const char* blk_version(void) { return "blkattn-b200 0.1 (sm_100a)"; }

// ---------------------------------------------------------------------------
// index helpers
// ---------------------------------------------------------------------------
static bool mul_ok(int64_t a, int64_t b, int64_t* out) {
    return !__builtin_mul_overflow(a, b, out);
}

extern "C" int blk_offsets_from_lists(const int64_t* M, const int64_t* N, const int64_t* K,
                                      int64_t S, int64_t* a1, int64_t* a2, int64_t* ao) {
    if (S < 0 || (S > 0 && (!M || !N || !K)) || !a1 || !a2 || !ao) {
        blk_set_error("blk_offsets_from_lists: null argument");
        return BLK_ERR_INVALID;
    }
    a1[0] = a2[0] = ao[0] = 0;
    for (int64_t s = 0; s < S; ++s) {
        int64_t mk, nk, mn;
        if (M[s] < 0 || N[s] < 0 || K[s] < 0 || !mul_ok(M[s], K[s], &mk) || !mul_ok(N[s], K[s], &nk) ||
            !mul_ok(M[s], N[s], &mn) || __builtin_add_overflow(a1[s], mk, &a1[s + 1]) ||
            __builtin_add_overflow(a2[s], nk, &a2[s + 1]) || __builtin_add_overflow(ao[s], mn, &ao[s + 1])) {
            blk_set_error("blk_offsets_from_lists: negative extent or int64 overflow at segment " + std::to_string(s));
            return BLK_ERR_INVALID;
        }
    }
    return BLK_OK;
}

extern "C" int blk_softmax_offsets(const int64_t* rows, const int64_t* cols, int64_t S, int64_t* acc) {
    if (S < 0 || (S > 0 && (!rows || !cols)) || !acc) {
        blk_set_error("blk_softmax_offsets: null argument");
        return BLK_ERR_INVALID;
    }
    acc[0] = 0;
    for (int64_t s = 0; s < S; ++s) {
        int64_t rc;
        if (rows[s] < 0 || cols[s] < 0 || !mul_ok(rows[s], cols[s], &rc) ||
            __builtin_add_overflow(acc[s], rc, &acc[s + 1])) {
            blk_set_error("blk_softmax_offsets: negative extent or int64 overflow at segment " + std::to_string(s));
            return BLK_ERR_INVALID;
        }
    }
    return BLK_OK;
}

static uint64_t isqrt_u128(unsigned __int128 v) {
    if (v == 0) return 0;
    long double approx = std::sqrt((long double)v);
    uint64_t r = (uint64_t)approx;
    while ((unsigned __int128)r * r > v) --r;
    while ((unsigned __int128)(r + 1) * (r + 1) <= v) ++r;
    return r;
}

extern "C" int blk_lists_from_offsets(const int64_t* a1, const int64_t* a2, const int64_t* ao, int64_t S,
                                      int64_t* M, int64_t* N, int64_t* K) {
    if (S < 0 || (S > 0 && (!a1 || !a2 || !ao || !M || !N || !K))) {
        blk_set_error("blk_lists_from_offsets: null argument");
        return BLK_ERR_INVALID;
    }
    for (int64_t s = 0; s < S; ++s) {
        const int64_t mk = a1[s + 1] - a1[s], nk = a2[s + 1] - a2[s], mn = ao[s + 1] - ao[s];
        if (mk <= 0 || nk <= 0 || mn <= 0) {
            blk_set_error("blk_lists_from_offsets: segment " + std::to_string(s) +
                          " has an empty extent; (M,N,K) cannot be recovered from offsets");
            return BLK_ERR_INVALID;
        }
        const unsigned __int128 num = (unsigned __int128)mk * (unsigned __int128)mn;
        bool ok = (num % (unsigned __int128)nk) == 0;
        uint64_t m = 0;
        if (ok) {
            const unsigned __int128 m2 = num / (unsigned __int128)nk;
            m = isqrt_u128(m2);
            ok = m > 0 && (unsigned __int128)m * m == m2 && mn % (int64_t)m == 0 && mk % (int64_t)m == 0 &&
                 (unsigned __int128)(mn / (int64_t)m) * (unsigned __int128)(mk / (int64_t)m) == (unsigned __int128)nk;
        }
        if (!ok) {
            blk_set_error("blk_lists_from_offsets: offsets of segment " + std::to_string(s) +
                          " are not those of an (M,N,K) segment");
            return BLK_ERR_INVALID;
        }
        M[s] = (int64_t)m;
        N[s] = mn / (int64_t)m;
        K[s] = mk / (int64_t)m;
    }
    return BLK_OK;
}

// ---------------------------------------------------------------------------
// partitioning
// ---------------------------------------------------------------------------
extern "C" int blk_segment_cost(const int64_t* M, const int64_t* N, const int64_t* K, int64_t S, int64_t H,
                                int in_bytes, int out_bytes, double flops_per_s, double bytes_per_s,
                                double* cost) {
    if (S < 0 || (S > 0 && (!M || !N || !K || !cost)) || flops_per_s <= 0 || bytes_per_s <= 0 || H < 0) {
        blk_set_error("blk_segment_cost: bad argument");
        return BLK_ERR_INVALID;
    }
    for (int64_t s = 0; s < S; ++s) {
        const double m = (double)M[s], n = (double)N[s], k = (double)K[s];
        const double fl = 2.0 * m * n * k;
        const double by = (m + n) * k * in_bytes + m * n * out_bytes;
        cost[s] = (double)H * std::max(fl / flops_per_s, by / bytes_per_s);
    }
    return BLK_OK;
}

// Number of ranges a greedy left-to-right fill needs when no range may exceed cap.
static int64_t ranges_needed(const double* cost, int64_t S, double cap) {
    int64_t cnt = 1;
    double cur = 0;
    for (int64_t s = 0; s < S; ++s) {
        if (cost[s] > cap) return INT64_MAX;
        if (cur + cost[s] > cap) {
            ++cnt;
            cur = 0;
        }
        cur += cost[s];
    }
    return cnt;
}

extern "C" int blk_partition_contiguous(const double* cost, int64_t S, int R, int64_t* bounds) {
    if (S < 0 || R < 1 || !bounds || (S > 0 && !cost)) {
        blk_set_error("blk_partition_contiguous: bad argument");
        return BLK_ERR_INVALID;
    }
    double total = 0, mx = 0;
    for (int64_t s = 0; s < S; ++s) {
        if (!(cost[s] >= 0)) {
            blk_set_error("blk_partition_contiguous: negative or NaN cost");
            return BLK_ERR_INVALID;
        }
        total += cost[s];
        mx = std::max(mx, cost[s]);
    }
    // bisection on the bottleneck value
    double lo = std::max(mx, total / R), hi = total;
    if (ranges_needed(cost, S, lo) <= R) hi = lo;
    for (int it = 0; it < 100 && hi - lo > 1e-10 * hi; ++it) {
        const double mid = 0.5 * (lo + hi);
        if (ranges_needed(cost, S, mid) <= R) hi = mid; else lo = mid;
    }
    // materialise the split for cap = hi: greedy fill, then spread empty tail ranges
    std::vector<int64_t> b(R + 1, S);
    b[0] = 0;
    {
        int r = 0;
        double cur = 0;
        int64_t start = 0;
        const double cap = hi * (1 + 1e-12);
        for (int64_t s = 0; s < S; ++s) {
            if (cur + cost[s] > cap && s > start && r + 1 < R) {  // s > start: never emit an empty range
                b[++r] = s;
                cur = 0;
                start = s;
            }
            cur += cost[s];
        }
        for (int q = r + 1; q <= R; ++q) b[q] = S;
    }
    for (int r = 0; r <= R; ++r) bounds[r] = b[r];
    return BLK_OK;
}

extern "C" int blk_partition_lpt(const double* cost, int64_t S, int R, int32_t* owner) {
    if (S < 0 || R < 1 || (S > 0 && (!cost || !owner))) {
        blk_set_error("blk_partition_lpt: bad argument");
        return BLK_ERR_INVALID;
    }
    std::vector<int64_t> order(S);
    std::iota(order.begin(), order.end(), 0);
    std::stable_sort(order.begin(), order.end(), [&](int64_t a, int64_t b) { return cost[a] > cost[b]; });
    typedef std::pair<double, int> Load;  // (load, rank); smallest load first, ties to the lowest rank
    std::priority_queue<Load, std::vector<Load>, std::greater<Load>> pq;
    for (int r = 0; r < R; ++r) pq.push(Load(0.0, r));
    for (int64_t i = 0; i < S; ++i) {
        Load l = pq.top();
        pq.pop();
        owner[order[i]] = l.second;
        l.first += cost[order[i]];
        pq.push(l);
    }
    return BLK_OK;
}

// ---------------------------------------------------------------------------
// scheduler
// ---------------------------------------------------------------------------
static int elem_bytes(int dtype) { return dtype == BLK_F32 ? 4 : 2; }

// Widest access class usable at `off` with row pitch `pitch` on every head of
// a (H, D) buffer of es-byte elements: 2 -> 16 bytes, 1 -> 4 bytes (a pair of
// 16-bit elements; one fp32 element), 0 -> one element.
static int access_class(int64_t H, int64_t D, int64_t off, int64_t pitch, int es) {
    const int64_t v16 = 16 / es, v4 = es == 2 ? 2 : 1;  // powers of two: masks instead of divisions
    const int64_t bits = (H <= 1 ? 0 : D) | off | pitch;
    auto ok = [&](int64_t v) { return (bits & (v - 1)) == 0; };
    if (ok(v16)) return 2;
    if (ok(v4)) return 1;
    return 0;
}

// Stable ascending order of (key, payload) records by their 64-bit keys: counting sort byte by byte, skipping the
// bytes on which all keys agree.  A comparison sort of a few thousand work items spends its time in mispredicted
// branches; this takes a fifth of it.
static void sort_by_key(std::vector<std::pair<uint64_t, int32_t>>& v) {
    uint64_t any = 0, all = ~(uint64_t)0;
    for (const auto& e : v) { any |= e.first; all &= e.first; }
    const uint64_t differ = any ^ all;
    std::vector<std::pair<uint64_t, int32_t>> tmp(v.size());
    for (int shift = 0; shift < 64; shift += 8) {
        if (((differ >> shift) & 255) == 0) continue;
        size_t start[256] = {0};
        for (const auto& e : v) ++start[(e.first >> shift) & 255];
        size_t at = 0;
        for (size_t& c : start) { const size_t n = c; c = at; at += n; }
        for (const auto& e : v) tmp[start[(e.first >> shift) & 255]++] = e;
        v.swap(tmp);
    }
}

// The distinct (K, residue) keys of an operand, numbered in the order of first appearance, behind a small
// open-addressing table (a batch of mixed contraction lengths has dozens of keys, looked up twice per segment).
struct BlkKeyTable {
    std::vector<std::pair<int64_t, int64_t>> keys;
    std::vector<int32_t> slots;  // key number or -1; a power of two, at most half full
    static size_t hash(int64_t k, int64_t r) {
        return (size_t)(((uint64_t)k * 0x9E3779B97F4A7C15ull) ^ ((uint64_t)r * 0xC2B2AE3D27D4EB4Full)) >> 20;
    }
    void place(int32_t i) {
        size_t h = hash(keys[i].first, keys[i].second) & (slots.size() - 1);
        while (slots[h] >= 0) h = (h + 1) & (slots.size() - 1);
        slots[h] = i;
    }
    int32_t number_of(int64_t k, int64_t r) {
        if (slots.empty()) slots.assign(64, -1);
        for (size_t h = hash(k, r) & (slots.size() - 1);; h = (h + 1) & (slots.size() - 1)) {
            const int32_t i = slots[h];
            if (i < 0) break;
            if (keys[i].first == k && keys[i].second == r) return i;
        }
        keys.push_back(std::make_pair(k, r));
        if (keys.size() * 2 > slots.size()) {
            slots.assign(slots.size() * 2, -1);
            for (size_t i = 0; i < keys.size(); ++i) place((int32_t)i);
        } else {
            place((int32_t)keys.size() - 1);
        }
        return (int32_t)keys.size() - 1;
    }
};

static int validate_offsets(const char* what, const std::vector<int64_t>& acc, const std::vector<int64_t>& need,
                            int64_t S) {
    if (acc[0] < 0) {
        blk_set_error(std::string(what) + ": first offset is negative");
        return BLK_ERR_INVALID;
    }
    for (int64_t s = 0; s < S; ++s) {
        if (acc[s + 1] < acc[s] || acc[s + 1] - acc[s] < need[s]) {
            blk_set_error(std::string(what) + ": offsets of segment " + std::to_string(s) +
                          " do not leave room for its extents (need " + std::to_string(need[s]) + " elements, have " +
                          std::to_string(acc[s + 1] - acc[s]) + ")");
            return BLK_ERR_INVALID;
        }
    }
    return BLK_OK;
}

int blk_build_gemm_schedule(blk_plan* p) {
    const int64_t S = p->S;
    const int es_in = elem_bytes(p->dtype_in), es_out = elem_bytes(p->dtype_out);
    std::vector<int64_t> needA(S), needB(S), needC(S);
    for (int64_t s = 0; s < S; ++s) {
        const int64_t m = p->M[s], n = p->N[s], k = p->K[s];
        if (m < 0 || n < 0 || k < 0 || m > INT32_MAX / 2 || n > INT32_MAX / 2 || k > INT32_MAX / 2) {
            blk_set_error("gemm plan: extent of segment " + std::to_string(s) + " is negative or exceeds 2^30");
            return BLK_ERR_INVALID;
        }
        if (!mul_ok(m, k, &needA[s]) || !mul_ok(n, k, &needB[s]) || !mul_ok(m, n, &needC[s])) {
            blk_set_error("gemm plan: int64 overflow");
            return BLK_ERR_INVALID;
        }
        if (p->attn) needC[s] = needA[s];  // an attention plan's output holds result rows, not scores
    }
    int rc;
    if ((rc = validate_offsets("gemm plan: mat1Accum", p->a1, needA, S)) != BLK_OK) return rc;
    if ((rc = validate_offsets("gemm plan: mat2Accum", p->a2, needB, S)) != BLK_OK) return rc;
    if ((rc = validate_offsets("gemm plan: outAccum", p->ao, needC, S)) != BLK_OK) return rc;
    p->Dm1 = p->a1[S];
    p->Dm2 = p->a2[S];
    p->Dout = p->ao[S];

    bool allow_small = !blk_env_flag("BLK_DISABLE_SMALL");
    const bool allow_umma = !blk_env_flag("BLK_DISABLE_UMMA") && p->dtype_in != BLK_F32 && !p->ta && !p->tb &&
                            p->Dm1 % 8 == 0 && p->Dm2 % 8 == 0;
    // The tcgen05 kernel reads each operand through (K, rows, heads) views (BlkUmmaView): a segment needs the view of
    // its K that starts at its offset modulo K.  It takes the 16-bit segments that are not for the small-segment
    // kernels (too big, or a K other than theirs) whose K and offsets are multiples of 8 elements (16-byte rows for the tensor maps) and whose views are
    // among the BLK_UMMA_VIEWS per operand that carry the most work.
    // Per segment, once: whether the kernel could take it at all, its multiply-adds, and the number of its (K, residue)
    // key among the distinct keys of each operand (BlkKeyTable).
    typedef std::pair<int64_t, int64_t> Key;  // (K, residue)
    BlkKeyTable tableA, tableB;
    const std::vector<Key>&keysA = tableA.keys, &keysB = tableB.keys;
    std::vector<int32_t> keyA(allow_umma ? (size_t)S : 0, -1), keyB(allow_umma ? (size_t)S : 0, -1);
    std::vector<double> seg_work(allow_umma ? (size_t)S : 0, 0.0);
    double all_work = 0;
    // segments the small-segment kernels would take get their keys only if they end up riding along (below): a batch
    // of thousands of small graphs does not pay for keys it never uses
    auto small_shaped = [&](int64_t s) {
        return p->M[s] <= BLK_SMALL_MAXM && p->N[s] <= BLK_SMALL_MAXN && (p->K[s] == 32 || p->K[s] == 64);
    };
    auto make_keys = [&](bool small_ones) {
        for (int64_t s = 0; s < S; ++s) {
            const int64_t m = p->M[s], n = p->N[s], k = p->K[s];
            if (!small_ones) {
                seg_work[s] = (double)m * (double)n * (double)k;
                all_work += seg_work[s];
            }
            if (small_shaped(s) != small_ones) continue;
            // (rows of a view must fit 32 bits: D / k < INT32_MAX, written without the division)
            if (m > 0 && n > 0 && k >= 16 && k % 8 == 0 && p->a1[s] % 8 == 0 && p->a2[s] % 8 == 0 &&
                p->Dm1 < (int64_t)INT32_MAX * k && p->Dm2 < (int64_t)INT32_MAX * k) {
                const bool pow2 = (k & (k - 1)) == 0;
                keyA[s] = tableA.number_of(k, pow2 ? (p->a1[s] & (k - 1)) : p->a1[s] % k);
                keyB[s] = tableB.number_of(k, pow2 ? (p->a2[s] & (k - 1)) : p->a2[s] % k);
            }
        }
    };
    if (allow_umma) {
        make_keys(false);
        if (!allow_small) make_keys(true);
    }
    // a capable segment is a candidate unless the small-segment kernels take it
    auto umma_candidate = [&](int64_t s) {
        const int64_t m = p->M[s], n = p->N[s], k = p->K[s];
        return allow_umma && keyA[s] >= 0 &&
               (m > BLK_SMALL_MAXM || n > BLK_SMALL_MAXN || (k != 32 && k != 64) || !allow_small);
    };
    std::vector<int32_t> umma_views(allow_umma ? (size_t)S : 0, -1);  // per segment: view of A | view of B << 8, or -1
    size_t umma_segments = 0;  // segments with views
    auto select_views = [&]() {
        p->umma_K = 0;
        umma_segments = 0;
        p->umma_viewsA.clear();
        p->umma_viewsB.clear();
        std::fill(umma_views.begin(), umma_views.end(), -1);
        if (!allow_umma) return;
        std::vector<double> workA(keysA.size(), 0.0), workB(keysB.size(), 0.0);
        std::vector<char> usedA(keysA.size(), 0), usedB(keysB.size(), 0);
        for (int64_t s = 0; s < S; ++s) {
            if (!umma_candidate(s)) continue;
            workA[keyA[s]] += seg_work[s];
            workB[keyB[s]] += seg_work[s];
            usedA[keyA[s]] = usedB[keyB[s]] = 1;
        }
        // the BLK_UMMA_VIEWS keys with the most work, ties in the order of (K, residue); slot[key] = view or -1
        auto pick = [](const std::vector<Key>& keys, const std::vector<double>& work, const std::vector<char>& used,
                       std::vector<BlkUmmaView>* out, std::vector<int32_t>* slot) {
            std::vector<int32_t> order;
            for (size_t i = 0; i < keys.size(); ++i)
                if (used[i]) order.push_back((int32_t)i);
            std::sort(order.begin(), order.end(), [&](int32_t x, int32_t y) { return keys[x] < keys[y]; });
            std::stable_sort(order.begin(), order.end(), [&](int32_t x, int32_t y) { return work[x] > work[y]; });
            slot->assign(keys.size(), -1);
            for (size_t i = 0; i < order.size() && i < (size_t)BLK_UMMA_VIEWS; ++i) {
                out->push_back(BlkUmmaView{keys[order[i]].first, keys[order[i]].second});
                (*slot)[order[i]] = (int32_t)i;
            }
        };
        std::vector<int32_t> slotA, slotB;
        pick(keysA, workA, usedA, &p->umma_viewsA, &slotA);
        pick(keysB, workB, usedB, &p->umma_viewsB, &slotB);
        double taken = 0;
        for (int64_t s = 0; s < S; ++s) {
            if (!umma_candidate(s)) continue;
            const int va = slotA[keyA[s]], vb = slotB[keyB[s]];
            if (va < 0 || vb < 0) continue;
            umma_views[s] = va | (vb << 8);
            taken += seg_work[s];
            ++umma_segments;
        }
        // A separate launch pays only if it takes a real share of the batch: when the segments it could take
        // carry under a tenth of all multiply-adds, they stay with the staged kernel.
        if (taken == 0 || (taken < 0.1 * all_work && !blk_env_flag("BLK_FORCE_UMMA"))) {
            std::fill(umma_views.begin(), umma_views.end(), -1);
            p->umma_viewsA.clear();
            p->umma_viewsB.clear();
            umma_segments = 0;
        } else if (p->umma_viewsA.size() == 1 && p->umma_viewsB.size() == 1 && p->umma_viewsA[0].residue == 0 &&
                   p->umma_viewsB[0].residue == 0) {
            p->umma_K = (int)p->umma_viewsA[0].K;
        } else {
            p->umma_K = -1;
        }
    };
    select_views();
    // A launch of the small-segment kernel of its own pays only for enough segments: when the tcgen05 kernel is
    // launched anyway and fewer than BLK_SMALL_MIN_PAIRS (default 300: two per SM) pairs of a small segment and a head
    // exist, they ride along with it (those it cannot take go to the staged kernel).  Attention plans keep their packs.
    if (allow_small && allow_umma && !p->attn && !p->umma_viewsA.empty()) {
        int64_t pairs = 0, sk = 0;
        for (int64_t s = 0; s < S; ++s) {
            const int64_t m = p->M[s], n = p->N[s], k = p->K[s];
            if (m > 0 && n > 0 && m <= BLK_SMALL_MAXM && n <= BLK_SMALL_MAXN && (k == 32 || k == 64) && (sk == 0 || sk == k)) {
                sk = k;
                pairs += p->H;
            }
        }
        const char* e = std::getenv("BLK_SMALL_MIN_PAIRS");
        const int64_t min_pairs = e ? std::atoll(e) : 300;
        if (pairs < min_pairs) {
            allow_small = false;
            make_keys(true);
            select_views();
        }
    }
    // The tcgen05 kernel for a second operand stored (K, D) -- the product of a probability block with the values --
    // takes 16-bit segments whose second operand has D = 64 or 128 columns (one D per plan: the one carrying the
    // most work), whose value rows are rows of the (rows, D) view of the strip and whose result rows are 16-byte
    // aligned.  The first operand may have any row length and alignment.
    const bool allow_pv = !blk_env_flag("BLK_DISABLE_UMMA") && p->dtype_in != BLK_F32 && p->dtype_out == p->dtype_in &&
                          !p->ta && p->tb && p->epi == BLK_EPI_SCORES && p->Dm2 % 8 == 0 && p->Dout % 8 == 0 && !p->attn;
    auto pv_candidate = [&](int64_t s, int64_t D) {
        return allow_pv && p->N[s] == D && p->M[s] > 0 && p->K[s] > 0 && p->a2[s] % D == 0 && p->ao[s] % 8 == 0 &&
               p->Dm2 / D < INT32_MAX;
    };
    p->pv_D = 0;
    if (allow_pv) {
        double w64 = 0, w128 = 0, all = 0;
        for (int64_t s = 0; s < S; ++s) {
            const double wk = (double)p->M[s] * (double)p->N[s] * (double)p->K[s];
            all += wk;
            if (pv_candidate(s, 64)) w64 += wk;
            if (pv_candidate(s, 128)) w128 += wk;
        }
        const double best = std::max(w64, w128);
        if (best > 0 && (best >= 0.1 * all || blk_env_flag("BLK_FORCE_UMMA"))) p->pv_D = w128 >= w64 ? 128 : 64;
    }
    p->segs.resize(S);
    p->umma_items.reserve(umma_segments + umma_segments / 2);  // an item per 128-row block (or tile): a first guess
    p->flops = p->bytes = 0;
    std::vector<int64_t> small_segs;  // segments of the small bin, in batch order
    for (int64_t s = 0; s < S; ++s) {
        const int64_t m = p->M[s], n = p->N[s], k = p->K[s];
        BlkSeg& sd = p->segs[s];
        sd.offA = p->a1[s];
        sd.offB = p->a2[s];
        sd.offC = p->ao[s];
        sd.M = (int32_t)m;
        sd.N = (int32_t)n;
        sd.K = (int32_t)k;
        const int cA = access_class(p->H, p->Dm1, sd.offA, p->ta ? m : k, es_in);
        const int cB = access_class(p->H, p->Dm2, sd.offB, p->tb ? n : k, es_in);
        sd.clsIn = (uint8_t)std::min(cA, cB);
        sd.clsOut = (uint8_t)access_class(p->H, p->Dout, sd.offC, n, es_out);
        sd.pad[0] = sd.pad[1] = 0;
        p->flops += 2.0 * (double)p->H * (double)m * (double)n * (double)k;
        p->bytes += (double)p->H * ((double)(m + n) * (double)k * es_in + (double)m * (double)n * es_out);
        if (m == 0 || n == 0) continue;

        if (p->dtype_in == BLK_F32) {
            const int32_t tms = (int32_t)((m + BLK_SIMT_BM - 1) / BLK_SIMT_BM);
            const int32_t tns = (int32_t)((n + BLK_SIMT_BN - 1) / BLK_SIMT_BN);
            for (int32_t tm = 0; tm < tms; ++tm)
                for (int32_t tn = 0; tn < tns; ++tn) p->simt_items.push_back(BlkTileItem{(int32_t)s, tm, tn, 1});
            continue;
        }
        // Packed small-segment kernel: one warp per (segment, head).
        const bool small_ok = allow_small && !p->ta && !p->tb && n <= BLK_SMALL_MAXN && m <= BLK_SMALL_MAXM &&
                              (k == 32 || k == 64) && sd.clsIn == 2 &&
                              (p->small_K == 0 || p->small_K == (int)k);
        if (small_ok) {
            p->small_K = (int)k;
            small_segs.push_back(s);  // packs or per-warp items: decided below, once the whole bin is known
            continue;
        }
        if (p->pv_D != 0 && pv_candidate(s, p->pv_D)) {
            for (int64_t tm = 0; tm * BLK_UMMA_BM < m; ++tm)
                p->pv_items.push_back(BlkPvItem{sd.offA + tm * BLK_UMMA_BM * k, sd.offC + tm * BLK_UMMA_BM * n,
                                                (int32_t)(sd.offB / n), (int32_t)(m - tm * BLK_UMMA_BM), (int32_t)k, 0});
            continue;
        }
        if (allow_umma && umma_views[s] >= 0) {
            const int32_t tms = (int32_t)((m + BLK_UMMA_BM - 1) / BLK_UMMA_BM);
            const int64_t ra = p->umma_viewsA[umma_views[s] & 255].residue, rb = p->umma_viewsB[umma_views[s] >> 8].residue;
            // Scores only: one item per 256-column chunk of a row block when the contraction is long (a k loop of
            // 8 blocks or more keeps a CTA busy for longer than it takes to start an item), so that a batch of few big
            // segments still fills the SMs and the CTAs running at one time share a few segments' operands in L2.
            // With the fused softmax an item is the whole row block.
            const int32_t chunks = (int32_t)((n + 255) / 256);
            const bool per_chunk = p->epi != BLK_EPI_SOFTMAX && k >= 512 && chunks > 1;
            for (int32_t tm = 0; tm < tms; ++tm)
                for (int32_t c = 0; c < (per_chunk ? chunks : 1); ++c)
                    p->umma_items.push_back(BlkUmmaItem{umma_views[s], tm, (int32_t)((sd.offA - ra) / k + (int64_t)tm * BLK_UMMA_BM),
                                                        (int32_t)((sd.offB - rb) / k), sd.offC, (int32_t)m, (int32_t)n, (int32_t)k,
                                                        per_chunk ? c : 0, per_chunk ? 1 : 0, 0});
            continue;
        }
        const int32_t tms = (int32_t)((m + BLK_TILE_BM - 1) / BLK_TILE_BM);
        const int32_t tns = (int32_t)((n + BLK_TILE_BN - 1) / BLK_TILE_BN);
        for (int32_t tm = 0; tm < tms; ++tm) {
            if (p->epi == BLK_EPI_SOFTMAX) {
                p->tile_items.push_back(BlkTileItem{(int32_t)s, tm, 0, tns});
            } else {
                for (int32_t tn = 0; tn < tns; ++tn) p->tile_items.push_back(BlkTileItem{(int32_t)s, tm, tn, 1});
            }
        }
    }
    // Persistent CTAs of the tcgen05 kernel take items with a fixed stride (alternating direction from round to
    // round): heaviest first evens the tails.  What an item costs that kernel is its number of 256-column chunks --
    // twice that when the fused softmax takes two sweeps (more than two chunks) -- whatever the rows of the block;
    // ordering by rows x columns instead left the CTAs 5 % apart on a long-tailed batch.
    const bool two_sweeps = p->epi == BLK_EPI_SOFTMAX;
    auto umma_cost = [two_sweeps](const BlkUmmaItem& a) {
        const int64_t chunks = a.nch ? a.nch : ((int64_t)a.N + 255) / 256;
        const int64_t rows = std::min(a.M - a.tm * BLK_UMMA_BM, BLK_UMMA_BM);
        const int64_t kblocks = ((int64_t)a.K + 63) / 64;  // a chunk costs the epilogue (about four k-blocks' worth) plus its k-blocks
        const int64_t work = std::min<int64_t>((two_sweeps && chunks > 2 ? 2 * chunks : chunks) * (4 + kblocks), (1 << 27) - 1);
        return (work << 36) + ((int64_t)a.N << 8) + rows;  // below 2^63: the ordering key is its complement
    };
    {
        // the cost of an item is computed once, the (cost, position) pairs are sorted and the items moved into that order
        std::vector<std::pair<uint64_t, int32_t>> order(p->umma_items.size());
        for (size_t i = 0; i < order.size(); ++i)
            order[i] = std::make_pair(~(uint64_t)umma_cost(p->umma_items[i]), (int32_t)i);
        sort_by_key(order);  // descending cost, ties in the order of generation (a stable sort)
        // in place, cycle by cycle: position i receives the item that was at order[i].second
        BlkUmmaItem* const items = p->umma_items.data();
        for (size_t i = 0; i < order.size(); ++i) {
            if (order[i].second == (int32_t)i) continue;
            const BlkUmmaItem first = items[i];
            size_t to = i;
            for (;;) {
                const size_t from = (size_t)order[to].second;
                order[to].second = (int32_t)to;  // done
                if (from == i) { items[to] = first; break; }
                items[to] = items[from];
                to = from;
            }
        }
    }
    p->umma_long_rows = 0;
    for (const BlkUmmaItem& it : p->umma_items)
        if (it.N > 512) p->umma_long_rows = 1;
    // longest contractions first for the same reason
    std::stable_sort(p->pv_items.begin(), p->pv_items.end(), [](const BlkPvItem& a, const BlkPvItem& b) { return a.K > b.K; });
    // K = 64 with 16-bit output: the small segments run on the pipelined kernel, grouped into packs of
    // consecutive segments whose operands are contiguous in memory (one bulk copy per operand per pack).
    p->small_pipe = 0;
    // The pack kernel fetches operands through (64, rows, heads) tensor maps: every small segment and every head
    // strip must start on a row of that view.
    bool rows_ok = p->Dm1 % 64 == 0 && p->Dm2 % 64 == 0 && p->Dm1 / 64 < INT32_MAX && p->Dm2 / 64 < INT32_MAX;
    for (size_t q = 0; rows_ok && q < small_segs.size(); ++q)
        rows_ok = p->segs[small_segs[q]].offA % 64 == 0 && p->segs[small_segs[q]].offB % 64 == 0;
    if (p->small_K == 64 && p->dtype_out != BLK_F32 && rows_ok && !blk_env_flag("BLK_DISABLE_PIPE") && !small_segs.empty()) {
        p->small_pipe = 1;
        const int pack_rows = p->attn ? BLK_PACK_ROWS_ATTN : BLK_PACK_ROWS;
        // First the packs in batch order (extents, cost and the first segment of each), then the block table written
        // once, pack by pack, heaviest pack first: persistent CTAs take packs with a fixed stride.
        std::vector<BlkPack> pk;
        std::vector<std::pair<double, int32_t>> order;  // (-cost, pack)
        std::vector<int32_t> first_seg;                 // index into small_segs
        pk.reserve(small_segs.size() / 4 + 1);
        order.reserve(small_segs.size() / 4 + 1);
        first_seg.reserve(small_segs.size() / 4 + 2);
        size_t nblocks = 0;
        for (size_t q = 0; q < small_segs.size(); ++q) {
            const BlkSeg& sd = p->segs[small_segs[q]];
            const int32_t mblocks = (sd.M + 15) / 16;  // one block per 16 first-operand rows of the segment
            bool extend = false;
            if (!pk.empty()) {
                const BlkPack& t = pk.back();
                extend = t.offA + (int64_t)t.rowsA * 64 == sd.offA && t.offB + (int64_t)t.rowsB * 64 == sd.offB &&
                         t.rowsA + sd.M <= pack_rows && t.rowsB + sd.N <= pack_rows &&
                         t.nblocks + mblocks <= BLK_PACK_BLOCKS;
            }
            if (!extend) {
                pk.push_back(BlkPack{sd.offA, sd.offB, 0, 0, 0, 0});
                order.push_back(std::make_pair(-0.0, (int32_t)order.size()));
                first_seg.push_back((int32_t)q);
            }
            BlkPack& t = pk.back();
            t.rowsA += sd.M;
            t.rowsB += sd.N;
            t.nblocks += mblocks;
            nblocks += (size_t)mblocks;
            order.back().first -= (double)sd.M * sd.N + (double)(sd.M + sd.N) * 64;
        }
        first_seg.push_back((int32_t)small_segs.size());
        std::sort(order.begin(), order.end());  // descending cost, equal costs in batch order
        p->packs.resize(pk.size());
        // the block table is read in 16-record pieces: 16 records of slack (zeros) behind the last pack
        p->pack_blocks.assign(nblocks + BLK_PACK_BLOCKS, BlkPackBlock{0, 0, 0, 0, 0, 0, 0});
        BlkPackBlock* dst = p->pack_blocks.data();
        const BlkSeg* const segs = p->segs.data();
        const int64_t* const small = small_segs.data();
        const bool attn = p->attn != 0;
        for (size_t i = 0; i < order.size(); ++i) {
            const int32_t pi = order[i].second;
            BlkPack t = pk[pi];
            t.first_block = (int32_t)(dst - p->pack_blocks.data());
            // consumers claim blocks in table order: widest segment first, equal widths in batch order (at most
            // BLK_PACK_BLOCKS segments, every one has a block: insertion sort)
            struct Member { int32_t N, q, rowA, rowB; } member[BLK_PACK_BLOCKS];
            int32_t rowsA = 0, rowsB = 0, members = 0;
            for (int32_t q = first_seg[pi]; q < first_seg[pi + 1]; ++q) {
                const BlkSeg& sd = segs[small[q]];
                int32_t at = members++;
                for (; at > 0 && member[at - 1].N < sd.N; --at) member[at] = member[at - 1];
                member[at] = Member{sd.N, q, rowsA, rowsB};
                rowsA += sd.M;
                rowsB += sd.N;
            }
            BlkPackBlock* out = dst;
            for (int32_t e = 0; e < members; ++e) {
                const BlkSeg& sd = segs[small[member[e].q]];
                // output of a block: 16 x N scores, or for an attention plan 16 x 64 result rows
                const int64_t step = 16 * (int64_t)(attn ? 64 : sd.N);
                for (int32_t mb = 0; mb * 16 < sd.M; ++mb)
                    *out++ = BlkPackBlock{sd.offC + mb * step, member[e].rowA + 16 * mb, member[e].rowB,
                                          std::min<int32_t>(16, sd.M - 16 * mb), sd.N, t.nblocks, 0};
            }
            dst += t.nblocks;
            p->packs[i] = t;
        }
    } else {
        // One warp per (segment, head).  Persistent warps take the items in list order with a fixed stride: heaviest
        // first evens the tails.
        for (int64_t s : small_segs) {
            const BlkSeg& sd = p->segs[s];
            p->small_items[sd.N <= 32 ? 0 : 1].push_back(BlkSmallItem{sd.offA, sd.offB, sd.offC, sd.M, sd.N});
        }
        for (auto& v : p->small_items)
            std::stable_sort(v.begin(), v.end(), [](const BlkSmallItem& a, const BlkSmallItem& b) {
                return (int64_t)a.M * a.N + (int64_t)(a.M + a.N) * 64 > (int64_t)b.M * b.N + (int64_t)(b.M + b.N) * 64;
            });
    }
    p->small_segments = (int64_t)small_segs.size();
    // fp32 inputs with the softmax epilogue: SIMT GEMM, then the softmax kernel in place.
    if (p->dtype_in == BLK_F32 && p->epi == BLK_EPI_SOFTMAX) {
        blk_plan tmp;
        tmp.kind = 1;
        tmp.S = S;
        tmp.H = p->H;
        tmp.dtype_in = tmp.dtype_out = BLK_F32;
        tmp.M = p->M;
        tmp.N = p->N;
        tmp.a1 = p->ao;
        if ((rc = blk_build_softmax_schedule(&tmp)) != BLK_OK) return rc;
        p->smx_chunks.swap(tmp.smx_chunks);
    }
    return BLK_OK;
}

int blk_build_softmax_schedule(blk_plan* p) {
    const int64_t S = p->S;
    const int es = elem_bytes(p->dtype_in);
    std::vector<int64_t> need(S);
    for (int64_t s = 0; s < S; ++s) {
        if (p->M[s] < 0 || p->N[s] < 0 || p->M[s] > INT32_MAX / 2 || p->N[s] > INT32_MAX / 2 ||
            !mul_ok(p->M[s], p->N[s], &need[s])) {
            blk_set_error("softmax plan: extent of segment " + std::to_string(s) + " is negative or too large");
            return BLK_ERR_INVALID;
        }
    }
    int rc;
    if ((rc = validate_offsets("softmax plan: srcAccum", p->a1, need, S)) != BLK_OK) return rc;
    p->Dm1 = p->Dout = p->a1[S];
    p->Dm2 = 0;
    p->flops = 0;
    p->bytes = 0;
    const int64_t window = BLK_SMX_WINDOW_BYTES / es;  // elements
    // Count the chunks before making them: a batch of very many long rows must be refused, not materialised.
    int64_t count = 0;
    {
        const int64_t cap = p->max_chunks > 0 ? p->max_chunks : (int64_t)0x7fffffff / std::max<int64_t>(p->H, 1);
        for (int64_t s = 0; s < S && count <= cap; ++s) {
            const int64_t rows = p->M[s], cols = p->N[s];
            if (rows == 0 || cols == 0) continue;
            const int64_t rpc = cols > window ? 1 : window / cols;
            count += (rows + rpc - 1) / rpc;
        }
        if (count > cap) {
            blk_set_error("softmax plan: this batch needs more than " + std::to_string(cap) +
                          " chunks of 12 KB (a row longer than 12 KB is one chunk)");
            return BLK_ERR_UNSUPPORTED;
        }
    }
    // Chunks, and in the same pass the windows of the pipelined kernels: consecutive chunks that are contiguous in
    // memory, up to the window size.
    p->smx_chunks.resize((size_t)count);
    p->smx_windows.clear();
    p->smx_windows.reserve((size_t)count / 2 + 16);
    BlkSmxChunk* const chunks = p->smx_chunks.data();
    int64_t c = 0;
    int64_t open_end = -1;  // element offset one past the last piece of the window being filled (-1: none)
    auto add_chunk = [&](int64_t off, int64_t rows, int64_t cols) {
        chunks[c] = BlkSmxChunk{off, (int32_t)rows, (int32_t)cols};
        const int64_t ne = rows * cols, nb = ne * es;
        bool extend = false;
        if (open_end == off && nb <= BLK_SMX_WINDOW_BYTES) {
            const BlkSmxWindow& wd = p->smx_windows.back();
            extend = wd.nbytes + nb <= BLK_SMX_WINDOW_BYTES && wd.npieces < BLK_SMX_WINDOW_PIECES;
        }
        if (extend) {
            BlkSmxWindow& wd = p->smx_windows.back();
            wd.nbytes += (int32_t)nb;
            wd.npieces += 1;
            open_end += ne;
        } else {
            // a one-row piece longer than the window keeps its own window; its byte count only has to exceed the
            // window size for the kernel to stream it (and no later piece continues such a window)
            const int64_t capped = std::min<int64_t>(nb, (int64_t)BLK_SMX_WINDOW_BYTES + 1);
            p->smx_windows.push_back(BlkSmxWindow{off, (int32_t)capped, (int32_t)c, 1, 0});
            open_end = nb <= BLK_SMX_WINDOW_BYTES ? off + ne : -1;
        }
        ++c;
    };
    for (int64_t s = 0; s < S; ++s) {
        const int64_t rows = p->M[s], cols = p->N[s];
        p->bytes += 2.0 * (double)p->H * (double)rows * (double)cols * es;
        if (rows == 0 || cols == 0) continue;
        const int64_t rpc = cols > window ? 1 : window / cols;
        for (int64_t r = 0; r < rows; r += rpc) add_chunk(p->a1[s] + r * cols, std::min(rpc, rows - r), cols);
    }
    return BLK_OK;
}
