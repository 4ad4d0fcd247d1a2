// C ABI of libblkattn: plan life cycle and the run entry points declared in
// include/blkattn.h.  Thin by design -- argument checks, one upload of the
// schedule at plan creation, kernel launches on the caller's stream.
#include <cuda_runtime.h>
#include <nvtx3/nvToolsExt.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <new>
#include <string>

#include "blk_internal.h"
#include "blk_kernels.h"

// A named range around every plan creation and every run, for timelines of tools that collect NVTX (header-only:
// without such a tool attached a range is a call through a pointer to an empty function).  BLK_NVTX=0 in the
// environment leaves them out.
namespace {
struct BlkRange {
    bool on;
    explicit BlkRange(const char* name) : on(enabled()) {
        if (on) nvtxRangePushA(name);
    }
    ~BlkRange() {
        if (on) nvtxRangePop();
    }
    BlkRange(const BlkRange&) = delete;
    BlkRange& operator=(const BlkRange&) = delete;
    static bool enabled() {
        static const bool v = [] {
            const char* e = std::getenv("BLK_NVTX");
            return !(e && e[0] == '0' && e[1] == 0);
        }();
        return v;
    }
};
}  // namespace

namespace {

int cuda_fail(const char* what, cudaError_t e) {
    blk_set_error(std::string(what) + ": " + cudaGetErrorString(e));
    return BLK_ERR_CUDA;
}

struct DeviceScope {
    int prev = -1;
    bool ok = true;
    explicit DeviceScope(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) { ok = false; return; }
        if (prev != dev && cudaSetDevice(dev) != cudaSuccess) ok = false;
        target = dev;
    }
    ~DeviceScope() {
        if (ok && prev >= 0 && prev != target) cudaSetDevice(prev);
    }
    int target = -1;
};

// All device tables of a plan live in one allocation, filled by one copy: the tables are laid out in a host
// staging block (kept per thread and reused, so a new plan touches no fresh pages) at 256-byte aligned offsets,
// followed by the status / counter words, and the block goes up with a single cudaMemcpy.
int upload_plan(blk_plan* p) {
    if (p->device < 0) return BLK_OK;
    DeviceScope scope(p->device);
    if (!scope.ok) {
        blk_set_error("cannot select CUDA device " + std::to_string(p->device));
        return BLK_ERR_CUDA;
    }
    {
        int sms = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, p->device) == cudaSuccess && sms > 0)
            p->num_sms = sms;
    }
    struct Piece { const void* src; size_t bytes; void** dst; size_t off; };
    std::vector<Piece> pieces;
    size_t total = 0;
    auto add = [&](const void* src, size_t bytes, void** dst) {
        *dst = nullptr;
        if (bytes == 0) return;
        pieces.push_back(Piece{src, bytes, dst, total});
        total += (bytes + 255) & ~(size_t)255;
    };
    auto add_vec = [&](const auto& v, auto** dst) {
        add(v.data(), v.size() * sizeof(v[0]), reinterpret_cast<void**>(dst));
    };
    add_vec(p->segs, &p->d_segs);
    add_vec(p->tile_items, &p->d_tile_items);
    // the staged kernel reads an item and its segment as one record: built straight into the staging block
    const size_t nrecs = p->dtype_in != BLK_F32 ? p->tile_items.size() : 0;
    add(nullptr, nrecs * sizeof(BlkTileRec), reinterpret_cast<void**>(&p->d_tile_recs));
    add_vec(p->simt_items, &p->d_simt_items);
    for (int b = 0; b < BLK_SMALL_BUCKETS; ++b) add_vec(p->small_items[b], &p->d_small_items[b]);
    add_vec(p->umma_items, &p->d_umma_items);
    add_vec(p->pv_items, &p->d_pv_items);
    add_vec(p->flash_items, &p->d_flash_items);
    add_vec(p->packs, &p->d_packs);
    add_vec(p->pack_blocks, &p->d_pack_blocks);
    add_vec(p->smx_chunks, &p->d_smx_chunks);
    add_vec(p->smx_windows, &p->d_smx_windows);
    const size_t status_off = total;
    total += 256;
    static thread_local std::vector<unsigned char> stage;
    if (stage.size() < total) stage.resize(total);
    for (const Piece& pc : pieces) {
        if (pc.src) {
            std::memcpy(stage.data() + pc.off, pc.src, pc.bytes);
        } else {
            BlkTileRec* recs = reinterpret_cast<BlkTileRec*>(stage.data() + pc.off);
            for (size_t i = 0; i < nrecs; ++i) recs[i] = BlkTileRec{p->segs[p->tile_items[i].seg], p->tile_items[i], 0};
        }
    }
    std::memset(stage.data() + status_off, 0, 256);
    cudaError_t e = cudaMalloc(&p->d_pool, total);
    if (e != cudaSuccess) return cuda_fail("allocate plan tables", e);
    e = cudaMemcpy(p->d_pool, stage.data(), total, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) return cuda_fail("upload plan tables", e);
    unsigned char* base = reinterpret_cast<unsigned char*>(p->d_pool);
    for (const Piece& pc : pieces) *pc.dst = base + pc.off;
    p->d_status = reinterpret_cast<int*>(base + status_off);
    p->d_counter = p->d_status + 1;
    return BLK_OK;
}

bool grid_ok(int64_t items, int64_t H, const char* what) {
    if (items * H > 0x7fffffffLL) {
        blk_set_error(std::string(what) + ": work items x heads exceeds 2^31-1 CTAs");
        return false;
    }
    return true;
}

size_t small_count(const blk_plan* p) { return (size_t)p->small_segments; }

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

extern "C" int blk_gemm_plan_create(blk_plan_t** plan, const int64_t* M, const int64_t* N, const int64_t* K,
                                    const int64_t* accum1, const int64_t* accum2, const int64_t* accumOut, int64_t S,
                                    int64_t H, int dtype_in, int dtype_out, int transpose1, int transpose2,
                                    int epilogue, int device) {
    BlkRange range("blk_gemm_plan_create");
    if (!plan) {
        blk_set_error("blk_gemm_plan_create: plan is null");
        return BLK_ERR_INVALID;
    }
    *plan = nullptr;
    if (S < 0 || H < 0 || (S > 0 && (!M || !N || !K))) {
        blk_set_error("blk_gemm_plan_create: negative count or null list");
        return BLK_ERR_INVALID;
    }
    const int given = (accum1 != nullptr) + (accum2 != nullptr) + (accumOut != nullptr);
    if (given != 0 && given != 3) {
        blk_set_error("blk_gemm_plan_create: give all three offset arrays or none");
        return BLK_ERR_INVALID;
    }
    if (dtype_in < BLK_F16 || dtype_in > BLK_F32 || dtype_out < BLK_F16 || dtype_out > BLK_F32 ||
        (dtype_in == BLK_F32 && dtype_out != BLK_F32) ||
        (dtype_in != BLK_F32 && dtype_out != BLK_F32 && dtype_out != dtype_in)) {
        blk_set_error("blk_gemm_plan_create: unsupported dtype combination (out must be the input dtype or fp32)");
        return BLK_ERR_UNSUPPORTED;
    }
    if (epilogue != BLK_EPI_SCORES && epilogue != BLK_EPI_SOFTMAX) {
        blk_set_error("blk_gemm_plan_create: unknown epilogue");
        return BLK_ERR_INVALID;
    }
    blk_plan* p = new (std::nothrow) blk_plan();
    if (!p) return BLK_ERR_NOMEM;
    p->kind = 0;
    p->S = S;
    p->H = H;
    p->dtype_in = dtype_in;
    p->dtype_out = dtype_out;
    p->ta = transpose1 ? 1 : 0;
    p->tb = transpose2 ? 1 : 0;
    p->epi = epilogue;
    p->device = device;
    p->M.assign(M, M + S);
    p->N.assign(N, N + S);
    p->K.assign(K, K + S);
    p->a1.resize(S + 1);
    p->a2.resize(S + 1);
    p->ao.resize(S + 1);
    int rc;
    if (given == 3) {
        std::memcpy(p->a1.data(), accum1, (S + 1) * sizeof(int64_t));
        std::memcpy(p->a2.data(), accum2, (S + 1) * sizeof(int64_t));
        std::memcpy(p->ao.data(), accumOut, (S + 1) * sizeof(int64_t));
        rc = BLK_OK;
    } else {
        rc = blk_offsets_from_lists(M, N, K, S, p->a1.data(), p->a2.data(), p->ao.data());
    }
    if (rc == BLK_OK) rc = blk_build_gemm_schedule(p);
    if (rc == BLK_OK && !(grid_ok((int64_t)p->tile_items.size(), H, "gemm plan") &&
                          grid_ok((int64_t)p->simt_items.size(), H, "gemm plan") &&
                          grid_ok((int64_t)p->smx_chunks.size(), H, "gemm plan") &&
                          grid_ok((int64_t)small_count(p), H, "gemm plan") &&
                          grid_ok((int64_t)p->umma_items.size(), H, "gemm plan") &&
                          grid_ok((int64_t)p->pv_items.size(), H, "gemm plan") &&
                          grid_ok((int64_t)p->packs.size(), H, "gemm plan")))
        rc = BLK_ERR_UNSUPPORTED;
    if (rc == BLK_OK) rc = upload_plan(p);
    if (rc != BLK_OK) {
        blk_plan_destroy(p);
        return rc;
    }
    *plan = p;
    return BLK_OK;
}

extern "C" int blk_softmax_plan_create(blk_plan_t** plan, const int64_t* rows, const int64_t* cols,
                                       const int64_t* accum, int64_t S, int64_t H, int dtype, int device) {
    BlkRange range("blk_softmax_plan_create");
    if (!plan) {
        blk_set_error("blk_softmax_plan_create: plan is null");
        return BLK_ERR_INVALID;
    }
    *plan = nullptr;
    if (S < 0 || H < 0 || (S > 0 && (!rows || !cols))) {
        blk_set_error("blk_softmax_plan_create: negative count or null list");
        return BLK_ERR_INVALID;
    }
    if (dtype < BLK_F16 || dtype > BLK_F32) {
        blk_set_error("blk_softmax_plan_create: unsupported dtype");
        return BLK_ERR_UNSUPPORTED;
    }
    blk_plan* p = new (std::nothrow) blk_plan();
    if (!p) return BLK_ERR_NOMEM;
    p->kind = 1;
    p->S = S;
    p->H = H;
    p->dtype_in = p->dtype_out = dtype;
    p->device = device;
    p->M.assign(rows, rows + S);
    p->N.assign(cols, cols + S);
    p->a1.resize(S + 1);
    int rc;
    if (accum) {
        std::memcpy(p->a1.data(), accum, (S + 1) * sizeof(int64_t));
        rc = BLK_OK;
    } else {
        rc = blk_softmax_offsets(rows, cols, S, p->a1.data());
    }
    if (rc == BLK_OK) rc = blk_build_softmax_schedule(p);
    if (rc == BLK_OK && !grid_ok((int64_t)p->smx_chunks.size(), H, "softmax plan")) rc = BLK_ERR_UNSUPPORTED;
    if (rc == BLK_OK) rc = upload_plan(p);
    if (rc != BLK_OK) {
        blk_plan_destroy(p);
        return rc;
    }
    p->ao = p->a1;
    *plan = p;
    return BLK_OK;
}

extern "C" void blk_plan_destroy(blk_plan_t* p) {
    if (!p) return;
    if (p->device >= 0) {
        DeviceScope scope(p->device);
        cudaFree(p->d_pool);  // every table and the status words are pieces of this one allocation
    }
    delete p;
}

extern "C" int blk_plan_extents(const blk_plan_t* p, int64_t* Dm1, int64_t* Dm2, int64_t* Dout) {
    if (!p) {
        blk_set_error("blk_plan_extents: plan is null");
        return BLK_ERR_INVALID;
    }
    if (Dm1) *Dm1 = p->Dm1;
    if (Dm2) *Dm2 = p->Dm2;
    if (Dout) *Dout = p->Dout;
    return BLK_OK;
}

extern "C" int blk_plan_offsets(const blk_plan_t* p, int64_t* a1, int64_t* a2, int64_t* ao) {
    if (!p) {
        blk_set_error("blk_plan_offsets: plan is null");
        return BLK_ERR_INVALID;
    }
    const size_t n = (size_t)(p->S + 1) * sizeof(int64_t);
    if (a1) std::memcpy(a1, p->a1.data(), n);
    if (a2 && p->kind == 0) std::memcpy(a2, p->a2.data(), n);
    if (ao) std::memcpy(ao, p->ao.data(), n);
    return BLK_OK;
}

static int launches_per_run(const blk_plan* p) {
    if (p->attn) return (p->flash_items.empty() ? 0 : 1) + (p->packs.empty() ? 0 : 1);
    int n = (!p->tile_items.empty()) + (!p->simt_items.empty()) + (!p->umma_items.empty()) + (!p->smx_chunks.empty()) +
            (!p->pv_items.empty());
    if (p->small_pipe) return n + 1;
    for (const auto& v : p->small_items) n += !v.empty();
    return n;
}

extern "C" int blk_plan_summary(const blk_plan_t* p, int64_t counts[8]) {
    if (!p || !counts) {
        blk_set_error("blk_plan_summary: null argument");
        return BLK_ERR_INVALID;
    }
    counts[0] = p->S;
    counts[1] = (int64_t)small_count(p);
    counts[2] = (int64_t)p->tile_items.size();
    counts[3] = (int64_t)(p->attn ? p->flash_items.size() : p->umma_items.size() + p->pv_items.size());
    counts[4] = (int64_t)p->smx_chunks.size();
    counts[5] = p->H > 0 ? launches_per_run(p) : 0;
    counts[6] = (int64_t)p->simt_items.size();
    counts[7] = (int64_t)p->packs.size();
    return BLK_OK;
}

extern "C" int blk_plan_table(const blk_plan_t* p, int table, void* dst, int64_t capacity, int64_t* bytes,
                              int64_t* record_bytes) {
    if (!p || !bytes) {
        blk_set_error("blk_plan_table: null argument");
        return BLK_ERR_INVALID;
    }
    const void* src = nullptr;
    size_t n = 0, rec = 0;
    auto take = [&](const auto& v) { src = v.data(); rec = sizeof(v[0]); n = v.size() * rec; };
    switch (table) {
        case BLK_TABLE_SEGMENTS: take(p->segs); break;
        case BLK_TABLE_TILE_ITEMS: take(p->tile_items); break;
        case BLK_TABLE_SIMT_ITEMS: take(p->simt_items); break;
        case BLK_TABLE_SMALL_ITEMS_32: take(p->small_items[0]); break;
        case BLK_TABLE_SMALL_ITEMS_64: take(p->small_items[1]); break;
        case BLK_TABLE_UMMA_ITEMS: take(p->umma_items); break;
        case BLK_TABLE_PV_ITEMS: take(p->pv_items); break;
        case BLK_TABLE_PACKS: take(p->packs); break;
        case BLK_TABLE_PACK_BLOCKS: take(p->pack_blocks); break;
        case BLK_TABLE_SMX_CHUNKS: take(p->smx_chunks); break;
        case BLK_TABLE_SMX_WINDOWS: take(p->smx_windows); break;
        case BLK_TABLE_FLASH_ITEMS: take(p->flash_items); break;
        case BLK_TABLE_UMMA_VIEWS_A: take(p->umma_viewsA); break;
        case BLK_TABLE_UMMA_VIEWS_B: take(p->umma_viewsB); break;
        default:
            blk_set_error("blk_plan_table: no table " + std::to_string(table));
            return BLK_ERR_INVALID;
    }
    *bytes = (int64_t)n;
    if (record_bytes) *record_bytes = (int64_t)rec;
    if (dst) {
        if (capacity < (int64_t)n) {
            blk_set_error("blk_plan_table: the table has " + std::to_string(n) + " bytes, the buffer " + std::to_string(capacity));
            return BLK_ERR_INVALID;
        }
        if (n) std::memcpy(dst, src, n);
    }
    return BLK_OK;
}

extern "C" int blk_plan_work(const blk_plan_t* p, double* flops, double* bytes) {
    if (!p) {
        blk_set_error("blk_plan_work: plan is null");
        return BLK_ERR_INVALID;
    }
    if (flops) *flops = p->flops;
    if (bytes) *bytes = p->bytes;
    return BLK_OK;
}

extern "C" int blk_plan_check(const blk_plan_t* p, void* cuda_stream) {
    if (!p || p->device < 0) {
        blk_set_error("blk_plan_check: plan has no device");
        return BLK_ERR_INVALID;
    }
    cudaStream_t st = reinterpret_cast<cudaStream_t>(cuda_stream);
    cudaError_t e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return cuda_fail("blk_plan_check: synchronize", e);
    int status = 0;
    e = cudaMemcpy(&status, p->d_status, sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return cuda_fail("blk_plan_check: read status", e);
    if (status != 0) {
        blk_set_error("a device-side bounded wait gave up (status " + std::to_string(status) + ")");
        cudaMemset(p->d_status, 0, sizeof(int));
        return BLK_ERR_TIMEOUT;
    }
    return BLK_OK;
}

// Schedule of the tcgen05 attention kernel: one item per 128-row block of the queries of a segment, longest
// key/value sweeps first (the persistent CTAs take the items round-robin in this order).
static int build_flash_items(blk_plan* p, bool skip_small) {
    const int64_t d = p->head_dim;
    if (p->a1[p->S] / d >= (int64_t)1 << 31 || p->a2[p->S] / d >= (int64_t)1 << 31) {
        blk_set_error("attention plan: more than 2^31 rows");
        return BLK_ERR_UNSUPPORTED;
    }
    for (int64_t s = 0; s < p->S; ++s) {
        const int64_t M = p->M[s], N = p->N[s];
        if (M == 0) continue;
        if (skip_small && M <= BLK_SMALL_MAXM && N <= BLK_SMALL_MAXN) continue;  // in a pack
        for (int64_t tm = 0; tm * BLK_FLASH_BM < M; ++tm)
            p->flash_items.push_back(BlkFlashItem{(int32_t)(p->a1[s] / d + tm * BLK_FLASH_BM), (int32_t)(p->a2[s] / d),
                                                  (int32_t)(M - tm * BLK_FLASH_BM), (int32_t)N});
    }
    std::stable_sort(p->flash_items.begin(), p->flash_items.end(),
                     [](const BlkFlashItem& a, const BlkFlashItem& b) { return a.N > b.N; });
    return BLK_OK;
}

static int attention_plan_impl(blk_plan_t** plan, const int64_t* M, const int64_t* N, int64_t S, int64_t H,
                               int64_t head_dim, bool any_length, int dtype, int device) {
    BlkRange range("blk_attention_plan_create");
    if (!plan) {
        blk_set_error("blk_attention_plan_create: plan is null");
        return BLK_ERR_INVALID;
    }
    *plan = nullptr;
    if (S < 0 || H < 0 || (S > 0 && (!M || !N))) {
        blk_set_error("blk_attention_plan_create: negative count or null list");
        return BLK_ERR_INVALID;
    }
    if (dtype != BLK_F16 && dtype != BLK_BF16) {
        blk_set_error("blk_attention_plan_create: fp16 or bf16 only");
        return BLK_ERR_UNSUPPORTED;
    }
    if (head_dim != 64 && head_dim != 128) {
        blk_set_error("blk_attention_plan_create: head dimension 64 or 128 only");
        return BLK_ERR_UNSUPPORTED;
    }
    bool small = head_dim == 64;
    for (int64_t s = 0; s < S; ++s) {
        if (M[s] < 0 || N[s] < 0) {
            blk_set_error("blk_attention_plan_create: negative extent in segment " + std::to_string(s));
            return BLK_ERR_INVALID;
        }
        if (M[s] > 0 && N[s] == 0) {
            blk_set_error("blk_attention_plan_create: segment " + std::to_string(s) + " has queries but no keys");
            return BLK_ERR_UNSUPPORTED;
        }
        if (M[s] > BLK_SMALL_MAXM || N[s] > BLK_SMALL_MAXN) small = false;
    }
    if (!small && !any_length) {
        blk_set_error("blk_attention_plan_create: the small-segment kernel takes segments of 0..64 queries and 1..64 "
                      "keys; blk_attention_plan_create_dim takes any batch");
        return BLK_ERR_UNSUPPORTED;
    }
    blk_plan* p = new (std::nothrow) blk_plan();
    if (!p) return BLK_ERR_NOMEM;
    p->kind = 0;
    p->attn = 1;
    p->head_dim = (int)head_dim;
    p->S = S;
    p->H = H;
    p->dtype_in = p->dtype_out = dtype;
    p->ta = p->tb = 0;
    p->epi = BLK_EPI_SOFTMAX;
    p->device = device;
    p->M.assign(M, M + S);
    p->N.assign(N, N + S);
    p->K.assign((size_t)S, head_dim);
    p->a1.assign((size_t)S + 1, 0);
    p->a2.assign((size_t)S + 1, 0);
    for (int64_t s = 0; s < S; ++s) {
        p->a1[s + 1] = p->a1[s] + M[s] * head_dim;
        p->a2[s + 1] = p->a2[s] + N[s] * head_dim;
    }
    p->ao = p->a1;  // the result has one row of head_dim per query row, laid out like the queries
    size_t nonempty = 0;
    for (int64_t s = 0; s < S; ++s) nonempty += M[s] > 0 && N[s] > 0;
    int rc = BLK_OK;
    // d = 64: the segments of at most 64 x 64 go into packs of the small-segment kernel (the scheduler of the GEMM
    // bins them; what it schedules for the other segments is of no use here), the rest to the tcgen05 kernel
    bool packs = false;
    if (head_dim == 64) {
        rc = blk_build_gemm_schedule(p);
        packs = rc == BLK_OK && p->small_pipe && !p->packs.empty();
        p->tile_items.clear();
        p->umma_items.clear();
        p->simt_items.clear();
        if (!packs) {
            p->packs.clear(); p->pack_blocks.clear(); p->small_pipe = 0; p->small_segments = 0;
            for (auto& v : p->small_items) v.clear();
        }
        if (rc == BLK_OK && !any_length && nonempty > 0 && !(small && packs)) {
            blk_set_error("blk_attention_plan_create: the pack kernel cannot take this batch (BLK_DISABLE_PIPE or "
                          "BLK_DISABLE_SMALL set?)");
            rc = BLK_ERR_UNSUPPORTED;
        }
    }
    if (rc == BLK_OK && !(small && packs)) {
        p->Dm1 = p->Dout = p->a1[S];
        p->Dm2 = p->a2[S];
        rc = build_flash_items(p, packs);
        if (rc == BLK_OK && (int64_t)p->flash_items.size() * H >= ((int64_t)1 << 31)) {
            blk_set_error("attention plan: more than 2^31 work items");
            rc = BLK_ERR_UNSUPPORTED;
        }
        if (!p->flash_items.empty()) p->attn = packs ? 3 : 2;  // 3: packs and tcgen05 items, two launches
    }
    if (rc == BLK_OK) {
        p->flops = p->bytes = 0;
        for (int64_t s = 0; s < S; ++s) {
            p->flops += 4.0 * (double)H * (double)M[s] * (double)N[s] * (double)head_dim;
            p->bytes += (double)H * 2.0 * (double)head_dim * (double)(2 * M[s] + 2 * N[s]);
        }
    }
    if (rc == BLK_OK && !p->packs.empty() && !grid_ok((int64_t)p->packs.size(), H, "attention plan")) rc = BLK_ERR_UNSUPPORTED;
    if (rc == BLK_OK) rc = upload_plan(p);
    if (rc != BLK_OK) {
        blk_plan_destroy(p);
        return rc;
    }
    *plan = p;
    return BLK_OK;
}

extern "C" int blk_attention_plan_create(blk_plan_t** plan, const int64_t* M, const int64_t* N, int64_t S, int64_t H,
                                         int dtype, int device) {
    return attention_plan_impl(plan, M, N, S, H, 64, false, dtype, device);
}

extern "C" int blk_attention_plan_create_dim(blk_plan_t** plan, const int64_t* M, const int64_t* N, int64_t S, int64_t H,
                                             int64_t head_dim, int dtype, int device) {
    return attention_plan_impl(plan, M, N, S, H, head_dim, true, dtype, device);
}

// Shared body of blk_attention_run (strides 0: packed head-major strips) and blk_attention_run_strided.
static int attention_run_impl(const blk_plan* p, const void* q, const void* k, const void* v, void* out,
                              int64_t row_stride, int64_t head_stride, float scale, void* cuda_stream);

extern "C" int blk_attention_run(const blk_plan_t* p, const void* q, const void* k, const void* v, void* out,
                                 float scale, void* cuda_stream) {
    return attention_run_impl(p, q, k, v, out, 0, 0, scale, cuda_stream);
}

extern "C" int blk_attention_run_strided(const blk_plan_t* p, const void* q, const void* k, const void* v, void* out,
                                         int64_t row_stride, int64_t head_stride, float scale, void* cuda_stream) {
    if (row_stride < (p && p->attn ? p->head_dim : 64) || head_stride <= 0 || row_stride % 8 || head_stride % 8) {
        blk_set_error("blk_attention_run_strided: strides must be multiples of 8 elements, the row stride at least "
                      "the head dimension");
        return BLK_ERR_INVALID;
    }
    return attention_run_impl(p, q, k, v, out, row_stride, head_stride, scale, cuda_stream);
}

static int attention_run_impl(const blk_plan* p, const void* q, const void* k, const void* v, void* out,
                              int64_t row_stride, int64_t head_stride, float scale, void* cuda_stream) {
    BlkRange range("blk_attention_run");
    if (!p || p->kind != 0 || !p->attn) {
        blk_set_error("blk_attention_run: not an attention plan");
        return BLK_ERR_INVALID;
    }
    if (p->device < 0) {
        blk_set_error("blk_attention_run: the plan was created without a device");
        return BLK_ERR_INVALID;
    }
    if ((p->packs.empty() && p->flash_items.empty()) || p->H == 0) return BLK_OK;
    if (!q || !k || !v || !out) {
        blk_set_error("blk_attention_run: null buffer");
        return BLK_ERR_INVALID;
    }
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out)) {
        blk_set_error("blk_attention_run: device pointers must be 16-byte aligned");
        return BLK_ERR_UNALIGNED;
    }
    if (scale == 0.f) scale = 1.17549435e-38f;  // softmax(0 * S) is the uniform distribution
    if (!p->flash_items.empty()) {
        const int64_t d = p->head_dim;
        const bool strips = row_stride == 0;
        BlkFlashParams fp{};
        fp.out = out;
        fp.items = p->d_flash_items;
        fp.num_items = (int)p->flash_items.size();
        fp.H = (int)p->H;
        fp.D = (int)d;
        fp.bf16 = p->dtype_in == BLK_BF16;
        fp.scale = scale;
        fp.status = p->d_status;
        fp.layQ = BlkOperandLayout{p->Dm1 / d, strips ? d : row_stride, strips ? p->Dm1 : head_stride};
        fp.layK = BlkOperandLayout{p->Dm2 / d, strips ? d : row_stride, strips ? p->Dm2 : head_stride};
        fp.layV = fp.layK;
        fp.out_row_stride = strips ? d : row_stride;
        fp.out_head_stride = strips ? p->Dm1 : head_stride;
        cudaError_t e = blk_launch_attn_umma(fp, q, k, v, p->num_sms, reinterpret_cast<cudaStream_t>(cuda_stream));
        if (e != cudaSuccess) return cuda_fail("attention launch", e);
    }
    if (p->packs.empty()) return BLK_OK;
    BlkPackParams pp{};
    pp.A = reinterpret_cast<const uint16_t*>(q);
    pp.B = reinterpret_cast<const uint16_t*>(k);
    pp.V = reinterpret_cast<const uint16_t*>(v);
    pp.C = out;
    pp.packs = p->d_packs;
    pp.blocks = p->d_pack_blocks;
    pp.Dm1 = p->Dm1; pp.Dm2 = p->Dm2; pp.Dout = p->Dm1;
    pp.num_packs = (int)p->packs.size();
    pp.H = (int)p->H;
    pp.epi = BLK_EPI_SOFTMAX;
    pp.scale = scale;
    pp.status = p->d_status;
    const bool packed = row_stride == 0;
    pp.layA = BlkOperandLayout{p->Dm1 / 64, packed ? 64 : row_stride, packed ? p->Dm1 : head_stride};
    pp.layB = BlkOperandLayout{p->Dm2 / 64, packed ? 64 : row_stride, packed ? p->Dm2 : head_stride};
    pp.layV = pp.layB;
    pp.out_row_stride = packed ? 64 : row_stride;
    pp.out_head_stride = packed ? p->Dm1 : head_stride;
    cudaError_t e = blk_launch_scores_pipe(pp, p->dtype_in, p->num_sms, reinterpret_cast<cudaStream_t>(cuda_stream));
    if (e != cudaSuccess) return cuda_fail("attention launch", e);
    return BLK_OK;
}

// Shared body of blk_gemm_run and blk_gemm_run_strided; layA / layB say where the operands' rows are (null:
// packed head-major strips, whose row view depends on the contraction length of the kernel that reads them).
static int gemm_run_impl(const blk_plan* p, const void* mat1, const void* mat2, void* out, float scale,
                         const BlkOperandLayout* layA, const BlkOperandLayout* layB, void* cuda_stream) {
    BlkRange range("blk_gemm_run");
    if (p && p->attn) {
        blk_set_error("blk_gemm_run: this is an attention plan, run it with blk_attention_run");
        return BLK_ERR_INVALID;
    }
    auto layout = [](const BlkOperandLayout* given, int64_t D, int64_t K) {
        return given ? *given : BlkOperandLayout{D / K, K, D};
    };
    if (!p || p->kind != 0) {
        blk_set_error("blk_gemm_run: not a GEMM plan");
        return BLK_ERR_INVALID;
    }
    if (p->device < 0) {
        blk_set_error("blk_gemm_run: the plan was created without a device");
        return BLK_ERR_INVALID;
    }
    if (p->S == 0 || p->H == 0 || p->Dout == 0) return BLK_OK;
    if (!out || (!mat1 && p->Dm1 > 0) || (!mat2 && p->Dm2 > 0)) {
        blk_set_error("blk_gemm_run: null buffer");
        return BLK_ERR_INVALID;
    }
    if (!aligned16(mat1) || !aligned16(mat2) || !aligned16(out)) {
        blk_set_error("blk_gemm_run: device pointers must be 16-byte aligned");
        return BLK_ERR_UNALIGNED;
    }
    cudaStream_t st = reinterpret_cast<cudaStream_t>(cuda_stream);
    cudaError_t e;
    // softmax(0 * S) is the uniform distribution; a denormal-free tiny scale gives exactly that and keeps
    // the kernels' "-inf times scale" column masks well defined
    if (p->epi == BLK_EPI_SOFTMAX && scale == 0.f) scale = 1.17549435e-38f;
    if (!p->simt_items.empty()) {
        BlkSimtParams sp{};
        sp.A = reinterpret_cast<const float*>(mat1);
        sp.B = reinterpret_cast<const float*>(mat2);
        sp.C = reinterpret_cast<float*>(out);
        sp.segs = p->d_segs;
        sp.items = p->d_simt_items;
        sp.Dm1 = p->Dm1; sp.Dm2 = p->Dm2; sp.Dout = p->Dout;
        sp.num_items = (int)p->simt_items.size();
        sp.H = (int)p->H;
        sp.ta = p->ta; sp.tb = p->tb;
        sp.scale = scale;
        if ((e = blk_launch_gemm_simt(sp, st)) != cudaSuccess) return cuda_fail("fp32 GEMM launch", e);
        if (!p->smx_chunks.empty()) {
            BlkSmxParams xp{};
            xp.src = out; xp.dst = out;
            xp.chunks = p->d_smx_chunks;
            xp.D = p->Dout;
            xp.num_chunks = (int)p->smx_chunks.size();
            xp.H = (int)p->H;
            xp.scale = 1.f;
            if ((e = blk_launch_softmax(xp, BLK_F32, st)) != cudaSuccess) return cuda_fail("softmax launch", e);
        }
    }
    if (p->small_pipe) {
        BlkPackParams pp{};
        pp.A = reinterpret_cast<const uint16_t*>(mat1);
        pp.B = reinterpret_cast<const uint16_t*>(mat2);
        pp.C = out;
        pp.packs = p->d_packs;
        pp.blocks = p->d_pack_blocks;
        pp.Dm1 = p->Dm1; pp.Dm2 = p->Dm2; pp.Dout = p->Dout;
        pp.num_packs = (int)p->packs.size();
        pp.H = (int)p->H;
        pp.epi = p->epi;
        pp.scale = scale;
        pp.status = p->d_status;
        pp.layA = layout(layA, p->Dm1, 64);
        pp.layB = layout(layB, p->Dm2, 64);
        if ((e = blk_launch_scores_pipe(pp, p->dtype_in, p->num_sms, st)) != cudaSuccess)
            return cuda_fail("pipelined small-segment launch", e);
    }
    for (int b = 0; b < BLK_SMALL_BUCKETS && !p->small_pipe; ++b) {
        if (p->small_items[b].empty()) continue;
        BlkSmallParams mp{};
        mp.A = reinterpret_cast<const uint16_t*>(mat1);
        mp.B = reinterpret_cast<const uint16_t*>(mat2);
        mp.C = out;
        mp.items = p->d_small_items[b];
        mp.Dm1 = p->Dm1; mp.Dm2 = p->Dm2; mp.Dout = p->Dout;
        mp.num_items = (int)p->small_items[b].size();
        mp.H = (int)p->H;
        mp.out_f32 = p->dtype_out == BLK_F32;
        mp.epi = p->epi;
        mp.scale = scale;
        if ((e = blk_launch_scores_small(mp, p->dtype_in, p->small_K, b, p->num_sms, st)) != cudaSuccess)
            return cuda_fail("small-segment launch", e);
    }
    if (!p->umma_items.empty()) {
        BlkUmmaParams up{};
        up.C = out;
        up.items = p->d_umma_items;
        up.Dout = p->Dout;
        up.num_items = (int)p->umma_items.size();
        up.H = (int)p->H;
        up.bf16 = p->dtype_in == BLK_BF16;
        up.out_f32 = p->dtype_out == BLK_F32;
        up.epi = p->epi;
        up.scale = scale;
        up.status = p->d_status;
        up.long_rows = p->umma_long_rows;
        if (blk_env_flag("BLK_TEST_STALL_PRODUCER")) {  // test hook: see BlkUmmaParams::stall
            up.stall = 1;
            up.spin_limit = 4096;
        }
        const BlkUmmaOperand opA{mat1, p->Dm1, p->umma_viewsA.data(), (int)p->umma_viewsA.size(), layA};
        const BlkUmmaOperand opB{mat2, p->Dm2, p->umma_viewsB.data(), (int)p->umma_viewsB.size(), layB};
        if ((e = blk_launch_gemm_umma(up, opA, opB, p->num_sms, st)) != cudaSuccess)
            return cuda_fail("tcgen05 GEMM launch", e);
    }
    if (!p->pv_items.empty()) {
        BlkPvParams vp{};
        vp.A = mat1;
        vp.C = out;
        vp.items = p->d_pv_items;
        vp.Dm1 = p->Dm1; vp.Dm2 = p->Dm2; vp.Dout = p->Dout;
        vp.num_items = (int)p->pv_items.size();
        vp.H = (int)p->H;
        vp.D = p->pv_D;
        vp.bf16 = p->dtype_in == BLK_BF16;
        vp.scale = scale;
        vp.status = p->d_status;
        if ((e = blk_launch_pv_umma(vp, mat2, p->num_sms, st)) != cudaSuccess) return cuda_fail("tcgen05 P V launch", e);
    }
    if (!p->tile_items.empty()) {
        BlkGemmParams gp{};
        gp.A = reinterpret_cast<const uint16_t*>(mat1);
        gp.B = reinterpret_cast<const uint16_t*>(mat2);
        gp.C = out;
        gp.segs = p->d_segs;
        gp.items = p->d_tile_items;
        gp.recs = p->d_tile_recs;
        gp.Dm1 = p->Dm1; gp.Dm2 = p->Dm2; gp.Dout = p->Dout;
        gp.num_items = (int)p->tile_items.size();
        gp.H = (int)p->H;
        gp.out_f32 = p->dtype_out == BLK_F32;
        gp.epi = p->epi;
        gp.scale = scale;
        if ((e = blk_launch_gemm_tile(gp, p->dtype_in, p->ta, p->tb, st)) != cudaSuccess)
            return cuda_fail("tile GEMM launch", e);
    }
    return BLK_OK;
}

extern "C" int blk_gemm_run(const blk_plan_t* p, const void* mat1, const void* mat2, void* out, float scale,
                            void* cuda_stream) {
    if (!p || p->kind != 0) {
        blk_set_error("blk_gemm_run: not a GEMM plan");
        return BLK_ERR_INVALID;
    }
    return gemm_run_impl(p, mat1, mat2, out, scale, nullptr, nullptr, cuda_stream);
}

extern "C" int blk_gemm_run_strided(const blk_plan_t* p, const void* mat1, int64_t row_stride1, int64_t head_stride1,
                                    const void* mat2, int64_t row_stride2, int64_t head_stride2, void* out,
                                    float scale, void* cuda_stream) {
    if (!p || p->kind != 0) {
        blk_set_error("blk_gemm_run_strided: not a GEMM plan");
        return BLK_ERR_INVALID;
    }
    if (p->S == 0 || p->H == 0 || p->Dout == 0) return BLK_OK;
    // Only the kernels that fetch operands through tensor maps take strides: every segment must be on the
    // pack kernel or the tcgen05 kernel, which also means one contraction length for the whole batch.
    const bool small_ok = p->small_pipe || small_count(p) == 0;
    if (!small_ok || !p->tile_items.empty() || !p->simt_items.empty() || !p->pv_items.empty()) {
        blk_set_error("blk_gemm_run_strided: this batch needs a kernel that reads packed operands only "
                      "(16-bit inputs, not transposed, packed offsets, one K that is a multiple of 8 are required)");
        return BLK_ERR_UNSUPPORTED;
    }
    const int64_t K = p->small_pipe ? 64 : p->umma_K;
    if (K <= 0 || (p->small_pipe && p->umma_K != 0 && p->umma_K != 64)) {
        blk_set_error("blk_gemm_run_strided: the batch does not have one contraction length");
        return BLK_ERR_UNSUPPORTED;
    }
    for (const int64_t v : {row_stride1, head_stride1, row_stride2, head_stride2})
        if (v <= 0 || v % 8) {
            blk_set_error("blk_gemm_run_strided: strides must be positive multiples of 8 elements");
            return BLK_ERR_INVALID;
        }
    if (row_stride1 < K || row_stride2 < K) {
        blk_set_error("blk_gemm_run_strided: a row stride is shorter than the contraction length");
        return BLK_ERR_INVALID;
    }
    const BlkOperandLayout layA{p->Dm1 / K, row_stride1, head_stride1}, layB{p->Dm2 / K, row_stride2, head_stride2};
    return gemm_run_impl(p, mat1, mat2, out, scale, &layA, &layB, cuda_stream);
}

extern "C" int blk_softmax_run(const blk_plan_t* p, const void* src, void* out, float scale, void* cuda_stream) {
    BlkRange range("blk_softmax_run");
    if (!p || p->kind != 1) {
        blk_set_error("blk_softmax_run: not a softmax plan");
        return BLK_ERR_INVALID;
    }
    if (p->device < 0) {
        blk_set_error("blk_softmax_run: the plan was created without a device");
        return BLK_ERR_INVALID;
    }
    if (p->smx_chunks.empty() || p->H == 0) return BLK_OK;
    if (!src || !out) {
        blk_set_error("blk_softmax_run: null buffer");
        return BLK_ERR_INVALID;
    }
    if (!aligned16(src) || !aligned16(out)) {
        blk_set_error("blk_softmax_run: device pointers must be 16-byte aligned");
        return BLK_ERR_UNALIGNED;
    }
    BlkSmxPipeParams xp{};
    xp.in0 = src;
    xp.in1 = nullptr;
    xp.out = out;
    xp.windows = p->d_smx_windows;
    xp.pieces = p->d_smx_chunks;
    xp.D = p->Dm1;
    xp.num_windows = (int)p->smx_windows.size();
    xp.H = (int)p->H;
    xp.scale = scale;
    xp.status = p->d_status;
    cudaError_t e = blk_launch_softmax_pipe(xp, p->dtype_in, 0, p->num_sms, reinterpret_cast<cudaStream_t>(cuda_stream));
    if (e != cudaSuccess) return cuda_fail("softmax launch", e);
    return BLK_OK;
}

extern "C" int blk_softmax_backward_run(const blk_plan_t* p, const void* out, const void* grad_out, void* grad_src,
                                        float scale, void* cuda_stream) {
    BlkRange range("blk_softmax_backward_run");
    if (!p || p->kind != 1) {
        blk_set_error("blk_softmax_backward_run: not a softmax plan");
        return BLK_ERR_INVALID;
    }
    if (p->device < 0) {
        blk_set_error("blk_softmax_backward_run: the plan was created without a device");
        return BLK_ERR_INVALID;
    }
    if (p->smx_chunks.empty() || p->H == 0) return BLK_OK;
    if (!out || !grad_out || !grad_src) {
        blk_set_error("blk_softmax_backward_run: null buffer");
        return BLK_ERR_INVALID;
    }
    if (!aligned16(out) || !aligned16(grad_out) || !aligned16(grad_src)) {
        blk_set_error("blk_softmax_backward_run: device pointers must be 16-byte aligned");
        return BLK_ERR_UNALIGNED;
    }
    BlkSmxPipeParams xp{};
    xp.in0 = out;
    xp.in1 = grad_out;
    xp.out = grad_src;
    xp.windows = p->d_smx_windows;
    xp.pieces = p->d_smx_chunks;
    xp.D = p->Dm1;
    xp.num_windows = (int)p->smx_windows.size();
    xp.H = (int)p->H;
    xp.scale = scale;
    xp.status = p->d_status;
    cudaError_t e = blk_launch_softmax_pipe(xp, p->dtype_in, 1, p->num_sms, reinterpret_cast<cudaStream_t>(cuda_stream));
    if (e != cudaSuccess) return cuda_fail("softmax backward launch", e);
    return BLK_OK;
}
