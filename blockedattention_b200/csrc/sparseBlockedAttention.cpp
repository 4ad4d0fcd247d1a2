// The extension module `blockAttention._C`: upstream's two operators and three launchers (see the header) as a
// shim over libblkattn's C ABI.  Host work per call: the list tensors are read to the host once per distinct
// tensor (remembered while alive), the plan -- schedule, upload -- is built once per distinct list *values* and
// reused, the result is allocated by torch, and the kernels go to torch's current stream on the operand's device.
#include "sparseBlockedAttention.h"

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <list>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "blkattn.h"

namespace {

using torch::Tensor;
typedef std::vector<int64_t> I64;

void check_operand(const Tensor& t, const char* name) {
    // upstream csrc/sparseBlockedAttention.h:6-8
    TORCH_CHECK(t.is_cuda(), name, " must be CUDA Tensor");
    TORCH_CHECK(t.is_contiguous(), name, " must be contiguous Tensor");
}

int dtype_code(const Tensor& t) {
    switch (t.scalar_type()) {
        case at::kHalf: return BLK_F16;
        case at::kBFloat16: return BLK_BF16;
        case at::kFloat: return BLK_F32;
        default: TORCH_CHECK(false, "blockAttention: dtype ", t.scalar_type(), " is not supported (half, bfloat16, float)");
    }
    return -1;
}

void ok(int rc) { TORCH_CHECK(rc == BLK_OK, "libblkattn error ", rc, ": ", blk_last_error()); }

// ---- list tensors on the host --------------------------------------------------------------------
// A device list tensor is copied to the host the first time it is seen; the memo keeps the tensor alive, so its
// address cannot come back with other values, and an in-place write changes its version.
struct ListMemo {
    struct Entry { Tensor keep; I64 values; };
    std::mutex mu;
    std::unordered_map<std::string, std::list<std::pair<std::string, Entry>>::iterator> index;
    std::list<std::pair<std::string, Entry>> lru;
    static constexpr size_t kMax = 256;

    I64 get(const Tensor& t) {
        TORCH_CHECK(t.dim() <= 1 || t.numel() == t.size(-1), "offset and list tensors must be one-dimensional");
        if (!t.is_cuda()) {
            Tensor h = t.to(at::kLong).contiguous();
            return I64(h.data_ptr<int64_t>(), h.data_ptr<int64_t>() + h.numel());
        }
        const std::string key = std::to_string(reinterpret_cast<uintptr_t>(t.data_ptr())) + ":" + std::to_string(t._version()) +
                                ":" + std::to_string(t.numel()) + ":" + std::to_string((int)t.scalar_type()) + ":" +
                                std::to_string(t.get_device());
        {
            std::lock_guard<std::mutex> g(mu);
            auto it = index.find(key);
            if (it != index.end()) {
                lru.splice(lru.begin(), lru, it->second);
                return it->second->second.values;
            }
        }
        Tensor h = t.to(at::kCPU, at::kLong).contiguous();   // the one device->host copy of this list
        I64 v(h.data_ptr<int64_t>(), h.data_ptr<int64_t>() + h.numel());
        std::lock_guard<std::mutex> g(mu);
        lru.emplace_front(key, Entry{t, v});
        index[key] = lru.begin();
        while (lru.size() > kMax) {
            index.erase(lru.back().first);
            lru.pop_back();
        }
        return v;
    }
} g_lists;

// ---- plans, cached under the list values ------------------------------------------------------------
struct PlanCache {
    std::mutex mu;
    std::list<std::pair<std::string, blk_plan_t*>> lru;
    std::unordered_map<std::string, std::list<std::pair<std::string, blk_plan_t*>>::iterator> index;
    static constexpr size_t kMax = 64;

    template <typename Make>
    blk_plan_t* get(const std::string& key, Make make) {
        std::lock_guard<std::mutex> g(mu);
        auto it = index.find(key);
        if (it != index.end()) {
            lru.splice(lru.begin(), lru, it->second);
            return it->second->second;
        }
        blk_plan_t* p = make();
        lru.emplace_front(key, p);
        index[key] = lru.begin();
        while (lru.size() > kMax) {
            // kernels already queued only read the plan's device tables; cudaFree waits for them
            blk_plan_destroy(lru.back().second);
            index.erase(lru.back().first);
            lru.pop_back();
        }
        return p;
    }
    ~PlanCache() {
        // process exit: the CUDA context may already be gone, so the device tables are left to it
    }
} g_plans;

void append(std::string& key, const I64& v) {
    key.append(reinterpret_cast<const char*>(v.data()), v.size() * sizeof(int64_t));
    key.push_back('|');
}

Tensor to_list_tensor(const I64& v, const Tensor& like) {
    return torch::tensor(v, torch::dtype(at::kLong)).to(like.device());
}

int64_t heads_of(const Tensor& t, int64_t D, const char* name) {
    TORCH_CHECK(D > 0 && t.numel() % D == 0, name, " has ", t.numel(), " elements, not a multiple of the packed extent ", D);
    return t.numel() / D;
}

Tensor gemm_launch_host(const Tensor& mat1, const Tensor& mat2, const I64& a1, const I64& a2, const I64& ao, const I64& M,
                        const I64& N, const I64& K, bool t1, bool t2) {
    check_operand(mat1, "mat1");
    check_operand(mat2, "mat2");
    TORCH_CHECK(mat1.scalar_type() == mat2.scalar_type(), "mat1 and mat2 must have the same dtype");
    const int64_t S = (int64_t)M.size();
    TORCH_CHECK((int64_t)N.size() == S && (int64_t)K.size() == S && (int64_t)a1.size() == S + 1 &&
                    (int64_t)a2.size() == S + 1 && (int64_t)ao.size() == S + 1,
                "offset tensors must have one more entry than the lists");
    const int64_t H = heads_of(mat1, a1[S], "mat1");          // any leading shape flattens (upstream spBlkGEMM.cu:999)
    TORCH_CHECK(mat2.numel() == H * a2[S], "mat2 does not match mat2Accum[-1] x heads");
    const int dt = dtype_code(mat1), dev = mat1.get_device();
    c10::cuda::CUDAGuard guard(mat1.device());
    std::string key = "g" + std::to_string(dt) + (t1 ? "T" : "n") + (t2 ? "T" : "n") + std::to_string(dev) + ":" +
                      std::to_string(H) + "|";
    append(key, M); append(key, N); append(key, K); append(key, a1); append(key, a2); append(key, ao);
    blk_plan_t* plan = g_plans.get(key, [&]() {
        blk_plan_t* p = nullptr;
        ok(blk_gemm_plan_create(&p, M.data(), N.data(), K.data(), a1.data(), a2.data(), ao.data(), S, H, dt, dt, t1, t2,
                                BLK_EPI_SCORES, dev));
        return p;
    });
    Tensor out = torch::empty({H, ao[S]}, mat1.options());      // 2-D, dtype of the inputs (upstream spBlkGEMM.cu:1008)
    Tensor m1 = reinterpret_cast<uintptr_t>(mat1.data_ptr()) % 16 ? mat1.clone() : mat1;
    Tensor m2 = reinterpret_cast<uintptr_t>(mat2.data_ptr()) % 16 ? mat2.clone() : mat2;
    ok(blk_gemm_run(plan, m1.data_ptr(), m2.data_ptr(), out.data_ptr(), 1.0f, at::cuda::getCurrentCUDAStream().stream()));
    return out;
}

blk_plan_t* softmax_plan(const Tensor& src, const I64& acc, const I64& rows, const I64& cols, int64_t* H_out) {
    const int64_t S = (int64_t)rows.size();
    TORCH_CHECK((int64_t)cols.size() == S && (int64_t)acc.size() == S + 1, "srcAccum must have one more entry than the lists");
    const int64_t H = heads_of(src, acc[S], "src");
    const int dt = dtype_code(src), dev = src.get_device();
    std::string key = "s" + std::to_string(dt) + std::to_string(dev) + ":" + std::to_string(H) + "|";
    append(key, rows); append(key, cols); append(key, acc);
    *H_out = H;
    return g_plans.get(key, [&]() {
        blk_plan_t* p = nullptr;
        ok(blk_softmax_plan_create(&p, rows.data(), cols.data(), acc.data(), S, H, dt, dev));
        return p;
    });
}

Tensor aligned(const Tensor& t) { return reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 ? t.clone() : t; }

// ---- autograd nodes: the same backward as upstream (csrc/sparseBlockedAttention.cpp:52-72, :103-114) ----
struct GemmNode : public torch::autograd::Function<GemmNode> {
    static Tensor forward(torch::autograd::AutogradContext* ctx, const Tensor& mat1, const Tensor& mat2, const Tensor& a1,
                          const Tensor& a2, const Tensor& ao, const Tensor& M, const Tensor& N, const Tensor& K, bool t1,
                          bool t2) {
        ctx->save_for_backward({mat1, mat2, a1, a2, ao, M, N, K});
        ctx->saved_data["t1"] = t1;
        ctx->saved_data["t2"] = t2;
        return sparseBlockedGEMMLaunch(mat1, mat2, a1, a2, ao, M, N, K, t1, t2);
    }
    static torch::autograd::variable_list backward(torch::autograd::AutogradContext* ctx,
                                                   torch::autograd::variable_list grads) {
        const auto sv = ctx->get_saved_variables();
        const Tensor g = grads[0].contiguous();
        const Tensor m1 = sv[0].to(g.scalar_type()), m2 = sv[1].to(g.scalar_type());
        const bool t1 = ctx->saved_data["t1"].toBool(), t2 = ctx->saved_data["t2"].toBool();
        // d mat1 = dOut mat2 with lists (M, K, N); d mat2 = dOut^T mat1 with lists (N, K, M)
        Tensor g1 = sparseBlockedGEMMLaunch(g, m2, sv[4], sv[3], sv[2], sv[5], sv[7], sv[6], false, !t2);
        Tensor g2 = sparseBlockedGEMMLaunch(g, m1, sv[4], sv[2], sv[3], sv[6], sv[7], sv[5], true, !t1);
        return {g1.reshape(sv[0].sizes()), g2.reshape(sv[1].sizes()), Tensor(), Tensor(), Tensor(), Tensor(), Tensor(), Tensor(),
                Tensor(), Tensor()};
    }
};

struct SoftmaxNode : public torch::autograd::Function<SoftmaxNode> {
    static Tensor forward(torch::autograd::AutogradContext* ctx, const Tensor& src, const Tensor& acc, const Tensor& rows,
                          const Tensor& cols) {
        Tensor out = sparseBlockedSoftmaxLaunch(src, acc, rows, cols);
        ctx->save_for_backward({out, acc, rows, cols});
        ctx->saved_data["shape"] = src.sizes().vec();
        return out;
    }
    static torch::autograd::variable_list backward(torch::autograd::AutogradContext* ctx,
                                                   torch::autograd::variable_list grads) {
        const auto sv = ctx->get_saved_variables();
        const Tensor g = grads[0].contiguous();
        Tensor gs = sparseBlockedSoftmaxBackwardLaunch(sv[0].to(g.scalar_type()), g, sv[1], sv[2], sv[3]);
        return {gs.reshape(ctx->saved_data["shape"].toIntVector()), Tensor(), Tensor(), Tensor()};
    }
};

}  // namespace

Tensor sparseBlockedGEMMLaunch(const Tensor& mat1, const Tensor& mat2, const Tensor& mat1Accum, const Tensor& mat2Accum,
                               const Tensor& outAccum, const Tensor& MList, const Tensor& NList, const Tensor& KList,
                               const bool transpose1, const bool transpose2) {
    return gemm_launch_host(mat1, mat2, g_lists.get(mat1Accum), g_lists.get(mat2Accum), g_lists.get(outAccum),
                            g_lists.get(MList), g_lists.get(NList), g_lists.get(KList), transpose1, transpose2);
}

Tensor sparseBlockedSoftmaxLaunch(const Tensor& src, const Tensor& accumSrc, const Tensor& rowList, const Tensor& colList) {
    check_operand(src, "src");
    c10::cuda::CUDAGuard guard(src.device());
    int64_t H = 0;
    const I64 acc = g_lists.get(accumSrc);
    blk_plan_t* plan = softmax_plan(src, acc, g_lists.get(rowList), g_lists.get(colList), &H);
    Tensor out = torch::empty({H, acc.back()}, src.options());   // upstream csrc/cuda/spBlkSoftmax.cu:398
    Tensor s = aligned(src);
    ok(blk_softmax_run(plan, s.data_ptr(), out.data_ptr(), 1.0f, at::cuda::getCurrentCUDAStream().stream()));
    return out;
}

Tensor sparseBlockedSoftmaxBackwardLaunch(const Tensor& out, const Tensor& dout, const Tensor& accumSrc, const Tensor& rowList,
                                          const Tensor& colList) {
    check_operand(out, "out");
    check_operand(dout, "dout");
    TORCH_CHECK(out.scalar_type() == dout.scalar_type() && out.numel() == dout.numel(), "out and dout must match");
    c10::cuda::CUDAGuard guard(out.device());
    int64_t H = 0;
    const I64 acc = g_lists.get(accumSrc);
    blk_plan_t* plan = softmax_plan(out, acc, g_lists.get(rowList), g_lists.get(colList), &H);
    Tensor gs = torch::empty({H, acc.back()}, out.options());
    Tensor o = aligned(out), g = aligned(dout);
    ok(blk_softmax_backward_run(plan, o.data_ptr(), g.data_ptr(), gs.data_ptr(), 1.0f,
                                at::cuda::getCurrentCUDAStream().stream()));
    return gs;
}

Tensor sparseBlockedGEMM_op(const Tensor& mat1, const Tensor& mat2, const std::optional<Tensor>& mat1Accum,
                            const std::optional<Tensor>& mat2Accum, const std::optional<Tensor>& outAccum,
                            const std::optional<Tensor>& MList, const std::optional<Tensor>& NList,
                            const std::optional<Tensor>& KList, const bool transpose1, const bool transpose2) {
    const bool have_acc = mat1Accum.has_value() && mat2Accum.has_value() && outAccum.has_value();
    const bool have_lists = MList.has_value() && NList.has_value() && KList.has_value();
    // upstream leaves this to an assert (csrc/sparseBlockedAttention.cpp:17); here it is an error
    TORCH_CHECK(have_acc || have_lists, "sparseBlockedGEMM needs either mat1Accum/mat2Accum/outAccum or MList/NList/KList");
    Tensor a1, a2, ao, M, N, K;
    if (have_acc) { a1 = *mat1Accum; a2 = *mat2Accum; ao = *outAccum; }
    if (have_lists) { M = *MList; N = *NList; K = *KList; }
    if (!have_acc) {
        // offsets = cumsum([0, M*K]) and so on (upstream :22-29), in overflow-checked integer arithmetic
        const I64 m = g_lists.get(M), n = g_lists.get(N), k = g_lists.get(K);
        TORCH_CHECK(m.size() == n.size() && m.size() == k.size(), "MList, NList and KList must have the same length");
        I64 v1(m.size() + 1), v2(m.size() + 1), vo(m.size() + 1);
        ok(blk_offsets_from_lists(m.data(), n.data(), k.data(), (int64_t)m.size(), v1.data(), v2.data(), vo.data()));
        a1 = to_list_tensor(v1, M); a2 = to_list_tensor(v2, M); ao = to_list_tensor(vo, M);
    } else if (!have_lists) {
        // lists from the offsets (upstream :30-40 in float32; exact here)
        const I64 v1 = g_lists.get(a1), v2 = g_lists.get(a2), vo = g_lists.get(ao);
        TORCH_CHECK(v1.size() == v2.size() && v1.size() == vo.size() && !v1.empty(), "the offset tensors must have equal, non-zero lengths");
        I64 m(v1.size() - 1), n(v1.size() - 1), k(v1.size() - 1);
        ok(blk_lists_from_offsets(v1.data(), v2.data(), vo.data(), (int64_t)m.size(), m.data(), n.data(), k.data()));
        M = to_list_tensor(m, a1); N = to_list_tensor(n, a1); K = to_list_tensor(k, a1);
    }
    return GemmNode::apply(mat1, mat2, a1, a2, ao, M, N, K, transpose1, transpose2);
}

Tensor sparseBlockedSoftmax_op(const Tensor& src, const std::optional<Tensor>& rowList, const std::optional<Tensor>& colList,
                               const std::optional<Tensor>& srcAccum) {
    TORCH_CHECK(rowList.has_value() && colList.has_value(), "sparseBlockedSoftmax needs rowList and colList");
    Tensor acc;
    if (srcAccum.has_value()) {
        acc = *srcAccum;
    } else {
        const I64 r = g_lists.get(*rowList), c = g_lists.get(*colList);
        TORCH_CHECK(r.size() == c.size(), "rowList and colList must have the same length");
        I64 v(r.size() + 1);
        ok(blk_softmax_offsets(r.data(), c.data(), (int64_t)r.size(), v.data()));
        acc = to_list_tensor(v, *rowList);
    }
    return SoftmaxNode::apply(src, acc, *rowList, *colList);
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "blockAttention: sparseBlockedGEMM / sparseBlockedSoftmax over libblkattn (NVIDIA B200, sm_100a)";
    namespace py = pybind11;
    m.def("sparseBlockedGEMM", &sparseBlockedGEMM_op, "sparseBlockedGEMM forward", py::arg("mat1"), py::arg("mat2"),
          py::arg("mat1Accum") = py::none(), py::arg("mat2Accum") = py::none(), py::arg("outAccum") = py::none(),
          py::arg("MList") = py::none(), py::arg("NList") = py::none(), py::arg("KList") = py::none(),
          py::arg("transpose1") = false, py::arg("transpose2") = false);
    m.def("sparseBlockedSoftmax", &sparseBlockedSoftmax_op, "sparseBlockedSoftmax forward", py::arg("src"),
          py::arg("rowList") = py::none(), py::arg("colList") = py::none(), py::arg("srcAccum") = py::none());
    m.def("sparseBlockedGEMMLaunch", &sparseBlockedGEMMLaunch, py::arg("mat1"), py::arg("mat2"), py::arg("mat1Accum"),
          py::arg("mat2Accum"), py::arg("outAccum"), py::arg("MList"), py::arg("NList"), py::arg("KList"),
          py::arg("transpose1") = false, py::arg("transpose2") = false);
    m.def("sparseBlockedSoftmaxLaunch", &sparseBlockedSoftmaxLaunch);
    m.def("sparseBlockedSoftmaxBackwardLaunch", &sparseBlockedSoftmaxBackwardLaunch);
}
