// CudaBackend / CudaSegment — the host side of the B200 backend, written against VKNN's pluggable backend
// interface (include/vknn/backend_class.h:15-47, include/vknn/segment.h:12-23) and registered with
// VKNN_REGISTER_BACKEND (include/vknn/backend_registry.h:29-32). It never touches CUDA directly: all device
// work goes through the C-ABI of libvknn_cuda (include/vknn_cuda.h).
//
// What the reference's planner hands over (src/core/session.cpp:393-422,486-585): a contiguous run of nodes in
// topological order and, after compileSegment() returns, the segment's boundary input/output sets. Initializers
// used by MatMul are erased from the graph once all segments are compiled (session.cpp:594-625), so weights are
// uploaded inside compileSegment(); everything that depends on the boundary sets (which intermediates must stay
// materialised) is planned lazily on the first run().
//
// Planning turns the node run into a short list of kernel launches:
//   * Reshape / Transpose / Gather(scalar index) / Squeeze / Unsqueeze / Flatten / Identity become VIEWS (offset +
//     strides over a device buffer); a copy is made only where a consumer cannot take the strides;
//   * Transpose(K) -> MatMul -> Mul(scale) [FusedPointwise{Mul, Add mask}] -> Softmax -> MatMul collapses into one
//     fused attention launch reading Q/K/V through their strides, and writes its output directly in the layout
//     the following head-merge Transpose/Reshape asks for;
//   * MatMul carries its fusedBias, an exported erf-GELU tail (Div, Erf, Add, FusedPointwise{Mul, Mul}) and a
//     following residual Add in the GEMM epilogue;
//   * anything else on the supported list runs as its own kernel (LayerNorm, Softmax, pointwise programs).
// After one eager run the launch list is captured into a CUDA graph (the analogue of the reference's pre-recorded
// command buffer, src/backend/vulkan/vk_backend.cpp:1009-1210) and replayed.
//
// There is no CPU fallback: what supportsNode() declines is refused by the planner (Status::Unsupported) when no
// other backend is configured, and a failing device call surfaces as vknn::Error.
#include "vknn/backend.h"
#include "vknn/binary_type.h"
#include "vknn/error.h"
#include "vknn/logging.h"
#include "vknn/profiler.h"
#include "vknn/unary_type.h"
#include "vknn_cuda.h"

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <sstream>
#include <map>
#include <memory>
#include <set>
#include <string>
#include <vector>

namespace vknn {

    // The reference leaves DeviceStorage to the backend (include/vknn/device_storage.h:8). Host builds contain no
    // other definition.
    struct DeviceStorage {
        void  *ptr   = nullptr;
        size_t bytes = 0;
    };

    namespace {

        constexpr BackendKind kCuda = static_cast<BackendKind>(2); // first value after Vulkan = 0, Cpu = 1
        // Device selection travels in a spare slot of Config::hints (include/vknn/config_struct.h:74-88; the reference's
        // Hint enum ends at 4, include/vknn/hint.h:9-15): cfg.setHint(static_cast<Hint>(8), ordinal + 1). 0 (the production
        // default of every hint) means "not set": then the environment variable VKNN_CUDA_DEVICE, else device 0. One
        // Session drives one device; a multi-GPU application creates one Session per device (per thread or process).
        constexpr int kHintCudaDevice = 8;

        [[noreturn]] void fail(Status s, const std::string &msg) { throw Error(s, "CUDA backend: " + msg); }

        void check(vkc_ctx *ctx, int rc, const char *what) {
            if (rc == VKC_OK) return;
            std::string msg = std::string(what) + ": " + (ctx ? vkc_last_error(ctx) : "no context");
            switch (rc) {
                case VKC_ERR_INVALID: fail(Status::InvalidArgument, msg);
                case VKC_ERR_UNSUPPORTED: fail(Status::Unsupported, msg);
                case VKC_ERR_DEVICE: fail(Status::DeviceLost, msg);
                default: fail(Status::RuntimeError, msg);
            }
        }

        // dtype of a caller-registered device buffer: fp32 or fp16, row-major (the only boundary formats this backend has)
        int extDtype(DType d, const std::string &name) {
            if (d == DType::Float32) return VKC_F32;
            if (d == DType::Float16) return VKC_F16;
            fail(Status::Unsupported, "device-resident tensor " + name + ": only Float32 and Float16 buffers are supported");
        }

        int64_t prod(const Shape &s) {
            int64_t n = 1;
            for (int64_t d : s) n *= d;
            return n;
        }
        std::vector<int64_t> denseStrides(const Shape &s) {
            std::vector<int64_t> st(s.size(), 1);
            for (int i = (int) s.size() - 2; i >= 0; --i) st[i] = st[i + 1] * s[i + 1];
            return st;
        }

        struct View {
            int                  buf = -1; // index into CudaSegment::bufs_
            int64_t              offset = 0;
            Shape                shape;
            std::vector<int64_t> strides;
            bool                 contiguous() const {
                int64_t expect = 1;
                for (int i = (int) shape.size() - 1; i >= 0; --i) {
                    if (shape[i] != 1 && strides[i] != expect) return false;
                    expect *= shape[i];
                }
                return true;
            }
        };

        struct Step {
            enum Kind { Gemm, Attn, LayerNorm, Pointwise, Softmax, Copy, Reduce, Rows, GatherRt } kind;
            // Rows: a -> d through the offset tables b (source) / c (destination), `rows` rows of `norm` elements.
            // GatherRt: data a, index tensor b, M = outer, N = axis size, K = index count, norm = inner elements.
            int reduceOp = 0;
            // generic operands (device pointers resolved at plan time)
            const void *a = nullptr, *b = nullptr, *c = nullptr;
            void       *d = nullptr;
            const float *bias = nullptr, *gamma = nullptr, *beta = nullptr, *mask = nullptr;
            int64_t     M = 0, N = 0, K = 0, batch = 1, sa = 0, sb = 0, sd = 0, lda = 0, ldb = 0, ldd = 0;
            int         bLayout = VKC_B_KN, epilogue = 0;
            int         gemmConfig = -1; // tensor-core kernel configuration chosen by the autotune (-1: built-in choice)
            int64_t     B = 0, Hq = 0, Hkv = 0, Sq = 0, Skv = 0, D = 0;
            int64_t     qs[3], ks[3], vs[3], os[3];
            float       scale = 1.f, eps = 1e-5f;
            int64_t     rows = 0, norm = 0;
            std::vector<int64_t>      shape, opStrides, inStrides, outStrides; // outStrides empty: dense output
            std::vector<int32_t>      pwSteps;
            std::vector<float>        pwParams;
            std::vector<const void *> operands;
            int64_t                   inOffset = 0;
            std::string               label;
            int                       node = -1; // graph node this launch was planned for (profiler records)
        };

        bool isScalarInit(const Graph &g, TensorId id, float *value) {
            auto it = g.initializers.find(id);
            if (it == g.initializers.end()) return false;
            const TensorDesc &d = g.desc(id);
            if (prod(d.shape) != 1 && !d.shape.empty()) return false;
            if (d.dtype == DType::Float32) *value = it->second.f32()[0];
            else if (d.dtype == DType::Float16) *value = halfToFloat(reinterpret_cast<const fp16_t *>(it->second.bytes.data())[0]);
            else return false;
            return true;
        }

    } // namespace

    class CudaBackend;

    class CudaSegment: public Segment {
      public:
        CudaSegment(CudaBackend *be, vkc_ctx *ctx, const std::vector<int> &nodes, Graph &g, const Config &cfg);
        ~CudaSegment() override;
        void run(ExecContext &ctx) override;

      private:
        struct DevBuf {
            void  *ptr   = nullptr;
            size_t bytes = 0;
        };
        vkc_ctx     *ctx_;
        const Graph *g_;
        int          dtype_;     // storage type of activations and matrices
        size_t       esize_;
        bool         useGraph_ = true;
        bool         planned_  = false;
        int          runs_     = 0;
        vkc_graph   *graph_    = nullptr;

        std::vector<DevBuf>         bufs_;
        std::map<TensorId, View>    views_;     // every tensor the segment touches on the device
        std::map<TensorId, float *> f32Inits_;  // biases, LayerNorm gamma/beta, masks: kept fp32
        std::map<TensorId, std::vector<int64_t>> i64Inits_; // Reshape shapes, Gather indices (host only)
        std::map<TensorId, float>   scalarInits_;
        std::set<TensorId>          initIds_;   // initializers seen at compile time (the graph forgets MatMul weights afterwards)
        std::vector<Step>           steps_;
        std::set<TensorId>          boundaryOut_;

        int   newBuffer(size_t bytes);
        View  newTensor(TensorId id, const Shape &shape);
        const void *ptrOf(const View &v) const { return static_cast<const char *>(bufs_[v.buf].ptr) + v.offset * (int64_t) esize_; }
        void *ptrOf(const View &v) { return static_cast<char *>(bufs_[v.buf].ptr) + v.offset * (int64_t) esize_; }
        View  materialize(const View &v, const std::string &why);
        const float *f32Init(TensorId id);
        void  uploadInitializers(const std::vector<int> &nodes, Graph &g);
        void  plan();
        void  launch(const Step &s);
        int   consumersInSegment(TensorId id, std::vector<int> *who) const;
        bool  internalOnly(TensorId id) const { return boundaryOut_.count(id) == 0; }

        void tuneGemms();
        CudaBackend *be_ = nullptr;
        int          tuning_ = 0; // Hint::Tuning: 0 none, 1 fast, 2 thorough

        bool tryAttention(size_t pos, std::set<int> &done);
        void planMatMul(size_t pos, std::set<int> &done);
        void planPointwise(const Node &n);
        void planPatchConv(const Node &n);
    };

    class CudaBackend: public Backend {
      public:
        CudaBackend() {
            // The context is created in configure(), which knows the device the Config asks for; available() is asked
            // before that (src/core/session.cpp:340-348) and only needs to know that a usable GPU exists.
            if (vkc_device_count(&deviceCount_) != VKC_OK) deviceCount_ = 0;
        }
        ~CudaBackend() override {
            if (ctx_) vkc_ctx_destroy(ctx_);
        }
        BackendKind kind() const override { return kCuda; }
        const char *name() const override { return "CUDA"; }
        bool        available() const override { return deviceCount_ > 0; }
        void        configure(const Config &cfg) override {
            precision_ = cfg.precision;
            int want   = cfg.hint(static_cast<Hint>(kHintCudaDevice), 0) - 1;
            if (want < 0) {
                const char *e = std::getenv("VKNN_CUDA_DEVICE");
                want          = e ? std::atoi(e) : 0;
            }
            if (ctx_ && want == device_) return;
            if (want < 0 || want >= deviceCount_) fail(Status::InvalidArgument, "device ordinal " + std::to_string(want) + " does not exist (" + std::to_string(deviceCount_) + " visible)");
            if (ctx_) vkc_ctx_destroy(ctx_);
            ctx_ = nullptr;
            if (vkc_ctx_create(want, &ctx_) != VKC_OK) {
                ctx_ = nullptr;
                fail(Status::RuntimeError, "device " + std::to_string(want) + " is not a usable sm_100 GPU");
            }
            device_ = want;
        }
        int device() const { return device_; }

        bool supports(OpType t, DType dt) const override {
            if (dt != DType::Float32 && dt != DType::Float16) return false;
            switch (t) {
                case OpType::MatMul:
                case OpType::Softmax:
                case OpType::LayerNorm:
                case OpType::Binary:
                case OpType::Add:
                case OpType::Unary:
                case OpType::FusedPointwise:
                case OpType::Transpose:
                case OpType::Reshape:
                case OpType::Gather:
                case OpType::Squeeze:
                case OpType::Unsqueeze:
                case OpType::Flatten:
                case OpType::Identity:
                case OpType::Slice:
                case OpType::Split:
                case OpType::Expand:
                case OpType::Tile:
                case OpType::Concat:
                case OpType::Conv:
                case OpType::Reduce:
                case OpType::Where:
                case OpType::ScatterND:
                case OpType::Einsum:
                case OpType::Equal:
                case OpType::Greater:
                case OpType::GreaterEqual: return true;
                default: return false;
            }
        }

        // Shape-aware refusals mirror what the kernels cover; the reference's Vulkan backend gates the same way
        // (src/backend/vulkan/vk_backend.cpp:189-434).
        bool supportsNode(const Graph &g, const Node &nd, DType dt) const override {
            if (!supports(nd.type, dt)) return false;
            if (nd.type != OpType::FusedPointwise && nd.attr.has("pw_steps")) return false; // producer-carried epilogue: not emitted today
            auto rank = [&](TensorId id) { return (int) g.desc(id).shape.size(); };
            for (TensorId o : nd.outputs)
                if (o != kNoTensor && (rank(o) == 0 || rank(o) > 8)) return false;
            switch (nd.type) {
                case OpType::Softmax: {
                    int64_t axis = nd.attr.geti("axis", -1), r = rank(nd.inputs[0]);
                    return axis == -1 || axis == r - 1;
                }
                case OpType::LayerNorm: {
                    if (nd.inputs.size() < 2 || !g.isInitializer(nd.inputs[1])) return false;
                    if (nd.inputs.size() > 2 && nd.inputs[2] != kNoTensor && !g.isInitializer(nd.inputs[2])) return false;
                    int64_t axis = nd.attr.geti("axis", -1), r = rank(nd.inputs[0]);
                    return axis == -1 || axis == r - 1;
                }
                case OpType::Gather: {
                    // constant int64 indices (one: a view; several: a row table built at plan time) or a floating
                    // index tensor computed inside the segment (src/backend/cpu/ops/gather.cpp:27-30)
                    const TensorDesc &d = g.desc(nd.inputs[1]);
                    if (g.desc(nd.inputs[0]).dtype == DType::Int64) return false;
                    if (g.isInitializer(nd.inputs[1])) return d.dtype == DType::Int64 && prod(d.shape) >= 1;
                    if (d.dtype != DType::Float32 && d.dtype != DType::Float16) return false;
                    // The index tensor lives in the segment's storage type. The reference casts from fp32
                    // (gather.cpp:27-30); f16 storage holds integers exactly only up to 2048, so a longer axis would
                    // fetch wrong rows silently: leave such a node to another backend.
                    const Shape &ds   = g.desc(nd.inputs[0]).shape;
                    int64_t      axis = nd.attr.geti("axis", 0);
                    if (axis < 0) axis += (int64_t) ds.size();
                    if (axis < 0 || axis >= (int64_t) ds.size()) return false;
                    return precision_ == Precision::High ? ds[(size_t) axis] <= (1 << 24) : ds[(size_t) axis] <= 2048;
                }
                case OpType::Einsum: {
                    // only the outer product (the rotary frequency tables); the two batched equations arrive as MatMul
                    // (src/import/lower_einsum.cpp:36-110)
                    std::string eq;
                    for (char c : nd.attr.gets("equation", ""))
                        if (c != ' ' && c != '\t') eq += c;
                    if (eq != "i,j->ij" || nd.inputs.size() != 2) return false;
                    for (TensorId in : nd.inputs)
                        if (g.desc(in).dtype != DType::Float32 && g.desc(in).dtype != DType::Float16) return false;
                    return true;
                }
                case OpType::ScatterND: {
                    // constant int64 indices: destinations (and which duplicate wins) are resolved at plan time
                    if (nd.inputs.size() != 3 || !g.isInitializer(nd.inputs[1]) || g.desc(nd.inputs[1]).dtype != DType::Int64) return false;
                    const TensorDesc &dd = g.desc(nd.inputs[0]), &ud = g.desc(nd.inputs[2]);
                    // int64 data is shape arithmetic: its consumers (Reshape / Expand / Slice parameters) need constants at
                    // plan time, so such a node is of no use on a device; it stays with the backend that owns the host tensors
                    if (dd.dtype == DType::Int64 || ud.dtype == DType::Int64 || dd.shape.empty()) return false;
                    const Shape &is = g.desc(nd.inputs[1]).shape;
                    return !is.empty() && is.back() >= 1 && is.back() <= (int64_t) dd.shape.size();
                }
                case OpType::MatMul: {
                    const Shape &a = g.desc(nd.inputs[0]).shape, &b = g.desc(nd.inputs[1]).shape;
                    if (a.size() < 2 || b.size() < 2) return false;
                    if (b.size() > 2 && b.size() != a.size()) return false; // mixed-rank batch broadcast: not covered
                    for (size_t i = 0; i + 2 < b.size() && b.size() > 2; ++i)
                        if (b[i] != a[i] && b[i] != 1) return false;
                    return true;
                }
                case OpType::Binary:
                case OpType::Add: {
                    // one operand must already have the output shape (it becomes the primary of the step program)
                    const Shape &o = g.desc(nd.outputs[0]).shape;
                    bool         a = g.desc(nd.inputs[0]).shape == o && !g.isInitializer(nd.inputs[0]);
                    bool         b = g.desc(nd.inputs[1]).shape == o && !g.isInitializer(nd.inputs[1]);
                    if (a) return true;
                    int code = nd.type == OpType::Add ? (int) BinaryType::Add : nd.subOp;
                    bool commutative = code == (int) BinaryType::Mul || code == (int) BinaryType::Add || code == (int) BinaryType::Max ||
                                       code == (int) BinaryType::Min;
                    return b && commutative;
                }
                case OpType::FusedPointwise: return !g.isInitializer(nd.inputs[0]);
                case OpType::Equal:
                case OpType::Greater:
                case OpType::GreaterEqual: {
                    // like Binary: one runtime operand must already have the output shape (the other may broadcast)
                    const Shape &o = g.desc(nd.outputs[0]).shape;
                    return (g.desc(nd.inputs[0]).shape == o && !g.isInitializer(nd.inputs[0])) || (g.desc(nd.inputs[1]).shape == o && !g.isInitializer(nd.inputs[1]));
                }
                case OpType::Where: { // the condition drives the step program; one that broadcasts is expanded to the output shape first
                    if (nd.inputs.size() != 3) return false;
                    for (TensorId in : nd.inputs)
                        if (g.desc(in).dtype != DType::Float32 && g.desc(in).dtype != DType::Float16) return false;
                    const Shape &c = g.desc(nd.inputs[0]).shape, &o = g.desc(nd.outputs[0]).shape;
                    if (c.size() > o.size()) return false;
                    for (size_t i = 0; i < c.size(); ++i) {
                        const int64_t cd = c[c.size() - 1 - i], od = o[o.size() - 1 - i];
                        if (cd != od && cd != 1) return false;
                    }
                    return true;
                }
                case OpType::Reduce: {
                    if (nd.inputs.size() > 1 && nd.inputs[1] != kNoTensor && !g.isInitializer(nd.inputs[1])) return false;
                    return nd.subOp >= 0 && nd.subOp <= 5 && !g.isInitializer(nd.inputs[0]);
                }
                case OpType::Slice:
                case OpType::Expand:
                case OpType::Tile: {
                    // parameters must be attributes or int64 initializers (they are read at plan time); Slice steps > 0
                    for (size_t i = 1; i < nd.inputs.size(); ++i)
                        if (nd.inputs[i] != kNoTensor && !g.isInitializer(nd.inputs[i])) return false;
                    if (nd.type == OpType::Slice) {
                        std::vector<int64_t> steps = nd.attr.getints("steps");
                        if (steps.empty() && nd.inputs.size() > 4 && nd.inputs[4] != kNoTensor) {
                            auto it = g.initializers.find(nd.inputs[4]);
                            if (it != g.initializers.end()) steps.assign(it->second.i64(), it->second.i64() + prod(g.desc(nd.inputs[4]).shape));
                        }
                        for (int64_t st : steps)
                            if (st <= 0) return false;
                    }
                    return !g.isInitializer(nd.inputs[0]);
                }
                case OpType::Conv: {
                    // patch embedding only: kernel == stride, no padding, no dilation, one group, constant weights —
                    // a non-overlapping convolution is a GEMM over [B*outH*outW, C*kh*kw] patches
                    if (nd.inputs.size() < 2 || !g.isInitializer(nd.inputs[1]) || g.isInitializer(nd.inputs[0])) return false;
                    if (nd.inputs.size() > 2 && nd.inputs[2] != kNoTensor && !g.isInitializer(nd.inputs[2])) return false;
                    const Shape &x = g.desc(nd.inputs[0]).shape, &w = g.desc(nd.inputs[1]).shape;
                    if (x.size() != 4 || w.size() != 4 || w[1] != x[1]) return false;
                    auto ints = [&](const char *k, std::vector<int64_t> d) {
                        const auto &v = nd.attr.getints(k);
                        return v.empty() ? d : v;
                    };
                    const auto st = ints("strides", {1, 1}), pad = ints("pads", {0, 0, 0, 0}), dil = ints("dilations", {1, 1});
                    if (nd.attr.geti("group", 1) != 1 || st[0] != w[2] || st[1] != w[3] || dil[0] != 1 || dil[1] != 1) return false;
                    for (int64_t v : pad)
                        if (v != 0) return false;
                    return nd.fusedAct == ActType::None && nd.fusedResidual == kNoTensor && x[2] >= w[2] && x[3] >= w[3];
                }
                default: return true;
            }
        }

        std::unique_ptr<Segment> compileSegment(const std::vector<int> &nodeIdx, Graph &g, const Config &cfg) override {
            if (!ctx_) configure(cfg);
            return std::unique_ptr<Segment>(new CudaSegment(this, ctx_, nodeIdx, g, cfg));
        }

        Precision precision() const { return precision_; }

        // ---- GEMM autotune table and its file (the CUDA counterpart of the tuning section of the reference's unified
        // cache, src/backend/vulkan/vk_backend.cpp:445-545; flushed by finalize() like saveCaches there). The file is
        // "<cfg.cacheFile>.cuda": text, one "key config" pair per line under a header that names the format and the GPU,
        // so a table measured on another device is ignored. Weights need no cache section: the kernels read the
        // reference's row-major [K,N] initializers as they are (fp16 ".vxm" weights upload byte for byte).
        void loadTuning(const Config &cfg) {
            if (tuneLoaded_) return;
            tuneLoaded_ = true;
            if (cfg.cacheFile.empty() || !cfg.cachesTuning()) return;
            tuneFile_ = cfg.cacheFile + ".cuda";
            std::ifstream f(tuneFile_);
            std::string   magic, gpu;
            if (!f || !std::getline(f, magic) || magic != "VKNNCUDA-TUNE-1" || !std::getline(f, gpu) || gpu != gpuTag()) return;
            std::string key;
            int         cfgIdx;
            while (f >> key >> cfgIdx)
                if (cfgIdx >= -1 && cfgIdx < vkc_gemm_config_count()) tune_[key] = cfgIdx;
        }
        bool lookupTuning(const std::string &key, int *cfgIdx) const {
            auto it = tune_.find(key);
            if (it == tune_.end()) return false;
            *cfgIdx = it->second;
            return true;
        }
        void storeTuning(const std::string &key, int cfgIdx) {
            tune_[key]  = cfgIdx;
            tuneDirty_ = true;
        }
        void finalize() override {
            if (!tuneDirty_ || tuneFile_.empty()) return;
            std::ofstream f(tuneFile_, std::ios::trunc);
            if (!f) {
                VKNN_WARN << "CUDA backend: cannot write " << tuneFile_;
                return;
            }
            f << "VKNNCUDA-TUNE-1\n" << gpuTag() << "\n";
            for (const auto &kv : tune_) f << kv.first << " " << kv.second << "\n";
            tuneDirty_ = false;
        }
        std::string gpuTag() const {
            char name[128] = "unknown";
            int  sms = 0, mhz = 0;
            if (ctx_) vkc_device_info(ctx_, name, sizeof name, &sms, &mhz);
            std::string tag = name;
            for (char &c : tag)
                if (c == ' ') c = '_';
            return tag + "/sms=" + std::to_string(sms) + "/mhz=" + std::to_string(mhz) + "/configs=" + std::to_string(vkc_gemm_config_count());
        }

      private:
        vkc_ctx  *ctx_         = nullptr;
        int       deviceCount_ = 0, device_ = -1;
        Precision precision_   = Precision::Low;
        std::map<std::string, int> tune_;
        std::string                tuneFile_;
        bool                       tuneLoaded_ = false, tuneDirty_ = false;
    };

    VKNN_REGISTER_BACKEND(kCuda, CudaBackend);

    // ------------------------------------------------------------------------------------------------------------
    CudaSegment::CudaSegment(CudaBackend *be, vkc_ctx *ctx, const std::vector<int> &nodes, Graph &g, const Config &cfg): ctx_(ctx), g_(&g) {
        backend = be;
        nodeIdx = nodes;
        dtype_  = cfg.precision == Precision::High ? VKC_F32 : VKC_F16;
        be_     = be;
        tuning_ = cfg.hint(Hint::Tuning, (int) Mode::Fast);
        be->loadTuning(cfg);
        esize_  = dtype_ == VKC_F32 ? 4 : 2;
        uploadInitializers(nodes, g);
    }

    CudaSegment::~CudaSegment() {
        if (graph_) vkc_graph_destroy(ctx_, graph_);
        vkc_sync(ctx_, nullptr);
        for (auto &b : bufs_)
            if (b.ptr) vkc_free(ctx_, b.ptr);
        for (auto &kv : f32Inits_)
            if (kv.second) vkc_free(ctx_, kv.second);
    }

    int CudaSegment::newBuffer(size_t bytes) {
        DevBuf b;
        b.bytes = std::max<size_t>(bytes, 16);
        check(ctx_, vkc_alloc(ctx_, b.bytes, &b.ptr), "vkc_alloc");
        bufs_.push_back(b);
        return (int) bufs_.size() - 1;
    }

    View CudaSegment::newTensor(TensorId id, const Shape &shape) {
        View v;
        v.buf     = newBuffer((size_t) prod(shape) * esize_);
        v.shape   = shape;
        v.strides = denseStrides(shape);
        if (id != kNoTensor) views_[id] = v;
        return v;
    }

    // Weights and constants go to the device while the graph still holds them.
    void CudaSegment::uploadInitializers(const std::vector<int> &nodes, Graph &g) {
        for (int ni : nodes) {
            const Node &n = g.nodes[ni];
            for (TensorId in : n.inputs) {
                if (in == kNoTensor || !g.isInitializer(in) || views_.count(in) || f32Inits_.count(in) || i64Inits_.count(in)) continue;
                const TensorDesc &d  = g.desc(in);
                const HostBuffer &hb = g.initializers.at(in);
                initIds_.insert(in);
                const int64_t     ne = std::max<int64_t>(prod(d.shape), d.shape.empty() ? 1 : 0);
                if (d.dtype == DType::Int64) {
                    i64Inits_[in].assign(hb.i64(), hb.i64() + ne);
                    continue;
                }
                if (d.dtype != DType::Float32 && d.dtype != DType::Float16) fail(Status::Unsupported, "initializer " + d.name + " has an unsupported dtype");
                const int src = d.dtype == DType::Float32 ? VKC_F32 : VKC_F16;
                float     sv;
                if (isScalarInit(g, in, &sv)) scalarInits_[in] = sv;
                const bool keepF32 = (n.type == OpType::MatMul && in == n.fusedBias) || (n.type == OpType::Conv && n.inputs.size() > 2 && in == n.inputs[2]) || (n.type == OpType::LayerNorm && (in == n.inputs[1] || (n.inputs.size() > 2 && in == n.inputs[2])));
                if (keepF32) {
                    void *p = nullptr;
                    check(ctx_, vkc_alloc(ctx_, (size_t) ne * 4, &p), "vkc_alloc");
                    check(ctx_, vkc_upload(ctx_, p, VKC_F32, hb.bytes.data(), src, ne, nullptr), "vkc_upload");
                    f32Inits_[in] = static_cast<float *>(p);
                    continue;
                }
                Shape shape = d.shape.empty() ? Shape {1} : d.shape;
                View  v     = newTensor(in, shape);
                check(ctx_, vkc_upload(ctx_, ptrOf(v), dtype_, hb.bytes.data(), src, ne, nullptr), "vkc_upload");
            }
        }
        check(ctx_, vkc_sync(ctx_, nullptr), "vkc_sync"); // the host buffers may be freed right after compileSegment
    }

    const float *CudaSegment::f32Init(TensorId id) {
        auto it = f32Inits_.find(id);
        if (it != f32Inits_.end()) return it->second;
        // an initializer that was uploaded in storage precision for another use: convert a private fp32 copy
        auto vt = views_.find(id);
        if (vt == views_.end()) fail(Status::RuntimeError, "missing initializer on the device");
        const int64_t ne = prod(vt->second.shape);
        void         *p  = nullptr;
        check(ctx_, vkc_alloc(ctx_, (size_t) ne * 4, &p), "vkc_alloc");
        check(ctx_, vkc_convert(ctx_, p, VKC_F32, ptrOf(vt->second), dtype_, ne, nullptr), "vkc_convert");
        f32Inits_[id] = static_cast<float *>(p);
        return f32Inits_[id];
    }

    int CudaSegment::consumersInSegment(TensorId id, std::vector<int> *who) const {
        int c = 0;
        for (size_t k = 0; k < nodeIdx.size(); ++k) {
            const Node &n = g_->nodes[nodeIdx[k]];
            for (TensorId in : n.inputs)
                if (in == id) {
                    ++c;
                    if (who) who->push_back((int) k);
                }
        }
        return c;
    }

    View CudaSegment::materialize(const View &v, const std::string &why) {
        if (v.contiguous()) {
            View d    = v;
            d.strides = denseStrides(v.shape);
            return d;
        }
        View d = newTensor(kNoTensor, v.shape);
        Step s;
        s.kind      = Step::Copy;
        s.a         = bufs_[v.buf].ptr;
        s.d         = ptrOf(d);
        s.shape     = v.shape;
        s.inStrides = v.strides;
        s.inOffset  = v.offset;
        s.label     = "copy(" + why + ")";
        steps_.push_back(s);
        return d;
    }

    // Transpose(K) -> MatMul(Q,K^T) -> Mul(scale) | FusedPointwise{Mul scale, Add mask} -> Softmax -> MatMul(P,V)
    bool CudaSegment::tryAttention(size_t pos, std::set<int> &done) {
        const Graph &g  = *g_;
        const Node  &m1 = g.nodes[nodeIdx[pos]];
        if (m1.type != OpType::MatMul || m1.fusedBias != kNoTensor) return false;
        auto single = [&](TensorId t, int *k) {
            std::vector<int> who;
            if (consumersInSegment(t, &who) != 1 || !internalOnly(t)) return false;
            *k = who[0];
            return true;
        };
        int kScale, kSoft, kPV;
        if (!single(m1.outputs[0], &kScale)) return false;
        const Node &sc    = g.nodes[nodeIdx[kScale]];
        float       scale = 0.f;
        const float *mask = nullptr;
        TensorId    maskId = kNoTensor;
        if (sc.type == OpType::Binary && sc.subOp == (int) BinaryType::Mul) {
            TensorId other = sc.inputs[0] == m1.outputs[0] ? sc.inputs[1] : sc.inputs[0];
            if (!scalarInits_.count(other)) return false;
            scale = scalarInits_[other];
        } else if (sc.type == OpType::FusedPointwise && sc.inputs[0] == m1.outputs[0]) {
            const auto &st = sc.attr.getints("pw_steps");
            if (st.size() != 8 || st[0] != 0 || st[1] != (int) BinaryType::Mul || st[4] != 0 || st[5] != (int) BinaryType::Add) return false;
            TensorId sId = sc.inputs[(size_t) st[2]], mId = sc.inputs[(size_t) st[6]];
            if (!scalarInits_.count(sId) || !initIds_.count(mId)) return false;
            scale  = scalarInits_[sId];
            maskId = mId;
        } else {
            return false;
        }
        if (!(scale > 0.f)) return false;
        if (!single(sc.outputs[0], &kSoft)) return false;
        const Node &sm = g.nodes[nodeIdx[kSoft]];
        if (sm.type != OpType::Softmax) return false;
        if (!single(sm.outputs[0], &kPV)) return false;
        const Node &m2 = g.nodes[nodeIdx[kPV]];
        if (m2.type != OpType::MatMul || m2.inputs[0] != sm.outputs[0] || m2.fusedBias != kNoTensor) return false;

        View q = views_.at(m1.inputs[0]), kt = views_.at(m1.inputs[1]), v = views_.at(m2.inputs[1]);
        const size_t r = q.shape.size();
        if (r < 2 || r > 4 || kt.shape.size() != r || v.shape.size() != r) return false;
        // K^T must be a transposed view of a tensor whose head dim is contiguous
        if (kt.strides[r - 2] != 1 || q.strides[r - 1] != 1 || v.strides[r - 1] != 1) return false;
        auto pad4 = [&](View x) {
            while (x.shape.size() < 4) {
                x.shape.insert(x.shape.begin(), 1);
                x.strides.insert(x.strides.begin(), x.shape[1] * x.strides[0]);
            }
            return x;
        };
        q  = pad4(q);
        kt = pad4(kt);
        v  = pad4(v);
        const int64_t B = q.shape[0], Hq = q.shape[1], Sq = q.shape[2], D = q.shape[3], Skv = kt.shape[3];
        const int64_t Hkv = kt.shape[1];
        if (kt.shape[0] != B || kt.shape[2] != D || v.shape[0] != B || v.shape[1] != Hkv || v.shape[2] != Skv || v.shape[3] != D) return false;
        if (Hkv != Hq) return false; // grouped heads reach this backend as the batch-broadcast MatMul form, see supportsNode
        if (maskId != kNoTensor) {
            const Shape &ms = g.desc(maskId).shape;
            if (prod(ms) != Sq * Skv || ms.size() < 2 || ms[ms.size() - 1] != Skv || ms[ms.size() - 2] != Sq) return false; // one [Sq,Skv] mask shared by all units
            mask = f32Init(maskId);
        }
        // Output layout: if the only consumer is the head-merge Transpose(0,2,1,3), write [B,Sq,H,D] directly.
        const TensorId outId = m2.outputs[0];
        const Shape    oshape = g.desc(outId).shape;
        int            kT;
        bool           merged = false;
        View           o;
        if (r == 4 && single(outId, &kT)) {
            const Node &tn = g.nodes[nodeIdx[kT]];
            std::vector<int64_t> perm = tn.attr.getints("perm");
            if (tn.type == OpType::Transpose && perm == std::vector<int64_t> {0, 2, 1, 3}) {
                View t = newTensor(tn.outputs[0], Shape {B, Sq, Hq, D});
                o      = t; // view of the same buffer in [B,H,Sq,D] index order
                o.shape   = Shape {B, Hq, Sq, D};
                o.strides = {t.strides[0], t.strides[2], t.strides[1], t.strides[3]};
                views_[outId] = o;
                done.insert(kT);
                merged = true;
            }
        }
        if (!merged) {
            o = newTensor(outId, oshape);
            o = pad4(o);
        }
        Step s;
        s.kind = Step::Attn;
        s.a = ptrOf(q), s.b = static_cast<const char *>(bufs_[kt.buf].ptr) + kt.offset * (int64_t) esize_, s.c = ptrOf(v), s.d = ptrOf(o);
        s.B = B, s.Hq = Hq, s.Hkv = Hkv, s.Sq = Sq, s.Skv = Skv, s.D = D;
        for (int i = 0; i < 3; ++i) {
            s.qs[i] = q.strides[i];
            s.vs[i] = v.strides[i];
            s.os[i] = o.strides[i];
        }
        s.ks[0] = kt.strides[0], s.ks[1] = kt.strides[1], s.ks[2] = kt.strides[3]; // undo the transpose: seq stride is K^T's last
        s.scale = scale;
        s.mask  = mask;
        s.label = "attention";
        steps_.push_back(s);
        done.insert(kScale);
        done.insert(kSoft);
        done.insert(kPV);
        return true;
    }

    void CudaSegment::planMatMul(size_t pos, std::set<int> &done) {
        const Graph &g = *g_;
        const Node  &n = g.nodes[nodeIdx[pos]];
        View         a = views_.at(n.inputs[0]), b = views_.at(n.inputs[1]);
        const size_t ra = a.shape.size(), rb = b.shape.size();
        const int64_t M = a.shape[ra - 2], K = a.shape[ra - 1], N = b.shape[rb - 1];
        // A: rows with unit stride along K and a dense batch; otherwise copy
        if (a.strides[ra - 1] != 1) a = materialize(a, "matmul A");
        int64_t batch = 1;
        for (size_t i = 0; i + 2 < ra; ++i) batch *= a.shape[i];
        bool aDenseBatch = true;
        {
            int64_t expect = a.strides[ra - 2] * M;
            for (int i = (int) ra - 3; i >= 0; --i) {
                if (a.shape[i] != 1 && a.strides[i] != expect) aDenseBatch = false;
                expect *= a.shape[i];
            }
        }
        if (!aDenseBatch) a = materialize(a, "matmul A batch");
        Step s;
        s.kind = Step::Gemm;
        s.K = K, s.N = N;
        s.lda = a.strides[ra - 2];
        if (b.strides[rb - 1] == 1) {
            s.bLayout = VKC_B_KN;
            s.ldb     = b.strides[rb - 2];
        } else if (b.strides[rb - 2] == 1) {
            s.bLayout = VKC_B_NK; // a transposed view: read it as [N,K] rows
            s.ldb     = b.strides[rb - 1];
        } else {
            b         = materialize(b, "matmul B");
            s.bLayout = VKC_B_KN;
            s.ldb     = b.strides[rb - 2];
        }
        bool bBatched = false;
        if (rb > 2) {
            for (size_t i = 0; i + 2 < rb; ++i)
                if (b.shape[i] != 1) bBatched = true;
        }
        if (!bBatched && s.lda == K) {
            // weights shared by every batch element: fold the batch into M
            s.M = batch * M, s.batch = 1, s.sa = 0, s.sb = 0;
        } else {
            s.M = M, s.batch = batch, s.sa = M * s.lda;
            if (bBatched) {
                // dense batch over B (partial broadcast was refused in supportsNode unless all-ones or equal)
                bool dense = true;
                int64_t expect = (s.bLayout == VKC_B_KN ? K : N) * s.ldb;
                for (int i = (int) rb - 3; i >= 0; --i) {
                    if (b.shape[i] != 1 && b.strides[i] != expect) dense = false;
                    if (b.shape[i] == 1 && a.shape[i] != 1) dense = false;
                    expect *= b.shape[i];
                }
                if (!dense) {
                    b = materialize(b, "matmul B batch");
                    if (s.bLayout == VKC_B_NK) { // materialize() keeps the logical [.., K, N] shape: now row-major KN
                        s.bLayout = VKC_B_KN;
                    }
                    s.ldb = N;
                    // broadcast along some batch dims only is not covered
                    for (size_t i = 0; i + 2 < rb; ++i)
                        if (b.shape[i] != a.shape[i]) fail(Status::Unsupported, "MatMul with a partially broadcast B batch");
                }
                s.sb = (s.bLayout == VKC_B_KN ? K : N) * s.ldb;
            } else {
                s.sb = 0;
            }
        }
        s.a = ptrOf(a);
        s.b = ptrOf(b);
        if (n.fusedBias != kNoTensor) {
            s.bias = f32Init(n.fusedBias);
            s.epilogue |= VKC_EPI_BIAS;
        }
        TensorId outId = n.outputs[0];
        // --- erf-GELU tail: Div(sqrt2) -> Erf -> Add(1) -> FusedPointwise{Mul h, Mul 0.5}
        std::vector<int> who;
        if (internalOnly(outId) && consumersInSegment(outId, &who) == 2) {
            int kDiv = -1, kFp = -1;
            for (int k : who) {
                const Node &c = g.nodes[nodeIdx[k]];
                if (c.type == OpType::Binary && c.subOp == (int) BinaryType::Div && c.inputs[0] == outId) kDiv = k;
                if (c.type == OpType::FusedPointwise) kFp = k;
            }
            if (kDiv >= 0 && kFp >= 0) {
                const Node &dv = g.nodes[nodeIdx[kDiv]];
                auto it = scalarInits_.find(dv.inputs[1]);
                std::vector<int> w2;
                if (it != scalarInits_.end() && std::fabs(it->second - 1.41421356f) < 1e-5f && internalOnly(dv.outputs[0]) &&
                    consumersInSegment(dv.outputs[0], &w2) == 1) {
                    const Node &er = g.nodes[nodeIdx[w2[0]]];
                    std::vector<int> w3;
                    if (er.type == OpType::Unary && er.subOp == (int) UnaryType::Erf && internalOnly(er.outputs[0]) &&
                        consumersInSegment(er.outputs[0], &w3) == 1) {
                        const Node &ad = g.nodes[nodeIdx[w3[0]]];
                        TensorId    one = ad.inputs[0] == er.outputs[0] ? ad.inputs[1] : ad.inputs[0];
                        std::vector<int> w4;
                        const bool isAdd = ad.type == OpType::Add || (ad.type == OpType::Binary && ad.subOp == (int) BinaryType::Add);
                        if (isAdd && scalarInits_.count(one) && scalarInits_[one] == 1.0f && internalOnly(ad.outputs[0]) &&
                            consumersInSegment(ad.outputs[0], &w4) == 1 && w4[0] == kFp) {
                            const Node &fp = g.nodes[nodeIdx[kFp]];
                            const auto &st = fp.attr.getints("pw_steps");
                            if (fp.inputs[0] == ad.outputs[0] && st.size() == 8 && st[0] == 0 && st[1] == (int) BinaryType::Mul && st[4] == 0 &&
                                st[5] == (int) BinaryType::Mul) {
                                TensorId o1 = fp.inputs[(size_t) st[2]], o2 = fp.inputs[(size_t) st[6]];
                                TensorId hId = o1 == outId ? o1 : o2, cId = o1 == outId ? o2 : o1;
                                if (hId == outId && scalarInits_.count(cId) && scalarInits_[cId] == 0.5f) {
                                    s.epilogue |= VKC_EPI_GELU_ERF;
                                    done.insert(kDiv);
                                    done.insert(w2[0]);
                                    done.insert(w3[0]);
                                    done.insert(kFp);
                                    outId = fp.outputs[0];
                                }
                            }
                        }
                    }
                }
            }
        }
        // --- residual Add
        who.clear();
        if (!(s.epilogue & VKC_EPI_GELU_ERF) && internalOnly(outId) && consumersInSegment(outId, &who) == 1) {
            const Node &ad = g.nodes[nodeIdx[who[0]]];
            const bool  isAdd = (ad.type == OpType::Add && ad.fusedAct == ActType::None) || (ad.type == OpType::Binary && ad.subOp == (int) BinaryType::Add);
            if (isAdd && !done.count(who[0])) {
                TensorId other = ad.inputs[0] == outId ? ad.inputs[1] : ad.inputs[0];
                auto     ov    = views_.find(other);
                if (ov != views_.end() && !initIds_.count(other) && g.desc(other).shape == g.desc(outId).shape && ov->second.contiguous()) {
                    s.c = ptrOf(ov->second);
                    s.epilogue |= VKC_EPI_RESIDUAL;
                    done.insert(who[0]);
                    outId = ad.outputs[0];
                }
            }
        }
        View d = newTensor(outId, g.desc(outId).shape);
        s.d    = ptrOf(d);
        s.ldd  = N;
        s.sd   = s.batch > 1 ? M * N : 0;
        s.label = "matmul";
        steps_.push_back(s);
    }

    void CudaSegment::planPointwise(const Node &n) {
        const Graph &g = *g_;
        Step         s;
        s.kind = Step::Pointwise;
        const Shape oshape = g.desc(n.outputs[0]).shape;
        s.shape.assign(oshape.begin(), oshape.end());
        const int rank = (int) oshape.size();
        auto addOperand = [&](TensorId id) -> int {
            View v = materialize(views_.at(id), "pointwise operand");
            s.operands.push_back(ptrOf(v));
            const int off = rank - (int) v.shape.size();
            for (int d = 0; d < rank; ++d) {
                int64_t dim = d < off ? 1 : v.shape[d - off];
                s.opStrides.push_back(dim == 1 ? 0 : v.strides[d - off]);
            }
            return (int) s.operands.size(); // 1-based
        };
        TensorId primary = n.inputs[0];
        if (n.type == OpType::Binary || n.type == OpType::Add) {
            const int code = n.type == OpType::Add ? (int) BinaryType::Add : n.subOp;
            TensorId  other = n.inputs[1];
            if (!(g.desc(primary).shape == oshape && !initIds_.count(primary))) std::swap(primary, other);
            const int oi = addOperand(other);
            s.pwSteps = {0, code, oi, 0};
            s.pwParams = {0.f, 0.f};
            if (n.type == OpType::Add && n.fusedAct != ActType::None) {
                s.pwSteps.insert(s.pwSteps.end(), {2, (int) n.fusedAct, -1, 0});
                s.pwParams.insert(s.pwParams.end(), {n.actLo, n.actHi});
            }
        } else if (n.type == OpType::Equal || n.type == OpType::Greater || n.type == OpType::GreaterEqual) {
            // comparison codes of the step program: 16 ==, 17 >, 18 >=; with the operands swapped 19 <, 20 <=
            int      code  = n.type == OpType::Equal ? 16 : (n.type == OpType::Greater ? 17 : 18);
            TensorId other = n.inputs[1];
            if (!(g.desc(primary).shape == oshape && !initIds_.count(primary))) {
                std::swap(primary, other);
                code = code == 16 ? 16 : (code == 17 ? 19 : 20);
            }
            const int oi = addOperand(other);
            s.pwSteps  = {0, code, oi, 0};
            s.pwParams = {0.f, 0.f};
        } else if (n.type == OpType::Where) {
            const int ix = addOperand(n.inputs[1]), iy = addOperand(n.inputs[2]);
            s.pwSteps  = {3, iy, ix, 0};
            s.pwParams = {0.f, 0.f};
        } else if (n.type == OpType::Unary) {
            s.pwSteps  = {1, n.subOp, -1, 0};
            s.pwParams = {n.actLo, n.actHi};
        } else { // FusedPointwise
            const auto &st = n.attr.getints("pw_steps");
            const auto &pr = n.attr.getfloats("pw_params");
            std::map<int, int> remap; // reference operand index (into node.inputs) -> step-program operand index
            for (size_t i = 0; i + 3 < st.size(); i += 4) {
                int oi = -1;
                if (st[i] == 0) {
                    const int ref = (int) st[i + 2];
                    if (!remap.count(ref)) remap[ref] = addOperand(n.inputs[(size_t) ref]);
                    oi = remap[ref];
                }
                s.pwSteps.insert(s.pwSteps.end(), {(int32_t) st[i], (int32_t) st[i + 1], oi, 0});
            }
            s.pwParams.assign(pr.begin(), pr.end());
            s.pwParams.resize(s.pwSteps.size() / 2, 0.f);
        }
        View px = views_.at(primary);
        if (n.type == OpType::Where && px.shape != oshape) {
            // a broadcasting condition: read it through stride-0 axes, written out once at the output shape
            View      e   = px;
            const int off = rank - (int) px.shape.size();
            e.shape = oshape;
            e.strides.assign((size_t) rank, 0);
            for (int d = off; d < rank; ++d) e.strides[(size_t) d] = px.shape[(size_t) (d - off)] == 1 ? 0 : px.strides[(size_t) (d - off)];
            px = e;
        }
        View x = materialize(px, "pointwise primary");
        View y = newTensor(n.outputs[0], oshape);
        s.a = ptrOf(x);
        s.d = ptrOf(y);
        s.label = "pointwise";
        steps_.push_back(s);
    }

    // Patch embedding: Conv with kernel == stride and no padding over X [B,C,H,W] is Y^T = patches . W^T with
    // patches [B*oh*ow, C*kh*kw] (one strided copy of the [B,oh,ow,C,kh,kw] view of X) and W [O, C*kh*kw] read as [N,K] rows;
    // the GEMM writes [B, oh*ow, O] and the node's NCHW output [B,O,oh,ow] is the transposed view of that buffer.
    // Reference arithmetic: src/backend/cpu/ops/conv.cpp:10-75 (bias, then products in (c, ky, kx) order).
    void CudaSegment::planPatchConv(const Node &n) {
        const Graph &g = *g_;
        const View  &x = views_.at(n.inputs[0]);
        const View  &w = views_.at(n.inputs[1]);
        const int64_t B = x.shape[0], C = x.shape[1], O = w.shape[0], kh = w.shape[2], kw = w.shape[3];
        const Shape  &os = g.desc(n.outputs[0]).shape;
        const int64_t oh = os[2], ow = os[3];
        View p6 = x;
        p6.shape   = {B, oh, ow, C, kh, kw};
        p6.strides = {x.strides[0], x.strides[2] * kh, x.strides[3] * kw, x.strides[1], x.strides[2], x.strides[3]};
        View a = materialize(p6, "conv patches"); // dense [B, oh, ow, C*kh*kw]
        View d = newTensor(kNoTensor, Shape {B, oh * ow, O});
        Step s;
        s.kind = Step::Gemm;
        s.M = B * oh * ow, s.N = O, s.K = C * kh * kw;
        s.batch = 1, s.sa = 0, s.sb = 0, s.sd = 0;
        s.lda = s.K, s.ldb = s.K, s.ldd = O;
        s.bLayout = VKC_B_NK;
        s.a = ptrOf(a), s.b = ptrOf(w), s.d = ptrOf(d);
        if (n.inputs.size() > 2 && n.inputs[2] != kNoTensor) {
            s.bias = f32Init(n.inputs[2]);
            s.epilogue |= VKC_EPI_BIAS;
        }
        s.label = "conv (patch embedding)";
        steps_.push_back(s);
        View y    = d;
        y.shape   = {B, O, oh, ow};
        y.strides = {oh * ow * O, 1, ow * O, O};
        views_[n.outputs[0]] = y;
    }

    void CudaSegment::plan() {
        const Graph &g = *g_;
        boundaryOut_.insert(boundaryOutputs.begin(), boundaryOutputs.end());
        // boundary inputs that are not initializers get a device buffer each
        for (TensorId id : boundaryInputs)
            if (!initIds_.count(id) && !views_.count(id)) newTensor(id, g.desc(id).shape);

        std::set<int> done;
        for (size_t pos = 0; pos < nodeIdx.size(); ++pos) {
            if (done.count((int) pos)) continue;
            const Node  &n      = g.nodes[nodeIdx[pos]];
            const size_t first_ = steps_.size();
            struct TagSteps { // every launch planned for this node carries its index, for the profiler records
                std::vector<Step> &st;
                size_t             from;
                int                node;
                ~TagSteps() {
                    for (size_t i = from; i < st.size(); ++i)
                        if (st[i].node < 0) st[i].node = node;
                }
            } tag_ {steps_, first_, nodeIdx[pos]};
            switch (n.type) {
                case OpType::Reshape:
                case OpType::Squeeze:
                case OpType::Unsqueeze:
                case OpType::Flatten:
                case OpType::Identity: {
                    View v    = materialize(views_.at(n.inputs[0]), "reshape");
                    v.shape   = g.desc(n.outputs[0]).shape; // inferred statically; the shape initializer is not needed
                    v.strides = denseStrides(v.shape);
                    views_[n.outputs[0]] = v;
                    break;
                }
                case OpType::Transpose: {
                    const View          &x    = views_.at(n.inputs[0]);
                    std::vector<int64_t> perm = n.attr.getints("perm");
                    const int            r    = (int) x.shape.size();
                    if ((int) perm.size() != r) {
                        perm.clear();
                        for (int i = r - 1; i >= 0; --i) perm.push_back(i);
                    }
                    View y = x;
                    for (int i = 0; i < r; ++i) {
                        int64_t p = perm[i] < 0 ? perm[i] + r : perm[i];
                        y.shape[i]   = x.shape[p];
                        y.strides[i] = x.strides[p];
                    }
                    views_[n.outputs[0]] = y;
                    break;
                }
                case OpType::Gather: {
                    const View &x    = views_.at(n.inputs[0]);
                    int64_t     axis = n.attr.geti("axis", 0);
                    const int   r    = (int) x.shape.size();
                    if (axis < 0) axis += r;
                    const TensorDesc &id = g.desc(n.inputs[1]);
                    const bool constIdx  = i64Inits_.count(n.inputs[1]) != 0;
                    if (constIdx && i64Inits_.at(n.inputs[1]).size() == 1) {
                        // one constant index: a view
                        int64_t idx = i64Inits_.at(n.inputs[1])[0];
                        if (idx < 0) idx += x.shape[axis];
                        View y = x;
                        y.offset += idx * x.strides[axis];
                        const bool scalar = id.shape.empty() || (id.shape.size() == 1 && id.shape[0] == 1);
                        if (scalar) {
                            y.shape.erase(y.shape.begin() + axis);
                            y.strides.erase(y.strides.begin() + axis);
                            if (y.shape.empty()) {
                                y.shape   = {1};
                                y.strides = {1};
                            }
                        } else {
                            y.shape[axis] = 1;
                        }
                        views_[n.outputs[0]] = y;
                        break;
                    }
                    // several indices: rows of `inner` elements move from a dense copy of the data
                    // (src/backend/cpu/ops/gather.cpp:31-76: out = data[:axis] + indices.shape + data[axis+1:])
                    View    xd    = materialize(x, "gather data");
                    int64_t outer = 1, inner = 1;
                    for (int i = 0; i < axis; ++i) outer *= x.shape[i];
                    for (int i = (int) axis + 1; i < r; ++i) inner *= x.shape[i];
                    const int64_t axisSize = x.shape[axis];
                    View          y        = newTensor(n.outputs[0], g.desc(n.outputs[0]).shape);
                    Step          s;
                    s.a    = ptrOf(xd);
                    s.d    = ptrOf(y);
                    s.norm = inner;
                    if (constIdx) {
                        const std::vector<int64_t> &ix = i64Inits_.at(n.inputs[1]);
                        const int64_t               nidx = (int64_t) ix.size();
                        std::vector<int64_t>        table((size_t) (outer * nidx));
                        for (int64_t o = 0; o < outer; ++o)
                            for (int64_t k = 0; k < nidx; ++k) {
                                int64_t v = ix[(size_t) k] < 0 ? ix[(size_t) k] + axisSize : ix[(size_t) k];
                                if (v < 0 || v >= axisSize) fail(Status::InvalidArgument, "Gather index out of range in " + n.name);
                                table[(size_t) (o * nidx + k)] = (o * axisSize + v) * inner;
                            }
                        const int tb = newBuffer(table.size() * 8);
                        check(ctx_, vkc_upload(ctx_, bufs_[tb].ptr, VKC_I32, table.data(), VKC_I32, (int64_t) table.size() * 2, nullptr), "vkc_upload");
                        s.kind  = Step::Rows;
                        s.b     = bufs_[tb].ptr;
                        s.rows  = outer * nidx;
                        s.label = "gather(rows)";
                    } else {
                        View iv = materialize(views_.at(n.inputs[1]), "gather index");
                        s.kind  = Step::GatherRt;
                        s.b     = ptrOf(iv);
                        s.M     = outer;
                        s.N     = axisSize;
                        s.K     = prod(iv.shape);
                        s.label = "gather(runtime index)";
                    }
                    steps_.push_back(s);
                    break;
                }
                case OpType::ScatterND: {
                    // out = data, then every index row overwrites one slice (src/backend/cpu/ops/scatternd.cpp:13-84). The
                    // indices are constants: destinations are computed here, and of several rows aimed at one slice only the
                    // last survives, which is what the reference's sequential loop leaves behind.
                    const View                 &x  = views_.at(n.inputs[0]);
                    const std::vector<int64_t> &ix = i64Inits_.at(n.inputs[1]);
                    const Shape                &is = g.desc(n.inputs[1]).shape;
                    const int                   r  = (int) x.shape.size();
                    const int                   q  = (int) is.back();
                    const int64_t               nrows = (int64_t) ix.size() / q;
                    std::vector<int64_t>        stride((size_t) r, 1);
                    for (int k = r - 2; k >= 0; --k) stride[(size_t) k] = stride[(size_t) k + 1] * x.shape[(size_t) k + 1];
                    int64_t slice = 1;
                    for (int k = q; k < r; ++k) slice *= x.shape[(size_t) k];
                    View y = newTensor(n.outputs[0], x.shape);
                    {
                        Step c;
                        c.kind      = Step::Copy;
                        c.a         = bufs_[x.buf].ptr;
                        c.d         = ptrOf(y);
                        c.shape     = x.shape;
                        c.inStrides = x.strides;
                        c.inOffset  = x.offset;
                        c.label     = "copy(scatter data)";
                        steps_.push_back(c);
                    }
                    std::map<int64_t, int64_t> last; // destination offset -> the row that writes it last
                    for (int64_t rr = 0; rr < nrows; ++rr) {
                        int64_t off = 0;
                        for (int c = 0; c < q; ++c) {
                            int64_t v = ix[(size_t) (rr * q + c)];
                            if (v < 0) v += x.shape[(size_t) c];
                            if (v < 0 || v >= x.shape[(size_t) c]) fail(Status::InvalidArgument, "ScatterND index out of range in " + n.name);
                            off += v * stride[(size_t) c];
                        }
                        last[off] = rr;
                    }
                    std::vector<int64_t> table;
                    for (const auto &kv : last) table.push_back(kv.second * slice);
                    for (const auto &kv : last) table.push_back(kv.first);
                    if (!last.empty()) {
                        View      u  = materialize(views_.at(n.inputs[2]), "scatter updates");
                        const int tb = newBuffer(table.size() * 8);
                        check(ctx_, vkc_upload(ctx_, bufs_[tb].ptr, VKC_I32, table.data(), VKC_I32, (int64_t) table.size() * 2, nullptr), "vkc_upload");
                        Step s;
                        s.kind  = Step::Rows;
                        s.a     = ptrOf(u);
                        s.d     = ptrOf(y);
                        s.b     = bufs_[tb].ptr;
                        s.c     = static_cast<const int64_t *>(bufs_[tb].ptr) + last.size();
                        s.rows  = (int64_t) last.size();
                        s.norm  = slice;
                        s.label = "scatter(rows)";
                        steps_.push_back(s);
                    }
                    break;
                }
                case OpType::Slice: {
                    // a view: offset and strides (reference semantics src/backend/cpu/ops/slice.cpp:24-52; steps > 0 here)
                    const View &x = views_.at(n.inputs[0]);
                    const int   r = (int) x.shape.size();
                    auto rd = [&](const char *attr, size_t idx) {
                        std::vector<int64_t> v = n.attr.getints(attr);
                        if (v.empty() && idx < n.inputs.size() && n.inputs[idx] != kNoTensor) v = i64Inits_.at(n.inputs[idx]);
                        return v;
                    };
                    const auto starts = rd("starts", 1), ends = rd("ends", 2), axes = rd("axes", 3), steps = rd("steps", 4);
                    View       y      = x;
                    for (size_t k = 0; k < starts.size(); ++k) {
                        int ax = (int) (axes.empty() ? (int64_t) k : axes[k]);
                        if (ax < 0) ax += r;
                        if (ax < 0 || ax >= r) continue;
                        const int64_t dim = x.shape[ax], sp = k < steps.size() ? steps[k] : 1;
                        int64_t       st  = starts[k] < 0 ? starts[k] + dim : starts[k];
                        int64_t       en  = ends[k] < 0 ? ends[k] + dim : ends[k];
                        st                = std::max<int64_t>(0, std::min(st, dim));
                        en                = std::max<int64_t>(0, std::min(en, dim));
                        y.offset += st * x.strides[ax];
                        y.strides[ax] = x.strides[ax] * sp;
                        y.shape[ax]   = std::max<int64_t>(0, (en - st + sp - 1) / sp);
                    }
                    if (y.shape != g.desc(n.outputs[0]).shape) fail(Status::RuntimeError, "Slice: planned shape differs from the inferred one");
                    views_[n.outputs[0]] = y;
                    break;
                }
                case OpType::Split: {
                    // views at running offsets along the axis (src/backend/cpu/ops/split.cpp:9-62)
                    const View &x    = views_.at(n.inputs[0]);
                    int64_t     axis = n.attr.geti("axis", 0);
                    if (axis < 0) axis += (int64_t) x.shape.size();
                    int64_t off = 0;
                    for (TensorId o : n.outputs) {
                        if (o == kNoTensor) continue;
                        View y = x;
                        y.shape[axis] = g.desc(o).shape[axis];
                        y.offset += off * x.strides[axis];
                        off += y.shape[axis];
                        views_[o] = y;
                    }
                    break;
                }
                case OpType::Expand: {
                    // a view with stride 0 along the broadcast dimensions (src/backend/cpu/ops/expand.cpp:17-45)
                    const View  &x   = views_.at(n.inputs[0]);
                    const Shape &out = g.desc(n.outputs[0]).shape;
                    const int    r = (int) out.size(), off = r - (int) x.shape.size();
                    View         y = x;
                    y.shape        = out;
                    y.strides.assign(r, 0);
                    for (int k = 0; k < r; ++k) {
                        const int64_t dim = k < off ? 1 : x.shape[k - off];
                        if (dim != 1) {
                            if (dim != out[k]) fail(Status::InvalidArgument, "Expand: shapes do not broadcast");
                            y.strides[k] = x.strides[k - off];
                        }
                    }
                    views_[n.outputs[0]] = y;
                    break;
                }
                case OpType::Tile: {
                    // [d0, d1, ..] repeated [r0, r1, ..]: the view [r0, d0, r1, d1, ..] with stride 0 on the repeat axes, copied
                    // once into a dense buffer and read as [r0*d0, r1*d1, ..] (src/backend/cpu/ops/tile.cpp:17-30)
                    const View &x    = views_.at(n.inputs[0]);
                    const int   r    = (int) x.shape.size();
                    std::vector<int64_t> reps = n.attr.getints("repeats");
                    if (reps.empty() && n.inputs.size() > 1 && n.inputs[1] != kNoTensor) reps = i64Inits_.at(n.inputs[1]);
                    View v2 = x;
                    v2.shape.clear(), v2.strides.clear();
                    for (int k = 0; k < r; ++k) {
                        v2.shape.push_back(std::max<int64_t>(k < (int) reps.size() ? reps[k] : 1, 1));
                        v2.strides.push_back(0);
                        v2.shape.push_back(x.shape[k]);
                        v2.strides.push_back(x.strides[k]);
                    }
                    View y    = materialize(v2, "tile");
                    y.shape   = g.desc(n.outputs[0]).shape;
                    y.strides = denseStrides(y.shape);
                    views_[n.outputs[0]] = y;
                    break;
                }
                case OpType::Concat: {
                    // each input is copied into its slab of the output (src/backend/cpu/ops/concat.cpp:9-66)
                    const Shape &out  = g.desc(n.outputs[0]).shape;
                    int64_t      axis = n.attr.geti("axis", 0);
                    if (axis < 0) axis += (int64_t) out.size();
                    View    y   = newTensor(n.outputs[0], out);
                    int64_t off = 0;
                    for (TensorId in : n.inputs) {
                        const View &x = views_.at(in);
                        Step        s;
                        s.kind = Step::Copy;
                        s.a    = bufs_[x.buf].ptr;
                        s.shape.assign(x.shape.begin(), x.shape.end());
                        s.inStrides = x.strides;
                        s.inOffset  = x.offset;
                        s.outStrides = y.strides;
                        s.d          = static_cast<char *>(ptrOf(y)) + off * y.strides[axis] * (int64_t) esize_;
                        s.label      = "concat";
                        steps_.push_back(s);
                        off += x.shape[axis];
                    }
                    break;
                }
                case OpType::Einsum: {
                    // "i,j->ij" (src/backend/cpu/ops/einsum.cpp:33-44): y[i,j] = a[i] * b[j]. a is read through a stride-0
                    // column axis and written out once at [I,J]; b joins as a broadcast operand of a one-step Mul program.
                    View a = materialize(views_.at(n.inputs[0]), "einsum a"), b = materialize(views_.at(n.inputs[1]), "einsum b");
                    const int64_t I = prod(a.shape), J = prod(b.shape);
                    View          e = a;
                    e.shape   = {I, J};
                    e.strides = {1, 0};
                    View x = materialize(e, "einsum a rows");
                    View y = newTensor(n.outputs[0], Shape {I, J});
                    Step s;
                    s.kind      = Step::Pointwise;
                    s.shape     = {I, J};
                    s.operands  = {ptrOf(b)};
                    s.opStrides = {0, 1};
                    s.pwSteps   = {0, (int) BinaryType::Mul, 1, 0};
                    s.pwParams  = {0.f, 0.f};
                    s.a = ptrOf(x), s.d = ptrOf(y);
                    s.label = "einsum(outer)";
                    steps_.push_back(s);
                    break;
                }
                case OpType::Conv: planPatchConv(n); break;
                case OpType::MatMul:
                    if (!tryAttention(pos, done)) planMatMul(pos, done);
                    break;
                case OpType::LayerNorm: {
                    View x = materialize(views_.at(n.inputs[0]), "layernorm");
                    View y = newTensor(n.outputs[0], g.desc(n.outputs[0]).shape);
                    Step s;
                    s.kind  = Step::LayerNorm;
                    s.a     = ptrOf(x);
                    s.d     = ptrOf(y);
                    s.norm  = x.shape.back();
                    s.rows  = prod(x.shape) / s.norm;
                    s.gamma = f32Init(n.inputs[1]);
                    s.beta  = (n.inputs.size() > 2 && n.inputs[2] != kNoTensor) ? f32Init(n.inputs[2]) : nullptr;
                    s.eps   = n.attr.getf("epsilon", 1e-5f);
                    s.label = "layernorm";
                    steps_.push_back(s);
                    break;
                }
                case OpType::Softmax: {
                    View x = materialize(views_.at(n.inputs[0]), "softmax");
                    View y = newTensor(n.outputs[0], g.desc(n.outputs[0]).shape);
                    Step s;
                    s.kind  = Step::Softmax;
                    s.a     = ptrOf(x);
                    s.d     = ptrOf(y);
                    s.norm  = x.shape.back();
                    s.rows  = prod(x.shape) / s.norm;
                    s.label = "softmax";
                    steps_.push_back(s);
                    break;
                }
                case OpType::Reduce: {
                    // move the reduced axes last (one strided copy), then one warp per output element
                    // (src/backend/cpu/ops/reduce.cpp:11-108)
                    const View &x = views_.at(n.inputs[0]);
                    const int   r = (int) x.shape.size();
                    std::vector<int64_t> axes = n.attr.getints("axes");
                    if (axes.empty() && n.inputs.size() > 1 && n.inputs[1] != kNoTensor) axes = i64Inits_.at(n.inputs[1]);
                    std::set<int> ax;
                    for (int64_t a : axes) ax.insert((int) (a < 0 ? a + r : a));
                    if (axes.empty())
                        for (int i = 0; i < r; ++i) ax.insert(i);
                    View    v2 = x;
                    int64_t rows = 1, red = 1;
                    v2.shape.clear(), v2.strides.clear();
                    for (int i = 0; i < r; ++i)
                        if (!ax.count(i)) v2.shape.push_back(x.shape[i]), v2.strides.push_back(x.strides[i]), rows *= x.shape[i];
                    for (int i = 0; i < r; ++i)
                        if (ax.count(i)) v2.shape.push_back(x.shape[i]), v2.strides.push_back(x.strides[i]), red *= x.shape[i];
                    View a = materialize(v2, "reduce");
                    View y = newTensor(n.outputs[0], g.desc(n.outputs[0]).shape);
                    if (prod(y.shape) != rows) fail(Status::RuntimeError, "Reduce: planned size differs from the inferred one");
                    Step s;
                    s.kind = Step::Reduce;
                    s.a = ptrOf(a), s.d = ptrOf(y);
                    s.rows = rows, s.norm = red, s.reduceOp = n.subOp;
                    s.label = "reduce";
                    steps_.push_back(s);
                    break;
                }
                case OpType::Binary:
                case OpType::Add:
                case OpType::Unary:
                case OpType::Where:
                case OpType::Equal:
                case OpType::Greater:
                case OpType::GreaterEqual:
                case OpType::FusedPointwise: planPointwise(n); break;
                default: fail(Status::Unsupported, std::string("node type ") + opTypeName(n.type));
            }
        }
        // boundary outputs must be contiguous buffers for the download
        for (TensorId id : boundaryOutputs) {
            auto it = views_.find(id);
            if (it == views_.end()) fail(Status::RuntimeError, "boundary output was not produced");
            if (!it->second.contiguous()) it->second = materialize(it->second, "boundary output");
        }
        planned_ = true;
        if (tuning_ != (int) Mode::NoTune && dtype_ != VKC_F32) tuneGemms();
    }

    // Per-shape choice of the tensor-core GEMM configuration by measurement (Hint::Tuning: Fast = 10 timed launches per
    // configuration, Thorough = 40), as the reference times its convolution kernels per shape. The buffers exist by now;
    // their contents are irrelevant for timing and every tuned output is overwritten by the first real run.
    void CudaSegment::tuneGemms() {
        const int nCfg  = vkc_gemm_config_count();
        const int iters = tuning_ == (int) Mode::Thorough ? 40 : 10;
        for (Step &s : steps_) {
            if (s.kind != Step::Gemm || s.M < 32 || s.N < 32 || s.K < 32) continue;
            std::ostringstream key;
            key << "gemm:" << dtype_ << ":" << s.M << "x" << s.N << "x" << s.K << "x" << s.batch << ":" << s.bLayout << ":" << s.epilogue << ":"
                << (s.lda % 8 == 0) << (s.ldb % 8 == 0) << (s.ldd % 8 == 0);
            if (be_->lookupTuning(key.str(), &s.gemmConfig)) continue;
            int   best   = -1;
            float bestMs = 1e30f;
            for (int c = -1; c < nCfg; ++c) {
                auto once = [&]() {
                    return vkc_gemm_ex(ctx_, s.a, s.b, s.bias, s.c, s.d, s.M, s.N, s.K, s.batch, s.sa, s.sb, s.sd, s.lda, s.ldb, s.ldd, s.bLayout, s.epilogue,
                                       dtype_, c, nullptr);
                };
                if (once() != VKC_OK) continue; // a configuration this shape cannot run
                // time on the device: the launches are recorded into a graph and replayed, so that host launch cost
                // (tensor-map encoding, driver calls) does not rank the configurations
                vkc_graph *tg = nullptr;
                if (vkc_graph_begin(ctx_) != VKC_OK) break;
                bool okc = true;
                for (int i = 0; i < iters && okc; ++i) okc = once() == VKC_OK;
                if (vkc_graph_end(ctx_, &tg) != VKC_OK || !tg || !okc) {
                    if (tg) vkc_graph_destroy(ctx_, tg);
                    continue;
                }
                float ms = 1e30f;
                if (vkc_graph_launch(ctx_, tg) == VKC_OK && vkc_timer_start(ctx_, nullptr) == VKC_OK && vkc_graph_launch(ctx_, tg) == VKC_OK) {
                    if (vkc_timer_stop(ctx_, nullptr, &ms) != VKC_OK) ms = 1e30f;
                }
                vkc_graph_destroy(ctx_, tg);
                if (ms < bestMs * 0.97f) bestMs = ms, best = c; // a later configuration must win clearly
            }
            s.gemmConfig = best;
            be_->storeTuning(key.str(), best);
        }
        check(ctx_, vkc_sync(ctx_, nullptr), "vkc_sync after GEMM tuning");
    }

    void CudaSegment::launch(const Step &s) {
        switch (s.kind) {
            case Step::Gemm:
                check(ctx_, vkc_gemm_ex(ctx_, s.a, s.b, s.bias, s.c, s.d, s.M, s.N, s.K, s.batch, s.sa, s.sb, s.sd, s.lda, s.ldb, s.ldd, s.bLayout,
                                        s.epilogue, dtype_, s.gemmConfig, nullptr), "vkc_gemm");
                break;
            case Step::Attn:
                check(ctx_, vkc_attn_prefill(ctx_, s.a, s.b, s.c, s.d, s.B, s.Hq, s.Hkv, s.Sq, s.Skv, s.D, s.qs, s.ks, s.vs, s.os, s.scale, 0, s.mask,
                                             nullptr, dtype_, nullptr), "vkc_attn_prefill");
                break;
            case Step::LayerNorm:
                check(ctx_, vkc_layernorm(ctx_, s.a, s.gamma, s.beta, s.d, s.rows, s.norm, s.eps, dtype_, nullptr), "vkc_layernorm");
                break;
            case Step::Softmax: check(ctx_, vkc_softmax(ctx_, s.a, s.d, s.rows, s.norm, dtype_, nullptr), "vkc_softmax"); break;
            case Step::Pointwise:
                check(ctx_, vkc_pointwise(ctx_, s.a, s.d, s.shape.data(), (int) s.shape.size(), (int) s.pwSteps.size() / 4, s.pwSteps.data(),
                                          s.pwParams.data(), (int) s.operands.size(), s.operands.data(), s.opStrides.data(), dtype_, nullptr),
                      "vkc_pointwise");
                break;
            case Step::Reduce:
                check(ctx_, vkc_reduce_rows(ctx_, s.a, s.d, s.rows, s.norm, s.reduceOp, dtype_, nullptr), "vkc_reduce_rows");
                break;
            case Step::Rows:
                check(ctx_, vkc_copy_rows(ctx_, s.a, s.d, static_cast<const int64_t *>(s.b), static_cast<const int64_t *>(s.c), s.rows, s.norm, dtype_, nullptr),
                      "vkc_copy_rows");
                break;
            case Step::GatherRt:
                check(ctx_, vkc_gather_rows(ctx_, s.a, s.b, s.d, s.M, s.N, s.K, s.norm, dtype_, dtype_, nullptr), "vkc_gather_rows");
                break;
            case Step::Copy:
                if (s.outStrides.empty())
                    check(ctx_, vkc_strided_copy(ctx_, s.a, s.d, s.shape.data(), s.inStrides.data(), (int) s.shape.size(), s.inOffset, dtype_, nullptr),
                          "vkc_strided_copy");
                else
                    check(ctx_, vkc_strided_copy2(ctx_, s.a, s.d, s.shape.data(), s.inStrides.data(), s.outStrides.data(), (int) s.shape.size(), s.inOffset,
                                                  dtype_, nullptr), "vkc_strided_copy2");
                break;
        }
    }

    void CudaSegment::run(ExecContext &ctx) {
        if (!planned_) plan();
        const Graph &g = *g_;
        // boundary inputs: host fp32 -> device storage precision (conversion on the device)
        for (TensorId id : boundaryInputs) {
            if (initIds_.count(id)) continue; // uploaded in compileSegment; the pool holds no host data for it
            RtTensor   &rt = ctx.t(id);
            const View &v  = views_.at(id);
            if (rt.dmaBufFd >= 0) {
                // device-resident input: the integer names a registered CUDA buffer (the CUDA form of the reference's
                // dma-buf input, src/backend/vulkan/vk_backend.cpp:1218-1260); converted on the device, no host staging
                void  *ext   = nullptr;
                size_t bytes = 0;
                if (vkc_extbuf_lookup(rt.dmaBufFd, &ext, &bytes) != VKC_OK)
                    fail(Status::InvalidArgument, "boundary input " + g.desc(id).name + ": handle is not a registered device buffer");
                const int     sdt = extDtype(rt.dmaBufDtype, g.desc(id).name);
                const int64_t n   = prod(v.shape);
                if ((size_t) n * (sdt == VKC_F32 ? 4 : 2) > bytes) fail(Status::InvalidArgument, "boundary input " + g.desc(id).name + ": device buffer too small");
                check(ctx_, vkc_convert(ctx_, ptrOf(v), dtype_, ext, sdt, n, nullptr), "vkc_convert");
                continue;
            }
            if (!rt.hostValid) fail(Status::RuntimeError, "boundary input " + g.desc(id).name + " has no host data");
            if (rt.elems() != prod(v.shape)) fail(Status::InvalidArgument, "boundary input " + g.desc(id).name + " has an unexpected size");
            check(ctx_, vkc_upload(ctx_, ptrOf(v), dtype_, rt.host.bytes.data(), VKC_F32, rt.elems(), nullptr), "vkc_upload");
        }
        if (ctx.profiler && ctx.profiler->enabled()) {
            // Profiled run: launches go out one by one between device timers and every launch leaves an OpRecord under the
            // node it was planned for (the counterpart of the per-node records of src/backend/cpu/cpu_backend.cpp:133-142 and
            // the timestamp records of src/backend/vulkan/vk_backend.cpp:1436-1457). Nodes folded into a neighbour's launch
            // (views, fused attention, GEMM epilogues) have no record of their own.
            for (const Step &s : steps_) {
                float ms = -1.f;
                check(ctx_, vkc_timer_start(ctx_, nullptr), "vkc_timer_start");
                launch(s);
                check(ctx_, vkc_timer_stop(ctx_, nullptr, &ms), "vkc_timer_stop");
                OpRecord r;
                r.name     = (s.node >= 0 ? g.nodes[(size_t) s.node].name : std::string()) + " [" + s.label + "]";
                r.type     = s.node >= 0 ? g.nodes[(size_t) s.node].type : OpType::Unknown;
                r.backend  = "CUDA";
                r.cpuMs    = ms;
                r.gpuMs    = ms;
                r.fellBack = false;
                ctx.profiler->add(r);
            }
        } else if (graph_) {
            check(ctx_, vkc_graph_launch(ctx_, graph_), "vkc_graph_launch");
        } else if (useGraph_ && runs_ == 1) {
            // the eager first run sized every scratch buffer; record the launch list once and replay it from now on
            check(ctx_, vkc_graph_begin(ctx_), "vkc_graph_begin");
            try {
                for (const Step &s : steps_) launch(s);
            } catch (...) {
                vkc_graph *tmp = nullptr;
                vkc_graph_end(ctx_, &tmp);
                if (tmp) vkc_graph_destroy(ctx_, tmp);
                throw;
            }
            check(ctx_, vkc_graph_end(ctx_, &graph_), "vkc_graph_end");
            check(ctx_, vkc_graph_launch(ctx_, graph_), "vkc_graph_launch");
        } else {
            for (const Step &s : steps_) launch(s);
        }
        // boundary outputs: device -> host fp32
        for (TensorId id : boundaryOutputs) {
            RtTensor   &rt = ctx.t(id);
            const View &v  = views_.at(id);
            rt.shape = g.desc(id).shape;
            if (rt.dmaBufFd >= 0) {
                // device-resident output (the reference's toDmaBuf binding, vk_backend.cpp:1339-1382): written into the
                // caller's registered buffer in the declared dtype; the Session then skips its host read-back
                void  *ext   = nullptr;
                size_t bytes = 0;
                if (vkc_extbuf_lookup(rt.dmaBufFd, &ext, &bytes) != VKC_OK)
                    fail(Status::InvalidArgument, "output " + g.desc(id).name + ": handle is not a registered device buffer");
                const int     ddt = extDtype(rt.dmaBufDtype, g.desc(id).name);
                const int64_t n   = prod(v.shape);
                if ((size_t) n * (ddt == VKC_F32 ? 4 : 2) > bytes) fail(Status::InvalidArgument, "output " + g.desc(id).name + ": device buffer too small");
                check(ctx_, vkc_convert(ctx_, ext, ddt, ptrOf(v), dtype_, n, nullptr), "vkc_convert");
                rt.dtype       = rt.dmaBufDtype;
                rt.hostValid   = false;
                rt.deviceValid = false;
                continue;
            }
            rt.dtype = DType::Float32;
            rt.allocHost();
            check(ctx_, vkc_download(ctx_, rt.host.bytes.data(), VKC_F32, ptrOf(v), dtype_, rt.elems(), nullptr), "vkc_download");
            rt.hostValid   = true;
            rt.deviceValid = false;
        }
        check(ctx_, vkc_sync(ctx_, nullptr), "vkc_sync");
        ++runs_;
    }

} // namespace vknn
