// TEST INFRASTRUCTURE — not part of the shipped product.
//
// vknn_ref_driver: runs a small graph through the UNMODIFIED reference engine (vknn::Session) so that
// the CPU restatement in vknn_oracle.c can be pinned against the reference's own CPU backend, golden
// vectors can be generated, and the reference CPU path can be timed. It is compiled against the
// reference sources where they lie (see the Makefile beside this file) and its outputs go to
// oracle/_ref/ only. When the Makefile also links the CUDA backend plug-in, `--backend cuda`
// plans the same graph on the plug-in through the reference's own planner.
//
// The graph is described by a line-oriented text spec (written by oracle/vko.py, class RefGraph):
//
//   tensor <name> <input|init|inter|output> <f32|i64> <rank> <d0> <d1> ...
//   node <OpType> <name> subop=<int> in=<a,b,c> out=<y> [fusedbias=<name>] [i:<k>=<int>] [f:<k>=<float>]
//        [ints:<k>=<a,b,c>] [floats:<k>=<a,b,c>] [s:<k>=<string without blanks>]
//
// Tensor payloads of inputs and initializers are raw little-endian values concatenated in spec order
// in <data.bin>; outputs are written concatenated in graph-output order to <out.bin> as fp32.
//
// usage: vknn_ref_driver <spec.txt> <data.bin> <out.bin> [--backend cpu|cuda] [--precision low|high]
//                        [--iters N] [--warmup W] [--quiet] [--vxm-fp16 <file.vxm>] [--device N] [--profile]
// --device N selects the CUDA device through the plug-in's spare Config::hints slot; --profile turns Config::profile on and
// adds the Session profiler's records of the last run to the JSON line.
// --vxm-fp16 takes the route of the reference's model compiler (convert/compile.cpp:36-96): run the standard
// passes, store every fp32 initializer as fp16, write the ".vxm" file, and create the Session from that file
// (Session::createFromVxm, include/vknn/session_class.h:24), so the backend sees fp16 weights.
// prints one line of JSON: node list after the reference's passes, per-node backend, median run ms.
//
// Reference interfaces used: Session::create(Graph&&, Config) include/vknn/session_class.h:26,
// Session::run session_class.h:36, Graph/Node/TensorDesc include/vknn/graph.h:12-39, node.h:14-32,
// and the graph-in-code idiom of tests/test_ops.cpp:42-107.
#include "import/passes.h"
#include "vknn/graph.h"
#include "vknn/session.h"
#ifdef VKNN_DRIVER_HAS_CUDA
#include "vknn_cuda.h"
#endif
#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <map>
#include <sstream>
#include <string>
#include <vector>

using namespace vknn;

namespace {

    std::vector<std::string> splitc(const std::string &s, char c) {
        std::vector<std::string> out;
        std::string              cur;
        for (char ch : s) {
            if (ch == c) {
                out.push_back(cur);
                cur.clear();
            } else {
                cur.push_back(ch);
            }
        }
        if (!cur.empty() || !s.empty()) out.push_back(cur);
        return out;
    }

    OpType opFromName(const std::string &n) {
        static const std::map<std::string, OpType> m = {
            {"MatMul", OpType::MatMul},       {"Softmax", OpType::Softmax},     {"LayerNorm", OpType::LayerNorm},
            {"Binary", OpType::Binary},       {"Add", OpType::Add},             {"Unary", OpType::Unary},
            {"Transpose", OpType::Transpose}, {"Reshape", OpType::Reshape},     {"Gather", OpType::Gather},
            {"FusedPointwise", OpType::FusedPointwise}, {"Identity", OpType::Identity},
            {"Conv", OpType::Conv},           {"Slice", OpType::Slice},         {"Split", OpType::Split},
            {"Expand", OpType::Expand},       {"Tile", OpType::Tile},           {"Concat", OpType::Concat},
            {"Squeeze", OpType::Squeeze},     {"Unsqueeze", OpType::Unsqueeze},
            {"Reduce", OpType::Reduce},       {"Where", OpType::Where},         {"Equal", OpType::Equal},
            {"Greater", OpType::Greater},     {"GreaterEqual", OpType::GreaterEqual}, {"ScatterND", OpType::ScatterND},
            {"Einsum", OpType::Einsum},
        };
        auto it = m.find(n);
        if (it == m.end()) {
            std::fprintf(stderr, "ref_driver: unknown op %s\n", n.c_str());
            std::exit(2);
        }
        return it->second;
    }

    struct IoSpec {
        std::string name;
        Shape       shape;
        DType       dtype;
        size_t      bytes;
    };

} // namespace

int main(int argc, char **argv) {
    if (argc < 4) {
        std::fprintf(stderr, "usage: %s spec.txt data.bin out.bin [--backend cpu|cuda] [--precision low|high] [--iters N] [--warmup W] [--vxm-fp16 file] [--device-io] [--cache-file path] [--tuning off|fast|thorough]\n", argv[0]);
        return 2;
    }
    std::string specPath = argv[1], dataPath = argv[2], outPath = argv[3];
    std::string backend = "cpu", precision = "high";
    int         iters = 1, warmup = 0;
    bool        quiet = false;
    std::string vxmPath;
    bool        deviceIo = false;
    std::string cacheFile, tuning;
    int         device  = -1;
    bool        profile = false;
    for (int i = 4; i < argc; ++i) {
        std::string a = argv[i];
        if (a == "--backend" && i + 1 < argc) backend = argv[++i];
        else if (a == "--precision" && i + 1 < argc) precision = argv[++i];
        else if (a == "--iters" && i + 1 < argc) iters = std::atoi(argv[++i]);
        else if (a == "--warmup" && i + 1 < argc) warmup = std::atoi(argv[++i]);
        else if (a == "--quiet") quiet = true;
        else if (a == "--vxm-fp16" && i + 1 < argc) vxmPath = argv[++i];
        else if (a == "--device-io") deviceIo = true;
        else if (a == "--cache-file" && i + 1 < argc) cacheFile = argv[++i];
        else if (a == "--tuning" && i + 1 < argc) tuning = argv[++i];
        else if (a == "--device" && i + 1 < argc) device = std::atoi(argv[++i]);
        else if (a == "--profile") profile = true;
    }

    std::ifstream spec(specPath);
    std::ifstream data(dataPath, std::ios::binary);
    if (!spec || !data) {
        std::fprintf(stderr, "ref_driver: cannot open spec/data\n");
        return 2;
    }

    Graph                 g;
    std::vector<IoSpec>   inputs;
    std::vector<IOTensor> ioIn;
    std::string           line;
    while (std::getline(spec, line)) {
        if (line.empty() || line[0] == '#') continue;
        std::istringstream ls(line);
        std::string        kind;
        ls >> kind;
        if (kind == "tensor") {
            std::string name, role, dt;
            int         rank = 0;
            ls >> name >> role >> dt >> rank;
            TensorDesc d;
            d.name = name;
            d.dtype = dt == "i64" ? DType::Int64 : DType::Float32;
            for (int i = 0; i < rank; ++i) {
                int64_t v;
                ls >> v;
                d.shape.push_back(v);
            }
            d.isInput       = role == "input";
            d.isOutput      = role == "output";
            d.isInitializer = role == "init";
            Shape  shp   = d.shape;
            DType  dtype = d.dtype;
            size_t bytes = (size_t) numElements(shp) * dtypeSize(dtype);
            if (role == "inter" || role == "output") {
                d.shape.clear(); // let the reference's shape inference fill it in
            }
            TensorId id = g.addTensor(d);
            g.tensorByName[name] = id;
            if (role == "input") {
                g.inputs.push_back(id);
                IOTensor t;
                t.name  = name;
                t.shape = shp;
                t.dtype = dtype;
                t.data.resize(bytes);
                data.read(reinterpret_cast<char *>(t.data.data()), (std::streamsize) bytes);
                ioIn.push_back(std::move(t));
            } else if (role == "init") {
                HostBuffer hb;
                hb.resizeElems(numElements(shp), dtype);
                data.read(reinterpret_cast<char *>(hb.bytes.data()), (std::streamsize) bytes);
                g.initializers[id] = std::move(hb);
            } else if (role == "output") {
                g.outputs.push_back(id);
            }
        } else if (kind == "node") {
            std::string op, name, tok;
            ls >> op >> name;
            Node n;
            n.type = opFromName(op);
            n.name = name;
            while (ls >> tok) {
                auto eq = tok.find('=');
                if (eq == std::string::npos) continue;
                std::string k = tok.substr(0, eq), v = tok.substr(eq + 1);
                if (k == "subop") n.subOp = std::atoi(v.c_str());
                else if (k == "in") {
                    for (auto &s : splitc(v, ',')) n.inputs.push_back(g.find(s));
                } else if (k == "out") {
                    for (auto &s : splitc(v, ',')) n.outputs.push_back(g.find(s));
                } else if (k == "fusedbias") {
                    n.fusedBias = g.find(v);
                } else if (k.rfind("i:", 0) == 0) {
                    Attr a;
                    a.kind = Attr::Int;
                    a.i    = std::atoll(v.c_str());
                    n.attr.map[k.substr(2)] = a;
                } else if (k.rfind("f:", 0) == 0) {
                    Attr a;
                    a.kind = Attr::Float;
                    a.f    = std::strtof(v.c_str(), nullptr);
                    n.attr.map[k.substr(2)] = a;
                } else if (k.rfind("ints:", 0) == 0) {
                    Attr a;
                    a.kind = Attr::Ints;
                    for (auto &s : splitc(v, ',')) a.ints.push_back(std::atoll(s.c_str()));
                    n.attr.map[k.substr(5)] = a;
                } else if (k.rfind("s:", 0) == 0) {
                    Attr a;
                    a.kind = Attr::String;
                    a.str  = v;
                    n.attr.map[k.substr(2)] = a;
                } else if (k.rfind("floats:", 0) == 0) {
                    Attr a;
                    a.kind = Attr::Floats;
                    for (auto &s : splitc(v, ',')) a.floats.push_back(std::strtof(s.c_str(), nullptr));
                    n.attr.map[k.substr(7)] = a;
                }
            }
            g.nodes.push_back(std::move(n));
        }
    }

    Config cfg;
    cfg.verbosity = quiet ? 0 : 1;
    cfg.precision = precision == "low" ? Precision::Low : Precision::High;
    if (backend == "cuda") {
        // The plug-in registers itself as the first free BackendKind value after the reference's own
        // two (include/vknn/backend_kind.h:7). No CPU backend is active: nothing may fall back.
        cfg.backend          = static_cast<BackendKind>(2);
        cfg.fallback         = {};
        cfg.allowCpuFallback = false;
    } else {
        cfg.backend  = BackendKind::Cpu;
        cfg.fallback = {};
    }
    if (device >= 0) cfg.setHint(static_cast<Hint>(8), device + 1); // the CUDA plug-in's device slot: ordinal + 1, 0 = unset
    cfg.profile   = profile;
    cfg.cacheFile = cacheFile; // empty: no cache file (the default of a session built from an in-memory graph)
    if (!tuning.empty()) cfg.setHint(Hint::Tuning, tuning == "off" ? Mode::NoTune : tuning == "thorough" ? Mode::Thorough : Mode::Fast);
    cfg.applyLogLevel();

    std::unique_ptr<Session> sess;
    try {
        if (!vxmPath.empty()) {
            runStandardPasses(g, PassOptions {});
            for (auto &kv : g.initializers) {
                TensorDesc &d = g.tensors[kv.first];
                if (d.dtype != DType::Float32) continue;
                const int64_t        n   = numElements(d.shape);
                const float         *src = kv.second.f32();
                std::vector<uint8_t> half((size_t) n * 2);
                for (int64_t i = 0; i < n; ++i) reinterpret_cast<fp16_t *>(half.data())[i] = floatToHalf(src[i]);
                kv.second.bytes = std::move(half);
                d.dtype         = DType::Float16;
            }
            if (!saveGraphBin(g, vxmPath)) {
                std::printf("{\"ok\": false, \"error\": \"saveGraphBin failed\"}\n");
                return 1;
            }
            sess = Session::createFromVxm(vxmPath, cfg);
        } else
            sess = Session::create(std::move(g), cfg);
    } catch (const std::exception &e) {
        std::printf("{\"ok\": false, \"error\": \"plan: %s\"}\n", e.what());
        return 1;
    }
    if (!sess) {
        std::printf("{\"ok\": false, \"error\": \"Session::create returned null\"}\n");
        return 1;
    }

    std::vector<IOTensor> outs;
    std::vector<double>   ms;
#ifdef VKNN_DRIVER_HAS_CUDA
    // --device-io: inputs and outputs live in caller-owned CUDA buffers registered with the CUDA library; the Session
    // carries only their handles (IOTensor::dmaBufFd), exactly as it carries dma-buf fds for the reference's GPU backend.
    vkc_ctx            *ioCtx = nullptr;
    std::vector<void *> inDev, outDev;
    std::vector<int>    outHandle;
    std::vector<int64_t> outElems;
    if (deviceIo) {
        if (backend != "cuda" || vkc_ctx_create(device >= 0 ? device : 0, &ioCtx) != VKC_OK) {
            std::printf("{\"ok\": false, \"error\": \"--device-io needs the cuda backend and a device\"}\n");
            return 1;
        }
        for (auto &t : ioIn) {
            void *d = nullptr;
            int   h = -1;
            const int64_t n = numElements(t.shape);
            if (vkc_alloc(ioCtx, t.data.size(), &d) || vkc_upload(ioCtx, d, VKC_F32, t.data.data(), VKC_F32, n, nullptr) || vkc_sync(ioCtx, nullptr) ||
                vkc_extbuf_register(d, t.data.size(), &h)) {
                std::printf("{\"ok\": false, \"error\": \"device-io input set-up: %s\"}\n", vkc_last_error(ioCtx));
                return 1;
            }
            inDev.push_back(d);
            t.dmaBufFd    = h;
            t.dmaBufDtype = DType::Float32;
            t.data.clear();
        }
        for (TensorId oid : sess->graph().outputs) {
            const int64_t n = numElements(sess->graph().tensors[oid].shape);
            void         *d = nullptr;
            int           h = -1;
            if (vkc_alloc(ioCtx, (size_t) n * 4, &d) || vkc_extbuf_register(d, (size_t) n * 4, &h)) {
                std::printf("{\"ok\": false, \"error\": \"device-io output set-up\"}\n");
                return 1;
            }
            outDev.push_back(d);
            outHandle.push_back(h);
            outElems.push_back(n);
        }
    }
#else
    if (deviceIo) {
        std::printf("{\"ok\": false, \"error\": \"--device-io is only built into the cuda driver\"}\n");
        return 1;
    }
#endif
    for (int it = 0; it < warmup + iters; ++it) {
        outs.clear();
#ifdef VKNN_DRIVER_HAS_CUDA
        if (deviceIo) {
            size_t k = 0;
            for (TensorId oid : sess->graph().outputs) {
                IOTensor b;
                b.name        = sess->graph().tensors[oid].name;
                b.dmaBufFd    = outHandle[k++];
                b.dmaBufDtype = DType::Float32;
                outs.push_back(std::move(b));
            }
        }
#endif
        auto   t0 = std::chrono::steady_clock::now();
        Status st = sess->run(ioIn, outs);
        auto   t1 = std::chrono::steady_clock::now();
        if (st != Status::Ok) {
            std::printf("{\"ok\": false, \"error\": \"run status %d\"}\n", (int) st);
            return 1;
        }
        if (it >= warmup) ms.push_back(std::chrono::duration<double, std::milli>(t1 - t0).count());
    }
    std::sort(ms.begin(), ms.end());

#ifdef VKNN_DRIVER_HAS_CUDA
    if (deviceIo) {
        // the results never touched host memory inside the Session: fetch them from the registered buffers now
        for (size_t k = 0; k < outs.size(); ++k) {
            if (!outs[k].data.empty() || outs[k].dmaBufFd != outHandle[k]) {
                std::printf("{\"ok\": false, \"error\": \"device-io output %zu came back through host memory\"}\n", k);
                return 1;
            }
            outs[k].data.resize((size_t) outElems[k] * 4);
            if (vkc_download(ioCtx, outs[k].data.data(), VKC_F32, outDev[k], VKC_F32, outElems[k], nullptr) || vkc_sync(ioCtx, nullptr)) {
                std::printf("{\"ok\": false, \"error\": \"device-io download: %s\"}\n", vkc_last_error(ioCtx));
                return 1;
            }
            vkc_extbuf_unregister(outHandle[k]);
            vkc_free(ioCtx, outDev[k]);
        }
        for (size_t k = 0; k < inDev.size(); ++k) {
            vkc_extbuf_unregister(ioIn[k].dmaBufFd);
            vkc_free(ioCtx, inDev[k]);
        }
    }
#endif
    std::ofstream out(outPath, std::ios::binary);
    for (auto &o : outs) {
        out.write(reinterpret_cast<const char *>(o.data.data()), (std::streamsize) o.data.size());
    }
    out.close();

    std::ostringstream js;
    js << "{\"ok\": true, \"backend\": \"" << backend << "\", \"median_ms\": " << ms[ms.size() / 2] << ", \"min_ms\": " << ms.front()
       << ", \"nodes\": [";
    auto        nb    = sess->nodeBackends();
    const auto &nodes = sess->graph().nodes;
    for (size_t i = 0; i < nodes.size(); ++i) {
        js << (i ? ", " : "") << "[\"" << opTypeName(nodes[i].type) << "\", " << (i < nb.size() ? (int) nb[i] : -1) << ", " << nodes[i].subOp
           << ", " << (nodes[i].fusedBias != kNoTensor ? 1 : 0) << "]";
    }
    js << "], \"profile\": [";
    {
        const auto &recs = sess->profiler().records();
        for (size_t i = 0; i < recs.size(); ++i)
            js << (i ? ", " : "") << "[\"" << recs[i].name << "\", \"" << opTypeName(recs[i].type) << "\", \"" << recs[i].backend << "\", " << recs[i].gpuMs << "]";
    }
    js << "], \"outputs\": [";
    for (size_t i = 0; i < outs.size(); ++i) {
        js << (i ? ", " : "") << "{\"name\": \"" << outs[i].name << "\", \"shape\": [";
        for (size_t d = 0; d < outs[i].shape.size(); ++d) js << (d ? ", " : "") << outs[i].shape[d];
        js << "]}";
    }
    js << "]}";
    std::printf("%s\n", js.str().c_str());
    return 0;
}
