// C++ host harness for a whole Qwen3 W8A8 forward pass and greedy generation over the C ABI.
//
// The reference host is Rust (crates/inferrous-qwen3/src/gpu.rs, src/model.rs); no Rust toolchain is available to
// this build, so the same call sequence is written in C++:
//   Model::load            src/model.rs:46-165      -> Qwen3Bundle::load (the on-disk bundle of tools/prepare.py)
//   GpuModel::new          src/gpu.rs:245-336       -> Qwen3Model::Qwen3Model (upload, workspaces, caches, control buffer)
//   GpuModel::forward      src/gpu.rs:528-817       -> Qwen3Model::forward
//   GpuModel::generate     src/gpu.rs:818-929       -> Qwen3Model::generate (prefill eager; one decode step captured as a
//                                                      CUDA graph with programmatic edges and replayed, src/gpu.rs:303-333)
// Like the reference: f32 activation buffers holding bf16 values, one stream, caller-visible errors instead of traps,
// {token, position} uploaded and the selected token read back every step.
// Unlike the reference: Q|K|V are one concatenated matrix (identical channel for channel with per-channel scales); the
// head runs as the reference's bf16 head with the selection fused (qwen3_head_bf16; logits bit-identical to `head`,
// src/kernels.rs:2233-2257) or, on request (HeadKind::W8A8), quantized per output channel when the bundle is loaded
// (tools/prepare.py:79-81) as a W8A8 projection (w8a8_linear_argmax); sha256 digests of the manifest are not verified here (the
// Python reader does), only names, sizes, finiteness and the weight checks of src/model.rs:143-145.
#pragma once

#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <memory>
#include <sstream>
#include <string>
#include <vector>

#include "../../include/qwen3_glue.h"
#include "gpu_linear.hpp"

namespace w8a8 {

struct Qwen3Config {
    int layers = 36, hidden = 4096, q_heads = 32, kv_heads = 8, intermediate = 12288, vocab = 151936, context = 4096;
    float eps = 1e-6f;
    int q_width() const { return q_heads * 128; }
    int kv_width() const { return kv_heads * 128; }
    int qkv_width() const { return (q_heads + 2 * kv_heads) * 128; }
};

namespace detail {
inline std::string slurp(const std::string &path) {
    std::ifstream f(path, std::ios::binary);
    if (!f) throw std::runtime_error("cannot open " + path);
    std::ostringstream s;
    s << f.rdbuf();
    return s.str();
}
// The unsigned integer that follows `"key":` in a machine-written JSON document (json.dumps of tools/prepare.py).
inline long json_uint(const std::string &text, const std::string &key) {
    const std::string needle = "\"" + key + "\":";
    size_t at = text.find(needle);
    if (at == std::string::npos) throw std::runtime_error("manifest: missing " + key);
    at += needle.size();
    while (at < text.size() && (text[at] == ' ' || text[at] == '\n')) ++at;
    size_t end = at;
    while (end < text.size() && text[end] >= '0' && text[end] <= '9') ++end;
    if (end == at) throw std::runtime_error("manifest: " + key + " is not an unsigned integer");
    return std::stol(text.substr(at, end - at));
}
template <class T> std::vector<T> read_tensor(const std::string &dir, const std::string &name, size_t count) {
    const std::string raw = slurp(dir + "/" + name + ".bin");
    if (raw.size() != count * sizeof(T)) throw std::runtime_error(name + ": size mismatch");
    std::vector<T> v(count);
    memcpy(v.data(), raw.data(), raw.size());
    return v;
}
inline std::vector<float> read_floats(const std::string &dir, const std::string &name, size_t count) {
    auto v = read_tensor<float>(dir, name, count);
    for (float x : v)
        if (!std::isfinite(x)) throw std::runtime_error(name + ": nonfinite float");
    return v;
}
// An int8 weight matrix and its per-channel scales as Model::load admits them (src/model.rs:143-145): the code -128
// never occurs in symmetric quantization, and a scale must be positive.
inline std::vector<int8_t> read_codes(const std::string &dir, const std::string &name, size_t count) {
    auto v = read_tensor<int8_t>(dir, name, count);
    for (int8_t x : v)
        if (x == -128) throw std::runtime_error(name + ": invalid quantized weight");
    return v;
}
inline std::vector<float> read_scales(const std::string &dir, const std::string &name, size_t count) {
    auto v = read_floats(dir, name, count);
    for (float x : v)
        if (!(x > 0.0f)) throw std::runtime_error(name + ": invalid weight scale");
    return v;
}
inline float widen(uint16_t b) {
    const uint32_t u = (uint32_t)b << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}
}  // namespace detail

enum class HeadKind { Bf16, W8A8 };

// Host copy of a bundle (src/model.rs `Model`, without the tokenizer).
struct Qwen3Bundle {
    struct LayerTensors {
        std::vector<float> norm1, norm2, qnorm, knorm;
        std::vector<int8_t> qkv, o, gate, up, down;
        std::vector<float> qkv_scale, o_scale, gate_scale, up_scale, down_scale;
    };
    Qwen3Config config;
    std::vector<uint16_t> embedding;
    std::vector<uint16_t> head_bf16;  // HeadKind::Bf16: the checkpoint's head as it is
    std::vector<int8_t> head;         // HeadKind::W8A8: its per-channel int8 quantization
    std::vector<float> head_scale, final_gain, rope;
    std::vector<LayerTensors> layers;

    static Qwen3Bundle load(const std::string &dir, HeadKind head_kind = HeadKind::Bf16) {
        using namespace detail;
        const std::string manifest = slurp(dir + "/manifest.json");
        if (json_uint(manifest, "format_version") != 1) throw std::runtime_error("unsupported bundle format version");
        if (json_uint(manifest, "head_dim") != 128) throw std::runtime_error("unsupported head_dim");
        Qwen3Bundle b;
        Qwen3Config &c = b.config;
        c.layers = (int)json_uint(manifest, "num_hidden_layers");
        c.hidden = (int)json_uint(manifest, "hidden_size");
        c.q_heads = (int)json_uint(manifest, "num_attention_heads");
        c.kv_heads = (int)json_uint(manifest, "num_key_value_heads");
        c.intermediate = (int)json_uint(manifest, "intermediate_size");
        c.vocab = (int)json_uint(manifest, "vocab_size");
        c.context = (int)json_uint(manifest, "max_context");
        const size_t H = c.hidden, I = c.intermediate, V = c.vocab;
        b.embedding = read_tensor<uint16_t>(dir, "embedding", V * H);
        b.final_gain = read_floats(dir, "final_gain", H);
        b.rope = read_floats(dir, "rope", (size_t)c.context * 128);
        if (head_kind == HeadKind::Bf16) {
            b.head_bf16 = read_tensor<uint16_t>(dir, "head", V * H);
        } else {
            // W8A8 head: per-output-channel symmetric int8 of the bf16 head (the formula of tools/prepare.py:79-81)
            const auto head = read_tensor<uint16_t>(dir, "head", V * H);
            b.head.resize(V * H);
            b.head_scale.resize(V);
            for (size_t n = 0; n < V; ++n) {
                float m = 0.0f;
                for (size_t k = 0; k < H; ++k) m = std::fmax(m, std::fabs(widen(head[n * H + k])));
                const float s = std::fmax(m, 1e-8f) / 127.0f;
                b.head_scale[n] = s;
                for (size_t k = 0; k < H; ++k) {
                    float r = std::nearbyint(widen(head[n * H + k]) / s);  // round-half-even in the default rounding mode
                    r = r < -127.0f ? -127.0f : (r > 127.0f ? 127.0f : r);
                    b.head[n * H + k] = (int8_t)r;
                }
            }
        }
        b.layers.resize(c.layers);
        for (int l = 0; l < c.layers; ++l) {
            const std::string p = "layer." + std::to_string(l) + ".";
            LayerTensors &t = b.layers[l];
            t.norm1 = read_floats(dir, p + "norm1", H);
            t.norm2 = read_floats(dir, p + "norm2", H);
            t.qnorm = read_floats(dir, p + "qnorm", 128);
            t.knorm = read_floats(dir, p + "knorm", 128);
            for (const char *name : {"q", "k", "v"}) {
                const size_t n = name[0] == 'q' ? c.q_width() : c.kv_width();
                const auto w = read_codes(dir, p + name + ".w", n * H);
                const auto s = read_scales(dir, p + name + ".scale", n);
                t.qkv.insert(t.qkv.end(), w.begin(), w.end());
                t.qkv_scale.insert(t.qkv_scale.end(), s.begin(), s.end());
            }
            t.o = read_codes(dir, p + "o.w", H * c.q_width());
            t.o_scale = read_scales(dir, p + "o.scale", H);
            t.gate = read_codes(dir, p + "gate.w", I * H);
            t.gate_scale = read_scales(dir, p + "gate.scale", I);
            t.up = read_codes(dir, p + "up.w", I * H);
            t.up_scale = read_scales(dir, p + "up.scale", I);
            t.down = read_codes(dir, p + "down.w", H * I);
            t.down_scale = read_scales(dir, p + "down.scale", H);
        }
        return b;
    }
};

// gpu::Workspace (src/gpu.rs:76-143) for a fixed row count.
struct Qwen3Workspace {
    int rows;
    Buffer hidden, residual, qkv, attention, gate, up, act, scales;
    DeviceBuffer<int8_t> quant4, quant_o, quant12;
    DeviceBuffer<uint32_t> maxima;
    Qwen3Workspace(const Qwen3Config &c, int rows_)
        : rows(rows_), hidden((size_t)rows_ * c.hidden), residual((size_t)rows_ * c.hidden), qkv((size_t)rows_ * c.qkv_width()),
          attention((size_t)rows_ * c.q_width()), gate((size_t)rows_ * c.intermediate), up((size_t)rows_ * c.intermediate),
          act((size_t)rows_ * c.intermediate), scales(rows_), quant4((size_t)rows_ * c.hidden),
          quant_o((size_t)rows_ * c.q_width()), quant12((size_t)rows_ * c.intermediate), maxima(rows_) {}
};

class Qwen3Model {
   public:
    struct Generation {
        std::vector<uint32_t> token_ids;
        std::vector<double> step_seconds;
    };

    explicit Qwen3Model(const Qwen3Bundle &b, int device = 0)
        : c_(b.config), gpu_(device), embedding_(DeviceBuffer<uint16_t>::from_host(b.embedding)),
          final_gain_(Buffer::from_host(b.final_gain)), rope_(Buffer::from_host(b.rope)),
          control_(DeviceBuffer<uint32_t>::zeroed(2)), next_(DeviceBuffer<uint32_t>::zeroed(1)), head_q_(b.config.hidden),
          head_scale_(1), head_x_(b.config.hidden), decode_(b.config, 1) {
        if (!b.head_bf16.empty())
            head_bf16_ = DeviceBuffer<uint16_t>::from_host(b.head_bf16);
        else
            head_ = std::make_unique<Matrix>(b.head, b.head_scale, b.config.vocab, b.config.hidden);
        for (const auto &t : b.layers) {
            auto l = std::make_unique<Layer>(t, c_);
            l->k_cache = DeviceBuffer<uint16_t>::zeroed((size_t)c_.context * c_.kv_width());
            l->v_cache = DeviceBuffer<uint16_t>::zeroed((size_t)c_.context * c_.kv_width());
            layers_.push_back(std::move(l));
        }
        make_plan();
    }
    ~Qwen3Model() {
        if (exec_) cudaGraphExecDestroy(exec_);
        if (graph_) cudaGraphDestroy(graph_);
        if (plan_) qwen3_decode_plan_destroy(plan_);
    }
    // true when one-token steps run as the single resident kernel (qwen3_decode_layers)
    bool resident_decode() const { return plan_ != nullptr; }
    const Qwen3Config &config() const { return c_; }

    // Queues one forward pass of ws.rows rows: `ids` holds their token ids (the control buffer in decode, whose word
    // 0 is the token), control_[1] the position of the first row.  The selected token lands in next_.
    void forward(Qwen3Workspace &ws, const uint32_t *ids) {
        cudaStream_t s = gpu_.stream();
        const int rows = ws.rows, H = c_.hidden;
        ensure(qwen3_embedding(ids, embedding_.ptr(), rows, H, c_.vocab, ws.hidden.ptr(), W8A8_F32, s), "embedding");
        if (rows == 1 && plan_) {  // every layer of the step inside one kernel; the same bits as the launches below
            ensure(qwen3_decode_layers(plan_, ws.hidden.ptr(), control_.ptr(), s), "decode layers");
            return head(ws);
        }
        for (auto &lp : layers_) {
            Layer &l = *lp;
            gpu_.norm_quantize(ws.hidden, l.norm1, nullptr, ws.quant4, ws.scales, &ws.maxima);
            gpu_.linear_quantized(ws.quant4, ws.scales, l.qkv, ws.qkv, rows);
            ensure(qwen3_prepare_qk(ws.qkv.ptr(), W8A8_F32, c_.qkv_width(), rows, c_.q_heads, c_.kv_heads, l.qnorm.ptr(),
                                    l.knorm.ptr(), rope_.ptr(), control_.ptr(), l.k_cache.ptr(), l.v_cache.ptr(), c_.context, s),
                   "prepare_qk");
            ensure(qwen3_attention(ws.qkv.ptr(), W8A8_F32, c_.qkv_width(), rows, c_.q_heads, c_.kv_heads, l.k_cache.ptr(),
                                   l.v_cache.ptr(), control_.ptr(), ws.attention.ptr(), c_.q_width(), c_.context, nullptr, s),
                   "attention");
            gpu_.quantize(ws.attention, c_.q_width(), ws.quant_o, ws.scales);
            ensure(w8a8_linear(ws.quant_o.ptr(), ws.scales.ptr(), l.o.handle, rows, ws.hidden.ptr(), nullptr, ws.residual.ptr(),
                               W8A8_F32, s),
                   "o projection");
            gpu_.norm_quantize(ws.residual, l.norm2, nullptr, ws.quant4, ws.scales, &ws.maxima);
            if (rows == 1) {  // src/gpu.rs:727-748
                gpu_.linear_swiglu(ws.quant4, ws.scales, l.gate, ws.gate, l.up, ws.up, ws.act, ws.maxima, rows);
                gpu_.quantize_with_max(ws.act, c_.intermediate, ws.maxima, ws.quant12, ws.scales);
            } else {          // src/gpu.rs:749-779
                gpu_.linear_quantized(ws.quant4, ws.scales, l.gate, ws.gate, rows);
                gpu_.linear_quantized(ws.quant4, ws.scales, l.up, ws.up, rows);
                gpu_.swiglu(ws.gate, ws.up, ws.act, nullptr, rows);
                gpu_.quantize(ws.act, c_.intermediate, ws.quant12, ws.scales);
            }
            ensure(w8a8_linear(ws.quant12.ptr(), ws.scales.ptr(), l.down.handle, rows, ws.residual.ptr(), nullptr, ws.hidden.ptr(),
                               W8A8_F32, s),
                   "down projection");
        }
        head(ws);
    }

    // Final norm of the last row, output head and greedy selection; the token lands in next_.
    void head(Qwen3Workspace &ws) {
        cudaStream_t s = gpu_.stream();
        const int H = c_.hidden;
        const float *last = ws.hidden.ptr() + (size_t)(ws.rows - 1) * H;
        const bool bf16_head = head_ == nullptr;
        // the final norm; with the bf16 head its output row is what the head multiplies (`norm`, src/gpu.rs:798)
        ensure(w8a8_rmsnorm_quantize(last, final_gain_.ptr(), W8A8_F32, c_.eps, 1, H, H, head_q_.ptr(), head_scale_.ptr(),
                                     bf16_head ? head_x_.ptr() : nullptr, nullptr, s),
               "final norm");
        if (bf16_head)
            ensure(qwen3_head_bf16(head_x_.ptr(), W8A8_F32, head_bf16_.ptr(), c_.vocab, H, nullptr, next_.ptr(), nullptr, s), "head");
        else
            ensure(w8a8_linear_argmax(head_q_.ptr(), head_scale_.ptr(), head_->handle, 1, next_.ptr(), nullptr, s), "head");
    }

    Generation generate(const std::vector<uint32_t> &prompt, int max_tokens, bool use_graph = true) {
        if (prompt.empty() || (int)prompt.size() + max_tokens > c_.context)
            throw std::invalid_argument("prompt must be non-empty and prompt + max_tokens must fit the context");
        cudaStream_t s = gpu_.stream();
        if (use_graph && !exec_) capture_decode();
        Qwen3Workspace prefill(c_, (int)prompt.size());
        auto ids = DeviceBuffer<uint32_t>::from_host(prompt);
        Generation out;
        uint32_t token = 0, position = 0;
        int rows = (int)prompt.size();
        for (int step = 0; step < max_tokens; ++step) {
            const auto start = std::chrono::steady_clock::now();
            const uint32_t control[2] = {token, position};
            cuda_ensure(cudaMemcpyAsync(control_.ptr(), control, sizeof control, cudaMemcpyHostToDevice, s), "control upload");
            if (step == 0)
                forward(prefill, ids.ptr());
            else if (use_graph)
                cuda_ensure(cudaGraphLaunch(exec_, s), "cudaGraphLaunch");
            else
                forward(decode_, control_.ptr());
            cuda_ensure(cudaMemcpyAsync(&token, next_.ptr(), sizeof token, cudaMemcpyDeviceToHost, s), "token read-back");
            cuda_ensure(cudaStreamSynchronize(s), "cudaStreamSynchronize");
            out.step_seconds.push_back(std::chrono::duration<double>(std::chrono::steady_clock::now() - start).count());
            if (token == 0xffffffffu) throw std::runtime_error("nonfinite or empty logits");
            out.token_ids.push_back(token);
            position += (uint32_t)rows;
            rows = 1;
        }
        uint32_t detail = 0;
        ensure(w8a8_device_status(s, &detail), "device status");
        return out;
    }

   private:
    struct Layer {
        Buffer norm1, norm2, qnorm, knorm;
        Matrix qkv, o, gate, up, down;
        DeviceBuffer<uint16_t> k_cache, v_cache;
        Layer(const Qwen3Bundle::LayerTensors &t, const Qwen3Config &c)
            : norm1(Buffer::from_host(t.norm1)), norm2(Buffer::from_host(t.norm2)), qnorm(Buffer::from_host(t.qnorm)),
              knorm(Buffer::from_host(t.knorm)), qkv(t.qkv, t.qkv_scale, c.qkv_width(), c.hidden),
              o(t.o, t.o_scale, c.hidden, c.q_width()), gate(t.gate, t.gate_scale, c.intermediate, c.hidden),
              up(t.up, t.up_scale, c.intermediate, c.hidden), down(t.down, t.down_scale, c.hidden, c.intermediate) {}
    };

    // The resident decode kernel's plan, where the library supports the shape and the device (W8A8_RESIDENT_DECODE=0
    // keeps the launch-per-operator step).
    void make_plan() {
        const char *off = std::getenv("W8A8_RESIDENT_DECODE");
        if (off && off[0] == '0') return;
        std::vector<qwen3_layer_desc> table;
        for (auto &lp : layers_) {
            Layer &l = *lp;
            qwen3_layer_desc d{};
            d.norm1 = l.norm1.ptr(); d.norm2 = l.norm2.ptr(); d.q_gain = l.qnorm.ptr(); d.k_gain = l.knorm.ptr();
            d.qkv = l.qkv.handle; d.o = l.o.handle; d.gate = l.gate.handle; d.up = l.up.handle; d.down = l.down.handle;
            d.k_cache = l.k_cache.ptr(); d.v_cache = l.v_cache.ptr();
            table.push_back(d);
        }
        const int st = qwen3_decode_plan_create(table.data(), (int)table.size(), c_.hidden, c_.q_heads, c_.kv_heads, c_.intermediate,
                                                c_.context, c_.eps, rope_.ptr(), W8A8_F32, &plan_);
        if (st == W8A8_ERR_UNSUPPORTED) plan_ = nullptr;
        else ensure(st, "decode plan");
    }

    // One decode step as a graph (src/gpu.rs:303-333, src/graph.rs:63-127): a warm-up launch outside the capture, then
    // the capture with every kernel on a programmatic edge.
    void capture_decode() {
        cudaStream_t s = gpu_.stream();
        ensure(w8a8_set_programmatic_launch(1), "programmatic launch");
        cuda_ensure(cudaMemsetAsync(control_.ptr(), 0, 8, s), "cudaMemsetAsync");
        forward(decode_, control_.ptr());
        cuda_ensure(cudaStreamSynchronize(s), "cudaStreamSynchronize");
        cuda_ensure(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal), "cudaStreamBeginCapture");
        try {
            forward(decode_, control_.ptr());
        } catch (...) {
            cudaGraph_t broken = nullptr;
            cudaStreamEndCapture(s, &broken);
            if (broken) cudaGraphDestroy(broken);
            w8a8_set_programmatic_launch(0);
            throw;
        }
        cuda_ensure(cudaStreamEndCapture(s, &graph_), "cudaStreamEndCapture");
        ensure(w8a8_set_programmatic_launch(0), "programmatic launch");
        cuda_ensure(cudaGraphInstantiate(&exec_, graph_, 0), "cudaGraphInstantiate");
    }

    Qwen3Config c_;
    GpuLinear gpu_;
    DeviceBuffer<uint16_t> embedding_;
    Buffer final_gain_, rope_;
    std::unique_ptr<Matrix> head_;        // W8A8 head, or
    DeviceBuffer<uint16_t> head_bf16_;    // the reference's bf16 head
    std::vector<std::unique_ptr<Layer>> layers_;
    DeviceBuffer<uint32_t> control_, next_;
    DeviceBuffer<int8_t> head_q_;
    Buffer head_scale_, head_x_;
    Qwen3Workspace decode_;
    cudaGraph_t graph_ = nullptr;
    cudaGraphExec_t exec_ = nullptr;
    qwen3_decode_plan_t plan_ = nullptr;
};

}  // namespace w8a8
