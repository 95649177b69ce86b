// GPU conformance of the C++ host mirror (inferrous_b200/host/gpu_linear.hpp) with closed-form inputs.
// The two tests follow crates/inferrous-qwen3/src/conformance.rs of the reference:
//   fused_gate_up_matches_separate   :741-839   linear_swiglu == linear_pair + swiglu, bitwise, incl. the maximum
//   integer_rounding_boundaries      :841-871   1 328 443 inputs against f64 clamp + round-half-even
// plus a worst-case accumulator check of `linear` (+-K*127^2, docs/qwen3-8b-w8a8/safety.md:34).
// Exit code 0 and a line "conformance ok" on success.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <vector>

#include "../../inferrous_b200/host/gpu_linear.hpp"

using namespace w8a8;

static uint32_t bits(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    return u;
}
static float from_bits(uint32_t u) {
    float x;
    memcpy(&x, &u, 4);
    return x;
}
static float bf16(float x) {  // src/kernels.rs:12-15
    uint32_t u = bits(x);
    u = (u + 0x7fffu + ((u >> 16) & 1u)) & 0xffff0000u;
    return from_bits(u);
}
#define CHECK(cond, ...)                  \
    do {                                  \
        if (!(cond)) {                    \
            fprintf(stderr, __VA_ARGS__); \
            fprintf(stderr, "\n");        \
            return 1;                     \
        }                                 \
    } while (0)

static int fused_gate_up_matches_separate(GpuLinear &gpu) {
    const int shapes[2][2] = {{128, 33}, {4096, 12288}};
    for (auto &sh : shapes) {
        const int k = sh[0], n = sh[1];
        std::vector<int8_t> q(k), w0((size_t)k * n), w1((size_t)k * n);
        for (int i = 0; i < k; ++i) q[i] = (int8_t)((i * 13 % 255) - 127);
        for (size_t i = 0; i < w0.size(); ++i) {
            w0[i] = (int8_t)((int)(i * 31 % 255) - 127);
            w1[i] = (int8_t)((int)(i * 17 % 251) - 125);
        }
        std::vector<float> s0(n), s1(n);
        for (int i = 0; i < n; ++i) {
            s0[i] = 0.0001f * (float)(i % 7 + 1);
            s1[i] = 0.0001f * (float)(i % 11 + 1);
        }
        auto dq = DeviceBuffer<int8_t>::from_host(q);
        auto asc = Buffer::from_host({0.002f});
        Matrix m0(w0, s0, n, k), m1(w1, s1, n, k);
        Buffer g = Buffer::zeroed(n), u = Buffer::zeroed(n), act = Buffer::zeroed(n);
        const uint32_t floor_bits = bits(1e-8f);
        auto maximum = DeviceBuffer<uint32_t>::from_host({floor_bits});
        gpu.linear_pair(dq, asc, m0, g, m1, u, 1);
        gpu.swiglu(g, u, act, &maximum, 1);
        auto eg = g.to_host_vec(gpu.stream()), eu = u.to_host_vec(gpu.stream()), ea = act.to_host_vec(gpu.stream());
        float emax = 1e-8f;
        for (float v : ea) emax = std::fmax(emax, std::fabs(v));
        CHECK(maximum.to_host_vec(gpu.stream())[0] == bits(emax), "swiglu maximum (k=%d n=%d)", k, n);
        // host check of a few gate values: bf16((acc * 0.002) * s0)
        for (int c : {0, 1, n - 1}) {
            long long acc = 0;
            for (int j = 0; j < k; ++j) acc += (long long)q[j] * w0[(size_t)c * k + j];
            volatile float a = (float)(int)acc * 0.002f;
            volatile float b = a * s0[c];
            CHECK(bits(eg[c]) == bits(bf16(b)), "gate[%d] differs from the host formula (k=%d n=%d)", c, k, n);
        }
        maximum.copy_from_host({floor_bits});
        Buffer g2 = Buffer::zeroed(n), u2 = Buffer::zeroed(n), a2 = Buffer::zeroed(n);
        gpu.linear_swiglu(dq, asc, m0, g2, m1, u2, a2, maximum, 1);
        auto hg = g2.to_host_vec(gpu.stream()), hu = u2.to_host_vec(gpu.stream()), ha = a2.to_host_vec(gpu.stream());
        for (int i = 0; i < n; ++i) {
            CHECK(bits(hg[i]) == bits(eg[i]), "gate bits at %d (k=%d n=%d)", i, k, n);
            CHECK(bits(hu[i]) == bits(eu[i]), "up bits at %d (k=%d n=%d)", i, k, n);
            CHECK(bits(ha[i]) == bits(ea[i]), "activation bits at %d (k=%d n=%d)", i, k, n);
        }
        CHECK(maximum.to_host_vec(gpu.stream())[0] == bits(emax), "activation maximum (k=%d n=%d)", k, n);
    }
    printf("fused_gate_up_matches_separate ok\n");
    return 0;
}

static int integer_rounding_boundaries(GpuLinear &gpu) {
    std::vector<float> input;
    for (uint32_t x = 0; x <= 0xffff; ++x) input.push_back(from_bits(x << 16));
    for (int x = -131072; x <= 131072; ++x) input.push_back((float)x / 1024.0f);
    for (int i = -127; i < 127; ++i) {
        const float tie = (float)i + 0.5f;
        for (uint32_t b : {bits(tie) - 1, bits(tie), bits(tie) + 1}) input.push_back(from_bits(b));
    }
    for (uint32_t x = 0; x < 1000000u; ++x) input.push_back(from_bits(x * 2654435761u));
    CHECK(input.size() == 1328443, "input count %zu", input.size());
    auto din = Buffer::from_host(input);
    DeviceBuffer<int8_t> out = DeviceBuffer<int8_t>::zeroed(input.size());
    gpu.rounding_probe(din, out);
    auto actual = out.to_host_vec(gpu.stream());
    for (size_t i = 0; i < input.size(); ++i) {
        double d = (double)input[i];
        int8_t e = 0;
        if (!std::isnan(d)) {
            d = d < -127.0 ? -127.0 : (d > 127.0 ? 127.0 : d);
            e = (int8_t)std::nearbyint(d);  // default rounding mode: ties to even
        }
        CHECK(actual[i] == e, "input bits %08x: got %d want %d", bits(input[i]), actual[i], e);
    }
    printf("integer_rounding_boundaries ok\n");
    return 0;
}

static int worst_case_accumulator(GpuLinear &gpu) {
    for (int k : {4096, 12288}) {
        const int n = 33;
        std::vector<int8_t> q(k, 127), w((size_t)n * k, 1);
        for (int j = 0; j < k; ++j) {
            w[j] = 127;
            w[(size_t)k + j] = -127;
        }
        std::vector<float> ws(n, 1.0f / 64);
        auto dq = DeviceBuffer<int8_t>::from_host(q);
        auto asc = Buffer::from_host({1.0f / 128});
        Matrix m(w, ws, n, k);
        Buffer out = Buffer::zeroed(n), res = Buffer::from_host(std::vector<float>(n, 0.0625f)), comb = Buffer::zeroed(n);
        gpu.linear_quantized(dq, asc, m, out, 1);
        auto y = out.to_host_vec(gpu.stream());
        const int acc = k * 127 * 127;  // exceeds 2^24: the int -> float conversion must round to nearest even
        auto expect = [&](int a) {
            volatile float f = (float)a;
            volatile float g = f * (1.0f / 128);
            volatile float h = g * (1.0f / 64);
            return bf16(h);
        };
        CHECK(bits(y[0]) == bits(expect(acc)), "k=%d +worst case", k);
        CHECK(bits(y[1]) == bits(expect(-acc)), "k=%d -worst case", k);
        CHECK(bits(y[2]) == bits(expect(k * 127)), "k=%d plain row", k);
        // linear_residual: quantize on the device from bf16-valued activations, then projection + residual sum
        std::vector<float> x(k, 2.0f);
        x[0] = 127.0f;
        Buffer dx = Buffer::from_host(x), scale(1);
        DeviceBuffer<int8_t> dq2(k);
        gpu.linear_residual(dx, m, dq2, scale, out, nullptr, res, comb, 1);
        auto y2 = out.to_host_vec(gpu.stream()), c2 = comb.to_host_vec(gpu.stream());
        for (int i = 0; i < n; ++i) {
            volatile float s = 0.0625f + y2[i];
            CHECK(bits(c2[i]) == bits(bf16(s)), "k=%d combined[%d]", k, i);
        }
        CHECK(scale.to_host_vec(gpu.stream())[0] == 1.0f, "k=%d scale of a row whose absmax is 127", k);
    }
    printf("worst_case_accumulator ok\n");
    return 0;
}

int main() {
    try {
        GpuLinear gpu(0);
        if (integer_rounding_boundaries(gpu)) return 1;
        if (worst_case_accumulator(gpu)) return 1;
        if (fused_gate_up_matches_separate(gpu)) return 1;
        // error behaviour: a failed precondition is an error value, never a trap
        try {
            Buffer x(100), s(1);
            DeviceBuffer<int8_t> q(100);
            gpu.quantize(x, 100, q, s);  // width not a multiple of 128
            fprintf(stderr, "bad width was accepted\n");
            return 1;
        } catch (const Error &e) {
            if (e.status != W8A8_ERR_ALIGNMENT) return 1;
        }
    } catch (const std::exception &e) {
        fprintf(stderr, "error: %s\n", e.what());
        return 1;
    }
    printf("conformance ok\n");
    return 0;
}
