// Device helpers shared by every kernel of the W8A8 linear-layer library (sm_100a).
//
// Arithmetic contracts restated from the reference (paths under crates/inferrous-qwen3/):
//   bf16_rne   src/kernels.rs:12-15    f32 -> nearest-even bf16 via the integer bit trick
//   round_i8   src/kernels.rs:25-34    clamp(+-127), cvt.rni.s32.f32, NaN -> 0
//   every FP32 multiply / add / divide is a separately rounded IEEE operation
//   (src/kernels.rs:4-7; the reference builds with --no-fmad, tools/cuda.sh:21).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace w8a8 {

// Code of a device-side wait that expired; written to the per-device status word (w8a8_device_status).
enum DeviceWait : uint32_t {
    WAIT_NONE = 0,
    WAIT_TMA_FULL = 1,    // consumer waited for a TMA stage to land
    WAIT_STAGE_EMPTY = 2, // producer waited for the MMA to release a stage
    WAIT_ACC_FULL = 3,    // epilogue waited for an accumulator
    WAIT_ACC_EMPTY = 4,   // MMA waited for the epilogue to drain an accumulator
    WAIT_PEER = 5,        // tensor-parallel all-reduce waited for another rank's partial outputs
    FAULT_CACHE_RANGE = 6,  // not a wait: a token id or cache position read from device memory was out of range; the access was skipped
    WAIT_GRID = 7,        // a CTA of the resident decode kernel waited for the others at a grid-wide barrier
};

__device__ __forceinline__ float bf16_rne(float x) {
    uint32_t u = __float_as_uint(x);
    u = (u + 0x7fffu + ((u >> 16) & 1u)) & 0xffff0000u;
    return __uint_as_float(u);
}
__device__ __forceinline__ uint16_t bf16_bits(float x) { return (uint16_t)(__float_as_uint(bf16_rne(x)) >> 16); }
__device__ __forceinline__ float bf16_to_f32(uint16_t b) { return __uint_as_float(((uint32_t)b) << 16); }

__device__ __forceinline__ int round_i8(float x) {
    // Selects (not fminf/fmaxf) so that NaN stays NaN, as Rust's f32::clamp does.
    x = (x < -127.0f) ? -127.0f : x;
    x = (x > 127.0f) ? 127.0f : x;
    int r;
    asm("cvt.rni.s32.f32 %0, %1;" : "=r"(r) : "f"(x));  // NaN converts to 0
    return r;
}

// q = round_i8(x / s) with one multiply instead of one IEEE division per element, bit-identical to the
// division the reference performs (src/kernels.rs:448: round(div(x, s))), and without the two conversion-unit
// instructions (floor, float -> int) that made the quantizers issue-bound on that unit.
// inv = rcp.rn(s) is computed once per row.  t = x * inv differs from the true quotient by at most
// (1 + 2^-24)^2 - 1 < 1.2e-7 relative, i.e. by less than 1.6e-5 for |t| <= 127, and the correctly rounded
// quotient differs from the true one by at most half an ulp (3.8e-6 below 128).  Two numbers that close
// round to different integers only if a rounding boundary k + 0.5 lies between or on them, so whenever t is
// farther than 4e-5 from every k + 0.5 both round alike; otherwise (about one element in 12 000) the exact
// division decides.  Values beyond +-127 (infinities included) clamp to the same code either way; NaN gives 0.
// Rounding: c + 1.5 * 2^23 has an ulp of 1, so the addition rounds c (|c| <= 127) to the nearest even integer
// and leaves that integer in the low mantissa bits; subtracting the constant again gives it back as a float.
__device__ __forceinline__ int quant_code(float x, float s, float inv) {
    const float t = __fmul_rn(x, inv);
    const float c = fminf(fmaxf(t, -127.0f), 127.0f);  // a NaN becomes -127 here and is put right below
    const float y = __fadd_rn(c, 12582912.0f);
    const float r = __fadd_rn(y, -12582912.0f);        // rne(c)
    if (fabsf(__fadd_rn(c, -r)) > 0.49996f) return round_i8(__fdiv_rn(x, s));
    const int code = __float_as_int(y) - 0x4B400000;
    return t == t ? code : 0;
}

// exp(x) as the reference writes it: ex2.approx(x * log2(e)) (src/kernels.rs:21-23).
__device__ __forceinline__ float exp_approx(float x) {
    float y = __fmul_rn(x, 1.4426950408889634f);
    float r;
    asm("ex2.approx.f32 %0, %1;" : "=f"(r) : "f"(y));
    return r;
}
// src/kernels.rs:2181: bf16((g / (1 + exp(-g))) * u)
__device__ __forceinline__ float swiglu_value(float g, float u) {
    return bf16_rne(__fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, exp_approx(-g))), u));
}
__device__ __forceinline__ float rsqrt_approx(float x) {
    float r;
    asm("rsqrt.approx.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

// |v| as an order-preserving unsigned key; NaN contributes 0 (src/kernels.rs:134-137).
__device__ __forceinline__ uint32_t absmax_key(float v) {
    uint32_t bits = __float_as_uint(v) & 0x7fffffffu;
    return bits > 0x7f800000u ? 0u : bits;
}

// Greedy selection key: larger value wins, equal values (0.0 == -0.0 included) go to the LOWER index, as the
// reference's select_token does (src/kernels.rs:2191-2231).  A non-finite value poisons the row (index ~0).
__device__ __forceinline__ unsigned long long argmax_key(float v, uint32_t index) {
    if (!(fabsf(v) <= 3.402823466e38f)) return ~0ull;  // NaN or infinity: wins every max, flags the row as bad
    v = v + 0.0f;                                       // -0.0 -> +0.0
    const uint32_t b = __float_as_uint(v);
    const uint32_t ordered = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
    return ((unsigned long long)ordered << 32) | (unsigned long long)(0xffffffffu - index);
}

// The epilogue of every projection (src/kernels.rs:290): two separately rounded multiplies, then bf16.
__device__ __forceinline__ float dequant(int acc, float a_scale, float w_scale) {
    return bf16_rne(__fmul_rn(__fmul_rn(__int2float_rn(acc), a_scale), w_scale));
}

// Programmatic dependent launch (src/kernels.rs:173-184): wait for the predecessor's
// memory, then let the successor start launching.  No-ops for ordinary launches.
__device__ __forceinline__ void dependency_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ---- element carriers: bf16 storage or the reference's f32 carrier ---------------------
struct Bf16 {  // 2-byte storage
    typedef uint16_t storage;
    static constexpr int kVec = 8;  // elements per 16-byte vector
    __device__ static __forceinline__ float load(const storage *p) { return bf16_to_f32(*p); }
    __device__ static __forceinline__ void store(storage *p, float v) { *p = (uint16_t)(__float_as_uint(v) >> 16); }
};
struct F32 {
    typedef float storage;
    static constexpr int kVec = 4;
    __device__ static __forceinline__ float load(const storage *p) { return *p; }
    __device__ static __forceinline__ void store(storage *p, float v) { *p = v; }
};

// 16-byte vector load of kVec elements into floats.
template <class T> struct Vec;
template <> struct Vec<Bf16> {
    __device__ static __forceinline__ void load(const uint16_t *p, float (&v)[8]) {
        uint4 r = *reinterpret_cast<const uint4 *>(p);
        v[0] = __uint_as_float(r.x << 16); v[1] = __uint_as_float(r.x & 0xffff0000u);
        v[2] = __uint_as_float(r.y << 16); v[3] = __uint_as_float(r.y & 0xffff0000u);
        v[4] = __uint_as_float(r.z << 16); v[5] = __uint_as_float(r.z & 0xffff0000u);
        v[6] = __uint_as_float(r.w << 16); v[7] = __uint_as_float(r.w & 0xffff0000u);
    }
    // a 16-byte vector fetched earlier, kept packed until it is needed
    __device__ static __forceinline__ void unpack(const uint4 &r, float (&v)[8]) {
        v[0] = __uint_as_float(r.x << 16); v[1] = __uint_as_float(r.x & 0xffff0000u);
        v[2] = __uint_as_float(r.y << 16); v[3] = __uint_as_float(r.y & 0xffff0000u);
        v[4] = __uint_as_float(r.z << 16); v[5] = __uint_as_float(r.z & 0xffff0000u);
        v[6] = __uint_as_float(r.w << 16); v[7] = __uint_as_float(r.w & 0xffff0000u);
    }
    // v holds bf16-representable floats
    __device__ static __forceinline__ void store(uint16_t *p, const float (&v)[8]) {
        uint4 r;
        r.x = (__float_as_uint(v[0]) >> 16) | (__float_as_uint(v[1]) & 0xffff0000u);
        r.y = (__float_as_uint(v[2]) >> 16) | (__float_as_uint(v[3]) & 0xffff0000u);
        r.z = (__float_as_uint(v[4]) >> 16) | (__float_as_uint(v[5]) & 0xffff0000u);
        r.w = (__float_as_uint(v[6]) >> 16) | (__float_as_uint(v[7]) & 0xffff0000u);
        *reinterpret_cast<uint4 *>(p) = r;
    }
};
template <> struct Vec<F32> {
    __device__ static __forceinline__ void load(const float *p, float (&v)[4]) {
        float4 r = *reinterpret_cast<const float4 *>(p);
        v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
    }
    __device__ static __forceinline__ void unpack(const uint4 &r, float (&v)[4]) {
        v[0] = __uint_as_float(r.x); v[1] = __uint_as_float(r.y); v[2] = __uint_as_float(r.z); v[3] = __uint_as_float(r.w);
    }
    __device__ static __forceinline__ void store(float *p, const float (&v)[4]) {
        *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};

// Streaming 16-byte weight load: read-only path, do not keep the line in L1.
__device__ __forceinline__ uint4 ld_stream_16(const void *p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}

__device__ __forceinline__ int warp_sum_i32(int v) { return __reduce_add_sync(0xffffffffu, v); }
__device__ __forceinline__ uint32_t warp_max_u32(uint32_t v) { return __reduce_max_sync(0xffffffffu, v); }

// ---- shared by the standalone quantizers and the quantizing GEMV prologue ------------------------------------
template <int N> __device__ __forceinline__ void store_codes(int8_t *dst, const int (&c)[N]);
// the low bytes of four ints as one word (three byte permutes)
__device__ __forceinline__ uint32_t pack_codes4(int c0, int c1, int c2, int c3) {
    const uint32_t lo = __byte_perm((uint32_t)c0, (uint32_t)c1, 0x0040);  // bytes: c0.0 c1.0 . .
    const uint32_t hi = __byte_perm((uint32_t)c2, (uint32_t)c3, 0x0040);
    return __byte_perm(lo, hi, 0x5410);
}
template <> __device__ __forceinline__ void store_codes<8>(int8_t *dst, const int (&c)[8]) {
    uint2 p;
    p.x = pack_codes4(c[0], c[1], c[2], c[3]);
    p.y = pack_codes4(c[4], c[5], c[6], c[7]);
    *reinterpret_cast<uint2 *>(dst) = p;
}
template <> __device__ __forceinline__ void store_codes<4>(int8_t *dst, const int (&c)[4]) {
    *reinterpret_cast<uint32_t *>(dst) = pack_codes4(c[0], c[1], c[2], c[3]);
}

// Block-wide maximum of non-negative floats (compared as unsigned bit patterns); up to 32 warps.
__device__ __forceinline__ float block_max(float m, uint32_t *slots, int tid) {
    const int nwarps = blockDim.x >> 5;
    uint32_t k = warp_max_u32(__float_as_uint(m));
    if ((tid & 31) == 0) slots[tid >> 5] = k;
    __syncthreads();
    uint32_t v = (tid & 31) < nwarps ? slots[tid & 31] : 0u;
    v = warp_max_u32(v);
    __syncthreads();  // slots may be reused by the next row
    return __uint_as_float(v);
}

}  // namespace w8a8
