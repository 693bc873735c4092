// Device helpers shared by the attention kernels (attention.cu) and the single-sequence persistent decode kernel
// (decode_persistent.cu): byte -> float conversion, the rotation, and the three order-preserving loops of the
// reference's softmax(QK)V (src/runtime/TenzoEngine.cpp:662-694, :823-851 of the reference).
#pragma once
#include "common.cuh"

namespace tz {

constexpr int kChunk = 128;          // V rows per bulk copy (two in flight)
constexpr int kHd = 128;             // head_dim (the reference hard-wires 16 x 8 lanes, :833-850)

// signed byte -> float without I2F: place (b ^ 0x80) in the mantissa of 2^23, subtract 2^23+128.
__device__ __forceinline__ float s8_to_f(uint32_t word_xor80, int byte) {
    const uint32_t sel = 0x7540u | (uint32_t)byte;
    return __uint_as_float(prmt(word_xor80, 0x4B000000u, sel)) - 8388736.0f;
}

__device__ __forceinline__ void rope_pair(float x0, float x1, const float* cs, const float* sn, int i, float& r0, float& r1) {
    r0 = x0;
    r1 = x1;
    if (cs) {
        const float c = cs[i], s = sn[i];
        r0 = __fmaf_rn(x0, c, -(x1 * s));      // fmsub(x0, c, x1*s)   :475
        r1 = __fmaf_rn(x0, s, x1 * c);         // fmadd(x0, s, x1*c)   :476
    }
}

// The same rotation with the coefficients already in registers.
__device__ __forceinline__ void rope_rotate(float x0, float x1, bool rotate, float c, float s, float& r0, float& r1) {
    r0 = x0;
    r1 = x1;
    if (rotate) {
        r0 = __fmaf_rn(x0, c, -(x1 * s));
        r1 = __fmaf_rn(x0, s, x1 * c);
    }
}

// The scores / e_t / weights of one (sequence, kv-head group) live in shared memory head-major: w[g][t] at
// base + g * tp + t, tp = max_len rounded up to 4. A head's values for consecutive keys are then contiguous: the
// scoring lanes store without bank conflicts, the sequential softmax sum reads four keys per load, and the value sum
// fetches four keys of one head per LDS.128.

// Value sum over one staged chunk for output dim `vcol - chunk base`: o[g] = fma(V[t][d], w[g][t], o[g])
// for t in order (:842-851). Keys are taken eight at a time with the next eight already requested
// from shared memory (two register sets, alternating), so the loads stay off the dependent chain.
// wg = weights of head 0 at the chunk's first key (16-byte aligned: chunks start at multiples of 128 keys).
template <int GH>
__device__ __forceinline__ void value_sum_chunk(const unsigned char* vcol, const float* wg, int tp, int nkeys, float (&o)[GH]) {
    constexpr int U = 8;
    uint32_t va[U], vb[U];
    float wa[GH][U], wb[GH][U];
    auto loadg = [&](int gi, uint32_t (&v)[U], float (&w)[GH][U]) {
#pragma unroll
        for (int u = 0; u < U; ++u) v[u] = vcol[(gi * U + u) * kHd];
#pragma unroll
        for (int g = 0; g < GH; ++g) {
            const float4* p = reinterpret_cast<const float4*>(wg + (size_t)g * tp + gi * U);
            const float4 lo = p[0], hi = p[1];
            w[g][0] = lo.x; w[g][1] = lo.y; w[g][2] = lo.z; w[g][3] = lo.w;
            w[g][4] = hi.x; w[g][5] = hi.y; w[g][6] = hi.z; w[g][7] = hi.w;
        }
    };
    auto compg = [&](const uint32_t (&v)[U], const float (&w)[GH][U]) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const float vf = __uint_as_float((v[u] ^ 0x80u) | 0x4B000000u) - 8388736.0f;
#pragma unroll
            for (int g = 0; g < GH; ++g) o[g] = __fmaf_rn(vf, w[g][u], o[g]);
        }
    };
    const int full = nkeys / U;
    int gi = 0;
    if (full > 0) loadg(0, va, wa);
    while (gi + 1 < full) {
        loadg(gi + 1, vb, wb);
        compg(va, wa);
        if (gi + 2 < full) loadg(gi + 2, va, wa);
        compg(vb, wb);
        gi += 2;
    }
    if (gi < full) compg(va, wa);
    for (int kl = full * U; kl < nkeys; ++kl) {
        const uint32_t b = vcol[kl * kHd];
        const float vf = __uint_as_float((b ^ 0x80u) | 0x4B000000u) - 8388736.0f;
#pragma unroll
        for (int g = 0; g < GH; ++g) o[g] = __fmaf_rn(vf, wg[(size_t)g * tp + kl], o[g]);
    }
}

// sum_t e[t], left to right (:824-829), e 16-byte aligned and contiguous: four keys per load, sixteen keys in flight
// while the previous sixteen are added (a dependent fp32 add takes 4.5 cycles; one load per add would double that).
__device__ __forceinline__ float sequential_sum(const float* e, int T) {
    const float4* p = reinterpret_cast<const float4*>(e);
    float4 a[4], b[4];
    float sum = 0.0f;
    auto loadg = [&](int gi, float4 (&v)[4]) {
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = p[gi * 4 + u];
    };
    auto addg = [&](const float4 (&v)[4]) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            sum = __fadd_rn(sum, v[u].x);
            sum = __fadd_rn(sum, v[u].y);
            sum = __fadd_rn(sum, v[u].z);
            sum = __fadd_rn(sum, v[u].w);
        }
    };
    const int full = T / 16;
    int gi = 0;
    if (full > 0) loadg(0, a);
    while (gi + 1 < full) {
        loadg(gi + 1, b);
        addg(a);
        if (gi + 2 < full) loadg(gi + 2, a);
        addg(b);
        gi += 2;
    }
    if (gi < full) addg(a);
    for (int t = full * 16; t < T; ++t) sum = __fadd_rn(sum, e[t]);
    return sum;
}

// e[g][t] = expf(e[g][t] - max[g]) for t < T, by all `n_threads` threads of the CTA (whole warps: the table
// lookup is a shuffle, so every lane makes every call).
template <int GH>
__device__ __forceinline__ void exp_in_place(float* e, int T, int tp, const float* mx, int tid, int n_threads) {
    const int lane = tid & 31;
    const unsigned long long tab = kExp2fTab[lane];
    const uint32_t tab_lo = (uint32_t)tab, tab_hi = (uint32_t)(tab >> 32);
    constexpr int U = 4;
#pragma unroll
    for (int g = 0; g < GH; ++g) {
        float* row = e + (size_t)g * tp;
        const float m = mx[g];
        for (int base = 0; base < T; base += U * n_threads) {
            float x[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int t = base + u * n_threads + tid;
                x[u] = t < T ? row[t] - m : 0.0f;
            }
#pragma unroll
            for (int u = 0; u < U; ++u) x[u] = expf_reference_bits_lanes(x[u], tab_lo, tab_hi);
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int t = base + u * n_threads + tid;
                if (t < T) row[t] = x[u];
            }
        }
    }
}

}  // namespace tz
