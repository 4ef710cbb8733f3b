// Per-channel statistics (count, mean, M2) taken in a convolution kernel's epilogue for the Batch_Norm that follows
// (CNN/models/CNN_classes_cupy.py:467-470 computes them in a pass of its own).
//
// Every epilogue warp keeps, per output column it owns, a running sum and sum of squares of (a - pivot), where a is
// the accumulator value (the output before the bias) and the pivot is the column's mean over the warp's FIRST tile.
// Sums about a value that close to the mean stay small, so M2 = Q - S*S/n does not cancel when a channel's mean is
// far from zero compared with its spread (inputs with an offset, outputs of a ReLU).  The first tile itself is
// summed without a pivot (it is not known yet) and converted once: S <- 0, Q <- Q - S*P.
//
// Shared memory per warp: float[3][128] = running sum, running sum of squares, pivot (all zero at the start).
#pragma once
#include <cuda_runtime.h>

namespace aether {

static constexpr int STATS_WARP_FLOATS = 3 * 128;

// Two fp32 values in one 64-bit register, and the packed arithmetic of sm_100 (one instruction for two results, each
// rounded exactly like the scalar add / fma): the per-element work of the statistics is three such instructions per
// two elements instead of three scalar ones per element.
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("add.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("mul.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
// Running (sum, sum of squares) of four consecutive columns, as two packed pairs each.
struct Stats4 {
    f32x2 s01, s23, q01, q23;
    __device__ __forceinline__ void clear() { s01 = s23 = q01 = q23 = 0ull; }
    // adds the four values d (already taken about the pivot, zero for rows that do not count)
    __device__ __forceinline__ void add(f32x2 d01, f32x2 d23) {
        s01 = add2(s01, d01); s23 = add2(s23, d23);
        q01 = fma2(d01, d01, q01); q23 = fma2(d23, d23, q23);
    }
    __device__ __forceinline__ float4 sum() const { float4 r; unpack2(s01, r.x, r.y); unpack2(s23, r.z, r.w); return r; }
    __device__ __forceinline__ float4 sumsq() const { float4 r; unpack2(q01, r.x, r.y); unpack2(q23, r.z, r.w); return r; }
};

// Lanes 0..3 of a warp add one tile's column sums (s, q: four consecutive columns from `off` on, already reduced
// over the warp's rows) to the running sums.  `first` marks the warp's first tile with any valid row: its sums were
// taken without a pivot, so the pivot is set from them (`rows` = valid rows of the tile in this warp's quarter).
__device__ __forceinline__ void stats_fold(float* stat_w, int off, float4 s, float4 q, bool first, float rows) {
    float4* ps = reinterpret_cast<float4*>(stat_w + off);
    float4* pq = reinterpret_cast<float4*>(stat_w + 128 + off);
    if (first) {
        const float inv = 1.f / rows;
        const float4 piv = make_float4(s.x * inv, s.y * inv, s.z * inv, s.w * inv);
        *reinterpret_cast<float4*>(stat_w + 256 + off) = piv;
        q.x -= s.x * piv.x; q.y -= s.y * piv.y; q.z -= s.z * piv.z; q.w -= s.w * piv.w;
        s = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float4 rs = *ps, rq = *pq;
    rs.x += s.x; rs.y += s.y; rs.z += s.z; rs.w += s.w;
    rq.x += q.x; rq.y += q.y; rq.z += q.z; rq.w += q.w;
    *ps = rs;
    *pq = rq;
}

// (mean without the bias, M2) of column `c` (warp-local index) after `rows` rows.
__device__ __forceinline__ void stats_result(const float* stat_w, int c, float rows, float& mean, float& m2) {
    const float s = stat_w[c], q = stat_w[128 + c];
    const float m = rows > 0.f ? s / rows : 0.f;
    mean = stat_w[256 + c] + m;
    m2 = fmaxf(q - s * m, 0.f);
}

}  // namespace aether
