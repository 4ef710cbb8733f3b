// First-layer convolutions: very few input channels (grey or RGB images; Conv_Layer with input depth 1 or 3,
// CNN/models/CNN_classes_cupy.py:52-66).  K = fH*fW*Cin is 9 or 27, far below one tensor-core K block, and
// the layer moves ~10 FLOP per byte, so these are fp32 CUDA-core kernels built around HBM traffic:
// the activation (x) is tiny, the output / upstream gradient is read or written exactly once, coalesced.
//
//   forward : y[p][d]  = b[d] + sum_k col[p][k] * w[k][d]       col = the K input values under pixel p
//   dW, dB  : dw[k][d] = sum_p col[p][k] * dy[p][d],  db[d] = sum_p dy[p][d]
//
// A CTA stages the im2col values of a tile of pixels (transposed, [K][TP]) in shared memory; a thread owns
// four consecutive output channels and works on four pixels at a time, so each shared-memory read feeds
// eight or more FMAs.  dW keeps its accumulators in registers across all tiles of the CTA and writes one
// partial per CTA; a second kernel adds the partials in fixed order (bit-reproducible, no atomics).
#include "common.cuh"

namespace aether {

static constexpr int SC_THREADS = 256;
static constexpr int SC_MAX_K = 64;

struct SmallcGeom {
    int S, H, W, Cin, Cout, fH, fW, sH, sW, pH, pW, Ho, Wo, K;
    long long P;      // output pixels
    int lanes;        // thread groups along pixels (forward) / along K (dW) = 256 / (Cout/4)
    int TP;           // pixels per tile
    int R;            // 4-pixel groups per thread and tile (forward)
    int KPG;          // filter entries per thread (dW)
};

// Gathers col^T for the tile starting at pixel p0 into colT[K][TP] (zero outside the image / past the end).
__device__ __forceinline__ void stage_colT(const SmallcGeom& g, const float* __restrict__ x, long long p0, float* colT) {
    for (int e = threadIdx.x; e < g.K * g.TP; e += SC_THREADS) {
        const int k = e / g.TP, pl = e - k * g.TP;
        const long long p = p0 + pl;
        float v = 0.f;
        if (p < g.P) {
            const int wo = (int)(p % g.Wo);
            const long long q = p / g.Wo;
            const int ho = (int)(q % g.Ho);
            const int s = (int)(q / g.Ho);
            const int c = k % g.Cin;
            const int tap = k / g.Cin;
            const int i = tap / g.fW, j = tap - i * g.fW;
            const int hi = ho * g.sH + i - g.pH, wi = wo * g.sW + j - g.pW;
            if (hi >= 0 && hi < g.H && wi >= 0 && wi < g.W) v = x[(((size_t)s * g.H + hi) * g.W + wi) * g.Cin + c];
        }
        colT[e] = v;
    }
}

__global__ void __launch_bounds__(SC_THREADS) smallc_fwd_kernel(const SmallcGeom g, const float* __restrict__ x,
                                                                const float* __restrict__ w, const float* __restrict__ b,
                                                                float* __restrict__ y, long long ntiles) {
    extern __shared__ float sm[];
    float* wsm = sm;                          // [K][Cout]
    float* colT = sm + g.K * g.Cout;          // [K][TP]
    for (int e = threadIdx.x; e < g.K * g.Cout; e += SC_THREADS) wsm[e] = w[e];
    const int cgs = g.Cout >> 2;
    const int cg = threadIdx.x % cgs, pl = threadIdx.x / cgs;
    const float4 bias = b ? *reinterpret_cast<const float4*>(b + cg * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
    for (long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        const long long p0 = tile * g.TP;
        __syncthreads();                      // previous tile's readers are done (and weights are staged)
        stage_colT(g, x, p0, colT);
        __syncthreads();
        for (int r = 0; r < g.R; ++r) {
            const int pb = (r * g.lanes + pl) * 4;            // first of this thread's 4 pixels in the tile
            float4 acc[4] = {bias, bias, bias, bias};
            for (int k = 0; k < g.K; ++k) {
                const float4 wv = *reinterpret_cast<const float4*>(wsm + k * g.Cout + cg * 4);
                const float4 cv = *reinterpret_cast<const float4*>(colT + k * g.TP + pb);
                acc[0].x = fmaf(cv.x, wv.x, acc[0].x); acc[0].y = fmaf(cv.x, wv.y, acc[0].y);
                acc[0].z = fmaf(cv.x, wv.z, acc[0].z); acc[0].w = fmaf(cv.x, wv.w, acc[0].w);
                acc[1].x = fmaf(cv.y, wv.x, acc[1].x); acc[1].y = fmaf(cv.y, wv.y, acc[1].y);
                acc[1].z = fmaf(cv.y, wv.z, acc[1].z); acc[1].w = fmaf(cv.y, wv.w, acc[1].w);
                acc[2].x = fmaf(cv.z, wv.x, acc[2].x); acc[2].y = fmaf(cv.z, wv.y, acc[2].y);
                acc[2].z = fmaf(cv.z, wv.z, acc[2].z); acc[2].w = fmaf(cv.z, wv.w, acc[2].w);
                acc[3].x = fmaf(cv.w, wv.x, acc[3].x); acc[3].y = fmaf(cv.w, wv.y, acc[3].y);
                acc[3].z = fmaf(cv.w, wv.z, acc[3].z); acc[3].w = fmaf(cv.w, wv.w, acc[3].w);
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const long long p = p0 + pb + q;
                if (p < g.P) *reinterpret_cast<float4*>(y + (size_t)p * g.Cout + cg * 4) = acc[q];
            }
        }
    }
}

// Partial sums per CTA: part[block][K + 1][Cout]  (row K holds the dB partial).
template <int KPG>
__global__ void __launch_bounds__(SC_THREADS) smallc_dw_kernel(const SmallcGeom g, const float* __restrict__ x,
                                                               const float* __restrict__ dy, float* __restrict__ part,
                                                               long long ntiles) {
    extern __shared__ float sm[];
    float* colT = sm;                         // [K][TP]
    float* dys = sm + g.K * g.TP;             // [TP][Cout]
    const int cgs = g.Cout >> 2;
    const int cg = threadIdx.x % cgs, kg = threadIdx.x / cgs;      // this thread's filter entries: kg, kg+lanes, ...
    float4 acc[KPG];
#pragma unroll
    for (int a = 0; a < KPG; ++a) acc[a] = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 bsum = make_float4(0.f, 0.f, 0.f, 0.f);
    const bool want_x = (x != nullptr);
    for (long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        const long long p0 = tile * g.TP;
        __syncthreads();
        if (want_x) stage_colT(g, x, p0, colT);
        for (int e = threadIdx.x; e < g.TP * cgs; e += SC_THREADS) {
            const int pl = e / cgs, c4 = e - pl * cgs;
            const long long p = p0 + pl;
            reinterpret_cast<float4*>(dys)[e] =
                (p < g.P) ? *reinterpret_cast<const float4*>(dy + (size_t)p * g.Cout + c4 * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        __syncthreads();
        for (int pb = 0; pb < g.TP; pb += 4) {
            const float4 d0 = *reinterpret_cast<const float4*>(dys + (size_t)(pb + 0) * g.Cout + cg * 4);
            const float4 d1 = *reinterpret_cast<const float4*>(dys + (size_t)(pb + 1) * g.Cout + cg * 4);
            const float4 d2 = *reinterpret_cast<const float4*>(dys + (size_t)(pb + 2) * g.Cout + cg * 4);
            const float4 d3 = *reinterpret_cast<const float4*>(dys + (size_t)(pb + 3) * g.Cout + cg * 4);
            if (kg == 0) {
                bsum.x += (d0.x + d1.x) + (d2.x + d3.x); bsum.y += (d0.y + d1.y) + (d2.y + d3.y);
                bsum.z += (d0.z + d1.z) + (d2.z + d3.z); bsum.w += (d0.w + d1.w) + (d2.w + d3.w);
            }
            if (want_x) {
#pragma unroll
                for (int a = 0; a < KPG; ++a) {
                    const int k = kg + a * g.lanes;
                    if (k < g.K) {
                        const float4 cv = *reinterpret_cast<const float4*>(colT + k * g.TP + pb);
                        acc[a].x = fmaf(cv.x, d0.x, acc[a].x); acc[a].y = fmaf(cv.x, d0.y, acc[a].y);
                        acc[a].z = fmaf(cv.x, d0.z, acc[a].z); acc[a].w = fmaf(cv.x, d0.w, acc[a].w);
                        acc[a].x = fmaf(cv.y, d1.x, acc[a].x); acc[a].y = fmaf(cv.y, d1.y, acc[a].y);
                        acc[a].z = fmaf(cv.y, d1.z, acc[a].z); acc[a].w = fmaf(cv.y, d1.w, acc[a].w);
                        acc[a].x = fmaf(cv.z, d2.x, acc[a].x); acc[a].y = fmaf(cv.z, d2.y, acc[a].y);
                        acc[a].z = fmaf(cv.z, d2.z, acc[a].z); acc[a].w = fmaf(cv.z, d2.w, acc[a].w);
                        acc[a].x = fmaf(cv.w, d3.x, acc[a].x); acc[a].y = fmaf(cv.w, d3.y, acc[a].y);
                        acc[a].z = fmaf(cv.w, d3.z, acc[a].z); acc[a].w = fmaf(cv.w, d3.w, acc[a].w);
                    }
                }
            }
        }
    }
    float* out = part + (size_t)blockIdx.x * (g.K + 1) * g.Cout;
#pragma unroll
    for (int a = 0; a < KPG; ++a) {
        const int k = kg + a * g.lanes;
        if (k < g.K) *reinterpret_cast<float4*>(out + (size_t)k * g.Cout + cg * 4) = acc[a];
    }
    if (kg == 0) *reinterpret_cast<float4*>(out + (size_t)g.K * g.Cout + cg * 4) = bsum;
}

// dw[e] / db[d] = sum over CTAs of the partials, 8 lanes per output combined in fixed order.
__global__ void __launch_bounds__(256) smallc_reduce_kernel(const float* __restrict__ part, int nblocks, int K, int Cout,
                                                            float* __restrict__ dw, float* __restrict__ db) {
    __shared__ float red[8][32];
    const int el = threadIdx.x & 31, ln = threadIdx.x >> 5;
    const int e = blockIdx.x * 32 + el;
    const int total = (K + 1) * Cout;
    float s = 0.f;
    if (e < total)
        for (int b = ln; b < nblocks; b += 8) s += part[(size_t)b * total + e];
    red[ln][el] = s;
    __syncthreads();
    if (ln == 0 && e < total) {
        float t = 0.f;
#pragma unroll
        for (int l = 0; l < 8; ++l) t += red[l][el];
        if (e < K * Cout) {
            if (dw) dw[e] = t;
        } else if (db) {
            db[e - K * Cout] = t;
        }
    }
}

// ---------------------------------------------------------------------------------- host
static bool smallc_geom(const AetherConvDesc& d, SmallcGeom& g) {
    g.K = d.fH * d.fW * d.Cin;
    if (g.K > SC_MAX_K || d.Cin > 4) return false;
    if (d.Cout < 16 || d.Cout > 256 || (d.Cout & (d.Cout - 1))) return false;    // 4-channel groups must divide 256 threads
    g.S = d.S; g.H = d.H; g.W = d.W; g.Cin = d.Cin; g.Cout = d.Cout; g.fH = d.fH; g.fW = d.fW;
    g.sH = d.sH; g.sW = d.sW; g.pH = d.padH; g.pW = d.padW;
    conv_out_hw(d, g.Ho, g.Wo);
    g.P = 1LL * d.S * g.Ho * g.Wo;
    g.lanes = SC_THREADS / (d.Cout >> 2);
    g.R = 64 / (g.lanes * 4) > 1 ? 64 / (g.lanes * 4) : 1;
    g.TP = g.lanes * 4 * g.R;
    g.KPG = ceil_div(g.K, g.lanes);
    return g.KPG <= 16;
}

bool smallc_conv_eligible(const AetherConvDesc& d) {
    SmallcGeom g;
    return smallc_geom(d, g);
}

static int smallc_blocks(const SmallcGeom& g) {
    const long long ntiles = (g.P + g.TP - 1) / g.TP;
    long long nb = 2LL * 148;
    if (nb > ntiles) nb = ntiles;
    return (int)(nb < 1 ? 1 : nb);
}

size_t smallc_conv_workspace_bytes(const AetherConvDesc& d) {
    SmallcGeom g;
    if (!smallc_geom(d, g)) return 0;
    return align_up((size_t)smallc_blocks(g) * (g.K + 1) * g.Cout * sizeof(float), 1024);
}

int smallc_conv_fwd(const AetherConvDesc& d, const float* x, const float* w, const float* b, float* y, cudaStream_t st) {
    SmallcGeom g;
    if (!smallc_geom(d, g)) return set_error(AE_UNSUPPORTED, "smallc_conv_fwd: shape not supported");
    const long long ntiles = (g.P + g.TP - 1) / g.TP;
    const size_t smem = (size_t)(g.K * g.Cout + g.K * g.TP) * sizeof(float);
    static size_t configured = 0;
    if (smem > 48 * 1024 && smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(smallc_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return set_error(AE_CUDA, "cudaFuncSetAttribute(smallc_fwd): %s", cudaGetErrorString(e));
        configured = smem;
    }
    long long nb = 4LL * 148;
    if (nb > ntiles) nb = ntiles;
    smallc_fwd_kernel<<<(int)nb, SC_THREADS, smem, st>>>(g, x, w, b, y, ntiles);
    count_launch();
    return check_launch("smallc_fwd_kernel");
}

template <int KPG>
static int launch_smallc_dw(const SmallcGeom& g, const float* x, const float* dy, float* part, int nb, long long ntiles,
                            size_t smem, cudaStream_t st) {
    static size_t configured = 0;
    if (smem > 48 * 1024 && smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(smallc_dw_kernel<KPG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return set_error(AE_CUDA, "cudaFuncSetAttribute(smallc_dw): %s", cudaGetErrorString(e));
        configured = smem;
    }
    smallc_dw_kernel<KPG><<<nb, SC_THREADS, smem, st>>>(g, x, dy, part, ntiles);
    count_launch();
    return check_launch("smallc_dw_kernel");
}

int smallc_conv_bwd_filter(const AetherConvDesc& d, const float* x, const float* dy, float* dw, float* db, void* ws,
                           size_t ws_bytes, cudaStream_t st) {
    SmallcGeom g;
    if (!smallc_geom(d, g)) return set_error(AE_UNSUPPORTED, "smallc_conv_bwd_filter: shape not supported");
    if (!ws || ws_bytes < smallc_conv_workspace_bytes(d))
        return set_error(AE_BAD_ARG, "conv workspace too small: %zu < %zu", ws_bytes, smallc_conv_workspace_bytes(d));
    const long long ntiles = (g.P + g.TP - 1) / g.TP;
    const int nb = smallc_blocks(g);
    const size_t smem = (size_t)(g.K * g.TP + g.TP * g.Cout) * sizeof(float);
    float* part = static_cast<float*>(ws);
    const float* xs = dw ? x : nullptr;       // only dB requested: skip the filter-gradient work
    int rc;
    if (g.KPG <= 1) rc = launch_smallc_dw<1>(g, xs, dy, part, nb, ntiles, smem, st);
    else if (g.KPG <= 2) rc = launch_smallc_dw<2>(g, xs, dy, part, nb, ntiles, smem, st);
    else if (g.KPG <= 4) rc = launch_smallc_dw<4>(g, xs, dy, part, nb, ntiles, smem, st);
    else if (g.KPG <= 8) rc = launch_smallc_dw<8>(g, xs, dy, part, nb, ntiles, smem, st);
    else rc = launch_smallc_dw<16>(g, xs, dy, part, nb, ntiles, smem, st);
    if (rc) return rc;
    smallc_reduce_kernel<<<ceil_div((g.K + 1) * g.Cout, 32), 256, 0, st>>>(part, nb, g.K, g.Cout, dw, db);
    count_launch();
    return check_launch("smallc_reduce_kernel");
}

}  // namespace aether
