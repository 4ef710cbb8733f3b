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
// eight or more FMAs.  Pixel and filter-entry coordinates are decoded once into small shared tables, so the
// gather itself has no divisions.  dW keeps its accumulators in registers across all tiles of the CTA and
// writes one partial per CTA; a second kernel adds the partials in fixed order (bit-reproducible, no atomics).
#include "common.cuh"

namespace aether {

static constexpr int SC_THREADS = 256;
static constexpr int SC_MAX_K = 64;
static constexpr int SC_MAX_TP = 256;

struct SmallcGeom {
    int S, H, W, Cin, Cout, fH, fW, sH, sW, pH, pW, Ho, Wo, K;
    long long P;      // output pixels
    int lanes;        // thread groups along pixels (forward) / along K (dW) = 256 / (Cout/4)
    int TP;           // pixels per tile (power of two)
    int tp_shift;     // log2(TP)
    int cg_shift;     // log2(Cout/4)
    int R;            // 4-pixel groups per thread and tile (forward)
    int KPG;          // filter entries per thread (dW)
};

struct SmallcTables {
    int k_i[SC_MAX_K], k_j[SC_MAX_K], k_c[SC_MAX_K];            // filter entry k -> (row, column, channel)
    int pix_s[SC_MAX_TP], pix_h[SC_MAX_TP], pix_w[SC_MAX_TP];   // tile pixel -> (sample*H, top input row, left input column)
};

__device__ __forceinline__ void fill_ktab(const SmallcGeom& g, SmallcTables& t) {
    for (int k = threadIdx.x; k < g.K; k += SC_THREADS) {
        const int tap = k / g.Cin;
        t.k_c[k] = k - tap * g.Cin;
        t.k_i[k] = tap / g.fW;
        t.k_j[k] = tap - (tap / g.fW) * g.fW;
    }
}

// Gathers col^T for the tile starting at pixel p0 into colT[K][TP] (zero outside the image / past the end).
// Contains two block barriers; every thread of the CTA must call it.
__device__ __forceinline__ void stage_colT(const SmallcGeom& g, SmallcTables& t, const float* __restrict__ x, long long p0,
                                           float* colT) {
    for (int q = threadIdx.x; q < g.TP; q += SC_THREADS) {
        const long long p = p0 + q;
        if (p < g.P) {
            const int wo = (int)(p % g.Wo);
            const long long r = p / g.Wo;
            t.pix_w[q] = wo * g.sW - g.pW;
            t.pix_h[q] = (int)(r % g.Ho) * g.sH - g.pH;
            t.pix_s[q] = (int)(r / g.Ho) * g.H;
        } else {
            t.pix_w[q] = 0; t.pix_h[q] = -(1 << 20); t.pix_s[q] = 0;   // fails the row test below
        }
    }
    __syncthreads();
    const int n = g.K << g.tp_shift;
    for (int e = threadIdx.x; e < n; e += SC_THREADS) {
        const int k = e >> g.tp_shift, pl = e & (g.TP - 1);
        const int hi = t.pix_h[pl] + t.k_i[k], wi = t.pix_w[pl] + t.k_j[k];
        float v = 0.f;
        if (hi >= 0 && hi < g.H && wi >= 0 && wi < g.W) v = x[((size_t)(t.pix_s[pl] + hi) * g.W + wi) * g.Cin + t.k_c[k]];
        colT[e] = v;
    }
    __syncthreads();
}

#define SC_FMA4(A, S, V)                                                                  \
    A.x = fmaf(S, V.x, A.x); A.y = fmaf(S, V.y, A.y); A.z = fmaf(S, V.z, A.z); A.w = fmaf(S, V.w, A.w)

template <int R>
__global__ void __launch_bounds__(SC_THREADS) smallc_fwd_kernel(const SmallcGeom g, const float* __restrict__ x,
                                                                const float* __restrict__ w, const float* __restrict__ b,
                                                                float* __restrict__ y, float* __restrict__ stats,
                                                                long long ntiles) {
    extern __shared__ float sm[];
    __shared__ SmallcTables tab;
    __shared__ __align__(16) float red_s[SC_THREADS * 4];    // statistics, used once at the end of the kernel
    __shared__ __align__(16) float red_q[SC_THREADS * 4];
    __shared__ float red_n[SC_THREADS];
    // Statistics of this thread's pixels: count, sum and sum of squares of (y - pivot).  The pivot is the thread's
    // first output value, so the sums stay small whatever the channel's mean is (no cancellation when |mean| >> std).
    float4 st_s = make_float4(0.f, 0.f, 0.f, 0.f), st_q = st_s, st_p = st_s;
    float st_n = 0.f;
    float* wsm = sm;                          // [K][Cout]
    float* colT = sm + g.K * g.Cout;          // [K][TP]
    for (int e = threadIdx.x; e < g.K * g.Cout; e += SC_THREADS) wsm[e] = w[e];
    fill_ktab(g, tab);
    const int cg = threadIdx.x & ((1 << g.cg_shift) - 1), pl = threadIdx.x >> g.cg_shift;
    const float4 bias = b ? *reinterpret_cast<const float4*>(b + cg * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
    __syncthreads();
    for (long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        const long long p0 = tile << g.tp_shift;
        stage_colT(g, tab, x, p0, colT);
        float4 acc[R][4];
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int q = 0; q < 4; ++q) acc[r][q] = bias;
        for (int k = 0; k < g.K; ++k) {
            const float4 wv = *reinterpret_cast<const float4*>(wsm + k * g.Cout + cg * 4);
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const float4 cv = *reinterpret_cast<const float4*>(colT + (k << g.tp_shift) + (r * g.lanes + pl) * 4);
                SC_FMA4(acc[r][0], cv.x, wv);
                SC_FMA4(acc[r][1], cv.y, wv);
                SC_FMA4(acc[r][2], cv.z, wv);
                SC_FMA4(acc[r][3], cv.w, wv);
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const long long p = p0 + (r * g.lanes + pl) * 4 + q;
                if (p < g.P) {
                    __stcs(reinterpret_cast<float4*>(y + (size_t)p * g.Cout + cg * 4), acc[r][q]);
                    if (stats) {
                        if (st_n == 0.f) st_p = acc[r][q];
                        const float dx = acc[r][q].x - st_p.x, dy = acc[r][q].y - st_p.y;
                        const float dz = acc[r][q].z - st_p.z, dw = acc[r][q].w - st_p.w;
                        st_s.x += dx; st_s.y += dy; st_s.z += dz; st_s.w += dw;
                        st_q.x = fmaf(dx, dx, st_q.x); st_q.y = fmaf(dy, dy, st_q.y);
                        st_q.z = fmaf(dz, dz, st_q.z); st_q.w = fmaf(dw, dw, st_q.w);
                        st_n += 1.f;
                    }
                }
            }
        __syncthreads();                      // colT is rewritten by the next tile's gather
    }
    if (stats) {
        // One (count, mean, M2) triple per channel and CTA: every thread turns its pivoted sums into (n, mean, M2),
        // and the pixel lanes are merged in fixed order with Chan's formula.
        const float inv = st_n > 0.f ? 1.f / st_n : 0.f;
        float4 mean, m2;
        mean.x = st_p.x + st_s.x * inv; m2.x = st_q.x - st_s.x * st_s.x * inv;
        mean.y = st_p.y + st_s.y * inv; m2.y = st_q.y - st_s.y * st_s.y * inv;
        mean.z = st_p.z + st_s.z * inv; m2.z = st_q.z - st_s.z * st_s.z * inv;
        mean.w = st_p.w + st_s.w * inv; m2.w = st_q.w - st_s.w * st_s.w * inv;
        reinterpret_cast<float4*>(red_s)[threadIdx.x] = mean;
        reinterpret_cast<float4*>(red_q)[threadIdx.x] = m2;
        red_n[threadIdx.x] = st_n;
        __syncthreads();
        if (threadIdx.x < g.Cout) {
            const int c = threadIdx.x, cgi = c >> 2, k = c & 3;
            float N = 0.f, M = 0.f, M2 = 0.f;
            for (int l = 0; l < g.lanes; ++l) {
                const int t = (l << g.cg_shift) + cgi;
                const float nl = red_n[t];
                if (nl == 0.f) continue;
                const float tot = N + nl, delta = red_s[t * 4 + k] - M;
                M2 += red_q[t * 4 + k] + delta * delta * N * nl / tot;
                M += delta * nl / tot;
                N = tot;
            }
            float* out = stats + (size_t)blockIdx.x * 3 * g.Cout;
            out[c] = N;
            out[g.Cout + c] = M;
            out[2 * g.Cout + c] = fmaxf(M2, 0.f);
        }
    }
}

// Partial sums per CTA: part[block][K + 1][Cout]  (row K holds the dB partial).
template <int KPG>
__global__ void __launch_bounds__(SC_THREADS) smallc_dw_kernel(const SmallcGeom g, const float* __restrict__ x,
                                                               const float* __restrict__ dy, float* __restrict__ part,
                                                               long long ntiles) {
    extern __shared__ float sm[];
    __shared__ SmallcTables tab;
    float* colT = sm;                         // [K][TP]
    float* dys = sm + (g.K << g.tp_shift);    // [TP][Cout]
    const int cgs = 1 << g.cg_shift;
    const int cg = threadIdx.x & (cgs - 1), kg = threadIdx.x >> g.cg_shift;   // filter entries kg, kg+lanes, ...
    float4 acc[KPG];
#pragma unroll
    for (int a = 0; a < KPG; ++a) acc[a] = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 bsum = make_float4(0.f, 0.f, 0.f, 0.f);
    const bool want_x = (x != nullptr);
    fill_ktab(g, tab);
    __syncthreads();
    for (long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        const long long p0 = tile << g.tp_shift;
        for (int e = threadIdx.x; e < (g.TP << g.cg_shift); e += SC_THREADS) {
            const long long p = p0 + (e >> g.cg_shift);
            reinterpret_cast<float4*>(dys)[e] =
                (p < g.P) ? __ldcs(reinterpret_cast<const float4*>(dy + (size_t)p * g.Cout) + (e & (cgs - 1)))
                          : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        if (want_x) stage_colT(g, tab, x, p0, colT);
        else __syncthreads();
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
                        const float4 cv = *reinterpret_cast<const float4*>(colT + (k << g.tp_shift) + pb);
                        SC_FMA4(acc[a], cv.x, d0);
                        SC_FMA4(acc[a], cv.y, d1);
                        SC_FMA4(acc[a], cv.z, d2);
                        SC_FMA4(acc[a], cv.w, d3);
                    }
                }
            }
        }
        __syncthreads();                      // dys / colT are rewritten by the next tile
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
static int ilog2(int v) {
    int s = 0;
    while ((1 << s) < v) ++s;
    return s;
}

static bool smallc_geom(const AetherConvDesc& d, SmallcGeom& g) {
    g.K = d.fH * d.fW * d.Cin;
    if (g.K > SC_MAX_K || d.Cin > 4) return false;
    if (d.Cout < 16 || d.Cout > 256 || (d.Cout & (d.Cout - 1))) return false;    // 4-channel groups must divide 256 threads
    g.S = d.S; g.H = d.H; g.W = d.W; g.Cin = d.Cin; g.Cout = d.Cout; g.fH = d.fH; g.fW = d.fW;
    g.sH = d.sH; g.sW = d.sW; g.pH = d.padH; g.pW = d.padW;
    conv_out_hw(d, g.Ho, g.Wo);
    g.P = 1LL * d.S * g.Ho * g.Wo;
    g.cg_shift = ilog2(d.Cout >> 2);
    g.lanes = SC_THREADS >> g.cg_shift;
    g.R = 64 / (g.lanes * 4) > 1 ? 64 / (g.lanes * 4) : 1;
    g.TP = g.lanes * 4 * g.R;
    g.tp_shift = ilog2(g.TP);
    g.KPG = ceil_div(g.K, g.lanes);
    return g.KPG <= 16 && g.TP <= SC_MAX_TP && g.R <= 4;
}

bool smallc_conv_eligible(const AetherConvDesc& d) {
    SmallcGeom g;
    return smallc_geom(d, g);
}

static int smallc_blocks(const SmallcGeom& g) {
    const long long ntiles = (g.P + g.TP - 1) / g.TP;
    long long nb = 4LL * 148;                 // four resident CTAs per SM hide each other's staging latency
    if (nb > ntiles) nb = ntiles;
    return (int)(nb < 1 ? 1 : nb);
}

size_t smallc_conv_workspace_bytes(const AetherConvDesc& d) {
    SmallcGeom g;
    if (!smallc_geom(d, g)) return 0;
    return align_up((size_t)smallc_blocks(g) * (g.K + 1) * g.Cout * sizeof(float), 1024);
}

template <typename Kern>
static int smallc_smem(Kern kernel, size_t smem, PerDeviceSmem& configured, const char* what) {
    if (smem <= 32 * 1024) return AE_OK;              // static + dynamic above 48 KB needs the opt-in
    return ensure_dynamic_smem(kernel, (int)smem, configured, what);
}

template <int R>
static int launch_smallc_fwd(const SmallcGeom& g, const float* x, const float* w, const float* b, float* y, float* stats,
                             int nb, long long ntiles, size_t smem, cudaStream_t st) {
    static PerDeviceSmem configured;
    int rc = smallc_smem(smallc_fwd_kernel<R>, smem, configured, "smallc_fwd");
    if (rc) return rc;
    smallc_fwd_kernel<R><<<nb, SC_THREADS, smem, st>>>(g, x, w, b, y, stats, ntiles);
    count_launch();
    return check_launch("smallc_fwd_kernel");
}

static int smallc_fwd_blocks(const SmallcGeom& g) {
    const long long ntiles = (g.P + g.TP - 1) / g.TP;
    long long nb = 4LL * 148;
    if (nb > ntiles) nb = ntiles;
    return (int)(nb < 1 ? 1 : nb);
}

// Blocks of [3][Cout] (count, mean, M2) partial statistics the forward kernel writes when asked to: one per CTA.
long long smallc_conv_stats_blocks(const AetherConvDesc& d) {
    SmallcGeom g;
    return smallc_geom(d, g) ? smallc_fwd_blocks(g) : 0;
}

int smallc_conv_fwd(const AetherConvDesc& d, const float* x, const float* w, const float* b, float* y, float* stats,
                    cudaStream_t st) {
    SmallcGeom g;
    if (!smallc_geom(d, g)) return set_error(AE_UNSUPPORTED, "smallc_conv_fwd: shape not supported");
    const long long ntiles = (g.P + g.TP - 1) / g.TP;
    const size_t smem = (size_t)(g.K * g.Cout + g.K * g.TP) * sizeof(float);
    const int nb = smallc_fwd_blocks(g);
    if (g.R == 1) return launch_smallc_fwd<1>(g, x, w, b, y, stats, nb, ntiles, smem, st);
    if (g.R == 2) return launch_smallc_fwd<2>(g, x, w, b, y, stats, nb, ntiles, smem, st);
    return launch_smallc_fwd<4>(g, x, w, b, y, stats, nb, ntiles, smem, st);
}

template <int KPG>
static int launch_smallc_dw(const SmallcGeom& g, const float* x, const float* dy, float* part, int nb, long long ntiles,
                            size_t smem, cudaStream_t st) {
    static PerDeviceSmem configured;
    int rc = smallc_smem(smallc_dw_kernel<KPG>, smem, configured, "smallc_dw");
    if (rc) return rc;
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

// Sums nb partials of [K + 1][Cout] floats (row K = dB) into dw / db in fixed order (also used by conv_first_tc.cu).
int smallc_reduce_partials(const float* part, int nb, int K, int Cout, float* dw, float* db, cudaStream_t st) {
    smallc_reduce_kernel<<<ceil_div((K + 1) * Cout, 32), 256, 0, st>>>(part, nb, K, Cout, dw, db);
    count_launch();
    return check_launch("smallc_reduce_kernel");
}

}  // namespace aether
