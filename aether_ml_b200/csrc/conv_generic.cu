// fp32 CUDA-core convolution for every filter size / stride / padding Conv_Layer accepts
// (CNN/models/CNN_classes_cupy.py:70-154).  It serves the shapes the tensor-core kernels do not
// take: the first layers with 1 or 3 input channels (HBM-bound, a few FLOP per byte), strided
// convolutions, channel counts that are not a multiple of 4, and AETHER_MATH_FP32.
#include "common.cuh"
#include "tc_host.cuh"

namespace aether {

static constexpr int GEN_MAX_W_SMEM = 12 * 1024;  // floats of filter kept in shared memory (48 KB)

// ---------------------------------------------------------------------------------- forward
// One thread per output element, consecutive threads on consecutive output channels (coalesced
// filter reads and output writes); the filter sits in shared memory when it fits.
template <bool W_IN_SMEM>
__global__ void __launch_bounds__(256) gen_fwd_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                      const float* __restrict__ b, float* __restrict__ y, int S, int H,
                                                      int W, int Cin, int Cout, int fH, int fW, int sH, int sW, int pH,
                                                      int pW, int Ho, int Wo) {
    extern __shared__ float wsm[];
    const int wcount = fH * fW * Cin * Cout;
    if (W_IN_SMEM) {
        for (int i = threadIdx.x; i < wcount; i += blockDim.x) wsm[i] = w[i];
        __syncthreads();
    }
    const float* wp = W_IN_SMEM ? wsm : w;
    // rows of x are 16-byte aligned: four channels per load and four independent sums (a Dense layer is one long row)
    const bool vec = (Cin & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
    const long long total = 1LL * S * Ho * Wo * Cout;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const int d = (int)(idx % Cout);
        long long pix = idx / Cout;
        const int wo = (int)(pix % Wo);
        pix /= Wo;
        const int ho = (int)(pix % Ho);
        const int s = (int)(pix / Ho);
        float acc = b ? b[d] : 0.f;
        for (int i = 0; i < fH; ++i) {
            const int hi = ho * sH + i - pH;
            if (hi < 0 || hi >= H) continue;
            for (int j = 0; j < fW; ++j) {
                const int wi = wo * sW + j - pW;
                if (wi < 0 || wi >= W) continue;
                const float* xp = x + (((size_t)s * H + hi) * W + wi) * Cin;
                const float* wq = wp + ((size_t)(i * fW + j) * Cin) * Cout + d;
                if (vec) {
                    const float4* xp4 = reinterpret_cast<const float4*>(xp);
                    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll 4
                    for (int c4 = 0; c4 < (Cin >> 2); ++c4) {
                        const float4 v = xp4[c4];
                        const float* wr = wq + (size_t)(4 * c4) * Cout;
                        a0 = fmaf(v.x, wr[0], a0);
                        a1 = fmaf(v.y, wr[Cout], a1);
                        a2 = fmaf(v.z, wr[2 * Cout], a2);
                        a3 = fmaf(v.w, wr[3 * Cout], a3);
                    }
                    acc += (a0 + a1) + (a2 + a3);
                } else {
                    for (int c = 0; c < Cin; ++c) acc = fmaf(xp[c], wq[(size_t)c * Cout], acc);
                }
            }
        }
        y[idx] = acc;
    }
}

// Pointwise layers with very few outputs per pixel (a classifier head: Dense 1024 -> 10 is a 1x1 convolution with
// Cout = 10): with one thread per output element a batch of 512 rows is 5120 threads walking 1024 channels each.
// Here a warp takes a row: the lanes split the channels (float4 loads of x, the row is read once), keep Cout partial
// sums each and combine them with shuffles in a fixed order.
// The filter is kept transposed in shared memory, wT[d][Cin], so a lane's four channels of output d are one 16-byte
// shared-memory read (4 * Cout scalar global loads per four channels before).
__device__ __forceinline__ void head_load_filter_T(const float* __restrict__ w, float* wT, int Cin, int Cout) {
    for (int i = threadIdx.x; i < Cin * Cout; i += blockDim.x) {
        const int c = i / Cout, d = i - c * Cout;
        wT[d * Cin + c] = w[i];
    }
    __syncthreads();
}

template <int MAXD>
__global__ void __launch_bounds__(256) gen_fwd_pointwise_few_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                                    const float* __restrict__ b, float* __restrict__ y,
                                                                    long long rows, int Cin, int Cout) {
    extern __shared__ __align__(16) float head_wT[];
    head_load_filter_T(w, head_wT, Cin, Cout);
    const int lane = threadIdx.x & 31;
    const long long warp0 = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    const int C4 = Cin >> 2;
    for (long long row = warp0; row < rows; row += nwarps) {
        float acc[MAXD];
#pragma unroll
        for (int d = 0; d < MAXD; ++d) acc[d] = 0.f;
        const float4* xr = reinterpret_cast<const float4*>(x + (size_t)row * Cin);
        for (int c4 = lane; c4 < C4; c4 += 32) {
            const float4 v = xr[c4];
#pragma unroll
            for (int d = 0; d < MAXD; ++d) {
                if (d < Cout) {
                    const float4 k = *reinterpret_cast<const float4*>(head_wT + d * Cin + 4 * c4);
                    acc[d] = fmaf(v.x, k.x, fmaf(v.y, k.y, fmaf(v.z, k.z, fmaf(v.w, k.w, acc[d]))));
                }
            }
        }
#pragma unroll
        for (int d = 0; d < MAXD; ++d) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc[d] += __shfl_xor_sync(0xffffffffu, acc[d], o);
        }
        if (lane < Cout) {
            float r = 0.f;
#pragma unroll
            for (int d = 0; d < MAXD; ++d) r = (d == lane) ? acc[d] : r;
            y[(size_t)row * Cout + lane] = r + (b ? b[lane] : 0.f);
        }
    }
}

// ---------------------------------------------------------------------------------- dX (gather form)
// dx[s,h,w,c] = sum over taps (i,j) and d of dy[s,ho,wo,d] * w[i,j,c,d] with ho*sH + i - pH == h.
__global__ void __launch_bounds__(256) gen_dx_kernel(const float* __restrict__ dy, const float* __restrict__ w,
                                                     float* __restrict__ dx, int S, int H, int W, int Cin, int Cout,
                                                     int fH, int fW, int sH, int sW, int pH, int pW, int Ho, int Wo) {
    const long long total = 1LL * S * H * W * Cin;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(idx % Cin);
        long long pix = idx / Cin;
        const int wi = (int)(pix % W);
        pix /= W;
        const int hi = (int)(pix % H);
        const int s = (int)(pix / H);
        float acc = 0.f;
        for (int i = 0; i < fH; ++i) {
            const int hn = hi + pH - i;
            if (hn < 0 || hn % sH) continue;
            const int ho = hn / sH;
            if (ho >= Ho) continue;
            for (int j = 0; j < fW; ++j) {
                const int wn = wi + pW - j;
                if (wn < 0 || wn % sW) continue;
                const int wo = wn / sW;
                if (wo >= Wo) continue;
                const float* dyp = dy + (((size_t)s * Ho + ho) * Wo + wo) * Cout;
                const float* wq = w + ((size_t)(i * fW + j) * Cin + c) * Cout;
                for (int d = 0; d < Cout; ++d) acc = fmaf(dyp[d], wq[d], acc);
            }
        }
        dx[idx] = acc;
    }
}

// The same for layers with 1..4 input channels and a filter count that is a multiple of 4 (the first layer of a
// network): one thread per input pixel keeps all CIN sums, so every dy vector is loaded once as float4 and the
// filter reads are the same address for the whole warp.
template <int CIN>
__global__ void __launch_bounds__(256) gen_dx_fewc_kernel(const float* __restrict__ dy, const float* __restrict__ w,
                                                          float* __restrict__ dx, int S, int H, int W, int Cout, int fH,
                                                          int fW, int sH, int sW, int pH, int pW, int Ho, int Wo) {
    const long long total = 1LL * S * H * W;
    const int C4 = Cout >> 2;
    for (long long pix = blockIdx.x * (long long)blockDim.x + threadIdx.x; pix < total;
         pix += (long long)gridDim.x * blockDim.x) {
        const int wi = (int)(pix % W);
        const long long q = pix / W;
        const int hi = (int)(q % H);
        const int s = (int)(q / H);
        float acc[CIN];
#pragma unroll
        for (int c = 0; c < CIN; ++c) acc[c] = 0.f;
        for (int i = 0; i < fH; ++i) {
            const int hn = hi + pH - i;
            if (hn < 0 || hn % sH) continue;
            const int ho = hn / sH;
            if (ho >= Ho) continue;
            for (int j = 0; j < fW; ++j) {
                const int wn = wi + pW - j;
                if (wn < 0 || wn % sW) continue;
                const int wo = wn / sW;
                if (wo >= Wo) continue;
                const float4* dyp = reinterpret_cast<const float4*>(dy + (((size_t)s * Ho + ho) * Wo + wo) * Cout);
                const float4* wq = reinterpret_cast<const float4*>(w + (size_t)(i * fW + j) * CIN * Cout);
#pragma unroll 4
                for (int d = 0; d < C4; ++d) {
                    const float4 g = dyp[d];
#pragma unroll
                    for (int c = 0; c < CIN; ++c) {
                        const float4 k = __ldg(wq + c * C4 + d);
                        acc[c] = fmaf(g.x, k.x, fmaf(g.y, k.y, fmaf(g.z, k.z, fmaf(g.w, k.w, acc[c]))));
                    }
                }
            }
        }
#pragma unroll
        for (int c = 0; c < CIN; ++c) dx[pix * CIN + c] = acc[c];
    }
}

// ---------------------------------------------------------------------------------- dW, dB
// Block b owns a contiguous chunk of output pixels; thread t accumulates filter entries t, t+256, ...
// over that chunk and writes them to part[b][entry].  A second kernel adds the chunks in fixed order.
static constexpr int GEN_DW_CHUNK = 256;
__global__ void __launch_bounds__(256) gen_dw_partial_kernel(const float* __restrict__ x, const float* __restrict__ dy,
                                                             float* __restrict__ part, int S, int H, int W, int Cin,
                                                             int Cout, int fH, int fW, int sH, int sW, int pH, int pW,
                                                             int Ho, int Wo, long long pix_per_block) {
    const long long npix = 1LL * S * Ho * Wo;
    const long long p0 = blockIdx.x * pix_per_block;
    long long p1 = p0 + pix_per_block;
    if (p1 > npix) p1 = npix;
    const int entries = fH * fW * Cin * Cout;
    // Pixel coordinates are decoded once per chunk of GEN_DW_CHUNK pixels into shared memory
    // (sample row base s*H, top-left input row, top-left input column), not once per (entry, pixel).
    __shared__ int pix_s[GEN_DW_CHUNK], pix_h[GEN_DW_CHUNK], pix_w[GEN_DW_CHUNK];
    // blockIdx.y walks the filter entries in groups of 256: every (pixel chunk, entry group) pair is a CTA of its own,
    // so the dependent load chains of the inner loop are hidden by occupancy instead of running one after another.
    for (int e0 = blockIdx.y * blockDim.x; e0 < entries + Cout; e0 += gridDim.y * blockDim.x) {
        const int e = e0 + threadIdx.x;
        const bool is_w = e < entries && x != nullptr;
        const bool is_b = e >= entries && e < entries + Cout;
        const int d = is_b ? e - entries : e % Cout;
        const int c = (e / Cout) % Cin;
        const int tap = e / (Cout * Cin);
        const int i = tap / fW, j = tap % fW;
        float acc = 0.f;
        for (long long c0 = p0; c0 < p1; c0 += GEN_DW_CHUNK) {
            const int n = (int)((p1 - c0 < GEN_DW_CHUNK) ? (p1 - c0) : GEN_DW_CHUNK);
            __syncthreads();
            for (int q = threadIdx.x; q < n; q += blockDim.x) {
                const long long p = c0 + q;
                const int wo = (int)(p % Wo);
                const long long r = p / Wo;
                pix_w[q] = wo * sW - pW;
                pix_h[q] = (int)(r % Ho) * sH - pH;
                pix_s[q] = (int)(r / Ho) * H;
            }
            __syncthreads();
            if (is_w) {
                for (int q = 0; q < n; ++q) {
                    const int hi = pix_h[q] + i, wi = pix_w[q] + j;
                    if (hi < 0 || hi >= H || wi < 0 || wi >= W) continue;
                    acc = fmaf(x[((size_t)(pix_s[q] + hi) * W + wi) * Cin + c], dy[(size_t)(c0 + q) * Cout + d], acc);
                }
            } else if (is_b) {                     // trailing Cout entries: dB
                for (int q = 0; q < n; ++q) acc += dy[(size_t)(c0 + q) * Cout + d];
            }
        }
        if (e < entries + Cout) part[(size_t)blockIdx.x * (entries + Cout) + e] = acc;
    }
}

__global__ void gen_dw_reduce_kernel(const float* __restrict__ part, int nblocks, int entries, int Cout,
                                     float* __restrict__ dw, float* __restrict__ db) {
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= entries + Cout) return;
    float s = 0.f;
    for (int b = 0; b < nblocks; ++b) s += part[(size_t)b * (entries + Cout) + e];
    if (e < entries) {
        if (dw) dw[e] = s;
    } else if (db) {
        db[e - entries] = s;
    }
}

// ---------------------------------------------------------------------------------- classifier heads, backward
// dx[p][c] = sum_d dy[p][d] * w[c][d] for a pointwise layer with few outputs: a block takes a row at a time, a thread
// four channels; the filter is read transposed from shared memory, the row of dy is the same address for every thread.
template <int MAXD>
__global__ void __launch_bounds__(256) head_dx_kernel(const float* __restrict__ dy, const float* __restrict__ w,
                                                      float* __restrict__ dx, long long rows, int Cin, int Cout) {
    extern __shared__ __align__(16) float head_wT[];
    head_load_filter_T(w, head_wT, Cin, Cout);
    const int C4 = Cin >> 2;
    float gn[MAXD];                                     // the next row's dy values, requested one row ahead
#pragma unroll
    for (int d = 0; d < MAXD; ++d) gn[d] = (d < Cout && blockIdx.x < rows) ? __ldg(dy + (size_t)blockIdx.x * Cout + d) : 0.f;
    for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
        float g[MAXD];
        const long long nrow = row + gridDim.x;
#pragma unroll
        for (int d = 0; d < MAXD; ++d) {
            g[d] = gn[d];
            gn[d] = (d < Cout && nrow < rows) ? __ldg(dy + (size_t)nrow * Cout + d) : 0.f;
        }
        float4* out = reinterpret_cast<float4*>(dx + (size_t)row * Cin);
        for (int c4 = threadIdx.x; c4 < C4; c4 += blockDim.x) {
            float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int d = 0; d < MAXD; ++d) {
                if (d < Cout) {
                    const float4 k = *reinterpret_cast<const float4*>(head_wT + d * Cin + 4 * c4);
                    a.x = fmaf(g[d], k.x, a.x); a.y = fmaf(g[d], k.y, a.y); a.z = fmaf(g[d], k.z, a.z); a.w = fmaf(g[d], k.w, a.w);
                }
            }
            out[c4] = a;
        }
    }
}

// dw[c][d] = sum_p x[p][c] * dy[p][d], db[d] = sum_p dy[p][d] over this block's rows, written as the partials
// gen_dw_reduce_kernel adds up ([block][Cin * Cout + Cout]).  A thread keeps four channels x Cout sums; x is read once,
// coalesced; the row of dy is the same address for every thread.  blockIdx.y walks the channels in groups of 1024.
template <int MAXD>
__global__ void __launch_bounds__(256) head_dw_partial_kernel(const float* __restrict__ x, const float* __restrict__ dy,
                                                              float* __restrict__ part, long long rows, int Cin, int Cout,
                                                              long long rows_per_block) {
    const long long r0 = blockIdx.x * rows_per_block;
    long long r1 = r0 + rows_per_block;
    if (r1 > rows) r1 = rows;
    const int C4 = Cin >> 2;
    const int c4 = blockIdx.y * blockDim.x + threadIdx.x;
    const int entries = Cin * Cout;
    float* out = part + (size_t)blockIdx.x * (entries + Cout);
    if (c4 < C4) {
        float4 acc[MAXD];
#pragma unroll
        for (int d = 0; d < MAXD; ++d) acc[d] = make_float4(0.f, 0.f, 0.f, 0.f);
        const float4* xp = reinterpret_cast<const float4*>(x) + c4;
#pragma unroll 2
        for (long long r = r0; r < r1; ++r) {
            const float4 v = xp[(size_t)r * C4];
            const float* gr = dy + (size_t)r * Cout;
#pragma unroll
            for (int d = 0; d < MAXD; ++d) {
                if (d < Cout) {
                    const float g = __ldg(gr + d);
                    acc[d].x = fmaf(v.x, g, acc[d].x); acc[d].y = fmaf(v.y, g, acc[d].y);
                    acc[d].z = fmaf(v.z, g, acc[d].z); acc[d].w = fmaf(v.w, g, acc[d].w);
                }
            }
        }
#pragma unroll
        for (int d = 0; d < MAXD; ++d) {
            if (d < Cout) {
                out[(size_t)(4 * c4 + 0) * Cout + d] = acc[d].x; out[(size_t)(4 * c4 + 1) * Cout + d] = acc[d].y;
                out[(size_t)(4 * c4 + 2) * Cout + d] = acc[d].z; out[(size_t)(4 * c4 + 3) * Cout + d] = acc[d].w;
            }
        }
    }
    if (blockIdx.y == 0 && (int)threadIdx.x < Cout) {
        float sdy = 0.f;
        for (long long r = r0; r < r1; ++r) sdy += dy[(size_t)r * Cout + threadIdx.x];
        out[entries + threadIdx.x] = sdy;
    }
}

// Pointwise layer with at most 16 outputs whose transposed filter fits in shared memory (a classifier head).
static bool head_shape(const AetherConvDesc& d) {
    return d.fH == 1 && d.fW == 1 && d.sH == 1 && d.sW == 1 && d.padH == 0 && d.padW == 0 && d.Cout <= 16 && d.Cin >= 128 &&
           (d.Cin & 3) == 0 && (size_t)d.Cin * d.Cout * sizeof(float) <= 96 * 1024;
}

// ---------------------------------------------------------------------------------- host
static int gen_blocks(long long total, int threads) {
    long long b = (total + threads - 1) / threads;
    const long long cap = 148LL * 16;
    if (b > cap) b = cap;
    if (b < 1) b = 1;
    return (int)b;
}

int generic_conv_fwd(const AetherConvDesc& d, const float* x, const float* w, const float* b, float* y, cudaStream_t st) {
    int Ho, Wo;
    conv_out_hw(d, Ho, Wo);
    const long long total = 1LL * d.S * Ho * Wo * d.Cout;
    const int wcount = d.fH * d.fW * d.Cin * d.Cout;
    if (head_shape(d) && (reinterpret_cast<uintptr_t>(x) & 15u) == 0) {
        const long long rows = 1LL * d.S * d.H * d.W;
        const int smem = d.Cin * d.Cout * (int)sizeof(float);
        static PerDeviceSmem configured;
        if (int rc = ensure_dynamic_smem(gen_fwd_pointwise_few_kernel<16>, 96 * 1024, configured, "head forward")) return rc;
        long long nb = (rows + 7) / 8;                        // a warp per row, 8 rows per block and pass
        if (nb > 2LL * num_sms()) nb = 2LL * num_sms();       // every block loads the filter once
        gen_fwd_pointwise_few_kernel<16><<<(int)nb, 256, smem, st>>>(x, w, b, y, rows, d.Cin, d.Cout);
        count_launch();
        return check_launch("gen_fwd_pointwise_few_kernel");
    }
    if (wcount <= GEN_MAX_W_SMEM) {
        gen_fwd_kernel<true><<<gen_blocks(total, 256), 256, wcount * sizeof(float), st>>>(
            x, w, b, y, d.S, d.H, d.W, d.Cin, d.Cout, d.fH, d.fW, d.sH, d.sW, d.padH, d.padW, Ho, Wo);
    } else {
        gen_fwd_kernel<false><<<gen_blocks(total, 256), 256, 0, st>>>(x, w, b, y, d.S, d.H, d.W, d.Cin, d.Cout, d.fH,
                                                                      d.fW, d.sH, d.sW, d.padH, d.padW, Ho, Wo);
    }
    count_launch();
    return check_launch("gen_fwd_kernel");
}

int generic_conv_bwd_data(const AetherConvDesc& d, const float* dy, const float* w, float* dx, cudaStream_t st) {
    int Ho, Wo;
    conv_out_hw(d, Ho, Wo);
    const long long total = 1LL * d.S * d.H * d.W * d.Cin;
    if (d.Cin <= 4 && d.Cout % 4 == 0 && (reinterpret_cast<uintptr_t>(dy) & 15u) == 0 && (reinterpret_cast<uintptr_t>(w) & 15u) == 0) {
        const int nb = gen_blocks(1LL * d.S * d.H * d.W, 256);
#define AETHER_DX_FEWC(CIN)                                                                                          \
    gen_dx_fewc_kernel<CIN><<<nb, 256, 0, st>>>(dy, w, dx, d.S, d.H, d.W, d.Cout, d.fH, d.fW, d.sH, d.sW, d.padH, d.padW, \
                                               Ho, Wo)
        switch (d.Cin) {
            case 1: AETHER_DX_FEWC(1); break;
            case 2: AETHER_DX_FEWC(2); break;
            case 3: AETHER_DX_FEWC(3); break;
            default: AETHER_DX_FEWC(4); break;
        }
#undef AETHER_DX_FEWC
        count_launch();
        return check_launch("gen_dx_fewc_kernel");
    }
    if (head_shape(d) && (reinterpret_cast<uintptr_t>(dx) & 15u) == 0) {
        const long long rows = 1LL * d.S * d.H * d.W;
        const int smem = d.Cin * d.Cout * (int)sizeof(float);
        static PerDeviceSmem configured;
        if (int rc = ensure_dynamic_smem(head_dx_kernel<16>, 96 * 1024, configured, "head dX")) return rc;
        long long nb = rows < 2LL * num_sms() ? rows : 2LL * num_sms();
        head_dx_kernel<16><<<(int)nb, 256, smem, st>>>(dy, w, dx, rows, d.Cin, d.Cout);
        count_launch();
        return check_launch("head_dx_kernel");
    }
    gen_dx_kernel<<<gen_blocks(total, 256), 256, 0, st>>>(dy, w, dx, d.S, d.H, d.W, d.Cin, d.Cout, d.fH, d.fW, d.sH,
                                                          d.sW, d.padH, d.padW, Ho, Wo);
    count_launch();
    return check_launch("gen_dx_kernel");
}

static int gen_dw_blocks(const AetherConvDesc& d) {
    int Ho, Wo;
    conv_out_hw(d, Ho, Wo);
    const long long npix = 1LL * d.S * Ho * Wo;
    long long nb = npix / 32;
    if (nb > 148LL * 4) nb = 148LL * 4;
    if (nb < 1) nb = 1;
    return (int)nb;
}

size_t generic_conv_workspace_bytes(const AetherConvDesc& d) {
    const size_t entries = (size_t)d.fH * d.fW * d.Cin * d.Cout + d.Cout;
    return align_up((size_t)gen_dw_blocks(d) * entries * sizeof(float), 1024);
}

int generic_conv_bwd_filter(const AetherConvDesc& d, const float* x, const float* dy, float* dw, float* db, void* ws,
                            size_t ws_bytes, cudaStream_t st) {
    int Ho, Wo;
    conv_out_hw(d, Ho, Wo);
    if (!ws || ws_bytes < generic_conv_workspace_bytes(d))
        return set_error(AE_BAD_ARG, "conv workspace too small: %zu < %zu", ws_bytes, generic_conv_workspace_bytes(d));
    const int nb = gen_dw_blocks(d);
    const long long npix = 1LL * d.S * Ho * Wo;
    const long long ppb = (npix + nb - 1) / nb;
    const int entries = d.fH * d.fW * d.Cin * d.Cout;
    float* part = static_cast<float*>(ws);
    if (head_shape(d) && x != nullptr && (reinterpret_cast<uintptr_t>(x) & 15u) == 0) {
        head_dw_partial_kernel<16><<<dim3(nb, ceil_div(d.Cin / 4, 256)), 256, 0, st>>>(x, dy, part, npix, d.Cin, d.Cout, ppb);
        count_launch();
        int rc = check_launch("head_dw_partial_kernel");
        if (rc) return rc;
        gen_dw_reduce_kernel<<<ceil_div(entries + d.Cout, 256), 256, 0, st>>>(part, nb, entries, d.Cout, dw, db);
        count_launch();
        return check_launch("gen_dw_reduce_kernel");
    }
    int egroups = ceil_div(entries + d.Cout, 256);
    if (egroups > 4096) egroups = 4096;
    gen_dw_partial_kernel<<<dim3(nb, egroups), 256, 0, st>>>(x, dy, part, d.S, d.H, d.W, d.Cin, d.Cout, d.fH, d.fW, d.sH, d.sW, d.padH,
                                              d.padW, Ho, Wo, ppb);
    count_launch();
    int rc = check_launch("gen_dw_partial_kernel");
    if (rc) return rc;
    gen_dw_reduce_kernel<<<ceil_div(entries + d.Cout, 256), 256, 0, st>>>(part, nb, entries, d.Cout, dw, db);
    count_launch();
    return check_launch("gen_dw_reduce_kernel");
}

}  // namespace aether
