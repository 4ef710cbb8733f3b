// Bandwidth-bound layers that sit next to the convolution in Aether-ML's networks
// (CNN/models/CNN_classes_cupy.py): Batch_Norm :430-526, Pooling :204-312, ReLU :406-415,
// Leaky_ReLU :417-428, Layer_Dropout_Spatial :384-404, Layer_Dropout :364-382, Optimizer_Adam
// :685-736, SoftMax + categorical cross-entropy :541-680.  All arrays are fp32 with the channel
// (last) axis contiguous; kernels use 128-bit accesses along it whenever the channel count allows.
#include <math.h>

#include "common.cuh"

namespace aether {

static int blocks_for(long long items, int threads, int per_sm = 8) {
    long long b = (items + threads - 1) / threads;
    const long long cap = 148LL * per_sm;
    if (b > cap) b = cap;
    if (b < 1) b = 1;
    return (int)b;
}

// Derivative of the (leaky) ReLU fused behind a Batch_Norm at pre-activation v = gamma * xhat + beta, which the
// backward kernels recompute from x: alpha where v < 0, else 1 -- the gradient passes at v == 0 exactly as in the
// reference (CNN_classes_cupy.py:412-428).
__device__ __forceinline__ float act_grad(float v, float alpha) { return v < 0.f ? alpha : 1.f; }

// ====================================================================================== batch norm
// Per-channel reductions over a [rows][C] matrix.  Thread t of a block owns column (t % cols) and row
// lane (t / cols); a block walks a contiguous slab of rows, so a warp reads consecutive addresses.
// MODE 0: partial (count, mean, M2) of x         -> part[block][3][C]
// MODE 1: partial sum(dy), sum(dy * xhat)        -> part[block][2][C]   (xhat from mean/inv_std)
template <int MODE>
__global__ void __launch_bounds__(256) bn_reduce_kernel(const float* __restrict__ x, const float* __restrict__ dy,
                                                        const float* __restrict__ mean, const float* __restrict__ var,
                                                        float eps, long long rows, int C, float* __restrict__ part,
                                                        long long rows_per_block, const float* __restrict__ act_gamma,
                                                        const float* __restrict__ act_beta, float alpha) {
    const long long r0 = blockIdx.x * rows_per_block;
    long long r1 = r0 + rows_per_block;
    if (r1 > rows) r1 = rows;
    const int cols = C < 256 ? C : 256;
    const int lanes = 256 / cols;
    __shared__ float sh_a[256], sh_b[256], sh_n[256];
    constexpr int NOUT = MODE == 0 ? 3 : 2;
    for (int cbase = 0; cbase < C; cbase += cols) {
        const int c = cbase + threadIdx.x % cols;
        const int rl = threadIdx.x / cols;
        float a = 0.f, b = 0.f, n = 0.f;
        if (rl < lanes && c < C) {
            if (MODE == 0) {
                // shifted sums: subtract the first element of the slab to avoid cancellation
                const float shift = (r0 < r1) ? x[(size_t)r0 * C + c] : 0.f;
                for (long long r = r0 + rl; r < r1; r += lanes) {
                    const float v = x[(size_t)r * C + c] - shift;
                    a += v;
                    b = fmaf(v, v, b);
                    n += 1.f;
                }
                // convert to (n, mean, M2) about the true local mean
                if (n > 0.f) {
                    const float m = a / n;
                    b = b - a * m;
                    a = m + shift;
                }
            } else {
                const float mu = mean[c];
                const float inv = rsqrtf(var[c] + eps);
                const float ag = act_gamma ? act_gamma[c] : 0.f, ab = act_gamma ? act_beta[c] : 0.f;
                for (long long r = r0 + rl; r < r1; r += lanes) {
                    float g = dy[(size_t)r * C + c];
                    const float xh = (x[(size_t)r * C + c] - mu) * inv;
                    if (act_gamma) g *= act_grad(fmaf(ag, xh, ab), alpha);     // gradient through the fused activation
                    a += g;
                    b = fmaf(g, xh, b);
                }
            }
        }
        sh_a[threadIdx.x] = a;
        sh_b[threadIdx.x] = b;
        sh_n[threadIdx.x] = n;
        __syncthreads();
        if (threadIdx.x < cols && c < C) {
            float* out = part + (size_t)blockIdx.x * NOUT * C;
            if (MODE == 0) {
                // Chan's parallel merge of the row lanes, in fixed order
                float N = 0.f, M = 0.f, M2 = 0.f;
                for (int l = 0; l < lanes; ++l) {
                    const float nl = sh_n[l * cols + threadIdx.x];
                    if (nl == 0.f) continue;
                    const float ml = sh_a[l * cols + threadIdx.x], m2l = sh_b[l * cols + threadIdx.x];
                    const float tot = N + nl;
                    const float delta = ml - M;
                    M2 += m2l + delta * delta * N * nl / tot;
                    M += delta * nl / tot;
                    N = tot;
                }
                out[c] = N;
                out[C + c] = M;
                out[2 * C + c] = M2;
            } else {
                float sa = 0.f, sb = 0.f;
                for (int l = 0; l < lanes; ++l) {
                    sa += sh_a[l * cols + threadIdx.x];
                    sb += sh_b[l * cols + threadIdx.x];
                }
                out[c] = sa;
                out[C + c] = sb;
            }
        }
        __syncthreads();
    }
}

// The same reductions with four consecutive channels per thread (C % 4 == 0, 16-byte aligned rows):
// float4 loads keep four times the bytes in flight per thread, which is what the HBM latency needs.
template <int MODE>
__global__ void __launch_bounds__(256) bn_reduce_vec4_kernel(const float* __restrict__ x, const float* __restrict__ dy,
                                                             const float* __restrict__ mean, const float* __restrict__ var,
                                                             float eps, long long rows, int C, float* __restrict__ part,
                                                             long long rows_per_block, const float* __restrict__ act_gamma,
                                                             const float* __restrict__ act_beta, float alpha) {
    const long long r0 = blockIdx.x * rows_per_block;
    long long r1 = r0 + rows_per_block;
    if (r1 > rows) r1 = rows;
    const int CV = C >> 2;
    const int cols = CV < 256 ? CV : 256;
    const int lanes = 256 / cols;
    __shared__ float4 sh_a4[256], sh_b4[256];
    __shared__ float sh_n[256];
    constexpr int NOUT = MODE == 0 ? 3 : 2;
    for (int cbase = 0; cbase < CV; cbase += cols) {
        const int cv = cbase + threadIdx.x % cols;
        const int rl = threadIdx.x / cols;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
        float n = 0.f;
        if (rl < lanes && cv < CV) {
            const float4* xr = reinterpret_cast<const float4*>(x) + cv;          // row r is xr[r * CV]
            if (MODE == 0) {
                const float4 sh = (r0 < r1) ? xr[(size_t)r0 * CV] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
                for (long long r = r0 + rl; r < r1; r += lanes) {
                    float4 v = xr[(size_t)r * CV];
                    v.x -= sh.x; v.y -= sh.y; v.z -= sh.z; v.w -= sh.w;
                    a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
                    b.x = fmaf(v.x, v.x, b.x); b.y = fmaf(v.y, v.y, b.y);
                    b.z = fmaf(v.z, v.z, b.z); b.w = fmaf(v.w, v.w, b.w);
                    n += 1.f;
                }
                if (n > 0.f) {
                    float m;
                    m = a.x / n; b.x -= a.x * m; a.x = m + sh.x;
                    m = a.y / n; b.y -= a.y * m; a.y = m + sh.y;
                    m = a.z / n; b.z -= a.z * m; a.z = m + sh.z;
                    m = a.w / n; b.w -= a.w * m; a.w = m + sh.w;
                }
            } else {
                const int c = cv * 4;
                const float4 mu = make_float4(mean[c], mean[c + 1], mean[c + 2], mean[c + 3]);
                const float4 inv = make_float4(rsqrtf(var[c] + eps), rsqrtf(var[c + 1] + eps), rsqrtf(var[c + 2] + eps),
                                               rsqrtf(var[c + 3] + eps));
                const float4* gr = reinterpret_cast<const float4*>(dy) + cv;
                const float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f);
                const float4 ag = act_gamma ? *reinterpret_cast<const float4*>(act_gamma + c) : z4;
                const float4 ab = act_gamma ? *reinterpret_cast<const float4*>(act_beta + c) : z4;
#pragma unroll 4
                for (long long r = r0 + rl; r < r1; r += lanes) {
                    float4 g = gr[(size_t)r * CV];
                    const float4 v = xr[(size_t)r * CV];
                    const float4 xh = make_float4((v.x - mu.x) * inv.x, (v.y - mu.y) * inv.y, (v.z - mu.z) * inv.z,
                                                  (v.w - mu.w) * inv.w);
                    if (act_gamma) {                                              // gradient through the fused activation
                        g.x *= act_grad(fmaf(ag.x, xh.x, ab.x), alpha); g.y *= act_grad(fmaf(ag.y, xh.y, ab.y), alpha);
                        g.z *= act_grad(fmaf(ag.z, xh.z, ab.z), alpha); g.w *= act_grad(fmaf(ag.w, xh.w, ab.w), alpha);
                    }
                    a.x += g.x; a.y += g.y; a.z += g.z; a.w += g.w;
                    b.x = fmaf(g.x, xh.x, b.x); b.y = fmaf(g.y, xh.y, b.y);
                    b.z = fmaf(g.z, xh.z, b.z); b.w = fmaf(g.w, xh.w, b.w);
                }
            }
        }
        sh_a4[threadIdx.x] = a;
        sh_b4[threadIdx.x] = b;
        sh_n[threadIdx.x] = n;
        __syncthreads();
        if (threadIdx.x < cols && cv < CV) {
            float* out = part + (size_t)blockIdx.x * NOUT * C + cv * 4;
            const float* pa = reinterpret_cast<const float*>(sh_a4);
            const float* pb = reinterpret_cast<const float*>(sh_b4);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                if (MODE == 0) {
                    float N = 0.f, M = 0.f, M2 = 0.f;          // Chan's merge of the row lanes, in fixed order
                    for (int l = 0; l < lanes; ++l) {
                        const int t = l * cols + threadIdx.x;
                        const float nl = sh_n[t];
                        if (nl == 0.f) continue;
                        const float tot = N + nl;
                        const float delta = pa[t * 4 + k] - M;
                        M2 += pb[t * 4 + k] + delta * delta * N * nl / tot;
                        M += delta * nl / tot;
                        N = tot;
                    }
                    out[k] = N;
                    out[C + k] = M;
                    out[2 * C + k] = M2;
                } else {
                    float sa = 0.f, sb = 0.f;
                    for (int l = 0; l < lanes; ++l) {
                        sa += pa[(l * cols + threadIdx.x) * 4 + k];
                        sb += pb[(l * cols + threadIdx.x) * 4 + k];
                    }
                    out[k] = sa;
                    out[C + k] = sb;
                }
            }
        }
        __syncthreads();
    }
}

template <int MODE>
static void launch_bn_reduce(int nb, cudaStream_t st, const float* x, const float* dy, const float* mean, const float* var,
                             float eps, long long rows, int C, float* part, const float* act_gamma = nullptr,
                             const float* act_beta = nullptr, float alpha = 0.f) {
    const long long rpb = (rows + nb - 1) / nb;
    const bool vec = (C & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0 &&
                     (MODE == 0 || (reinterpret_cast<uintptr_t>(dy) & 15u) == 0) &&
                     (act_gamma == nullptr || ((reinterpret_cast<uintptr_t>(act_gamma) | reinterpret_cast<uintptr_t>(act_beta)) & 15u) == 0);
    if (vec) bn_reduce_vec4_kernel<MODE><<<nb, 256, 0, st>>>(x, dy, mean, var, eps, rows, C, part, rpb, act_gamma, act_beta, alpha);
    else bn_reduce_kernel<MODE><<<nb, 256, 0, st>>>(x, dy, mean, var, eps, rows, C, part, rpb, act_gamma, act_beta, alpha);
}

// Merges the per-block (n, mean, M2) triples in double precision, writes batch mean / biased variance,
// updates the running statistics (momentum * old + (1 - momentum) * batch) and the affine
// coefficients scale = gamma / sqrt(var + eps), shift = beta - mean * scale used by the apply kernel.
// Finalize kernels: FIN_CH channels x FIN_LANES lanes per CTA.  The merge is a chain of L2 round trips per lane, so
// it is spread over many lanes (a few blocks each); a network with 32 channels still gets 4 CTAs.
static constexpr int FIN_CH = 8, FIN_LANES = 64, FIN_THREADS = FIN_CH * FIN_LANES;

__global__ void __launch_bounds__(FIN_THREADS) bn_finalize_fwd_kernel(const float* __restrict__ part, int nblocks, int C,
                                       const float* __restrict__ gamma, const float* __restrict__ beta, float eps,
                                       float momentum, float* __restrict__ running_mean,
                                       float* __restrict__ running_var, float* __restrict__ batch_mean,
                                       float* __restrict__ batch_var, float* __restrict__ scale_shift) {
    // One pass over the per-block triples, all in double: N = sum n, S = sum n * mean, Q = sum (M2 + n * mean^2); then
    // M2 = Q - N * M^2.  The subtraction loses log2(mean^2 / var) of double's 53 bits, harmless for any ratio a float
    // tensor can show (the per-block M2 themselves carry 24 bits).  Lanes are combined in fixed order.
    __shared__ double red_a[FIN_LANES][FIN_CH], red_b[FIN_LANES][FIN_CH], red_c[FIN_LANES][FIN_CH];
    const int cl = threadIdx.x % FIN_CH, ln = threadIdx.x / FIN_CH;
    const int c = blockIdx.x * FIN_CH + cl;
    double n_sum = 0.0, s_sum = 0.0, q_sum = 0.0;
    if (c < C)
#pragma unroll 4
        for (int b = ln; b < nblocks; b += FIN_LANES) {
            const float* p = part + (size_t)b * 3 * C;
            const double nl = p[c], ml = p[C + c];
            n_sum += nl;
            s_sum += nl * ml;
            q_sum += (double)p[2 * C + c] + nl * ml * ml;
        }
    red_a[ln][cl] = n_sum;
    red_b[ln][cl] = s_sum;
    red_c[ln][cl] = q_sum;
    __syncthreads();
    if (ln != 0 || c >= C) return;
    double N = 0.0, S1 = 0.0, Q = 0.0;
#pragma unroll 8
    for (int l = 0; l < FIN_LANES; ++l) { N += red_a[l][cl]; S1 += red_b[l][cl]; Q += red_c[l][cl]; }
    const double M = N > 0 ? S1 / N : 0.0;
    double M2 = Q - N * M * M;
    if (M2 < 0.0) M2 = 0.0;
    const double var = N > 0 ? M2 / N : 0.0;
    batch_mean[c] = (float)M;
    batch_var[c] = (float)var;
    running_mean[c] = momentum * running_mean[c] + (1.f - momentum) * (float)M;
    running_var[c] = momentum * running_var[c] + (1.f - momentum) * (float)var;
    const double sc = (double)gamma[c] / sqrt(var + (double)eps);
    scale_shift[c] = (float)sc;
    scale_shift[C + c] = (float)((double)beta[c] - M * sc);
}

__global__ void bn_eval_coeff_kernel(int C, const float* __restrict__ gamma, const float* __restrict__ beta, float eps,
                                     const float* __restrict__ running_mean, const float* __restrict__ running_var,
                                     float* __restrict__ scale_shift) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const float sc = gamma[c] / sqrtf(running_var[c] + eps);
    scale_shift[c] = sc;
    scale_shift[C + c] = beta[c] - running_mean[c] * sc;
}

// y = x * scale[c] + shift[c], optionally followed by y = y > 0 ? y : act_alpha * y (act_alpha < 0: no activation)
__global__ void __launch_bounds__(256) affine_channels_kernel(const float* __restrict__ x, float* __restrict__ y,
                                                              const float* __restrict__ scale,
                                                              const float* __restrict__ shift, long long n, int C,
                                                              float act_alpha) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    const bool act = act_alpha >= 0.f;
    if ((C & 3) == 0) {
        const long long n4 = n >> 2;
        const int C4 = C >> 2;
        const float4* x4 = reinterpret_cast<const float4*>(x);
        float4* y4 = reinterpret_cast<float4*>(y);
        const long long i0 = blockIdx.x * (long long)blockDim.x + threadIdx.x;
        const int cstep = (int)(stride % C4);          // the channel group advances by this much per iteration
        int cq = (int)(i0 % C4);
        for (long long i = i0; i < n4; i += stride) {
            const int c = cq * 4;
            cq += cstep;
            if (cq >= C4) cq -= C4;
            const float4 v = x4[i];
            const float4 s = *reinterpret_cast<const float4*>(scale + c);
            float4 o;
            if (shift) {
                const float4 t = *reinterpret_cast<const float4*>(shift + c);
                o = make_float4(fmaf(v.x, s.x, t.x), fmaf(v.y, s.y, t.y), fmaf(v.z, s.z, t.z), fmaf(v.w, s.w, t.w));
            } else {
                o = make_float4(v.x * s.x, v.y * s.y, v.z * s.z, v.w * s.w);
            }
            if (act) {
                o.x = o.x > 0.f ? o.x : act_alpha * o.x; o.y = o.y > 0.f ? o.y : act_alpha * o.y;
                o.z = o.z > 0.f ? o.z : act_alpha * o.z; o.w = o.w > 0.f ? o.w : act_alpha * o.w;
            }
            y4[i] = o;
        }
    } else {
        for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += stride) {
            const int c = (int)(i % C);
            const float o = shift ? fmaf(x[i], scale[c], shift[c]) : x[i] * scale[c];
            y[i] = (act && o <= 0.f) ? act_alpha * o : o;
        }
    }
}

// dgamma = sum(dy * xhat), dbeta = sum(dy); coefficients for
// dx = k1[c] * dy + k2[c] * x + k3[c]  with  k1 = gamma*inv, k2 = -gamma*inv^2*dgamma/N * ... (see below)
__global__ void __launch_bounds__(FIN_THREADS) bn_finalize_bwd_kernel(const float* __restrict__ part, int nblocks, int C, long long rows,
                                       const float* __restrict__ gamma, const float* __restrict__ mean,
                                       const float* __restrict__ var, float eps, float* __restrict__ dgamma,
                                       float* __restrict__ dbeta, float* __restrict__ coeff,
                                       const float* __restrict__ pscale) {
    // pscale (nullable): per-channel factor that multiplied the layer's output (a fused spatial-dropout mask).  The
    // upstream gradient is that factor times what the kernels summed, so it scales both sums and the dy coefficient.
    __shared__ double red_a[FIN_LANES][FIN_CH], red_b[FIN_LANES][FIN_CH];
    const int cl = threadIdx.x % FIN_CH, ln = threadIdx.x / FIN_CH;
    const int c = blockIdx.x * FIN_CH + cl;
    double pa = 0.0, pb = 0.0;
    if (c < C)
#pragma unroll 4
        for (int b = ln; b < nblocks; b += FIN_LANES) {
            pa += part[(size_t)b * 2 * C + c];
            pb += part[(size_t)b * 2 * C + C + c];
        }
    red_a[ln][cl] = pa;
    red_b[ln][cl] = pb;
    __syncthreads();
    if (ln != 0 || c >= C) return;
    double sdy = 0.0, sdyx = 0.0;
#pragma unroll 8
    for (int l = 0; l < FIN_LANES; ++l) { sdy += red_a[l][cl]; sdyx += red_b[l][cl]; }
    const double ms = pscale ? (double)pscale[c] : 1.0;
    sdy *= ms;
    sdyx *= ms;
    dgamma[c] = (float)sdyx;
    dbeta[c] = (float)sdy;
    // dx = gamma*inv/N * (N*dy - sum(dy) - xhat * sum(dy*xhat)),  xhat = (x - mean) * inv
    //    = k1*dy + k2*x + k3
    const double inv = 1.0 / sqrt((double)var[c] + (double)eps);
    const double g = gamma[c], N = (double)rows, mu = mean[c];
    const double k1 = g * inv * ms;
    const double k2 = -g * inv * inv * sdyx / N;
    const double k3 = -g * inv * sdy / N - k2 * mu;
    coeff[c] = (float)k1;
    coeff[C + c] = (float)k2;
    coeff[2 * C + c] = (float)k3;
}

// act_gamma / act_beta (nullable): a fused activation's derivative is applied to dy first, taken at the pre-activation
// v = gamma * ((x - mean) * rsqrt(var + eps)) + beta -- the same expression, operation for operation, as in the
// reduction kernels above, so both passes judge every element alike.
__global__ void __launch_bounds__(256) bn_bwd_apply_kernel(const float* __restrict__ x, const float* __restrict__ dy,
                                                           float* __restrict__ dx, const float* __restrict__ coeff,
                                                           long long n, int C, const float* __restrict__ act_gamma,
                                                           const float* __restrict__ act_beta,
                                                           const float* __restrict__ mean, const float* __restrict__ var,
                                                           float eps, float alpha) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    if ((C & 3) == 0) {
        const long long n4 = n >> 2;
        const int C4 = C >> 2;
        const long long i0 = blockIdx.x * (long long)blockDim.x + threadIdx.x;
        const int cstep = (int)(stride % C4);
        int cq = (int)(i0 % C4);
        for (long long i = i0; i < n4; i += stride) {
            const int c = cq * 4;
            cq += cstep;
            if (cq >= C4) cq -= C4;
            const float4 xv = reinterpret_cast<const float4*>(x)[i];
            float4 g = reinterpret_cast<const float4*>(dy)[i];
            if (act_gamma) {                                                      // gradient through the fused activation
                const float4 ag = *reinterpret_cast<const float4*>(act_gamma + c);
                const float4 ab = *reinterpret_cast<const float4*>(act_beta + c);
                const float4 mu = *reinterpret_cast<const float4*>(mean + c);
                const float4 vr = *reinterpret_cast<const float4*>(var + c);
                g.x *= act_grad(fmaf(ag.x, (xv.x - mu.x) * rsqrtf(vr.x + eps), ab.x), alpha);
                g.y *= act_grad(fmaf(ag.y, (xv.y - mu.y) * rsqrtf(vr.y + eps), ab.y), alpha);
                g.z *= act_grad(fmaf(ag.z, (xv.z - mu.z) * rsqrtf(vr.z + eps), ab.z), alpha);
                g.w *= act_grad(fmaf(ag.w, (xv.w - mu.w) * rsqrtf(vr.w + eps), ab.w), alpha);
            }
            const float4 k1 = *reinterpret_cast<const float4*>(coeff + c);
            const float4 k2 = *reinterpret_cast<const float4*>(coeff + C + c);
            const float4 k3 = *reinterpret_cast<const float4*>(coeff + 2 * C + c);
            float4 o;
            o.x = fmaf(k1.x, g.x, fmaf(k2.x, xv.x, k3.x));
            o.y = fmaf(k1.y, g.y, fmaf(k2.y, xv.y, k3.y));
            o.z = fmaf(k1.z, g.z, fmaf(k2.z, xv.z, k3.z));
            o.w = fmaf(k1.w, g.w, fmaf(k2.w, xv.w, k3.w));
            reinterpret_cast<float4*>(dx)[i] = o;
        }
    } else {
        for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += stride) {
            const int c = (int)(i % C);
            const float g = act_gamma ? dy[i] * act_grad(fmaf(act_gamma[c], (x[i] - mean[c]) * rsqrtf(var[c] + eps), act_beta[c]), alpha)
                                      : dy[i];
            dx[i] = fmaf(coeff[c], g, fmaf(coeff[C + c], x[i], coeff[2 * C + c]));
        }
    }
}

static int bn_blocks(long long rows) {
    long long nb = rows / 32;
    if (nb > 148LL * 4) nb = 148LL * 4;
    if (nb < 1) nb = 1;
    return (int)nb;
}

__global__ void coeff_scale_kernel(float* __restrict__ scale_shift, const float* __restrict__ m, int C) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    scale_shift[c] *= m[c];
    scale_shift[C + c] *= m[c];
}

// ---- pieces of Batch_Norm shared with block_fused.cu ----------------------------------------------------------
int bn_partial_blocks(long long rows) { return bn_blocks(rows); }

// Batch statistics (reduced here unless `partials` come from the producer of x), running-statistics update and the
// per-channel affine coefficients scale/shift (times channel_scale when given) at ws + nb*3*C floats; returns them.
float* bn_forward_coeffs(const float* x, const float* partials, long long nblocks, const float* gamma, const float* beta,
                         float* running_mean, float* running_var, float* batch_mean, float* batch_var, long long rows,
                         int C, float eps, float momentum, const float* channel_scale, float* ws, cudaStream_t st) {
    int nb = bn_blocks(rows);
    float* coeff = ws + (size_t)nb * 3 * C;
    const float* src = partials;
    if (!partials) {
        launch_bn_reduce<0>(nb, st, x, nullptr, nullptr, nullptr, eps, rows, C, ws);
        count_launch();
        src = ws;
    } else {
        nb = (int)nblocks;
    }
    bn_finalize_fwd_kernel<<<ceil_div(C, FIN_CH), FIN_THREADS, 0, st>>>(src, nb, C, gamma, beta, eps, momentum, running_mean, running_var,
                                                            batch_mean, batch_var, coeff);
    count_launch();
    if (channel_scale) {
        coeff_scale_kernel<<<ceil_div(C, 128), 128, 0, st>>>(coeff, channel_scale, C);
        count_launch();
    }
    return coeff;
}

// Inference coefficients from the running statistics into ws (2*C floats).
float* bn_eval_coeffs(const float* gamma, const float* beta, const float* running_mean, const float* running_var, int C,
                      float eps, float* ws, cudaStream_t st) {
    bn_eval_coeff_kernel<<<ceil_div(C, 128), 128, 0, st>>>(C, gamma, beta, eps, running_mean, running_var, ws);
    count_launch();
    return ws;
}

// dgamma, dbeta and the dx coefficients (k1, k2, k3) from nb partial (sum g, sum g*xhat) pairs.
void bn_backward_coeffs(const float* part, int nb, int C, long long rows, const float* gamma, const float* mean,
                        const float* var, float eps, float* dgamma, float* dbeta, float* coeff, const float* pscale,
                        cudaStream_t st) {
    bn_finalize_bwd_kernel<<<ceil_div(C, FIN_CH), FIN_THREADS, 0, st>>>(part, nb, C, rows, gamma, mean, var, eps, dgamma, dbeta, coeff,
                                                            pscale);
    count_launch();
}

}  // namespace aether

using namespace aether;

extern "C" size_t aether_bn_workspace_bytes(int64_t rows, int C) {
    if (rows <= 0 || C <= 0) return 0;
    return align_up(((size_t)bn_blocks(rows) * 3 + 3) * (size_t)C * sizeof(float), 256);
}

extern "C" int aether_bn_fwd_train(const float* x, const float* gamma, const float* beta, float* running_mean,
                                   float* running_var, float* batch_mean, float* batch_var, float* y, int64_t rows,
                                   int C, float eps, float momentum, void* ws, size_t ws_bytes, void* stream) {
    if (!x || !gamma || !beta || !running_mean || !running_var || !batch_mean || !batch_var || !y || !ws)
        return set_error(AE_BAD_ARG, "aether_bn_fwd_train: null pointer");
    if (rows <= 0 || C <= 0) return set_error(AE_BAD_ARG, "aether_bn_fwd_train: rows=%lld C=%d", (long long)rows, C);
    if (ws_bytes < aether_bn_workspace_bytes(rows, C)) return set_error(AE_BAD_ARG, "aether_bn_fwd_train: workspace too small");
    if ((C & 3) == 0 && (!aligned16(x) || !aligned16(y))) return set_error(AE_BAD_ARG, "aether_bn_fwd_train: arrays must be 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int nb = bn_blocks(rows);
    float* part = static_cast<float*>(ws);
    float* coeff = part + (size_t)nb * 3 * C;
    launch_bn_reduce<0>(nb, st, x, nullptr, nullptr, nullptr, eps, rows, C, part);
    bn_finalize_fwd_kernel<<<ceil_div(C, FIN_CH), FIN_THREADS, 0, st>>>(part, nb, C, gamma, beta, eps, momentum, running_mean,
                                                            running_var, batch_mean, batch_var, coeff);
    const long long n = rows * C;
    affine_channels_kernel<<<blocks_for(n / 4 + 1, 256), 256, 0, st>>>(x, y, coeff, coeff + C, n, C, -1.f);
    count_launch(3);
    return check_launch("aether_bn_fwd_train");
}

// Batch_Norm training forward when the producer of x (a convolution's epilogue) already wrote per-block
// (count, mean, M2) partials of every channel: only the merge and the apply pass run, x is read once instead of twice.
extern "C" int aether_bn_fwd_train_partials(const float* x, const float* partials, int64_t nblocks, const float* gamma,
                                            const float* beta, float* running_mean, float* running_var, float* batch_mean,
                                            float* batch_var, float* y, int64_t rows, int C, float eps, float momentum,
                                            void* ws, size_t ws_bytes, void* stream) {
    if (!x || !partials || !gamma || !beta || !running_mean || !running_var || !batch_mean || !batch_var || !y || !ws)
        return set_error(AE_BAD_ARG, "aether_bn_fwd_train_partials: null pointer");
    if (rows <= 0 || C <= 0 || nblocks <= 0 || nblocks > (1 << 30))
        return set_error(AE_BAD_ARG, "aether_bn_fwd_train_partials: rows=%lld C=%d nblocks=%lld", (long long)rows, C, (long long)nblocks);
    if (ws_bytes < 2 * (size_t)C * sizeof(float) || !aligned16(ws))
        return set_error(AE_BAD_ARG, "aether_bn_fwd_train_partials: workspace too small or misaligned (needs 2*C floats)");
    if ((C & 3) == 0 && (!aligned16(x) || !aligned16(y))) return set_error(AE_BAD_ARG, "aether_bn_fwd_train_partials: arrays must be 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    float* coeff = static_cast<float*>(ws);
    bn_finalize_fwd_kernel<<<ceil_div(C, FIN_CH), FIN_THREADS, 0, st>>>(partials, (int)nblocks, C, gamma, beta, eps, momentum, running_mean,
                                                            running_var, batch_mean, batch_var, coeff);
    const long long n = rows * C;
    affine_channels_kernel<<<blocks_for(n / 4 + 1, 256), 256, 0, st>>>(x, y, coeff, coeff + C, n, C, -1.f);
    count_launch(2);
    return check_launch("aether_bn_fwd_train_partials");
}

// ---- Batch_Norm training forward for callers that cannot hand over a workspace ---------------------------
// Scratch lives in a fixed device array that is part of the library image: every GPU that loads the library
// carries these AETHER_BN_STATIC_SCRATCH_FLOATS * 4 bytes (about 1.8 MB) until the process exits.
// Layout per call: [blocks][3][C] partial (count, mean, M2) triples, then [3][C] coefficients.
static constexpr int BN_STATIC_MAX_BLOCKS = 148;
static constexpr size_t AETHER_BN_STATIC_SCRATCH_FLOATS = ((size_t)BN_STATIC_MAX_BLOCKS * 3 + 3) * AETHER_BN_STATIC_MAX_CHANNELS;
static __device__ __align__(256) float g_bn_static_scratch[AETHER_BN_STATIC_SCRATCH_FLOATS];

// Host code cannot use the array's name as a pointer (on the host it is only a handle for the symbol): the
// device address is looked up once per device and cached here.
static std::atomic<float*> g_bn_static_ptr[64];   // zero-initialised; two threads racing here look the same address up twice

static int bn_static_scratch(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return set_error(AE_CUDA, "aether_bn_fwd_train_static: cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= 64) return set_error(AE_UNSUPPORTED, "aether_bn_fwd_train_static: device ordinal %d out of range", dev);
    float* ptr = g_bn_static_ptr[dev].load(std::memory_order_acquire);
    if (ptr == nullptr) {
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_bn_static_scratch);   // address on the CURRENT device
        if (e != cudaSuccess || ptr == nullptr)
            return set_error(AE_CUDA, "aether_bn_fwd_train_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        g_bn_static_ptr[dev].store(ptr, std::memory_order_release);
    }
    *out = ptr;
    return AE_OK;
}

extern "C" int aether_bn_fwd_train_static(const float* x, const float* gamma, const float* beta, float* running_mean,
                                          float* running_var, float* batch_mean, float* batch_var, float* y,
                                          int64_t rows, int C, float eps, float momentum, void* stream) {
    if (!x || !gamma || !beta || !running_mean || !running_var || !batch_mean || !batch_var || !y)
        return set_error(AE_BAD_ARG, "aether_bn_fwd_train_static: null pointer");
    if (rows <= 0 || C <= 0) return set_error(AE_BAD_ARG, "aether_bn_fwd_train_static: rows=%lld C=%d", (long long)rows, C);
    if (C > AETHER_BN_STATIC_MAX_CHANNELS)
        return set_error(AE_UNSUPPORTED,
                         "aether_bn_fwd_train_static: C=%d exceeds the built-in scratch (at most %d channels); use "
                         "aether_bn_fwd_train with a caller-provided workspace", C, AETHER_BN_STATIC_MAX_CHANNELS);
    if ((C & 3) == 0 && (!aligned16(x) || !aligned16(y)))
        return set_error(AE_BAD_ARG, "aether_bn_fwd_train_static: arrays must be 16-byte aligned");
    float* scratch = nullptr;
    int rc = bn_static_scratch(&scratch);
    if (rc) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int nb = bn_blocks(rows);
    if (nb > BN_STATIC_MAX_BLOCKS) nb = BN_STATIC_MAX_BLOCKS;
    float* part = scratch;
    float* coeff = scratch + (size_t)nb * 3 * C;
    // Every scratch element read below is written earlier in this same call (each block stores all 3*C of its
    // partials, the finalize kernel stores all coefficients), so stale contents of a previous call never matter
    // and nothing has to be cleared.
    launch_bn_reduce<0>(nb, st, x, nullptr, nullptr, nullptr, eps, rows, C, part);
    bn_finalize_fwd_kernel<<<ceil_div(C, FIN_CH), FIN_THREADS, 0, st>>>(part, nb, C, gamma, beta, eps, momentum, running_mean,
                                                            running_var, batch_mean, batch_var, coeff);
    const long long n = rows * C;
    affine_channels_kernel<<<blocks_for(n / 4 + 1, 256), 256, 0, st>>>(x, y, coeff, coeff + C, n, C, -1.f);
    count_launch(3);
    return check_launch("aether_bn_fwd_train_static");
}

extern "C" int aether_bn_fwd_eval(const float* x, const float* gamma, const float* beta, const float* running_mean,
                                  const float* running_var, float* y, int64_t rows, int C, float eps, void* ws,
                                  size_t ws_bytes, void* stream) {
    if (!x || !gamma || !beta || !running_mean || !running_var || !y || !ws)
        return set_error(AE_BAD_ARG, "aether_bn_fwd_eval: null pointer");
    if (rows <= 0 || C <= 0) return set_error(AE_BAD_ARG, "aether_bn_fwd_eval: rows=%lld C=%d", (long long)rows, C);
    if (ws_bytes < 2 * (size_t)C * sizeof(float)) return set_error(AE_BAD_ARG, "aether_bn_fwd_eval: workspace too small");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    float* coeff = static_cast<float*>(ws);
    bn_eval_coeff_kernel<<<ceil_div(C, 128), 128, 0, st>>>(C, gamma, beta, eps, running_mean, running_var, coeff);
    const long long n = rows * C;
    affine_channels_kernel<<<blocks_for(n / 4 + 1, 256), 256, 0, st>>>(x, y, coeff, coeff + C, n, C, -1.f);
    count_launch(2);
    return check_launch("aether_bn_fwd_eval");
}

extern "C" int aether_bn_bwd(const float* x, const float* dy, const float* gamma, const float* batch_mean,
                             const float* batch_var, float* dx, float* dgamma, float* dbeta, int64_t rows, int C,
                             float eps, void* ws, size_t ws_bytes, void* stream) {
    if (!x || !dy || !gamma || !batch_mean || !batch_var || !dx || !dgamma || !dbeta || !ws)
        return set_error(AE_BAD_ARG, "aether_bn_bwd: null pointer");
    if (rows <= 0 || C <= 0) return set_error(AE_BAD_ARG, "aether_bn_bwd: rows=%lld C=%d", (long long)rows, C);
    if (ws_bytes < aether_bn_workspace_bytes(rows, C)) return set_error(AE_BAD_ARG, "aether_bn_bwd: workspace too small");
    if ((C & 3) == 0 && (!aligned16(x) || !aligned16(dy) || !aligned16(dx)))
        return set_error(AE_BAD_ARG, "aether_bn_bwd: arrays must be 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int nb = bn_blocks(rows);
    float* part = static_cast<float*>(ws);
    float* coeff = part + (size_t)nb * 3 * C;
    launch_bn_reduce<1>(nb, st, x, dy, batch_mean, batch_var, eps, rows, C, part);
    bn_finalize_bwd_kernel<<<ceil_div(C, FIN_CH), FIN_THREADS, 0, st>>>(part, nb, C, rows, gamma, batch_mean, batch_var, eps, dgamma,
                                                            dbeta, coeff, nullptr);
    const long long n = rows * C;
    bn_bwd_apply_kernel<<<blocks_for(n / 4 + 1, 256), 256, 0, st>>>(x, dy, dx, coeff, n, C, nullptr, nullptr, nullptr, nullptr, eps, 0.f);
    count_launch(3);
    return check_launch("aether_bn_bwd");
}

// ---- Batch_Norm with the (leaky) ReLU that follows it applied in the same passes ------------------------------
// forward : y = act(bn(x)); the normalised, not yet activated tensor is never written.
// backward: dy is the gradient w.r.t. y; the activation's derivative is taken from the sign of y while the
//           statistics pass and the dx pass read it, so the ReLU's own backward pass disappears as well.
static int bn_act_check(const char* who, int64_t rows, int C, float alpha, const void* a, const void* b, const void* c) {
    if (rows <= 0 || C <= 0) return set_error(AE_BAD_ARG, "%s: rows=%lld C=%d", who, (long long)rows, C);
    if (!(alpha >= 0.f && alpha < 1.f)) return set_error(AE_BAD_ARG, "%s: alpha must be in [0, 1)", who);
    if ((C & 3) == 0 && (!aligned16(a) || !aligned16(b) || !aligned16(c)))
        return set_error(AE_BAD_ARG, "%s: arrays must be 16-byte aligned", who);
    return AE_OK;
}

extern "C" int aether_bn_act_fwd_train(const float* x, const float* partials, int64_t nblocks, const float* gamma,
                                       const float* beta, float* running_mean, float* running_var, float* batch_mean,
                                       float* batch_var, float* y, int64_t rows, int C, float eps, float momentum,
                                       float alpha, const float* channel_scale, void* ws, size_t ws_bytes, void* stream) {
    if (!x || !gamma || !beta || !running_mean || !running_var || !batch_mean || !batch_var || !y || !ws)
        return set_error(AE_BAD_ARG, "aether_bn_act_fwd_train: null pointer");
    int rc = bn_act_check("aether_bn_act_fwd_train", rows, C, alpha, x, y, ws);
    if (rc) return rc;
    if (ws_bytes < aether_bn_workspace_bytes(rows, C)) return set_error(AE_BAD_ARG, "aether_bn_act_fwd_train: workspace too small");
    if (partials && (nblocks <= 0 || nblocks > (1 << 30))) return set_error(AE_BAD_ARG, "aether_bn_act_fwd_train: nblocks");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int nb = bn_blocks(rows);
    float* part = static_cast<float*>(ws);
    float* coeff = part + (size_t)nb * 3 * C;
    const float* src = partials;
    if (!partials) {                       // no producer-side statistics: reduce x here
        launch_bn_reduce<0>(nb, st, x, nullptr, nullptr, nullptr, eps, rows, C, part);
        count_launch();
        src = part;
    } else {
        nb = (int)nblocks;
    }
    bn_finalize_fwd_kernel<<<ceil_div(C, FIN_CH), FIN_THREADS, 0, st>>>(src, nb, C, gamma, beta, eps, momentum, running_mean, running_var,
                                                            batch_mean, batch_var, coeff);
    if (channel_scale) {
        // act(v) * m = act(m * v) for m >= 0 (ReLU and Leaky_ReLU are positively homogeneous): a spatial-dropout
        // mask behind the activation is folded into the affine coefficients, at no cost per element
        coeff_scale_kernel<<<ceil_div(C, 128), 128, 0, st>>>(coeff, channel_scale, C);
        count_launch();
    }
    const long long n = rows * C;
    affine_channels_kernel<<<blocks_for(n / 4 + 1, 256), 256, 0, st>>>(x, y, coeff, coeff + C, n, C, alpha);
    count_launch(2);
    return check_launch("aether_bn_act_fwd_train");
}

extern "C" int aether_bn_act_fwd_eval(const float* x, const float* gamma, const float* beta, const float* running_mean,
                                      const float* running_var, float* y, int64_t rows, int C, float eps, float alpha,
                                      void* ws, size_t ws_bytes, void* stream) {
    if (!x || !gamma || !beta || !running_mean || !running_var || !y || !ws)
        return set_error(AE_BAD_ARG, "aether_bn_act_fwd_eval: null pointer");
    int rc = bn_act_check("aether_bn_act_fwd_eval", rows, C, alpha, x, y, ws);
    if (rc) return rc;
    if (ws_bytes < 2 * (size_t)C * sizeof(float)) return set_error(AE_BAD_ARG, "aether_bn_act_fwd_eval: workspace too small");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    float* coeff = static_cast<float*>(ws);
    bn_eval_coeff_kernel<<<ceil_div(C, 128), 128, 0, st>>>(C, gamma, beta, eps, running_mean, running_var, coeff);
    const long long n = rows * C;
    affine_channels_kernel<<<blocks_for(n / 4 + 1, 256), 256, 0, st>>>(x, y, coeff, coeff + C, n, C, alpha);
    count_launch(2);
    return check_launch("aether_bn_act_fwd_eval");
}

extern "C" int aether_bn_act_bwd(const float* x, const float* beta, const float* dy, const float* gamma,
                                 const float* batch_mean, const float* batch_var, float* dx, float* dgamma, float* dbeta,
                                 int64_t rows, int C, float eps, float alpha, const float* channel_scale, void* ws,
                                 size_t ws_bytes, void* stream) {
    if (!x || !beta || !dy || !gamma || !batch_mean || !batch_var || !dx || !dgamma || !dbeta || !ws)
        return set_error(AE_BAD_ARG, "aether_bn_act_bwd: null pointer");
    int rc = bn_act_check("aether_bn_act_bwd", rows, C, alpha, x, dy, dx);
    if (rc) return rc;
    if (ws_bytes < aether_bn_workspace_bytes(rows, C)) return set_error(AE_BAD_ARG, "aether_bn_act_bwd: workspace too small");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int nb = bn_blocks(rows);
    float* part = static_cast<float*>(ws);
    float* coeff = part + (size_t)nb * 3 * C;
    launch_bn_reduce<1>(nb, st, x, dy, batch_mean, batch_var, eps, rows, C, part, gamma, beta, alpha);
    bn_finalize_bwd_kernel<<<ceil_div(C, FIN_CH), FIN_THREADS, 0, st>>>(part, nb, C, rows, gamma, batch_mean, batch_var, eps, dgamma,
                                                            dbeta, coeff, channel_scale);
    const long long n = rows * C;
    // the four per-channel vectors are read as float4 when C % 4 == 0
    if ((C & 3) == 0 && (!aligned16(gamma) || !aligned16(beta) || !aligned16(batch_mean) || !aligned16(batch_var)))
        return set_error(AE_BAD_ARG, "aether_bn_act_bwd: gamma, beta, batch_mean and batch_var must be 16-byte aligned");
    bn_bwd_apply_kernel<<<blocks_for(n / 4 + 1, 256), 256, 0, st>>>(x, dy, dx, coeff, n, C, gamma, beta, batch_mean, batch_var, eps, alpha);
    count_launch(3);
    return check_launch("aether_bn_act_bwd");
}

namespace aether {
// ====================================================================================== pooling
// Forward: one thread per (output pixel, 4 channels).  The argmax code is the window-local index
// i*fW + j of the FIRST maximum in row-major window order (ties keep the earlier cell).
// I is the flat-index type: unsigned int whenever the element count fits (32-bit divisions are several times
// cheaper than 64-bit ones and the index decode is most of the kernel's instructions), else long long.
// F > 0: F x F windows known at compile time (vec == 4 only): the window's loads are issued together -- one 16-byte
// load in flight per thread does not cover the HBM latency.
template <bool MAX, typename I, int F>
__global__ void __launch_bounds__(256) pool_fwd_kernel(const float* __restrict__ x, float* __restrict__ y,
                                                       uint8_t* __restrict__ arg, int S, int H, int W, int C, int fH_,
                                                       int fW_, int sH, int sW, int Ho, int Wo, int vec) {
    const int fH = F ? F : fH_, fW = F ? F : fW_;
    const int Cv = C / vec;
    const I total = (I)(1LL * S * Ho * Wo * Cv);
    const float inv = 1.f / (float)(fH * fW);
    for (I idx = blockIdx.x * (I)blockDim.x + threadIdx.x; idx < total; idx += (I)gridDim.x * (I)blockDim.x) {
        const int cv = (int)(idx % (I)Cv);
        I pix = idx / (I)Cv;
        const int wo = (int)(pix % Wo);
        pix /= Wo;
        const int ho = (int)(pix % Ho);
        const int s = (int)(pix / Ho);
        const size_t obase = ((size_t)(((size_t)s * Ho + ho) * Wo + wo)) * C + (size_t)cv * vec;
        if (vec == 4) {
            float4 best = make_float4(0.f, 0.f, 0.f, 0.f);
            uchar4 code = make_uchar4(0, 0, 0, 0);
            float4 pre[F ? F * F : 1];
            if (F) {
#pragma unroll
                for (int k = 0; k < F * F; ++k)
                    pre[k] = *reinterpret_cast<const float4*>(
                        x + (((size_t)s * H + ho * sH + k / (F ? F : 1)) * W + wo * sW + k % (F ? F : 1)) * C + cv * 4);
            }
#pragma unroll
            for (int i = 0; i < fH; ++i)
#pragma unroll
                for (int j = 0; j < fW; ++j) {
                    const float4 v = F ? pre[F ? i * F + j : 0]
                                       : *reinterpret_cast<const float4*>(
                                             x + (((size_t)s * H + ho * sH + i) * W + wo * sW + j) * C + cv * 4);
                    const unsigned char k = (unsigned char)(i * fW + j);
                    if (MAX) {
                        if (k == 0) { best = v; }
                        else {
                            if (v.x > best.x) { best.x = v.x; code.x = k; }
                            if (v.y > best.y) { best.y = v.y; code.y = k; }
                            if (v.z > best.z) { best.z = v.z; code.z = k; }
                            if (v.w > best.w) { best.w = v.w; code.w = k; }
                        }
                    } else {
                        best.x += v.x; best.y += v.y; best.z += v.z; best.w += v.w;
                    }
                }
            if (!MAX) { best.x *= inv; best.y *= inv; best.z *= inv; best.w *= inv; }
            *reinterpret_cast<float4*>(y + obase) = best;
            if (MAX) *reinterpret_cast<uchar4*>(arg + obase) = code;
        } else {
            float best = 0.f;
            unsigned char code = 0;
            for (int i = 0; i < fH; ++i)
                for (int j = 0; j < fW; ++j) {
                    const float v = x[(((size_t)s * H + ho * sH + i) * W + wo * sW + j) * C + cv];
                    const unsigned char k = (unsigned char)(i * fW + j);
                    if (MAX) {
                        if (k == 0 || v > best) { best = v; code = k; }
                    } else {
                        best += v;
                    }
                }
            y[obase] = MAX ? best : best * inv;
            if (MAX) arg[obase] = code;
        }
    }
}

// Backward for windows that tile the input exactly (stride == filter, H and W multiples of it; the 2x2/2 pooling of
// every reference network): one thread per (window, 4 channels) reads dy and the argmax code once and writes the
// fH*fW cells of its window -- no per-cell index decode, every byte moved exactly once.
template <bool MAX>
__global__ void __launch_bounds__(256) pool_bwd_tiled_kernel(const float* __restrict__ dy, const uint8_t* __restrict__ arg,
                                                             float* __restrict__ dx, unsigned total, int W, int C4,
                                                             int fH, int fW, int Ho, int Wo) {
    const float inv = 1.f / (float)(fH * fW);
    for (unsigned idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
        const unsigned cv = idx % (unsigned)C4;
        unsigned pix = idx / (unsigned)C4;
        const unsigned wo = pix % (unsigned)Wo;
        pix /= (unsigned)Wo;                                   // = s * Ho + ho
        const float4 g = __ldcs(reinterpret_cast<const float4*>(dy) + idx);
        uchar4 a = make_uchar4(0, 0, 0, 0);
        if (MAX) a = reinterpret_cast<const uchar4*>(arg)[idx];
        // first cell of the window: input row pix*fH (rows of all samples are stacked: H = Ho*fH), column wo*fW
        float4* out = reinterpret_cast<float4*>(dx) + ((size_t)pix * fH * W + (size_t)wo * fW) * C4 + cv;
        for (int i = 0; i < fH; ++i)
            for (int j = 0; j < fW; ++j) {
                float4 o;
                if (MAX) {
                    const unsigned char code = (unsigned char)(i * fW + j);
                    o = make_float4(a.x == code ? g.x : 0.f, a.y == code ? g.y : 0.f, a.z == code ? g.z : 0.f,
                                    a.w == code ? g.w : 0.f);
                } else {
                    o = make_float4(g.x * inv, g.y * inv, g.z * inv, g.w * inv);
                }
                out[((size_t)i * W + j) * C4] = o;
            }
    }
}

// Backward in gather form: each input cell sums the dy of every window that selected it (max) or
// that covers it (average).  No atomics; cells outside every window get zero.
template <bool MAX, int VEC, typename I>
__global__ void __launch_bounds__(256) pool_bwd_kernel(const float* __restrict__ dy, const uint8_t* __restrict__ arg,
                                                       float* __restrict__ dx, int S, int H, int W, int C, int fH,
                                                       int fW, int sH, int sW, int Ho, int Wo) {
    const int Cv = C / VEC;
    const I total = (I)(1LL * S * H * W * Cv);
    const float inv = 1.f / (float)(fH * fW);
    for (I idx = blockIdx.x * (I)blockDim.x + threadIdx.x; idx < total; idx += (I)gridDim.x * (I)blockDim.x) {
        const int cv = (int)(idx % (I)Cv);
        I pix = idx / (I)Cv;
        const int w = (int)(pix % W);
        pix /= W;
        const int h = (int)(pix % H);
        const int s = (int)(pix / H);
        float acc[VEC];
#pragma unroll
        for (int k = 0; k < VEC; ++k) acc[k] = 0.f;
        // windows (ho, wo) with ho*sH <= h < ho*sH + fH
        const int ho_hi = min(Ho - 1, h / sH);
        const int wo_hi = min(Wo - 1, w / sW);
        for (int ho = ho_hi; ho >= 0 && ho * sH + fH > h; --ho) {
            const int i = h - ho * sH;
            for (int wo = wo_hi; wo >= 0 && wo * sW + fW > w; --wo) {
                const int j = w - wo * sW;
                const size_t o = (((size_t)s * Ho + ho) * Wo + wo) * C + (size_t)cv * VEC;
                const unsigned char code = (unsigned char)(i * fW + j);
                if (VEC == 4) {
                    const float4 g = *reinterpret_cast<const float4*>(dy + o);
                    if (MAX) {
                        const uchar4 a = *reinterpret_cast<const uchar4*>(arg + o);
                        if (a.x == code) acc[0] += g.x;
                        if (a.y == code) acc[1] += g.y;
                        if (a.z == code) acc[2] += g.z;
                        if (a.w == code) acc[3] += g.w;
                    } else {
                        acc[0] += g.x * inv; acc[1] += g.y * inv; acc[2] += g.z * inv; acc[3] += g.w * inv;
                    }
                } else {
                    if (MAX) {
                        if (arg[o] == code) acc[0] += dy[o];
                    } else {
                        acc[0] += dy[o] * inv;
                    }
                }
            }
        }
        if (VEC == 4) *reinterpret_cast<float4*>(dx + (size_t)idx * 4) = make_float4(acc[0], acc[1], acc[2], acc[3]);
        else dx[idx] = acc[0];
    }
}

// ====================================================================================== activations
// y = x > 0 ? x : alpha * x   (alpha = 0 gives ReLU)
__global__ void __launch_bounds__(256) lrelu_fwd_kernel(const float* __restrict__ x, float* __restrict__ y, long long n,
                                                        float alpha) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    const long long n4 = n >> 2;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += stride) {
        float4 v = reinterpret_cast<const float4*>(x)[i];
        v.x = v.x > 0.f ? v.x : alpha * v.x;
        v.y = v.y > 0.f ? v.y : alpha * v.y;
        v.z = v.z > 0.f ? v.z : alpha * v.z;
        v.w = v.w > 0.f ? v.w : alpha * v.w;
        reinterpret_cast<float4*>(y)[i] = v;
    }
    for (long long i = (n4 << 2) + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += stride)
        y[i] = x[i] > 0.f ? x[i] : alpha * x[i];
}
// dx = x < 0 ? alpha * dy : dy   (the gradient passes where x == 0, as in the reference)
__global__ void __launch_bounds__(256) lrelu_bwd_kernel(const float* __restrict__ x, const float* __restrict__ dy,
                                                        float* __restrict__ dx, long long n, float alpha) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    const long long n4 = n >> 2;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += stride) {
        const float4 v = reinterpret_cast<const float4*>(x)[i];
        float4 g = reinterpret_cast<const float4*>(dy)[i];
        g.x = v.x < 0.f ? alpha * g.x : g.x;
        g.y = v.y < 0.f ? alpha * g.y : g.y;
        g.z = v.z < 0.f ? alpha * g.z : g.z;
        g.w = v.w < 0.f ? alpha * g.w : g.w;
        reinterpret_cast<float4*>(dx)[i] = g;
    }
    for (long long i = (n4 << 2) + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += stride)
        dx[i] = x[i] < 0.f ? alpha * dy[i] : dy[i];
}

// ====================================================================================== dropout
// Counter-based generator (Philox-4x32-10, Salmon et al. 2011): 4 uniforms per (seed, index).
__device__ __forceinline__ uint4 philox4x32_10(uint2 key, uint4 ctr) {
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const unsigned int hi0 = __umulhi(0xD2511F53u, ctr.x), lo0 = 0xD2511F53u * ctr.x;
        const unsigned int hi1 = __umulhi(0xCD9E8D57u, ctr.z), lo1 = 0xCD9E8D57u * ctr.z;
        ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
        key.x += 0x9E3779B9u;
        key.y += 0xBB67AE85u;
    }
    return ctr;
}
// mask[i] = (u < keep) / keep ; y = x * mask.  4 elements per thread.
__global__ void __launch_bounds__(256) dropout_fwd_kernel(const float* __restrict__ x, float* __restrict__ y,
                                                          float* __restrict__ mask, long long n, float keep,
                                                          unsigned long long seed, unsigned long long offset,
                                                          const long long* __restrict__ calls_dev) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    const float scale = 1.f / keep;
    // a call counter kept in device memory (replayed CUDA graphs cannot change kernel arguments) selects the stream
    if (calls_dev) offset += ((unsigned long long)*calls_dev) << 40;
    for (long long q = blockIdx.x * (long long)blockDim.x + threadIdx.x; q * 4 < n; q += stride) {
        const unsigned long long ctr = (unsigned long long)q + offset;
        const uint4 r = philox4x32_10(make_uint2((unsigned)seed, (unsigned)(seed >> 32)),
                                      make_uint4((unsigned)ctr, (unsigned)(ctr >> 32), 0u, 0u));
        const unsigned int rr[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const long long i = q * 4 + k;
            if (i < n) {
                const float u = (float)(rr[k] >> 8) * (1.0f / 16777216.0f);
                const float m = u < keep ? scale : 0.f;
                mask[i] = m;
                y[i] = x[i] * m;
            }
        }
    }
}
// Channel mask of Layer_Dropout_Spatial drawn on the device: mask[c] = Bernoulli(keep) / keep, one Philox stream per call.
__global__ void channel_mask_kernel(float* __restrict__ mask, int C, float keep, unsigned long long seed,
                                    const long long* __restrict__ calls_dev) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const unsigned long long ctr = (unsigned long long)c + (((unsigned long long)*calls_dev) << 40);
    const uint4 r = philox4x32_10(make_uint2((unsigned)seed, (unsigned)(seed >> 32)),
                                  make_uint4((unsigned)ctr, (unsigned)(ctr >> 32), 0x5Du, 0u));
    const float u = (float)(r.x >> 8) * (1.0f / 16777216.0f);
    mask[c] = u < keep ? 1.f / keep : 0.f;
}
__global__ void __launch_bounds__(256) mul_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                  float* __restrict__ y, long long n) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += stride) y[i] = a[i] * b[i];
}

// ====================================================================================== Adam
// One launch updates a whole flat parameter buffer (Optimizer_Adam.update_parameters, :710-734):
//   g' = g * gscale;  m = b1*m + (1-b1)*g';  v = b2*v + (1-b2)*g'^2
//   p -= lr * (m / bc1) / (sqrt(v / bc2) + eps)        with bc = 1 - beta^(iterations+1)
__global__ void __launch_bounds__(256) adam_kernel(float* __restrict__ p, const float* __restrict__ g,
                                                   float* __restrict__ m, float* __restrict__ v, long long n, float lr,
                                                   float b1, float b2, float eps, float inv_bc1, float inv_bc2,
                                                   float gscale) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += stride) {
        const float gi = g[i] * gscale;
        const float mi = b1 * m[i] + (1.f - b1) * gi;
        const float vi = b2 * v[i] + (1.f - b2) * gi * gi;
        m[i] = mi;
        v[i] = vi;
        p[i] -= lr * (mi * inv_bc1) / (sqrtf(vi * inv_bc2) + eps);
    }
}

// The same update with the step count read from device memory, so that a captured CUDA graph replays it with the
// right learning-rate decay (:705-707) and bias corrections (:716-723) every time: `iterations` is the number of
// updates already made, as Optimizer_Adam.iterations.
__global__ void __launch_bounds__(256) adam_dev_kernel(float* __restrict__ p, const float* __restrict__ g,
                                                       float* __restrict__ m, float* __restrict__ v, long long n, float lr0,
                                                       float decay, float b1, float b2, float eps, float gscale,
                                                       const long long* __restrict__ iterations) {
    const double it = (double)*iterations;
    const float lr = decay != 0.f ? (float)((double)lr0 * (1.0 / (1.0 + (double)decay * it))) : lr0;
    const float inv_bc1 = (float)(1.0 / (1.0 - pow((double)b1, it + 1.0)));
    const float inv_bc2 = (float)(1.0 / (1.0 - pow((double)b2, it + 1.0)));
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += stride) {
        const float gi = g[i] * gscale;
        const float mi = b1 * m[i] + (1.f - b1) * gi;
        const float vi = b2 * v[i] + (1.f - b2) * gi * gi;
        m[i] = mi;
        v[i] = vi;
        p[i] -= lr * (mi * inv_bc1) / (sqrtf(vi * inv_bc2) + eps);
    }
}

// g += l1 * sign(w) + 2 * l2 * w   (Layer_Dense.backward regulariser terms, :337-351; sign(0) = +1)
__global__ void __launch_bounds__(256) reg_grad_kernel(const float* __restrict__ w, float* __restrict__ g, long long n,
                                                       float l1, float l2) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += stride) {
        const float wi = w[i];
        g[i] += l1 * (wi < 0.f ? -1.f : 1.f) + 2.f * l2 * wi;
    }
}

// out[0] += l1 * sum|w| + l2 * sum w^2   (Loss.regularization_loss, :593-609); single block, fixed order.
__global__ void __launch_bounds__(256) reg_loss_kernel(const float* __restrict__ w, long long n, float l1, float l2,
                                                       float* __restrict__ out) {
    __shared__ double sh[256];
    double acc = 0.0;
    for (long long i = threadIdx.x; i < n; i += blockDim.x) {
        const double wi = w[i];
        acc += l1 * fabs(wi) + l2 * wi * wi;
    }
    sh[threadIdx.x] = acc;
    __syncthreads();
    for (int s = 128; s > 0; s >>= 1) {
        if (threadIdx.x < s) sh[threadIdx.x] += sh[threadIdx.x + s];
        __syncthreads();
    }
    if (threadIdx.x == 0) out[0] += (float)sh[0];
}

// ====================================================================================== softmax + CCE
// One warp per sample: probabilities, clipped cross-entropy with label smoothing, the combined
// gradient (p - y_smooth) / rows, and whether argmax(p) == label.
__global__ void __launch_bounds__(256) softmax_cce_kernel(const float* __restrict__ z, const int* __restrict__ labels,
                                                          float* __restrict__ prob, float* __restrict__ loss,
                                                          float* __restrict__ dz, int* __restrict__ correct, int rows,
                                                          int classes, float smooth_fwd, float smooth_bwd,
                                                          int input_is_prob, const float* __restrict__ targets) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= rows) return;
    const float* zr = z + (size_t)warp * classes;
    float mx = -INFINITY;
    int amax = 0;
    for (int k = lane; k < classes; k += 32) {
        const float v = zr[k];
        if (v > mx) { mx = v; amax = k; }
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float om = __shfl_xor_sync(0xffffffffu, mx, o);
        const int oa = __shfl_xor_sync(0xffffffffu, amax, o);
        if (om > mx || (om == mx && oa < amax)) { mx = om; amax = oa; }
    }
    float sum = 0.f;
    if (!input_is_prob) {
        for (int k = lane; k < classes; k += 32) sum += expf(zr[k] - mx);
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    }
    // targets: class indices (labels) or rows of target probabilities (one-hot or soft, :625-637); for the accuracy a
    // row of targets stands for its arg-max (CNN_model_cupy.py:383-385)
    int label = labels ? labels[warp] : -1;
    if (targets) {
        const float* tr = targets + (size_t)warp * classes;
        float tm = -INFINITY;
        int ta = 0;
        for (int k = lane; k < classes; k += 32) {
            const float v = tr[k];
            if (v > tm) { tm = v; ta = k; }
        }
        for (int o = 16; o > 0; o >>= 1) {
            const float om = __shfl_xor_sync(0xffffffffu, tm, o);
            const int oa = __shfl_xor_sync(0xffffffffu, ta, o);
            if (om > tm || (om == tm && oa < ta)) { tm = om; ta = oa; }
        }
        label = ta;
    }
    const float inv_rows = 1.f / (float)rows;
    float l = 0.f;
    for (int k = lane; k < classes; k += 32) {
        const float pk = input_is_prob ? zr[k] : expf(zr[k] - mx) / sum;
        if (prob) prob[(size_t)warp * classes + k] = pk;
        if (labels || targets) {
            const float onehot = targets ? targets[(size_t)warp * classes + k] : ((k == label) ? 1.f : 0.f);
            const float tf = onehot * (1.f - smooth_fwd) + smooth_fwd / classes;
            const float tb = onehot * (1.f - smooth_bwd) + smooth_bwd / classes;
            const float pc = fminf(fmaxf(pk, 1e-7f), 1.f - 1e-7f);
            l -= tf * logf(pc);
            if (dz) dz[(size_t)warp * classes + k] = (pk - tb) * inv_rows;
        }
    }
    for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
    if (lane == 0) {
        if (loss) loss[warp] = l;
        if (correct) correct[warp] = (amax == label) ? 1 : 0;
    }
}

// SoftMax.backward (CNN_classes_cupy.py:549-560): per sample dinputs = (diag(p) - p p^T) dvalues = p * (dv - <p, dv>).
// One warp per sample, the dot product reduced with shuffles in a fixed order.
__global__ void __launch_bounds__(256) softmax_bwd_kernel(const float* __restrict__ p, const float* __restrict__ dv,
                                                          float* __restrict__ dx, int rows, int classes) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= rows) return;
    const float* pr = p + (size_t)warp * classes;
    const float* dr = dv + (size_t)warp * classes;
    float dot = 0.f;
    for (int k = lane; k < classes; k += 32) dot = fmaf(pr[k], dr[k], dot);
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    for (int k = lane; k < classes; k += 32) dx[(size_t)warp * classes + k] = pr[k] * (dr[k] - dot);
}

}  // namespace aether

// ====================================================================================== C ABI
extern "C" int aether_softmax_bwd(const float* p, const float* dvalues, float* dinputs, int rows, int classes, void* stream) {
    if (!p || !dvalues || !dinputs || rows <= 0 || classes <= 0) return set_error(AE_BAD_ARG, "aether_softmax_bwd: bad argument");
    softmax_bwd_kernel<<<ceil_div(rows * 32, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(p, dvalues, dinputs, rows, classes);
    count_launch();
    return check_launch("aether_softmax_bwd");
}

extern "C" int aether_pool_fwd(const float* x, float* y, uint8_t* argmax, int S, int H, int W, int C, int fH, int fW,
                               int sH, int sW, int kind, void* stream) {
    if (!x || !y || (kind == AETHER_POOL_MAX && !argmax)) return set_error(AE_BAD_ARG, "aether_pool_fwd: null pointer");
    if (S <= 0 || C <= 0 || fH <= 0 || fW <= 0 || sH <= 0 || sW <= 0 || H < fH || W < fW || fH * fW > 255)
        return set_error(AE_BAD_ARG, "aether_pool_fwd: bad shape S=%d H=%d W=%d C=%d f=%dx%d s=%dx%d", S, H, W, C, fH, fW, sH, sW);
    if (kind != AETHER_POOL_MAX && kind != AETHER_POOL_AVG) return set_error(AE_UNSUPPORTED, "aether_pool_fwd: kind %d", kind);
    const int Ho = (H - fH) / sH + 1, Wo = (W - fW) / sW + 1;
    const int vec = ((C & 3) == 0 && aligned16(x) && aligned16(y) && (!argmax || (reinterpret_cast<uintptr_t>(argmax) & 3) == 0)) ? 4 : 1;
    const long long total = 1LL * S * Ho * Wo * (C / vec);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int nb = blocks_for(total, 256, 16);
    const bool small = total < (1LL << 31);
    const bool two = vec == 4 && fH == 2 && fW == 2;
#define AETHER_POOL_FWD(MAXK, I, ARG)                                                                                  \
    do {                                                                                                               \
        if (two) pool_fwd_kernel<MAXK, I, 2><<<nb, 256, 0, st>>>(x, y, ARG, S, H, W, C, fH, fW, sH, sW, Ho, Wo, vec);  \
        else pool_fwd_kernel<MAXK, I, 0><<<nb, 256, 0, st>>>(x, y, ARG, S, H, W, C, fH, fW, sH, sW, Ho, Wo, vec);      \
    } while (0)
    if (kind == AETHER_POOL_MAX) {
        if (small) AETHER_POOL_FWD(true, unsigned, argmax);
        else AETHER_POOL_FWD(true, long long, argmax);
    } else {
        if (small) AETHER_POOL_FWD(false, unsigned, nullptr);
        else AETHER_POOL_FWD(false, long long, nullptr);
    }
#undef AETHER_POOL_FWD
    count_launch();
    return check_launch("aether_pool_fwd");
}

extern "C" int aether_pool_bwd(const float* dy, const uint8_t* argmax, float* dx, int S, int H, int W, int C, int fH,
                               int fW, int sH, int sW, int kind, void* stream) {
    if (!dy || !dx || (kind == AETHER_POOL_MAX && !argmax)) return set_error(AE_BAD_ARG, "aether_pool_bwd: null pointer");
    if (S <= 0 || C <= 0 || fH <= 0 || fW <= 0 || sH <= 0 || sW <= 0 || H < fH || W < fW || fH * fW > 255)
        return set_error(AE_BAD_ARG, "aether_pool_bwd: bad shape");
    if (kind != AETHER_POOL_MAX && kind != AETHER_POOL_AVG) return set_error(AE_UNSUPPORTED, "aether_pool_bwd: kind %d", kind);
    const int Ho = (H - fH) / sH + 1, Wo = (W - fW) / sW + 1;
    const bool vec = (C & 3) == 0 && aligned16(dy) && aligned16(dx) && (!argmax || (reinterpret_cast<uintptr_t>(argmax) & 3) == 0);
    const long long total = 1LL * S * H * W * (vec ? C / 4 : C);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int nb = blocks_for(total, 256, 16);
    const long long windows4 = 1LL * S * Ho * Wo * (C / 4);
    if (vec && sH == fH && sW == fW && H == Ho * fH && W == Wo * fW && windows4 < (1LL << 32) - (1LL << 22)) {
        const int nbt = blocks_for(windows4, 256, 16);
        if (kind == AETHER_POOL_MAX)
            pool_bwd_tiled_kernel<true><<<nbt, 256, 0, st>>>(dy, argmax, dx, (unsigned)windows4, W, C / 4, fH, fW, Ho, Wo);
        else
            pool_bwd_tiled_kernel<false><<<nbt, 256, 0, st>>>(dy, nullptr, dx, (unsigned)windows4, W, C / 4, fH, fW, Ho, Wo);
        count_launch();
        return check_launch("aether_pool_bwd");
    }
#define AETHER_POOL_BWD(MAXK, V, I, ARG) \
    pool_bwd_kernel<MAXK, V, I><<<nb, 256, 0, st>>>(dy, ARG, dx, S, H, W, C, fH, fW, sH, sW, Ho, Wo)
    const bool small = total < (1LL << 31);
    if (kind == AETHER_POOL_MAX) {
        if (vec && small) AETHER_POOL_BWD(true, 4, unsigned, argmax);
        else if (vec) AETHER_POOL_BWD(true, 4, long long, argmax);
        else if (small) AETHER_POOL_BWD(true, 1, unsigned, argmax);
        else AETHER_POOL_BWD(true, 1, long long, argmax);
    } else {
        if (vec && small) AETHER_POOL_BWD(false, 4, unsigned, nullptr);
        else if (vec) AETHER_POOL_BWD(false, 4, long long, nullptr);
        else if (small) AETHER_POOL_BWD(false, 1, unsigned, nullptr);
        else AETHER_POOL_BWD(false, 1, long long, nullptr);
    }
#undef AETHER_POOL_BWD
    count_launch();
    return check_launch("aether_pool_bwd");
}

extern "C" int aether_leaky_relu_fwd(const float* x, float* y, int64_t n, float alpha, void* stream) {
    if (!x || !y || n <= 0) return set_error(AE_BAD_ARG, "aether_leaky_relu_fwd: bad argument");
    if (!aligned16(x) || !aligned16(y)) return set_error(AE_BAD_ARG, "aether_leaky_relu_fwd: arrays must be 16-byte aligned");
    lrelu_fwd_kernel<<<blocks_for(n / 4 + 1, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(x, y, n, alpha);
    count_launch();
    return check_launch("aether_leaky_relu_fwd");
}

extern "C" int aether_leaky_relu_bwd(const float* x, const float* dy, float* dx, int64_t n, float alpha, void* stream) {
    if (!x || !dy || !dx || n <= 0) return set_error(AE_BAD_ARG, "aether_leaky_relu_bwd: bad argument");
    if (!aligned16(x) || !aligned16(dy) || !aligned16(dx)) return set_error(AE_BAD_ARG, "aether_leaky_relu_bwd: arrays must be 16-byte aligned");
    lrelu_bwd_kernel<<<blocks_for(n / 4 + 1, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(x, dy, dx, n, alpha);
    count_launch();
    return check_launch("aether_leaky_relu_bwd");
}

extern "C" int aether_channel_scale(const float* x, const float* scale, float* y, int64_t n, int C, void* stream) {
    if (!x || !scale || !y || n <= 0 || C <= 0 || n % C) return set_error(AE_BAD_ARG, "aether_channel_scale: bad argument");
    if ((C & 3) == 0 && (!aligned16(x) || !aligned16(y) || !aligned16(scale)))
        return set_error(AE_BAD_ARG, "aether_channel_scale: arrays must be 16-byte aligned");
    affine_channels_kernel<<<blocks_for(n / 4 + 1, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(x, y, scale, nullptr, n, C, -1.f);
    count_launch();
    return check_launch("aether_channel_scale");
}

extern "C" int aether_dropout_fwd(const float* x, float* y, float* mask, int64_t n, float keep_prob, uint64_t seed,
                                  uint64_t offset, void* stream) {
    if (!x || !y || !mask || n <= 0 || !(keep_prob > 0.f) || keep_prob > 1.f)
        return set_error(AE_BAD_ARG, "aether_dropout_fwd: bad argument");
    dropout_fwd_kernel<<<blocks_for(n / 4 + 1, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(x, y, mask, n, keep_prob, seed, offset,
                                                                                                  nullptr);
    count_launch();
    return check_launch("aether_dropout_fwd");
}

// Variants for captured CUDA graphs: whatever changes from step to step is read from device memory.
extern "C" int aether_dropout_fwd_dev(const float* x, float* y, float* mask, int64_t n, float keep_prob, uint64_t seed,
                                      uint64_t offset, const int64_t* calls_dev, void* stream) {
    if (!x || !y || !mask || !calls_dev || n <= 0 || !(keep_prob > 0.f) || keep_prob > 1.f)
        return set_error(AE_BAD_ARG, "aether_dropout_fwd_dev: bad argument");
    dropout_fwd_kernel<<<blocks_for(n / 4 + 1, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        x, y, mask, n, keep_prob, seed, offset, reinterpret_cast<const long long*>(calls_dev));
    count_launch();
    return check_launch("aether_dropout_fwd_dev");
}

extern "C" int aether_channel_mask_dev(float* mask, int C, float keep_prob, uint64_t seed, const int64_t* calls_dev,
                                       void* stream) {
    if (!mask || !calls_dev || C <= 0 || !(keep_prob > 0.f) || keep_prob > 1.f)
        return set_error(AE_BAD_ARG, "aether_channel_mask_dev: bad argument");
    channel_mask_kernel<<<ceil_div(C, 128), 128, 0, static_cast<cudaStream_t>(stream)>>>(
        mask, C, keep_prob, seed, reinterpret_cast<const long long*>(calls_dev));
    count_launch();
    return check_launch("aether_channel_mask_dev");
}

extern "C" int aether_adam_step_dev(float* p, const float* g, float* m, float* v, int64_t n, float lr0, float decay,
                                    float beta1, float beta2, float eps, float grad_scale, const int64_t* iterations_dev,
                                    void* stream) {
    if (!p || !g || !m || !v || !iterations_dev || n <= 0) return set_error(AE_BAD_ARG, "aether_adam_step_dev: bad argument");
    if (!(beta1 >= 0.f && beta1 < 1.f) || !(beta2 >= 0.f && beta2 < 1.f))
        return set_error(AE_BAD_ARG, "aether_adam_step_dev: betas must be in [0, 1)");
    adam_dev_kernel<<<blocks_for(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        p, g, m, v, n, lr0, decay, beta1, beta2, eps, grad_scale, reinterpret_cast<const long long*>(iterations_dev));
    count_launch();
    return check_launch("aether_adam_step_dev");
}

extern "C" int aether_mul(const float* a, const float* b, float* y, int64_t n, void* stream) {
    if (!a || !b || !y || n <= 0) return set_error(AE_BAD_ARG, "aether_mul: bad argument");
    mul_kernel<<<blocks_for(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(a, b, y, n);
    count_launch();
    return check_launch("aether_mul");
}

extern "C" int aether_adam_step(float* p, const float* g, float* m, float* v, int64_t n, float lr, float beta1,
                                float beta2, float eps, float bias_corr1, float bias_corr2, float grad_scale,
                                void* stream) {
    if (!p || !g || !m || !v || n <= 0) return set_error(AE_BAD_ARG, "aether_adam_step: bad argument");
    if (!(bias_corr1 > 0.f) || !(bias_corr2 > 0.f)) return set_error(AE_BAD_ARG, "aether_adam_step: bias corrections must be > 0");
    adam_kernel<<<blocks_for(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(p, g, m, v, n, lr, beta1, beta2, eps, 1.f / bias_corr1,
                                                                                   1.f / bias_corr2, grad_scale);
    count_launch();
    return check_launch("aether_adam_step");
}

extern "C" int aether_regularizer_grad(const float* w, float* g, int64_t n, float l1, float l2, void* stream) {
    if (!w || !g || n <= 0) return set_error(AE_BAD_ARG, "aether_regularizer_grad: bad argument");
    reg_grad_kernel<<<blocks_for(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(w, g, n, l1, l2);
    count_launch();
    return check_launch("aether_regularizer_grad");
}

extern "C" int aether_regularizer_loss(const float* w, int64_t n, float l1, float l2, float* out, void* stream) {
    if (!w || !out || n <= 0) return set_error(AE_BAD_ARG, "aether_regularizer_loss: bad argument");
    reg_loss_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(w, n, l1, l2, out);
    count_launch();
    return check_launch("aether_regularizer_loss");
}

extern "C" int aether_softmax_cce(const float* z, const int32_t* labels, float* prob, float* loss, float* dz,
                                  int32_t* correct, int rows, int classes, float smooth_fwd, float smooth_bwd,
                                  int input_is_prob, void* stream) {
    if (!z || rows <= 0 || classes <= 0) return set_error(AE_BAD_ARG, "aether_softmax_cce: bad argument");
    if (!labels && (loss || dz || correct)) return set_error(AE_BAD_ARG, "aether_softmax_cce: labels required for loss/gradient");
    const int threads = 256;
    const int blocks = ceil_div(rows * 32, threads);
    softmax_cce_kernel<<<blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(z, labels, prob, loss, dz, correct, rows, classes, smooth_fwd, smooth_bwd, input_is_prob, nullptr);
    count_launch();
    return check_launch("aether_softmax_cce");
}

extern "C" int aether_softmax_cce_targets(const float* z, const float* targets, float* prob, float* loss, float* dz,
                                          int32_t* correct, int rows, int classes, float smooth_fwd, float smooth_bwd,
                                          int input_is_prob, void* stream) {
    if (!z || !targets || rows <= 0 || classes <= 0) return set_error(AE_BAD_ARG, "aether_softmax_cce_targets: bad argument");
    const int threads = 256;
    const int blocks = ceil_div(rows * 32, threads);
    softmax_cce_kernel<<<blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(z, nullptr, prob, loss, dz, correct, rows, classes, smooth_fwd, smooth_bwd, input_is_prob, targets);
    count_launch();
    return check_launch("aether_softmax_cce_targets");
}
