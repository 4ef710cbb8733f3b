// The tail of a convolution block of the reference's networks -- Batch_Norm, ReLU / Leaky_ReLU, optional
// Layer_Dropout_Spatial, max Pooling whose windows tile the input (CNN_classes_cupy.py:430-526, 406-428, 384-404,
// 204-312) -- in one pass each way.  The activation between the convolution and the pooling is never written:
//
//   forward : pooled = maxpool( act(x * scale[c] + shift[c]) ), argmax codes kept   (mask folded into scale/shift)
//             reads x once, writes |x|/4 floats + |x|/4 bytes  (layer by layer: 3 reads and 3 writes of |x|)
//   backward: the gradient of an input cell is d_pooled of its window if the cell was the window's maximum, times
//             the activation's derivative, recomputed from x (v = gamma * xhat + beta); a statistics pass and a
//             dx pass, each reading x and d_pooled once.
//
// Every thread owns one window and four channels.  Statistics, running averages, coefficient algebra and the
// fixed-order reductions are the Batch_Norm kernels of layers.cu.
#include <cuda_bf16.h>

#include "common.cuh"

namespace aether {

// Operand copy hand-off.  The tensor these passes write (the pooled activation going forward, dx going back) is the
// next convolution's x, respectively the previous convolution's dy, whose tensor-core kernels read a bf16 copy with
// the channels padded to `ld`.  When the consumer's workspace is known the copy is written here, from the values
// already in registers, instead of by a cast pass that reads the fp32 tensor again: 4 channels = 8 bytes per thread,
// and the threads of the first channel groups also zero the padding [C, ld) of their pixel.
__device__ __forceinline__ void store_operand_copy(__nv_bfloat16* copy, int ld, size_t pixel, int cv, int C4, float4 v) {
    __nv_bfloat162 o[2] = {__floats2bfloat162_rn(v.x, v.y), __floats2bfloat162_rn(v.z, v.w)};
    __nv_bfloat16* row = copy + pixel * (size_t)ld;
    *reinterpret_cast<uint2*>(row + cv * 4) = *reinterpret_cast<uint2*>(o);
    for (int pg = C4 + cv; pg * 4 < ld; pg += C4) *reinterpret_cast<uint2*>(row + pg * 4) = make_uint2(0u, 0u);
}

__device__ __forceinline__ float lrelu(float v, float alpha) { return v > 0.f ? v : alpha * v; }
// derivative of the activation at pre-activation v (the reference passes the gradient at v == 0, :412-428)
__device__ __forceinline__ float lrelu_grad(float v, float alpha) { return v < 0.f ? alpha : 1.f; }

// F > 0: square F x F windows known at compile time -- the window's loads are issued together (one load in flight
// per thread does not cover the HBM latency); F == 0: any window, cells one after the other.
template <int F>
__global__ void __launch_bounds__(256) bn_act_pool_fwd_kernel(const float* __restrict__ x, const float* __restrict__ scale,
                                                              const float* __restrict__ shift, float alpha,
                                                              float* __restrict__ y, uint8_t* __restrict__ arg,
                                                              unsigned total, int W, int C4, int fH_, int fW_, int Wo,
                                                              __nv_bfloat16* __restrict__ copy, int copy_ld,
                                                              float* __restrict__ xsel) {
    const int fH = F ? F : fH_, fW = F ? F : fW_;
    for (unsigned idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
        const unsigned cv = idx % (unsigned)C4;
        unsigned pix = idx / (unsigned)C4;
        const unsigned opix = pix;                             // output pixel of this window
        const unsigned wo = pix % (unsigned)Wo;
        pix /= (unsigned)Wo;                                   // = s * Ho + ho; input rows of all samples are stacked
        const float4 s = *reinterpret_cast<const float4*>(scale + cv * 4);
        const float4 t = *reinterpret_cast<const float4*>(shift + cv * 4);
        const float4* in = reinterpret_cast<const float4*>(x) + ((size_t)pix * fH * W + (size_t)wo * fW) * C4 + cv;
        float4 best = make_float4(0.f, 0.f, 0.f, 0.f), sel = best;     // sel: the input value at the selected cell
        uchar4 code = make_uchar4(0, 0, 0, 0);
        float4 pre[F ? F * F : 1];
        if (F) {
#pragma unroll
            for (int k = 0; k < F * F; ++k) pre[k] = __ldcs(in + ((size_t)(k / (F ? F : 1)) * W + k % (F ? F : 1)) * C4);
        }
#pragma unroll
        for (int i = 0; i < fH; ++i)
#pragma unroll
            for (int j = 0; j < fW; ++j) {
                const float4 v = F ? pre[F ? i * F + j : 0] : __ldcs(in + ((size_t)i * W + j) * C4);
                float4 o;
                o.x = lrelu(fmaf(v.x, s.x, t.x), alpha); o.y = lrelu(fmaf(v.y, s.y, t.y), alpha);
                o.z = lrelu(fmaf(v.z, s.z, t.z), alpha); o.w = lrelu(fmaf(v.w, s.w, t.w), alpha);
                const unsigned char k = (unsigned char)(i * fW + j);
                if (k == 0) {
                    best = o;
                    sel = v;
                } else {                                      // first maximum in row-major window order, as Pooling
                    if (o.x > best.x) { best.x = o.x; code.x = k; sel.x = v.x; }
                    if (o.y > best.y) { best.y = o.y; code.y = k; sel.y = v.y; }
                    if (o.z > best.z) { best.z = o.z; code.z = k; sel.z = v.z; }
                    if (o.w > best.w) { best.w = o.w; code.w = k; sel.w = v.w; }
                }
            }
        if (y != nullptr) reinterpret_cast<float4*>(y)[idx] = best;       // not written when only the bf16 copy is wanted
        reinterpret_cast<uchar4*>(arg)[idx] = code;
        if (copy != nullptr) store_operand_copy(copy, copy_ld, opix, (int)cv, C4, best);
        if (xsel != nullptr) reinterpret_cast<float4*>(xsel)[idx] = sel;
    }
}

// The backward statistics pass when the forward pass kept the input value at every window's selected cell (xsel,
// shaped like the pooled tensor): only that cell has a gradient, so sum(g) and sum(g * xhat) need xsel and d_pooled
// alone -- half of |x| in coalesced reads instead of all of x gathered cell by cell.  part[block][2][C].
__global__ void __launch_bounds__(256) bn_act_pool_bwd_reduce_sel_kernel(
    const float* __restrict__ xsel, const float* __restrict__ dpool, const float* __restrict__ gamma,
    const float* __restrict__ beta, const float* __restrict__ mean, const float* __restrict__ var, float eps, float alpha,
    long long windows, long long win_per_block, int C, float* __restrict__ part) {
    const long long w0 = blockIdx.x * win_per_block;
    long long w1 = w0 + win_per_block;
    if (w1 > windows) w1 = windows;
    const int CV = C >> 2;
    const int cols = CV < 256 ? CV : 256;
    const int lanes = 256 / cols;
    __shared__ float4 sh_a4[256], sh_b4[256];
    for (int cbase = 0; cbase < CV; cbase += cols) {
        const int cv = cbase + threadIdx.x % cols;
        const int rl = threadIdx.x / cols;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
        if (rl < lanes && cv < CV) {
            const int c = cv * 4;
            const float4 mu = *reinterpret_cast<const float4*>(mean + c);
            const float4 vr = *reinterpret_cast<const float4*>(var + c);
            const float4 inv = make_float4(rsqrtf(vr.x + eps), rsqrtf(vr.y + eps), rsqrtf(vr.z + eps), rsqrtf(vr.w + eps));
            const float4 ga = *reinterpret_cast<const float4*>(gamma + c);
            const float4 be = *reinterpret_cast<const float4*>(beta + c);
            const float4* gp = reinterpret_cast<const float4*>(dpool) + cv;
            const float4* xp = reinterpret_cast<const float4*>(xsel) + cv;
#pragma unroll 4
            for (long long wdx = w0 + rl; wdx < w1; wdx += lanes) {
                const float4 g = __ldcs(gp + (size_t)wdx * CV);
                const float4 v = __ldcs(xp + (size_t)wdx * CV);
                const float hx = (v.x - mu.x) * inv.x, hy = (v.y - mu.y) * inv.y;
                const float hz = (v.z - mu.z) * inv.z, hw = (v.w - mu.w) * inv.w;
                const float gx = g.x * lrelu_grad(fmaf(ga.x, hx, be.x), alpha), gy = g.y * lrelu_grad(fmaf(ga.y, hy, be.y), alpha);
                const float gz = g.z * lrelu_grad(fmaf(ga.z, hz, be.z), alpha), gw = g.w * lrelu_grad(fmaf(ga.w, hw, be.w), alpha);
                a.x += gx; a.y += gy; a.z += gz; a.w += gw;
                b.x = fmaf(gx, hx, b.x); b.y = fmaf(gy, hy, b.y); b.z = fmaf(gz, hz, b.z); b.w = fmaf(gw, hw, b.w);
            }
        }
        sh_a4[threadIdx.x] = a;
        sh_b4[threadIdx.x] = b;
        __syncthreads();
        if (threadIdx.x < cols && cv < CV) {
            float* out = part + (size_t)blockIdx.x * 2 * C + cv * 4;
            const float* pa = reinterpret_cast<const float*>(sh_a4);
            const float* pb = reinterpret_cast<const float*>(sh_b4);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float sa = 0.f, sb = 0.f;
                for (int l = 0; l < lanes; ++l) {
                    sa += pa[(l * cols + threadIdx.x) * 4 + k];
                    sb += pb[(l * cols + threadIdx.x) * 4 + k];
                }
                out[k] = sa;
                out[C + k] = sb;
            }
        }
        __syncthreads();
    }
}

// Per-channel partial sums of g and g * xhat over a slab of windows: part[block][2][C].  Thread = (channel group,
// window lane) like bn_reduce_vec4_kernel; only the window's selected cell has a non-zero g.
__global__ void __launch_bounds__(256) bn_act_pool_bwd_reduce_kernel(
    const float* __restrict__ x, const float* __restrict__ dpool, const uint8_t* __restrict__ arg,
    const float* __restrict__ gamma, const float* __restrict__ beta, const float* __restrict__ mean,
    const float* __restrict__ var, float eps, float alpha, long long windows, long long win_per_block, int W, int C, int fH,
    int fW, int Wo, float* __restrict__ part) {
    const long long w0 = blockIdx.x * win_per_block;
    long long w1 = w0 + win_per_block;
    if (w1 > windows) w1 = windows;
    const int CV = C >> 2;
    const int cols = CV < 256 ? CV : 256;
    const int lanes = 256 / cols;
    __shared__ float4 sh_a4[256], sh_b4[256];
    for (int cbase = 0; cbase < CV; cbase += cols) {
        const int cv = cbase + threadIdx.x % cols;
        const int rl = threadIdx.x / cols;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
        if (rl < lanes && cv < CV) {
            const int c = cv * 4;
            const float4 mu = make_float4(mean[c], mean[c + 1], mean[c + 2], mean[c + 3]);
            const float4 inv = make_float4(rsqrtf(var[c] + eps), rsqrtf(var[c + 1] + eps), rsqrtf(var[c + 2] + eps),
                                           rsqrtf(var[c + 3] + eps));
            const float4 ga = *reinterpret_cast<const float4*>(gamma + c);
            const float4 be = *reinterpret_cast<const float4*>(beta + c);
            for (long long wdx = w0 + rl; wdx < w1; wdx += lanes) {
                const long long pix = wdx / Wo;                // s * Ho + ho
                const int wo = (int)(wdx - pix * Wo);
                const float4 g = (reinterpret_cast<const float4*>(dpool) + cv)[(size_t)wdx * CV];
                const uchar4 cd = (reinterpret_cast<const uchar4*>(arg) + cv)[(size_t)wdx * CV];
                const float4* in = reinterpret_cast<const float4*>(x) + ((size_t)pix * fH * W + (size_t)wo * fW) * CV + cv;
                // the selected cell of each of the four channels (window-local code = i * fW + j)
                const float4 vx = in[((size_t)(cd.x / fW) * W + cd.x % fW) * CV];
                const float4 vy = in[((size_t)(cd.y / fW) * W + cd.y % fW) * CV];
                const float4 vz = in[((size_t)(cd.z / fW) * W + cd.z % fW) * CV];
                const float4 vw = in[((size_t)(cd.w / fW) * W + cd.w % fW) * CV];
                const float hx = (vx.x - mu.x) * inv.x, hy = (vy.y - mu.y) * inv.y;
                const float hz = (vz.z - mu.z) * inv.z, hw = (vw.w - mu.w) * inv.w;
                const float gx = g.x * lrelu_grad(fmaf(ga.x, hx, be.x), alpha), gy = g.y * lrelu_grad(fmaf(ga.y, hy, be.y), alpha);
                const float gz = g.z * lrelu_grad(fmaf(ga.z, hz, be.z), alpha), gw = g.w * lrelu_grad(fmaf(ga.w, hw, be.w), alpha);
                a.x += gx; a.y += gy; a.z += gz; a.w += gw;
                b.x = fmaf(gx, hx, b.x); b.y = fmaf(gy, hy, b.y); b.z = fmaf(gz, hz, b.z); b.w = fmaf(gw, hw, b.w);
            }
        }
        sh_a4[threadIdx.x] = a;
        sh_b4[threadIdx.x] = b;
        __syncthreads();
        if (threadIdx.x < cols && cv < CV) {
            float* out = part + (size_t)blockIdx.x * 2 * C + cv * 4;
            const float* pa = reinterpret_cast<const float*>(sh_a4);
            const float* pb = reinterpret_cast<const float*>(sh_b4);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float sa = 0.f, sb = 0.f;
                for (int l = 0; l < lanes; ++l) {
                    sa += pa[(l * cols + threadIdx.x) * 4 + k];
                    sb += pb[(l * cols + threadIdx.x) * 4 + k];
                }
                out[k] = sa;
                out[C + k] = sb;
            }
        }
        __syncthreads();
    }
}

// dx = k1 * g + k2 * x + k3 for every cell of every window (g is non-zero only at the window's selected cell).
template <int F>
__global__ void __launch_bounds__(256) bn_act_pool_bwd_apply_kernel(
    const float* __restrict__ x, const float* __restrict__ dpool, const uint8_t* __restrict__ arg,
    const float* __restrict__ gamma, const float* __restrict__ beta, const float* __restrict__ mean,
    const float* __restrict__ var, float eps, float alpha, const float* __restrict__ coeff, float* __restrict__ dx,
    unsigned total, int W, int C, int fH_, int fW_, int Wo, __nv_bfloat16* __restrict__ copy, int copy_ld,
    float* __restrict__ colsum_part) {
    const int fH = F ? F : fH_, fW = F ? F : fW_;
    const int C4 = C >> 2;
    // column sums of dx (the bias gradient of the convolution in front): only with grids whose stride keeps a thread on
    // one channel group (gridDim.x * 256 a multiple of C4; the host checks), so four running sums per thread suffice
    float4 csum = make_float4(0.f, 0.f, 0.f, 0.f);
    for (unsigned idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
        const unsigned cv = idx % (unsigned)C4;
        unsigned pix = idx / (unsigned)C4;
        const unsigned wo = pix % (unsigned)Wo;
        pix /= (unsigned)Wo;
        const int c = cv * 4;
        const float4 g = __ldcs(reinterpret_cast<const float4*>(dpool) + idx);
        const uchar4 cd = reinterpret_cast<const uchar4*>(arg)[idx];
        const float4 k1 = *reinterpret_cast<const float4*>(coeff + c);
        const float4 k2 = *reinterpret_cast<const float4*>(coeff + C + c);
        const float4 k3 = *reinterpret_cast<const float4*>(coeff + 2 * C + c);
        const float4 mu = *reinterpret_cast<const float4*>(mean + c);
        const float4 vr = *reinterpret_cast<const float4*>(var + c);
        const float4 ga = *reinterpret_cast<const float4*>(gamma + c);
        const float4 be = *reinterpret_cast<const float4*>(beta + c);
        const float4 inv = make_float4(rsqrtf(vr.x + eps), rsqrtf(vr.y + eps), rsqrtf(vr.z + eps), rsqrtf(vr.w + eps));
        const size_t first = ((size_t)pix * fH * W + (size_t)wo * fW) * C4 + cv;
        float4 pre[F ? F * F : 1];
        if (F) {
#pragma unroll
            for (int k = 0; k < F * F; ++k)
                pre[k] = __ldcs(reinterpret_cast<const float4*>(x) + first + ((size_t)(k / (F ? F : 1)) * W + k % (F ? F : 1)) * C4);
        }
#pragma unroll
        for (int i = 0; i < fH; ++i)
#pragma unroll
            for (int j = 0; j < fW; ++j) {
                const size_t cell = first + ((size_t)i * W + j) * C4;
                const float4 v = F ? pre[F ? i * F + j : 0] : __ldcs(reinterpret_cast<const float4*>(x) + cell);
                const unsigned char k = (unsigned char)(i * fW + j);
                float4 o;
                o.x = fmaf(k2.x, v.x, k3.x); o.y = fmaf(k2.y, v.y, k3.y); o.z = fmaf(k2.z, v.z, k3.z); o.w = fmaf(k2.w, v.w, k3.w);
                if (cd.x == k) o.x = fmaf(k1.x, g.x * lrelu_grad(fmaf(ga.x, (v.x - mu.x) * inv.x, be.x), alpha), o.x);
                if (cd.y == k) o.y = fmaf(k1.y, g.y * lrelu_grad(fmaf(ga.y, (v.y - mu.y) * inv.y, be.y), alpha), o.y);
                if (cd.z == k) o.z = fmaf(k1.z, g.z * lrelu_grad(fmaf(ga.z, (v.z - mu.z) * inv.z, be.z), alpha), o.z);
                if (cd.w == k) o.w = fmaf(k1.w, g.w * lrelu_grad(fmaf(ga.w, (v.w - mu.w) * inv.w, be.w), alpha), o.w);
                if (dx != nullptr) reinterpret_cast<float4*>(dx)[cell] = o;   // not written when only the bf16 copy is wanted
                if (copy != nullptr) {
                    store_operand_copy(copy, copy_ld, (size_t)pix * fH * W + (size_t)wo * fW + (size_t)i * W + j, (int)cv, C4, o);
                    csum.x += o.x; csum.y += o.y; csum.z += o.z; csum.w += o.w;
                }
            }
    }
    if (colsum_part != nullptr) {
        // threads t, t + C4, ... of the block hold the same four channels: added in that order, one row per block
        __shared__ float4 red[256];
        red[threadIdx.x] = csum;
        __syncthreads();
        if ((int)threadIdx.x < C4) {
            float4 t = red[threadIdx.x];
            for (int l = threadIdx.x + C4; l < 256; l += C4) { const float4 v = red[l]; t.x += v.x; t.y += v.y; t.z += v.z; t.w += v.w; }
            *reinterpret_cast<float4*>(colsum_part + (size_t)blockIdx.x * C + threadIdx.x * 4) = t;
        }
    }
}

static int fused_blocks(long long items, int threads, int per_sm) {
    long long b = (items + threads - 1) / threads;
    const long long cap = 148LL * per_sm;
    if (b > cap) b = cap;
    return (int)(b < 1 ? 1 : b);
}

static int block_check(const char* who, int S, int H, int W, int C, int fH, int fW, float alpha, long long* windows4) {
    if (S <= 0 || H <= 0 || W <= 0 || C <= 0 || fH <= 0 || fW <= 0) return set_error(AE_BAD_ARG, "%s: non-positive dimension", who);
    if (C % 4 || H % fH || W % fW || fH * fW > 255)
        return set_error(AE_UNSUPPORTED, "%s: needs C %% 4 == 0 and pooling windows that tile the input (H=%d W=%d f=%dx%d C=%d)",
                         who, H, W, fH, fW, C);
    if (!(alpha >= 0.f && alpha < 1.f)) return set_error(AE_BAD_ARG, "%s: alpha must be in [0, 1)", who);
    *windows4 = 1LL * S * (H / fH) * (W / fW) * (C / 4);
    if (*windows4 >= (1LL << 32) - (1LL << 22)) return set_error(AE_UNSUPPORTED, "%s: tensor too large for 32-bit window indices", who);
    return AE_OK;
}

}  // namespace aether

using namespace aether;

extern "C" size_t aether_bn_workspace_bytes(int64_t rows, int C);

extern "C" int aether_bn_act_pool_fwd(const float* x, const float* partials, int64_t nblocks, const float* gamma,
                                      const float* beta, float* running_mean, float* running_var, float* batch_mean,
                                      float* batch_var, float* pooled, uint8_t* argmax, int S, int H, int W, int C, int fH,
                                      int fW, float eps, float momentum, float alpha, const float* channel_scale,
                                      int training, void* ws, size_t ws_bytes, void* stream) {
    return aether_bn_act_pool_fwd_copy(x, partials, nblocks, gamma, beta, running_mean, running_var, batch_mean, batch_var,
                                       pooled, argmax, S, H, W, C, fH, fW, eps, momentum, alpha, channel_scale, training,
                                       nullptr, 0, nullptr, ws, ws_bytes, stream);
}

extern "C" int aether_bn_act_pool_fwd_copy(const float* x, const float* partials, int64_t nblocks, const float* gamma,
                                           const float* beta, float* running_mean, float* running_var, float* batch_mean,
                                           float* batch_var, float* pooled, uint8_t* argmax, int S, int H, int W, int C,
                                           int fH, int fW, float eps, float momentum, float alpha,
                                           const float* channel_scale, int training, void* operand_copy, int copy_ld,
                                           float* selected_x, void* ws, size_t ws_bytes, void* stream) {
    if (!x || !gamma || !beta || !running_mean || !running_var || (!pooled && !operand_copy) || !argmax || !ws ||
        (training && (!batch_mean || !batch_var)))
        return set_error(AE_BAD_ARG, "aether_bn_act_pool_fwd: null pointer");
    if (operand_copy && (copy_ld < C || copy_ld % 4 || (reinterpret_cast<uintptr_t>(operand_copy) & 7)))
        return set_error(AE_BAD_ARG, "aether_bn_act_pool_fwd_copy: operand copy needs ld >= C, ld %% 4 == 0, 8-byte alignment");
    if (selected_x && !aligned16(selected_x)) return set_error(AE_BAD_ARG, "aether_bn_act_pool_fwd_copy: selected_x must be 16-byte aligned");
    long long windows4 = 0;
    int rc = block_check("aether_bn_act_pool_fwd", S, H, W, C, fH, fW, alpha, &windows4);
    if (rc) return rc;
    if (!aligned16(x) || (pooled && !aligned16(pooled)) || !aligned16(ws) || (reinterpret_cast<uintptr_t>(argmax) & 3))
        return set_error(AE_BAD_ARG, "aether_bn_act_pool_fwd: arrays must be 16-byte aligned (argmax: 4)");
    const long long rows = 1LL * S * H * W;
    if (ws_bytes < aether_bn_workspace_bytes(rows, C)) return set_error(AE_BAD_ARG, "aether_bn_act_pool_fwd: workspace too small");
    if (partials && (nblocks <= 0 || nblocks > (1 << 30))) return set_error(AE_BAD_ARG, "aether_bn_act_pool_fwd: nblocks");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    float* coeff = training ? bn_forward_coeffs(x, partials, nblocks, gamma, beta, running_mean, running_var, batch_mean,
                                                batch_var, rows, C, eps, momentum, channel_scale, static_cast<float*>(ws), st)
                            : bn_eval_coeffs(gamma, beta, running_mean, running_var, C, eps, static_cast<float*>(ws), st);
    const int fb = fused_blocks(windows4, 256, 16);
    __nv_bfloat16* copy = static_cast<__nv_bfloat16*>(operand_copy);
    if (fH == 2 && fW == 2)
        bn_act_pool_fwd_kernel<2><<<fb, 256, 0, st>>>(x, coeff, coeff + C, alpha, pooled, argmax, (unsigned)windows4, W, C / 4,
                                                     fH, fW, W / fW, copy, copy_ld, selected_x);
    else
        bn_act_pool_fwd_kernel<0><<<fb, 256, 0, st>>>(x, coeff, coeff + C, alpha, pooled, argmax, (unsigned)windows4, W, C / 4,
                                                     fH, fW, W / fW, copy, copy_ld, selected_x);
    count_launch();
    return check_launch("aether_bn_act_pool_fwd");
}

extern "C" int aether_bn_act_pool_bwd(const float* x, const float* dpooled, const uint8_t* argmax, const float* gamma,
                                      const float* beta, const float* batch_mean, const float* batch_var, float* dx,
                                      float* dgamma, float* dbeta, int S, int H, int W, int C, int fH, int fW, float eps,
                                      float alpha, const float* channel_scale, void* ws, size_t ws_bytes, void* stream) {
    return aether_bn_act_pool_bwd_copy(x, dpooled, argmax, gamma, beta, batch_mean, batch_var, dx, dgamma, dbeta, S, H, W, C, fH,
                                       fW, eps, alpha, channel_scale, nullptr, 0, nullptr, 0, nullptr, nullptr, ws, ws_bytes, stream);
}

extern "C" int aether_bn_act_pool_bwd_copy(const float* x, const float* dpooled, const uint8_t* argmax, const float* gamma,
                                           const float* beta, const float* batch_mean, const float* batch_var, float* dx,
                                           float* dgamma, float* dbeta, int S, int H, int W, int C, int fH, int fW, float eps,
                                           float alpha, const float* channel_scale, void* operand_copy, int copy_ld,
                                           float* colsum_part, int colsum_rows_max, int* colsum_rows,
                                           const float* selected_x, void* ws, size_t ws_bytes, void* stream) {
    if (!x || !dpooled || !argmax || !gamma || !beta || !batch_mean || !batch_var || (!dx && !operand_copy) || !dgamma ||
        !dbeta || !ws)
        return set_error(AE_BAD_ARG, "aether_bn_act_pool_bwd: null pointer");
    if (operand_copy) {
        if (copy_ld < C || copy_ld % 4 || (reinterpret_cast<uintptr_t>(operand_copy) & 7) || !colsum_part || !colsum_rows ||
            colsum_rows_max < 1 || !aligned16(colsum_part))
            return set_error(AE_BAD_ARG, "aether_bn_act_pool_bwd_copy: operand copy needs ld >= C, ld %% 4 == 0, 8-byte alignment "
                                         "and a column-sum buffer");
        if (256 % (C / 4 > 0 ? C / 4 : 1) || C / 4 > 256)
            return set_error(AE_UNSUPPORTED, "aether_bn_act_pool_bwd_copy: the column sums need C / 4 to divide 256 (C = %d)", C);
    }
    long long windows4 = 0;
    int rc = block_check("aether_bn_act_pool_bwd", S, H, W, C, fH, fW, alpha, &windows4);
    if (rc) return rc;
    if (!aligned16(x) || !aligned16(dpooled) || (dx && !aligned16(dx)) || !aligned16(ws) || !aligned16(gamma) || !aligned16(beta) ||
        !aligned16(batch_mean) || !aligned16(batch_var) || (reinterpret_cast<uintptr_t>(argmax) & 3))
        return set_error(AE_BAD_ARG, "aether_bn_act_pool_bwd: arrays must be 16-byte aligned (argmax: 4)");
    const long long rows = 1LL * S * H * W;
    if (ws_bytes < aether_bn_workspace_bytes(rows, C)) return set_error(AE_BAD_ARG, "aether_bn_act_pool_bwd: workspace too small");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const long long windows = windows4 / (C / 4);
    int nb = bn_partial_blocks(rows);
    if (nb > windows) nb = (int)windows;
    float* part = static_cast<float*>(ws);
    float* coeff = part + (size_t)bn_partial_blocks(rows) * 3 * C;
    if (selected_x) {
        if (!aligned16(selected_x)) return set_error(AE_BAD_ARG, "aether_bn_act_pool_bwd_copy: selected_x must be 16-byte aligned");
        bn_act_pool_bwd_reduce_sel_kernel<<<nb, 256, 0, st>>>(selected_x, dpooled, gamma, beta, batch_mean, batch_var, eps, alpha,
                                                              windows, (windows + nb - 1) / nb, C, part);
    } else {
        bn_act_pool_bwd_reduce_kernel<<<nb, 256, 0, st>>>(x, dpooled, argmax, gamma, beta, batch_mean, batch_var, eps, alpha, windows,
                                                          (windows + nb - 1) / nb, W, C, fH, fW, W / fW, part);
    }
    count_launch();
    bn_backward_coeffs(part, nb, C, rows, gamma, batch_mean, batch_var, eps, dgamma, dbeta, coeff, channel_scale, st);
    int fb = fused_blocks(windows4, 256, 16);
    __nv_bfloat16* copy = static_cast<__nv_bfloat16*>(operand_copy);
    if (copy) {                                  // one row of column sums per CTA: no more CTAs than rows offered
        if (fb > colsum_rows_max) fb = colsum_rows_max;
        *colsum_rows = fb;
    }
    if (fH == 2 && fW == 2)
        bn_act_pool_bwd_apply_kernel<2><<<fb, 256, 0, st>>>(x, dpooled, argmax, gamma, beta, batch_mean, batch_var, eps, alpha,
                                                           coeff, dx, (unsigned)windows4, W, C, fH, fW, W / fW, copy, copy_ld,
                                                           copy ? colsum_part : nullptr);
    else
        bn_act_pool_bwd_apply_kernel<0><<<fb, 256, 0, st>>>(x, dpooled, argmax, gamma, beta, batch_mean, batch_var, eps, alpha,
                                                           coeff, dx, (unsigned)windows4, W, C, fH, fW, W / fW, copy, copy_ld,
                                                           copy ? colsum_part : nullptr);
    count_launch();
    return check_launch("aether_bn_act_pool_bwd");
}
