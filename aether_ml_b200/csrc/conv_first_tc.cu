// First-layer convolution (1..4 input channels, K = fH*fW*Cin <= 64) on the tensor cores, bf16 mode.
//
//   y[p][d] = b[d] + sum_k col[p][k] * w[k][d]            (Conv_Layer.forward, CNN_classes_cupy.py:70-120)
//
// With 3 input channels a pixel's 12 bytes cannot be the inner extent of a TMA box and K = 27 is less than one
// 128-byte operand row, so the im2col rows are built by threads: four producer warps gather the K input values of
// 128 output pixels (one pixel per thread), convert them to bf16 and write them as a K-major, 128-byte-swizzled
// operand tile (16-byte chunk c of row r is stored at chunk c ^ (r % 8)); the filter is laid out the same way once
// per CTA.  One warp issues K/16 (two for a 3x3 RGB filter) 128 x Cout x 16 MMAs per tile into one of up to four
// TMEM accumulators; eight epilogue warps add the bias and write 64-byte row segments straight from registers, and
// optionally accumulate the per-channel statistics the following Batch_Norm needs.  The layer is bound by the HBM
// write of its output (the CUDA-core version of the same layer, conv_smallc.cu, is bound by its FMAs).
#include <cuda_bf16.h>
#include <string.h>

#include "common.cuh"
#include "sm100_ptx.cuh"
#include "stats_epilogue.cuh"
#include "tc_host.cuh"
#include "tc_host.cuh"

namespace aether {

struct FirstParams {
    const float* x;
    const float* w;      // (fH, fW, Cin, Cout) = [K][Cout]
    const float* bias;   // nullable
    float* y;
    float* stats;        // nullable: [cta][4][3][Cout] (count, mean, M2) partials
    int* status;
    int H, W, Cin, Cout, NT, fH, fW, sH, sW, pH, pW, Ho, Wo, K, KP;
    long long P;         // output pixels
    int stages, ntiles;
};

// Producer warps: about two threads per pixel -- a lone producer warp per scheduler cannot hide the gather latency.
// The kernel with the statistics epilogue runs 7 of them: 16 warps are four per scheduler and 128 registers per thread,
// 17 warps put five on one scheduler and cap every thread at 96, which the statistics' running sums do not fit in.
static constexpr int FT_EPI_WARPS = 8;
template <bool STATS> struct FirstCfg {
    static constexpr int PROD_WARPS = STATS ? 7 : 8;
    static constexpr int THREADS = 32 * (PROD_WARPS + 1 + FT_EPI_WARPS);   // producers, MMA issuer, epilogue
};
static constexpr int FT_STAGE_BYTES = 128 * 128;                             // 128 pixel rows of 128 bytes
static constexpr int FT_TAIL = 2048;                                         // barriers, TMEM pointer, bias, k tables
static constexpr int FT_STATS_BYTES = FT_EPI_WARPS * STATS_WARP_FLOATS * 4;

__device__ __forceinline__ void ft_umma(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t hi, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %5, 0;\n\tmov.b64 da, {%1, %4};\n\tmov.b64 db, {%2, %4};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(hi), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&v);
}

template <bool STATS>
__global__ void __launch_bounds__(FirstCfg<STATS>::THREADS, 1) first_conv_kernel(const __grid_constant__ FirstParams p) {
    constexpr int FT_PROD_WARPS = FirstCfg<STATS>::PROD_WARPS;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (smem_base - smem_u32(smem_raw));
    const int NT = p.NT, S = p.stages;
    const uint32_t sW = smem_base;                                  // filter: NT rows of 128 bytes
    const uint32_t sA = sW + (uint32_t)NT * 128u;                   // NT is a multiple of 64: stays 1024-byte aligned
    const uint32_t sBar = sA + (uint32_t)S * FT_STAGE_BYTES;
    auto full_bar = [&](int s) { return sBar + 8u * s; };
    auto empty_bar = [&](int s) { return sBar + 8u * (S + s); };
    auto tfull_bar = [&](int b) { return sBar + 8u * (2 * S + b); };
    auto tempty_bar = [&](int b) { return sBar + 8u * (2 * S + 4 + b); };
    const uint32_t sTmemPtr = sBar + 8u * (2 * S + 8);
    volatile uint32_t* tmem_ptr_generic = reinterpret_cast<volatile uint32_t*>(gen_base + (sTmemPtr - smem_base));
    float* bias_s = reinterpret_cast<float*>(gen_base + (sBar - smem_base) + 256);         // NT <= 256 floats
    int* koff_s = reinterpret_cast<int*>(gen_base + (sBar - smem_base) + 256 + 1024);      // K <= 64 entries each
    int* ki_s = koff_s + 64;
    int* kj_s = ki_s + 64;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t NB = (4 * NT <= 512) ? 4u : (3 * NT <= 512) ? 3u : 2u;
    const uint32_t need_cols = NB * (uint32_t)NT;
    const uint32_t tmem_cols = (need_cols <= 32) ? 32u : (need_cols <= 64) ? 64u : (need_cols <= 128) ? 128u : (need_cols <= 256) ? 256u : 512u;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(full_bar(s), 32 * FT_PROD_WARPS);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 4; ++b) {
            mbar_init(tfull_bar(b), 1);
            mbar_init(tempty_bar(b), FT_EPI_WARPS);
        }
        mbar_fence_init();
    }
    for (int i = threadIdx.x; i < NT; i += blockDim.x) bias_s[i] = (p.bias != nullptr && i < p.Cout) ? p.bias[i] : 0.f;
    for (int k = threadIdx.x; k < 64; k += blockDim.x) {
        const int kk = k < p.K ? k : 0;
        const int tap = kk / p.Cin, c = kk - tap * p.Cin;
        const int i = tap / p.fW, j = tap - i * p.fW;
        ki_s[k] = k < p.K ? i : (1 << 20);                         // entries past K fail the bounds test: zero
        kj_s[k] = j;
        koff_s[k] = (i * p.W + j) * p.Cin + c;
    }
    // filter operand: row n = output channel, element k at byte (k/8 ^ n%8)*16 + (k%8)*2 of the row
    for (int it = threadIdx.x; it < NT * (p.KP >> 3); it += blockDim.x) {
        const int n = it / (p.KP >> 3), ch = it - n * (p.KP >> 3);
        float v[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const int k = ch * 8 + e;
            v[e] = (n < p.Cout && k < p.K) ? p.w[(size_t)k * p.Cout + n] : 0.f;
        }
        const uint4 q = make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
        *reinterpret_cast<uint4*>(gen_base + (sW - smem_base) + n * 128 + ((ch ^ (n & 7)) << 4)) = q;
    }
    fence_proxy_async_smem();
    if (warp == FT_PROD_WARPS) {
        tmem_alloc(sTmemPtr, tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr_generic;
    const int grid = (int)gridDim.x;

    if (warp < FT_PROD_WARPS) {
        // ------------------------------------------------------------------ producers
        // A tile is 128 rows x (KP / 8) 16-byte chunks; the producer threads take the (row, chunk) pairs round robin.
        constexpr int NPT = 32 * FT_PROD_WARPS;
        uint8_t* tile_gen = gen_base + (sA - smem_base);
        const int ntasks = (p.KP >> 3) << 7;
        const long long HoWo = (long long)p.Ho * p.Wo;
        int s = 0;
        uint32_t ph = 0;
        for (int t = blockIdx.x; t < p.ntiles; t += grid) {
            if (!mbar_wait(empty_bar(s), ph ^ 1u, p.status, DS_TIMEOUT_EMPTY)) break;
            uint8_t* stage_gen = tile_gen + s * FT_STAGE_BYTES;
            int r_prev = -1, h0 = 0, w0 = 0;
            long long base = 0;
            for (int task = threadIdx.x; task < ntasks; task += NPT) {
                const int r = task & 127, ch = task >> 7;
                if (r != r_prev) {                                  // with 256 producer threads: once per thread and tile
                    r_prev = r;
                    const long long pix = (long long)t * 128 + r;
                    h0 = -(1 << 20); w0 = 0; base = 0;
                    if (pix < p.P) {
                        const long long n = pix / HoWo;
                        const int rem = (int)(pix - n * HoWo);
                        const int ho = rem / p.Wo, wo = rem - ho * p.Wo;
                        h0 = ho * p.sH - p.pH;
                        w0 = wo * p.sW - p.pW;
                        base = ((n * p.H + h0) * p.W + w0) * p.Cin;  // may point before the image: only used with valid taps
                    }
                }
                float v[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const int k = ch * 8 + e;
                    const int hi = h0 + ki_s[k], wi = w0 + kj_s[k];
                    v[e] = (hi >= 0 && hi < p.H && wi >= 0 && wi < p.W) ? __ldg(p.x + base + koff_s[k]) : 0.f;
                }
                const uint4 q = make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
                *reinterpret_cast<uint4*>(stage_gen + r * 128 + ((ch ^ (r & 7)) << 4)) = q;
            }
            fence_proxy_async_smem();                               // generic-proxy writes -> visible to the tensor core
            mbar_arrive(full_bar(s));
            if (++s == S) { s = 0; ph ^= 1u; }
        }
    } else if (warp == FT_PROD_WARPS) {
        // ------------------------------------------------------------------ MMA issuer
        const bool leader = elect_one();
        const uint32_t idesc = make_idesc(1u, 0u, 0u, 128u, (uint32_t)NT);
        const uint64_t proto = make_smem_desc(0, 16, 1024);
        const uint32_t hi = (uint32_t)(proto >> 32);
        const uint32_t lo_proto = (uint32_t)proto;
        const uint32_t w_lo = lo_proto + ((sW & 0x3FFFFu) >> 4);
        const uint32_t a_lo0 = lo_proto + ((sA & 0x3FFFFu) >> 4);
        const int ksteps = p.KP >> 4;
        int s = 0;
        uint32_t ph = 0, buf = 0, aph = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < p.ntiles && ok; t += grid) {
            bool w_ok = mbar_wait_spin(tempty_bar(buf), aph ^ 1u, p.status, DS_TIMEOUT_TMEM_EMPTY);
            w_ok = __all_sync(0xffffffffu, w_ok);
            if (!w_ok) { ok = false; break; }
            bool f_ok = mbar_wait_spin(full_bar(s), ph, p.status, DS_TIMEOUT_FULL);
            f_ok = __all_sync(0xffffffffu, f_ok);
            if (!f_ok) { ok = false; break; }
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + buf * NT;
            const uint32_t a_lo = a_lo0 + (uint32_t)s * (FT_STAGE_BYTES >> 4);
            if (leader) {
                for (int ks = 0; ks < ksteps; ++ks) ft_umma(d_tmem, a_lo + 2u * ks, w_lo + 2u * ks, hi, idesc, ks ? 1u : 0u);
                umma_commit(empty_bar(s));
                umma_commit(tfull_bar(buf));
            }
            if (++s == S) { s = 0; ph ^= 1u; }
            if (++buf == NB) { buf = 0; aph ^= 1u; }
            __syncwarp();
        }
    } else {
        // ------------------------------------------------------------------ epilogue (same scheme as conv_halo.cu)
        const int ew = warp - FT_PROD_WARPS - 1;
        const int q = warp & 3;                                      // TMEM lane quarter this warp may access
        const int half = ew >> 2;
        const int ncols = NT >> 1;
        const int col_begin = half * ncols;
        const int trow = lane >> 2, tcol4 = (lane & 3) * 4;
        const bool lo2 = (lane & 2) == 0, odd = (lane & 1) != 0;
        const bool all_cols = (p.Cout == NT);
        float* stat_w = reinterpret_cast<float*>(gen_base + (sBar - smem_base) + FT_TAIL) + ew * STATS_WARP_FLOATS;
        float st_rows = 0.f;
        if (STATS) {
            for (int i = lane; i < STATS_WARP_FLOATS; i += 32) stat_w[i] = 0.f;
            __syncwarp();
        }
        int row_in_tile[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) row_in_tile[j] = q * 32 + (j >> 1) * 16 + trow + (j & 1) * 8;
        const float* bias4 = bias_s + col_begin + tcol4;
        const f32x2 one2 = pack2(1.f, 1.f);
        // Statistics: per-thread sums of its (4 rows x 4 columns) cells per 16-column group.  With one column batch
        // per tile (ncols <= 64) they run over all tiles of the CTA and the lanes are combined once at the end --
        // the epilogue is this kernel's critical path, and a per-tile lane reduction doubles its length.
        const bool persist = ncols <= 64;
        Stats4 st[4];                              // packed running sums of this thread's four 16-column groups
#pragma unroll
        for (int u = 0; u < 4; ++u) st[u].clear();
        // adds the lanes with equal lane%4 (same 4 columns, 8 row groups) and accumulates into the warp's sums
        // (about the columns' pivots, see stats_epilogue.cuh; `first`: the sums are the warp's first tile, taken
        // without pivots, which are set from them)
        auto flush_stats = [&](int cb, bool first, float rows) {
            float4 st_s[4], st_q[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) { st_s[u] = st[u].sum(); st_q[u] = st[u].sumsq(); }
#pragma unroll
            for (int m = 4; m <= 16; m <<= 1) {
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    st_s[u].x += __shfl_xor_sync(0xffffffffu, st_s[u].x, m); st_s[u].y += __shfl_xor_sync(0xffffffffu, st_s[u].y, m);
                    st_s[u].z += __shfl_xor_sync(0xffffffffu, st_s[u].z, m); st_s[u].w += __shfl_xor_sync(0xffffffffu, st_s[u].w, m);
                    st_q[u].x += __shfl_xor_sync(0xffffffffu, st_q[u].x, m); st_q[u].y += __shfl_xor_sync(0xffffffffu, st_q[u].y, m);
                    st_q[u].z += __shfl_xor_sync(0xffffffffu, st_q[u].z, m); st_q[u].w += __shfl_xor_sync(0xffffffffu, st_q[u].w, m);
                }
            }
            if (lane < 4) {
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int cc = cb + u * 16;
                    if (cc < ncols) stats_fold(stat_w, cc + tcol4, st_s[u], st_q[u], first, rows);
                }
            }
            if (first) __syncwarp();               // the pivots must be visible to the whole warp before its next tile
        };
        uint32_t buf = 0, aph = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < p.ntiles && ok; t += grid) {
            float* rowp[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const long long pix = (long long)t * 128 + row_in_tile[j];
                rowp[j] = pix < p.P ? p.y + (size_t)pix * p.Cout + col_begin + tcol4 : nullptr;
            }
            float tile_rows = 0.f;                 // valid rows of this tile in this warp's quarter
            if (STATS) {
#pragma unroll
                for (int j = 0; j < 4; ++j) tile_rows += (rowp[j] != nullptr) ? 1.f : 0.f;
                tile_rows += __shfl_xor_sync(0xffffffffu, tile_rows, 4);
                tile_rows += __shfl_xor_sync(0xffffffffu, tile_rows, 8);
                tile_rows += __shfl_xor_sync(0xffffffffu, tile_rows, 16);
            }
            const bool first_stats = STATS && st_rows == 0.f && tile_rows > 0.f;      // the tile that sets the pivots
            if (!mbar_wait(tfull_bar(buf), aph, p.status, DS_TIMEOUT_TMEM_FULL)) { ok = false; break; }
            tc_fence_after();
            const uint32_t taddr0 = tmem_base + ((uint32_t)(q * 32) << 16) + buf * NT + col_begin;
#pragma unroll 1
            for (int cb0 = 0; cb0 < ncols; cb0 += 64) {
                if (STATS && !persist) {
#pragma unroll
                    for (int u = 0; u < 4; ++u) st[u].clear();
                }
                // two half batches of 2 x 16 columns: 32 accumulator registers in flight beside the running sums
#pragma unroll
                for (int hb = 0; hb < 2; ++hb) {
                    const int cb = cb0 + hb * 32;
                    if (cb >= ncols) break;
                    uint32_t v[2][2][8];
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        if (cb + u * 16 < ncols) {
                            tmem_ld_16x256b_x2(taddr0 + cb + u * 16, v[0][u]);
                            tmem_ld_16x256b_x2(taddr0 + (16u << 16) + cb + u * 16, v[1][u]);
                        }
                    }
                    tmem_ld_wait();
                    if (cb + 32 >= ncols) {                       // accumulator fully read by this warp
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(tempty_bar(buf));
                    }
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        if (cb + u * 16 < ncols) {
                            const int cc = cb + u * 16;
                            const int g = hb * 2 + u;             // 16-column group within the 64-column batch
                            const float4 b4 = *reinterpret_cast<const float4*>(bias4 + cc);
                            const bool cols_ok = all_cols || col_begin + tcol4 + cc < p.Cout;
                            f32x2 npv01 = 0ull, npv23 = 0ull;             // minus the pivots of this lane's four columns
                            if (STATS) {
                                const float4 pv = *reinterpret_cast<const float4*>(stat_w + 256 + cc + tcol4);
                                npv01 = pack2(-pv.x, -pv.y);
                                npv23 = pack2(-pv.z, -pv.w);
                            }
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                // quad exchange: 2+2 columns per lane -> 4 consecutive columns per lane (64-byte row segments)
                                const uint32_t a0 = v[j >> 1][u][(j & 1) * 2 + 0], a1 = v[j >> 1][u][(j & 1) * 2 + 1];
                                const uint32_t b0 = v[j >> 1][u][4 + (j & 1) * 2 + 0], b1 = v[j >> 1][u][4 + (j & 1) * 2 + 1];
                                const uint32_t s0 = lo2 ? b0 : a0, s1 = lo2 ? b1 : a1;
                                const uint32_t r0 = __shfl_xor_sync(0xffffffffu, s0, 2), r1 = __shfl_xor_sync(0xffffffffu, s1, 2);
                                const uint32_t x0 = lo2 ? a0 : r0, x1 = lo2 ? a1 : r1;
                                const uint32_t y0 = lo2 ? r0 : b0, y1 = lo2 ? r1 : b1;
                                const uint32_t t0 = odd ? x0 : y0, t1 = odd ? x1 : y1;
                                const uint32_t q0 = __shfl_xor_sync(0xffffffffu, t0, 1), q1 = __shfl_xor_sync(0xffffffffu, t1, 1);
                                float4 a;
                                a.x = __uint_as_float(odd ? q0 : x0);
                                a.y = __uint_as_float(odd ? q1 : x1);
                                a.z = __uint_as_float(odd ? y0 : q0);
                                a.w = __uint_as_float(odd ? y1 : q1);
                                const bool wr = cols_ok && rowp[j] != nullptr;
                                if (wr)
                                    __stcs(reinterpret_cast<float4*>(rowp[j] + cc),
                                           make_float4(a.x + b4.x, a.y + b4.y, a.z + b4.z, a.w + b4.w));
                                if (STATS) {
                                    // rows past the last pixel hold zeros (their operand rows are zero): a product with
                                    // the row's 0/1 factor removes them from the sums
                                    const f32x2 m2 = (cols_ok && rowp[j] != nullptr) ? one2 : 0ull;
                                    st[g].add(mul2(add2(pack2(a.x, a.y), npv01), m2), mul2(add2(pack2(a.z, a.w), npv23), m2));
                                }
                            }
                        }
                    }
                }
                if (STATS) {
                    // the first tile is always folded at once (it sets the pivots); with running per-thread sums the
                    // other tiles are folded together after the last one
                    if (!persist || first_stats) {
                        flush_stats(cb0, first_stats, tile_rows);
                        if (persist) {
#pragma unroll
                            for (int u = 0; u < 4; ++u) st[u].clear();
                        }
                    }
                }
            }
            st_rows += tile_rows;
            if (++buf == NB) { buf = 0; aph ^= 1u; }
        }
        if (STATS && persist) flush_stats(0, false, 0.f);
        if (STATS && lane < 4) {
            float* sp = p.stats + ((size_t)blockIdx.x * 4 + q) * 3 * (size_t)p.Cout;
            for (int cc = 0; cc < ncols; cc += 16) {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int col = col_begin + tcol4 + cc + k;
                    if (col < p.Cout) {
                        float m, m2;
                        stats_result(stat_w, cc + tcol4 + k, st_rows, m, m2);
                        sp[col] = st_rows;
                        sp[p.Cout + col] = m + bias_s[col];
                        sp[2 * p.Cout + col] = m2;
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == FT_PROD_WARPS) {
        tc_fence_after();
        tmem_dealloc(tmem_base, tmem_cols);
    }
}

// ====================================================================================== filter / bias gradient
//   dw[k][d] = sum_p col[p][k] * dy[p][d],  db[d] = sum_p dy[p][d]            (Conv_Layer.backward, :132-134)
// as D[d][k] += dy^T[d][pixels] * col[pixels][k]: M = 128 output channels (two 64-channel chunks of an MN-major
// operand), N = K padded to 16, reduction over the 128 pixels of a tile in eight K=16 steps.  The producers build
// both operands: the col tile exactly as in the forward kernel (the same bytes serve as an MN-major B operand) and
// the dy tile converted from fp32 to bf16; they also keep the fp32 column sums of dy for db.  The accumulators stay
// in TMEM for the CTA's whole life; one partial per CTA, summed in fixed order by smallc_reduce_kernel.
struct FirstDwParams {
    const float* x;
    const float* dy;
    float* part;         // [cta][K + 1][Cout]
    int* status;
    int H, W, Cin, Cout, fH, fW, sH, sW, pH, pW, Ho, Wo, K, KP;
    int dblocks;         // 128-channel blocks of dy
    long long P;
    int stages, ntiles, stage_bytes;
    int groups;          // producer groups (divides FD_NP; <= stages)
    // dy handed in as a bf16 copy [P][dy_ld] by the kernel that produced it (aether_conv2d_operand_layout): TMA brings
    // the tile in already in operand form, the producers only gather the col tile, and dB comes from the column sums
    // that arrived with the copy
    CUtensorMap tm_dy;   // (dy_ld, P), box (64 channels, 128 pixels), 128-byte swizzle
    int dy_bf16;
};

// Twelve producer warps: with one producer warp per scheduler every round of dy loads costs a full HBM round trip
// and the kernel ran at a third of the HBM rate; 384 threads cover a 128-pixel tile of dy in one or two rounds.
static constexpr int FD_PROD_WARPS = 12;
static constexpr int FD_NP = 32 * FD_PROD_WARPS;
// Producer groups, each building every groups-th tile.  At most as many groups as operand stages: a group that
// could run two phases ahead of a stage's barrier would pass its parity wait early.
static constexpr int FD_MAX_GROUPS = 3;
static constexpr int FD_ROWS = 6;                                            // dy rows per thread and round
static constexpr int FD_TAIL = 1024 + FD_NP * 8 * 4 + 1024;                  // barriers, k tables, dB staging
static constexpr int FD_THREADS = 32 * (FD_PROD_WARPS + 1 + 4);              // producers, MMA issuer, 4 epilogue warps

__global__ void __launch_bounds__(FD_THREADS, 1) first_dw_kernel(const __grid_constant__ FirstDwParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (smem_base - smem_u32(smem_raw));
    const int S = p.stages;
    const uint32_t sBar = smem_base + (uint32_t)S * p.stage_bytes;           // stage: col tile, then 2*dblocks dy chunks
    auto full_bar = [&](int s) { return sBar + 8u * s; };
    auto empty_bar = [&](int s) { return sBar + 8u * (S + s); };
    const uint32_t done_bar = sBar + 8u * (2 * S);
    const uint32_t sTmemPtr = sBar + 8u * (2 * S + 1);
    volatile uint32_t* tmem_ptr_generic = reinterpret_cast<volatile uint32_t*>(gen_base + (sTmemPtr - smem_base));
    int* koff_s = reinterpret_cast<int*>(gen_base + (sBar - smem_base) + 256);
    int* ki_s = koff_s + 64;
    int* kj_s = ki_s + 64;
    float* dbsum_s = reinterpret_cast<float*>(gen_base + (sBar - smem_base) + 1024);      // [producer threads][8]

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t tmem_cols = 128;                                          // dblocks (<= 2) x KP (<= 64) columns

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(full_bar(s), FD_NP / p.groups + (p.dy_bf16 ? 1 : 0));    // + the thread that posts the TMA bytes
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(done_bar, 1);
        mbar_fence_init();
        if (p.dy_bf16) tma_prefetch_desc(&p.tm_dy);
    }
    for (int k = threadIdx.x; k < 64; k += blockDim.x) {
        const int kk = k < p.K ? k : 0;
        const int tap = kk / p.Cin, c = kk - tap * p.Cin;
        const int i = tap / p.fW, j = tap - i * p.fW;
        ki_s[k] = k < p.K ? i : (1 << 20);
        kj_s[k] = j;
        koff_s[k] = (i * p.W + j) * p.Cin + c;
    }
    if (warp == FD_PROD_WARPS) {
        tmem_alloc(sTmemPtr, tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr_generic;
    const int grid = (int)gridDim.x;
    const bool any = (int)blockIdx.x < p.ntiles;

    if (warp < FD_PROD_WARPS) {
        // ------------------------------------------------------------------ producers
        // Groups of warps build alternate tiles: while one group converts and gathers, the other groups' dy loads are
        // in flight (all twelve warps in lock step left the HBM pipe idle for two thirds of every tile).
        const int r = threadIdx.x;                                   // 0 .. FD_NP-1
        const int FD_GRP = FD_NP / p.groups;
        const int grp = r / FD_GRP, rg = r - grp * FD_GRP;
        const int chunks = p.KP >> 3;
        const int col_items = 128 * chunks;                          // item -> pixel = item % 128, 16-byte chunk = item / 128
        const int C8 = p.Cout >> 3;                                  // 8-channel chunks of a dy row (power of two <= 32)
        const int my_chunk = rg & (C8 - 1);                          // fixed for this thread: FD_GRP % C8 == 0
        const int prow0 = rg / C8, prow_step = FD_GRP / C8;
        const int dchunks = p.dblocks * 16;                          // 8-channel chunks the operand holds (zero padded)
        const long long HoWo = (long long)p.Ho * p.Wo;
        float bs[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) bs[e] = 0.f;
        if (C8 < dchunks) {
            // fewer than 128 channels: the chunks past Cout of the M = 128 operand are zero and stay zero (nobody
            // writes them again); published to the tensor core before any producer arrives on a stage
            for (int i = r; i < S * p.stage_bytes / 16; i += FD_NP)
                reinterpret_cast<uint4*>(gen_base)[i] = make_uint4(0, 0, 0, 0);
            fence_proxy_async_smem();
            named_bar_sync(1, FD_NP);
        }
        int k = grp;                                                 // index of the tile among this CTA's tiles
        for (int t = blockIdx.x + grp * grid; t < p.ntiles; t += p.groups * grid, k += p.groups) {
            const int s = k % S;
            const uint32_t ph = (uint32_t)(k / S) & 1u;
            const long long pix0 = (long long)t * 128;
            if (!mbar_wait(empty_bar(s), ph ^ 1u, p.status, DS_TIMEOUT_EMPTY)) break;
            uint8_t* stage = gen_base + (size_t)s * p.stage_bytes;
            // dy tile first (the long-latency loads): rows = pixels, 64-channel chunks of 128 bytes; chunk region c64
            // starts at 16 KB * (1 + c64).  All loads of a round are issued before the first use.
            uint8_t* reg = stage + FT_STAGE_BYTES * (1 + (my_chunk >> 3));
            if (p.dy_bf16 && rg == 0) {
                // the tile of the bf16 copy: one box per 64-channel chunk, rows past the last pixel are zero filled
                const int real_chunks = (p.Cout + 63) >> 6;
                mbar_arrive_expect_tx(full_bar(s), (uint32_t)real_chunks * FT_STAGE_BYTES);
                for (int c64 = 0; c64 < real_chunks; ++c64)
                    tma_load_2d(smem_base + (uint32_t)s * p.stage_bytes + FT_STAGE_BYTES * (1 + c64), &p.tm_dy, full_bar(s),
                                c64 * 64, (int)pix0);
            }
            for (int pr0 = prow0; pr0 < 128 && !p.dy_bf16; pr0 += FD_ROWS * prow_step) {
                float4 a[FD_ROWS], b[FD_ROWS];
#pragma unroll
                for (int u = 0; u < FD_ROWS; ++u) {
                    const int pr = pr0 + u * prow_step;
                    const long long pp = pix0 + pr;
                    a[u] = b[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (pr < 128 && pp < p.P) {
                        const float4* src = reinterpret_cast<const float4*>(p.dy + (size_t)pp * p.Cout + my_chunk * 8);
                        a[u] = __ldcs(src);
                        b[u] = __ldcs(src + 1);
                    }
                }
#pragma unroll
                for (int u = 0; u < FD_ROWS; ++u) {
                    const int pr = pr0 + u * prow_step;
                    if (pr < 128) {
                        bs[0] += a[u].x; bs[1] += a[u].y; bs[2] += a[u].z; bs[3] += a[u].w;
                        bs[4] += b[u].x; bs[5] += b[u].y; bs[6] += b[u].z; bs[7] += b[u].w;
                        const uint4 q = make_uint4(pack_bf16(a[u].x, a[u].y), pack_bf16(a[u].z, a[u].w),
                                                   pack_bf16(b[u].x, b[u].y), pack_bf16(b[u].z, b[u].w));
                        *reinterpret_cast<uint4*>(reg + pr * 128 + (((my_chunk & 7) ^ (pr & 7)) << 4)) = q;
                    }
                }
            }
            // col tile: row = pixel of the tile (the forward kernel's operand, read here as MN-major B)
            for (int it = rg; it < col_items; it += FD_GRP) {
                const int pr = it & 127, ch = it >> 7;
                const long long pix = pix0 + pr;
                int h0 = -(1 << 20), w0 = 0;
                long long base = 0;
                if (pix < p.P) {
                    const long long n = pix / HoWo;
                    const int rem = (int)(pix - n * HoWo);
                    const int ho = rem / p.Wo, wo = rem - ho * p.Wo;
                    h0 = ho * p.sH - p.pH;
                    w0 = wo * p.sW - p.pW;
                    base = ((n * p.H + h0) * p.W + w0) * p.Cin;
                }
                float v[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const int k = ch * 8 + e;
                    const int hi = h0 + ki_s[k], wi = w0 + kj_s[k];
                    v[e] = (hi >= 0 && hi < p.H && wi >= 0 && wi < p.W) ? __ldg(p.x + base + koff_s[k]) : 0.f;
                }
                const uint4 q = make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
                *reinterpret_cast<uint4*>(stage + pr * 128 + ((ch ^ (pr & 7)) << 4)) = q;
            }
            fence_proxy_async_smem();
            mbar_arrive(full_bar(s));
        }
        // db: fp32 column sums of this thread's 8 channels; threads with the same chunk are added in fixed order
#pragma unroll
        for (int e = 0; e < 8; ++e) dbsum_s[r * 8 + e] = bs[e];
        named_bar_sync(1, FD_NP);
        for (int c = r; c < p.Cout; c += FD_NP) {          // (all zero when dy came as a copy: dB is taken elsewhere)
            const int ck = c >> 3, e = c & 7;
            float tsum = 0.f;
            for (int th = ck; th < FD_NP; th += C8) tsum += dbsum_s[th * 8 + e];
            p.part[(size_t)blockIdx.x * (p.K + 1) * p.Cout + (size_t)p.K * p.Cout + c] = tsum;
        }
    } else if (warp == FD_PROD_WARPS) {
        // ------------------------------------------------------------------ MMA issuer
        const bool leader = elect_one();
        const uint32_t idesc = make_idesc(1u, 1u, 1u, 128u, (uint32_t)p.KP);      // A and B MN-major
        const uint32_t hi = (uint32_t)(make_smem_desc(0, 0, 1024) >> 32);          // SBO = 8 reduction rows
        const uint32_t a_lbo = ((uint32_t)FT_STAGE_BYTES >> 4) << 16;              // next 64-channel chunk of dy
        int s = 0;
        uint32_t ph = 0, acc = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < p.ntiles && ok; t += grid) {
            bool f_ok = mbar_wait_spin(full_bar(s), ph, p.status, DS_TIMEOUT_FULL);
            f_ok = __all_sync(0xffffffffu, f_ok);
            if (!f_ok) { ok = false; break; }
            tc_fence_after();
            const uint32_t st16 = ((smem_base + (uint32_t)s * p.stage_bytes) & 0x3FFFFu) >> 4;
            if (leader) {
                for (int db = 0; db < p.dblocks; ++db) {
                    const uint32_t a0 = st16 + ((uint32_t)FT_STAGE_BYTES >> 4) * (1u + 2u * db);
                    for (uint32_t ks = 0; ks < 8; ++ks)
                        asm volatile(
                            "{\n\t.reg .pred pp;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 pp, %5, 0;\n\t"
                            "mov.b64 da, {%1, %4};\n\tmov.b64 db, {%2, %4};\n\t"
                            "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, pp;\n\t}"
                            ::"r"(tmem_base + (uint32_t)(db * 64)), "r"((a0 + ks * 128u) | a_lbo), "r"(st16 + ks * 128u),
                              "r"(idesc), "r"(hi), "r"((ks | acc) ? 1u : 0u)
                            : "memory");
                }
                umma_commit(empty_bar(s));
            }
            acc = 1u;
            if (++s == S) { s = 0; ph ^= 1u; }
            __syncwarp();
        }
        if (leader) umma_commit(done_bar);
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ epilogue: one partial per CTA
        const int q = warp & 3;
        bool ok = true;
        if (any) ok = mbar_wait(done_bar, 0, p.status, DS_TIMEOUT_TMEM_FULL);
        tc_fence_after();
        if (ok) {
            float* out = p.part + (size_t)blockIdx.x * (p.K + 1) * p.Cout;
            for (int db = 0; db < p.dblocks; ++db) {
                const int d = db * 128 + q * 32 + lane;
                for (int cg = 0; cg < p.KP; cg += 32) {
                    uint32_t v[32];
                    if (any) {
                        tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + db * 64 + cg, v);
                        tmem_ld_wait();
                    } else {
#pragma unroll
                        for (int k = 0; k < 32; ++k) v[k] = 0u;
                    }
                    if (d < p.Cout) {
#pragma unroll
                        for (int k = 0; k < 32; ++k)
                            if (cg + k < p.K) out[(size_t)(cg + k) * p.Cout + d] = __uint_as_float(v[k]);
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == FD_PROD_WARPS) {
        tc_fence_after();
        tmem_dealloc(tmem_base, tmem_cols);
    }
}

// ---------------------------------------------------------------------------------- host
static bool first_tc_shape(const AetherConvDesc& d, int& K, int& KP, int& NT, int& Ho, int& Wo) {
    if (d.math_mode != AETHER_MATH_BF16) return false;
    K = d.fH * d.fW * d.Cin;
    if (d.Cin > 4 || K > 64) return false;
    if (d.Cout % 4 || d.Cout < 16 || d.Cout > 256) return false;
    KP = (K + 15) / 16 * 16;
    NT = (d.Cout + 63) / 64 * 64;              // two column halves of 16-column groups; filter rows fill whole 8-row atoms
    conv_out_hw(d, Ho, Wo);
    if (Ho < 1 || Wo < 1) return false;
    const long long P = 1LL * d.S * Ho * Wo;
    return (P + 127) / 128 < 0x7fffffffLL && 1LL * d.S * d.H * d.W * d.Cin < (1LL << 40);
}

bool first_tc_eligible(const AetherConvDesc& d) {
    int K, KP, NT, Ho, Wo;
    return first_tc_shape(d, K, KP, NT, Ho, Wo);
}

static int first_tc_grid(long long ntiles) { return (int)(ntiles < num_sms() ? ntiles : num_sms()); }

long long first_tc_stats_blocks(const AetherConvDesc& d) {
    int K, KP, NT, Ho, Wo;
    if (!first_tc_shape(d, K, KP, NT, Ho, Wo)) return 0;
    const long long P = 1LL * d.S * Ho * Wo;
    return 4LL * first_tc_grid((P + 127) / 128);
}

int first_tc_fwd(const AetherConvDesc& d, const float* x, const float* w, const float* b, float* y, float* stats,
                 cudaStream_t st) {
    int K, KP, NT, Ho, Wo;
    if (!first_tc_shape(d, K, KP, NT, Ho, Wo)) return set_error(AE_UNSUPPORTED, "first_tc_fwd: shape not supported");
    FirstParams p;
    memset(&p, 0, sizeof(p));
    p.x = x; p.w = w; p.bias = b; p.y = y; p.stats = stats; p.status = device_status_word();
    p.H = d.H; p.W = d.W; p.Cin = d.Cin; p.Cout = d.Cout; p.NT = NT; p.fH = d.fH; p.fW = d.fW; p.sH = d.sH; p.sW = d.sW;
    p.pH = d.padH; p.pW = d.padW; p.Ho = Ho; p.Wo = Wo; p.K = K; p.KP = KP;
    p.P = 1LL * d.S * Ho * Wo;
    p.ntiles = (int)((p.P + 127) / 128);
    p.stages = 4;
    const int smem = 1024 + NT * 128 + p.stages * FT_STAGE_BYTES + FT_TAIL + FT_STATS_BYTES;
    static PerDeviceSmem configured[2];
    if (int rc = stats ? ensure_dynamic_smem(first_conv_kernel<true>, 232448, configured[1], "first_conv")
                       : ensure_dynamic_smem(first_conv_kernel<false>, 232448, configured[0], "first_conv"))
        return rc;
    const int grid = first_tc_grid(p.ntiles);
    if (stats) first_conv_kernel<true><<<grid, FirstCfg<true>::THREADS, smem, st>>>(p);
    else first_conv_kernel<false><<<grid, FirstCfg<false>::THREADS, smem, st>>>(p);
    count_launch();
    return check_launch("first_conv_kernel");
}

// dW / dB on the tensor cores need, on top of the forward's conditions, a power-of-two filter count (the producers'
// thread -> channel-chunk mapping) -- the same shapes conv_smallc.cu takes.
bool first_tc_bwd_eligible(const AetherConvDesc& d) {
    return first_tc_eligible(d) && smallc_conv_eligible(d) && d.Cout % 8 == 0;
}

// Workspace of the first-layer filter gradient: the per-CTA partials, then room for a bf16 copy of dy handed in by its
// producer ([P][ld], ld = Cout padded to 64) and for the column sums that come with it.
struct FirstDwLayout {
    size_t part_bytes, dy_off, colsum_off, total;
    int ld, rows_max;
};
static FirstDwLayout first_dw_layout(const AetherConvDesc& d, int K, long long P) {
    FirstDwLayout l;
    l.part_bytes = align_up((size_t)first_tc_grid((P + 127) / 128) * (K + 1) * d.Cout * sizeof(float), 1024);
    l.ld = (d.Cout + 63) / 64 * 64;
    l.dy_off = l.part_bytes;
    l.colsum_off = l.dy_off + align_up((size_t)P * l.ld * 2, 1024);
    l.rows_max = 8 * num_sms();
    l.total = l.colsum_off + align_up((size_t)l.rows_max * d.Cout * sizeof(float), 1024);
    return l;
}

size_t first_tc_bwd_workspace_bytes(const AetherConvDesc& d) {
    int K, KP, NT, Ho, Wo;
    if (!first_tc_bwd_eligible(d) || !first_tc_shape(d, K, KP, NT, Ho, Wo)) return 0;
    return first_dw_layout(d, K, 1LL * d.S * Ho * Wo).total;
}

bool first_tc_operand_layout(const AetherConvDesc& d, AetherOperandLayout* out) {
    int K, KP, NT, Ho, Wo;
    if (!first_tc_bwd_eligible(d) || !first_tc_shape(d, K, KP, NT, Ho, Wo)) return false;
    const FirstDwLayout l = first_dw_layout(d, K, 1LL * d.S * Ho * Wo);
    out->x_copy_offset = 0;
    out->x_copy_ld = 0;                     // the forward kernel gathers x itself: no copy of x to hand in
    out->dy_copy_offset = l.dy_off;
    out->dy_copy_ld = l.ld;
    out->dy_colsum_offset = l.colsum_off;
    out->dy_colsum_rows_max = l.rows_max;
    return true;
}

int first_tc_bwd_filter(const AetherConvDesc& d, const float* x, const float* dy, float* dw, float* db, void* ws,
                        size_t ws_bytes, int dy_colsum_rows, cudaStream_t st) {
    int K, KP, NT, Ho, Wo;
    if (!first_tc_bwd_eligible(d) || !first_tc_shape(d, K, KP, NT, Ho, Wo))
        return set_error(AE_UNSUPPORTED, "first_tc_bwd_filter: shape not supported");
    FirstDwParams p;
    memset(&p, 0, sizeof(p));
    p.x = x; p.dy = dy; p.part = static_cast<float*>(ws); p.status = device_status_word();
    p.H = d.H; p.W = d.W; p.Cin = d.Cin; p.Cout = d.Cout; p.fH = d.fH; p.fW = d.fW; p.sH = d.sH; p.sW = d.sW;
    p.pH = d.padH; p.pW = d.padW; p.Ho = Ho; p.Wo = Wo; p.K = K; p.KP = KP;
    p.dblocks = (d.Cout + 127) / 128;
    p.P = 1LL * d.S * Ho * Wo;
    p.ntiles = (int)((p.P + 127) / 128);
    p.stage_bytes = FT_STAGE_BYTES * (1 + 2 * p.dblocks);
    const int tail = FD_TAIL;
    p.stages = (232448 - 1024 - tail) / p.stage_bytes;
    if (p.stages > 4) p.stages = 4;
    p.groups = p.stages < FD_MAX_GROUPS ? p.stages : FD_MAX_GROUPS;      // 1, 2 or 3: all divide FD_NP, FD_NP / groups is a multiple of 32
    const int grid = first_tc_grid(p.ntiles);
    const FirstDwLayout lay = first_dw_layout(d, K, p.P);
    const size_t need = dy_colsum_rows > 0 ? lay.total : (size_t)grid * (K + 1) * d.Cout * sizeof(float);
    if (!ws || ws_bytes < need) return set_error(AE_BAD_ARG, "conv workspace too small: %zu < %zu", ws_bytes, need);
    if (dy_colsum_rows > 0) {              // dy arrives as a bf16 copy with its column sums
        if (dy_colsum_rows > lay.rows_max)
            return set_error(AE_BAD_ARG, "aether_conv2d_bwd_ex: dy_colsum_rows %d outside [1, %d]", dy_colsum_rows, lay.rows_max);
        int rc0 = make_map_2d(&p.tm_dy, static_cast<uint8_t*>(ws) + lay.dy_off, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, lay.ld, p.P,
                              64, 128);
        if (rc0) return rc0;
        p.dy_bf16 = 1;
    }
    const int smem = 1024 + p.stages * p.stage_bytes + tail;
    static PerDeviceSmem configured;
    if (int rc0 = ensure_dynamic_smem(first_dw_kernel, 232448, configured, "first_dw")) return rc0;
    first_dw_kernel<<<grid, FD_THREADS, smem, st>>>(p);
    count_launch();
    int rc = check_launch("first_dw_kernel");
    if (rc) return rc;
    if (p.dy_bf16) {
        if ((rc = smallc_reduce_partials(p.part, grid, K, d.Cout, dw, nullptr, st))) return rc;
        return db ? colsum_finish(reinterpret_cast<const float*>(static_cast<uint8_t*>(ws) + lay.colsum_off), dy_colsum_rows,
                                  d.Cout, db, st)
                  : AE_OK;
    }
    return smallc_reduce_partials(p.part, grid, K, d.Cout, dw, db, st);
}

}  // namespace aether
