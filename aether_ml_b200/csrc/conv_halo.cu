// Halo-reuse implicit GEMM for stride-1 convolutions on wide images (forward and dX).
//
// One tile = a strip of BH full-width output rows of one image.  Its input window -- (BH+fH-1) rows
// by Wp = Wout+fW-1 columns, one 128-byte channel block per pixel -- is brought into shared memory
// by ONE TMA box whose out-of-range coordinates are zero filled (that is the 'same' padding).
// Shared-memory pixel q = hh*Wp + ww sits in row q of a 128-byte-swizzled K-major operand, so the A
// operand of filter tap (i,j) is the SAME buffer read from row i*Wp + j on: the tensor core's
// operand descriptor simply starts (i*Wp + j) * 128 bytes later (the swizzle is a function of the
// absolute shared-memory address, so row-shifted starts address the data the TMA wrote).
// Accumulator row r then holds output pixel (h_l, w) = (r / Wp, r % Wp); rows with w >= Wout or
// h_l >= BH are by-products that are never stored.  The whole filter stays resident in shared
// memory for the life of the CTA.  Compared with fetching one shifted tile per tap this cuts the
// L2 -> shared-memory traffic per output pixel by roughly fH*fW.
//
// Warp roles (320 threads): warp 0 = TMA producer (it also prefetches the window of the tile after
// next into L2), warp 1 = MMA issuer (the warp runs the loop so that descriptor arithmetic is
// warp-uniform: 32-bit adds on the descriptors' low word; one elected lane issues), warps 2..9 =
// epilogue.  Up to four accumulators live in TMEM so the issuer can run ahead of the epilogue.  Two
// epilogue warps share each 32-lane quarter of TMEM and split its columns; they read the accumulator
// in the 16-lane x 256-bit shape, whose register layout spreads 16 columns of an output row over
// four neighbouring threads; two butterfly shuffles inside the quad give every thread 4 consecutive
// columns, the bias (kept in shared memory) is added and 64-byte row segments go straight to global
// memory (the store path handles about one cache line per cycle, so fewer, wider segments matter).
// Everything that does not change from tile to tile (row -> pixel mapping, column offsets) is
// computed once per thread.
#include <string.h>

#include "common.cuh"
#include "sm100_ptx.cuh"
#include "stats_epilogue.cuh"
#include "tc_host.cuh"

namespace aether {

struct HaloParams {
    CUtensorMap tm_in;   // activations (C, W, H, N), box (128 B of channels, Wp, BH+fH-1, 1)
    CUtensorMap tm_w;    // filter matrix (K, taps*rows_per_tap), box (128 B of K, NT)
    float* out;          // (N, Hout, Wout, n_out) fp32
    const float* bias;   // nullable
    float* stats;        // nullable: per CTA and 32-row quarter (count, mean, M2) of every output channel,
                         // [cta][4][3][n_out] -- the partials Batch_Norm's statistics are merged from
    int* status;
    int n_out;           // real output channels
    int NT;              // accumulator columns (padded output channels), multiple of 32, <= 256
    int Hout, Wout, Wp, BH;
    int tiles_h, n_images;
    int fH, fW, padT, padL, flip;
    int kchunks, rows_per_tap;
    int region_rows;     // (BH+fH-1) * Wp
    int region_stride;   // bytes between stages (multiple of 1024)
    int stages;
    int w_bytes;         // resident filter bytes = taps * kchunks * NT * 128
};

static constexpr int HALO_EPI_WARPS = 8;                          // 4 lane quadrants x HALO_EPI_PARTS column parts
static constexpr int HALO_EPI_PARTS = HALO_EPI_WARPS / 4;
static constexpr int HALO_EPI_UB = 8 / HALO_EPI_PARTS;            // 16-column TMEM loads in flight per batch
static constexpr int HALO_THREADS = 64 + 32 * HALO_EPI_WARPS;
static constexpr int HALO_TAIL = 2048;          // barriers, TMEM pointer, bias
static constexpr int HALO_STATS_BYTES = HALO_EPI_WARPS * STATS_WARP_FLOATS * 4;   // per-warp running column sums and pivots

// MMA with descriptors given as (low word, shared high word); K-major 128-byte-swizzle operands.
// PAIR: the 256-row form issued by the even CTA of a CTA pair (cta_group::2).
template <bool TF32, bool PAIR>
__device__ __forceinline__ void umma_lohi(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t hi, uint32_t idesc,
                                          uint32_t accumulate) {
    if constexpr (PAIR && TF32) {
        asm volatile(
            "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %5, 0;\n\tmov.b64 da, {%1, %4};\n\tmov.b64 db, {%2, %4};\n\t"
            "tcgen05.mma.cta_group::2.kind::tf32 [%0], da, db, %3, p;\n\t}"
            ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(hi), "r"(accumulate)
            : "memory");
    } else if constexpr (PAIR) {
        asm volatile(
            "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %5, 0;\n\tmov.b64 da, {%1, %4};\n\tmov.b64 db, {%2, %4};\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %3, p;\n\t}"
            ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(hi), "r"(accumulate)
            : "memory");
    } else if constexpr (TF32) {
        asm volatile(
            "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %5, 0;\n\tmov.b64 da, {%1, %4};\n\tmov.b64 db, {%2, %4};\n\t"
            "tcgen05.mma.cta_group::1.kind::tf32 [%0], da, db, %3, p;\n\t}"
            ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(hi), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %5, 0;\n\tmov.b64 da, {%1, %4};\n\tmov.b64 db, {%2, %4};\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n\t}"
            ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(hi), "r"(accumulate)
            : "memory");
    }
}

// STATS: the epilogue also accumulates per-channel statistics of the output (p.stats must be set).
// PAIR (clusters of two CTAs, cta_group::2): CTA rank r of a pair takes tile 2u + r of unit u and keeps filter rows
// [r * NT/2, (r+1) * NT/2) of every tap resident; the even CTA issues 256-row MMAs that read both CTAs' windows and
// filter halves and write both CTAs' accumulators.  Half a filter per SM leaves room for more window stages (and lets a
// TF32 filter of 9 x 128 x 64 fit at all), and each MMA reads half as many filter bytes from each SM's shared memory.
template <bool TF32, bool STATS, bool PAIR>
__global__ void __launch_bounds__(HALO_THREADS, 1) halo_conv_kernel(const __grid_constant__ HaloParams p) {
    constexpr int KC = TF32 ? 32 : 64;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t sW = smem_base;
    const uint32_t sR = sW + ((p.w_bytes + 1023) & ~1023);
    const uint32_t sBar = sR + p.stages * p.region_stride;
    const int S = p.stages;
    auto full_bar = [&](int s) { return sBar + 8u * s; };
    auto empty_bar = [&](int s) { return sBar + 8u * (S + s); };
    auto tfull_bar = [&](int b) { return sBar + 8u * (2 * S + b); };
    auto tempty_bar = [&](int b) { return sBar + 8u * (2 * S + 4 + b); };
    const uint32_t wfull_bar = sBar + 8u * (2 * S + 8);
    const uint32_t sTmemPtr = sBar + 8u * (2 * S + 9);
    volatile uint32_t* tmem_ptr_generic = reinterpret_cast<volatile uint32_t*>(gen_base + (sTmemPtr - smem_base));
    float* bias_s = reinterpret_cast<float*>(gen_base + (sBar - smem_base) + 256);     // NT floats

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int NT = p.NT;
    const int cta_rank = PAIR ? (int)cluster_cta_rank() : 0;
    const bool issuer = cta_rank == 0;
    constexpr int PF = PAIR ? 2 : 1;
    // up to four accumulators (the 512 TMEM columns allow it) so the MMA issuer can run ahead of the epilogue
    const uint32_t NB = (4 * NT <= 512) ? 4u : (3 * NT <= 512) ? 3u : 2u;
    const uint32_t need_cols = NB * (uint32_t)NT;
    const uint32_t tmem_cols = (need_cols <= 32) ? 32u : (need_cols <= 64) ? 64u : (need_cols <= 128) ? 128u : (need_cols <= 256) ? 256u : 512u;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 4; ++b) {
            mbar_init(tfull_bar(b), 1);
            mbar_init(tempty_bar(b), PF * HALO_EPI_WARPS);
        }
        mbar_init(wfull_bar, 1);
        mbar_fence_init();
        tma_prefetch_desc(&p.tm_in);
        tma_prefetch_desc(&p.tm_w);
    }
    for (int i = threadIdx.x; i < NT; i += blockDim.x) bias_s[i] = (p.bias != nullptr && i < p.n_out) ? p.bias[i] : 0.f;
    if (warp == 1) {
        if (PAIR) {
            tmem_alloc_pair(sTmemPtr, tmem_cols);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(sTmemPtr, tmem_cols);
            tmem_relinquish();
        }
    }
    tc_fence_before();
    if (PAIR) cluster_sync_all();
    else __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr_generic;

    const int taps = p.fH * p.fW;
    const int total_tiles = p.tiles_h * p.n_images;          // host guarantees it fits in 31 bits
    const int grid = (int)gridDim.x;                         // tiles per round: CTA b takes tiles b, b + grid, ...
    // PAIR: with an odd tile count the odd CTA's last tile is one past the end: its window is zero-filled (image index
    // out of range) and none of its rows is stored; the loops of a pair run while the EVEN CTA's tile exists
    const int t_first = blockIdx.x, t_lead = blockIdx.x - cta_rank;
    const uint32_t region_tx = (uint32_t)p.region_rows * 128u * (uint32_t)PF;     // both CTAs' windows
    const uint32_t wtile_bytes = (uint32_t)(NT / PF) * 128u;                       // this CTA's rows of one filter tile

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            // resident filter: p.w_bytes per CTA; a pair's two halves are counted on the even CTA's barrier
            if (issuer) mbar_arrive_expect_tx(wfull_bar, (uint32_t)p.w_bytes * (uint32_t)PF);
            const uint32_t wbar = PAIR ? cluster_map_shared(wfull_bar, 0) : wfull_bar;
            for (int t = 0; t < taps; ++t)
                for (int kc = 0; kc < p.kchunks; ++kc) {
                    const uint32_t dst = sW + (uint32_t)(t * p.kchunks + kc) * wtile_bytes;
                    if (PAIR) tma_load_2d_pair(dst, &p.tm_w, wbar, kc * KC, t * p.rows_per_tap + cta_rank * (NT / 2));
                    else tma_load_2d(dst, &p.tm_w, wbar, kc * KC, t * p.rows_per_tap);
                }
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int t = t_first; t - cta_rank < total_tiles && ok; t += grid) {
                const int n = t / p.tiles_h;
                const int h0 = (t - n * p.tiles_h) * p.BH;
                const int tp = t + 2 * grid;                       // tile after next: warm L2 with its window
                const int np = tp / p.tiles_h;
                const int hp = (tp - np * p.tiles_h) * p.BH;
                for (int kc = 0; kc < p.kchunks; ++kc) {
                    if (!mbar_wait(empty_bar(s), ph ^ 1u, p.status, DS_TIMEOUT_EMPTY)) { ok = false; break; }
                    if (issuer) mbar_arrive_expect_tx(full_bar(s), region_tx);
                    if (PAIR)
                        tma_load_4d_pair(sR + s * p.region_stride, &p.tm_in, cluster_map_shared(full_bar(s), 0), kc * KC,
                                         -p.padL, h0 - p.padT, n);
                    else
                        tma_load_4d(sR + s * p.region_stride, &p.tm_in, full_bar(s), kc * KC, -p.padL, h0 - p.padT, n);
                    if (tp < total_tiles) tma_prefetch_l2_4d(&p.tm_in, kc * KC, -p.padL, hp - p.padT, np);
                    if (++s == S) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 1 && issuer) {
        // ------------------------------------------------------------------ MMA issuer
        const bool leader = elect_one();
        const uint32_t idesc = make_idesc(TF32 ? 2u : 1u, 0u, 0u, 128u * PF, (uint32_t)NT);
        const uint64_t proto = make_smem_desc(0, 16, 1024);
        const uint32_t hi = (uint32_t)(proto >> 32);
        const uint32_t lo_proto = (uint32_t)proto;                         // LBO field; start address added below
        const uint32_t wt16 = wtile_bytes >> 4;
        const uint32_t bstep = wt16 * (uint32_t)p.kchunks;                 // one filter tap, in 16-byte units
        const uint32_t w_lo = lo_proto + ((sW & 0x3FFFFu) >> 4);
        const uint32_t row_step = (uint32_t)p.Wp * 8u;                     // one window row, in 16-byte units
        const uint32_t r_lo = lo_proto + ((sR & 0x3FFFFu) >> 4);
        const uint32_t rs16 = (uint32_t)p.region_stride >> 4;
        // every lane observes each barrier itself (non-suspending polls, so no lane lags behind)
        bool ok = __all_sync(0xffffffffu, mbar_wait_spin(wfull_bar, 0, p.status, DS_TIMEOUT_FULL));
        int s = 0;
        uint32_t ph = 0, buf = 0, aph = 0;
        for (int t = t_lead; t < total_tiles && ok; t += grid) {
            bool w_ok = mbar_wait_spin(tempty_bar(buf), aph ^ 1u, p.status, DS_TIMEOUT_TMEM_EMPTY);
            w_ok = __all_sync(0xffffffffu, w_ok);
            if (!w_ok) { ok = false; break; }
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + buf * NT;
            uint32_t acc = 0;
            for (int kc = 0; kc < p.kchunks; ++kc) {
                bool f_ok = mbar_wait_spin(full_bar(s), ph, p.status, DS_TIMEOUT_FULL);
                f_ok = __all_sync(0xffffffffu, f_ok);
                if (!f_ok) { ok = false; break; }
                tc_fence_after();
                uint32_t a_row = r_lo + (uint32_t)s * rs16;
                // filter tap that multiplies window shift (ti,tj): the same index, or the mirrored one for dX
                uint32_t b_cur = w_lo + (uint32_t)kc * wt16 + (p.flip ? (uint32_t)(taps - 1) * bstep : 0u);
                for (int ti = 0; ti < p.fH; ++ti) {
                    uint32_t a_tap = a_row;
                    for (int tj = 0; tj < p.fW; ++tj) {
                        if (leader) {
                            umma_lohi<TF32, PAIR>(d_tmem, a_tap, b_cur, hi, idesc, acc);
                            umma_lohi<TF32, PAIR>(d_tmem, a_tap + 2, b_cur + 2, hi, idesc, 1u);
                            umma_lohi<TF32, PAIR>(d_tmem, a_tap + 4, b_cur + 4, hi, idesc, 1u);
                            umma_lohi<TF32, PAIR>(d_tmem, a_tap + 6, b_cur + 6, hi, idesc, 1u);
                        }
                        acc = 1u;
                        a_tap += 8u;
                        b_cur = p.flip ? b_cur - bstep : b_cur + bstep;
                    }
                    a_row += row_step;
                }
                if (leader) {
                    if (PAIR) {
                        umma_commit_pair(empty_bar(s));
                        umma_commit_pair(cluster_map_shared(empty_bar(s), 1));
                    } else {
                        umma_commit(empty_bar(s));
                    }
                }
                if (++s == S) { s = 0; ph ^= 1u; }
            }
            if (ok && leader) {
                if (PAIR) {
                    umma_commit_pair(tfull_bar(buf));
                    umma_commit_pair(cluster_map_shared(tfull_bar(buf), 1));
                } else {
                    umma_commit(tfull_bar(buf));
                }
            }
            if (++buf == NB) { buf = 0; aph ^= 1u; }
            __syncwarp();
        }
    } else if (warp >= 2) {
        // ------------------------------------------------------------------ epilogue
        // Warp (q, half): TMEM lanes [32q, 32q+32), columns [half*NT/2, (half+1)*NT/2).  Accumulators are read
        // with the 16-lane x 256-bit shape: thread t receives, per 8-column group, columns 2*(t%4)+{0,1} of rows
        // t/4 and t/4+8 of the 16-lane half -- i.e. four threads hold one 32-byte sector of an output row, so
        // the registers go straight to global memory as full sectors (no shared-memory staging).
        const int ew = warp - 2;
        const int q = warp & 3;
        const int part = ew >> 2;
        const int ncols = NT / HALO_EPI_PARTS;     // columns this warp owns (multiple of 16)
        const int col_begin = part * ncols;
        const int trow = lane >> 2, tcol4 = (lane & 3) * 4;   // after the quad exchange a lane owns 4 consecutive columns
        const bool lo2 = (lane & 2) == 0, odd = (lane & 1) != 0;
        const bool all_cols = (p.n_out == NT);     // no padded output channels: no per-column bound checks
        constexpr bool do_stats = STATS;
        // running per-column sums of this warp over all its tiles (stats_epilogue.cuh): warp-private shared memory
        float* stat_w = reinterpret_cast<float*>(gen_base + (sBar - smem_base) + HALO_TAIL) + ew * STATS_WARP_FLOATS;
        float st_rows = 0.f;                       // rows (pixels) summed so far, identical in every lane
        if (do_stats) {
            for (int i = lane; i < STATS_WARP_FLOATS; i += 32) stat_w[i] = 0.f;
            __syncwarp();
        }
        // The four accumulator rows this thread holds map to fixed pixels of every strip: precompute their
        // offsets (in floats, relative to the strip's first pixel, including this thread's column offset).
        int row_off[4], row_hl[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int r = q * 32 + (j >> 1) * 16 + trow + (j & 1) * 8;      // rows: lane half j>>1, sub-row j&1
            const int hl = r / p.Wp, w = r - hl * p.Wp;
            row_hl[j] = (w < p.Wout && hl < p.BH) ? hl : (1 << 30);           // never valid
            row_off[j] = (hl * p.Wout + w) * p.n_out + col_begin + tcol4;
        }
        const float* bias4 = bias_s + col_begin + tcol4;
        const size_t strip_floats = (size_t)p.BH * p.Wout * p.n_out;
        const size_t image_floats = (size_t)p.Hout * p.Wout * p.n_out;
        uint32_t buf = 0, aph = 0;
        bool ok = true;
        for (int t = t_first; t - cta_rank < total_tiles && ok; t += grid) {
            const int n = t / p.tiles_h;
            const int th = t - n * p.tiles_h;
            const int rows_left = t < total_tiles ? p.Hout - th * p.BH : 0;      // a pair's tile past the end stores nothing
            float* tile_base = p.out + (size_t)n * image_floats + (size_t)th * strip_floats;
            float* rowp[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) rowp[j] = (row_hl[j] < rows_left) ? tile_base + row_off[j] : nullptr;
            float tile_rows = 0.f;                 // valid rows of this tile in this warp's quarter
            if (do_stats) {
#pragma unroll
                for (int j = 0; j < 4; ++j) tile_rows += (rowp[j] != nullptr) ? 1.f : 0.f;
                tile_rows += __shfl_xor_sync(0xffffffffu, tile_rows, 4);
                tile_rows += __shfl_xor_sync(0xffffffffu, tile_rows, 8);
                tile_rows += __shfl_xor_sync(0xffffffffu, tile_rows, 16);
            }
            const bool first_stats = do_stats && st_rows == 0.f && tile_rows > 0.f;   // the tile that sets the pivots
            if (!mbar_wait(tfull_bar(buf), aph, p.status, DS_TIMEOUT_TMEM_FULL)) { ok = false; break; }
            tc_fence_after();
            const uint32_t taddr0 = tmem_base + ((uint32_t)(q * 32) << 16) + buf * NT + col_begin;
#pragma unroll 1
            for (int cb = 0; cb < ncols; cb += 16 * HALO_EPI_UB) {   // batches of HALO_EPI_UB x 16 columns
                uint32_t v[2][HALO_EPI_UB][8];
                float4 st_s[HALO_EPI_UB], st_q[HALO_EPI_UB];         // per-column sum / sum of squares of this tile's rows
#pragma unroll
                for (int u = 0; u < HALO_EPI_UB; ++u) st_s[u] = st_q[u] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int u = 0; u < HALO_EPI_UB; ++u) {
                    if (cb + u * 16 < ncols) {
                        tmem_ld_16x256b_x2(taddr0 + cb + u * 16, v[0][u]);
                        tmem_ld_16x256b_x2(taddr0 + (16u << 16) + cb + u * 16, v[1][u]);
                    }
                }
                tmem_ld_wait();
                if (cb + 16 * HALO_EPI_UB >= ncols) {            // accumulator fully read by this warp
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        if (PAIR) mbar_arrive_cluster(cluster_map_shared(tempty_bar(buf), 0));
                        else mbar_arrive(tempty_bar(buf));
                    }
                }
#pragma unroll
                for (int u = 0; u < HALO_EPI_UB; ++u) {
                    if (cb + u * 16 < ncols) {
#pragma unroll
                        // A quad holds 16 columns of a row as 2+2 columns per lane (groups 0 and 1).  Two
                        // butterfly exchanges inside the quad turn that into 4 consecutive columns per lane,
                        // so each store instruction writes 64 contiguous bytes per row instead of 32.
                        const int cc = cb + u * 16;              // column relative to this thread's first column
                        const float4 b4 = *reinterpret_cast<const float4*>(bias4 + cc);
                        const bool cols_ok = all_cols || col_begin + tcol4 + cc < p.n_out;
                        float4 pv = make_float4(0.f, 0.f, 0.f, 0.f);      // pivot of this lane's four columns
                        if (do_stats) pv = *reinterpret_cast<const float4*>(stat_w + 256 + cc + tcol4);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const uint32_t a0 = v[j >> 1][u][(j & 1) * 2 + 0], a1 = v[j >> 1][u][(j & 1) * 2 + 1];
                            const uint32_t b0 = v[j >> 1][u][4 + (j & 1) * 2 + 0], b1 = v[j >> 1][u][4 + (j & 1) * 2 + 1];
                            // step 1 (lane ^ 2): lanes 0,1 collect group 0, lanes 2,3 collect group 1
                            const uint32_t s0 = lo2 ? b0 : a0, s1 = lo2 ? b1 : a1;
                            const uint32_t r0 = __shfl_xor_sync(0xffffffffu, s0, 2), r1 = __shfl_xor_sync(0xffffffffu, s1, 2);
                            const uint32_t x0 = lo2 ? a0 : r0, x1 = lo2 ? a1 : r1;       // piece from the even source lane
                            const uint32_t y0 = lo2 ? r0 : b0, y1 = lo2 ? r1 : b1;       // piece from the source lane + 2
                            // step 2 (lane ^ 1): even lanes keep the lower pair of pieces, odd lanes the upper pair
                            const uint32_t t0 = odd ? x0 : y0, t1 = odd ? x1 : y1;
                            const uint32_t q0 = __shfl_xor_sync(0xffffffffu, t0, 1), q1 = __shfl_xor_sync(0xffffffffu, t1, 1);
                            float4 a;                                                     // accumulator values (before the bias)
                            a.x = __uint_as_float(odd ? q0 : x0);
                            a.y = __uint_as_float(odd ? q1 : x1);
                            a.z = __uint_as_float(odd ? y0 : q0);
                            a.w = __uint_as_float(odd ? y1 : q1);
                            const bool wr = cols_ok && rowp[j] != nullptr;
                            if (wr)
                                __stcs(reinterpret_cast<float4*>(rowp[j] + cc),
                                       make_float4(a.x + b4.x, a.y + b4.y, a.z + b4.z, a.w + b4.w));
                            if (do_stats) {                                  // branch-free: by-product rows count as zero
                                a.x = wr ? a.x - pv.x : 0.f; a.y = wr ? a.y - pv.y : 0.f;  // selects, not products: a by-product may be NaN
                                a.z = wr ? a.z - pv.z : 0.f; a.w = wr ? a.w - pv.w : 0.f;
                                st_s[u].x += a.x; st_s[u].y += a.y; st_s[u].z += a.z; st_s[u].w += a.w;
                                st_q[u].x = fmaf(a.x, a.x, st_q[u].x); st_q[u].y = fmaf(a.y, a.y, st_q[u].y);
                                st_q[u].z = fmaf(a.z, a.z, st_q[u].z); st_q[u].w = fmaf(a.w, a.w, st_q[u].w);
                            }
                        }
                    }
                }
                if (do_stats) {
                    // Lanes with equal lane%4 hold the same 4 columns of 8 different row groups: add them up
                    // (xor 4, 8, 16); lanes 0..3 then add the tile's sums to this warp's running sums in
                    // shared memory (about the column's pivot, see stats_epilogue.cuh).
#pragma unroll
                    for (int m = 4; m <= 16; m <<= 1) {
#pragma unroll
                        for (int u = 0; u < HALO_EPI_UB; ++u) {
                            st_s[u].x += __shfl_xor_sync(0xffffffffu, st_s[u].x, m); st_s[u].y += __shfl_xor_sync(0xffffffffu, st_s[u].y, m);
                            st_s[u].z += __shfl_xor_sync(0xffffffffu, st_s[u].z, m); st_s[u].w += __shfl_xor_sync(0xffffffffu, st_s[u].w, m);
                            st_q[u].x += __shfl_xor_sync(0xffffffffu, st_q[u].x, m); st_q[u].y += __shfl_xor_sync(0xffffffffu, st_q[u].y, m);
                            st_q[u].z += __shfl_xor_sync(0xffffffffu, st_q[u].z, m); st_q[u].w += __shfl_xor_sync(0xffffffffu, st_q[u].w, m);
                        }
                    }
                    if (lane < 4) {
#pragma unroll
                        for (int u = 0; u < HALO_EPI_UB; ++u) {
                            const int cc = cb + u * 16;
                            if (cc < ncols) stats_fold(stat_w, cc + tcol4, st_s[u], st_q[u], first_stats, tile_rows);
                        }
                    }
                    if (first_stats) __syncwarp();     // the pivots must be visible to the whole warp before its next tile
                }
            }
            st_rows += tile_rows;
            if (++buf == NB) { buf = 0; aph ^= 1u; }
        }
        if (do_stats && lane < 4) {
            // (count, mean, M2) of this warp's rows over all tiles of the CTA: block blockIdx.x*4 + q of [3][n_out]
            float* sp = p.stats + ((size_t)blockIdx.x * 4 + q) * 3 * (size_t)p.n_out;
            for (int cc = 0; cc < ncols; cc += 16) {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int col = col_begin + tcol4 + cc + k;
                    if (col < p.n_out) {
                        float m, m2;
                        stats_result(stat_w, cc + tcol4 + k, st_rows, m, m2);
                        sp[col] = st_rows;
                        sp[p.n_out + col] = m + bias_s[col];
                        sp[2 * p.n_out + col] = m2;
                    }
                }
            }
        }
    }

    tc_fence_before();
    if (PAIR) cluster_sync_all();
    else __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        if (PAIR) tmem_dealloc_pair(tmem_base, tmem_cols);
        else tmem_dealloc(tmem_base, tmem_cols);
    }
}

// Decides whether the halo kernel takes this problem; if so launches it and sets *used.
struct HaloGeom {
    int Wp, BH, tiles_h, kchunks, w_bytes, region_rows, region_stride, stages, fixed;
    bool pair;      // CTA pairs: w_bytes is then the half filter each CTA keeps
    int grid;       // CTAs (2 x pairs)
};
static constexpr int HALO_SMEM_MAX = 232448;

// Decides whether the halo kernel takes the problem and, if so, its tiling.
static bool halo_geometry(bool tf32, int in_C, int S, int taps, int out_C, int out_H, int out_W, int n_padded, int fH,
                          int fW, HaloGeom& g) {
    const int KC = tf32 ? 32 : 64;
    g.Wp = out_W + fW - 1;
    if (n_padded > 256 || n_padded % (16 * HALO_EPI_PARTS) || out_C % 4) return false;
    if (g.Wp > 256 || out_W > 128 || out_W < 12) return false;
    g.BH = (128 - out_W) / g.Wp + 1;
    if (g.BH > out_H) g.BH = out_H;
    if (g.BH + fH - 1 > 256) return false;
    g.tiles_h = ceil_div(out_H, g.BH);
    if (1LL * g.tiles_h * S > 0x3fffffffLL) return false;
    // useful fraction of the 128 accumulator rows, including the ragged last strip of each image
    const double eff = (double)out_H * out_W / ((double)g.tiles_h * 128.0);
    if (eff < 0.70) return false;
    g.kchunks = ceil_div(in_C, KC);
    g.region_rows = (g.BH + fH - 1) * g.Wp;
    g.region_stride = (int)align_up((size_t)g.region_rows * 128, 1024);
    const long long total = 1LL * g.tiles_h * S;
    // Single CTAs where the whole filter fits beside two window stages.  Where it does not (TF32, 64 -> 128 channels:
    // 295 KB), CTA pairs keep half of it each -- if every pair of SMs gets at least two units of two tiles.  Pairs are
    // NOT used where single CTAs fit: measured on B200 (bf16, batch 256) the pair form took 0.144 ms against 0.117 ms
    // for the 56x56 64 -> 128 forward and 0.044 against 0.037 ms at 32x32 64 -> 64 (two SMs that wait for each
    // other's store-bound epilogues), and gained only 5 % on the 56x56 dX (0.127 against 0.134 ms).
    g.pair = false;
    for (int attempt = 0; attempt < 2; ++attempt) {
        g.w_bytes = taps * g.kchunks * (g.pair ? n_padded / 2 : n_padded) * 128;
        g.fixed = 1024 + (int)align_up(g.w_bytes, 1024) + HALO_TAIL + HALO_STATS_BYTES;
        g.stages = (HALO_SMEM_MAX - g.fixed) / g.region_stride;
        if (g.stages > 4) g.stages = 4;
        if (g.stages >= 2) break;
        if (attempt == 1 || n_padded % 32 != 0 || total < 4LL * (num_sms() / 2) || !cta_pairs_available()) return false;
        g.pair = true;
    }
    if (g.pair) {
        const long long units = (total + 1) / 2;
        g.grid = 2 * (int)(units < num_sms() / 2 ? units : num_sms() / 2);
    } else {
        g.grid = (int)(total < num_sms() ? total : num_sms());
    }
    // every tap reads 128 rows from its shifted start; the furthest read must stay inside the allocation
    const int overhang_rows = (fH - 1) * g.Wp + (fW - 1) + 128 - g.region_rows;
    // (what the last stage reads past its region -- barriers, bias, statistics -- only feeds by-product rows)
    if (overhang_rows > 0 && overhang_rows * 128 > HALO_TAIL + HALO_STATS_BYTES + (g.region_stride - g.region_rows * 128))
        return false;
    return true;
}

// Number of (count, mean, M2) partial blocks the kernel writes per output channel when asked for statistics
// (4 per tile), or 0 when the halo kernel does not take this problem.
long long halo_igemm_stats_blocks(bool tf32, int in_C, int S, int taps, int out_C, int out_H, int out_W, int n_padded,
                                  int fH, int fW) {
    HaloGeom g;
    if (!halo_geometry(tf32, in_C, S, taps, out_C, out_H, out_W, n_padded, fH, fW, g)) return 0;
    return 4LL * g.grid;       // one block per CTA and 32-row quarter
}

int run_halo_igemm(bool tf32, const void* in, int in_C, int in_H, int in_W, int S, const void* wmat, int w_inner,
                   int rows_per_tap, int taps, float* out, int out_C, int out_H, int out_W, int n_padded, int fH, int fW,
                   int padT, int padL, int flip, const float* bias, float* stats, int prof_kind, cudaStream_t st,
                   bool* used) {
    *used = false;
    const int elt = tf32 ? 4 : 2;
    const int KC = 128 / elt;
    HaloGeom g;
    if (!halo_geometry(tf32, in_C, S, taps, out_C, out_H, out_W, n_padded, fH, fW, g)) return AE_OK;
    const int Wp = g.Wp, BH = g.BH, tiles_h = g.tiles_h, kchunks = g.kchunks, w_bytes = g.w_bytes;
    const int region_rows = g.region_rows, region_stride = g.region_stride, stages = g.stages, fixed = g.fixed;
    const int smem_max = HALO_SMEM_MAX;

    HaloParams p;
    memset(&p, 0, sizeof(p));
    const CUtensorMapDataType dt = tf32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    int rc;
    if ((rc = make_map_nhwc(&p.tm_in, in, dt, elt, in_C, in_W, in_H, S, KC, Wp, BH + fH - 1, 1))) return rc;
    if ((rc = make_map_2d(&p.tm_w, wmat, dt, elt, w_inner, 1LL * taps * rows_per_tap, KC, g.pair ? n_padded / 2 : n_padded)))
        return rc;
    p.out = out;
    p.bias = bias;
    p.stats = stats;
    p.status = device_status_word();
    p.n_out = out_C;
    p.NT = n_padded;
    p.Hout = out_H; p.Wout = out_W; p.Wp = Wp; p.BH = BH;
    p.tiles_h = tiles_h; p.n_images = S;
    p.fH = fH; p.fW = fW; p.padT = padT; p.padL = padL; p.flip = flip;
    p.kchunks = kchunks; p.rows_per_tap = rows_per_tap;
    p.region_rows = region_rows; p.region_stride = region_stride; p.stages = stages; p.w_bytes = w_bytes;
    const int smem = fixed + stages * region_stride;

    // eight instantiations: operand type x (with / without the statistics epilogue) x (single CTAs / CTA pairs)
    using KernelFn = void (*)(const HaloParams);
    static const KernelFn kernels[8] = {halo_conv_kernel<false, false, false>, halo_conv_kernel<true, false, false>,
                                        halo_conv_kernel<false, true, false>,  halo_conv_kernel<true, true, false>,
                                        halo_conv_kernel<false, false, true>,  halo_conv_kernel<true, false, true>,
                                        halo_conv_kernel<false, true, true>,   halo_conv_kernel<true, true, true>};
    static PerDeviceSmem configured[8];
    const int ki = (tf32 ? 1 : 0) + (stats ? 2 : 0) + (g.pair ? 4 : 0);
    if ((rc = ensure_dynamic_smem(kernels[ki], smem_max, configured[ki], "halo_conv"))) return rc;
    prof_begin(prof_kind, st);
    if (g.pair) {
        cudaLaunchConfig_t cfg;
        memset(&cfg, 0, sizeof(cfg));
        cfg.gridDim = dim3(g.grid, 1, 1);
        cfg.blockDim = dim3(HALO_THREADS, 1, 1);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = st;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2;
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        const cudaError_t e = cudaLaunchKernelEx(&cfg, kernels[ki], p);
        if (e != cudaSuccess) return set_error(AE_CUDA, "halo_conv_kernel (CTA pairs): %s", cudaGetErrorString(e));
    } else {
        kernels[ki]<<<g.grid, HALO_THREADS, smem, st>>>(p);
    }
    prof_end(prof_kind, st);
    count_launch();
    *used = true;
    return check_launch("halo_conv_kernel");
}


}  // namespace aether
