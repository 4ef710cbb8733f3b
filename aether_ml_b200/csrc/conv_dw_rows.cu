// Filter gradient (dW) for 3-row filters on wide images with the upstream gradient as the M operand, bf16.
//
//   dW[(i,j)][c][d] = sum over output pixels p of x[p + (i,j)][c] * dy[p][d]        (CNN_classes_cupy.py:134)
//
// With a 64-channel block of x as M and a 64-channel block of dy as N (conv_halo_dw.cu) every MMA is a
// 128x64x16 product whose shared-memory operand reads (6 KB) take longer than its tensor-core time.  Here the
// roles are swapped and widened: M = 128 output channels of dy, N = fW taps x 64 input channels, so one MMA
// per filter row and 16 pixels does a 128 x (fW*64) x 16 product (10 KB of operand reads for 96 tensor clocks
// at fW = 3).  The three taps of a filter row are three 64-column chunks of the N operand whose
// leading-dimension offset is ONE pixel row (128 bytes) of the x window: tap j is the same window read one
// pixel further on.
//
// The accumulators of all three filter rows (3 x fW*64 columns) do not fit the 512 TMEM columns, so CTAs come
// in two classes that share the strips of the image: class A accumulates filter rows 0 and 1 (two MMAs per
// 16 pixels on the same dy operand), class B filter row 2; the CTAs are divided between the classes so that
// both finish together (rows_dw_splits).  Class-A CTA s walks strips s, s+a, ...; class-B CTA t walks
// t, t+b, ... at a faster pace, so both classes read a strip at about the same time and the second read
// comes from L2 (DRAM traffic measured by ncu equals one pass over x and dy).  Each CTA keeps its
// accumulators in TMEM for its whole life and writes one partial; the partials are added in fixed order by
// dw_reduce_kernel (which is told the two split counts).
#include <string.h>

#include "common.cuh"
#include "sm100_ptx.cuh"
#include "tc_host.cuh"

namespace aether {

struct DwRowsParams {
    CUtensorMap tm_x;    // (Cin_p, W, H, N) bf16, box (64, Wp, BH+1, 1)
    CUtensorMap tm_dy;   // (Cout_p, Wo, Ho, N) bf16, box (64, Wp, BH, 1)
    float* part;         // [split][taps*cblocks][64][ldn]
    int* status;
    int Wp, BH, tiles_h, n_images;
    int fW, taps, padT, padL;
    int cblocks, dblocks, ldn;            // dblocks counts 128-channel blocks of dy
    int x_box_rows, dy_box_rows;          // pixel rows written by the boxes
    int dyr_bytes, xr_bytes, stage_bytes; // one dy region (two per stage), the x region, a stage
    int stages, ksteps;
    int splits_a, splits_b, rows_a;       // CTAs per unit in class A / B, filter rows of class A
    int fH;
};

static constexpr int DWR_THREADS = 192;   // warp 0 producer, warp 1 MMA issuer, warps 2..5 epilogue

__global__ void __launch_bounds__(DWR_THREADS, 1) dw_rows_kernel(const __grid_constant__ DwRowsParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (smem_base - smem_u32(smem_raw));
    const int S = p.stages;
    const uint32_t sBar = smem_base + S * p.stage_bytes;
    auto full_bar = [&](int s) { return sBar + 8u * s; };
    auto empty_bar = [&](int s) { return sBar + 8u * (S + s); };
    const uint32_t done_bar = sBar + 8u * (2 * S);
    const uint32_t sTmemPtr = sBar + 8u * (2 * S + 1);
    volatile uint32_t* tmem_ptr_generic = reinterpret_cast<volatile uint32_t*>(gen_base + (sTmemPtr - smem_base));

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    // Rows that no TMA box writes (the tails of the regions) are read by the MMAs and must be zero.
    // Only those tails are cleared (a few KB), not the whole 220 KB of stages.
    {
        const int dy_tail0 = p.dy_box_rows * 128, x_tail0 = 2 * p.dyr_bytes + p.x_box_rows * 128;
        for (int s = 0; s < S; ++s) {
            uint8_t* st = gen_base + (size_t)s * p.stage_bytes;
            for (int o = dy_tail0 + threadIdx.x * 16; o < p.dyr_bytes; o += blockDim.x * 16) {
                *reinterpret_cast<uint4*>(st + o) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(st + p.dyr_bytes + o) = make_uint4(0, 0, 0, 0);
            }
            for (int o = x_tail0 + threadIdx.x * 16; o < p.stage_bytes; o += blockDim.x * 16)
                *reinterpret_cast<uint4*>(st + o) = make_uint4(0, 0, 0, 0);
        }
        fence_proxy_async_smem();
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(done_bar, 1);
        mbar_fence_init();
        tma_prefetch_desc(&p.tm_x);
        tma_prefetch_desc(&p.tm_dy);
    }
    if (warp == 1) {
        tmem_alloc(sTmemPtr, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr_generic;

    // CTA -> (unit = (x block, dy block), class, split)
    const int per_unit = p.splits_a + p.splits_b;
    const int unit = blockIdx.x / per_unit;
    const int wi = blockIdx.x - unit * per_unit;
    const bool cls_b = wi >= p.splits_a;
    const int split = cls_b ? wi - p.splits_a : wi;
    const int splits = cls_b ? p.splits_b : p.splits_a;
    const int row0 = cls_b ? p.rows_a : 0;                       // first filter row of this CTA
    const int nrows = cls_b ? p.fH - p.rows_a : p.rows_a;
    const int cb = unit / p.dblocks;
    const int db = unit - cb * p.dblocks;
    const int N = p.fW * 64;
    const long long total_strips = 1LL * p.tiles_h * p.n_images;
    const uint32_t stage_tx = (uint32_t)(p.x_box_rows + 2 * p.dy_box_rows) * 128u;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            for (long long st = split; st < total_strips; st += splits, ++it) {
                const int th = (int)(st % p.tiles_h);
                const int n = (int)(st / p.tiles_h);
                const int h0 = th * p.BH;
                const int s = it % S;
                const uint32_t ph = (it / S) & 1u;
                if (!mbar_wait(empty_bar(s), ph ^ 1u, p.status, DS_TIMEOUT_EMPTY)) break;
                mbar_arrive_expect_tx(full_bar(s), stage_tx);
                const uint32_t base = smem_base + s * p.stage_bytes;
                tma_load_4d(base, &p.tm_dy, full_bar(s), db * 128, 0, h0, n);
                tma_load_4d(base + p.dyr_bytes, &p.tm_dy, full_bar(s), db * 128 + 64, 0, h0, n);
                tma_load_4d(base + 2 * p.dyr_bytes, &p.tm_x, full_bar(s), cb * 64, -p.padL, h0 - p.padT + row0, n);
            }
        }
    } else if (warp == 1) {
        // The whole warp runs the loop (warp-uniform descriptor arithmetic); one elected lane issues.
        const bool leader = elect_one();
        const uint32_t idesc = make_idesc(1u, 1u, 1u, 128u, (uint32_t)N);       // bf16, A and B MN-major, M=128
        const uint32_t hi = (uint32_t)(make_smem_desc(0, 0, 1024) >> 32);       // SBO = 1024 (8 reduction rows), 128B swizzle
        const uint32_t a_lbo = ((uint32_t)p.dyr_bytes >> 4) << 16;              // second 64-channel block of dy
        const uint32_t b_lbo = 8u << 16;                                        // next tap = next pixel row (128 bytes)
        const uint32_t row_step = (uint32_t)p.Wp * 8u;                          // next filter row = Wp pixel rows
        uint32_t it = 0;
        bool ok = true;
        uint32_t acc = 0;
        for (long long st = split; st < total_strips && ok; st += splits, ++it) {
            const int s = it % S;
            const uint32_t ph = (it / S) & 1u;
            bool f_ok = mbar_wait_spin(full_bar(s), ph, p.status, DS_TIMEOUT_FULL);
            f_ok = __all_sync(0xffffffffu, f_ok);
            if (!f_ok) { ok = false; break; }
            tc_fence_after();
            const uint32_t base16 = ((smem_base + s * p.stage_bytes) & 0x3FFFFu) >> 4;
            uint32_t a_k = base16;                                               // advances 16 reduction rows per step
            uint32_t b_k = base16 + ((uint32_t)(2 * p.dyr_bytes) >> 4);
            for (int kk = 0; kk < p.ksteps; ++kk) {
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    if (r < nrows && leader) {
                        asm volatile(
                            "{\n\t.reg .pred pp;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 pp, %5, 0;\n\t"
                            "mov.b64 da, {%1, %4};\n\tmov.b64 db, {%2, %4};\n\t"
                            "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, pp;\n\t}"
                            ::"r"(tmem_base + (uint32_t)(r * N)), "r"(a_k | a_lbo), "r"((b_k + (uint32_t)r * row_step) | b_lbo),
                              "r"(idesc), "r"(hi), "r"(acc)
                            : "memory");
                    }
                }
                acc = 1u;
                a_k += 128u;
                b_k += 128u;
            }
            if (leader) umma_commit(empty_bar(s));
            __syncwarp();
        }
        if (leader) umma_commit(done_bar);
        __syncwarp();
    } else {
        const int q = warp & 3;
        const int d_in = q * 32 + lane;                                          // accumulator lane = dy channel in the block
        const bool any = split < total_strips;
        bool ok = true;
        if (any) ok = mbar_wait(done_bar, 0, p.status, DS_TIMEOUT_TMEM_FULL);
        tc_fence_after();
        if (ok) {
            for (int r = 0; r < nrows; ++r) {
                for (int j = 0; j < p.fW; ++j) {
                    const int tap = (row0 + r) * p.fW + j;
                    float* dst = p.part + (((size_t)split * (p.taps * p.cblocks) + (size_t)tap * p.cblocks + cb) * 64) * (size_t)p.ldn +
                                 db * 128 + d_in;
#pragma unroll 1
                    for (int ch = 0; ch < 2; ++ch) {
                        uint32_t v[32];
                        if (any) {
                            tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + r * N + j * 64 + ch * 32, v);
                            tmem_ld_wait();
                        } else {
#pragma unroll
                            for (int k = 0; k < 32; ++k) v[k] = 0u;
                        }
#pragma unroll
                        for (int k = 0; k < 32; ++k) dst[(size_t)(ch * 32 + k) * p.ldn] = __uint_as_float(v[k]);
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// Split counts of the two CTA classes for `units` (x block, dy block) pairs: class A gets two thirds of the
// CTAs of a unit.  Returns false when a unit would get fewer than three CTAs.
static bool rows_dw_splits(int units, long long strips, int* a, int* b) {
    const int per_unit = num_sms() / units;
    if (per_unit < 3) return false;
    // Class B does half the MMA work of class A per strip but loads the same bytes, and at that pace it is bound
    // by what one SM can pull from L2, not by its MMAs: measured on B200 (56x56, 64 -> 128 channels, batch 256)
    // the kernel is fastest with 60 of 148 CTAs in class B (0.091 ms, against 0.110 ms at 49 and 0.100 ms at 74).
    int sb = (per_unit * 13) / 32, sa = per_unit - sb;
    if (sb < 1) { sb = 1; sa = per_unit - 1; }
    if (sb > strips) sb = (int)strips;
    if (sa > strips) sa = (int)strips;
    *a = sa;
    *b = sb;
    return true;
}

static bool rows_dw_shape_ok(int Cin_p, int Cout_p, int Wo, int fH, int fW) {
    if (fH != 3 || fW < 2 || fW > 4) return false;          // N = fW*64 <= 256 columns, two rows <= 512 TMEM columns
    if (Cin_p % 64 || Cout_p % 128) return false;
    const int Wp = Wo + fW - 1;
    return Wp <= 256 && Wo >= 12;
}

// Largest split count the kernel can ask of the partial buffer for this problem (0: kernel not applicable).
int rows_dw_max_splits(int Cin_p, int Cout_p, int Ho, int Wo, int S, int fH, int fW) {
    if (!rows_dw_shape_ok(Cin_p, Cout_p, Wo, fH, fW)) return 0;
    int a = 0, b = 0;
    if (!rows_dw_splits((Cin_p / 64) * (Cout_p / 128), 1LL * Ho * S, &a, &b)) return 0;
    return a;
}

// Launches the kernel when the problem fits it; *used tells.  `part` must hold rows_dw_max_splits(...) splits.
// *splits_a / *splits_b are the partial counts of taps below / from *tap_split on.
int run_rows_dw(const void* x_sh, int Cin_p, int H, int W, int S, const void* dy_sh, int Cout_p, int Ho, int Wo, int fH,
                int fW, int padH, int padW, float* part, int* splits_a, int* splits_b, int* tap_split, cudaStream_t st,
                bool* used) {
    *used = false;
    if (!rows_dw_shape_ok(Cin_p, Cout_p, Wo, fH, fW)) return AE_OK;
    const int Wp = Wo + fW - 1;
    const int rows_a = 2;
    const int smem_max = 232448;
    const int avail = smem_max - 1024 - 256;
    int BH = 0, stages = 0, ksteps = 0, dyr = 0, xr = 0;
    for (int bh = (Ho < 16 ? Ho : 16); bh >= 1; --bh) {
        if (bh + rows_a - 1 > 256) continue;
        const int ks = ceil_div(bh * Wp, 16);
        const int dyr_b = (int)align_up((size_t)ks * 16 * 128, 1024);
        // the MMAs of filter row r, tap j read x rows up to ks*16 + (rows_a-1)*Wp + fW-1
        const int x_rows = ks * 16 + (rows_a - 1) * Wp + fW;
        const int x_need = (bh + rows_a - 1) * Wp;
        const int xr_b = (int)align_up((size_t)(x_rows > x_need ? x_rows : x_need) * 128, 1024);
        const int stage = 2 * dyr_b + xr_b;
        const int stg = avail / stage;
        if (stg >= 3) { BH = bh; stages = stg > 4 ? 4 : stg; ksteps = ks; dyr = dyr_b; xr = xr_b; break; }
        if (stg >= 2 && BH == 0) { BH = bh; stages = 2; ksteps = ks; dyr = dyr_b; xr = xr_b; }
    }
    if (BH == 0) return AE_OK;
    const int tiles_h = ceil_div(Ho, BH);
    const int units = (Cin_p / 64) * (Cout_p / 128);
    int sa = 0, sb = 0;
    if (!rows_dw_splits(units, 1LL * tiles_h * S, &sa, &sb)) return AE_OK;

    DwRowsParams p;
    memset(&p, 0, sizeof(p));
    int rc;
    if ((rc = make_map_nhwc(&p.tm_x, x_sh, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, Cin_p, W, H, S, 64, Wp, BH + rows_a - 1, 1))) return rc;
    if ((rc = make_map_nhwc(&p.tm_dy, dy_sh, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, Cout_p, Wo, Ho, S, 64, Wp, BH, 1))) return rc;
    p.part = part;
    p.status = device_status_word();
    p.Wp = Wp; p.BH = BH; p.tiles_h = tiles_h; p.n_images = S;
    p.fW = fW; p.fH = fH; p.taps = fH * fW; p.padT = padH; p.padL = padW;
    p.cblocks = Cin_p / 64; p.dblocks = Cout_p / 128; p.ldn = Cout_p;
    p.x_box_rows = (BH + rows_a - 1) * Wp;
    p.dy_box_rows = BH * Wp;
    p.dyr_bytes = dyr; p.xr_bytes = xr; p.stage_bytes = 2 * dyr + xr;
    p.stages = stages; p.ksteps = ksteps;
    p.splits_a = sa; p.splits_b = sb; p.rows_a = rows_a;
    *splits_a = sa; *splits_b = sb; *tap_split = rows_a * fW;
    const int smem = 1024 + p.stages * p.stage_bytes + 256;
    static PerDeviceSmem configured;
    if ((rc = ensure_dynamic_smem(dw_rows_kernel, smem_max, configured, "dw_rows"))) return rc;
    prof_begin(PK_DW, st);
    dw_rows_kernel<<<units * (sa + sb), DWR_THREADS, smem, st>>>(p);
    prof_end(PK_DW, st);
    count_launch();
    *used = true;
    return check_launch("dw_rows_kernel");
}

}  // namespace aether
