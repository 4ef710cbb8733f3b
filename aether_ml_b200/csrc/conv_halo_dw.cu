// Halo-reuse filter gradient (dW) for stride-1 convolutions on wide images, bf16 operands.
//
//   dW[tap][c][d] = sum over output pixels p of x[p + tap][c] * dy[p][d]        (CNN_classes_cupy.py:134)
//
// A CTA owns one 64-channel block of x and one 64-channel block of dy and walks over strips of BH output
// rows of the images assigned to it.  Per strip ONE TMA box brings the x window ((BH+fH-1) rows by
// Wp = Wo+fW-1 columns, zero filled outside the image) and one box the dy strip (BH rows by Wp columns;
// the fW-1 extra columns are out of range, hence zero) into shared memory; pixel q = row*Wp + col sits in
// row q of a 128-byte-swizzled MN-major operand (rows = reduction index).  Because both windows use the
// same pitch Wp, the x operand of filter tap (i,j) is the x window read from row i*Wp + j on: every tap
// re-reads the same shared memory through a row-shifted descriptor, and the zero columns of dy cancel the
// wrap-around rows.  Two taps are stacked into one M=128 MMA (the descriptor's leading-dimension offset is
// the row distance between the two taps), so a 3x3 filter needs five MMAs per 16 reduction rows and their
// accumulators (5 x 64 TMEM columns) stay resident for the whole kernel.  Partial sums per CTA go to the
// split workspace and are reduced in fixed order by dw_reduce_kernel.
#include <string.h>

#include "common.cuh"
#include "sm100_ptx.cuh"
#include "tc_host.cuh"

namespace aether {

struct DwHaloParams {
    CUtensorMap tm_x;    // (Cin_p, W, H, N) bf16, box (64, Wp, BH+fH-1, 1)
    CUtensorMap tm_dy;   // (Cout_p, Wo, Ho, N) bf16, box (64, Wp, BH, 1)
    float* part;         // [splits][taps*cblocks][64][ldn]
    int* status;
    int Ho, Wp, BH, tiles_h, n_images;
    int fH, fW, padT, padL;
    int cblocks, dblocks, ldn;
    int xr_rows, dyr_rows;        // rows written by the two boxes
    int xr_bytes, stage_bytes;    // x region size (1 KiB multiple), stage size
    int stages, ksteps, npairs;
};

static constexpr int DWH_THREADS = 192;   // warp 0 producer, warp 1 MMA issuer, warps 2..5 epilogue

__global__ void __launch_bounds__(DWH_THREADS, 1) dw_halo_kernel(const __grid_constant__ DwHaloParams p) {
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

    // Rows that no TMA box ever writes (the tail of each dy region up to a multiple of 16 rows) must read as zero.
    {
        uint4* z = reinterpret_cast<uint4*>(gen_base);
        const int n16 = S * p.stage_bytes / 16;
        for (int i = threadIdx.x; i < n16; i += blockDim.x) z[i] = make_uint4(0, 0, 0, 0);
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

    const int split = blockIdx.x, splits = gridDim.x;
    const int cb = blockIdx.y / p.dblocks;
    const int db = blockIdx.y % p.dblocks;
    const int taps = p.fH * p.fW;
    const long long total_strips = 1LL * p.tiles_h * p.n_images;
    const uint32_t stage_tx = (uint32_t)(p.xr_rows + p.dyr_rows) * 128u;

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
                tma_load_4d(base, &p.tm_x, full_bar(s), cb * 64, -p.padL, h0 - p.padT, n);
                tma_load_4d(base + p.xr_bytes, &p.tm_dy, full_bar(s), db * 64, 0, h0, n);
            }
        }
    } else if (warp == 1) {
        // The whole warp runs the loop (warp-uniform descriptor arithmetic); one elected lane issues.
        const bool leader = elect_one();
        constexpr uint32_t idesc = make_idesc(1u, 1u, 1u, 128u, 64u);           // bf16, A and B MN-major, M=128, N=64
        const uint32_t hi = (uint32_t)(make_smem_desc(0, 0, 1024) >> 32);       // SBO = 1024 (8 reduction rows), 128B swizzle
        // per pair of taps: row offset of the first tap and distance to the second (leading-dimension offset),
        // packed as the low descriptor word without the start address
        uint32_t pair_lo[8];
#pragma unroll
        for (int pr = 0; pr < 8; ++pr) {
            int ta = 2 * pr, tb = 2 * pr + 1;
            if (tb >= taps) { tb = taps - 1; ta = taps - 2; }           // odd tap count: last pair repeats a tap
            if (ta < 0) ta = 0;
            const uint32_t offa = (uint32_t)((ta / p.fW) * p.Wp + (ta % p.fW));
            const uint32_t offb = (uint32_t)((tb / p.fW) * p.Wp + (tb % p.fW));
            pair_lo[pr] = (offa * 8u) + (((offb - offa) * 8u) << 16);
        }
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
            const uint32_t xr16 = ((smem_base + s * p.stage_bytes) & 0x3FFFFu) >> 4;
            uint32_t a_k = xr16;                                                 // advances 16 reduction rows per step
            uint32_t b_lo = xr16 + ((uint32_t)p.xr_bytes >> 4);                  // one 64-channel block: LBO unused
            for (int kk = 0; kk < p.ksteps; ++kk) {
#pragma unroll
                for (int pr = 0; pr < 8; ++pr) {
                    if (pr < p.npairs && leader) {
                        asm volatile(
                            "{\n\t.reg .pred pp;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 pp, %5, 0;\n\t"
                            "mov.b64 da, {%1, %4};\n\tmov.b64 db, {%2, %4};\n\t"
                            "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, pp;\n\t}"
                            ::"r"(tmem_base + (uint32_t)pr * 64u), "r"(a_k + pair_lo[pr]), "r"(b_lo), "r"(idesc), "r"(hi),
                              "r"(acc)
                            : "memory");
                    }
                }
                acc = 1u;
                a_k += 128u;
                b_lo += 128u;
            }
            if (leader) umma_commit(empty_bar(s));
            __syncwarp();
        }
        if (leader) umma_commit(done_bar);
        __syncwarp();
    } else {
        const int q = warp & 3;
        const int row = q * 32 + lane;
        const bool any = split < total_strips;
        bool ok = true;
        if (any) ok = mbar_wait(done_bar, 0, p.status, DS_TIMEOUT_TMEM_FULL);
        tc_fence_after();
        if (ok) {
            const int m = row >> 6, c_in = row & 63;
            for (int pr = 0; pr < p.npairs; ++pr) {
                int ta = 2 * pr, tb = 2 * pr + 1;
                bool dup = false;
                if (tb >= taps) { tb = taps - 1; ta = taps - 2; dup = true; }
                const int tap = m ? tb : ta;
                const bool write = !(dup && m == 0);                             // the repeated tap was already stored
#pragma unroll 1
                for (int ch = 0; ch < 2; ++ch) {
                    uint32_t r[32];
                    if (any) {
                        tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + pr * 64 + ch * 32, r);
                        tmem_ld_wait();
                    } else {
#pragma unroll
                        for (int k = 0; k < 32; ++k) r[k] = 0u;
                    }
                    if (write) {
                        float4* dst = reinterpret_cast<float4*>(
                            p.part + (((size_t)split * (taps * p.cblocks) + (size_t)tap * p.cblocks + cb) * 64 + c_in) * (size_t)p.ldn +
                            db * 64 + ch * 32);
#pragma unroll
                        for (int k = 0; k < 8; ++k)
                            dst[k] = make_float4(__uint_as_float(r[4 * k]), __uint_as_float(r[4 * k + 1]),
                                                 __uint_as_float(r[4 * k + 2]), __uint_as_float(r[4 * k + 3]));
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

// Launches the halo dW kernel when the problem fits it (bf16 shadows with 64-channel blocks); *used tells.
// `part` must hold splits * taps * cblocks * 64 * ldn floats; the chosen split count is returned in *splits_out.
int run_halo_dw(const void* x_sh, int Cin_p, int H, int W, int S, const void* dy_sh, int Cout_p, int Ho, int Wo, int fH,
                int fW, int padH, int padW, float* part, int max_splits, int* splits_out, cudaStream_t st, bool* used) {
    *used = false;
    const int taps = fH * fW;
    if (taps < 2 || taps > 16) return AE_OK;
    if (Cin_p % 64 || Cout_p % 64) return AE_OK;
    const int Wp = Wo + fW - 1;
    if (Wp > 256 || Wo < 12) return AE_OK;
    const int npairs = (taps + 1) / 2;
    const int smem_max = 232448;
    const int avail = smem_max - 1024 - 256;
    int best_bh = 0, best_stages = 0;
    for (int bh = (Ho < 16 ? Ho : 16); bh >= 1; --bh) {
        if (bh + fH - 1 > 256) continue;
        const int xr = (int)align_up((size_t)(bh + fH - 1) * Wp * 128, 1024);
        const int ks = ceil_div(bh * Wp, 16);
        const int stage = xr + (int)align_up((size_t)ks * 16 * 128, 1024);
        const int stg = avail / stage;
        if (stg >= 3) { best_bh = bh; best_stages = stg > 4 ? 4 : stg; break; }
        if (stg >= 2 && best_bh == 0) { best_bh = bh; best_stages = 2; }
    }
    if (best_bh == 0) return AE_OK;
    const int BH = best_bh;
    DwHaloParams p;
    memset(&p, 0, sizeof(p));
    int rc;
    if ((rc = make_map_nhwc(&p.tm_x, x_sh, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, Cin_p, W, H, S, 64, Wp, BH + fH - 1, 1))) return rc;
    if ((rc = make_map_nhwc(&p.tm_dy, dy_sh, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, Cout_p, Wo, Ho, S, 64, Wp, BH, 1))) return rc;
    p.part = part;
    p.status = device_status_word();
    p.Ho = Ho; p.Wp = Wp; p.BH = BH; p.tiles_h = ceil_div(Ho, BH); p.n_images = S;
    p.fH = fH; p.fW = fW; p.padT = padH; p.padL = padW;
    p.cblocks = Cin_p / 64; p.dblocks = Cout_p / 64; p.ldn = Cout_p;
    p.xr_rows = (BH + fH - 1) * Wp;
    p.dyr_rows = BH * Wp;
    p.xr_bytes = (int)align_up((size_t)p.xr_rows * 128, 1024);
    p.ksteps = ceil_div(BH * Wp, 16);
    p.stage_bytes = p.xr_bytes + (int)align_up((size_t)p.ksteps * 16 * 128, 1024);
    p.stages = best_stages;
    p.npairs = npairs;
    const long long strips = 1LL * p.tiles_h * S;
    const int gy = p.cblocks * p.dblocks;
    long long splits = num_sms() / gy;
    if (splits < 1) splits = 1;
    if (splits > strips) splits = strips;
    if (splits > max_splits) splits = max_splits;
    *splits_out = (int)splits;
    const int smem = 1024 + p.stages * p.stage_bytes + 256;
    static PerDeviceSmem configured;
    if (int rc0 = ensure_dynamic_smem(dw_halo_kernel, smem_max, configured, "dw_halo")) return rc0;
    prof_begin(PK_DW, st);
    dw_halo_kernel<<<dim3((unsigned)splits, gy), DWH_THREADS, smem, st>>>(p);
    prof_end(PK_DW, st);
    count_launch();
    *used = true;
    return check_launch("dw_halo_kernel");
}

}  // namespace aether
