// extern "C" surface of the library: argument validation, dispatch between the tensor-core and the
// CUDA-core convolution, error strings, launch counter, device status word.
#include <atomic>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <mutex>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace aether {

static thread_local char g_err[512] = "";
static std::atomic<unsigned long long> g_launches{0};
static int* g_status_host = nullptr;   // pinned + mapped; the device pointer is identical under UVA

int set_error(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

void count_launch(int n) { g_launches.fetch_add((unsigned long long)n, std::memory_order_relaxed); }

int* device_status_word() {
    static std::once_flag once;
    std::call_once(once, [] {
        int* p = nullptr;
        if (cudaHostAlloc(reinterpret_cast<void**>(&p), sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable) ==
            cudaSuccess) {
            *p = 0;
            g_status_host = p;
        }
    });
    return g_status_host;   // may be null: kernels then skip reporting
}

// One thread waits on a barrier that nothing ever completes, with the same bounded wait the convolution kernels
// use, gives up after `limit` cycles, records its code and returns: the give-up path of every kernel, run alone.
__global__ void selftest_bounded_wait_kernel(int* status, long long limit) {
    __shared__ __align__(8) unsigned long long bar;
    if (threadIdx.x == 0) {
        const uint32_t b = smem_u32(&bar);
        mbar_init(b, 1);
        mbar_fence_init();
        mbar_wait(b, 0, status, DS_TIMEOUT_SELFTEST, limit);
    }
}

int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return set_error(AE_CUDA, "%s: %s", what, cudaGetErrorString(e));
    return AE_OK;
}

// ---- optional kernel timing ------------------------------------------------------------------
static constexpr int PROF_MAX = 2048;          // event pairs per kind; further launches are not timed
struct ProfSlot {
    cudaEvent_t beg[PROF_MAX], end[PROF_MAX];
    int used = 0;
    int seen = 0;        // launches of this kind since profiling was enabled
    bool open = false;   // the launch in progress is being timed
    bool created = false;
};
static ProfSlot g_prof[PK_COUNT];
static bool g_prof_on = false;
static int g_prof_stride = 1;   // every n-th launch of a kind is timed (event records cost stream time themselves)

void prof_begin(int kind, cudaStream_t st) {
    if (!g_prof_on) return;
    ProfSlot& s = g_prof[kind];
    s.open = (s.seen++ % g_prof_stride) == 0 && s.used < PROF_MAX;
    if (s.open) cudaEventRecord(s.beg[s.used], st);
}
void prof_end(int kind, cudaStream_t st) {
    if (!g_prof_on) return;
    ProfSlot& s = g_prof[kind];
    if (s.open) {
        cudaEventRecord(s.end[s.used], st);
        ++s.used;
        s.open = false;
    }
}

static int validate_desc(const AetherConvDesc* d, const char* fn) {
    if (!d) return set_error(AE_BAD_ARG, "%s: null descriptor", fn);
    if (d->S <= 0 || d->H <= 0 || d->W <= 0 || d->Cin <= 0 || d->Cout <= 0 || d->fH <= 0 || d->fW <= 0 || d->sH <= 0 ||
        d->sW <= 0 || d->padH < 0 || d->padW < 0)
        return set_error(AE_BAD_ARG, "%s: non-positive dimension in descriptor", fn);
    if (d->math_mode < AETHER_MATH_BF16 || d->math_mode > AETHER_MATH_FP32)
        return set_error(AE_BAD_ARG, "%s: unknown math_mode %d", fn, d->math_mode);
    int Ho, Wo;
    conv_out_hw(*d, Ho, Wo);
    if (d->H + 2 * d->padH < d->fH || d->W + 2 * d->padW < d->fW || Ho < 1 || Wo < 1)
        return set_error(AE_BAD_ARG, "%s: filter %dx%d larger than padded input %dx%d", fn, d->fH, d->fW,
                         d->H + 2 * d->padH, d->W + 2 * d->padW);
    return AE_OK;
}

static int pending_timeout(const char* fn) {
    if (g_status_host && *reinterpret_cast<volatile int*>(g_status_host) != 0)
        return set_error(AE_DEVICE_TIMEOUT, "%s: an earlier kernel abandoned a bounded wait (status %d)", fn,
                         *reinterpret_cast<volatile int*>(g_status_host));
    return AE_OK;
}

}  // namespace aether

using namespace aether;

int aether_conv2d_fwd_bnstats_flags(const AetherConvDesc* d, const float* x, const float* w, const float* b, float* y,
                                    float* stats, size_t stats_bytes, void* ws, size_t ws_bytes, int flags, void* stream);

extern "C" int aether_version(void) { return 101; }
extern "C" const char* aether_last_error(void) { return g_err; }
extern "C" uint64_t aether_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }
extern "C" int aether_device_status(void) { return g_status_host ? *reinterpret_cast<volatile int*>(g_status_host) : 0; }
extern "C" void aether_device_status_clear(void) {
    if (g_status_host) *reinterpret_cast<volatile int*>(g_status_host) = 0;
}

extern "C" int aether_selftest_bounded_wait(int64_t limit_cycles, void* stream) {
    if (limit_cycles < 1 || limit_cycles > 2000000000LL)
        return set_error(AE_BAD_ARG, "aether_selftest_bounded_wait: limit_cycles must be in [1, 2e9] (about a second at most)");
    int* status = device_status_word();
    if (!status) return set_error(AE_CUDA, "aether_selftest_bounded_wait: no status word (pinned allocation failed)");
    selftest_bounded_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(status, (long long)limit_cycles);
    count_launch();
    return check_launch("selftest_bounded_wait_kernel");
}

extern "C" int aether_profile_enable(int on) {
    if (on) {
        for (int k = 0; k < PK_COUNT; ++k) {
            ProfSlot& s = g_prof[k];
            if (!s.created) {
                for (int i = 0; i < PROF_MAX; ++i) {
                    if (cudaEventCreate(&s.beg[i]) != cudaSuccess || cudaEventCreate(&s.end[i]) != cudaSuccess)
                        return set_error(AE_CUDA, "aether_profile_enable: cudaEventCreate failed");
                }
                s.created = true;
            }
            s.used = 0;
            s.seen = 0;
            s.open = false;
        }
        g_prof_stride = on > 0 ? on : 1;
    }
    g_prof_on = on != 0;
    return AE_OK;
}

extern "C" int aether_profile_read(int kind, double* total_ms, int* launches) {
    if (kind < 0 || kind >= PK_COUNT || !total_ms || !launches)
        return set_error(AE_BAD_ARG, "aether_profile_read: bad argument");
    ProfSlot& s = g_prof[kind];
    double tot = 0.0;
    for (int i = 0; i < s.used; ++i) {
        float ms = 0.f;
        cudaError_t e = cudaEventSynchronize(s.end[i]);
        if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, s.beg[i], s.end[i]);
        if (e != cudaSuccess) return set_error(AE_CUDA, "aether_profile_read: %s", cudaGetErrorString(e));
        tot += ms;
    }
    *total_ms = tot;
    *launches = s.used;
    return AE_OK;
}

extern "C" void aether_profile_reset(void) {
    for (int k = 0; k < PK_COUNT; ++k) g_prof[k].used = g_prof[k].seen = 0;
}

extern "C" size_t aether_conv2d_workspace_bytes(const AetherConvDesc* d) {
    if (validate_desc(d, "aether_conv2d_workspace_bytes")) return 0;
    size_t g = generic_conv_workspace_bytes(*d);
    if (smallc_conv_eligible(*d)) {
        size_t s = smallc_conv_workspace_bytes(*d);
        if (s > g) g = s;
    }
    if (first_tc_bwd_eligible(*d)) {
        size_t s = first_tc_bwd_workspace_bytes(*d);
        if (s > g) g = s;
    }
    if (tc_conv_eligible(*d)) {
        size_t t = tc_conv_workspace_bytes(*d);
        return t > g ? t : g;
    }
    return g;
}

extern "C" int aether_conv2d_operand_layout(const AetherConvDesc* d, AetherOperandLayout* out) {
    if (!out) return 0;
    memset(out, 0, sizeof(*out));
    if (validate_desc(d, "aether_conv2d_operand_layout")) return 0;
    if (tc_conv_eligible(*d)) return tc_conv_operand_layout(*d, out) ? 1 : 0;
    return first_tc_operand_layout(*d, out) ? 1 : 0;       // first layers: a copy of dy only (x_copy_ld == 0)
}

extern "C" int aether_conv2d_fwd_ex(const AetherConvDesc* d, const float* x, const float* w, const float* b, float* y,
                                    float* stats, size_t stats_bytes, void* ws, size_t ws_bytes, int flags, void* stream) {
    int rc = validate_desc(d, "aether_conv2d_fwd_ex");
    if (rc) return rc;
    if (flags & ~AETHER_CONV_X_COPY_READY) return set_error(AE_BAD_ARG, "aether_conv2d_fwd_ex: unknown flag bits 0x%x", flags);
    if ((flags & AETHER_CONV_X_COPY_READY) && !(tc_conv_eligible(*d) && d->math_mode == AETHER_MATH_BF16))
        return set_error(AE_UNSUPPORTED, "aether_conv2d_fwd_ex: this shape / math mode reads no operand copy of x "
                                         "(aether_conv2d_operand_layout returned 0)");
    if (stats) return aether_conv2d_fwd_bnstats_flags(d, x, w, b, y, stats, stats_bytes, ws, ws_bytes, flags, stream);
    if (!x || !w || !y) return set_error(AE_BAD_ARG, "aether_conv2d_fwd_ex: null pointer");
    if (!aligned16(x) || !aligned16(w) || !aligned16(y) || (ws && !aligned16(ws)))
        return set_error(AE_BAD_ARG, "aether_conv2d_fwd_ex: arrays must be 16-byte aligned");
    if ((rc = pending_timeout("aether_conv2d_fwd_ex"))) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (tc_conv_eligible(*d)) return tc_conv_fwd(*d, x, w, b, y, nullptr, ws, ws_bytes, flags, st);
    return aether_conv2d_fwd(d, x, w, b, y, ws, ws_bytes, stream);
}

extern "C" int aether_conv2d_fwd(const AetherConvDesc* d, const float* x, const float* w, const float* b, float* y,
                                 void* ws, size_t ws_bytes, void* stream) {
    int rc = validate_desc(d, "aether_conv2d_fwd");
    if (rc) return rc;
    if (!x || !w || !y) return set_error(AE_BAD_ARG, "aether_conv2d_fwd: null pointer");
    if (!aligned16(x) || !aligned16(w) || !aligned16(y) || (ws && !aligned16(ws)))
        return set_error(AE_BAD_ARG, "aether_conv2d_fwd: arrays must be 16-byte aligned");
    if ((rc = pending_timeout("aether_conv2d_fwd"))) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (tc_conv_eligible(*d)) return tc_conv_fwd(*d, x, w, b, y, nullptr, ws, ws_bytes, 0, st);
    if (first_tc_eligible(*d)) return first_tc_fwd(*d, x, w, b, y, nullptr, st);
    if (smallc_conv_eligible(*d) && (!b || aligned16(b))) return smallc_conv_fwd(*d, x, w, b, y, nullptr, st);
    return generic_conv_fwd(*d, x, w, b, y, st);
}

extern "C" int64_t aether_conv2d_bnstats_blocks(const AetherConvDesc* d) {
    if (validate_desc(d, "aether_conv2d_bnstats_blocks")) return 0;
    if (tc_conv_eligible(*d)) return tc_conv_stats_blocks(*d);
    if (first_tc_eligible(*d)) return first_tc_stats_blocks(*d);
    if (smallc_conv_eligible(*d)) return smallc_conv_stats_blocks(*d);
    return 0;
}

extern "C" int aether_conv2d_fwd_bnstats(const AetherConvDesc* d, const float* x, const float* w, const float* b, float* y,
                                         float* stats, size_t stats_bytes, void* ws, size_t ws_bytes, void* stream) {
    return aether_conv2d_fwd_bnstats_flags(d, x, w, b, y, stats, stats_bytes, ws, ws_bytes, 0, stream);
}

int aether_conv2d_fwd_bnstats_flags(const AetherConvDesc* d, const float* x, const float* w, const float* b, float* y,
                                    float* stats, size_t stats_bytes, void* ws, size_t ws_bytes, int flags, void* stream) {
    int rc = validate_desc(d, "aether_conv2d_fwd_bnstats");
    if (rc) return rc;
    if (!x || !w || !y || !stats) return set_error(AE_BAD_ARG, "aether_conv2d_fwd_bnstats: null pointer");
    if (!aligned16(x) || !aligned16(w) || !aligned16(y) || !aligned16(stats) || (b && !aligned16(b)) || (ws && !aligned16(ws)))
        return set_error(AE_BAD_ARG, "aether_conv2d_fwd_bnstats: arrays must be 16-byte aligned");
    const int64_t blocks = aether_conv2d_bnstats_blocks(d);
    if (blocks <= 0)
        return set_error(AE_UNSUPPORTED, "aether_conv2d_fwd_bnstats: the forward kernel of this shape does not emit statistics "
                                         "(aether_conv2d_bnstats_blocks returned 0); use aether_conv2d_fwd");
    if (stats_bytes < (size_t)blocks * 3 * d->Cout * sizeof(float))
        return set_error(AE_BAD_ARG, "aether_conv2d_fwd_bnstats: statistics buffer too small: %zu < %zu", stats_bytes,
                         (size_t)blocks * 3 * d->Cout * sizeof(float));
    if ((rc = pending_timeout("aether_conv2d_fwd_bnstats"))) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (tc_conv_eligible(*d)) return tc_conv_fwd(*d, x, w, b, y, stats, ws, ws_bytes, flags, st);
    if (first_tc_eligible(*d)) return first_tc_fwd(*d, x, w, b, y, stats, st);
    return smallc_conv_fwd(*d, x, w, b, y, stats, st);
}

extern "C" int aether_conv2d_bwd(const AetherConvDesc* d, const float* x, const float* dy, const float* w, float* dx,
                                 float* dw, float* db, void* ws, size_t ws_bytes, int x_shadow_valid, void* stream) {
    if (x_shadow_valid & AETHER_CONV_DY_COPY_READY)
        return set_error(AE_BAD_ARG, "aether_conv2d_bwd: AETHER_CONV_DY_COPY_READY needs aether_conv2d_bwd_ex (row count)");
    return aether_conv2d_bwd_ex(d, x, dy, w, dx, dw, db, ws, ws_bytes, x_shadow_valid, 0, stream);
}

extern "C" int aether_conv2d_bwd_ex(const AetherConvDesc* d, const float* x, const float* dy, const float* w, float* dx,
                                    float* dw, float* db, void* ws, size_t ws_bytes, int x_shadow_valid,
                                    int dy_colsum_rows, void* stream) {
    int rc = validate_desc(d, "aether_conv2d_bwd");
    if (rc) return rc;
    if (!dy || !w || ((dw != nullptr) && !x)) return set_error(AE_BAD_ARG, "aether_conv2d_bwd: null pointer");
    if (!aligned16(x) || !aligned16(dy) || !aligned16(w) || !aligned16(dx) || !aligned16(dw) || (ws && !aligned16(ws)))
        return set_error(AE_BAD_ARG, "aether_conv2d_bwd: arrays must be 16-byte aligned");
    if ((rc = pending_timeout("aether_conv2d_bwd"))) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool dy_ready = (x_shadow_valid & AETHER_CONV_DY_COPY_READY) != 0;
    if (dy_ready && !((tc_conv_eligible(*d) && d->math_mode == AETHER_MATH_BF16) || (first_tc_bwd_eligible(*d) && !dx && dw)))
        return set_error(AE_UNSUPPORTED, "aether_conv2d_bwd_ex: this shape / math mode / request reads no operand copy of dy "
                                         "(aether_conv2d_operand_layout returned 0, or a first layer asked for dx)");
    if (tc_conv_eligible(*d)) return tc_conv_bwd(*d, x, dy, w, dx, dw, db, ws, ws_bytes, x_shadow_valid, dy_colsum_rows, st);
    if (dx && (rc = generic_conv_bwd_data(*d, dy, w, dx, st))) return rc;
    if (dw && first_tc_bwd_eligible(*d))
        return first_tc_bwd_filter(*d, x, dy, dw, db, ws, ws_bytes, dy_ready ? dy_colsum_rows : 0, st);
    if ((dw || db) && smallc_conv_eligible(*d) && (!db || aligned16(db)))
        return smallc_conv_bwd_filter(*d, x, dy, dw, db, ws, ws_bytes, st);
    if (dw || db) return generic_conv_bwd_filter(*d, x, dy, dw, db, ws, ws_bytes, st);
    return AE_OK;
}
