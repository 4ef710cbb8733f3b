// Shared host-side plumbing of the library: error reporting, the device status word that
// bounded waits report into, the launch counter, and the internal entry points of each .cu file.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include <atomic>

#include "../../include/aether_b200.h"

namespace aether {

// Return codes of every extern "C" entry point (0 = success).
enum : int {
    AE_OK = 0,
    AE_BAD_ARG = -1,       // null pointer, misaligned pointer, non-positive size, workspace too small
    AE_UNSUPPORTED = -2,   // shape/mode the library has no kernel for
    AE_CUDA = -3,          // a CUDA runtime/driver call failed
    AE_DEVICE_TIMEOUT = -4 // an earlier kernel gave up a bounded wait (see aether_device_status)
};

int set_error(int code, const char* fmt, ...);
void count_launch(int n = 1);
// Pinned, device-visible int that kernels write a DeviceStatus code into; allocated once per process.
int* device_status_word();
// Checks cudaGetLastError after a launch; returns AE_OK or AE_CUDA (with message).
int check_launch(const char* what);

// Optional per-kernel timing (off by default): CUDA events recorded around selected launches on the
// launch stream, read back through aether_profile_read.
enum ProfKind : int { PK_IGEMM_FWD = 0, PK_IGEMM_DX = 1, PK_DW = 2, PK_SHADOW = 3, PK_COUNT = 4 };
void prof_begin(int kind, cudaStream_t st);
void prof_end(int kind, cudaStream_t st);

// ---- per-device state.  Kernel attributes (the opt-in to more than 48 KB of dynamic shared memory) and the SM
// count belong to a device, not to the process: a host that drives several GPUs from one process, or switches
// device between calls, gets each of them configured on first use.  The flags are atomics, so any number of host
// threads may call into the library (a doubled cudaFuncSetAttribute is harmless).
static constexpr int AE_MAX_DEVICES = 64;
static inline int current_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= AE_MAX_DEVICES) dev = 0;
    return dev;
}
struct PerDeviceSmem {
    std::atomic<int> bytes[AE_MAX_DEVICES];      // largest dynamic shared-memory size configured so far (0: none)
};
// Makes sure `kernel` may be launched with `bytes` of dynamic shared memory on the current device.
template <typename K>
static inline int ensure_dynamic_smem(K kernel, int bytes, PerDeviceSmem& once, const char* what) {
    const int dev = current_device();
    if (once.bytes[dev].load(std::memory_order_acquire) >= bytes) return AE_OK;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return set_error(AE_CUDA, "cudaFuncSetAttribute(%s, %d): %s", what, bytes, cudaGetErrorString(e));
    once.bytes[dev].store(bytes, std::memory_order_release);
    return AE_OK;
}

static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- conv_generic.cu : fp32 CUDA-core convolution for any filter/stride/padding
int generic_conv_fwd(const AetherConvDesc& d, const float* x, const float* w, const float* b, float* y, cudaStream_t st);
int generic_conv_bwd_data(const AetherConvDesc& d, const float* dy, const float* w, float* dx, cudaStream_t st);
int generic_conv_bwd_filter(const AetherConvDesc& d, const float* x, const float* dy, float* dw, float* db, void* ws,
                            size_t ws_bytes, cudaStream_t st);
size_t generic_conv_workspace_bytes(const AetherConvDesc& d);

// ---- conv_smallc.cu : fp32 first-layer convolution (1..4 input channels, fH*fW*Cin <= 64): forward, dW, dB
bool smallc_conv_eligible(const AetherConvDesc& d);
size_t smallc_conv_workspace_bytes(const AetherConvDesc& d);
int smallc_conv_fwd(const AetherConvDesc& d, const float* x, const float* w, const float* b, float* y, float* stats,
                    cudaStream_t st);
long long smallc_conv_stats_blocks(const AetherConvDesc& d);
int smallc_conv_bwd_filter(const AetherConvDesc& d, const float* x, const float* dy, float* dw, float* db, void* ws,
                           size_t ws_bytes, cudaStream_t st);

// ---- conv_first_tc.cu : first-layer forward on tensor cores (bf16 mode, thread-built im2col operand)
bool first_tc_eligible(const AetherConvDesc& d);
long long first_tc_stats_blocks(const AetherConvDesc& d);
int first_tc_fwd(const AetherConvDesc& d, const float* x, const float* w, const float* b, float* y, float* stats,
                 cudaStream_t st);
bool first_tc_bwd_eligible(const AetherConvDesc& d);
int first_tc_bwd_filter(const AetherConvDesc& d, const float* x, const float* dy, float* dw, float* db, void* ws,
                        size_t ws_bytes, int dy_colsum_rows, cudaStream_t st);
size_t first_tc_bwd_workspace_bytes(const AetherConvDesc& d);
bool first_tc_operand_layout(const AetherConvDesc& d, AetherOperandLayout* out);
// out[c] = sum over `rows` rows of part[row][C] in fixed order (conv_tc.cu)
int colsum_finish(const float* part, int rows, int C, float* out, cudaStream_t st);
int smallc_reduce_partials(const float* part, int nb, int K, int Cout, float* dw, float* db, cudaStream_t st);

// ---- conv_tc.cu : tcgen05 implicit-GEMM convolution (stride 1)
bool tc_conv_eligible(const AetherConvDesc& d);
size_t tc_conv_workspace_bytes(const AetherConvDesc& d);
// `stats` (nullable): per-block (count, mean, M2) of every output channel, tc_conv_stats_blocks(d) blocks of [3][Cout]
int tc_conv_fwd(const AetherConvDesc& d, const float* x, const float* w, const float* b, float* y, float* stats, void* ws,
                size_t ws_bytes, int flags, cudaStream_t st);
bool tc_conv_operand_layout(const AetherConvDesc& d, AetherOperandLayout* out);
long long tc_conv_stats_blocks(const AetherConvDesc& d);
int tc_conv_bwd(const AetherConvDesc& d, const float* x, const float* dy, const float* w, float* dx, float* dw,
                float* db, void* ws, size_t ws_bytes, int x_shadow_valid, int dy_colsum_rows, cudaStream_t st);

// ---- layers.cu : pieces of Batch_Norm shared with block_fused.cu
int bn_partial_blocks(long long rows);
float* bn_forward_coeffs(const float* x, const float* partials, long long nblocks, const float* gamma, const float* beta,
                         float* running_mean, float* running_var, float* batch_mean, float* batch_var, long long rows,
                         int C, float eps, float momentum, const float* channel_scale, float* ws, cudaStream_t st);
float* bn_eval_coeffs(const float* gamma, const float* beta, const float* running_mean, const float* running_var, int C,
                      float eps, float* ws, cudaStream_t st);
void bn_backward_coeffs(const float* part, int nb, int C, long long rows, const float* gamma, const float* mean,
                        const float* var, float eps, float* dgamma, float* dbeta, float* coeff, const float* pscale,
                        cudaStream_t st);

static inline void conv_out_hw(const AetherConvDesc& d, int& Ho, int& Wo) {
    Ho = (d.H + 2 * d.padH - d.fH) / d.sH + 1;
    Wo = (d.W + 2 * d.padW - d.fW) / d.sW + 1;
}

}  // namespace aether
