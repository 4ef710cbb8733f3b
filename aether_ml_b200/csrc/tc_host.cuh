// Host-side helpers shared by the tensor-core convolution files.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

namespace aether {

int num_sms();
// Whether this device can co-schedule the CTA pairs (clusters of two CTAs with ~210 KB of shared memory each) the
// cta_group::2 kernels are launched as, on every pair of SMs; looked up once per device.  False keeps the single-CTA forms.
bool cta_pairs_available();
// NHWC tensor seen as 4-D (C, W, H, N), box (box_c, BW, BH, BN); 128-byte swizzle unless told otherwise.
int make_map_nhwc(CUtensorMap* m, const void* base, CUtensorMapDataType dt, int elt, int C, int W, int H, int N,
                  int box_c, int BW, int BH, int BN, CUtensorMapSwizzle swz = CU_TENSOR_MAP_SWIZZLE_128B);
// Row-major matrix (inner = K elements contiguous, `rows` rows), box (box_k, box_rows), 128-byte swizzle.
int make_map_2d(CUtensorMap* m, const void* base, CUtensorMapDataType dt, int elt, int inner, long long rows, int box_k,
                int box_rows);
// Halo-reuse kernel (conv_halo.cu): launches and sets *used when the problem fits it, else leaves *used false.
int run_halo_igemm(bool tf32, const void* in, int in_C, int in_H, int in_W, int S, const void* wmat, int w_inner,
                   int rows_per_tap, int taps, float* out, int out_C, int out_H, int out_W, int n_padded, int fH, int fW,
                   int padT, int padL, int flip, const float* bias, float* stats, int prof_kind, cudaStream_t st,
                   bool* used);
// Partial-statistics blocks ([block][3][out_C]: count, mean, M2) the halo kernel writes when `stats` is given; 0 when
// the halo kernel does not take the problem.
long long halo_igemm_stats_blocks(bool tf32, int in_C, int S, int taps, int out_C, int out_H, int out_W, int n_padded,
                                  int fH, int fW);

// Halo-reuse dW kernel (conv_halo_dw.cu), bf16 shadows with 64-channel blocks.  `part` must have room for
// max_splits split slices; the split count actually used is returned in *splits_out.
int run_halo_dw(const void* x_sh, int Cin_p, int H, int W, int S, const void* dy_sh, int Cout_p, int Ho, int Wo, int fH,
                int fW, int padH, int padW, float* part, int max_splits, int* splits_out, cudaStream_t st, bool* used);

// conv_dw_rows.cu: dW with dy as the M operand and the taps of a filter row as N (3-row filters, bf16).
int rows_dw_max_splits(int Cin_p, int Cout_p, int Ho, int Wo, int S, int fH, int fW);
int run_rows_dw(const void* x_sh, int Cin_p, int H, int W, int S, const void* dy_sh, int Cout_p, int Ho, int Wo, int fH,
                int fW, int padH, int padW, float* part, int* splits_a, int* splits_b, int* tap_split, cudaStream_t st,
                bool* used);

}  // namespace aether
