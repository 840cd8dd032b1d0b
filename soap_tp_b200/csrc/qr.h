// Host-side interface of the blocked Householder QR building blocks (qr.cu).
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace soapb200 {

constexpr int kQrPanelWidth = 128;     // columns factored per panel (also the GEMM K of the updates)
constexpr int kQrRowsPerCta = 256;     // rows of the panel held in one CTA's shared memory
constexpr int kQrMaxRows = 148 * kQrRowsPerCta;  // one CTA per SM at most (cooperative launch)

// Factor one panel: the r x b matrix given as hi/lo planes (column-major, pitch ldp) is reduced by
// b Householder reflectors H_c = I - tau_c v_c v_c^T (v_c[c] = 1, zeros above).
// Outputs, all as operand planes unless noted: V (r x b, unit lower trapezoid, pitch ldv), V^T
// (b x r, pitch ldvt), tau[b] (plain), and the triangular factor of the compact WY form
// H_0 ... H_{b-1} = I - V T V^T in both orientations (T and T^T, b x b, pitch ldt).
// `exchange` is 8-byte-aligned scratch of at least 4 * (gridsize + 1) * 128 floats that persists
// between calls; `status` is the device status word a timed-out exchange reports to.  Cooperative
// launch of ceil(r / 256) CTAs.  `trace` (optional, 16 x int64) receives clock64 stamps of one column step and
// `debug_skip` switches parts of the step off, both only in a build with -DSOAP_QR_TRACE.
void qr_panel(const float* p_hi, const float* p_lo, int64_t ldp, int r, int b, float* v_hi, float* v_lo, int64_t ldv,
              float* vt_hi, float* vt_lo, int64_t ldvt, float* tau, float* t_hi, float* t_lo, float* tt_hi, float* tt_lo,
              int64_t ldt, float* exchange, int* status, cudaStream_t stream, long long* trace = nullptr,
              int debug_skip = 0);

// Same contract, two Householder columns per exchange step where that is numerically safe (see
// qr_panel_pairs.cu).  `rows_per_cta` is 256 (fewest SMs) or 128 (fastest: twice the CTAs, half the registers
// per thread taken by the slab); the grid is ceil(r / rows_per_cta) CTAs.  `exchange` must hold at least
// 8 * (gridsize + 1) * 128 floats, 16-byte aligned.  `steps_taken` (optional, device) receives the number of
// exchange steps the panel needed (b / 2 when every step retired two columns).
void qr_panel_pairs(const float* p_hi, const float* p_lo, int64_t ldp, int r, int b, float* v_hi, float* v_lo, int64_t ldv,
                    float* vt_hi, float* vt_lo, int64_t ldvt, float* tau, float* t_hi, float* t_lo, float* tt_hi,
                    float* tt_lo, int64_t ldt, float* exchange, int* status, cudaStream_t stream,
                    int rows_per_cta = 256, long long* steps_taken = nullptr);

// planes <- sum over `splits` partial matrices (rows x cols, column-major pitch ld, `stride` floats apart).
void sum_partials_to_planes(const float* partials, int splits, int64_t stride, int64_t ld, float* hi, float* lo,
                            int64_t ldp, int rows, int cols, cudaStream_t stream);

// planes <- columns first_col .. first_col + cols - 1 of the rows x rows identity.
void identity_planes(float* hi, float* lo, int64_t ldp, int rows, int cols, cudaStream_t stream, int first_col = 0);

// out[c * ldo + k] = hi[k + c * ldp] + lo[k + c * ldp] for k < depth, c < cols (the fp32 values behind operand
// planes, every plane column as one contiguous row of `out`).
void planes_sum(const float* hi, const float* lo, int64_t ldp, float* out, int64_t ldo, int depth, int cols,
                cudaStream_t stream);

}  // namespace soapb200
