// Allocation-free entry point.  This file has no counterpart in the reference project.
//
// Who needs it: code that may not (or cannot) call cudaMalloc when it wants a panel factored --
// a host thread that is inside a CUDA-graph stream capture (allocation is illegal there), a plug-in
// running under a framework that owns every byte of device memory and forbids side allocations, a
// real-time loop that must not take the allocator's locks, or a process whose memory pool is already
// carved up to the last megabyte.  The regular path (`qr_panel` in qr.h) expects the caller to hand
// in a scratch buffer for the exchange between thread blocks; such callers have nowhere to get one.
//
// What it does: `soapb200_qr_panel_noalloc` factors one panel exactly like `qr_panel`, but the
// exchange scratch lives in a fixed array inside this library's device image.
//
// Limits and rules
//   * at most SOAPB200_NOALLOC_MAX_ROWS rows and 128 columns per call; larger panels are refused with
//     a message, nothing is launched;
//   * the array (about 130 KB) exists once per GPU that loads the library and stays until the process
//     exits;
//   * it is shared by every call and still holds what the previous call left there; the entry point
//     re-arms the part it is going to use before launching, on the caller's stream.  Two calls whose
//     kernels can run at the same time on one GPU (different streams, no ordering) would trample each
//     other's exchange words -- order them;
//   * the first call on each device looks up the array's device address.  Make that first call
//     outside any stream capture, and from one host thread: the per-device table of looked-up addresses
//     is not protected by a lock, so two threads that both make the FIRST call for a device race on it
//     (later calls only read the table);
//   * no cudaMalloc, cudaFree or other allocating routine is called, here or in what it calls.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define SOAPB200_NOALLOC_MAX_ROWS 16384
#define SOAPB200_NOALLOC_MAX_COLS 128

// Householder-factor the rows x cols panel given as hi/lo planes (column-major, pitch ldp floats).
// Outputs (all caller-owned device memory): V planes (rows x cols, pitch ldv), V^T planes (cols x rows,
// pitch ldvt), tau[cols], T and T^T planes (cols x cols, pitch ldt); `status` is a device int that stays
// 0 unless a bounded wait inside the kernel ran out.  `stream` is a cudaStream_t (may be null).
// Returns 0 on success.  On failure returns a non-zero code and, if `message` is not null, writes a
// NUL-terminated explanation of at most `message_capacity` bytes.
int soapb200_qr_panel_noalloc(const float* p_hi, const float* p_lo, long long ldp, int rows, int cols, float* v_hi,
                              float* v_lo, long long ldv, float* vt_hi, float* vt_lo, long long ldvt, float* tau,
                              float* t_hi, float* t_lo, float* tt_hi, float* tt_lo, long long ldt, int* status,
                              void* stream, char* message, int message_capacity);

#ifdef __cplusplus
}
#endif
