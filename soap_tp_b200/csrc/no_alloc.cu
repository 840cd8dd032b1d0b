// Allocation-free panel factorisation (see no_alloc.h for who needs it and the rules of use).
#include "no_alloc.h"

#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <exception>

#include "qr.h"

namespace {

constexpr int kMaxBlocks = (SOAPB200_NOALLOC_MAX_ROWS + soapb200::kQrRowsPerCta - 1) / soapb200::kQrRowsPerCta;
// Two parities x (one slot row per thread block + one for the pivot row) x 128 columns of 8-byte words.
constexpr size_t kScratchWords = 2ull * (kMaxBlocks + 1) * 128;

// The exchange scratch.  In host code this name is only a handle: the device address comes from
// cudaGetSymbolAddress, once per device, below.
static __device__ __align__(256) unsigned long long g_exchange[kScratchWords];

constexpr int kMaxDevices = 64;
unsigned long long* g_exchange_address[kMaxDevices] = {};

int fail(int code, char* message, int capacity, const char* text) {
  if (message != nullptr && capacity > 0) {
    std::strncpy(message, text, static_cast<size_t>(capacity) - 1);
    message[capacity - 1] = '\0';
  }
  return code;
}

}  // namespace

extern "C" __attribute__((visibility("default"))) int soapb200_qr_panel_noalloc(
    const float* p_hi, const float* p_lo, long long ldp, int rows, int cols, float* v_hi, float* v_lo, long long ldv,
    float* vt_hi, float* vt_lo, long long ldvt, float* tau, float* t_hi, float* t_lo, float* tt_hi, float* tt_lo,
    long long ldt, int* status, void* stream, char* message, int message_capacity) {
  char text[256];
  if (rows <= 0 || cols <= 0) return fail(1, message, message_capacity, "soapb200_qr_panel_noalloc: empty panel");
  if (rows > SOAPB200_NOALLOC_MAX_ROWS || cols > SOAPB200_NOALLOC_MAX_COLS) {
    std::snprintf(text, sizeof(text),
                  "soapb200_qr_panel_noalloc: a %d x %d panel exceeds the built-in scratch (at most %d rows, %d columns); "
                  "use qr_panel with a caller-provided exchange buffer",
                  rows, cols, SOAPB200_NOALLOC_MAX_ROWS, SOAPB200_NOALLOC_MAX_COLS);
    return fail(2, message, message_capacity, text);
  }
  if (!p_hi || !p_lo || !v_hi || !v_lo || !vt_hi || !vt_lo || !tau || !t_hi || !t_lo || !tt_hi || !tt_lo || !status)
    return fail(3, message, message_capacity, "soapb200_qr_panel_noalloc: null pointer argument");

  int device = -1;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess || device < 0 || device >= kMaxDevices) {
    std::snprintf(text, sizeof(text), "soapb200_qr_panel_noalloc: cudaGetDevice failed or device %d unsupported: %s", device,
                  cudaGetErrorString(err));
    return fail(4, message, message_capacity, text);
  }
  // Set-up, once per device, with that device current: resolve the device address of the scratch.
  if (g_exchange_address[device] == nullptr) {
    unsigned long long* address = nullptr;
    err = cudaGetSymbolAddress(reinterpret_cast<void**>(&address), g_exchange);
    if (err != cudaSuccess || address == nullptr) {
      std::snprintf(text, sizeof(text), "soapb200_qr_panel_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(err));
      return fail(5, message, message_capacity, text);
    }
    g_exchange_address[device] = address;
  }
  unsigned long long* exchange = g_exchange_address[device];
  cudaStream_t cuda_stream = static_cast<cudaStream_t>(stream);

  // The array still holds the previous call's words.  Re-arm the part this launch will poll so that
  // no stale sequence number can be mistaken for a fresh one.
  const int blocks = (rows + soapb200::kQrRowsPerCta - 1) / soapb200::kQrRowsPerCta;
  const size_t used_bytes = 2ull * (blocks + 1) * 128 * sizeof(unsigned long long);
  err = cudaMemsetAsync(exchange, 0, used_bytes, cuda_stream);
  if (err != cudaSuccess) {
    std::snprintf(text, sizeof(text), "soapb200_qr_panel_noalloc: clearing the scratch failed: %s", cudaGetErrorString(err));
    return fail(6, message, message_capacity, text);
  }
  try {
    soapb200::qr_panel(p_hi, p_lo, ldp, rows, cols, v_hi, v_lo, ldv, vt_hi, vt_lo, ldvt, tau, t_hi, t_lo, tt_hi, tt_lo, ldt,
                       reinterpret_cast<float*>(exchange), status, cuda_stream);
  } catch (const std::exception& error) {
    return fail(7, message, message_capacity, error.what());
  }
  if (message != nullptr && message_capacity > 0) message[0] = '\0';
  return 0;
}
