// Codes that kernels of this library store in the device status word when a bounded wait gives up or
// an argument is unusable.  The first code wins (atomicCAS from 0); the host reads the word after the
// stream has drained, or one step later through a pinned copy (engine/kernels.py).
#pragma once

namespace soapb200 {

enum StatusCode : int {
  kStatusOk = 0,
  kStatusTmaWaitTimeout = 1,          // GEMM consumer never saw a full stage
  kStatusSlotWaitTimeout = 2,         // GEMM producer never got an empty stage back
  kStatusAccumWaitTimeout = 3,        // GEMM epilogue never saw the accumulator commit
  kStatusBarrierTimeout = 4,          // cross-rank barrier flag never arrived
  kStatusBadArgument = 5,
  kStatusPanelExchangeTimeout = 6,    // QR panel: a poll of the exchange between its thread blocks ran out
  kStatusPeerFlagTimeout = 7,         // a wait for a peer's "data ready" flag ran out
  kStatusGridBarrierTimeout = 8,      // tridiagonalisation: a barrier over the CTAs of the launch ran out
};

}  // namespace soapb200
