// Symmetric-memory communicator over CUDA IPC and the kernels that move data between ranks.
//
// The reference talks to its peers through torch.distributed collectives issued tile by tile from
// Python (src/soap_tp/ops/preconditioners.py:339-406, src/soap_tp/ops/optimizer.py:362-368) and
// through MPI inside SLATE/ELPA.  Here every rank exports a set of device buffers ("symmetric
// segments": same size and meaning on every rank) with cudaIpcGetMemHandle; peers map them with
// cudaIpcOpenMemHandle, and kernels then read a peer's buffer with ordinary global loads that
// travel over NVLink/NVSwitch.  All data movement is PULL: a rank only ever reads its peers'
// segments and writes its own memory, so the only cross-rank hazards are "data ready" and "buffer
// free", both covered by the barrier below.
//
//   dist_gather_kernel  out(i, j) = source(map_i(i), map_j(j)), optionally transposed, where source
//                       is a matrix spread over the ranks (packed 2-D block-cyclic, or contiguous
//                       tensor-parallel row/column shards) and the maps are block-cyclic
//                       local->global maps optionally composed with a permutation vector.  Output
//                       is either a plain strided matrix or the hi/lo operand planes of the 3xTF32
//                       GEMM (all-gather fused with the operand split).  With `upper_only` only
//                       entries whose mapped row is above their mapped column are written (pull
//                       of the mirrored half of a symmetric matrix).
//   barrier_kernel      one flag per peer in each rank's signal pad, release store to every peer,
//                       bounded acquire spin on the own pad.  Used only when every rank has its own
//                       GPU; ranks that share a GPU order themselves on the host instead.
#include <cuda_runtime.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>

#include "comm.h"
#include "ptx.cuh"

namespace py = pybind11;

namespace soapb200 {
namespace {

void check(cudaError_t err, const char* what) {
  if (err != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(err));
}

// ---- distributed source description ----------------------------------------------------------
enum SourceKind : int { kBlockCyclic = 0, kRowShards = 1, kColShards = 2 };

struct DistSource {
  const float* const* peers;  // device array [world] of segment base pointers (element 0 of the matrix storage)
  int kind;
  int rows, cols;             // global shape
  int nb_r, nb_c, Pr, Pc;     // block-cyclic parameters (kBlockCyclic): row/column block sizes, grid
  int world;                  // number of shards (kRowShards / kColShards)
};

struct IndexMap {
  int p, P, nb;               // local -> global: g = ((l / nb) * P + p) * nb + l % nb   (P == 1: identity)
  int offset;                 // then g <- g + offset
  const int64_t* perm;        // optional, last: g <- perm[g]
  int local_offset;           // first of all: l <- l + local_offset (a chunk of the local index range)
};

__device__ __forceinline__ int map_index(const IndexMap& map, int local) {
  local += map.local_offset;
  int g = local;
  if (map.P > 1) g = ((local / map.nb) * map.P + map.p) * map.nb + local % map.nb;
  g += map.offset;
  if (map.perm) g = static_cast<int>(map.perm[g]);
  return g;
}

__device__ __forceinline__ int numroc_dev(int n, int nb, int p, int P) {
  const int full = n / nb, rem = n % nb;
  int count = (full / P) * nb;
  const int extra = full % P;
  if (p < extra) count += nb; else if (p == extra) count += rem;
  return count;
}

__device__ __forceinline__ float load_source(const DistSource& src, int gi, int gj) {
  const float* base;
  int64_t offset;
  if (src.kind == kBlockCyclic) {
    const int bi = gi / src.nb_r, bj = gj / src.nb_c;
    const int pr = bi % src.Pr, pc = bj % src.Pc;
    const int li = (bi / src.Pr) * src.nb_r + gi % src.nb_r;
    const int lj = (bj / src.Pc) * src.nb_c + gj % src.nb_c;
    int ld = numroc_dev(src.rows, src.nb_r, pr, src.Pr);
    if (ld < 1) ld = 1;
    base = src.peers[pr * src.Pc + pc];
    offset = li + static_cast<int64_t>(lj) * ld;
  } else if (src.kind == kRowShards) {
    const int per = src.rows / src.world;
    base = src.peers[gi / per];
    offset = static_cast<int64_t>(gi % per) * src.cols + gj;
  } else {
    const int per = src.cols / src.world;
    base = src.peers[gj / per];
    offset = static_cast<int64_t>(gi) * per + gj % per;
  }
  return __ldcg(base + offset);  // bypass L1: peers rewrite these buffers between launches
}

__device__ __forceinline__ float tf32_round_dev(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

// out(i, j), i < rows_out, j < cols_out.  Source element: transpose ? (map_j(j), map_i(i)) read as
// source(row = map_j(j), col = map_i(i)) : source(row = map_i(i), col = map_j(j)).
// read_i_fast tells whether consecutive i touch consecutive source addresses (chosen by the host).
__global__ void __launch_bounds__(256)
dist_gather_kernel(DistSource src, IndexMap map_i, IndexMap map_j, int transpose, int read_i_fast, int upper_only,
                   float* out_hi, float* out_lo, int64_t d_i, int64_t d_j, int rows_out, int cols_out) {
  __shared__ float tile[32][33];
  const int i0 = blockIdx.x * 32, j0 = blockIdx.y * 32;
  const int tx = threadIdx.x % 32, ty = threadIdx.x / 32;
  for (int t = ty; t < 32; t += 8) {
    const int i = read_i_fast ? i0 + tx : i0 + t;
    const int j = read_i_fast ? j0 + t : j0 + tx;
    float val = 0.f;
    if (i < rows_out && j < cols_out) {
      const int a = map_index(map_i, i), b = map_index(map_j, j);
      if (!upper_only || a < b) val = transpose ? load_source(src, b, a) : load_source(src, a, b);
    }
    if (read_i_fast) tile[t][tx] = val; else tile[tx][t] = val;
  }
  __syncthreads();
  for (int t = ty; t < 32; t += 8) {
    const int i = i0 + tx, j = j0 + t;
    if (i < rows_out && j < cols_out && (!upper_only || map_index(map_i, i) < map_index(map_j, j))) {
      const float x = tile[t][tx];
      const int64_t off = i * d_i + j * d_j;
      if (out_lo) {
        const float h = tf32_round_dev(x);
        out_hi[off] = h;
        out_lo[off] = x - h;
      } else {
        out_hi[off] = x;
      }
    }
  }
}

// ---- cross-rank barrier ----------------------------------------------------------------------
__global__ void barrier_kernel(int* const* pads, int rank, int world, int epoch, int* status, long long budget_ns) {
  const int peer = threadIdx.x;
  if (peer >= world) return;
  __threadfence_system();
  int* remote = pads[peer] + rank;
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
  const int* mine = pads[rank] + peer;
  unsigned long long start, now;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(start));
  for (;;) {
    int seen;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
    if (seen - epoch >= 0) break;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
    if (static_cast<long long>(now - start) > budget_ns) {
      atomicCAS(status, 0, kStatusBarrierTimeout);
      break;
    }
    __nanosleep(200);
  }
  __threadfence_system();
}

}  // namespace

void register_comm(py::module_& m) {
  m.def("ipc_alloc", [](int64_t bytes) {
    void* ptr = nullptr;
    check(cudaMalloc(&ptr, static_cast<size_t>(bytes < 256 ? 256 : bytes)), "cudaMalloc(symmetric segment)");
    check(cudaMemset(ptr, 0, static_cast<size_t>(bytes < 256 ? 256 : bytes)), "cudaMemset(symmetric segment)");
    cudaIpcMemHandle_t handle;
    check(cudaIpcGetMemHandle(&handle, ptr), "cudaIpcGetMemHandle");
    return py::make_tuple(reinterpret_cast<uint64_t>(ptr), py::bytes(reinterpret_cast<const char*>(&handle), sizeof(handle)));
  });
  m.def("ipc_open", [](const std::string& raw) {
    if (raw.size() != sizeof(cudaIpcMemHandle_t)) throw std::invalid_argument("bad IPC handle size");
    cudaIpcMemHandle_t handle;
    memcpy(&handle, raw.data(), sizeof(handle));
    void* ptr = nullptr;
    check(cudaIpcOpenMemHandle(&ptr, handle, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
    return reinterpret_cast<uint64_t>(ptr);
  });
  m.def("ipc_close", [](uint64_t ptr) { check(cudaIpcCloseMemHandle(reinterpret_cast<void*>(ptr)), "cudaIpcCloseMemHandle"); });
  m.def("ipc_free", [](uint64_t ptr) { check(cudaFree(reinterpret_cast<void*>(ptr)), "cudaFree"); });
  m.def("device_uuid", [](int device) {
    cudaDeviceProp prop;
    check(cudaGetDeviceProperties(&prop, device), "cudaGetDeviceProperties");
    return py::bytes(reinterpret_cast<const char*>(prop.uuid.bytes), 16);
  });

  m.def("dist_gather",
        [](uint64_t peers, int kind, int rows, int cols, int nb_r, int nb_c, int Pr, int Pc, int world, int ip, int iP,
           int inb, int ioff, uint64_t iperm, int jp, int jP, int jnb, int joff, uint64_t jperm, int transpose,
           int upper_only, int i_local_offset, int j_local_offset, uint64_t out_hi, uint64_t out_lo,
           int64_t d_i, int64_t d_j, int rows_out, int cols_out, uint64_t stream) {
          if (rows_out <= 0 || cols_out <= 0) return;
          DistSource src{reinterpret_cast<const float* const*>(peers), kind, rows, cols, nb_r, nb_c, Pr, Pc, world};
          IndexMap mi{ip, iP, inb, ioff, reinterpret_cast<const int64_t*>(iperm), i_local_offset};
          IndexMap mj{jp, jP, jnb, joff, reinterpret_cast<const int64_t*>(jperm), j_local_offset};
          // consecutive i are consecutive in the source when i indexes the source's contiguous dimension:
          // rows for column-major packed buffers, columns for row-major shards.
          const bool i_is_source_row = !transpose;
          const bool source_row_contiguous = (kind == kBlockCyclic);
          const int read_i_fast = (i_is_source_row == source_row_contiguous) ? 1 : 0;
          dim3 grid((rows_out + 31) / 32, (cols_out + 31) / 32);
          dist_gather_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
              src, mi, mj, transpose, read_i_fast, upper_only, reinterpret_cast<float*>(out_hi), reinterpret_cast<float*>(out_lo), d_i,
              d_j, rows_out, cols_out);
          check(cudaGetLastError(), "dist_gather_kernel");
        });

  m.def("device_barrier", [](uint64_t pads, int rank, int world, int epoch, uint64_t status, double budget_seconds,
                             uint64_t stream) {
    if (world > 1024) throw std::invalid_argument("device_barrier supports at most 1024 ranks");
    barrier_kernel<<<1, ((world + 31) / 32) * 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<int* const*>(pads), rank, world, epoch, reinterpret_cast<int*>(status),
        static_cast<long long>(budget_seconds * 1e9));
    check(cudaGetLastError(), "barrier_kernel");
  });
}

}  // namespace soapb200
