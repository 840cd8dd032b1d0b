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
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <utility>

#include "comm.h"
#include "ptx.cuh"

namespace py = pybind11;

namespace soapb200 {
namespace {

bool g_force_scalar_gather = false;   // tests: route every gather through the element-wise kernel

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

// Address of element (gi, gj) of the distributed matrix in the owner's segment.
__device__ __forceinline__ const float* source_address(const DistSource& src, int gi, int gj) {
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
  return base + offset;
}

__device__ __forceinline__ float load_source(const DistSource& src, int gi, int gj) {
  return __ldcg(source_address(src, gi, gj));  // bypass L1: peers rewrite these buffers between launches
}

// Where an output is written as operand planes: hi (fp32) and either lo (fp32) or the interleaved bf16 plane hl.
struct PlaneOut {
  float* hi;
  float* lo;          // null with hl: mixed planes; null without hl: plain copy into `hi`
  uint16_t* hl;
  int64_t d_j16;      // column pitch of the bf16 plane (elements)
};

// Position of element k of hb inside a column of the interleaved bf16 plane (lb: 32 further); as in gemm.h.
__device__ __forceinline__ int64_t plane16(int64_t k) { return ((k >> 5) << 6) | (k & 31); }

__device__ __forceinline__ uint16_t bf16_bits_dev(float v) {
  const __nv_bfloat16 b = __float2bfloat16_rn(v);
  return *reinterpret_cast<const uint16_t*>(&b);
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
                   PlaneOut out, int64_t d_i, int64_t d_j, int rows_out, int cols_out) {
  float* out_hi = out.hi;
  float* out_lo = out.lo;
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
      if (out.hl) {
        const float h = tf32_round_dev(x);
        out_hi[off] = h;
        out.hl[plane16(i) + j * out.d_j16] = bf16_bits_dev(x);          // (mixed planes always have d_i == 1)
        out.hl[plane16(i) + 32 + j * out.d_j16] = bf16_bits_dev(x - h);
      } else if (out_lo) {
        const float h = tf32_round_dev(x);
        out_hi[off] = h;
        out_lo[off] = x - h;
      } else {
        out_hi[off] = x;
      }
    }
  }
}

// ---- 16-byte paths ---------------------------------------------------------------------------------
// Both kernels below need what the host checks before choosing them: no permutation vector along the source's
// contiguous axis (one along the other axis is fine), no triangle mask, output pitch 1 along i with 16-byte aligned columns, and index maps under which four consecutive
// 4-aligned local indices along the source's contiguous axis stay four consecutive 4-aligned global indices
// inside one block / one shard.  A group whose source address still is not 16-byte aligned (a peer whose local
// pitch is odd) or that crosses the end of the output falls back to element loads inside the kernel.
__device__ __forceinline__ float4 load_group(const DistSource& src, bool transpose, int a, int b, int limit) {
  // four elements along the first mapped index a .. a+3 (only the first `limit` are needed)
  const float* p = transpose ? source_address(src, b, a) : source_address(src, a, b);
  if (limit >= 4 && (reinterpret_cast<uintptr_t>(p) & 15) == 0) return __ldcg(reinterpret_cast<const float4*>(p));
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  v.x = __ldcg(p);
  if (limit > 1) v.y = transpose ? load_source(src, b, a + 1) : load_source(src, a + 1, b);
  if (limit > 2) v.z = transpose ? load_source(src, b, a + 2) : load_source(src, a + 2, b);
  if (limit > 3) v.w = transpose ? load_source(src, b, a + 3) : load_source(src, a + 3, b);
  return v;
}

// `keep`: bit e set = element e of the group is written (all four: 0xF).
__device__ __forceinline__ void store_group(const PlaneOut& out, int64_t i, int64_t j, int64_t d_j, const float4& x, int limit,
                                            unsigned keep = 0xFu) {
  float* out_hi = out.hi;
  float* out_lo = out.lo;
  const int64_t off = i + j * d_j;
  if (keep != 0xFu) {
    // a group cut by the triangle mask (plain copies only: the mirrored half of a symmetric matrix)
    const float v[4] = {x.x, x.y, x.z, x.w};
    for (int e = 0; e < limit; ++e)
      if (keep & (1u << e)) out_hi[off + e] = v[e];
    return;
  }
  if (out.hl) {
    const int64_t off16 = plane16(i) + j * out.d_j16;
    const float v[4] = {x.x, x.y, x.z, x.w};
    float h[4], l[4];
    for (int e = 0; e < 4; ++e) {
      h[e] = tf32_round_dev(v[e]);
      l[e] = v[e] - h[e];
    }
    if (limit >= 4) {
      *reinterpret_cast<float4*>(out_hi + off) = make_float4(h[0], h[1], h[2], h[3]);
      const __nv_bfloat162 b0 = __floats2bfloat162_rn(v[0], v[1]), b1 = __floats2bfloat162_rn(v[2], v[3]);
      const __nv_bfloat162 c0 = __floats2bfloat162_rn(l[0], l[1]), c1 = __floats2bfloat162_rn(l[2], l[3]);
      uint2 pb, pc;
      pb.x = *reinterpret_cast<const uint32_t*>(&b0); pb.y = *reinterpret_cast<const uint32_t*>(&b1);
      pc.x = *reinterpret_cast<const uint32_t*>(&c0); pc.y = *reinterpret_cast<const uint32_t*>(&c1);
      *reinterpret_cast<uint2*>(out.hl + off16) = pb;
      *reinterpret_cast<uint2*>(out.hl + off16 + 32) = pc;
    } else {
      for (int e = 0; e < limit; ++e) {
        out_hi[off + e] = h[e];
        out.hl[off16 + e] = bf16_bits_dev(v[e]);
        out.hl[off16 + 32 + e] = bf16_bits_dev(l[e]);
      }
    }
    return;
  }
  if (limit >= 4) {
    if (out_lo) {
      const float4 h = make_float4(tf32_round_dev(x.x), tf32_round_dev(x.y), tf32_round_dev(x.z), tf32_round_dev(x.w));
      *reinterpret_cast<float4*>(out_hi + off) = h;
      *reinterpret_cast<float4*>(out_lo + off) = make_float4(x.x - h.x, x.y - h.y, x.z - h.z, x.w - h.w);
    } else {
      *reinterpret_cast<float4*>(out_hi + off) = x;
    }
    return;
  }
  const float v[4] = {x.x, x.y, x.z, x.w};
  for (int e = 0; e < limit; ++e) {
    if (out_lo) {
      const float h = tf32_round_dev(v[e]);
      out_hi[off + e] = h;
      out_lo[off + e] = v[e] - h;
    } else {
      out_hi[off + e] = v[e];
    }
  }
}

// Source contiguous along i (as the output is): a warp moves 512 contiguous bytes of one output column per
// pass, four passes (four columns) in flight per thread; no shared memory.
constexpr int kCopyTileI = 128, kCopyTileJ = 32;
__global__ void __launch_bounds__(256)
dist_gather_copy16_kernel(DistSource src, IndexMap map_i, IndexMap map_j, int transpose, int upper_only, PlaneOut out,
                          int64_t d_j, int rows_out, int cols_out) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int i = blockIdx.x * kCopyTileI + 4 * lane;
  if (i >= rows_out) return;
  const int limit = min(4, rows_out - i);
  const int a = map_index(map_i, i);
  const int j0 = blockIdx.y * kCopyTileJ + warp;
  float4 v[4];
  unsigned keep[4];
#pragma unroll
  for (int pass = 0; pass < 4; ++pass) {
    const int j = j0 + 8 * pass;
    keep[pass] = 0;
    if (j < cols_out) {
      const int b = map_index(map_j, j);
      // with the triangle mask only entries whose mapped row index is below their mapped column index move
      keep[pass] = upper_only ? ((a < b) | ((a + 1 < b) << 1) | ((a + 2 < b) << 2) | ((a + 3 < b) << 3)) : 0xFu;
      if (keep[pass]) v[pass] = load_group(src, transpose != 0, a, b, limit);
    }
  }
#pragma unroll
  for (int pass = 0; pass < 4; ++pass) {
    const int j = j0 + 8 * pass;
    if (keep[pass]) store_group(out, i, j, d_j, v[pass], limit, keep[pass]);
  }
}

// Source contiguous along j: 64 x 64 tile, read as 256-byte rows along j, turned in shared memory, written
// as 16-byte groups along i.
constexpr int kTurnTile = 64;
__global__ void __launch_bounds__(256)
dist_gather_turn16_kernel(DistSource src, IndexMap map_i, IndexMap map_j, int transpose, int upper_only, PlaneOut out,
                          int64_t d_j, int rows_out, int cols_out) {
  __shared__ float tile[kTurnTile][kTurnTile + 1];   // [i][j]
  const int i0 = blockIdx.x * kTurnTile, j0 = blockIdx.y * kTurnTile;
  const int group = threadIdx.x & 15, line = threadIdx.x >> 4;
  {
    const int j = j0 + 4 * group;
    const int limit = min(4, cols_out - j);
    const int b = (limit > 0) ? map_index(map_j, j) : 0;
    float4 v[4];
#pragma unroll
    for (int pass = 0; pass < 4; ++pass) {
      const int i = i0 + line + 16 * pass;
      v[pass] = make_float4(0.f, 0.f, 0.f, 0.f);
      // the group runs along the SECOND mapped index here: swap the roles for load_group
      if (i < rows_out && limit > 0) {
        const int a = map_index(map_i, i);
        if (!upper_only || a < b + 3) v[pass] = load_group(src, transpose == 0, b, a, limit);   // some element has a < b + e
      }
    }
#pragma unroll
    for (int pass = 0; pass < 4; ++pass) {
      float* row = &tile[line + 16 * pass][4 * group];
      row[0] = v[pass].x; row[1] = v[pass].y; row[2] = v[pass].z; row[3] = v[pass].w;
    }
  }
  __syncthreads();
  const int i = i0 + 4 * group;
  const int limit = min(4, rows_out - i);
  if (limit <= 0) return;
#pragma unroll
  for (int pass = 0; pass < 4; ++pass) {
    const int jl = line + 16 * pass, j = j0 + jl;
    if (j < cols_out) {
      const float4 x = make_float4(tile[4 * group][jl], tile[4 * group + 1][jl], tile[4 * group + 2][jl], tile[4 * group + 3][jl]);
      unsigned keep = 0xFu;
      if (upper_only) {
        const int a = map_index(map_i, i), b = map_index(map_j, j);     // a .. a+3 are consecutive (4-aligned group)
        keep = (a < b) | ((a + 1 < b) << 1) | ((a + 2 < b) << 2) | ((a + 3 < b) << 3);
      }
      if (keep) store_group(out, i, j, d_j, x, limit, keep);
    }
  }
}

// ---- cross-rank barrier ----------------------------------------------------------------------
// `slot0`: first word of this barrier's channel inside every pad (channels let barriers of different streams be in
// flight at the same time without seeing each other's epochs).
__global__ void barrier_kernel(int* const* pads, int rank, int world, int epoch, int* status, long long budget_ns, int slot0) {
  const int peer = threadIdx.x;
  if (peer >= world) return;
  __threadfence_system();
  int* remote = pads[peer] + slot0 + rank;
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
  const int* mine = pads[rank] + slot0 + peer;
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

// ---- one-way flags: a producer rank announces progress, consumer ranks wait for it -----------------
// The flag is an int32 in the PRODUCER's symmetric segment.  `signal_flag_kernel` runs on the producer's stream
// after the work it announces; `wait_flag_kernel` runs on a consumer's stream and polls the producer's memory
// over NVLink with a time budget.  Used only when every rank has its own GPU (a consumer that waited for a
// producer kernel queued behind it on the same GPU would never see the flag).
__global__ void signal_flag_kernel(int* flag, int value) {
  __threadfence_system();
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(flag), "r"(value) : "memory");
}

__global__ void wait_flag_kernel(const int* flag, int value, int* status, long long budget_ns) {
  unsigned long long start, now;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(start));
  for (;;) {
    int seen;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
    if (seen - value >= 0) break;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
    if (static_cast<long long>(now - start) > budget_ns) {
      atomicCAS(status, 0, kStatusPeerFlagTimeout);
      break;
    }
    __nanosleep(500);
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

  auto gather = [](uint64_t peers, int kind, int rows, int cols, int nb_r, int nb_c, int Pr, int Pc, int world, int ip, int iP,
           int inb, int ioff, uint64_t iperm, int jp, int jP, int jnb, int joff, uint64_t jperm, int transpose,
           int upper_only, int i_local_offset, int j_local_offset, uint64_t out_hi, uint64_t out_lo,
           int64_t d_i, int64_t d_j, int rows_out, int cols_out, uint64_t stream, uint64_t out_hl, int64_t d_j16) {
          if (rows_out <= 0 || cols_out <= 0) return;
          PlaneOut out{reinterpret_cast<float*>(out_hi), reinterpret_cast<float*>(out_lo), reinterpret_cast<uint16_t*>(out_hl),
                       d_j16};
          if (out_hl != 0 && d_i != 1) throw std::invalid_argument("dist_gather: mixed planes are written with unit row pitch");
          DistSource src{reinterpret_cast<const float* const*>(peers), kind, rows, cols, nb_r, nb_c, Pr, Pc, world};
          IndexMap mi{ip, iP, inb, ioff, reinterpret_cast<const int64_t*>(iperm), i_local_offset};
          IndexMap mj{jp, jP, jnb, joff, reinterpret_cast<const int64_t*>(jperm), j_local_offset};
          if (!upper_only && d_i != 1 && d_j == 1) {
            // a row-major output is the column-major output of the transposed problem: out'(j, i) = out(i, j)
            std::swap(mi, mj);
            std::swap(rows_out, cols_out);
            std::swap(d_i, d_j);
            transpose = !transpose;
          }
          // consecutive i are consecutive in the source when i indexes the source's contiguous dimension:
          // rows for column-major packed buffers, columns for row-major shards.
          const bool i_is_source_row = !transpose;
          const bool source_row_contiguous = (kind == kBlockCyclic);
          const int read_i_fast = (i_is_source_row == source_row_contiguous) ? 1 : 0;
          cudaStream_t cuda_stream = reinterpret_cast<cudaStream_t>(stream);
          // 16-byte paths: see the comment above load_group for what has to hold
          auto keeps_groups = [](const IndexMap& m) {
            return m.perm == nullptr && m.offset % 4 == 0 && m.local_offset % 4 == 0 && (m.P <= 1 || m.nb % 4 == 0);
          };
          const IndexMap& along = read_i_fast ? mi : mj;     // the map along the source's contiguous axis
          bool source_groups;                                // a 4-aligned global group stays in one block / shard
          if (kind == kBlockCyclic) source_groups = (nb_r % 4 == 0);
          else if (kind == kRowShards) source_groups = (cols % 4 == 0);
          else source_groups = (world > 0 && (cols / world) % 4 == 0);
          const bool aligned_out = d_i == 1 && d_j % 4 == 0 && (out_hi % 16 == 0) && (out_lo % 16 == 0) &&
                                   (out_hl == 0 || (d_j16 % 4 == 0 && out_hl % 8 == 0));
          // the triangle mask needs 4-aligned groups along i to be consecutive global indices as well
          const bool mask_ok = !upper_only || (out_lo == 0 && out_hl == 0 && keeps_groups(mi));
          if (mask_ok && keeps_groups(along) && source_groups && aligned_out && !g_force_scalar_gather) {
            if (read_i_fast) {
              dim3 grid((rows_out + kCopyTileI - 1) / kCopyTileI, (cols_out + kCopyTileJ - 1) / kCopyTileJ);
              dist_gather_copy16_kernel<<<grid, 256, 0, cuda_stream>>>(src, mi, mj, transpose, upper_only, out, d_j, rows_out, cols_out);
              check(cudaGetLastError(), "dist_gather_copy16_kernel");
            } else {
              dim3 grid((rows_out + kTurnTile - 1) / kTurnTile, (cols_out + kTurnTile - 1) / kTurnTile);
              dist_gather_turn16_kernel<<<grid, 256, 0, cuda_stream>>>(src, mi, mj, transpose, upper_only, out, d_j, rows_out, cols_out);
              check(cudaGetLastError(), "dist_gather_turn16_kernel");
            }
            return;
          }
          dim3 grid((rows_out + 31) / 32, (cols_out + 31) / 32);
          dist_gather_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
              src, mi, mj, transpose, read_i_fast, upper_only, out, d_i, d_j, rows_out, cols_out);
          check(cudaGetLastError(), "dist_gather_kernel");
        };
  m.def("dist_gather",
        [gather](uint64_t peers, int kind, int rows, int cols, int nb_r, int nb_c, int Pr, int Pc, int world, int ip, int iP,
                 int inb, int ioff, uint64_t iperm, int jp, int jP, int jnb, int joff, uint64_t jperm, int transpose,
                 int upper_only, int i_local_offset, int j_local_offset, uint64_t out_hi, uint64_t out_lo, int64_t d_i,
                 int64_t d_j, int rows_out, int cols_out, uint64_t stream) {
          gather(peers, kind, rows, cols, nb_r, nb_c, Pr, Pc, world, ip, iP, inb, ioff, iperm, jp, jP, jnb, joff, jperm,
                 transpose, upper_only, i_local_offset, j_local_offset, out_hi, out_lo, d_i, d_j, rows_out, cols_out, stream,
                 0, 0);
        });
  // the same with mixed operand planes as the output: hi (fp32) plus the interleaved bf16 plane (column pitch d_j16)
  m.def("dist_gather_mixed", gather);

  m.def("signal_flag", [](uint64_t flag, int value, uint64_t stream) {
    signal_flag_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(reinterpret_cast<int*>(flag), value);
    check(cudaGetLastError(), "signal_flag_kernel");
  });
  m.def("wait_flag", [](uint64_t flag, int value, uint64_t status, double budget_seconds, uint64_t stream) {
    wait_flag_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const int*>(flag), value, reinterpret_cast<int*>(status), static_cast<long long>(budget_seconds * 1e9));
    check(cudaGetLastError(), "wait_flag_kernel");
  });

  m.def("force_scalar_gather", [](bool on) { g_force_scalar_gather = on; },
        "Route every dist_gather through the element-wise kernel (cross-checks of the 16-byte paths)");

  m.def("device_barrier", [](uint64_t pads, int rank, int world, int epoch, uint64_t status, double budget_seconds,
                             uint64_t stream, int slot0) {
    if (world > 1024) throw std::invalid_argument("device_barrier supports at most 1024 ranks");
    barrier_kernel<<<1, ((world + 31) / 32) * 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<int* const*>(pads), rank, world, epoch, reinterpret_cast<int*>(status),
        static_cast<long long>(budget_seconds * 1e9), slot0);
    check(cudaGetLastError(), "barrier_kernel");
  }, py::arg("pads"), py::arg("rank"), py::arg("world"), py::arg("epoch"), py::arg("status"), py::arg("budget_seconds"),
     py::arg("stream"), py::arg("slot0") = 0);
}

}  // namespace soapb200
