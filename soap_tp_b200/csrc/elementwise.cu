// Memory-bound kernels of the SOAP pipeline: fused Adam, the 3xTF32 operand split (optionally
// transposing), column dot products for the eigenvalue estimates, and index-mapped gathers.
#include <stdexcept>
#include <string>

#include <cuda_bf16.h>

#include "elementwise.h"
#include "gemm.h"
#include "launch_util.h"

namespace soapb200 {
namespace {

inline void check_launch(const char* what) {
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(err));
}

__device__ __forceinline__ float tf32_hi(float x, int nearest) {
  if (nearest) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
  }
  return __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);
}

// ---- Adam ---------------------------------------------------------------------------------
// One pass over g, m, v (column-major with independent pitches); the reference issues ten elementwise
// launches for the same arithmetic (src/soap_tp/ops/optimizer.py:36-44).
__global__ void adam_kernel(const float* __restrict__ g, int64_t ldg, float* __restrict__ m, int64_t ldm,
                            float* __restrict__ v, int64_t ldv, float* __restrict__ u, int64_t ldu, int rows, int cols,
                            float beta1, float beta2, float eps, float inv_bc1, float inv_sqrt_bc2) {
  const int64_t total = static_cast<int64_t>(rows) * cols;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i % rows);
    const int64_t c = i / rows;
    const float gi = g[r + c * ldg];
    const float mo = fmaf(beta1, m[r + c * ldm], (1.0f - beta1) * gi);
    const float va = fmaf(beta2, v[r + c * ldv], (1.0f - beta2) * gi * gi);
    m[r + c * ldm] = mo;
    v[r + c * ldv] = va;
    u[r + c * ldu] = (mo * inv_bc1) / (sqrtf(va) * inv_sqrt_bc2 + eps);
  }
}

// Same arithmetic, four elements per thread with 16-byte accesses; used when all four matrices are dense
// (pitch == rows) and 16-byte aligned, i.e. one flat array each.
__global__ void adam_flat4_kernel(const float4* __restrict__ g, float4* __restrict__ m, float4* __restrict__ v,
                                  float4* __restrict__ u, int64_t quads, float beta1, float beta2, float eps, float inv_bc1,
                                  float inv_sqrt_bc2) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < quads;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const float4 gi = g[i];
    float4 mo = m[i], va = v[i], out;
#define SOAP_ADAM_LANE(c)                                              \
    mo.c = fmaf(beta1, mo.c, (1.0f - beta1) * gi.c);                   \
    va.c = fmaf(beta2, va.c, (1.0f - beta2) * gi.c * gi.c);            \
    out.c = (mo.c * inv_bc1) / (sqrtf(va.c) * inv_sqrt_bc2 + eps);
    SOAP_ADAM_LANE(x) SOAP_ADAM_LANE(y) SOAP_ADAM_LANE(z) SOAP_ADAM_LANE(w)
#undef SOAP_ADAM_LANE
    m[i] = mo;
    v[i] = va;
    u[i] = out;
  }
}

// ---- operand split --------------------------------------------------------------------------
// out(i, j) = src[i*s_i + j*s_j] for i < rows, j < cols, written as hi/lo planes with i contiguous
// (pitch ldo).  A 32x33 shared tile makes both the read and the write coalesced whichever of s_i,
// s_j is the unit stride, so the same kernel splits in place-order and transposes.
__device__ __forceinline__ uint16_t bf16_bits(float v) {
  const __nv_bfloat16 b = __float2bfloat16_rn(v);
  return *reinterpret_cast<const uint16_t*>(&b);
}

// With `hl` (interleaved bf16 plane, pitch ld16, see gemm.h) the low part is written there as bf16(x) and
// bf16(x - hi) instead of `lo`: the operand format of the GEMM's mixed-precision corrections.
__global__ void __launch_bounds__(256) split_planes_kernel(const float* __restrict__ src, int64_t s_i, int64_t s_j,
                                                           float* __restrict__ hi, float* __restrict__ lo, int64_t ldo,
                                                           int rows, int cols, float scale, int nearest,
                                                           uint16_t* __restrict__ hl, int64_t ld16) {
  __shared__ float tile[32][33];
  const int i0 = blockIdx.x * 32, j0 = blockIdx.y * 32;
  const int tx = threadIdx.x % 32, ty = threadIdx.x / 32;  // 32 x 8
  const bool read_i_fast = (s_i <= s_j);
  for (int t = ty; t < 32; t += 8) {
    const int i = read_i_fast ? i0 + tx : i0 + t;
    const int j = read_i_fast ? j0 + t : j0 + tx;
    float val = 0.f;
    if (i < rows && j < cols) val = src[i * s_i + j * s_j];
    if (read_i_fast) tile[t][tx] = val; else tile[tx][t] = val;  // tile[j - j0][i - i0]
  }
  __syncthreads();
  for (int t = ty; t < 32; t += 8) {
    const int i = i0 + tx, j = j0 + t;
    if (i < rows && j < cols) {
      const float x = tile[t][tx] * scale;
      const float h = tf32_hi(x, nearest);
      hi[i + j * ldo] = h;
      if (hl != nullptr) {
        const int64_t at = bf16_plane_index(i) + j * ld16;
        hl[at] = bf16_bits(x);
        hl[at + 32] = bf16_bits(x - h);
      } else {
        lo[i + j * ldo] = x - h;
      }
    }
  }
}

// ---- column dots: out[j] = sum_i a[i, j] * b[i, j] -----------------------------------------
__global__ void __launch_bounds__(256) column_dot_kernel(const float* __restrict__ a, int64_t lda,
                                                         const float* __restrict__ b, int64_t ldb,
                                                         float* __restrict__ out, int rows, int cols) {
  const int j = blockIdx.x;
  if (j >= cols) return;
  float acc = 0.f;
  for (int i = threadIdx.x; i < rows; i += blockDim.x) acc = fmaf(a[i + j * lda], b[i + j * ldb], acc);
  __shared__ float partial[256];
  partial[threadIdx.x] = acc;
  __syncthreads();
  for (int s = 128; s > 0; s >>= 1) {
    if (threadIdx.x < s) partial[threadIdx.x] += partial[threadIdx.x + s];
    __syncthreads();
  }
  if (threadIdx.x == 0) out[j] = partial[0];
}

// ---- stable descending order of column sums ------------------------------------------------------
// estimates[j] = sum_r table[r + j * ld] (r < parts, fixed order); order = indices sorted by descending estimate, ties by
// ascending index (what a stable descending argsort returns).  One CTA, bitonic sort of (value, index) pairs in shared
// memory; `padded` is the power of two >= n that the launch was sized for.
__global__ void __launch_bounds__(1024) order_by_estimate_kernel(const float* __restrict__ table, int64_t ld, int parts,
                                                                 int n, int padded, int64_t* __restrict__ order) {
  extern __shared__ unsigned char sort_raw[];
  float* keys = reinterpret_cast<float*>(sort_raw);
  int* index = reinterpret_cast<int*>(keys + padded);
  for (int j = threadIdx.x; j < padded; j += blockDim.x) {
    float total = -INFINITY;                       // padding sorts to the end
    if (j < n) {
      total = 0.f;
      for (int r = 0; r < parts; ++r) total += table[r + j * ld];
      if (total != total) total = -INFINITY;       // a NaN estimate goes last instead of poisoning the network
    }
    keys[j] = total;
    index[j] = j;
  }
  __syncthreads();
  // "a precedes b" in the wanted order: larger value first, smaller index first among equals
  auto precedes = [](float va, int ia, float vb, int ib) { return va > vb || (va == vb && ia < ib); };
  for (int size = 2; size <= padded; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int t = threadIdx.x; t < padded / 2; t += blockDim.x) {
        const int lo = 2 * t - (t & (stride - 1));
        const int hi = lo + stride;
        const bool ascending_block = (lo & size) == 0;        // blocks alternate direction
        const float va = keys[lo], vb = keys[hi];
        const int ia = index[lo], ib = index[hi];
        const bool in_order = precedes(va, ia, vb, ib);
        if (in_order != ascending_block) {
          keys[lo] = vb; keys[hi] = va;
          index[lo] = ib; index[hi] = ia;
        }
      }
      __syncthreads();
    }
  }
  for (int j = threadIdx.x; j < n; j += blockDim.x) order[j] = index[j];
}

// ---- gather: dst(i, j) = src(row_map[i], col_map[j]) with null maps meaning identity ----------
__global__ void gather2d_kernel(const float* __restrict__ src, int64_t s_i, int64_t s_j, float* __restrict__ dst,
                                int64_t d_i, int64_t d_j, const int64_t* __restrict__ row_map,
                                const int64_t* __restrict__ col_map, int rows, int cols) {
  const int64_t total = static_cast<int64_t>(rows) * cols;
  for (int64_t t = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; t < total;
       t += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int i = static_cast<int>(t % rows);
    const int j = static_cast<int>(t / rows);
    const int64_t si = row_map ? row_map[i] : i;
    const int64_t sj = col_map ? col_map[j] : j;
    dst[i * d_i + j * d_j] = src[si * s_i + sj * s_j];
  }
}

inline int grid_for(int64_t total, int threads) {
  int64_t blocks = (total + threads - 1) / threads;
  const int64_t cap = 148 * 16;
  return static_cast<int>(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

}  // namespace

void adam_update(const float* g, int64_t ldg, float* m, int64_t ldm, float* v, int64_t ldv, float* u, int64_t ldu,
                 int rows, int cols, float beta1, float beta2, float eps, float inv_bc1, float inv_sqrt_bc2,
                 cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return;
  const int64_t total = static_cast<int64_t>(rows) * cols;
  const bool dense = (cols == 1 || (ldg == rows && ldm == rows && ldv == rows && ldu == rows)) && total % 4 == 0;
  const bool aligned = ((reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v) |
                         reinterpret_cast<uintptr_t>(u)) & 15) == 0;
  if (dense && aligned) {
    adam_flat4_kernel<<<grid_for(total / 4, 256), 256, 0, stream>>>(
        reinterpret_cast<const float4*>(g), reinterpret_cast<float4*>(m), reinterpret_cast<float4*>(v),
        reinterpret_cast<float4*>(u), total / 4, beta1, beta2, eps, inv_bc1, inv_sqrt_bc2);
    check_launch("adam_flat4_kernel");
    return;
  }
  adam_kernel<<<grid_for(static_cast<int64_t>(rows) * cols, 256), 256, 0, stream>>>(
      g, ldg, m, ldm, v, ldv, u, ldu, rows, cols, beta1, beta2, eps, inv_bc1, inv_sqrt_bc2);
  check_launch("adam_kernel");
}

void split_planes(const float* src, int64_t s_i, int64_t s_j, float* hi, float* lo, int64_t ldo, int rows, int cols,
                  float scale, int nearest, cudaStream_t stream, uint16_t* hl, int64_t ld16) {
  if (rows <= 0 || cols <= 0) return;
  dim3 grid((rows + 31) / 32, (cols + 31) / 32);
  split_planes_kernel<<<grid, 256, 0, stream>>>(src, s_i, s_j, hi, lo, ldo, rows, cols, scale, nearest, hl, ld16);
  check_launch("split_planes_kernel");
}

void column_dot(const float* a, int64_t lda, const float* b, int64_t ldb, float* out, int rows, int cols,
                cudaStream_t stream) {
  if (cols <= 0) return;
  column_dot_kernel<<<cols, 256, 0, stream>>>(a, lda, b, ldb, out, rows, cols);
  check_launch("column_dot_kernel");
}

void order_by_estimate(const float* table, int64_t ld, int parts, int n, int64_t* order, cudaStream_t stream) {
  if (n <= 0) return;
  int padded = 1;
  while (padded < n) padded <<= 1;
  if (padded > kOrderMaxLength) throw std::invalid_argument("order_by_estimate: more entries than one CTA's shared memory sorts");
  const size_t smem = static_cast<size_t>(padded) * (sizeof(float) + sizeof(int));
  static PerDeviceOnce configured;
  allow_dynamic_smem(reinterpret_cast<const void*>(order_by_estimate_kernel), kOrderMaxLength * 8, configured, "order_by_estimate");
  order_by_estimate_kernel<<<1, 1024, smem, stream>>>(table, ld, parts, n, padded, order);
  check_launch("order_by_estimate_kernel");
}

void gather2d(const float* src, int64_t s_i, int64_t s_j, float* dst, int64_t d_i, int64_t d_j, const int64_t* row_map,
              const int64_t* col_map, int rows, int cols, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return;
  gather2d_kernel<<<grid_for(static_cast<int64_t>(rows) * cols, 256), 256, 0, stream>>>(src, s_i, s_j, dst, d_i, d_j,
                                                                                     row_map, col_map, rows, cols);
  check_launch("gather2d_kernel");
}

}  // namespace soapb200
