// Host-side interface of the GEMM kernels (gemm_tf32x3.cu, gemm_simt.cu).
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace soapb200 {

enum EpilogueMode : int {
  kEpiStore = 0,     // C[m + n*ldc] = alpha*acc + beta*C   (EMA when beta != 0); optional symmetric mirror
  kEpiSplit = 1,     // planes <- alpha*acc + beta*(old planes), as hi/lo (operand of the next GEMM); optional plain copy in C
  kEpiAdam = 2,      // acc is the projected gradient: update momentum/variance; update -> planes and/or C
  kEpiRowMajor = 3,  // C[m*ldc + n] = alpha*acc (tensor-parallel shard output)
  kEpiPairUpdate = 4,  // block-Jacobi column-pair update: the 128 result columns of a batch item go, in two
                       // halves of 64, to new column positions; written as planes in both orientations
  kEpiPush = 5,      // GEMM -> all-gather in one kernel: the result tile is this rank's block of a 2-D block-cyclic
                     // matrix T; every element alpha*acc is stored, as operand planes, straight into the gathered
                     // operand T[:, row class] of every rank that consumes it (peer memory over NVLink included)
};

// Operand planes.  a_* is the K x M column-major matrix Za (pitch lda floats), b_* the K x N matrix Zb.
struct GemmOperands {
  const float* a_hi;
  const float* a_lo;
  int64_t lda;
  const float* b_hi;
  const float* b_lo;
  int64_t ldb;
  // Extents of the whole operand buffers when a launch addresses sub-blocks of them per batch item
  // (0: the operand is exactly K x M, resp. K x N).
  int64_t a_k_total = 0, a_rows_total = 0, b_k_total = 0, b_rows_total = 0;
  // Mixed-precision corrections (both non-null selects them): one bf16 plane per operand that holds, for every
  // 32 elements of K, 32 values hb = bf16(x) followed by 32 values lb = bf16(x - hi) -- element k of hb at
  // (k / 32) * 64 + k % 32, of lb 32 further (`bf16_plane_index`); pitches in bf16 elements, multiples of 64, and
  // the elements past K in the last group are zero.  The two correction products hi*lo and lo*hi then run as
  // kind::f16 MMAs at twice the tf32 rate; a_lo and b_lo are not read.
  const uint16_t* a_hl = nullptr;
  int64_t lda16 = 0;
  const uint16_t* b_hl = nullptr;
  int64_t ldb16 = 0;
};

// Position of element k of hb inside a row of the interleaved bf16 plane (lb: 32 further).
__host__ __device__ inline int64_t bf16_plane_index(int64_t k) { return ((k >> 5) << 6) | (k & 31); }

struct GemmProblem {
  int M, N, K;
  int mode;
  int symmetric;     // 1: A == B, compute tiles on/below the diagonal and mirror the rest (kEpiStore only);
                     // 2: packed block-cyclic part of a symmetric result, entries on/below the GLOBAL diagonal only
  int tri_nb, tri_pr, tri_Pr, tri_pc, tri_Pc;   // symmetric == 2: block size and grid coordinates of this rank
  int tri_m0, tri_n0;                           // symmetric == 2: local row / column index of output element (0, 0)
  int force_narrow;  // use 128-wide tiles regardless of the problem size
  int k_splits;      // kEpiStore: split K over this many CTAs per tile, partial s written at C + s*split_stride
  int64_t split_stride;
  float alpha, beta;
  float* C;
  int64_t ldc;
  float* Chi;
  float* Clo;
  int64_t ldp;
  uint16_t* Chl;     // kEpiSplit / kEpiAdam with mixed output planes: the interleaved bf16 plane instead of Clo
  int64_t ldp16;
  float* mom;
  float* var;
  int64_t ldm, ldv;
  float beta1, beta2, eps, inv_bc1, inv_sqrt_bc2;
  // Batching (blockIdx.z = batch item): operand sub-blocks start at these multiples of the item index.
  int batches;
  int a_k_step, a_row_step, b_k_step, b_row_step;
  int64_t c_batch_stride;      // kEpiStore: item b writes at C + b * c_batch_stride
  // kEpiPairUpdate
  const int* remap;            // [batches][2]: destination position (in units of 64 columns) of each half
  float* C2hi;                 // second orientation: element (m, c') at [m + c' * ld2], only rows m < m_limit
  float* C2lo;
  int64_t ld2;
  int m_limit;
  int o1_row_start;            // rows m < o1_row_start are not written in the first orientation
  // kEpiPush.  Local element (m, n) is T(i, j) with i = ((m / nb) * Pr + pr) * nb + m % nb and
  // j = ((n / nb) * Pc + pc) * nb + n % nb.  Its consumers are the ranks of grid row (j / nb) % Pr; in their planes
  // (depth index i, column c = ((j / nb) / Pr) * nb + j % nb) it lands at hi[c * push_ld + i] and in the low plane
  // (fp32 lo at the same offset, or the interleaved bf16 plane at c * push_ld16 + bf16_plane_index(i)).
  const uint64_t* push_table = nullptr;   // device array [Pr * Pc][2]: hi plane and low plane of rank pr' * Pc + pc'
  int64_t push_ld = 0, push_ld16 = 0;
  int push_nb = 1, push_Pr = 1, push_Pc = 1, push_pr = 0, push_pc = 0;
  int push_mixed = 0;                     // 1: the low plane is the interleaved bf16 plane
};

// acc[m, n] = sum_k Za[k, m] * Zb[k, n] on tcgen05 with 3xTF32 compensation, then the epilogue.
// `status` is the device status word that bounded waits report to.
void gemm_tf32x3(const GemmOperands& ops, const GemmProblem& prob, int* status, cudaStream_t stream);

// Large plain problems run on CTA pairs (cta_group::2) by default; `false` keeps every launch on single CTAs.
void gemm_use_cta_pairs(bool on);

// Same contraction in plain fp32 FMA on CUDA cores from unsplit operands with arbitrary strides:
// acc[m, n] = sum_k A[k*a_sk + m*a_sm] * B[k*b_sk + n*b_sn];  C[m*c_sm + n*c_sn] = alpha*acc + beta*C.
// Used as the in-tree numerical cross-check of the tensor-core kernel and for problems far below one tile.
void gemm_simt(const float* A, int64_t a_sk, int64_t a_sm, const float* B, int64_t b_sk, int64_t b_sn, float* C,
               int64_t c_sm, int64_t c_sn, int M, int N, int K, float alpha, float beta, cudaStream_t stream);

}  // namespace soapb200
