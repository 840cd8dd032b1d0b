// Python bindings of the native library (module soap_tp_b200._C).
//
// The reference exposes two pybind11 modules that take raw integer addresses plus leading dimensions
// and release the GIL (src/soap_tp/csrc/slate_bindings.cpp:317-389, elpa_bindings.cpp:200-236).  The
// same calling convention is used here: tensors are passed as data_ptr() integers with explicit
// pitches, the CUDA stream as its integer handle.  Nothing here allocates device memory.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstdint>

#include "comm.h"
#include "elementwise.h"
#include "gemm.h"
#include "jacobi.h"
#include "qr.h"
#include "tridiag.h"

namespace py = pybind11;
using namespace soapb200;

namespace {
template <class T>
T* ptr(uint64_t address) {
  return reinterpret_cast<T*>(static_cast<uintptr_t>(address));
}
cudaStream_t stream_of(uint64_t handle) { return reinterpret_cast<cudaStream_t>(static_cast<uintptr_t>(handle)); }
}  // namespace

PYBIND11_MODULE(_C, m) {
  m.doc() = "sm_100a kernels of soap_tp_b200";
  m.def("compiled_gpu_backend", [] { return "cuda"; });
  m.def("compiled_arch", [] { return "sm_100a"; });

  m.def(
      "gemm_tf32x3",
      [](uint64_t a_hi, uint64_t a_lo, int64_t lda, uint64_t b_hi, uint64_t b_lo, int64_t ldb, int M, int N, int K,
         int mode, int symmetric, int force_narrow, float alpha, float beta, uint64_t C, int64_t ldc, uint64_t Chi,
         uint64_t Clo, int64_t ldp, uint64_t mom, uint64_t var, int64_t ldm, int64_t ldv, float beta1, float beta2,
         float eps, float inv_bc1, float inv_sqrt_bc2, int k_splits, int64_t split_stride, uint64_t status,
         uint64_t stream, int batches, int a_k_step, int a_row_step, int b_k_step, int b_row_step,
         int64_t c_batch_stride, int64_t a_k_total, int64_t a_rows_total, int64_t b_k_total, int64_t b_rows_total,
         uint64_t remap, uint64_t C2hi, uint64_t C2lo, int64_t ld2, int m_limit, int o1_row_start, int tri_nb,
         int tri_pr, int tri_Pr, int tri_pc, int tri_Pc, int tri_m0, int tri_n0, uint64_t a_hl, int64_t lda16,
         uint64_t b_hl, int64_t ldb16, uint64_t Chl, int64_t ldp16, uint64_t push_table, int64_t push_ld,
         int64_t push_ld16, int push_nb, int push_Pr, int push_Pc, int push_pr, int push_pc, int push_mixed) {
        GemmOperands ops{};
        ops.a_hi = ptr<const float>(a_hi); ops.a_lo = ptr<const float>(a_lo); ops.lda = lda;
        ops.b_hi = ptr<const float>(b_hi); ops.b_lo = ptr<const float>(b_lo); ops.ldb = ldb;
        GemmProblem prob{};
        prob.M = M; prob.N = N; prob.K = K;
        prob.mode = mode; prob.symmetric = symmetric; prob.force_narrow = force_narrow;
        prob.alpha = alpha; prob.beta = beta;
        prob.C = ptr<float>(C); prob.ldc = ldc;
        prob.Chi = ptr<float>(Chi); prob.Clo = ptr<float>(Clo); prob.ldp = ldp;
        prob.mom = ptr<float>(mom); prob.var = ptr<float>(var); prob.ldm = ldm; prob.ldv = ldv;
        prob.beta1 = beta1; prob.beta2 = beta2; prob.eps = eps;
        prob.inv_bc1 = inv_bc1; prob.inv_sqrt_bc2 = inv_sqrt_bc2;
        prob.k_splits = k_splits; prob.split_stride = split_stride;
        prob.batches = batches;
        prob.a_k_step = a_k_step; prob.a_row_step = a_row_step; prob.b_k_step = b_k_step; prob.b_row_step = b_row_step;
        prob.c_batch_stride = c_batch_stride;
        ops.a_k_total = a_k_total; ops.a_rows_total = a_rows_total; ops.b_k_total = b_k_total; ops.b_rows_total = b_rows_total;
        prob.remap = ptr<const int>(remap); prob.C2hi = ptr<float>(C2hi); prob.C2lo = ptr<float>(C2lo);
        prob.ld2 = ld2; prob.m_limit = m_limit; prob.o1_row_start = o1_row_start;
        prob.tri_nb = tri_nb > 0 ? tri_nb : 1; prob.tri_pr = tri_pr; prob.tri_Pr = tri_Pr > 0 ? tri_Pr : 1;
        prob.tri_pc = tri_pc; prob.tri_Pc = tri_Pc > 0 ? tri_Pc : 1; prob.tri_m0 = tri_m0; prob.tri_n0 = tri_n0;
        ops.a_hl = ptr<const uint16_t>(a_hl); ops.lda16 = lda16;
        ops.b_hl = ptr<const uint16_t>(b_hl); ops.ldb16 = ldb16;
        prob.Chl = ptr<uint16_t>(Chl); prob.ldp16 = ldp16;
        prob.push_table = ptr<const uint64_t>(push_table); prob.push_ld = push_ld; prob.push_ld16 = push_ld16;
        prob.push_nb = push_nb; prob.push_Pr = push_Pr; prob.push_Pc = push_Pc; prob.push_pr = push_pr;
        prob.push_pc = push_pc; prob.push_mixed = push_mixed;
        py::gil_scoped_release release;
        gemm_tf32x3(ops, prob, ptr<int>(status), stream_of(stream));
      },
      py::arg("a_hi"), py::arg("a_lo"), py::arg("lda"), py::arg("b_hi"), py::arg("b_lo"), py::arg("ldb"), py::arg("M"),
      py::arg("N"), py::arg("K"), py::arg("mode"), py::arg("symmetric"), py::arg("force_narrow"), py::arg("alpha"),
      py::arg("beta"), py::arg("C"), py::arg("ldc"), py::arg("Chi"), py::arg("Clo"), py::arg("ldp"), py::arg("mom"),
      py::arg("var"), py::arg("ldm"), py::arg("ldv"), py::arg("beta1"), py::arg("beta2"), py::arg("eps"),
      py::arg("inv_bc1"), py::arg("inv_sqrt_bc2"), py::arg("k_splits"), py::arg("split_stride"), py::arg("status"),
      py::arg("stream"), py::arg("batches") = 1, py::arg("a_k_step") = 0, py::arg("a_row_step") = 0,
      py::arg("b_k_step") = 0, py::arg("b_row_step") = 0, py::arg("c_batch_stride") = 0, py::arg("a_k_total") = 0,
      py::arg("a_rows_total") = 0, py::arg("b_k_total") = 0, py::arg("b_rows_total") = 0, py::arg("remap") = 0,
      py::arg("C2hi") = 0, py::arg("C2lo") = 0, py::arg("ld2") = 0, py::arg("m_limit") = 0, py::arg("o1_row_start") = 0, py::arg("tri_nb") = 1, py::arg("tri_pr") = 0,
      py::arg("tri_Pr") = 1, py::arg("tri_pc") = 0, py::arg("tri_Pc") = 1, py::arg("tri_m0") = 0, py::arg("tri_n0") = 0,
      py::arg("a_hl") = 0, py::arg("lda16") = 0, py::arg("b_hl") = 0, py::arg("ldb16") = 0, py::arg("Chl") = 0,
      py::arg("ldp16") = 0, py::arg("push_table") = 0, py::arg("push_ld") = 0, py::arg("push_ld16") = 0,
      py::arg("push_nb") = 1, py::arg("push_Pr") = 1, py::arg("push_Pc") = 1, py::arg("push_pr") = 0,
      py::arg("push_pc") = 0, py::arg("push_mixed") = 0,
      "3xTF32 tcgen05 GEMM acc[m,n] = sum_k Za[k,m] Zb[k,n] with fused epilogue");

  m.def("gemm_use_cta_pairs", [](bool on) { gemm_use_cta_pairs(on); },
        "Large plain GEMMs on CTA pairs (cta_group::2, default) or on single CTAs");

  m.def("gemm_simt",
        [](uint64_t A, int64_t a_sk, int64_t a_sm, uint64_t B, int64_t b_sk, int64_t b_sn, uint64_t C, int64_t c_sm,
           int64_t c_sn, int M, int N, int K, float alpha, float beta, uint64_t stream) {
          py::gil_scoped_release release;
          gemm_simt(ptr<const float>(A), a_sk, a_sm, ptr<const float>(B), b_sk, b_sn, ptr<float>(C), c_sm, c_sn, M, N,
                    K, alpha, beta, stream_of(stream));
        });

  m.def("adam_update",
        [](uint64_t g, int64_t ldg, uint64_t mo, int64_t ldm, uint64_t v, int64_t ldv, uint64_t u, int64_t ldu, int rows,
           int cols, float beta1, float beta2, float eps, float inv_bc1, float inv_sqrt_bc2, uint64_t stream) {
          adam_update(ptr<const float>(g), ldg, ptr<float>(mo), ldm, ptr<float>(v), ldv, ptr<float>(u), ldu, rows, cols,
                      beta1, beta2, eps, inv_bc1, inv_sqrt_bc2, stream_of(stream));
        });

  m.def("split_planes",
        [](uint64_t src, int64_t s_i, int64_t s_j, uint64_t hi, uint64_t lo, int64_t ldo, int rows, int cols,
           float scale, int nearest, uint64_t stream, uint64_t hl, int64_t ld16) {
          split_planes(ptr<const float>(src), s_i, s_j, ptr<float>(hi), ptr<float>(lo), ldo, rows, cols, scale, nearest,
                       stream_of(stream), ptr<uint16_t>(hl), ld16);
        },
        py::arg("src"), py::arg("s_i"), py::arg("s_j"), py::arg("hi"), py::arg("lo"), py::arg("ldo"), py::arg("rows"),
        py::arg("cols"), py::arg("scale"), py::arg("nearest"), py::arg("stream"), py::arg("hl") = 0, py::arg("ld16") = 0);

  m.def("column_dot",
        [](uint64_t a, int64_t lda, uint64_t b, int64_t ldb, uint64_t out, int rows, int cols, uint64_t stream) {
          column_dot(ptr<const float>(a), lda, ptr<const float>(b), ldb, ptr<float>(out), rows, cols, stream_of(stream));
        });

  m.def("order_by_estimate", [](uint64_t table, int64_t ld, int parts, int n, uint64_t order, uint64_t stream) {
    order_by_estimate(ptr<const float>(table), ld, parts, n, ptr<int64_t>(order), stream_of(stream));
  });
  m.attr("ORDER_MAX_LENGTH") = kOrderMaxLength;

  m.def("gather2d",
        [](uint64_t src, int64_t s_i, int64_t s_j, uint64_t dst, int64_t d_i, int64_t d_j, uint64_t row_map,
           uint64_t col_map, int rows, int cols, uint64_t stream) {
          gather2d(ptr<const float>(src), s_i, s_j, ptr<float>(dst), d_i, d_j, ptr<const int64_t>(row_map),
                   ptr<const int64_t>(col_map), rows, cols, stream_of(stream));
        });

  m.def("jacobi_small",
        [](uint64_t s_hi, uint64_t s_lo, int64_t lds, int batches, uint64_t u_hi, uint64_t u_lo, int64_t ldu,
           uint64_t offdiag, float scale, int max_sweeps, float tolerance, uint64_t stream) {
          jacobi_small(ptr<const float>(s_hi), ptr<const float>(s_lo), lds, batches, ptr<float>(u_hi), ptr<float>(u_lo), ldu,
                       ptr<float>(offdiag), scale, max_sweeps, tolerance, stream_of(stream));
        });
  m.def("qr_panel",
        [](uint64_t p_hi, uint64_t p_lo, int64_t ldp, int r, int b, uint64_t v_hi, uint64_t v_lo, int64_t ldv,
           uint64_t vt_hi, uint64_t vt_lo, int64_t ldvt, uint64_t tau, uint64_t t_hi, uint64_t t_lo, uint64_t tt_hi,
           uint64_t tt_lo, int64_t ldt, uint64_t exchange, uint64_t status, uint64_t stream, uint64_t trace, int debug_skip) {
          qr_panel(ptr<const float>(p_hi), ptr<const float>(p_lo), ldp, r, b, ptr<float>(v_hi), ptr<float>(v_lo), ldv,
                   ptr<float>(vt_hi), ptr<float>(vt_lo), ldvt, ptr<float>(tau), ptr<float>(t_hi), ptr<float>(t_lo),
                   ptr<float>(tt_hi), ptr<float>(tt_lo), ldt, ptr<float>(exchange), ptr<int>(status), stream_of(stream),
                   ptr<long long>(trace), debug_skip);
        },
        py::arg("p_hi"), py::arg("p_lo"), py::arg("ldp"), py::arg("r"), py::arg("b"), py::arg("v_hi"), py::arg("v_lo"),
        py::arg("ldv"), py::arg("vt_hi"), py::arg("vt_lo"), py::arg("ldvt"), py::arg("tau"), py::arg("t_hi"),
        py::arg("t_lo"), py::arg("tt_hi"), py::arg("tt_lo"), py::arg("ldt"), py::arg("exchange"), py::arg("status"),
        py::arg("stream"), py::arg("trace") = 0, py::arg("debug_skip") = 0);
  m.def("qr_panel_pairs",
        [](uint64_t p_hi, uint64_t p_lo, int64_t ldp, int r, int b, uint64_t v_hi, uint64_t v_lo, int64_t ldv,
           uint64_t vt_hi, uint64_t vt_lo, int64_t ldvt, uint64_t tau, uint64_t t_hi, uint64_t t_lo, uint64_t tt_hi,
           uint64_t tt_lo, int64_t ldt, uint64_t exchange, uint64_t status, uint64_t stream, int rows_per_cta,
           uint64_t steps_taken) {
          qr_panel_pairs(ptr<const float>(p_hi), ptr<const float>(p_lo), ldp, r, b, ptr<float>(v_hi), ptr<float>(v_lo),
                         ldv, ptr<float>(vt_hi), ptr<float>(vt_lo), ldvt, ptr<float>(tau), ptr<float>(t_hi),
                         ptr<float>(t_lo), ptr<float>(tt_hi), ptr<float>(tt_lo), ldt, ptr<float>(exchange),
                         ptr<int>(status), stream_of(stream), rows_per_cta, ptr<long long>(steps_taken));
        },
        py::arg("p_hi"), py::arg("p_lo"), py::arg("ldp"), py::arg("r"), py::arg("b"), py::arg("v_hi"), py::arg("v_lo"),
        py::arg("ldv"), py::arg("vt_hi"), py::arg("vt_lo"), py::arg("ldvt"), py::arg("tau"), py::arg("t_hi"),
        py::arg("t_lo"), py::arg("tt_hi"), py::arg("tt_lo"), py::arg("ldt"), py::arg("exchange"), py::arg("status"),
        py::arg("stream"), py::arg("rows_per_cta") = 256, py::arg("steps_taken") = 0);
  m.def("sum_partials_to_planes",
        [](uint64_t partials, int splits, int64_t stride, int64_t ld, uint64_t hi, uint64_t lo, int64_t ldp, int rows,
           int cols, uint64_t stream) {
          sum_partials_to_planes(ptr<const float>(partials), splits, stride, ld, ptr<float>(hi), ptr<float>(lo), ldp, rows,
                                 cols, stream_of(stream));
        });
  m.def("identity_planes", [](uint64_t hi, uint64_t lo, int64_t ldp, int rows, int cols, uint64_t stream, int first_col) {
    identity_planes(ptr<float>(hi), ptr<float>(lo), ldp, rows, cols, stream_of(stream), first_col);
  }, py::arg("hi"), py::arg("lo"), py::arg("ldp"), py::arg("rows"), py::arg("cols"), py::arg("stream"), py::arg("first_col") = 0);
  m.def("planes_sum", [](uint64_t hi, uint64_t lo, int64_t ldp, uint64_t out, int64_t ldo, int depth, int cols, uint64_t stream) {
    planes_sum(ptr<const float>(hi), ptr<const float>(lo), ldp, ptr<float>(out), ldo, depth, cols, stream_of(stream));
  });
  m.def("sytrd_panel",
        [](uint64_t A, int64_t lda, int n, int j0, int nb, uint64_t vw, uint64_t x, uint64_t y, uint64_t partial, uint64_t d,
           uint64_t e, uint64_t tau, uint64_t za_hi, uint64_t za_lo, uint64_t zb_hi, uint64_t zb_lo, uint64_t v_hi,
           uint64_t v_lo, int64_t ldv, uint64_t vt_hi, uint64_t vt_lo, int64_t ldvt, uint64_t t_hi, uint64_t t_lo,
           uint64_t tt_hi, uint64_t tt_lo, int64_t ldt, uint64_t barrier, uint64_t status, int last, uint64_t stream) {
          SytrdPanelArgs args{ptr<float>(A), lda, n, j0, nb, ptr<float>(vw), ptr<float>(x), ptr<float>(y), ptr<float>(partial),
                              ptr<double>(d), ptr<double>(e), ptr<float>(tau), ptr<float>(za_hi), ptr<float>(za_lo),
                              ptr<float>(zb_hi), ptr<float>(zb_lo), ptr<float>(v_hi), ptr<float>(v_lo), ldv, ptr<float>(vt_hi),
                              ptr<float>(vt_lo), ldvt, ptr<float>(t_hi), ptr<float>(t_lo), ptr<float>(tt_hi), ptr<float>(tt_lo),
                              ldt, ptr<unsigned int>(barrier), ptr<int>(status), last};
          sytrd_panel(args, stream_of(stream));
        });
  m.def("tridiagonal_bisect", [](uint64_t d, uint64_t e, int n, double lo, double hi, double pivmin, uint64_t lambda, uint64_t stream) {
    tridiagonal_bisect(ptr<const double>(d), ptr<const double>(e), n, lo, hi, pivmin, ptr<double>(lambda), stream_of(stream));
  });
  m.def("tridiagonal_vectors", [](uint64_t d, uint64_t e, int n, uint64_t lambda, double pivmin, uint64_t lplus, uint64_t dplus,
                                  uint64_t uminus, uint64_t z, uint64_t stream) {
    tridiagonal_vectors(ptr<const double>(d), ptr<const double>(e), n, ptr<const double>(lambda), pivmin, ptr<double>(lplus),
                        ptr<double>(dplus), ptr<double>(uminus), ptr<float>(z), stream_of(stream));
  });
  m.attr("TRIDIAG_PANEL") = kTridiagPanel;
  m.attr("QR_PANEL_WIDTH") = kQrPanelWidth;
  m.attr("QR_ROWS_PER_CTA") = kQrRowsPerCta;
  m.attr("QR_MAX_ROWS") = kQrMaxRows;

  register_comm(m);
}
