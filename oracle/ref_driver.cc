// TEST INFRASTRUCTURE ONLY (checker side).
//
// C-ABI wrappers around the reference's own CPU operator bodies.  The bodies
// themselves are NOT in this repository: oracle/Makefile compiles them from the
// reference checkout (jittor_geometric/ops/cpp/*_op.cc, -DJIT -DJIT_cpu) and
// links them with this file into oracle/_ref/libjgref.so.  This file supplies
// what the `#ifndef JIT` halves of those files would have supplied (the
// out-of-line constructors) and one plain-pointer entry point per operator.
#include "op.h"
#include "cootocsr_op.h"
#include "cootocsc_op.h"
#include "aggregate_op.h"
#include "edgesoftmax_op.h"
#include "edgesoftmaxbackward_op.h"
#include "scattertoedge_op.h"
#include "edgetovertex_op.h"
#include "toundirected_op.h"
#include "csctocsr_op.h"
#include "getweight_op.h"
#include "sampleprocessing_op.h"

namespace jittor {

// Constructors: member-wise stores only (flags/output of the real runtime are
// not needed to run jit_run()).
CootocsrOp::CootocsrOp(Var* ei, Var* w, Var* ci, Var* ro, Var* cw, int n)
    : column_indices(ci), row_offset(ro), csr_edge_weight(cw), edge_index(ei),
      coo_edge_weight(w), output(nullptr), v_num(n) {}
CootocscOp::CootocscOp(Var* ei, Var* w, Var* ri, Var* co, Var* cw, int n)
    : row_indices(ri), column_offset(co), csc_edge_weight(cw), edge_index(ei),
      coo_edge_weight(w), output(nullptr), v_num(n) {}
AggregateOp::AggregateOp(Var* o, Var* x_, Var* i, Var* off, Var* w, bool f)
    : x(x_), outputVar(o), indices(i), offset(off), weight(w), forward(f), output(nullptr) {}
EdgesoftmaxOp::EdgesoftmaxOp(Var* o, Var* x_, Var* i, Var* off)
    : x(x_), outputVar(o), indices(i), offset(off), edge_weight(nullptr), output(nullptr) {}
EdgesoftmaxbackwardOp::EdgesoftmaxbackwardOp(Var* o, Var* x_, Var* y_, Var* i, Var* off)
    : x(x_), outputVar(o), y(y_), indices(i), offset(off), edge_weight(nullptr), output(nullptr) {}
ScattertoedgeOp::ScattertoedgeOp(Var* o, Var* x_, Var* i, Var* off, bool ww, int fl)
    : x(x_), outputVar(o), edge_weight(nullptr), indices(i), offset(off), with_weight(ww),
      output(nullptr), flag(fl) {}
EdgetovertexOp::EdgetovertexOp(Var* o, Var* x_, Var* i, Var* off, int fl)
    : x(x_), outputVar(o), indices(i), offset(off), output(nullptr), flag(fl) {}
ToundirectedOp::ToundirectedOp(Var* ei, Var* ea, int ne, int nn, Var* nei, Var* nea, NanoString d)
    : output(nullptr), edge_index(ei), edge_attr(ea), new_edge_index(nei), new_edge_attr(nea),
      num_edges(ne), num_nodes(nn), dtype(d) {}
CsctocsrOp::CsctocsrOp(Var* co, Var* ri, Var* ro, Var* ci, Var* d, Var* s_)
    : output(nullptr), column_offset(co), row_indices(ri), row_offset(ro), column_indices(ci), src(s_), dst(d) {}
GetweightOp::GetweightOp(int n, Var* d, Var* s_, Var* co, Var* ri, Var* w)
    : output(nullptr), vtx_size(n), csc_layer_dst(d), csc_layer_src(s_), csc_layer_column_offset(co),
      csc_layer_row_indices(ri), csc_layer_edge_weight(w) {}
SampleprocessingOp::SampleprocessingOp(int f, Var* d, Var* co, Var* ri, Var* gco, Var* gri)
    : output(nullptr), fanout_i(f), csc_layer_dst(d), csc_layer_column_offset(co), csc_layer_row_indices(ri),
      csc_global_column_offset(gco), csc_global_row_indices(gri) {}

}  // namespace jittor

using jittor::Var;

static Var mk(void* p, int64_t d0, int64_t d1 = 0) {
    Var v;
    v.mem = p;
    v.shape[0] = d0;
    v.shape[1] = d1;
    v.ndim = d1 ? 2 : 1;
    return v;
}

extern "C" {

// edge_index is [2,E] row-major int32; outputs must be zero-filled by the caller
// (the reference wrapper allocates them with jt.zeros).
void ref_cootocsr(int* edge_index, float* w, long E, int n, int* col_idx, int* row_off, float* out_w) {
    Var ei = mk(edge_index, 2, E), vw = mk(w, E), ci = mk(col_idx, E), ro = mk(row_off, n + 1), cw = mk(out_w, E);
    jittor::CootocsrOp op(&ei, &vw, &ci, &ro, &cw, n);
    op.jit_run();
}

void ref_cootocsc(int* edge_index, float* w, long E, int n, int* row_idx, int* col_off, float* out_w) {
    Var ei = mk(edge_index, 2, E), vw = mk(w, E), ri = mk(row_idx, E), co = mk(col_off, n + 1), cw = mk(out_w, E);
    jittor::CootocscOp op(&ei, &vw, &ri, &co, &cw, n);
    op.jit_run();
}

// out must be zero-filled: the body accumulates into it.
void ref_aggregate(float* out, float* x, int* idx, int* off, float* w, long n, long f, long E) {
    Var o = mk(out, n, f), vx = mk(x, n, f), vi = mk(idx, E), vo = mk(off, n + 1), vw = mk(w, E);
    jittor::AggregateOp op(&o, &vx, &vi, &vo, &vw, true);
    op.jit_run();
}

void ref_edgesoftmax(float* out, float* x, int* idx, int* off, long n, long E) {
    Var o = mk(out, E), vx = mk(x, E), vi = mk(idx, E), vo = mk(off, n + 1);
    jittor::EdgesoftmaxOp op(&o, &vx, &vi, &vo);
    op.jit_run();
}

// x = incoming gradient, y = saved softmax output (argument order of the reference op).
void ref_edgesoftmax_backward(float* out, float* grad, float* y, int* idx, int* off, long n, long E) {
    Var o = mk(out, E), vg = mk(grad, E), vy = mk(y, E), vi = mk(idx, E), vo = mk(off, n + 1);
    jittor::EdgesoftmaxbackwardOp op(&o, &vg, &vy, &vi, &vo);
    op.jit_run();
}

// out [E,f] must be zero-filled.  flag 0: source row of each edge, 1: destination row.
void ref_scattertoedge(float* out, float* x, int* idx, int* off, long n, long f, long E, int flag) {
    Var o = mk(out, E, f), vx = mk(x, n, f), vi = mk(idx, E), vo = mk(off, n + 1);
    jittor::ScattertoedgeOp op(&o, &vx, &vi, &vo, false, flag);
    op.jit_run();
}

// out [n,f] must be zero-filled.
void ref_edgetovertex(float* out, float* x, int* idx, int* off, long n, long f, long E, int flag) {
    Var o = mk(out, n, f), vx = mk(x, E, f), vi = mk(idx, E), vo = mk(off, n + 1);
    jittor::EdgetovertexOp op(&o, &vx, &vi, &vo, flag);
    op.jit_run();
}

// new_edge_index / new_attr need room for 2*E entries; returns the new edge count.
long ref_toundirected(int* edge_index, float* attr, long E, int n, int* new_edge_index, float* new_attr) {
    Var ei = mk(edge_index, 2, E), ea = mk(attr, E), nei = mk(new_edge_index, 2, 2 * E), nea = mk(new_attr, 2 * E);
    jittor::ToundirectedOp op(&ei, &ea, (int)E, n, &nei, &nea, jittor::ns_float32);
    op.jit_run();
    return nei.shape[1];
}

// row_off [n_src+1] must be zero-filled (the reference wrapper allocates it with jt.zeros).  Source
// ids must stay below 2^20: the body's id table has that many slots.
void ref_csctocsr(int* col_off, int* row_idx, long n_dst, long E, int* dst_ids, int* src_ids, long n_src, int* row_off,
                  int* col_idx) {
    Var co = mk(col_off, n_dst + 1), ri = mk(row_idx, E), ro = mk(row_off, n_src + 1), ci = mk(col_idx, E);
    Var d = mk(dst_ids, n_dst), s = mk(src_ids, n_src);
    jittor::CsctocsrOp op(&co, &ri, &ro, &ci, &d, &s);
    op.jit_run();
}

void ref_getweight(int vtx_size, int* dst_ids, long n_dst, int* src_ids, long n_src, int* col_off, int* row_idx, long E,
                   float* out_w) {
    Var d = mk(dst_ids, n_dst), s = mk(src_ids, n_src), co = mk(col_off, n_dst + 1), ri = mk(row_idx, E), w = mk(out_w, E);
    jittor::GetweightOp op(vtx_size, &d, &s, &co, &ri, &w);
    op.jit_run();
}

// The body draws with rand(): `seed` goes to srand() first.
void ref_sampleprocessing(int fanout, int* dst_ids, long n_dst, int* layer_off, int* layer_idx, long E_layer, int* g_off,
                          long n_global, int* g_idx, long E_global, unsigned seed) {
    Var d = mk(dst_ids, n_dst), lo = mk(layer_off, n_dst + 1), li = mk(layer_idx, E_layer);
    Var go = mk(g_off, n_global + 1), gi = mk(g_idx, E_global);
    srand(seed);
    jittor::SampleprocessingOp op(fanout, &d, &lo, &li, &go, &gi);
    op.jit_run();
}

}  // extern "C"
