// TorchScript boundary: the custom class my_classes.DGLGraph and the my_ops::* operators,
// registered under the reference's exact names and schema strings so that its MP-DFG builder,
// optimizer passes and Python wrapper dispatch here unchanged.  Every operator is a thin
// shim: validate, allocate the output with torch::empty on the input's device, launch the
// C-ABI kernel (include/gphl.h) on the current PyTorch stream.  No operator synchronises the
// device, copies to the host or falls back to a CPU path; CPU tensors are rejected.
//
// Reference registrations: src/dglgraph.cpp:5-24 (class), src/ops/broadcast/broadcast.cu:102-122,
// src/ops/segment_softmax/segment_softmax.cu:27-30, src/ops/segment_mm/segment_mm.cu:35-42,
// src/ops/dgl_primitives/spmm.cu:391-406, src/ops/dgl_primitives/sddmm.cu:131-134.
// `int? t` is bound as optional<int64_t>: current PyTorch rejects optional<ScalarType> for it.
#include <cstdlib>
#include <vector>
#include <mutex>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/custom_class.h>
#include <torch/script.h>

#include <algorithm>

#include "gphl.h"

namespace {

using torch::Tensor;

void check_rc(int rc, const char *what) {
  TORCH_CHECK(rc == GPHL_OK, what, " failed (", rc, "): ", gphl_last_error());
}

int64_t feat_of(const Tensor &x) {
  int64_t f = 1;
  for (int64_t i = 1; i < x.dim(); ++i) f *= x.size(i);
  return f;
}

Tensor cuda_f32(const Tensor &x, const char *name) {
  TORCH_CHECK(x.is_cuda(), name, " must be a CUDA tensor (this library has no CPU path)");
  TORCH_CHECK(x.scalar_type() == torch::kFloat32, name, " must be float32");
  return x.contiguous();
}

Tensor cuda_idx(const Tensor &x, torch::ScalarType t, const char *name) {
  TORCH_CHECK(x.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(x.scalar_type() == t, name, " has the wrong index dtype");
  return x.contiguous();
}

// Address of a tensor's data; an empty tensor has none, and where the C ABI wants a non-null array
// that it will never read (index and edge arrays of an edgeless graph) `lender` gives its address.
template <typename T>
T *ptr_or(const Tensor &t, const Tensor &lender) {
  return t.numel() ? t.data_ptr<T>() : reinterpret_cast<T *>(lender.data_ptr());
}

void *stream_of(const Tensor &x) { return at::cuda::getCurrentCUDAStream(x.get_device()).stream(); }

}  // namespace

// Same field names and counts as the reference's struct (include/dglgraph.h:7-75), plus cached
// per-graph metadata: row-split plans for the reduce (CSC) and message (CSR) sides.
struct DGLGraph : torch::CustomClassHolder {
  DGLGraph(Tensor in_pointer, Tensor in_node_indices, Tensor in_edge_indices, Tensor out_pointer,
           Tensor out_node_indices, Tensor out_edge_indices, Tensor COO_src, Tensor COO_dst,
           c10::optional<Tensor> ntype_pointer, c10::optional<Tensor> etype_pointer)
      : in_pointer(in_pointer), in_node_indices(in_node_indices), in_edge_indices(in_edge_indices),
        out_pointer(out_pointer), out_node_indices(out_node_indices), out_edge_indices(out_edge_indices),
        COO_src(COO_src), COO_dst(COO_dst), ntype_pointer(ntype_pointer), etype_pointer(etype_pointer) {
    num_nodes = in_pointer.size(0) - 1;
    num_edges = in_node_indices.size(0);
    num_ntypes = ntype_pointer.has_value() ? ntype_pointer.value().size(0) - 1 : 1;
    num_etypes = etype_pointer.has_value() ? etype_pointer.value().size(0) - 1 : 1;
    TORCH_CHECK(out_pointer.size(0) == num_nodes + 1, "out_pointer has the wrong length");
    TORCH_CHECK(in_edge_indices.size(0) == num_edges && out_node_indices.size(0) == num_edges &&
                    out_edge_indices.size(0) == num_edges && COO_src.size(0) == num_edges &&
                    COO_dst.size(0) == num_edges,
                "edge arrays must all have num_edges entries");
    prepare();
  }
  // Everything that needs a host round trip happens here, once per graph, so that no operator call synchronises
  // or allocates outside PyTorch's caching allocator: the index arrays are validated (the kernels trust them; set
  // GPHL_SKIP_VALIDATION=1 to skip the pass) and the row-split plans of both sides are built.  Their scratch is
  // bound per call from the caching allocator (plan()).  CPU tensors are left alone: every operator rejects them.
  void prepare() {
    if (!in_pointer.is_cuda() || num_nodes >= INT32_MAX || num_edges >= INT32_MAX) return;
    c10::cuda::CUDAGuard guard(in_pointer.device());
    Tensor ip = cuda_idx(in_pointer, torch::kInt32, "in_pointer"), op = cuda_idx(out_pointer, torch::kInt32, "out_pointer");
    const char *skip = std::getenv("GPHL_SKIP_VALIDATION");
    if (!(skip && skip[0] == '1')) {
      Tensor inn = cuda_idx(in_node_indices, torch::kInt32, "in_node_indices");
      Tensor ine = cuda_idx(in_edge_indices, torch::kInt32, "in_edge_indices");
      Tensor outn = cuda_idx(out_node_indices, torch::kInt32, "out_node_indices");
      Tensor oute = cuda_idx(out_edge_indices, torch::kInt32, "out_edge_indices");
      Tensor cs = cuda_idx(COO_src, torch::kInt64, "COO_src"), cd = cuda_idx(COO_dst, torch::kInt64, "COO_dst");
      void *st = stream_of(ip);
      check_rc(gphl_validate_csr(ip.data_ptr<int32_t>(), num_nodes, num_edges, ptr_or<int32_t>(inn, ip), num_nodes,
                                 ptr_or<int32_t>(ine, ip), num_edges, st), "DGLGraph: in-edge arrays");
      check_rc(gphl_validate_csr(op.data_ptr<int32_t>(), num_nodes, num_edges, ptr_or<int32_t>(outn, op), num_nodes,
                                 ptr_or<int32_t>(oute, op), num_edges, st), "DGLGraph: out-edge arrays");
      check_rc(gphl_validate_index_i64(num_edges ? cs.data_ptr<int64_t>() : nullptr, num_edges, num_nodes, st), "DGLGraph: COO_src");
      check_rc(gphl_validate_index_i64(num_edges ? cd.data_ptr<int64_t>() : nullptr, num_edges, num_nodes, st), "DGLGraph: COO_dst");
      if (ntype_pointer.has_value()) check_type_pointer(ntype_pointer.value(), num_nodes, "ntype_pointer");
      if (etype_pointer.has_value()) check_type_pointer(etype_pointer.value(), num_edges, "etype_pointer");
    }
    check_rc(gphl_plan_create(ip.data_ptr<int32_t>(), num_nodes, GPHL_DEFAULT_CHUNK, 0, stream_of(ip), &plan_in), "gphl_plan_create");
    check_rc(gphl_plan_create(op.data_ptr<int32_t>(), num_nodes, GPHL_DEFAULT_CHUNK, 0, stream_of(op), &plan_out), "gphl_plan_create");
  }
  // A type pointer must be non-decreasing from 0 to the number of rows it partitions: the typed-linear kernels write
  // exactly the rows it covers (the reference's loop of at::mm + cat, segment_mm.cu:4-21, would return a shorter
  // tensor or raise for anything else).
  static void check_type_pointer(const Tensor &pointer, int64_t rows, const char *what) {
    if (!pointer.is_cuda()) return;
    const char *skip = std::getenv("GPHL_SKIP_VALIDATION");
    if (skip && skip[0] == '1') return;
    Tensor pc = cuda_idx(pointer, torch::kInt32, what);
    TORCH_CHECK(pc.numel() >= 1, what, " must have at least one entry");
    c10::cuda::CUDAGuard guard(pc.device());
    check_rc(gphl_validate_csr(pc.data_ptr<int32_t>(), pc.numel() - 1, rows, nullptr, 0, nullptr, 0, stream_of(pc)), what);
  }
  ~DGLGraph() override {
    gphl_plan_destroy(plan_in);
    gphl_plan_destroy(plan_out);
  }
  void SetNtypePointer(Tensor pointer) {
    check_type_pointer(pointer, num_nodes, "ntype_pointer");
    ntype_pointer = pointer;
    num_ntypes = pointer.size(0) - 1;
  }
  void SetEtypePointer(Tensor pointer) {
    check_type_pointer(pointer, num_edges, "etype_pointer");
    etype_pointer = pointer;
    num_etypes = pointer.size(0) - 1;
  }
  void SetNtypeCOO(Tensor t) {
    TORCH_CHECK(t.size(0) == num_nodes, "ntype_COO must have num_nodes entries");
    ntype_COO = t;
  }
  void SetEtypeCOO(Tensor t) {
    TORCH_CHECK(t.size(0) == num_edges, "etype_COO must have num_edges entries");
    etype_COO = t;
    build_pairs();
  }
  // The distinct (edge type, source node) pairs of a typed graph, grouped by type.  An edge-typed linear applied to
  // gathered source rows (SegmentMMEdgeSrc) yields the same row for every edge of one pair: where the pairs are at
  // most half as many as the edges it is computed once per pair and the rows are handed out to the edges.  Built
  // here, in a setter, because torch::unique synchronises; operator calls stay free of synchronisation.
  void build_pairs() {
    pair_src = Tensor();
    if (!etype_COO.has_value() || !etype_COO.value().is_cuda() || !COO_src.is_cuda() || num_edges == 0) return;
    c10::cuda::CUDAGuard guard(COO_src.device());
    Tensor key = etype_COO.value().to(torch::kInt64) * num_nodes + COO_src.to(torch::kInt64);
    auto res = at::_unique2(key, /*sorted=*/true, /*return_inverse=*/true, /*return_counts=*/false);
    Tensor uniq = std::get<0>(res);
    if (uniq.size(0) * 2 > num_edges) return;                      // too few repeats to pay for the hand-out pass
    Tensor ptype = at::floor_divide(uniq, num_nodes);
    pair_src = (uniq - ptype * num_nodes).contiguous();
    pair_pointer = at::searchsorted(ptype, torch::arange(num_etypes + 1, ptype.options())).to(torch::kInt32).contiguous();
    edge_pair = std::get<1>(res).contiguous();
  }

  // Plan for the reduce side (rows = destinations) or the message side (rows = sources).  The plans were built in the
  // constructor; here only the scratch of the cut rows is bound, from PyTorch's caching allocator (no cudaMalloc,
  // no synchronisation), kept per graph and grown when a wider feature arrives.  Calls on one graph from several
  // streams at once would share it, as they would share any per-graph state.
  const gphl_plan *plan(bool reduce_side, int64_t feat) {
    gphl_plan *&p = reduce_side ? plan_in : plan_out;
    TORCH_CHECK(p != nullptr, "DGLGraph was built from CPU tensors: this library has no CPU path");
    int64_t &width = reduce_side ? plan_in_width : plan_out_width;
    Tensor &scratch = reduce_side ? scratch_in : scratch_out;
    if (feat > width) {
      const int64_t pieces = gphl_plan_num_pieces(p);
      width = std::max<int64_t>((feat + 7) / 8 * 8, 256);
      if (pieces > 0) scratch = torch::empty({2 * pieces * width}, in_pointer.options().dtype(torch::kFloat32));
      check_rc(gphl_plan_bind_scratch(p, pieces > 0 ? scratch.data_ptr() : nullptr, width), "gphl_plan_bind_scratch");
    }
    return p;
  }

  // int32 edge positions 0..E-1 and an int32 copy of COO_dst, made on first use (edge-level left operand of e_dot_v)
  const Tensor &edge_positions32() {
    if (!edge_pos32.defined())
      edge_pos32 = torch::arange(num_edges, COO_dst.options().dtype(torch::kInt32));
    return edge_pos32;
  }
  const Tensor &coo_dst32() {
    if (!dst32.defined()) dst32 = COO_dst.to(torch::kInt32).contiguous();
    return dst32;
  }

  int64_t num_nodes, num_edges, num_ntypes, num_etypes;
  Tensor edge_pos32, dst32, scratch_in, scratch_out;
  Tensor pair_src, pair_pointer, edge_pair;      // see build_pairs()
  Tensor in_pointer, in_node_indices, in_edge_indices;
  Tensor out_pointer, out_node_indices, out_edge_indices;
  Tensor COO_src, COO_dst;
  c10::optional<Tensor> ntype_pointer, etype_pointer, ntype_COO, etype_COO;
  gphl_plan *plan_in = nullptr, *plan_out = nullptr;
  int64_t plan_in_width = 0, plan_out_width = 0;
};

namespace {

using GraphPtr = c10::intrusive_ptr<DGLGraph>;

// ---- broadcasts -------------------------------------------------------------------------
Tensor gather_rows(const Tensor &x, const Tensor &idx, const c10::optional<Tensor> &idx2) {
  TORCH_CHECK(x.is_cuda(), "broadcast input must be a CUDA tensor (this library has no CPU path)");
  TORCH_CHECK(x.dim() >= 1, "broadcast input needs at least one dimension");
  Tensor xc = x.contiguous();
  Tensor ic = cuda_idx(idx, torch::kInt64, "index");
  const Tensor *outer = &ic;
  Tensor i2;
  if (idx2.has_value()) {
    i2 = cuda_idx(idx2.value(), torch::kInt64, "index");
    outer = &i2;
  }
  auto sizes = xc.sizes().vec();
  sizes[0] = outer->size(0);
  Tensor y = torch::empty(sizes, xc.options());
  c10::cuda::CUDAGuard guard(xc.device());
  check_rc(gphl_gather_rows_i64(ic.data_ptr<int64_t>(), idx2.has_value() ? i2.data_ptr<int64_t>() : nullptr,
                                outer->size(0), feat_of(xc) * (int64_t)xc.element_size(), xc.data_ptr(), y.data_ptr(),
                                stream_of(xc)),
           "gphl_gather_rows");
  return y;
}

Tensor BroadcastSrcNode(Tensor x, const GraphPtr &g) { return gather_rows(x, g->COO_src, c10::nullopt); }
Tensor BroadcastDstNode(Tensor x, const GraphPtr &g) { return gather_rows(x, g->COO_dst, c10::nullopt); }
Tensor BroadcastNodeType(Tensor x, const GraphPtr &g) {
  TORCH_CHECK(g->ntype_COO.has_value(), "BroadcastNodeType needs SetNtypeCOO");
  return gather_rows(x, g->ntype_COO.value(), c10::nullopt);
}
Tensor BroadcastEdgeType(Tensor x, const GraphPtr &g) {
  TORCH_CHECK(g->etype_COO.has_value(), "BroadcastEdgeType needs SetEtypeCOO");
  return gather_rows(x, g->etype_COO.value(), c10::nullopt);
}
Tensor BroadcastSrcNodeType(Tensor x, const GraphPtr &g) {
  TORCH_CHECK(g->ntype_COO.has_value(), "BroadcastSrcNodeType needs SetNtypeCOO");
  return gather_rows(x, g->ntype_COO.value(), g->COO_src);
}
Tensor BroadcastDstNodeType(Tensor x, const GraphPtr &g) {
  TORCH_CHECK(g->ntype_COO.has_value(), "BroadcastDstNodeType needs SetNtypeCOO");
  return gather_rows(x, g->ntype_COO.value(), g->COO_dst);
}
int64_t get_feat_dim(Tensor x) { return feat_of(x); }

// ---- SpMM ---------------------------------------------------------------------------------
std::vector<int64_t> out_shape(const Tensor &x, int64_t rows) {
  if (x.dim() <= 1) return {rows, 1};
  auto s = x.sizes().vec();
  s[0] = rows;
  return s;
}

Tensor spmm_gather(const Tensor &x, const Tensor &idx, const GraphPtr &g, int64_t need_rows, const char *what) {
  Tensor xc = cuda_f32(x, what);
  TORCH_CHECK(xc.size(0) == need_rows, what, ": expected ", need_rows, " rows, got ", xc.size(0));
  const int64_t f = feat_of(xc);
  Tensor y = torch::empty(out_shape(xc, g->num_nodes), xc.options());
  Tensor ptr = cuda_idx(g->in_pointer, torch::kInt32, "in_pointer");
  Tensor ic = cuda_idx(idx, torch::kInt32, "index");
  c10::cuda::CUDAGuard guard(xc.device());
  check_rc(gphl_spmm_gather_sum_f32(g->plan(true, f), ptr.data_ptr<int32_t>(), ptr_or<int32_t>(ic, ptr), g->num_nodes, f,
                                    ptr_or<float>(xc, ptr), y.data_ptr<float>(), stream_of(xc)),
           "gphl_spmm_gather_sum_f32");
  return y;
}

Tensor SpMMEdge(Tensor x, std::vector<int64_t>, bool, c10::optional<int64_t>, const GraphPtr &g) {
  return spmm_gather(x, g->in_edge_indices, g, g->num_edges, "SpMMEdge input");
}
Tensor SpMMSrc(Tensor x, std::vector<int64_t>, bool, c10::optional<int64_t>, const GraphPtr &g) {
  return spmm_gather(x, g->in_node_indices, g, g->num_nodes, "SpMMSrc input");
}

Tensor mul_e_sum(const Tensor &x, const Tensor &w, const GraphPtr &g, bool reduce_side) {
  Tensor xc = cuda_f32(x, "node features");
  Tensor wc = cuda_f32(w, "edge weights");
  TORCH_CHECK(xc.size(0) == g->num_nodes, "node features must have num_nodes rows");
  TORCH_CHECK(wc.size(0) == g->num_edges, "edge weights must have num_edges rows");
  const int64_t f = feat_of(xc), h = feat_of(wc);
  TORCH_CHECK(h >= 1 && f % h == 0, "feature width ", f, " is not a multiple of the weight width ", h);
  Tensor y = torch::empty(out_shape(xc, g->num_nodes), xc.options());
  Tensor ptr = cuda_idx(reduce_side ? g->in_pointer : g->out_pointer, torch::kInt32, "pointer");
  Tensor nid = cuda_idx(reduce_side ? g->in_node_indices : g->out_node_indices, torch::kInt32, "node indices");
  Tensor eid = cuda_idx(reduce_side ? g->in_edge_indices : g->out_edge_indices, torch::kInt32, "edge indices");
  c10::cuda::CUDAGuard guard(xc.device());
  check_rc(gphl_spmm_u_mul_e_sum_f32(g->plan(reduce_side, f), ptr.data_ptr<int32_t>(), ptr_or<int32_t>(nid, ptr),
                                     ptr_or<int32_t>(eid, ptr), g->num_nodes, h, f / h, xc.data_ptr<float>(),
                                     ptr_or<float>(wc, ptr), y.data_ptr<float>(), stream_of(xc)),
           "gphl_spmm_u_mul_e_sum_f32");
  return y;
}

Tensor src_mul_e_sum(Tensor x, Tensor w, std::vector<int64_t>, bool, c10::optional<int64_t>, const GraphPtr &g) {
  return mul_e_sum(x, w, g, true);
}
Tensor dst_mul_e_sum(Tensor x, Tensor w, std::vector<int64_t>, bool, c10::optional<int64_t>, const GraphPtr &g) {
  return mul_e_sum(x, w, g, false);
}

// Not registered by the reference.  Replaces SpMMEdge(mul(a, b)): the product of an (E, F) message with an (E, H)
// per-edge weight (H divides F; either operand order) is folded into the segment sum, so the (E, F) product is never
// written.  Other shapes multiply first and sum afterwards, as the unfused graph did.
Tensor SpMMEdgeMul(Tensor a, Tensor b, const GraphPtr &g) {
  auto edge2d = [&](const Tensor &t) {
    return t.is_cuda() && t.scalar_type() == torch::kFloat32 && t.dim() == 2 && t.size(0) == g->num_edges;
  };
  const Tensor *x = nullptr, *w = nullptr;
  if (edge2d(a) && edge2d(b)) {
    if (b.size(1) >= 1 && a.size(1) % b.size(1) == 0 && b.size(1) < a.size(1)) x = &a, w = &b;
    else if (a.size(1) >= 1 && b.size(1) % a.size(1) == 0 && a.size(1) < b.size(1)) x = &b, w = &a;
  }
  if (x == nullptr) return spmm_gather(at::mul(a, b), g->in_edge_indices, g, g->num_edges, "SpMMEdgeMul input");
  Tensor xc = x->contiguous(), wc = w->contiguous();
  const int64_t f = xc.size(1), h = wc.size(1);
  Tensor y = torch::empty({g->num_nodes, f}, xc.options());
  Tensor ptr = cuda_idx(g->in_pointer, torch::kInt32, "in_pointer");
  Tensor eid = cuda_idx(g->in_edge_indices, torch::kInt32, "in_edge_indices");
  c10::cuda::CUDAGuard guard(xc.device());
  // rows of x and of w are both addressed by edge id
  check_rc(gphl_spmm_u_mul_e_sum_f32(g->plan(true, f), ptr.data_ptr<int32_t>(), ptr_or<int32_t>(eid, ptr),
                                     ptr_or<int32_t>(eid, ptr), g->num_nodes, h, f / h, ptr_or<float>(xc, ptr),
                                     ptr_or<float>(wc, ptr), y.data_ptr<float>(), stream_of(xc)),
           "gphl_spmm_u_mul_e_sum_f32");
  return y;
}

// ---- SDDMM --------------------------------------------------------------------------------
// Shapes the destination-row dot-product kernel covers (gphl_sddmm_u_dot_v_csc_f32): heads of 4, 8, ..., 128 columns
// that fit the lane layout, rows of at most 512 columns.  torch allocations are 16-byte aligned.
static bool csc_dot_fits(int64_t f, int64_t heads) {
  if (heads < 1 || f % heads != 0) return false;
  const int64_t dim = f / heads;
  if (dim % 4 != 0) return false;
  const int64_t dv = dim / 4, fv = f / 4;
  if ((dv & (dv - 1)) != 0 || dv > 32 || fv > 128) return false;
  const int64_t lpr = fv <= 1 ? 1 : fv <= 2 ? 2 : fv <= 4 ? 4 : fv <= 8 ? 8 : fv <= 16 ? 16 : 32;
  const int64_t nv = fv <= 32 ? 1 : fv <= 64 ? 2 : 4;
  return dv % nv == 0 && dv / nv <= lpr;
}

Tensor u_add_v_mul_alpha(Tensor l, Tensor r, int64_t /*alpha: ignored, as in the reference*/, const GraphPtr &g) {
  Tensor lc = cuda_f32(l, "source features"), rc_ = cuda_f32(r, "destination features");
  const int64_t f = feat_of(lc);
  TORCH_CHECK(feat_of(rc_) == f, "u_add_v: feature widths differ");
  TORCH_CHECK(lc.size(0) == g->num_nodes && rc_.size(0) == g->num_nodes, "u_add_v: inputs must have num_nodes rows");
  Tensor z = torch::empty(out_shape(lc, g->num_edges), lc.options());
  Tensor s = cuda_idx(g->COO_src, torch::kInt64, "COO_src"), d = cuda_idx(g->COO_dst, torch::kInt64, "COO_dst");
  c10::cuda::CUDAGuard guard(lc.device());
  check_rc(gphl_sddmm_u_add_v_f32_i64(s.data_ptr<int64_t>(), d.data_ptr<int64_t>(), g->num_edges, f,
                                      lc.data_ptr<float>(), rc_.data_ptr<float>(), z.data_ptr<float>(), stream_of(lc)),
           "gphl_sddmm_u_add_v_f32_i64");
  return z;
}

// Not registered by the reference (its HGT graph runs aten::mul + aten::sum on gathered rows).  Replaces
// sum(mul(BroadcastSrcNode(l), BroadcastDstNode(r)), [1], keepdim): the kernel covers two-dimensional fp32 operands of
// equal width; every other shape (trailing dimensions, widths that only broadcast, other dtypes) takes the unfused
// route, so the rewrite never changes what a graph accepts or returns.
Tensor u_dot_v(Tensor l, Tensor r, int64_t heads, const GraphPtr &g) {
  const bool fits = l.is_cuda() && r.is_cuda() && l.scalar_type() == torch::kFloat32 && r.scalar_type() == torch::kFloat32 &&
                    l.dim() == 2 && r.dim() == 2 && l.size(0) == g->num_nodes && r.size(0) == g->num_nodes &&
                    l.size(1) == r.size(1) && heads >= 1 && l.size(1) % heads == 0;
  if (!fits) {
    TORCH_CHECK(heads == 1, "gsddmm_u_dot_v: the general form needs heads == 1");
    return at::sum(at::mul(gather_rows(l, g->COO_src, c10::nullopt), gather_rows(r, g->COO_dst, c10::nullopt)), {1}, true);
  }
  Tensor lc = l.contiguous(), rc_ = r.contiguous();
  const int64_t f = lc.size(1);
  Tensor z = torch::empty({g->num_edges, heads}, lc.options());
  if (g->num_edges == 0) return z;
  c10::cuda::CUDAGuard guard(lc.device());
  if (csc_dot_fits(f, heads)) {          // destination-row order: r[v] once per row, half the gathered bytes
    Tensor ptr = cuda_idx(g->in_pointer, torch::kInt32, "in_pointer");
    Tensor nid = cuda_idx(g->in_node_indices, torch::kInt32, "in_node_indices");
    Tensor eid = cuda_idx(g->in_edge_indices, torch::kInt32, "in_edge_indices");
    check_rc(gphl_sddmm_u_dot_v_csc_f32(g->plan(true, f), ptr.data_ptr<int32_t>(), nid.data_ptr<int32_t>(),
                                        eid.data_ptr<int32_t>(), g->num_nodes, heads, f / heads, lc.data_ptr<float>(),
                                        rc_.data_ptr<float>(), z.data_ptr<float>(), stream_of(lc)),
             "gphl_sddmm_u_dot_v_csc_f32");
    return z;
  }
  Tensor s = cuda_idx(g->COO_src, torch::kInt64, "COO_src"), d = cuda_idx(g->COO_dst, torch::kInt64, "COO_dst");
  check_rc(gphl_sddmm_u_dot_v_f32_i64(s.data_ptr<int64_t>(), d.data_ptr<int64_t>(), g->num_edges, heads, f / heads,
                                      lc.data_ptr<float>(), rc_.data_ptr<float>(), z.data_ptr<float>(), stream_of(lc)),
           "gphl_sddmm_u_dot_v_f32_i64");
  return z;
}

// Not registered by the reference.  Replaces sum(mul(e, BroadcastDstNode(v)), [1], keepdim) where e already holds one
// row per edge (HGT: the relation-transformed keys): out[i, h] = sum_d e[i, h, d] * v[COO_dst[i], h, d].  Shapes the
// kernel does not cover take the unfused route so that the rewrite never changes what a graph accepts.
Tensor e_dot_v(Tensor e, Tensor v, int64_t heads, const GraphPtr &g) {
  const bool fits = e.is_cuda() && v.is_cuda() && e.scalar_type() == torch::kFloat32 && v.scalar_type() == torch::kFloat32 &&
                    e.dim() == 2 && v.dim() == 2 && e.size(0) == g->num_edges && v.size(0) == g->num_nodes &&
                    e.size(1) == v.size(1) && heads >= 1 && e.size(1) % heads == 0 && g->num_edges < INT32_MAX;
  if (!fits) {
    TORCH_CHECK(heads == 1, "gsddmm_e_dot_v: the general form needs heads == 1");
    return at::sum(at::mul(e, gather_rows(v, g->COO_dst, c10::nullopt)), {1}, true);
  }
  Tensor ec = e.contiguous(), vc = v.contiguous();
  const int64_t f = ec.size(1);
  Tensor z = torch::empty({g->num_edges, heads}, ec.options());
  if (g->num_edges == 0) return z;
  c10::cuda::CUDAGuard guard(ec.device());
  if (csc_dot_fits(f, heads)) {          // rows of e are addressed by edge id, v[dst] is read once per destination row
    Tensor ptr = cuda_idx(g->in_pointer, torch::kInt32, "in_pointer");
    Tensor eid = cuda_idx(g->in_edge_indices, torch::kInt32, "in_edge_indices");
    check_rc(gphl_sddmm_u_dot_v_csc_f32(g->plan(true, f), ptr.data_ptr<int32_t>(), eid.data_ptr<int32_t>(),
                                        eid.data_ptr<int32_t>(), g->num_nodes, heads, f / heads, ec.data_ptr<float>(),
                                        vc.data_ptr<float>(), z.data_ptr<float>(), stream_of(ec)),
             "gphl_sddmm_u_dot_v_csc_f32");
    return z;
  }
  const Tensor &pos = g->edge_positions32(), &dst = g->coo_dst32();
  check_rc(gphl_sddmm_u_dot_v_f32_i32(pos.data_ptr<int32_t>(), dst.data_ptr<int32_t>(), g->num_edges, heads, f / heads,
                                      ec.data_ptr<float>(), vc.data_ptr<float>(), z.data_ptr<float>(), stream_of(ec)),
           "gphl_sddmm_u_dot_v_f32_i32");
  return z;
}

// ---- segment softmax ------------------------------------------------------------------------
Tensor SegmentSoftmax(Tensor x, int64_t dim, c10::optional<int64_t>, const GraphPtr &g) {
  TORCH_CHECK(dim == 1, "SegmentSoftmax: dim must be 1 (the mailbox dimension)");
  Tensor xc = cuda_f32(x, "SegmentSoftmax input");
  TORCH_CHECK(xc.size(0) == g->num_edges, "SegmentSoftmax input must have num_edges rows");
  const int64_t h = feat_of(xc);
  Tensor y = torch::empty_like(xc);
  Tensor stats = torch::empty({std::max<int64_t>(1, 2 * g->num_nodes * h)}, xc.options());
  Tensor ptr = cuda_idx(g->in_pointer, torch::kInt32, "in_pointer");
  Tensor eid = cuda_idx(g->in_edge_indices, torch::kInt32, "in_edge_indices");
  c10::cuda::CUDAGuard guard(xc.device());
  check_rc(gphl_segment_softmax_f32(g->plan(true, h), ptr.data_ptr<int32_t>(), ptr_or<int32_t>(eid, ptr), g->num_nodes, h,
                                    ptr_or<float>(xc, ptr), ptr_or<float>(y, ptr), stats.data_ptr<float>(), stream_of(xc)),
           "gphl_segment_softmax_f32");
  return y;
}

// Not registered by the reference: one operator for u_add_v -> leaky-relu -> softmax -> u_mul_e_sum.
Tensor gat_fused(Tensor el, Tensor er, Tensor z, double slope, const GraphPtr &g) {
  Tensor elc = cuda_f32(el, "el"), erc = cuda_f32(er, "er"), zc = cuda_f32(z, "z");
  const int64_t h = feat_of(elc), f = feat_of(zc);
  TORCH_CHECK(feat_of(erc) == h && h >= 1 && f % h == 0, "gat_fused: bad head / feature widths");
  TORCH_CHECK(elc.size(0) == g->num_nodes && erc.size(0) == g->num_nodes && zc.size(0) == g->num_nodes,
              "gat_fused: inputs must have num_nodes rows");
  Tensor out = torch::empty(out_shape(zc, g->num_nodes), zc.options());
  Tensor stats = torch::empty({std::max<int64_t>(1, 2 * g->num_nodes * h)}, zc.options());
  Tensor ptr = cuda_idx(g->in_pointer, torch::kInt32, "in_pointer");
  Tensor nid = cuda_idx(g->in_node_indices, torch::kInt32, "in_node_indices");
  c10::cuda::CUDAGuard guard(zc.device());
  check_rc(gphl_gat_fused_f32(g->plan(true, f), ptr.data_ptr<int32_t>(), ptr_or<int32_t>(nid, ptr), nullptr, g->num_nodes,
                              h, f / h, elc.data_ptr<float>(), erc.data_ptr<float>(), zc.data_ptr<float>(), (float)slope,
                              out.data_ptr<float>(), nullptr, stats.data_ptr<float>(), stream_of(zc)),
           "gphl_gat_fused_f32");
  return out;
}

// ---- typed linear -----------------------------------------------------------------------------
// Split weights of the tensor-core typed linear, kept per weight tensor: weights are constants of a layer, so the
// split kernel runs once per (tensor, version) instead of once per call.  An entry is valid while the very same
// TensorImpl is alive (a weak reference keeps its address from being reused), its version counter and storage
// address are unchanged and the call comes on the stream the workspace was written on; anything else is a miss.
struct PreparedWeights {
  c10::weak_intrusive_ptr<c10::TensorImpl> impl;
  const void *data;
  uint32_t version;
  int64_t t, k, n;
  void *stream;
  Tensor ws;
};
Tensor prepared_weights(const Tensor &wc, int64_t t, int64_t k, int64_t n, void *stream) {
  static std::mutex mu;
  static std::vector<PreparedWeights> cache;
  const bool trackable = !wc.is_inference();
  std::lock_guard<std::mutex> lock(mu);
  if (trackable) {
    for (size_t i = 0; i < cache.size(); ++i) {
      PreparedWeights &e = cache[i];
      if (e.impl._unsafe_get_target() == wc.unsafeGetTensorImpl() && !e.impl.expired() && e.data == wc.data_ptr() &&
          e.version == wc._version() && e.t == t && e.k == k && e.n == n && e.stream == stream) {
        if (i + 1 != cache.size()) std::rotate(cache.begin() + i, cache.begin() + i + 1, cache.end());   // most recent last
        return cache.back().ws;
      }
    }
  }
  Tensor ws = torch::empty({std::max<int64_t>(16, gphl_segment_mm_tc_workspace_bytes(t, k, n))}, wc.options().dtype(torch::kUInt8));
  check_rc(gphl_segment_mm_tc_prepare_weights(wc.data_ptr<float>(), t, k, n, ws.data_ptr(), stream), "gphl_segment_mm_tc_prepare_weights");
  if (trackable) {
    cache.erase(std::remove_if(cache.begin(), cache.end(), [](const PreparedWeights &e) { return e.impl.expired(); }), cache.end());
    if (cache.size() >= 64) cache.erase(cache.begin());
    cache.push_back(PreparedWeights{c10::weak_intrusive_ptr<c10::TensorImpl>(wc.getIntrusivePtr()), wc.data_ptr(), wc._version(),
                                    t, k, n, stream, ws});
  }
  return ws;
}

Tensor segment_mm(const Tensor &x, const Tensor &w, const c10::optional<Tensor> &pointer, int64_t n_types, int64_t rows,
                  const c10::optional<Tensor> &gather, const char *what) {
  TORCH_CHECK(pointer.has_value(), what, " needs the type pointer (SetNtypePointer / SetEtypePointer)");
  Tensor xc = cuda_f32(x, "features"), wc = cuda_f32(w, "weights");
  TORCH_CHECK(xc.dim() == 2 && wc.dim() == 3, what, ": features must be 2-D and weights 3-D");
  TORCH_CHECK(wc.size(0) == n_types, what, ": expected ", n_types, " weight matrices, got ", wc.size(0));
  TORCH_CHECK(wc.size(1) == xc.size(1), what, ": inner dimensions differ");
  TORCH_CHECK(gather.has_value() || xc.size(0) == rows, what, ": expected ", rows, " feature rows, got ", xc.size(0));
  Tensor pc = cuda_idx(pointer.value(), torch::kInt32, "type pointer");
  Tensor y = torch::empty({rows, wc.size(2)}, xc.options());
  Tensor gi;
  if (gather.has_value()) gi = cuda_idx(gather.value(), torch::kInt64, "gather index");
  c10::cuda::CUDAGuard guard(xc.device());
  const int64_t k = xc.size(1), n = wc.size(2);
  // narrow weights (k <= 64, n <= 32) take the double-accumulating SIMT kernel: a 128-row tensor-core tile would be
  // mostly padding there
  const bool tc = (k % 4 == 0) && !(k <= 64 && n <= 32) && (reinterpret_cast<uintptr_t>(xc.data_ptr()) % 16 == 0) &&
                  (reinterpret_cast<uintptr_t>(y.data_ptr()) % 16 == 0);
  if (tc) {
    // tensor-core path: the split, transposed weights depend on the weight tensor alone and are kept per tensor
    Tensor ws = prepared_weights(wc, n_types, k, n, stream_of(xc));
    check_rc(gphl_segment_mm_tc_prepared_f32(xc.data_ptr<float>(), ws.data_ptr(), pc.data_ptr<int32_t>(), n_types, rows, k, n,
                                             gather.has_value() ? gi.data_ptr<int64_t>() : nullptr, nullptr, 0,
                                             y.data_ptr<float>(), stream_of(xc)),
             "gphl_segment_mm_tc_prepared_f32");
  } else {
    check_rc(gphl_segment_mm_f32(xc.data_ptr<float>(), wc.data_ptr<float>(), pc.data_ptr<int32_t>(), n_types, rows, k, n,
                                 gather.has_value() ? gi.data_ptr<int64_t>() : nullptr, y.data_ptr<float>(),
                                 stream_of(xc)),
             "gphl_segment_mm_f32");
  }
  return y;
}

Tensor SegmentMMNode(Tensor x, Tensor w, const GraphPtr &g) {
  return segment_mm(x, w, g->ntype_pointer, g->num_ntypes, g->num_nodes, c10::nullopt, "SegmentMMNode");
}
Tensor SegmentMMEdge(Tensor x, Tensor w, const GraphPtr &g) {
  return segment_mm(x, w, g->etype_pointer, g->num_etypes, g->num_edges, c10::nullopt, "SegmentMMEdge");
}
// Not registered by the reference: BroadcastSrcNode fused into SegmentMMEdge (x holds node rows).
Tensor SegmentMMEdgeSrc(Tensor x, Tensor w, const GraphPtr &g) {
  TORCH_CHECK(x.size(0) == g->num_nodes, "SegmentMMEdgeSrc: features must have num_nodes rows");
  if (g->pair_src.defined() && g->etype_pointer.has_value()) {
    // one product row per distinct (edge type, source) pair, then handed out to the edges: the same rows bit for bit
    Tensor per_pair = segment_mm(x, w, g->pair_pointer, g->num_etypes, g->pair_src.size(0), g->pair_src, "SegmentMMEdgeSrc");
    return gather_rows(per_pair, g->edge_pair, c10::nullopt);
  }
  return segment_mm(x, w, g->etype_pointer, g->num_etypes, g->num_edges, g->COO_src, "SegmentMMEdgeSrc");
}

#define GRAPH_T "__torch__.torch.classes.my_classes.DGLGraph"

}  // namespace

TORCH_LIBRARY(my_classes, m) {
  m.class_<DGLGraph>("DGLGraph")
      .def(torch::init<Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, c10::optional<Tensor>,
                       c10::optional<Tensor>>())
      .def("SetNtypePointer", &DGLGraph::SetNtypePointer)
      .def("SetEtypePointer", &DGLGraph::SetEtypePointer)
      .def("SetNtypeCOO", &DGLGraph::SetNtypeCOO)
      .def("SetEtypeCOO", &DGLGraph::SetEtypeCOO);
}

static auto registry =
    torch::RegisterOperators(
        "my_ops::BroadcastSrcNode(Tensor x, " GRAPH_T " g) -> Tensor y", &BroadcastSrcNode)
        .op("my_ops::BroadcastDstNode(Tensor x, " GRAPH_T " g) -> Tensor y", &BroadcastDstNode)
        .op("my_ops::BroadcastNodeType(Tensor x, " GRAPH_T " g) -> Tensor y", &BroadcastNodeType)
        .op("my_ops::BroadcastSrcNodeType(Tensor x, " GRAPH_T " g) -> Tensor y", &BroadcastSrcNodeType)
        .op("my_ops::BroadcastDstNodeType(Tensor x, " GRAPH_T " g) -> Tensor y", &BroadcastDstNodeType)
        .op("my_ops::BroadcastEdgeType(Tensor x, " GRAPH_T " g) -> Tensor y", &BroadcastEdgeType)
        .op("my_ops::get_feat_dim", &get_feat_dim)
        .op("my_ops::SegmentSoftmax(Tensor x, int dim, int? t, " GRAPH_T " g) -> Tensor y", &SegmentSoftmax)
        .op("my_ops::SegmentMMNode(Tensor x, Tensor y, " GRAPH_T " g) -> Tensor z", &SegmentMMNode)
        .op("my_ops::SegmentMMEdge(Tensor x, Tensor y, " GRAPH_T " g) -> Tensor z", &SegmentMMEdge)
        .op("my_ops::SpMMEdge(Tensor x, int[] dim, bool k, int? t, " GRAPH_T " g) -> Tensor y", &SpMMEdge)
        .op("my_ops::SpMMSrc(Tensor x, int[] dim, bool k, int? t, " GRAPH_T " g) -> Tensor y", &SpMMSrc)
        .op("my_ops::gspmm_src_mul_e_sum(Tensor x, Tensor y, int[] dim, bool k, int? t, " GRAPH_T " g) -> Tensor z",
            &src_mul_e_sum)
        .op("my_ops::gspmm_dst_mul_e_sum(Tensor x, Tensor y, int[] dim, bool k, int? t, " GRAPH_T " g) -> Tensor z",
            &dst_mul_e_sum)
        .op("my_ops::gsddmm_u_add_v_mul_alpha(Tensor x, Tensor y, int alpha," GRAPH_T " g) -> Tensor z",
            &u_add_v_mul_alpha)
        // additions with no counterpart in the reference's registry
        .op("my_ops::gsddmm_u_dot_v(Tensor x, Tensor y, int heads, " GRAPH_T " g) -> Tensor z", &u_dot_v)
        .op("my_ops::gat_fused(Tensor el, Tensor er, Tensor z, float slope, " GRAPH_T " g) -> Tensor y", &gat_fused)
        .op("my_ops::SegmentMMEdgeSrc(Tensor x, Tensor y, " GRAPH_T " g) -> Tensor z", &SegmentMMEdgeSrc)
        .op("my_ops::gsddmm_e_dot_v(Tensor x, Tensor y, int heads, " GRAPH_T " g) -> Tensor z", &e_dot_v)
        .op("my_ops::SpMMEdgeMul(Tensor x, Tensor y, " GRAPH_T " g) -> Tensor z", &SpMMEdgeMul);
