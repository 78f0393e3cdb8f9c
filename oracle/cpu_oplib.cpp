// CPU registration of the my_ops operators and the DGLGraph class.  TEST INFRASTRUCTURE ONLY.
//
// Lets the reference's own MP-DFG builder, optimizer passes and Python wrapper (compiled into
// oracle/_ref/ by oracle/build_ref.py) run on a machine without a GPU, so that the operator
// semantics restated in oracle/ops_oracle.py can be pinned against the reference's compiler:
// the graph it emits calls these bodies, and the result must equal the user-defined-function
// path.  Never linked into, loaded by or timed as part of the shipped package.  The bodies are
// plain ATen calls on whatever dtype comes in (float32 or float64); each cites the reference
// operator whose semantics it restates.
#include <torch/custom_class.h>
#include <torch/script.h>

using torch::Tensor;

struct DGLGraph : torch::CustomClassHolder {  // include/dglgraph.h:7-75
  DGLGraph(Tensor in_pointer, Tensor in_node_indices, Tensor in_edge_indices, Tensor out_pointer,
           Tensor out_node_indices, Tensor out_edge_indices, Tensor COO_src, Tensor COO_dst,
           c10::optional<Tensor> ntype_pointer, c10::optional<Tensor> etype_pointer)
      : in_pointer(in_pointer), in_node_indices(in_node_indices), in_edge_indices(in_edge_indices),
        out_pointer(out_pointer), out_node_indices(out_node_indices), out_edge_indices(out_edge_indices),
        COO_src(COO_src), COO_dst(COO_dst), ntype_pointer(ntype_pointer), etype_pointer(etype_pointer) {
    num_nodes = in_pointer.size(0) - 1;
    num_edges = in_node_indices.size(0);
  }
  void SetNtypePointer(Tensor t) { ntype_pointer = t; }
  void SetEtypePointer(Tensor t) { etype_pointer = t; }
  void SetNtypeCOO(Tensor t) { ntype_COO = t; }
  void SetEtypeCOO(Tensor t) { etype_COO = t; }
  // row id of every position of a pointer-grouped array
  static Tensor rows_of(const Tensor &pointer) {
    auto p = pointer.to(torch::kLong);
    auto deg = p.slice(0, 1) - p.slice(0, 0, -1);
    return torch::repeat_interleave(torch::arange(deg.size(0), torch::kLong), deg);
  }
  int64_t num_nodes, num_edges;
  Tensor in_pointer, in_node_indices, in_edge_indices, out_pointer, out_node_indices, out_edge_indices;
  Tensor COO_src, COO_dst;
  c10::optional<Tensor> ntype_pointer, etype_pointer, ntype_COO, etype_COO;
};

using G = c10::intrusive_ptr<DGLGraph>;

static Tensor two_d(const Tensor &x) { return x.dim() <= 1 ? x.reshape({x.size(0), 1}) : x.flatten(1); }

// broadcast.cu:58-100
static Tensor BroadcastSrcNode(Tensor x, const G &g) { return x.index_select(0, g->COO_src); }
static Tensor BroadcastDstNode(Tensor x, const G &g) { return x.index_select(0, g->COO_dst); }
static Tensor BroadcastNodeType(Tensor x, const G &g) { return x.index_select(0, g->ntype_COO.value()); }
static Tensor BroadcastEdgeType(Tensor x, const G &g) { return x.index_select(0, g->etype_COO.value()); }
static Tensor BroadcastSrcNodeType(Tensor x, const G &g) { return BroadcastSrcNode(BroadcastNodeType(x, g), g); }
static Tensor BroadcastDstNodeType(Tensor x, const G &g) { return BroadcastDstNode(BroadcastNodeType(x, g), g); }
static int64_t get_feat_dim(Tensor x) {  // broadcast.cu:3-9
  int64_t f = 1;
  for (int64_t i = 1; i < x.dim(); ++i) f *= x.size(i);
  return f;
}

// y[v] = sum over positions of row v of vals[pos]
static Tensor segment_sum(const Tensor &vals, const Tensor &pointer, int64_t rows) {
  auto out = torch::zeros({rows, vals.size(1)}, vals.options());
  return out.index_add_(0, DGLGraph::rows_of(pointer), vals);
}

// spmm.cu:359-389
static Tensor SpMMEdge(Tensor x, std::vector<int64_t>, bool, c10::optional<int64_t>, const G &g) {
  return segment_sum(two_d(x).index_select(0, g->in_edge_indices.to(torch::kLong)), g->in_pointer, g->num_nodes);
}
static Tensor SpMMSrc(Tensor x, std::vector<int64_t>, bool, c10::optional<int64_t>, const G &g) {
  return segment_sum(two_d(x).index_select(0, g->in_node_indices.to(torch::kLong)), g->in_pointer, g->num_nodes);
}
// spmm.cu:286-356, with the per-head broadcast of bcast.h:21-35
static Tensor mul_e_sum(const Tensor &x, const Tensor &w, const Tensor &pointer, const Tensor &nid, const Tensor &eid,
                        int64_t rows) {
  auto x2 = two_d(x), w2 = two_d(w);
  const int64_t h = w2.size(1), f = x2.size(1);
  auto xs = x2.index_select(0, nid.to(torch::kLong)).reshape({-1, h, f / h});
  auto ws = w2.index_select(0, eid.to(torch::kLong)).reshape({-1, h, 1});
  return segment_sum((xs * ws).reshape({-1, f}), pointer, rows);
}
static Tensor src_mul_e_sum(Tensor x, Tensor w, std::vector<int64_t>, bool, c10::optional<int64_t>, const G &g) {
  return mul_e_sum(x, w, g->in_pointer, g->in_node_indices, g->in_edge_indices, g->num_nodes);
}
static Tensor dst_mul_e_sum(Tensor x, Tensor w, std::vector<int64_t>, bool, c10::optional<int64_t>, const G &g) {
  return mul_e_sum(x, w, g->out_pointer, g->out_node_indices, g->out_edge_indices, g->num_nodes);
}
// sddmm.cu:118-129 (alpha ignored there too)
static Tensor u_add_v_mul_alpha(Tensor l, Tensor r, int64_t, const G &g) {
  return two_d(l).index_select(0, g->COO_src) + two_d(r).index_select(0, g->COO_dst);
}
// segment_softmax.cu:3-24 as a true softmax per destination
static Tensor SegmentSoftmax(Tensor x, int64_t dim, c10::optional<int64_t>, const G &g) {
  TORCH_CHECK(dim == 1, "dim must be 1");
  auto x2 = two_d(x);
  auto eid = g->in_edge_indices.to(torch::kLong);
  auto rows = DGLGraph::rows_of(g->in_pointer);
  auto xs = x2.index_select(0, eid);
  auto mx = torch::full({g->num_nodes, x2.size(1)}, -std::numeric_limits<double>::infinity(), x2.options());
  mx.index_reduce_(0, rows, xs, "amax", true);
  auto ex = (xs - mx.index_select(0, rows)).exp();
  auto den = torch::zeros({g->num_nodes, x2.size(1)}, x2.options()).index_add_(0, rows, ex);
  auto y = torch::zeros_like(x2);
  y.index_copy_(0, eid, ex / den.index_select(0, rows));
  return y.reshape(x.sizes());
}
// segment_mm.cu:4-33
static Tensor segment_mm(const Tensor &x, const Tensor &w, const Tensor &pointer) {
  auto p = pointer.to(torch::kLong);
  std::vector<Tensor> parts;
  for (int64_t t = 0; t + 1 < p.size(0); ++t)
    parts.push_back(at::mm(x.slice(0, p[t].item<int64_t>(), p[t + 1].item<int64_t>()), w[t]));
  return torch::cat(parts, 0);
}
static Tensor SegmentMMNode(Tensor x, Tensor w, const G &g) { return segment_mm(x, w, g->ntype_pointer.value()); }
static Tensor SegmentMMEdge(Tensor x, Tensor w, const G &g) { return segment_mm(x, w, g->etype_pointer.value()); }


// ---- operators the reference does not register: the targets of the added fusion patterns, restated as the
// unfused chains they replace so that a rewritten graph can be checked on the CPU -------------------------------
static Tensor u_dot_v(Tensor l, Tensor r, int64_t heads, const G &g) {
  if (l.dim() != 2 || r.dim() != 2 || l.size(1) != r.size(1))      // the chain the rewrite replaced, literally
    return at::mul(l.index_select(0, g->COO_src), r.index_select(0, g->COO_dst)).sum({1}, true);
  auto a = two_d(l).index_select(0, g->COO_src), b = two_d(r).index_select(0, g->COO_dst);
  return (a * b).reshape({a.size(0), heads, -1}).sum(2);
}
static Tensor e_dot_v(Tensor e, Tensor v, int64_t heads, const G &g) {
  auto p = at::mul(e, v.index_select(0, g->COO_dst));
  if (heads == 1) return p.sum({1}, true);
  return p.reshape({p.size(0), heads, -1}).sum(2);
}
static Tensor SpMMEdgeMul(Tensor a, Tensor b, const G &g) {
  std::vector<int64_t> dims{1};
  auto a2 = two_d(a), b2 = two_d(b);
  if (a2.size(1) != b2.size(1) && a2.size(1) > 1 && b2.size(1) > 1) {   // per-head weights
    const bool a_is_w = a2.size(1) < b2.size(1);
    const Tensor &x = a_is_w ? b2 : a2, &w = a_is_w ? a2 : b2;
    const int64_t h = w.size(1);
    return SpMMEdge((x.reshape({-1, h, x.size(1) / h}) * w.reshape({-1, h, 1})).reshape({-1, x.size(1)}), dims, false,
                    c10::nullopt, g);
  }
  return SpMMEdge(at::mul(a, b), dims, false, c10::nullopt, g);
}
static Tensor gat_fused(Tensor el, Tensor er, Tensor z, double slope, const G &g) {
  std::vector<int64_t> dims{1};
  auto e = at::leaky_relu(u_add_v_mul_alpha(el, er, 1, g), slope);
  return src_mul_e_sum(z, SegmentSoftmax(e, 1, c10::nullopt, g), dims, false, c10::nullopt, g);
}
static Tensor SegmentMMEdgeSrc(Tensor x, Tensor w, const G &g) { return SegmentMMEdge(BroadcastSrcNode(x, g), w, g); }

#define GRAPH_T "__torch__.torch.classes.my_classes.DGLGraph"

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
    torch::RegisterOperators("my_ops::BroadcastSrcNode(Tensor x, " GRAPH_T " g) -> Tensor y", &BroadcastSrcNode)
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
        .op("my_ops::gsddmm_u_dot_v(Tensor x, Tensor y, int heads, " GRAPH_T " g) -> Tensor z", &u_dot_v)
        .op("my_ops::gsddmm_e_dot_v(Tensor x, Tensor y, int heads, " GRAPH_T " g) -> Tensor z", &e_dot_v)
        .op("my_ops::SpMMEdgeMul(Tensor x, Tensor y, " GRAPH_T " g) -> Tensor z", &SpMMEdgeMul)
        .op("my_ops::gat_fused(Tensor el, Tensor er, Tensor z, float slope, " GRAPH_T " g) -> Tensor y", &gat_fused)
        .op("my_ops::SegmentMMEdgeSrc(Tensor x, Tensor y, " GRAPH_T " g) -> Tensor z", &SegmentMMEdgeSrc);
