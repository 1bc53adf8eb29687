// See dequant_dot_fusion_optimizer.hpp.
//
// The sub-graph the ONNX importer produces for Y = X . ((Cast(W) - zp) * scale)^T (opset >= 7; importer:
// src/nnfusion/frontend/onnx_import/op/cast.hpp:35-51, op/binaryop.hpp:89-107, broadcasting plan
// src/nnfusion/core/graph/util/autobroadcast.cpp:83-151):
//
//   W  u8[N,K] -- [Reshape] -- Convert(f32) ------------------------------------------+
//   zp u8[N,G,1] -- Convert(f32) -- Reshape -- Broadcast(inner = group) --------------+- Subtract -+
//   s  [N,G,1] ------------------- Reshape -- Broadcast(inner = group) ----------------------------+- Multiply -- [Reshape] -- Dot(transB)
//
// The walk below starts at Dot and goes up its second operand; Reshape nodes that keep the element count are
// skipped, Broadcast must be an inner broadcast (op_define/broadcast.cpp:71-117) whose inner size is the group.
#include "dequant_dot_fusion_optimizer.hpp"
#include "nnfusion/core/operators/op_define/broadcast.hpp"
#include "nnfusion/core/operators/op_define/dot.hpp"

using namespace nnfusion;
using namespace nnfusion::graph;
using namespace nnfusion::pass::graph;

namespace
{
    std::shared_ptr<GNode> skip_reshapes(std::shared_ptr<GNode> n)
    {
        while (n->get_op_type() == "Reshape" && n->get_out_edges().size() == 1)
            n = n->get_in_edge(0)->get_src();
        return n;
    }

    // Producer of a broadcast quantisation parameter; returns the pre-broadcast node and the inner size.
    bool match_param(std::shared_ptr<GNode> n, std::shared_ptr<GNode>& param, size_t& inner, bool expect_convert)
    {
        if (n->get_op_type() != "Broadcast")
            return false;
        auto bc = std::dynamic_pointer_cast<op::Broadcast>(n->get_op_ptr());
        if (!bc || !bc->is_inner_broadcast())
            return false;
        inner = bc->get_inner_broadcast_size();
        auto src = skip_reshapes(n->get_in_edge(0)->get_src());
        if (expect_convert)
        {
            if (src->get_op_type() != "Convert")
                return false;
            src = skip_reshapes(src->get_in_edge(0)->get_src());
        }
        param = src;
        return true;
    }
}

bool DequantDotFusionOptimizer::create_subgraphs()
{
    auto check_root = [](std::shared_ptr<GNode> gnode) -> bool {
        if (gnode->get_op_type() != "Dot")
            return false;
        auto dot = std::dynamic_pointer_cast<op::Dot>(gnode->get_op_ptr());
        return dot && dot->get_transpose_B() && !dot->get_transpose_A() && gnode->get_input_shape(0).size() == 2 &&
               gnode->get_input_shape(1).size() == 2;
    };
    SubGraph::Pointer sg = std::make_shared<SubGraph>();
    sg->name = "dequant_dot";
    sg->check_starting_node = check_root;
    {
        // the chain is matched upwards from Dot: Multiply <- Subtract <- Convert, with optional Reshapes handled
        // in fuse_subgraph (the matcher only anchors on the three arithmetic nodes)
        Pattern::Pointer p = std::make_shared<Pattern>();
        std::vector<std::string> ops{"Dot", "Multiply", "Subtract", "Convert"};
        p->descriptions.push_back(std::make_pair(ops, 1));
        p->reverse_order = true;
        sg->patterns.push_back(p);
    }
    m_subgraphs.push_back(sg);
    return true;
}

bool DequantDotFusionOptimizer::fuse_subgraph(SubGraphRecord::Pointer subgraph_record)
{
    auto pr = subgraph_record->pattern_records[0];
    auto dot = pr->nodes[0], mul = pr->nodes[1], sub = pr->nodes[2], cvt = pr->nodes[3];
    auto x = dot->get_in_edge(0)->get_src();
    auto wq = skip_reshapes(cvt->get_in_edge(0)->get_src());
    if (wq->get_output_element_type(0) != element::u8)
        return false;

    // which operand of Subtract / Multiply is the broadcast parameter
    std::shared_ptr<GNode> zp, scale;
    size_t inner_zp = 0, inner_s = 0;
    if (!match_param(sub->get_in_edge(1)->get_src(), zp, inner_zp, /*expect_convert*/ true))
        return false;
    bool found = false;
    for (auto e : mul->get_in_edges())
        if (skip_reshapes(e->get_src()) != sub && match_param(e->get_src(), scale, inner_s, false))
            found = true;
    if (!found || inner_zp != inner_s || zp->get_output_element_type(0) != element::u8)
        return false;

    const auto w_shape = wq->get_output_shape(0);
    const size_t K = dot->get_input_shape(1)[1];
    nnfusion::op::OpConfig::any cfg;
    cfg["w_bits"] = 8; // packed 4-bit weights reach the graph already as a DequantDot (no 4-bit element type exists)
    cfg["group_size"] = (inner_s == K) ? 0 : (int)inner_s;
    cfg["prologue"] = "none";
    cfg["epilogue"] = "none";
    cfg["rms_eps"] = 1e-6f;
    auto op = std::make_shared<nnfusion::op::GenericOp>(dot->get_name() + "_dq", "DequantDot", cfg);
    auto fused = graph->add_node_and_edge(
        op, {GNodeIndex{x, 0}, GNodeIndex{wq, 0}, GNodeIndex{scale, 0}, GNodeIndex{zp, 0}});

    for (auto out_edge : dot->get_out_edges())
    {
        auto dst = out_edge->get_dst();
        int slot = out_edge->get_dst_input();
        graph->remove_edge(out_edge);
        graph->add_edge(fused, 0, dst, slot);
    }
    // remove the arithmetic chain with its Reshape / Broadcast / Convert helpers when nothing else reads them
    std::unordered_set<std::shared_ptr<GNode>> dead{dot, mul, sub, cvt};
    std::queue<std::shared_ptr<GNode>> work;
    for (auto n : {mul, sub})
        for (auto e : n->get_in_edges())
            work.push(e->get_src());
    while (!work.empty())
    {
        auto n = work.front();
        work.pop();
        const auto t = n->get_op_type();
        if ((t == "Reshape" || t == "Broadcast" || t == "Convert") && n->get_out_edges().size() <= 1 && !dead.count(n))
        {
            dead.insert(n);
            for (auto e : n->get_in_edges())
                work.push(e->get_src());
        }
    }
    (void)w_shape;
    return RemoveNodes(dead, fused);
}
