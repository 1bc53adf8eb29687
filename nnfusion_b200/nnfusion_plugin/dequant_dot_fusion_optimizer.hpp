// Graph fold: Convert -> Subtract(Broadcast(zero-point)) -> Multiply(Broadcast(scale)) -> Dot(transpose_B)  ==>  DequantDot.
// Goes to src/nnfusion/engine/pass/graph/subgraph_fusion_optimizer/; base class:
// subgraph_fusion_optimizer.hpp:18-43; modelled on MatMulAddFusionOptimizer (matmuladd_fusion_optimizer.cpp:8-93).
// Invoked from SubGraphFusionPass::run_on_graph (subgraph_fusion_pass.cpp:27-140) through run_dequant_dot_fusion
// (dequant_dot_fusion_pass.cpp, which also defines the -fdequant_dot_fusion flag); it has to run before
// RuntimeConstantFoldingPass, which would otherwise fold constant weights to fp32.
#pragma once
#include "subgraph_fusion_optimizer.hpp"

namespace nnfusion
{
    namespace pass
    {
        namespace graph
        {
            class DequantDotFusionOptimizer : public SubGraphFusionOptimizer
            {
            public:
                DequantDotFusionOptimizer(std::shared_ptr<nnfusion::graph::Graph> g)
                    : SubGraphFusionOptimizer(g)
                {
                }
                bool create_subgraphs() override;
                bool fuse_subgraph(SubGraphRecord::Pointer subgraph_record) override;
            };

            bool run_dequant_dot_fusion(std::shared_ptr<nnfusion::graph::Graph>& graph);
        }
    }
}
