// The flag and the call that put DequantDotFusionOptimizer into the compiler's pass list.
// Both belong in src/nnfusion/engine/pass/graph/subgraph_fusion_pass.cpp: the flag next to
// DEFINE_bool(fmatmuladd_fusion, ...) (:17-25), the call at the top of SubGraphFusionPass::run_on_graph (:27-140), in
// front of the other optimizers, as
//
//     nnfusion::pass::graph::run_dequant_dot_fusion(graph);
//
// SubGraphFusionPass itself runs before RuntimeConstantFoldingPass in the CUDA pass list
// (src/nnfusion/engine/device/cuda.cpp:49), so constant weights still are uint8 when the fold sees them.
#include "dequant_dot_fusion_optimizer.hpp"
#include "nnfusion/util/util.hpp"

DEFINE_bool(fdequant_dot_fusion, false, "Fold the Cast-Sub-Mul dequantisation chain into Dot (B200 kernels).");
DECLARE_bool(fenable_all_subgraph_fusion);

namespace nnfusion
{
    namespace pass
    {
        namespace graph
        {
            // Returns false only when the optimizer ran and failed; a switched-off fold is not a failure.
            bool run_dequant_dot_fusion(std::shared_ptr<nnfusion::graph::Graph>& graph)
            {
                if (!(FLAGS_fdequant_dot_fusion || FLAGS_fenable_all_subgraph_fusion))
                    return true;
                NNFUSION_LOG(NNFUSION_WARNING) << "DequantDotFusion Optimization begin.";
                auto optimizer = std::make_shared<DequantDotFusionOptimizer>(graph);
                if (!optimizer->Optimize())
                {
                    NNFUSION_LOG(NNFUSION_WARNING) << "DequantDotFusion Optimization failed.";
                    return false;
                }
                NNFUSION_LOG(INFO) << "DequantDotFusion Optimization Done.";
                return true;
            }
        } // namespace graph
    }     // namespace pass
} // namespace nnfusion
