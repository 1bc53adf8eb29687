// DecodeAttention: one decoding step of an attention layer as a single graph node.
//   inputs : q [heads, head_dim], k [kv_heads, head_dim], v [kv_heads, head_dim] of the new token (fp16),
//            k_cache, v_cache [kv_heads, capacity, head_dim] (persistent tensors, updated in place at `position`)
//   output : [1, heads * head_dim]
// It stands for the sub-graph Slice/Negative/Concat/Multiply/Add (rotary embedding) -> BatchMatMul(adj_y) ->
// Softmax -> BatchMatMul plus the cache Concat; a frontend (or a SubGraphFusionOptimizer in the style of
// dequant_dot_fusion_optimizer.cpp) creates it.  Goes to
// src/nnfusion/core/operators/generic_op/generic_op_define/DecodeAttention.cpp
// (registration interface: src/nnfusion/core/operators/generic_op/generic_op.hpp:54-171; shape rules of the
// operators it replaces: generic_op_define/BatchMatMul.cpp:6-50).
#include "nnfusion/core/operators/generic_op/generic_op.hpp"

REGISTER_OP(DecodeAttention)
    .attr<int>("heads")
    .attr<int>("kv_heads")
    .attr<int>("head_dim", 128)
    .attr<int>("position")
    .attr<bool>("rotary", true)
    .attr<float>("rotary_base", 10000.0f)
    .attr<float>("softmax_scale", 0.0f) // 0: 1/sqrt(head_dim)
    .constrait([](const nnfusion::op::OpConfig::any& config) -> bool {
        const int heads = config["heads"], kv_heads = config["kv_heads"];
        return heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && (int)config["head_dim"] == 128 &&
               (int)config["position"] >= 0;
    })
    .infershape([](std::shared_ptr<graph::GNode> gnode) -> void {
        NNFUSION_CHECK(gnode->get_input_size() == 5) << "q, k, v, k_cache, v_cache";
        auto op = std::dynamic_pointer_cast<nnfusion::op::GenericOp>(gnode->get_op_ptr());
        auto& cfg = op->localOpConfig.getRoot();
        const size_t heads = (int)cfg["heads"], kv_heads = (int)cfg["kv_heads"], dim = (int)cfg["head_dim"];
        const nnfusion::Shape& cache = gnode->get_input_shape(3);
        NNFUSION_CHECK(cache.size() == 3 && cache[0] == kv_heads && cache[2] == dim);
        NNFUSION_CHECK(gnode->get_input_shape(4) == cache);
        NNFUSION_CHECK((size_t)(int)cfg["position"] < cache[1]) << "the caches are full";
        NNFUSION_CHECK(nnfusion::shape_size(gnode->get_input_shape(0)) == heads * dim);
        NNFUSION_CHECK(nnfusion::shape_size(gnode->get_input_shape(1)) == kv_heads * dim);
        NNFUSION_CHECK(nnfusion::shape_size(gnode->get_input_shape(2)) == kv_heads * dim);
        for (size_t i = 0; i < 5; i++)
            NNFUSION_CHECK(gnode->get_input_element_type(i) == nnfusion::element::f16);
        gnode->set_output_type_and_shape(0, nnfusion::element::f16, nnfusion::Shape{1, heads * dim});
    });
