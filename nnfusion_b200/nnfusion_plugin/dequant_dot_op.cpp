// Operator "DequantDot": Y[M,N] = epilogue(prologue(X)[M,K] . dequant(W)[N,K]^T), the node the fold pass puts in
// place of Convert -> Subtract -> Multiply -> Dot(transpose_B).
// Goes to src/nnfusion/core/operators/generic_op/generic_op_define/DequantDot.cpp; registration interface:
// src/nnfusion/core/operators/generic_op/generic_op.hpp:54-171 (same pattern as generic_op_define/MatMulAdd.cpp).
//
// Inputs : 0 X [M,K] (f16 / f32), 1 Wq (u8; [N,K] for 8-bit, [N,K/2] for packed 4-bit), 2 scale [N,K/group],
//          3 zero-point (u8, packed like Wq for 4-bit), then optionally, in this order,
//          gain [K] (prologue = "rmsnorm"), bias [N] (epilogue = "bias"), an addend [M,N] of the output's type
//          (epilogue = "add": MatMulAdd with its full-size C, generic_op_define/MatMulAdd.cpp:6-35), or
//          Wq2, scale2, zp2 (epilogue = "silu_mul").
// Attribute out_dtype ("", "float", "half"): element type of Y; empty keeps the element type of X.
#include "nnfusion/core/operators/generic_op/generic_op.hpp"

REGISTER_OP(DequantDot)
    .attr<int>("w_bits", 4)
    .attr<int>("group_size", 128) // 0: one scale / zero-point per output channel
    .attr<std::string>("prologue", "none")
    .attr<std::string>("epilogue", "none")
    .attr<float>("rms_eps", 1e-6f)
    .attr<std::string>("out_dtype", "") // empty: the element type of X
    .constrait([](const nnfusion::op::OpConfig::any& config) -> bool {
        const int bits = config["w_bits"];
        const int group = config["group_size"];
        const std::string pro = config["prologue"], epi = config["epilogue"];
        return (bits == 4 || bits == 8) && group >= 0 && (pro == "none" || pro == "rmsnorm") &&
               (epi == "none" || epi == "bias" || epi == "silu_mul" || epi == "add");
    })
    .infershape([](std::shared_ptr<graph::GNode> gnode) -> void {
        auto op = static_pointer_cast<nnfusion::op::GenericOp>(gnode->get_op_ptr());
        NNFUSION_CHECK_NOT_NULLPTR(op) << "Node type is not " << gnode->get_op_ptr()->get_op_type();
        auto& cfg = op->localOpConfig.getRoot();
        const int bits = cfg["w_bits"];
        NNFUSION_CHECK(gnode->get_input_size() >= 4) << "DequantDot takes X, Wq, scale and zero-point.";
        const auto x_shape = gnode->get_input_shape(0);
        const auto w_shape = gnode->get_input_shape(1);
        NNFUSION_CHECK(x_shape.size() == 2 && w_shape.size() == 2) << "DequantDot only supports matrices.";
        const size_t k = x_shape[1];
        const size_t k_stored = (bits == 4) ? w_shape[1] * 2 : w_shape[1];
        NNFUSION_CHECK(k == k_stored) << "Contraction sizes of X and Wq differ.";
        nnfusion::Shape out{x_shape[0], w_shape[0]};
        const std::string out_dtype = cfg["out_dtype"];
        nnfusion::element::Type out_type = gnode->get_input_element_type(0);
        if (out_dtype == "float")
            out_type = nnfusion::element::f32;
        else if (out_dtype == "half")
            out_type = nnfusion::element::f16;
        else
            NNFUSION_CHECK(out_dtype.empty()) << "DequantDot: out_dtype must be \"\", \"float\" or \"half\".";
        const std::string epi = cfg["epilogue"];
        if (epi == "add")
        {
            const size_t slot = 4 + (std::string(cfg["prologue"]) == "rmsnorm" ? 1 : 0);
            NNFUSION_CHECK(gnode->get_input_size() > slot) << "DequantDot: the add epilogue takes an [M,N] addend.";
            NNFUSION_CHECK(gnode->get_input_shape(slot) == out && gnode->get_input_element_type(slot) == out_type)
                << "DequantDot: the addend must have the output's shape and element type.";
        }
        gnode->set_output_type_and_shape(0, out_type, out);
    });
