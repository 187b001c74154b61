// Library nodes the B200 target adds to docc: scaled-dot-product attention and LayerNorm.
//
// docc has no node for either (its tensor nodes end at MatMul / Softmax / Mean / Std / element-wise ops), so a front
// end can only spell them as a chain of those, with every intermediate materialised. These two nodes keep the
// operation whole until code generation, where the B200 dispatchers turn each into one runtime call.
// Both follow the pattern of docc's own math nodes: a MathNode subclass (math_node.h:66-102) with validate / symbols /
// replace / clone / toStr, plus a LibraryNodeSerializer (gemm_node.h:89-96, conv_node.h:206) so that a dumped SDFG
// round-trips. Builds inside a docc source tree only.
#pragma once

#include <sdfg/data_flow/library_nodes/math/tensor/tensor_node.h>
#include <sdfg/serializer/json_serializer.h>

namespace docc::target::b200 {

inline sdfg::data_flow::LibraryNodeCode LibraryNodeType_Attention("ml::Attention");
inline sdfg::data_flow::LibraryNodeCode LibraryNodeType_LayerNorm("ml::LayerNorm");

// O[b,h,i,:] = sum_j softmax_j(scale * <Q[b,h,i,:], K[b,h,j,:]> [j <= i + seq_kv - seq_q]) * V[b,h,j,:]
// Connectors Q, K, V -> O; all four tensors are C-order [batch, heads, seq, head_dim].
class AttentionNode : public sdfg::math::tensor::TensorNode {
    sdfg::symbolic::Expression batch_, heads_, seq_q_, seq_kv_, head_dim_;
    double scale_;  // <= 0 selects 1 / sqrt(head_dim) at run time
    bool causal_;

public:
    AttentionNode(size_t element_id, const sdfg::DebugInfo& debug_info, const sdfg::graph::Vertex vertex,
                  sdfg::data_flow::DataFlowGraph& parent, sdfg::symbolic::Expression batch, sdfg::symbolic::Expression heads,
                  sdfg::symbolic::Expression seq_q, sdfg::symbolic::Expression seq_kv, sdfg::symbolic::Expression head_dim,
                  double scale, bool causal);

    const sdfg::symbolic::Expression& batch() const { return batch_; }
    const sdfg::symbolic::Expression& heads() const { return heads_; }
    const sdfg::symbolic::Expression& seq_q() const { return seq_q_; }
    const sdfg::symbolic::Expression& seq_kv() const { return seq_kv_; }
    const sdfg::symbolic::Expression& head_dim() const { return head_dim_; }
    double scale() const { return scale_; }
    bool causal() const { return causal_; }

    void validate(const sdfg::Function& function) const override;
    sdfg::symbolic::SymbolSet symbols() const override;
    void replace(const sdfg::symbolic::Expression old_expression, const sdfg::symbolic::Expression new_expression) override;
    std::unique_ptr<sdfg::data_flow::DataFlowNode> clone(size_t element_id, const sdfg::graph::Vertex vertex,
                                                         sdfg::data_flow::DataFlowGraph& parent) const override;
    std::string toStr() const override;
    // 4 * batch * heads * seq_q * seq_kv * head_dim (two contractions; halved by convention under a causal mask)
    sdfg::symbolic::Expression flop() const override;
    // No loop-nest form is provided: the node exists so that the score matrix is never materialised, which an
    // expansion into MatMul / Softmax / MatMul would undo. A target without a dispatcher for it must reject the SDFG.
    bool expand(sdfg::builder::StructuredSDFGBuilder& builder, sdfg::analysis::AnalysisManager& analysis_manager) override;
    bool supports_integer_types() const override { return false; }
};

class AttentionNodeSerializer : public sdfg::serializer::LibraryNodeSerializer {
public:
    nlohmann::json serialize(const sdfg::data_flow::LibraryNode& library_node) override;
    sdfg::data_flow::LibraryNode& deserialize(const nlohmann::json& j, sdfg::builder::StructuredSDFGBuilder& builder,
                                              sdfg::structured_control_flow::Block& parent) override;
};

// Y = (X - mean) / sqrt(var + eps) * G + B over the last dimension of `shape` (population variance, as StdNode).
// Connectors X, [G, B] -> Y; G and B are fp32 vectors of the last dimension's length.
class LayerNormNode : public sdfg::math::tensor::TensorNode {
    std::vector<sdfg::symbolic::Expression> shape_;
    double eps_;
    bool affine_;

public:
    LayerNormNode(size_t element_id, const sdfg::DebugInfo& debug_info, const sdfg::graph::Vertex vertex,
                  sdfg::data_flow::DataFlowGraph& parent, const std::vector<sdfg::symbolic::Expression>& shape, double eps,
                  bool affine);

    const std::vector<sdfg::symbolic::Expression>& shape() const { return shape_; }
    double eps() const { return eps_; }
    bool affine() const { return affine_; }
    sdfg::symbolic::Expression rows() const;  // product of all but the last dimension
    sdfg::symbolic::Expression cols() const { return shape_.back(); }

    void validate(const sdfg::Function& function) const override;
    sdfg::symbolic::SymbolSet symbols() const override;
    void replace(const sdfg::symbolic::Expression old_expression, const sdfg::symbolic::Expression new_expression) override;
    std::unique_ptr<sdfg::data_flow::DataFlowNode> clone(size_t element_id, const sdfg::graph::Vertex vertex,
                                                         sdfg::data_flow::DataFlowGraph& parent) const override;
    std::string toStr() const override;
    bool expand(sdfg::builder::StructuredSDFGBuilder& builder, sdfg::analysis::AnalysisManager& analysis_manager) override;
    bool supports_integer_types() const override { return false; }
};

class LayerNormNodeSerializer : public sdfg::serializer::LibraryNodeSerializer {
public:
    nlohmann::json serialize(const sdfg::data_flow::LibraryNode& library_node) override;
    sdfg::data_flow::LibraryNode& deserialize(const nlohmann::json& j, sdfg::builder::StructuredSDFGBuilder& builder,
                                              sdfg::structured_control_flow::Block& parent) override;
};

}  // namespace docc::target::b200
