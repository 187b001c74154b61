// AttentionNode and LayerNormNode (see b200_nodes.h). Compiled inside a docc tree.
#include "b200_nodes.h"

#include <sdfg/builder/structured_sdfg_builder.h>
#include <sdfg/symbolic/symbolic.h>

namespace docc::target::b200 {

using namespace sdfg;

namespace {
void add_atoms(symbolic::SymbolSet& syms, const symbolic::Expression& e) {
    for (auto& atom : symbolic::atoms(e)) syms.insert(atom);
}
}  // namespace

// ---- AttentionNode -------------------------------------------------------------------------------------
AttentionNode::AttentionNode(size_t element_id, const DebugInfo& debug_info, const graph::Vertex vertex,
                             data_flow::DataFlowGraph& parent, symbolic::Expression batch, symbolic::Expression heads,
                             symbolic::Expression seq_q, symbolic::Expression seq_kv, symbolic::Expression head_dim, double scale,
                             bool causal)
    : math::tensor::TensorNode(element_id, debug_info, vertex, parent, LibraryNodeType_Attention, {"O"}, {"Q", "K", "V"},
                               data_flow::ImplementationType_NONE),
      batch_(batch), heads_(heads), seq_q_(seq_q), seq_kv_(seq_kv), head_dim_(head_dim), scale_(scale), causal_(causal) {}

void AttentionNode::validate(const Function& function) const {
    math::tensor::TensorNode::validate(function);  // one primitive type on all connectors, no integers
    auto& graph = this->get_parent();
    if (graph.in_degree(*this) != 3 || graph.out_degree(*this) != 1)
        throw InvalidSDFGException("AttentionNode: expects the inputs Q, K, V and the output O");
    // Every connector carries a rank-4 tensor whose extents match the node's
    for (auto& edge : graph.in_edges(*this)) {
        auto& t = static_cast<const types::Tensor&>(edge.base_type());
        if (t.shape().size() != 4) throw InvalidSDFGException("AttentionNode: operands must be [batch, heads, seq, head_dim]");
        const bool is_q = edge.dst_conn() == "Q";
        if (!symbolic::eq(t.shape().at(0), batch_) || !symbolic::eq(t.shape().at(1), heads_) ||
            !symbolic::eq(t.shape().at(2), is_q ? seq_q_ : seq_kv_) || !symbolic::eq(t.shape().at(3), head_dim_))
            throw InvalidSDFGException("AttentionNode: shape of " + edge.dst_conn() + " does not match the node");
    }
}

symbolic::SymbolSet AttentionNode::symbols() const {
    symbolic::SymbolSet syms;
    for (auto& e : {batch_, heads_, seq_q_, seq_kv_, head_dim_}) add_atoms(syms, e);
    return syms;
}

void AttentionNode::replace(const symbolic::Expression old_expression, const symbolic::Expression new_expression) {
    for (auto* e : {&batch_, &heads_, &seq_q_, &seq_kv_, &head_dim_}) *e = symbolic::subs(*e, old_expression, new_expression);
}

std::unique_ptr<data_flow::DataFlowNode> AttentionNode::clone(size_t element_id, const graph::Vertex vertex,
                                                              data_flow::DataFlowGraph& parent) const {
    auto node = std::unique_ptr<AttentionNode>(new AttentionNode(element_id, this->debug_info(), vertex, parent, batch_, heads_,
                                                                 seq_q_, seq_kv_, head_dim_, scale_, causal_));
    node->implementation_type() = this->implementation_type();
    return node;
}

std::string AttentionNode::toStr() const {
    return LibraryNode::toStr() + "(" + batch_->__str__() + ", " + heads_->__str__() + ", " + seq_q_->__str__() + ", " +
           seq_kv_->__str__() + ", " + head_dim_->__str__() + ", scale=" + std::to_string(scale_) + (causal_ ? ", causal)" : ")");
}

symbolic::Expression AttentionNode::flop() const {
    auto f = symbolic::mul(symbolic::integer(causal_ ? 2 : 4),
                           symbolic::mul(symbolic::mul(batch_, heads_), symbolic::mul(symbolic::mul(seq_q_, seq_kv_), head_dim_)));
    return f;
}

bool AttentionNode::expand(builder::StructuredSDFGBuilder&, analysis::AnalysisManager&) { return false; }

nlohmann::json AttentionNodeSerializer::serialize(const data_flow::LibraryNode& library_node) {
    auto& n = static_cast<const AttentionNode&>(library_node);
    serializer::JSONSerializer s;
    nlohmann::json j;
    j["code"] = n.code().value();
    j["batch"] = s.expression(n.batch());
    j["heads"] = s.expression(n.heads());
    j["seq_q"] = s.expression(n.seq_q());
    j["seq_kv"] = s.expression(n.seq_kv());
    j["head_dim"] = s.expression(n.head_dim());
    j["scale"] = n.scale();
    j["causal"] = n.causal();
    return j;
}

data_flow::LibraryNode& AttentionNodeSerializer::deserialize(const nlohmann::json& j, builder::StructuredSDFGBuilder& builder,
                                                             structured_control_flow::Block& parent) {
    assert(j.contains("element_id"));
    assert(j.contains("code"));
    assert(j.contains("debug_info"));
    if (j["code"].get<std::string>() != LibraryNodeType_Attention.value()) throw std::runtime_error("Invalid library node code");
    serializer::JSONSerializer s;
    DebugInfo debug_info = s.json_to_debug_info(j["debug_info"]);
    auto& node = builder.add_library_node<AttentionNode>(
        parent, debug_info, symbolic::parse(j.at("batch").get<std::string>()), symbolic::parse(j.at("heads").get<std::string>()),
        symbolic::parse(j.at("seq_q").get<std::string>()), symbolic::parse(j.at("seq_kv").get<std::string>()),
        symbolic::parse(j.at("head_dim").get<std::string>()), j.at("scale").get<double>(), j.at("causal").get<bool>());
    if (j.contains("implementation_type")) node.implementation_type() = data_flow::ImplementationType(j["implementation_type"].get<std::string>());
    return node;
}

// ---- LayerNormNode -------------------------------------------------------------------------------------
static std::vector<std::string> layernorm_inputs(bool affine) {
    return affine ? std::vector<std::string>{"X", "G", "B"} : std::vector<std::string>{"X"};
}

LayerNormNode::LayerNormNode(size_t element_id, const DebugInfo& debug_info, const graph::Vertex vertex,
                             data_flow::DataFlowGraph& parent, const std::vector<symbolic::Expression>& shape, double eps, bool affine)
    : math::tensor::TensorNode(element_id, debug_info, vertex, parent, LibraryNodeType_LayerNorm, {"Y"}, layernorm_inputs(affine),
                               data_flow::ImplementationType_NONE),
      shape_(shape), eps_(eps), affine_(affine) {
    if (shape.empty()) throw InvalidSDFGException("LayerNormNode: empty shape");
}

symbolic::Expression LayerNormNode::rows() const {
    symbolic::Expression r = symbolic::one();
    for (size_t i = 0; i + 1 < shape_.size(); i++) r = symbolic::mul(r, shape_[i]);
    return r;
}

void LayerNormNode::validate(const Function& function) const {
    // G and B are fp32 whatever X is, so the one-primitive-type rule of TensorNode::validate does not apply here
    auto& graph = this->get_parent();
    if (graph.in_degree(*this) != (affine_ ? 3u : 1u) || graph.out_degree(*this) != 1)
        throw InvalidSDFGException("LayerNormNode: expects X" + std::string(affine_ ? ", G, B" : "") + " and the output Y");
    for (auto& edge : graph.in_edges(*this)) {
        if (edge.dst_conn() != "X") continue;
        auto& t = static_cast<const types::Tensor&>(edge.base_type());
        if (t.shape().size() != shape_.size()) throw InvalidSDFGException("LayerNormNode: rank of X does not match the node");
        for (size_t i = 0; i < shape_.size(); i++)
            if (!symbolic::eq(t.shape().at(i), shape_.at(i))) throw InvalidSDFGException("LayerNormNode: shape of X does not match the node");
    }
}

symbolic::SymbolSet LayerNormNode::symbols() const {
    symbolic::SymbolSet syms;
    for (auto& d : shape_) add_atoms(syms, d);
    return syms;
}

void LayerNormNode::replace(const symbolic::Expression old_expression, const symbolic::Expression new_expression) {
    for (auto& d : shape_) d = symbolic::subs(d, old_expression, new_expression);
}

std::unique_ptr<data_flow::DataFlowNode> LayerNormNode::clone(size_t element_id, const graph::Vertex vertex,
                                                              data_flow::DataFlowGraph& parent) const {
    auto node = std::unique_ptr<LayerNormNode>(new LayerNormNode(element_id, this->debug_info(), vertex, parent, shape_, eps_, affine_));
    node->implementation_type() = this->implementation_type();
    return node;
}

std::string LayerNormNode::toStr() const {
    std::string s = LibraryNode::toStr() + "([";
    for (size_t i = 0; i < shape_.size(); i++) s += (i ? ", " : "") + shape_[i]->__str__();
    return s + "], eps=" + std::to_string(eps_) + (affine_ ? ", affine)" : ")");
}

bool LayerNormNode::expand(builder::StructuredSDFGBuilder&, analysis::AnalysisManager&) { return false; }

nlohmann::json LayerNormNodeSerializer::serialize(const data_flow::LibraryNode& library_node) {
    auto& n = static_cast<const LayerNormNode&>(library_node);
    serializer::JSONSerializer s;
    nlohmann::json j;
    j["code"] = n.code().value();
    j["shape"] = nlohmann::json::array();
    for (auto& d : n.shape()) j["shape"].push_back(s.expression(d));
    j["eps"] = n.eps();
    j["affine"] = n.affine();
    return j;
}

data_flow::LibraryNode& LayerNormNodeSerializer::deserialize(const nlohmann::json& j, builder::StructuredSDFGBuilder& builder,
                                                             structured_control_flow::Block& parent) {
    assert(j.contains("element_id"));
    assert(j.contains("code"));
    assert(j.contains("debug_info"));
    assert(j.contains("shape"));
    if (j["code"].get<std::string>() != LibraryNodeType_LayerNorm.value()) throw std::runtime_error("Invalid library node code");
    std::vector<symbolic::Expression> shape;
    for (const auto& d : j["shape"]) shape.push_back(symbolic::parse(d.get<std::string>()));
    serializer::JSONSerializer s;
    DebugInfo debug_info = s.json_to_debug_info(j["debug_info"]);
    auto& node = builder.add_library_node<LayerNormNode>(parent, debug_info, shape, j.at("eps").get<double>(), j.at("affine").get<bool>());
    if (j.contains("implementation_type")) node.implementation_type() = data_flow::ImplementationType(j["implementation_type"].get<std::string>());
    return node;
}

}  // namespace docc::target::b200
