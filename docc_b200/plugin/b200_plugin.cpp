// B200 target plugin for docc (see b200_plugin.h). Not part of the runtime library: this file is
// compiled inside a docc tree. The text of every emitted call comes from b200_emit.h.
#include "b200_plugin.h"

#include <sdfg/passes/targets/target_mapping_pass.h>
#include <sdfg/targets/offloading/data_offloading_node.h>
#include <sdfg/types/utils.h>

#include "b200_emit.h"
#include "b200_map_dispatcher.h"

namespace docc::target::b200 {

using namespace sdfg;
namespace emit = docc_b200_plugin;

static std::filesystem::path B200_ROOT = "/opt/docc_b200";  // installation prefix of this package

int reduce_op_of(const std::string& code) {
    if (code == "ml::Sum") return 0;
    if (code == "ml::Max") return 1;
    if (code == "ml::Min") return 2;
    if (code == "ml::Mean") return 3;
    if (code == "ml::Std") return 4;
    return -1;
}
int unary_act_of(const std::string& code) {
    if (code == "ml::ReLU") return 2;
    if (code == "ml::Tanh") return 3;
    if (code == "ml::Sigmoid") return 4;
    if (code == "ml::Exp") return 5;
    if (code == "ml::Erf") return 6;
    if (code == "ml::Sqrt") return 7;
    if (code == "ml::Abs") return 8;
    return -1;
}
int binary_op_of(const std::string& code) {
    if (code == "ml::Add") return 0;
    if (code == "ml::Sub") return 1;
    if (code == "ml::Mul") return 2;
    if (code == "ml::Div") return 3;
    if (code == "ml::Maximum") return 4;
    if (code == "ml::Minimum") return 5;
    return -1;
}

static bool float_type(types::PrimitiveType t) {
    return t == types::PrimitiveType::Double || t == types::PrimitiveType::Float || t == types::PrimitiveType::Half ||
           t == types::PrimitiveType::BFloat;
}

// The batched matmul entry takes one leading dimension and one batch stride per operand, with unit stride along the
// last dimension: views whose strides say otherwise stay with docc's own expansion (matmul_node.cpp:194-269 copies them).
static bool matmul_is_plain(const math::tensor::MatMulNode& n) {
    auto plain = [](const symbolic::MultiExpression& shape, const symbolic::MultiExpression& strides) {
        if (strides.empty()) return true;
        symbolic::Expression expect = symbolic::one();
        for (size_t i = shape.size(); i-- > 0;) {
            if (!symbolic::eq(strides[i], expect)) return false;
            expect = symbolic::mul(expect, shape[i]);
        }
        return true;
    };
    return plain(n.shape_a(), n.strides_a()) && plain(n.shape_b(), n.strides_b()) && symbolic::eq(n.offset_a(), symbolic::zero()) &&
           symbolic::eq(n.offset_b(), symbolic::zero());
}

bool B200LibNodeMapper::try_map(builder::StructuredSDFGBuilder&, analysis::AnalysisManager&,
                                data_flow::LibraryNode& node) const {
    const auto& code = node.code().value();
    // transfer / allocation nodes of an offloaded region: same node, runtime pool behind it
    if (code == "CUDAOffloading") {
        node.implementation_type() = ImplementationType_B200;
        return true;
    }
    if (code == math::blas::LibraryNodeType_GEMM.value()) {
        auto& g = static_cast<math::blas::GEMMNode&>(node);
        if (!float_type(g.scalar_primitive())) return false;
    } else if (code == math::tensor::LibraryNodeType_MatMul.value()) {
        auto& m = static_cast<math::tensor::MatMulNode&>(node);
        if (!matmul_is_plain(m) || !float_type(m.primitive_type(node.get_parent()))) return false;
    } else if (code == math::tensor::LibraryNodeType_Softmax.value() || code == math::tensor::LibraryNodeType_Conv.value() ||
               reduce_op_of(code) >= 0 || unary_act_of(code) >= 0 || binary_op_of(code) >= 0 || code == "ml::Cast" ||
               code == LibraryNodeType_Attention.value()) {
        auto& t = static_cast<math::tensor::TensorNode&>(node);
        if (code != "ml::Cast" && !float_type(t.primitive_type(node.get_parent()))) return false;  // integer tensors: docc's expansion
    } else if (code != LibraryNodeType_LayerNorm.value()) {
        return false;
    }
    node.implementation_type() = ImplementationType_B200WithTransfers;
    return true;
}

static char precision_char(math::blas::BLAS_Precision p) { return static_cast<char>(p); }

static char precision_of(types::PrimitiveType t) {
    switch (t) {
        case types::PrimitiveType::Double: return 'd';
        case types::PrimitiveType::Float: return 's';
        case types::PrimitiveType::Half: return 'h';
        case types::PrimitiveType::BFloat: return 'b';
        default: throw InvalidSDFGException("B200 target: unsupported element type");
    }
}

void GEMMNodeDispatcher_B200::dispatch_code(codegen::PrettyPrinter& stream, codegen::PrettyPrinter& globals_stream,
                                            codegen::CodeSnippetFactory&) {
    auto& n = static_cast<const math::blas::GEMMNode&>(node_);
    emit::emit_include(globals_stream);
    emit::emit_gemm(stream, precision_char(n.precision()), static_cast<int>(n.layout()), static_cast<int>(n.trans_a()),
                    static_cast<int>(n.trans_b()), expr(n.m()), expr(n.n()), expr(n.k()), expr(n.lda()), expr(n.ldb()),
                    expr(n.ldc()), with_transfers_, emit::debug_checks_enabled());
}
codegen::InstrumentationInfo GEMMNodeDispatcher_B200::instrumentation_info() const {
    auto& n = static_cast<const math::blas::GEMMNode&>(node_);
    return codegen::InstrumentationInfo(node_.element_id(), codegen::ElementType_Math, TargetType_B200,
                                        analysis::LoopInfo{}, {{"flop", language_extension_.expression(n.flop())}});
}

void MatMulNodeDispatcher_B200::dispatch_code(codegen::PrettyPrinter& stream, codegen::PrettyPrinter& globals_stream,
                                              codegen::CodeSnippetFactory&) {
    auto& n = static_cast<const math::tensor::MatMulNode&>(node_);
    emit::emit_include(globals_stream);
    const auto& sa = n.shape_a();
    const auto& sb = n.shape_b();
    symbolic::Expression batch = symbolic::one();
    for (size_t i = 0; i + 2 < sa.size(); i++) batch = symbolic::mul(batch, sa[i]);
    const auto m = sa[sa.size() - 2], k = sa[sa.size() - 1], nn = sb[sb.size() - 1];
    const auto stride_a = sa.size() > 2 ? symbolic::mul(m, k) : symbolic::zero();
    const auto stride_b = sb.size() > 2 ? symbolic::mul(k, nn) : symbolic::zero();
    emit::emit_matmul(stream, precision_of(n.primitive_type(data_flow_graph_)), expr(batch), expr(m), expr(nn), expr(k), expr(k),
                      expr(stride_a), expr(nn), expr(stride_b), with_transfers_, emit::debug_checks_enabled());
}
codegen::InstrumentationInfo MatMulNodeDispatcher_B200::instrumentation_info() const {
    // 2 * batch * m * n * k, the count GEMMNode::flop gives per batch item (gemm_node.cpp:333-356) without the
    // alpha / beta terms (MatMulNode wraps GEMM with alpha = 1, beta = 0, matmul_node.cpp:463-489)
    auto& n = static_cast<const math::tensor::MatMulNode&>(node_);
    const auto& sa = n.shape_a();
    symbolic::Expression flop = symbolic::mul(symbolic::integer(2), symbolic::mul(symbolic::mul(n.m(), n.n()), n.k()));
    for (size_t i = 0; i + 2 < sa.size(); i++) flop = symbolic::mul(flop, sa[i]);
    return codegen::InstrumentationInfo(node_.element_id(), codegen::ElementType_Math, TargetType_B200,
                                        analysis::LoopInfo{}, {{"flop", language_extension_.expression(flop)}});
}

void SoftmaxNodeDispatcher_B200::dispatch_code(codegen::PrettyPrinter& stream, codegen::PrettyPrinter& globals_stream,
                                               codegen::CodeSnippetFactory&) {
    auto& n = static_cast<const math::tensor::SoftmaxNode&>(node_);
    emit::emit_include(globals_stream);
    std::vector<std::string> axes;
    for (auto a : n.axes()) axes.push_back(std::to_string(a));
    emit::emit_softmax(stream, precision_of(n.primitive_type(data_flow_graph_)), exprs(n.shape()), axes, with_transfers_,
                       emit::debug_checks_enabled());
}
codegen::InstrumentationInfo SoftmaxNodeDispatcher_B200::instrumentation_info() const {
    auto& n = static_cast<const math::tensor::SoftmaxNode&>(node_);
    // one read and one write of the tensor; get_type_size is a symbolic expression (types/utils.h:104)
    symbolic::Expression bytes = symbolic::mul(symbolic::integer(2), types::get_type_size(types::Scalar(n.primitive_type(data_flow_graph_)), false));
    for (auto& d : n.shape()) bytes = symbolic::mul(bytes, d);
    return codegen::InstrumentationInfo(node_.element_id(), codegen::ElementType_Math, TargetType_B200,
                                        analysis::LoopInfo{}, {{"hbm_bytes", language_extension_.expression(bytes)}});
}

void ConvNodeDispatcher_B200::dispatch_code(codegen::PrettyPrinter& stream, codegen::PrettyPrinter& globals_stream,
                                            codegen::CodeSnippetFactory&) {
    auto& n = static_cast<const math::tensor::ConvNode&>(node_);
    emit::emit_include(globals_stream);
    std::vector<symbolic::Expression> pads = n.pads_begin();
    pads.insert(pads.end(), n.pads_end().begin(), n.pads_end().end());
    emit::emit_conv(stream, precision_of(n.primitive_type(data_flow_graph_)), exprs(n.shape()), exprs(n.kernel_shape()),
                    exprs(n.strides()), exprs(pads), exprs(n.dilations()), expr(n.output_channels()), expr(n.group()),
                    n.has_bias(), with_transfers_, emit::debug_checks_enabled());
}
codegen::InstrumentationInfo ConvNodeDispatcher_B200::instrumentation_info() const {
    // flop = 2 * N * C_out * prod(out) * (C_in / group) * prod(kernel); hbm_bytes = one pass over X, W and Y.
    // Output extents as ConvNode::expand derives them (conv_node.cpp:225-233).
    auto& n = static_cast<const math::tensor::ConvNode&>(node_);
    const auto& x = n.shape();
    const size_t sr = n.kernel_shape().size();
    symbolic::Expression out = symbolic::mul(x[0], n.output_channels());
    symbolic::Expression taps = symbolic::div(x[1], n.group());
    symbolic::Expression x_elems = symbolic::mul(x[0], x[1]);
    for (size_t i = 0; i < sr; i++) {
        auto pad = symbolic::add(n.pads_begin()[i], n.pads_end()[i]);
        auto dk = symbolic::mul(n.dilations()[i], symbolic::sub(n.kernel_shape()[i], symbolic::one()));
        auto num = symbolic::sub(symbolic::add(x[2 + i], pad), symbolic::add(dk, symbolic::one()));
        out = symbolic::mul(out, symbolic::add(symbolic::div(num, n.strides()[i]), symbolic::one()));
        taps = symbolic::mul(taps, n.kernel_shape()[i]);
        x_elems = symbolic::mul(x_elems, x[2 + i]);
    }
    const auto es = types::get_type_size(types::Scalar(n.primitive_type(data_flow_graph_)), false);
    auto flop = symbolic::mul(symbolic::integer(2), symbolic::mul(out, taps));
    auto bytes = symbolic::mul(es, symbolic::add(symbolic::add(x_elems, symbolic::mul(n.output_channels(), taps)), out));
    return codegen::InstrumentationInfo(node_.element_id(), codegen::ElementType_Math, TargetType_B200, analysis::LoopInfo{},
                                        {{"flop", language_extension_.expression(flop)},
                                         {"hbm_bytes", language_extension_.expression(bytes)}});
}

// ---- reductions, element-wise nodes, cast ----------------------------------------------------------------
static symbolic::Expression product(const std::vector<symbolic::Expression>& shape) {
    symbolic::Expression p = symbolic::one();
    for (auto& d : shape) p = symbolic::mul(p, d);
    return p;
}
static symbolic::Expression tensor_bytes(const std::vector<symbolic::Expression>& shape, types::PrimitiveType t, int tensors) {
    return symbolic::mul(symbolic::mul(symbolic::integer(tensors), types::get_type_size(types::Scalar(t), false)), product(shape));
}

void ReduceNodeDispatcher_B200::dispatch_code(codegen::PrettyPrinter& stream, codegen::PrettyPrinter& globals_stream,
                                              codegen::CodeSnippetFactory&) {
    auto& n = static_cast<const math::tensor::ReduceNode&>(node_);
    emit::emit_include(globals_stream);
    std::vector<std::string> axes;
    for (auto a : n.axes()) axes.push_back(std::to_string(a));
    // keepdims only adds extents of one: the C-order output buffer is the same either way
    emit::emit_reduce(stream, reduce_op_of(n.code().value()), precision_of(n.primitive_type(data_flow_graph_)), exprs(n.shape()), axes,
                      with_transfers_, emit::debug_checks_enabled());
}
codegen::InstrumentationInfo ReduceNodeDispatcher_B200::instrumentation_info() const {
    auto& n = static_cast<const math::tensor::ReduceNode&>(node_);
    return codegen::InstrumentationInfo(
        node_.element_id(), codegen::ElementType_Math, TargetType_B200, analysis::LoopInfo{},
        {{"hbm_bytes", language_extension_.expression(tensor_bytes(n.shape(), n.primitive_type(data_flow_graph_), 1))}});
}

void UnaryNodeDispatcher_B200::dispatch_code(codegen::PrettyPrinter& stream, codegen::PrettyPrinter& globals_stream,
                                             codegen::CodeSnippetFactory&) {
    auto& n = static_cast<const math::tensor::ElementWiseUnaryNode&>(node_);
    emit::emit_include(globals_stream);
    emit::emit_unary(stream, precision_of(n.primitive_type(data_flow_graph_)), unary_act_of(n.code().value()), expr(product(n.shape())),
                     with_transfers_, emit::debug_checks_enabled());
}
codegen::InstrumentationInfo UnaryNodeDispatcher_B200::instrumentation_info() const {
    auto& n = static_cast<const math::tensor::ElementWiseUnaryNode&>(node_);
    return codegen::InstrumentationInfo(
        node_.element_id(), codegen::ElementType_Math, TargetType_B200, analysis::LoopInfo{},
        {{"hbm_bytes", language_extension_.expression(tensor_bytes(n.shape(), n.primitive_type(data_flow_graph_), 2))}});
}

void BinaryNodeDispatcher_B200::dispatch_code(codegen::PrettyPrinter& stream, codegen::PrettyPrinter& globals_stream,
                                              codegen::CodeSnippetFactory&) {
    auto& n = static_cast<const math::tensor::ElementWiseBinaryNode&>(node_);
    emit::emit_include(globals_stream);
    emit::emit_binary(stream, binary_op_of(n.code().value()), precision_of(n.primitive_type(data_flow_graph_)), expr(product(n.shape())),
                      with_transfers_, emit::debug_checks_enabled());
}
codegen::InstrumentationInfo BinaryNodeDispatcher_B200::instrumentation_info() const {
    auto& n = static_cast<const math::tensor::ElementWiseBinaryNode&>(node_);
    return codegen::InstrumentationInfo(
        node_.element_id(), codegen::ElementType_Math, TargetType_B200, analysis::LoopInfo{},
        {{"hbm_bytes", language_extension_.expression(tensor_bytes(n.shape(), n.primitive_type(data_flow_graph_), 3))}});
}

// the element type on one connector (CastNode and LayerNormNode carry more than one type)
static types::PrimitiveType connector_type(const data_flow::DataFlowGraph& graph, const data_flow::LibraryNode& node, const std::string& conn,
                                           bool input) {
    if (input) {
        for (auto& e : graph.in_edges(node))
            if (e.dst_conn() == conn) return static_cast<const types::Tensor&>(e.base_type()).primitive_type();
    } else {
        for (auto& e : graph.out_edges(node))
            if (e.src_conn() == conn) return static_cast<const types::Tensor&>(e.base_type()).primitive_type();
    }
    throw InvalidSDFGException("B200 target: connector " + conn + " is not connected");
}

void CastNodeDispatcher_B200::dispatch_code(codegen::PrettyPrinter& stream, codegen::PrettyPrinter& globals_stream,
                                            codegen::CodeSnippetFactory&) {
    auto& n = static_cast<const math::tensor::ElementWiseUnaryNode&>(node_);
    emit::emit_include(globals_stream);
    emit::emit_cast(stream, precision_of(connector_type(data_flow_graph_, node_, "X", true)),
                    precision_of(connector_type(data_flow_graph_, node_, "Y", false)), expr(product(n.shape())), with_transfers_,
                    emit::debug_checks_enabled());
}
codegen::InstrumentationInfo CastNodeDispatcher_B200::instrumentation_info() const {
    auto& n = static_cast<const math::tensor::ElementWiseUnaryNode&>(node_);
    auto bytes = symbolic::add(tensor_bytes(n.shape(), connector_type(data_flow_graph_, node_, "X", true), 1),
                               tensor_bytes(n.shape(), connector_type(data_flow_graph_, node_, "Y", false), 1));
    return codegen::InstrumentationInfo(node_.element_id(), codegen::ElementType_Math, TargetType_B200, analysis::LoopInfo{},
                                        {{"hbm_bytes", language_extension_.expression(bytes)}});
}

// ---- the nodes this target adds -----------------------------------------------------------------------------
void AttentionNodeDispatcher_B200::dispatch_code(codegen::PrettyPrinter& stream, codegen::PrettyPrinter& globals_stream,
                                                 codegen::CodeSnippetFactory&) {
    auto& n = static_cast<const AttentionNode&>(node_);
    emit::emit_include(globals_stream);
    globals_stream << "#include <math.h>\n";
    emit::emit_attention(stream, precision_of(n.primitive_type(data_flow_graph_)), expr(n.batch()), expr(n.heads()), expr(n.seq_q()),
                         expr(n.seq_kv()), expr(n.head_dim()), n.scale(), n.causal(), with_transfers_, emit::debug_checks_enabled());
}
codegen::InstrumentationInfo AttentionNodeDispatcher_B200::instrumentation_info() const {
    auto& n = static_cast<const AttentionNode&>(node_);
    return codegen::InstrumentationInfo(node_.element_id(), codegen::ElementType_Math, TargetType_B200, analysis::LoopInfo{},
                                        {{"flop", language_extension_.expression(n.flop())}});
}

void LayerNormNodeDispatcher_B200::dispatch_code(codegen::PrettyPrinter& stream, codegen::PrettyPrinter& globals_stream,
                                                 codegen::CodeSnippetFactory&) {
    auto& n = static_cast<const LayerNormNode&>(node_);
    emit::emit_include(globals_stream);
    emit::emit_layernorm(stream, precision_of(connector_type(data_flow_graph_, node_, "X", true)), expr(n.rows()), expr(n.cols()), n.eps(),
                         n.affine(), with_transfers_, emit::debug_checks_enabled());
}
codegen::InstrumentationInfo LayerNormNodeDispatcher_B200::instrumentation_info() const {
    auto& n = static_cast<const LayerNormNode&>(node_);
    return codegen::InstrumentationInfo(
        node_.element_id(), codegen::ElementType_Math, TargetType_B200, analysis::LoopInfo{},
        {{"hbm_bytes", language_extension_.expression(tensor_bytes(n.shape(), connector_type(data_flow_graph_, node_, "X", true), 2))}});
}

// ---- transfers and allocations -----------------------------------------------------------------------------
// Same node, same connector roles and the same order of operations as CUDADataOffloadingNodeDispatcher
// (cuda_data_offloading_node.cpp:139-173): "_ret" or "_dst" is output(0), "_src" or "_ptr" is input(0).
void OffloadingNodeDispatcher_B200::dispatch_code(codegen::PrettyPrinter& stream, codegen::PrettyPrinter& globals_stream,
                                                  codegen::CodeSnippetFactory&) {
    auto& n = static_cast<const sdfg::offloading::DataOffloadingNode&>(node_);
    emit::emit_include(globals_stream);
    const std::string dst = n.outputs().empty() ? std::string() : n.output(0);
    const std::string src = n.inputs().empty() ? std::string() : n.input(0);
    emit::emit_offload(stream, n.is_alloc(), n.is_h2d(), n.is_d2h(), n.is_free(), dst, src, expr(n.size()), emit::debug_checks_enabled());
}
codegen::InstrumentationInfo OffloadingNodeDispatcher_B200::instrumentation_info() const {
    auto& n = static_cast<const sdfg::offloading::DataOffloadingNode&>(node_);
    if (n.is_d2h() || n.is_h2d())
        return codegen::InstrumentationInfo(node_.element_id(), n.is_d2h() ? codegen::ElementType_D2HTransfer : codegen::ElementType_H2DTransfer,
                                            TargetType_B200, analysis::LoopInfo{}, {{"pcie_bytes", language_extension_.expression(n.size())}});
    return codegen::LibraryNodeDispatcher::instrumentation_info();
}

template <class D>
static auto make_factory(bool with_transfers) {
    return [with_transfers](codegen::LanguageExtension& le, const Function& fn, const data_flow::DataFlowGraph& dfg,
                            const data_flow::LibraryNode& node) -> std::unique_ptr<codegen::LibraryNodeDispatcher> {
        return std::make_unique<D>(le, fn, dfg, node, with_transfers);
    };
}

void register_plugin(plugins::Context& context) {
    auto& reg = context.library_node_dispatcher_registry;
    const std::string wt = "::" + ImplementationType_B200WithTransfers.value();
    const std::string wo = "::" + ImplementationType_B200WithoutTransfers.value();
    auto both = [&](const std::string& code, auto with, auto without) {
        reg.register_library_node_dispatcher(code + wt, with);
        reg.register_library_node_dispatcher(code + wo, without);
    };
    both(math::blas::LibraryNodeType_GEMM.value(), make_factory<GEMMNodeDispatcher_B200>(true), make_factory<GEMMNodeDispatcher_B200>(false));
    both(math::tensor::LibraryNodeType_MatMul.value(), make_factory<MatMulNodeDispatcher_B200>(true), make_factory<MatMulNodeDispatcher_B200>(false));
    both(math::tensor::LibraryNodeType_Softmax.value(), make_factory<SoftmaxNodeDispatcher_B200>(true), make_factory<SoftmaxNodeDispatcher_B200>(false));
    both(math::tensor::LibraryNodeType_Conv.value(), make_factory<ConvNodeDispatcher_B200>(true), make_factory<ConvNodeDispatcher_B200>(false));
    for (const char* code : {"ml::Sum", "ml::Max", "ml::Min", "ml::Mean", "ml::Std"})
        both(code, make_factory<ReduceNodeDispatcher_B200>(true), make_factory<ReduceNodeDispatcher_B200>(false));
    for (const char* code : {"ml::Exp", "ml::Erf", "ml::Tanh", "ml::Sqrt", "ml::Sigmoid", "ml::ReLU", "ml::Abs"})
        both(code, make_factory<UnaryNodeDispatcher_B200>(true), make_factory<UnaryNodeDispatcher_B200>(false));
    for (const char* code : {"ml::Add", "ml::Sub", "ml::Mul", "ml::Div", "ml::Maximum", "ml::Minimum"})
        both(code, make_factory<BinaryNodeDispatcher_B200>(true), make_factory<BinaryNodeDispatcher_B200>(false));
    both("ml::Cast", make_factory<CastNodeDispatcher_B200>(true), make_factory<CastNodeDispatcher_B200>(false));
    both(LibraryNodeType_Attention.value(), make_factory<AttentionNodeDispatcher_B200>(true), make_factory<AttentionNodeDispatcher_B200>(false));
    both(LibraryNodeType_LayerNorm.value(), make_factory<LayerNormNodeDispatcher_B200>(true), make_factory<LayerNormNodeDispatcher_B200>(false));
    // transfers / allocations: the CUDA offloading node (its serializer is registered by the CUDA plugin, plugin.h:47-52)
    reg.register_library_node_dispatcher("CUDAOffloading::" + ImplementationType_B200.value(), make_factory<OffloadingNodeDispatcher_B200>(false));

    // leftover element-wise maps: dispatcher by schedule type, scheduler by target name, as register_cuda_plugin() does for
    // "CUDA" / "cuda" (opt/include/sdfg/targets/cuda/plugin.h:21-34,119-120)
    context.map_dispatcher_registry.register_map_dispatcher(
        ScheduleType_B200::value(),
        [](codegen::LanguageExtension& language_extension, StructuredSDFG& sdfg, analysis::AnalysisManager& analysis_manager,
           structured_control_flow::Map& node, codegen::InstrumentationPlan& instrumentation_plan,
           codegen::ArgCapturePlan& arg_capture_plan) {
            return std::make_unique<B200MapDispatcher>(language_extension, sdfg, analysis_manager, node, instrumentation_plan,
                                                       arg_capture_plan);
        });
    context.scheduler_registry.register_loop_scheduler<B200Scheduler>(B200Scheduler::target());

    // serializers of the two new nodes, so that dumps (python_program.py:283,301) round-trip
    auto& ser = context.library_node_serializer_registry;
    ser.register_library_node_serializer(LibraryNodeType_Attention.value(), []() { return std::make_unique<AttentionNodeSerializer>(); });
    ser.register_library_node_serializer(LibraryNodeType_LayerNorm.value(), []() { return std::make_unique<LayerNormNodeSerializer>(); });
}

void b200_scheduling_passes(builder::StructuredSDFGBuilder& builder, analysis::AnalysisManager& analysis_manager,
                            const std::string&) {
    std::vector<std::shared_ptr<plugins::TargetMapper>> mappers{std::make_shared<B200LibNodeMapper>()};
    passes::TargetMappingPass mapping(mappers);
    mapping.run_pass(builder, analysis_manager);
}

std::string b200_get_host_additional_compile_args(const StructuredSDFG&, const codegen::CodeSnippetFactory&) {
    return "-I" + (B200_ROOT / "include").string();
}

std::string b200_get_host_additional_link_args(const StructuredSDFG&, const codegen::CodeSnippetFactory&) {
    const auto lib = (B200_ROOT / "docc_b200" / "lib").string();
    return "-L" + lib + " -Wl,-rpath," + lib + " -ldocc_b200_rt";
}

}  // namespace docc::target::b200
