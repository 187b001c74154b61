// B200 target plugin for docc (see b200_plugin.h). Not part of the runtime library: this file is
// compiled inside a docc tree. The text of every emitted call comes from b200_emit.h.
#include "b200_plugin.h"

#include <sdfg/passes/targets/target_mapping_pass.h>

#include "b200_emit.h"

namespace docc::target::b200 {

using namespace sdfg;
namespace emit = docc_b200_plugin;

static std::filesystem::path B200_ROOT = "/opt/docc_b200";  // installation prefix of this package

bool B200LibNodeMapper::try_map(builder::StructuredSDFGBuilder&, analysis::AnalysisManager&,
                                data_flow::LibraryNode& node) const {
    const auto& code = node.code().value();
    const bool gemm = code == math::blas::LibraryNodeType_GEMM.value();
    const bool tensor = code == math::tensor::LibraryNodeType_MatMul.value() ||
                        code == math::tensor::LibraryNodeType_Softmax.value() ||
                        code == math::tensor::LibraryNodeType_Conv.value();
    if (!gemm && !tensor) return false;
    if (gemm) {
        auto& g = static_cast<math::blas::GEMMNode&>(node);
        auto prim = g.scalar_primitive();
        if (prim != types::PrimitiveType::Double && prim != types::PrimitiveType::Float && prim != types::PrimitiveType::Half)
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
    return codegen::InstrumentationInfo(node_.element_id(), codegen::ElementType_LibraryNode, TargetType_B200,
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
    return codegen::InstrumentationInfo(node_.element_id(), codegen::ElementType_LibraryNode, TargetType_B200,
                                        analysis::LoopInfo{}, {});
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
    symbolic::Expression bytes = symbolic::integer(2 * types::get_type_size(types::Scalar(n.primitive_type(data_flow_graph_)), false));
    for (auto& d : n.shape()) bytes = symbolic::mul(bytes, d);
    return codegen::InstrumentationInfo(node_.element_id(), codegen::ElementType_LibraryNode, TargetType_B200,
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
    return codegen::InstrumentationInfo(node_.element_id(), codegen::ElementType_LibraryNode, TargetType_B200,
                                        analysis::LoopInfo{}, {});
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
    reg.register_library_node_dispatcher(math::blas::LibraryNodeType_GEMM.value() + wt, make_factory<GEMMNodeDispatcher_B200>(true));
    reg.register_library_node_dispatcher(math::blas::LibraryNodeType_GEMM.value() + wo, make_factory<GEMMNodeDispatcher_B200>(false));
    reg.register_library_node_dispatcher(math::tensor::LibraryNodeType_MatMul.value() + wt, make_factory<MatMulNodeDispatcher_B200>(true));
    reg.register_library_node_dispatcher(math::tensor::LibraryNodeType_MatMul.value() + wo, make_factory<MatMulNodeDispatcher_B200>(false));
    reg.register_library_node_dispatcher(math::tensor::LibraryNodeType_Softmax.value() + wt, make_factory<SoftmaxNodeDispatcher_B200>(true));
    reg.register_library_node_dispatcher(math::tensor::LibraryNodeType_Softmax.value() + wo, make_factory<SoftmaxNodeDispatcher_B200>(false));
    reg.register_library_node_dispatcher(math::tensor::LibraryNodeType_Conv.value() + wt, make_factory<ConvNodeDispatcher_B200>(true));
    reg.register_library_node_dispatcher(math::tensor::LibraryNodeType_Conv.value() + wo, make_factory<ConvNodeDispatcher_B200>(false));
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
