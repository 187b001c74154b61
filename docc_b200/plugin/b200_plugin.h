// B200 target plugin for docc: implementation types, target mapper, dispatchers, registration.
// Builds inside a docc source tree (needs sdfg/ and opt/ headers); shape follows targets/et
// (targets/et/include/docc/target/et/target.h, targets/et/src/et/target.cpp:21-58).
#pragma once

#include <sdfg/codegen/dispatchers/block_dispatcher.h>
#include <sdfg/codegen/dispatchers/node_dispatcher_registry.h>
#include <sdfg/codegen/instrumentation/instrumentation_info.h>
#include <sdfg/data_flow/library_nodes/math/blas/gemm_node.h>
#include <sdfg/data_flow/library_nodes/math/tensor/conv_node.h>
#include <sdfg/data_flow/library_nodes/math/tensor/elementwise_node.h>
#include <sdfg/data_flow/library_nodes/math/tensor/matmul_node.h>
#include <sdfg/data_flow/library_nodes/math/tensor/reduce_node.h>
#include <sdfg/data_flow/library_nodes/math/tensor/reduce_ops/softmax_node.h>
#include <sdfg/plugins/plugins.h>
#include <sdfg/plugins/target_mapping.h>

#include "b200_nodes.h"

namespace docc::target::b200 {

// Free strings (library_node.h:73,82); distinct from the cuBLAS keys in opt/include/sdfg/targets/cuda/cuda.h:20-26.
inline sdfg::data_flow::ImplementationType ImplementationType_B200WithTransfers{"B200WithTransfers"};
inline sdfg::data_flow::ImplementationType ImplementationType_B200WithoutTransfers{"B200WithoutTransfers"};
// Transfer / allocation nodes (code "CUDAOffloading", cuda_data_offloading_node.h:19) routed to the runtime's pool:
// the CUDA plugin owns the key "CUDAOffloading::" + NONE (plugin.h:35-45, first registration wins), so the mapper
// moves the nodes of a B200-scheduled SDFG to this implementation type and the plugin registers "CUDAOffloading::B200".
inline sdfg::data_flow::ImplementationType ImplementationType_B200{"B200"};
// Target name in instrumentation records (the CUDA target uses its schedule-type name, cuda.h:48).
inline sdfg::codegen::TargetType TargetType_B200{"B200"};

// Replaces CudaLibraryNodeRewriter (opt/src/passes/offloading/cuda_library_node_rewriter_pass.cpp:12-54).
// Must run before ExpansionPass: nodes whose implementation type is not NONE are not expanded
// (sdfg/src/passes/dataflow/expansion_pass.cpp:16-18).
class B200LibNodeMapper : public sdfg::plugins::TargetMapper {
public:
    bool try_map(sdfg::builder::StructuredSDFGBuilder& builder, sdfg::analysis::AnalysisManager& analysis_manager,
                 sdfg::data_flow::LibraryNode& node) const override;
};

class B200Dispatcher : public sdfg::codegen::LibraryNodeDispatcher {
public:
    B200Dispatcher(sdfg::codegen::LanguageExtension& language_extension, const sdfg::Function& function,
                   const sdfg::data_flow::DataFlowGraph& data_flow_graph, const sdfg::data_flow::LibraryNode& node,
                   bool with_transfers)
        : LibraryNodeDispatcher(language_extension, function, data_flow_graph, node), with_transfers_(with_transfers) {}

protected:
    std::string expr(const sdfg::symbolic::Expression& e) { return language_extension_.expression(e); }
    std::vector<std::string> exprs(const std::vector<sdfg::symbolic::Expression>& v) {
        std::vector<std::string> out;
        for (auto& e : v) out.push_back(expr(e));
        return out;
    }
    bool with_transfers_;
};

#define DOCC_B200_DECLARE_DISPATCHER(Name)                                                                              \
    class Name : public B200Dispatcher {                                                                                \
    public:                                                                                                             \
        using B200Dispatcher::B200Dispatcher;                                                                           \
        void dispatch_code(sdfg::codegen::PrettyPrinter& stream, sdfg::codegen::PrettyPrinter& globals_stream,          \
                           sdfg::codegen::CodeSnippetFactory& library_snippet_factory) override;                        \
        sdfg::codegen::InstrumentationInfo instrumentation_info() const override;                                       \
    }

DOCC_B200_DECLARE_DISPATCHER(GEMMNodeDispatcher_B200);
DOCC_B200_DECLARE_DISPATCHER(MatMulNodeDispatcher_B200);
DOCC_B200_DECLARE_DISPATCHER(SoftmaxNodeDispatcher_B200);
DOCC_B200_DECLARE_DISPATCHER(ConvNodeDispatcher_B200);
DOCC_B200_DECLARE_DISPATCHER(ReduceNodeDispatcher_B200);       // ml::Sum / Max / Min / Mean / Std
DOCC_B200_DECLARE_DISPATCHER(UnaryNodeDispatcher_B200);        // ml::Exp / Erf / Tanh / Sqrt / Sigmoid / ReLU / Abs
DOCC_B200_DECLARE_DISPATCHER(BinaryNodeDispatcher_B200);       // ml::Add / Sub / Mul / Div / Maximum / Minimum
DOCC_B200_DECLARE_DISPATCHER(CastNodeDispatcher_B200);         // ml::Cast
DOCC_B200_DECLARE_DISPATCHER(AttentionNodeDispatcher_B200);    // ml::Attention (b200_nodes.h)
DOCC_B200_DECLARE_DISPATCHER(LayerNormNodeDispatcher_B200);    // ml::LayerNorm (b200_nodes.h)
DOCC_B200_DECLARE_DISPATCHER(OffloadingNodeDispatcher_B200);   // CUDAOffloading::B200

// Node code -> runtime op code tables (DOCC_B200_RED_*, DOCC_B200_ACT_*, DOCC_B200_EW_* of rt.h); -1 = not covered.
int reduce_op_of(const std::string& code);
int unary_act_of(const std::string& code);
int binary_op_of(const std::string& code);

// Called at module import next to register_cuda_plugin() (python/bindings/bindings.cpp:51-60).
void register_plugin(sdfg::plugins::Context& context);

// Hooks of an out-of-tree target (targets/et/src/et/target.cpp:38-58).
void b200_scheduling_passes(sdfg::builder::StructuredSDFGBuilder& builder, sdfg::analysis::AnalysisManager& analysis_manager,
                            const std::string& category);
std::string b200_get_host_additional_compile_args(const sdfg::StructuredSDFG& sdfg,
                                                  const sdfg::codegen::CodeSnippetFactory& snippet_factory);
std::string b200_get_host_additional_link_args(const sdfg::StructuredSDFG& sdfg,
                                               const sdfg::codegen::CodeSnippetFactory& snippet_factory);

}  // namespace docc::target::b200
