#include "b200_map_dispatcher.h"

#include <algorithm>
#include <map>

#include <sdfg/analysis/arguments_analysis.h>
#include <sdfg/analysis/assumptions_analysis.h>
#include <sdfg/analysis/flop_analysis.h>
#include <sdfg/analysis/loop_analysis.h>
#include <sdfg/builder/structured_sdfg_builder.h>
#include <sdfg/codegen/dispatchers/sequence_dispatcher.h>
#include <sdfg/codegen/language_extensions/cuda_language_extension.h>
#include <sdfg/data_flow/access_node.h>
#include <sdfg/data_flow/library_node.h>
#include <sdfg/exceptions.h>
#include <sdfg/structured_control_flow/block.h>
#include <sdfg/targets/cuda/cuda.h>
#include <sdfg/types/pointer.h>
#include <sdfg/types/scalar.h>

#include "b200_plugin.h"

namespace docc::target::b200 {

using namespace sdfg;
using docc_b200_plugin::ElementwiseMap;
using docc_b200_plugin::MapOperand;

namespace {

// Pointer to a scalar element type: the only array form the vector kernel handles.
const types::Scalar* element_type_of(const types::IType& type) {
    auto pointer = dynamic_cast<const types::Pointer*>(&type);
    if (!pointer || !pointer->has_pointee_type()) return nullptr;
    return dynamic_cast<const types::Scalar*>(&pointer->pointee_type());
}

}  // namespace

bool recognise_elementwise_map(StructuredSDFG& sdfg, analysis::AnalysisManager& analysis_manager,
                               structured_control_flow::Map& map, codegen::LanguageExtension& language_extension,
                               ElementwiseMap* out) {
    // a loop 0 <= i < bound with unit stride (the form CUDAMapDispatcher requires as well: cuda_map_dispatcher.cpp:419-434)
    if (!symbolic::eq(map.init(), symbolic::zero())) return false;
    auto stride = analysis::LoopAnalysis::stride(&map);
    if (stride.is_null() || !symbolic::eq(stride, symbolic::one())) return false;
    auto& assumptions = analysis_manager.get<analysis::AssumptionsAnalysis>();
    auto bound = analysis::LoopAnalysis::canonical_bound(&map, assumptions);
    if (bound.is_null()) return false;

    const auto indvar = map.indvar();
    std::map<std::string, bool> read, written;  // array containers by name

    // the body: blocks of tasklets, nothing between them
    auto& root = map.root();
    for (size_t c = 0; c < root.size(); c++) {
        auto child = root.at(c);
        if (!child.second.assignments().empty()) return false;
        auto block = dynamic_cast<structured_control_flow::Block*>(&child.first);
        if (!block) return false;  // nested loops, branches, returns: the CUDA dispatcher's business
        auto& graph = block->dataflow();
        if (!graph.library_nodes().empty()) return false;
        for (auto& memlet : graph.edges()) {
            const data_flow::AccessNode* access = dynamic_cast<const data_flow::AccessNode*>(&memlet.src());
            const bool is_read = access != nullptr;
            if (!access) access = dynamic_cast<const data_flow::AccessNode*>(&memlet.dst());
            if (!access) return false;  // tasklet-to-tasklet edges do not exist in docc's graphs
            if (dynamic_cast<const data_flow::ConstantNode*>(access)) continue;
            const std::string& name = access->data();
            if (name == indvar->get_name()) return false;  // the induction variable as a value: lanes are not indices
            auto& type = sdfg.type(name);
            if (type.type_id() == types::TypeID::Scalar) {
                if (!memlet.subset().empty()) return false;
                continue;
            }
            if (!element_type_of(type)) return false;
            auto& subset = memlet.subset();
            if (subset.size() != 1 || !symbolic::eq(subset[0], indvar)) return false;  // exactly container[indvar]
            (is_read ? read : written)[name] = true;
        }
    }
    if (written.empty()) return false;
    if (!out) return true;

    // operands in name order; a container that is read and written is an in-place output
    auto operand = [&](const std::string& name, bool also_read) {
        auto scalar = element_type_of(sdfg.type(name));
        MapOperand o;
        o.name = name;
        o.ctype = language_extension.primitive_type(scalar->primitive_type());
        o.bytes = static_cast<int>(types::bit_width(scalar->primitive_type()) / 8);
        o.also_read = also_read;
        return o;
    };
    for (auto& [name, _] : read)
        if (!written.count(name)) out->inputs.push_back(operand(name, false));
    for (auto& [name, _] : written) out->outputs.push_back(operand(name, read.count(name) > 0));

    // scalars the body reads from outside: the kernel's by-value arguments (cuda_map_dispatcher.cpp:66-84)
    auto& arguments_analysis = analysis_manager.get<analysis::ArgumentsAnalysis>();
    std::vector<std::string> scalars;
    for (auto& argument : arguments_analysis.arguments(analysis_manager, map)) {
        auto& type = sdfg.type(argument.first);
        if (type.storage_type().is_nv_symbol()) continue;
        if (type.type_id() == types::TypeID::Scalar) scalars.push_back(argument.first);
    }
    std::sort(scalars.begin(), scalars.end());
    for (auto& name : scalars) {
        auto& scalar = static_cast<const types::Scalar&>(sdfg.type(name));
        out->scalars.push_back({name, language_extension.primitive_type(scalar.primitive_type()),
                                static_cast<int>(types::bit_width(scalar.primitive_type()) / 8)});
    }
    out->count = language_extension.expression(bound);
    out->indvar = indvar->get_name();
    out->kernel_name = "kernel_" + sdfg.name() + "_" + std::to_string(map.element_id());
    return true;
}

// ---- scheduler ----

passes::scheduler::SchedulerAction B200Scheduler::schedule(builder::StructuredSDFGBuilder& builder,
                                                           analysis::AnalysisManager& analysis_manager,
                                                           structured_control_flow::StructuredLoop& loop,
                                                           bool offload_unknown_sizes) {
    auto action = cuda_.schedule(builder, analysis_manager, loop, offload_unknown_sizes);
    // CUDATransform keeps the map node and moves its accesses to the device containers; what it offloaded carries the
    // CUDA schedule type now. Flat element-wise maps among those go to the B200 dispatcher.
    if (auto map = dynamic_cast<structured_control_flow::Map*>(&loop)) {
        if (map->schedule_type().value() == cuda::ScheduleType_CUDA::value()) {
            codegen::CUDALanguageExtension language_extension(builder.subject());
            if (recognise_elementwise_map(builder.subject(), analysis_manager, *map, language_extension, nullptr)) {
                builder.update_schedule_type(*map, ScheduleType_B200::create());
                analysis_manager.invalidate_all();
            }
        }
    }
    return action;
}

passes::scheduler::SchedulerAction B200Scheduler::schedule(builder::StructuredSDFGBuilder& builder,
                                                           analysis::AnalysisManager& analysis_manager,
                                                           structured_control_flow::While& loop, bool offload_unknown_sizes) {
    return cuda_.schedule(builder, analysis_manager, loop, offload_unknown_sizes);
}

std::unordered_set<structured_control_flow::ScheduleTypeCategory> B200Scheduler::compatible_types() {
    return {structured_control_flow::ScheduleTypeCategory::None};
}

void B200Scheduler::set_report(PassReportConsumer* report) {
    report_ = report;
    cuda_.set_report(report);
}

// ---- dispatcher ----

B200MapDispatcher::B200MapDispatcher(codegen::LanguageExtension& language_extension, StructuredSDFG& sdfg,
                                     analysis::AnalysisManager& analysis_manager, structured_control_flow::Map& node,
                                     codegen::InstrumentationPlan& instrumentation_plan, codegen::ArgCapturePlan& arg_capture_plan)
    : codegen::NodeDispatcher(language_extension, sdfg, analysis_manager, node, instrumentation_plan, arg_capture_plan), node_(node) {}

void B200MapDispatcher::dispatch_node(codegen::PrettyPrinter& main_stream, codegen::PrettyPrinter& globals_stream,
                                      codegen::CodeSnippetFactory& library_snippet_factory) {
    analysis::AnalysisManager analysis_manager(sdfg_);
    codegen::CUDALanguageExtension cuda_language_extension(sdfg_);
    ElementwiseMap map;
    if (!recognise_elementwise_map(sdfg_, analysis_manager, node_, cuda_language_extension, &map)) {
        // the scheduler only tags maps this function accepts; a graph edited afterwards has to be scheduled again
        throw InvalidSDFGException("B200 map " + std::to_string(node_.element_id()) + " is not a flat element-wise map");
    }

    // Body: docc's own text for the blocks, `container[i]` accesses and all, behind the declarations of the
    // tasklet-local scalars (the CUDA dispatcher declares them at the top of its kernel: cuda_map_dispatcher.cpp:186-199).
    codegen::PrettyPrinter body(12);
    body << "{" << std::endl;
    auto& arguments_analysis = analysis_manager.get<analysis::ArgumentsAnalysis>();
    std::vector<std::string> locals(arguments_analysis.locals(analysis_manager, node_).begin(),
                                    arguments_analysis.locals(analysis_manager, node_).end());
    std::sort(locals.begin(), locals.end());
    for (auto& local : locals) {
        if (local == node_.indvar()->get_name()) continue;
        std::string declaration = cuda_language_extension.declaration(local, sdfg_.type(local), false, true);
        if (!declaration.empty()) body << declaration << ";" << std::endl;
    }
    codegen::SequenceDispatcher sequence(cuda_language_extension, sdfg_, analysis_manager_, node_.root(), instrumentation_plan_,
                                         arg_capture_plan_);
    sequence.dispatch(body, body, library_snippet_factory);
    body << "}";
    map.body = body.str();

    // kernel + launcher into their own .cu snippet, the launcher's declaration into the host file, the call in place
    auto& library_stream = library_snippet_factory.require(map.kernel_name, "cu", true).stream();
    library_stream << "#include <cuda_runtime.h>" << std::endl << "#include <docc_b200/rt.h>" << std::endl;
    library_stream << "#include " << library_snippet_factory.header_path().filename() << std::endl << std::endl;
    std::ostringstream kernel_text;
    docc_b200_plugin::emit_map_kernel(kernel_text, map);
    docc_b200_plugin::emit_map_launcher(kernel_text, map);
    library_stream << kernel_text.str();

    std::ostringstream declaration_text;
    docc_b200_plugin::emit_map_launcher_declaration(declaration_text, map);
    globals_stream << declaration_text.str();

    std::vector<std::string> device_pointers;
    for (auto& o : map.inputs) device_pointers.push_back(o.name);
    for (auto& o : map.outputs) device_pointers.push_back(o.name);
    std::ostringstream call_text;
    docc_b200_plugin::emit_map_call(call_text, map, device_pointers);
    main_stream << call_text.str();
    // asynchronous like the library-node calls; with instrumentation on, the region has to cover the kernel
    if (instrumentation_plan_.should_instrument(node_)) main_stream << "docc_b200_sync();" << std::endl;
}

codegen::InstrumentationInfo B200MapDispatcher::instrumentation_info() const {
    auto& loop_analysis = analysis_manager_.get<analysis::LoopAnalysis>();
    analysis::LoopInfo loop_info = loop_analysis.loop_info(&node_);
    std::unordered_map<std::string, std::string> metrics;
    auto& flop_analysis = analysis_manager_.get<analysis::FlopAnalysis>();
    auto flop = flop_analysis.get_if_available_for_codegen(&node_);
    if (!flop.is_null()) metrics.insert({"flop", language_extension_.expression(flop)});
    return codegen::InstrumentationInfo(node_.element_id(), codegen::ElementType_Map, TargetType_B200, loop_info, metrics);
}

}  // namespace docc::target::b200
