// Generic-map side of the B200 target for docc: schedule type, loop scheduler and map dispatcher.
// Builds inside a docc source tree (needs sdfg/ and opt/ headers), next to b200_plugin.cpp.
//
// What the CUDA target does with a leftover map (a loop nest that is not a library node): CUDAScheduler applies
// CUDATransform with 32-thread blocks (opt/src/passes/scheduler/cuda_scheduler.cpp:13-70) and CUDAMapDispatcher writes a
// kernel that handles one element per thread under `if (i < n)` (opt/src/targets/cuda/cuda_map_dispatcher.cpp:42-168,
// 208-213). The B200 target keeps that pipeline for everything it does not recognise, and takes over flat element-wise
// maps: one loop, blocks of tasklets only, every array access `container[indvar]`. Those are re-tagged from "CUDA" to
// "B200" after the transform, and B200MapDispatcher writes them as vector kernels (b200_map_emit.h).
#pragma once

#include <sdfg/codegen/dispatchers/node_dispatcher.h>
#include <sdfg/codegen/instrumentation/instrumentation_info.h>
#include <sdfg/passes/scheduler/cuda_scheduler.h>
#include <sdfg/passes/scheduler/loop_scheduler.h>
#include <sdfg/structured_control_flow/map.h>

#include "b200_map_emit.h"

namespace docc::target::b200 {

// Registered like ScheduleType_CUDA (opt/include/sdfg/targets/cuda/cuda.h:32-46): an offloading schedule.
class ScheduleType_B200 {
public:
    static const std::string value() { return "B200"; }
    static sdfg::structured_control_flow::ScheduleType create() {
        return sdfg::structured_control_flow::ScheduleType(value(), sdfg::structured_control_flow::ScheduleTypeCategory::Offloader);
    }
};

// True if `map` is a flat element-wise map; fills `out` (operands sorted by name, as the CUDA dispatcher sorts its
// arguments) when it is. Used by the scheduler (to decide) and by the dispatcher (to emit).
bool recognise_elementwise_map(sdfg::StructuredSDFG& sdfg, sdfg::analysis::AnalysisManager& analysis_manager,
                               sdfg::structured_control_flow::Map& map, sdfg::codegen::LanguageExtension& language_extension,
                               docc_b200_plugin::ElementwiseMap* out);

// Loop scheduler for target "b200" (sdfg.schedule("b200", ...), python/docc/sdfg/__init__.py): CUDAScheduler's steps,
// then the re-tagging of the maps the B200 dispatcher covers.
class B200Scheduler : public sdfg::passes::scheduler::LoopScheduler {
public:
    sdfg::passes::scheduler::SchedulerAction schedule(sdfg::builder::StructuredSDFGBuilder& builder,
                                                      sdfg::analysis::AnalysisManager& analysis_manager,
                                                      sdfg::structured_control_flow::StructuredLoop& loop,
                                                      bool offload_unknown_sizes = false) override;
    sdfg::passes::scheduler::SchedulerAction schedule(sdfg::builder::StructuredSDFGBuilder& builder,
                                                      sdfg::analysis::AnalysisManager& analysis_manager,
                                                      sdfg::structured_control_flow::While& loop,
                                                      bool offload_unknown_sizes = false) override;
    static std::string target() { return "b200"; }
    std::unordered_set<sdfg::structured_control_flow::ScheduleTypeCategory> compatible_types() override;
    void set_report(sdfg::PassReportConsumer* report) override;

private:
    sdfg::passes::scheduler::CUDAScheduler cuda_;
};

class B200MapDispatcher : public sdfg::codegen::NodeDispatcher {
public:
    B200MapDispatcher(sdfg::codegen::LanguageExtension& language_extension, sdfg::StructuredSDFG& sdfg,
                      sdfg::analysis::AnalysisManager& analysis_manager, sdfg::structured_control_flow::Map& node,
                      sdfg::codegen::InstrumentationPlan& instrumentation_plan, sdfg::codegen::ArgCapturePlan& arg_capture_plan);

    void dispatch_node(sdfg::codegen::PrettyPrinter& main_stream, sdfg::codegen::PrettyPrinter& globals_stream,
                       sdfg::codegen::CodeSnippetFactory& library_snippet_factory) override;

    sdfg::codegen::InstrumentationInfo instrumentation_info() const override;

private:
    sdfg::structured_control_flow::Map& node_;
};

}  // namespace docc::target::b200
