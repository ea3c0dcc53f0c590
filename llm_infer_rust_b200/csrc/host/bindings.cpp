// Python bindings of the host runtime (cache manager, scheduler, batch builder).
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "batch_builder.h"
#include "page_cache.h"
#include "scheduler.h"

namespace py = pybind11;
using namespace b200;

PYBIND11_MODULE(_host_runtime, m) {
  m.doc() = "Host runtime: paged cache bookkeeping, scheduler and batch builder";

  py::class_<GroupSpec>(m, "GroupSpec")
      .def(py::init([](int page_size, int num_pages, int window) {
             GroupSpec s; s.page_size = page_size; s.num_pages = num_pages; s.window = window; return s;
           }), py::arg("page_size"), py::arg("num_pages"), py::arg("window") = 0)
      .def_readwrite("page_size", &GroupSpec::page_size)
      .def_readwrite("num_pages", &GroupSpec::num_pages)
      .def_readwrite("window", &GroupSpec::window);

  py::enum_<Acquire>(m, "Acquire")
      .value("Ready", Acquire::Ready).value("DeferredMemory", Acquire::DeferredMemory)
      .value("Impossible", Acquire::Impossible).value("DeferredSlots", Acquire::DeferredSlots);

  py::class_<PagePool>(m, "PagePool")
      .def(py::init<int>())
      .def("alloc", &PagePool::alloc)
      .def("release", &PagePool::release)
      .def("free_count", &PagePool::free_count)
      .def("is_held", &PagePool::is_held)
      .def("free_list", &PagePool::free_list);

  py::class_<CacheManager>(m, "CacheManager")
      .def(py::init<std::vector<GroupSpec>, int>(), py::arg("groups"), py::arg("num_state_slots"))
      .def("num_groups", &CacheManager::num_groups)
      .def("group", &CacheManager::group)
      .def("free_pages", &CacheManager::free_pages)
      .def("unpromised_pages", &CacheManager::unpromised_pages)
      .def("free_state_slots", &CacheManager::free_state_slots)
      .def("live_requests", &CacheManager::live_requests)
      .def("has", &CacheManager::has)
      .def("pages_needed", &CacheManager::pages_needed)
      .def("acquire", &CacheManager::acquire, py::arg("id"), py::arg("capacity_tokens"), py::arg("max_step_tokens"))
      .def("open", &CacheManager::open)
      .def("grow", &CacheManager::grow)
      .def("grow_all", &CacheManager::grow_all)
      .def("advance", &CacheManager::advance)
      .def("release", &CacheManager::release)
      .def("length", &CacheManager::length)
      .def("state_slot", &CacheManager::state_slot)
      .def("block_table", &CacheManager::block_table)
      .def("first_live_page", &CacheManager::first_live_page)
      .def("pages_held", &CacheManager::pages_held)
      .def("slot_of", &CacheManager::slot_of)
      .def("check", &CacheManager::check);

  py::class_<SamplingParams>(m, "SamplingParams")
      .def(py::init([](float temperature, int top_k, float top_p, bool ignore_eos, int max_tokens, uint64_t seed) {
             SamplingParams p; p.temperature = temperature; p.top_k = top_k; p.top_p = top_p;
             p.ignore_eos = ignore_eos; p.max_tokens = max_tokens; p.seed = seed; return p;
           }), py::arg("temperature") = 0.0f, py::arg("top_k") = -1, py::arg("top_p") = 1.0f,
           py::arg("ignore_eos") = false, py::arg("max_tokens") = 1024, py::arg("seed") = 0)
      .def("normalized", &SamplingParams::normalized)
      .def_readwrite("temperature", &SamplingParams::temperature)
      .def_readwrite("top_k", &SamplingParams::top_k)
      .def_readwrite("top_p", &SamplingParams::top_p)
      .def_readwrite("ignore_eos", &SamplingParams::ignore_eos)
      .def_readwrite("max_tokens", &SamplingParams::max_tokens)
      .def_readwrite("seed", &SamplingParams::seed);

  py::enum_<Status>(m, "Status")
      .value("Waiting", Status::Waiting).value("Prefilling", Status::Prefilling)
      .value("Decoding", Status::Decoding).value("Finished", Status::Finished);
  py::enum_<FinishReason>(m, "FinishReason")
      .value("NotFinished", FinishReason::None).value("Stop", FinishReason::Stop)
      .value("Length", FinishReason::Length).value("Abort", FinishReason::Abort)
      .value("Error", FinishReason::Error);

  py::class_<OutputToken>(m, "OutputToken")
      .def_readonly("uid", &OutputToken::uid)
      .def_readonly("token", &OutputToken::token)
      .def_readonly("finished", &OutputToken::finished)
      .def_readonly("reason", &OutputToken::reason);

  py::class_<PlanEntry>(m, "PlanEntry")
      .def_readonly("uid", &PlanEntry::uid)
      .def_readonly("start", &PlanEntry::start)
      .def_readonly("count", &PlanEntry::count)
      .def_readonly("sample", &PlanEntry::sample)
      .def_readonly("output_index", &PlanEntry::output_index);

  py::class_<StepPlan>(m, "StepPlan")
      .def_readonly("entries", &StepPlan::entries)
      .def_readonly("prefill_tokens", &StepPlan::prefill_tokens)
      .def_readonly("decode_rows", &StepPlan::decode_rows);

  py::class_<SchedulerOptions>(m, "SchedulerOptions")
      .def(py::init([](int max_running_req, int max_seq_len, int max_batch_tokens) {
             SchedulerOptions o; o.max_running_req = max_running_req; o.max_seq_len = max_seq_len;
             o.max_batch_tokens = max_batch_tokens; return o;
           }), py::arg("max_running_req") = 256, py::arg("max_seq_len") = 8192, py::arg("max_batch_tokens") = 8192)
      .def_readwrite("max_running_req", &SchedulerOptions::max_running_req)
      .def_readwrite("max_seq_len", &SchedulerOptions::max_seq_len)
      .def_readwrite("max_batch_tokens", &SchedulerOptions::max_batch_tokens);

  py::class_<Scheduler>(m, "Scheduler")
      .def(py::init<CacheManager*, SchedulerOptions, std::vector<int>>(), py::arg("cache"), py::arg("options"),
           py::arg("eos_ids"), py::keep_alive<1, 2>())
      .def("add_request", &Scheduler::add_request)
      .def("abort_request", &Scheduler::abort_request)
      .def("is_idle", &Scheduler::is_idle)
      .def("plan_step", &Scheduler::plan_step)
      .def("successor", &Scheduler::successor)
      .def("tokens_of", &Scheduler::tokens_of)
      .def("params_of", &Scheduler::params_of)
      .def("commit_step", &Scheduler::commit_step)
      .def("fail_step", &Scheduler::fail_step)
      .def("rollback_step", &Scheduler::rollback_step)
      .def("drain_outbox", &Scheduler::drain_outbox)
      .def("num_pending", &Scheduler::num_pending)
      .def("num_running", &Scheduler::num_running)
      .def("status_of", &Scheduler::status_of);

  py::class_<BatchLayout>(m, "BatchLayout")
      .def_readonly("num_tokens", &BatchLayout::num_tokens)
      .def_readonly("num_rows", &BatchLayout::num_rows)
      .def_readonly("num_real_rows", &BatchLayout::num_real_rows)
      .def_readonly("num_decode", &BatchLayout::num_decode)
      .def_readonly("num_prefill", &BatchLayout::num_prefill)
      .def_readonly("num_logits", &BatchLayout::num_logits)
      .def_readonly("max_q_len", &BatchLayout::max_q_len)
      .def_readonly("max_kv_len", &BatchLayout::max_kv_len)
      .def_readonly("off_tokens", &BatchLayout::off_tokens)
      .def_readonly("off_positions", &BatchLayout::off_positions)
      .def_readonly("off_row_of_token", &BatchLayout::off_row_of_token)
      .def_readonly("off_cu_q", &BatchLayout::off_cu_q)
      .def_readonly("off_kv_len", &BatchLayout::off_kv_len)
      .def_readonly("off_prefix_len", &BatchLayout::off_prefix_len)
      .def_readonly("off_state_slot", &BatchLayout::off_state_slot)
      .def_readonly("off_decode_rows", &BatchLayout::off_decode_rows)
      .def_readonly("off_prefill_rows", &BatchLayout::off_prefill_rows)
      .def_readonly("off_logit_rows", &BatchLayout::off_logit_rows)
      .def_readonly("off_slots", &BatchLayout::off_slots)
      .def_readonly("off_table", &BatchLayout::off_table)
      .def_readonly("table_width", &BatchLayout::table_width)
      .def_readonly("total_ints", &BatchLayout::total_ints);

  py::class_<BatchRequest>(m, "BatchRequest")
      .def(py::init<>())
      .def_readwrite("ids", &BatchRequest::ids)
      .def_readwrite("counts", &BatchRequest::counts)
      .def_readwrite("tokens", &BatchRequest::tokens)
      .def_readwrite("want_counts", &BatchRequest::want_counts)
      .def_readwrite("want_index", &BatchRequest::want_index)
      .def_readwrite("pad_rows_to", &BatchRequest::pad_rows_to)
      .def_readwrite("fixed_table_width", &BatchRequest::fixed_table_width);

  m.def("plan_batch", &plan_batch);
  m.def("build_batch", [](const CacheManager& cache, const BatchRequest& req,
                          py::array_t<int32_t, py::array::c_style> out) {
    auto info = out.request(true);
    return build_batch(cache, req, static_cast<int32_t*>(info.ptr), static_cast<int64_t>(info.size));
  });
}
