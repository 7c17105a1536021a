// Python bindings of the host-side runtime: cache manager and scheduler.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "cache_manager.hpp"
#include "scheduler.hpp"

namespace py = pybind11;
using namespace mxb;

PYBIND11_MODULE(_mxb_host, m) {
  m.doc() = "metallix_b200 host runtime: paged cache accounting and continuous batching";

  py::class_<GroupConfig>(m, "GroupConfig")
      .def(py::init([](int page_tokens, int window, int num_pages) {
             GroupConfig g;
             g.page_tokens = page_tokens;
             g.window = window;
             g.num_pages = num_pages;
             return g;
           }),
           py::arg("page_tokens"), py::arg("window") = 0, py::arg("num_pages") = 0)
      .def_readwrite("page_tokens", &GroupConfig::page_tokens)
      .def_readwrite("window", &GroupConfig::window)
      .def_readwrite("num_pages", &GroupConfig::num_pages);

  static py::exception<OutOfPages> out_of_pages(m, "OutOfPages", PyExc_RuntimeError);

  py::class_<CacheManager>(m, "CacheManager")
      .def(py::init<std::vector<GroupConfig>, int>(), py::arg("groups"), py::arg("max_requests"))
      .def("num_groups", &CacheManager::num_groups)
      .def("group", &CacheManager::group)
      .def("max_requests", &CacheManager::max_requests)
      .def("free_pages", &CacheManager::free_pages)
      .def("free_slots", &CacheManager::free_slots)
      .def("live_requests", &CacheManager::live_requests)
      .def("live_ids", &CacheManager::live_ids)
      .def("has", &CacheManager::has)
      .def("admit", &CacheManager::admit)
      .def("slot", &CacheManager::slot)
      .def("epoch", &CacheManager::epoch)
      .def("reserved", &CacheManager::reserved)
      .def("computed", &CacheManager::computed)
      .def("cost", &CacheManager::cost)
      .def("fits", &CacheManager::fits)
      .def("reserve", &CacheManager::reserve)
      .def("commit", &CacheManager::commit)
      .def("rollback", &CacheManager::rollback)
      .def("release", &CacheManager::release)
      .def("fork",
           [](CacheManager& manager, int64_t parent, int64_t child) {
             CacheManager::Fork f = manager.fork(parent, child);
             py::list copies;
             for (const auto& c : f.copies) copies.append(py::make_tuple(c.group, c.source, c.target));
             return py::make_tuple(f.source_slot, f.target_slot, copies);
           },
           "(source slot, target slot, [(group, source page, target page)]) the device has to copy")
      .def("references", &CacheManager::references)
      .def("table", &CacheManager::table)
      .def("first_live_page", &CacheManager::first_live_page)
      .def("pages_handed_out", &CacheManager::pages_handed_out)
      .def("pages_reused", &CacheManager::pages_reused)
      .def("check_invariants", &CacheManager::check_invariants);

  py::class_<Limits>(m, "Limits")
      .def(py::init([](int max_num_seqs, int max_tokens_per_step, int prefill_chunk) {
             Limits l;
             l.max_num_seqs = max_num_seqs;
             l.max_tokens_per_step = max_tokens_per_step;
             l.prefill_chunk = prefill_chunk;
             return l;
           }),
           py::arg("max_num_seqs") = 8, py::arg("max_tokens_per_step") = 8192,
           py::arg("prefill_chunk") = 0)
      .def_readwrite("max_num_seqs", &Limits::max_num_seqs)
      .def_readwrite("max_tokens_per_step", &Limits::max_tokens_per_step)
      .def_readwrite("prefill_chunk", &Limits::prefill_chunk);

  py::class_<SamplingParams>(m, "SamplingParams")
      .def(py::init([](double temperature, uint64_t seed, double top_p, int top_k, int sampler) {
             SamplingParams s;
             s.temperature = temperature;
             s.seed = seed;
             s.top_p = top_p;
             s.top_k = top_k;
             s.sampler = sampler;
             return s;
           }),
           py::arg("temperature") = 0.0, py::arg("seed") = 0, py::arg("top_p") = 1.0,
           py::arg("top_k") = 0, py::arg("sampler") = 0)
      .def_readwrite("temperature", &SamplingParams::temperature)
      .def_readwrite("seed", &SamplingParams::seed)
      .def_readwrite("top_p", &SamplingParams::top_p)
      .def_readwrite("top_k", &SamplingParams::top_k)
      .def_readwrite("sampler", &SamplingParams::sampler);

  py::class_<RequestInfo>(m, "RequestInfo")
      .def_readonly("id", &RequestInfo::id)
      .def_readonly("prompt", &RequestInfo::prompt)
      .def_readonly("output", &RequestInfo::output)
      .def_readonly("max_new_tokens", &RequestInfo::max_new_tokens)
      .def_readonly("stop_ids", &RequestInfo::stop_ids)
      .def_readonly("ignore_eos", &RequestInfo::ignore_eos)
      .def_readonly("sampling", &RequestInfo::sampling)
      .def_readonly("preemptions", &RequestInfo::preemptions)
      .def_readonly("finish_reason", &RequestInfo::finish_reason)
      .def_readonly("failed", &RequestInfo::failed);

  py::class_<PlanEntry>(m, "PlanEntry")
      .def_readonly("id", &PlanEntry::id)
      .def_readonly("start", &PlanEntry::start)
      .def_readonly("tokens", &PlanEntry::tokens)
      .def_readonly("wants_token", &PlanEntry::wants_token)
      .def_readonly("generated_position", &PlanEntry::generated_position);

  py::class_<StepPlan>(m, "StepPlan")
      .def_readonly("entries", &StepPlan::entries)
      .def_readonly("preempted", &StepPlan::preempted)
      .def_readonly("failed", &StepPlan::failed)
      .def_readonly("decode_tokens", &StepPlan::decode_tokens)
      .def_readonly("prefill_tokens", &StepPlan::prefill_tokens);

  py::class_<Event>(m, "Event")
      .def_readonly("id", &Event::id)
      .def_readonly("token", &Event::token)
      .def_readonly("finished", &Event::finished)
      .def_readonly("finish_reason", &Event::finish_reason);

  py::class_<Scheduler>(m, "Scheduler")
      .def(py::init<CacheManager*, Limits>(), py::arg("cache"), py::arg("limits"),
           py::keep_alive<1, 2>())
      .def("add", &Scheduler::add, py::arg("prompt"), py::arg("max_new_tokens"),
           py::arg("stop_ids") = std::vector<int32_t>{}, py::arg("ignore_eos") = false,
           py::arg("sampling") = SamplingParams{}, py::arg("deadline") = 0.0)
      .def("cancel", &Scheduler::cancel)
      .def("idle", &Scheduler::idle)
      .def("num_waiting", &Scheduler::num_waiting)
      .def("num_running", &Scheduler::num_running)
      .def("running", &Scheduler::running)
      .def("waiting", &Scheduler::waiting)
      .def("request", &Scheduler::request, py::return_value_policy::copy)
      .def("forget", &Scheduler::forget)
      .def("plan", &Scheduler::plan, py::arg("now") = 0.0)
      .def("update", &Scheduler::update)
      .def("fail_plan", &Scheduler::fail_plan);
}
