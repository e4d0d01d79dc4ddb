// Python bindings of the host runtime (cache manager and scheduler).
#include <algorithm>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "cache_manager.hpp"
#include "scheduler.hpp"

namespace py = pybind11;
using namespace dlm;

PYBIND11_MODULE(_dlm_host, m) {
    m.doc() = "dlm_b200 host runtime: page pools, block tables, state slots, scheduler";

    py::register_exception<CacheExhausted>(m, "CacheExhausted", PyExc_RuntimeError);

    py::class_<GroupSpec>(m, "GroupSpec")
        .def(py::init([](int page_size, int window, int num_pages) {
                 GroupSpec g; g.page_size = page_size; g.window = window; g.num_pages = num_pages; return g;
             }), py::arg("page_size"), py::arg("window"), py::arg("num_pages"))
        .def_readwrite("page_size", &GroupSpec::page_size)
        .def_readwrite("window", &GroupSpec::window)
        .def_readwrite("num_pages", &GroupSpec::num_pages);

    py::class_<GroupStats>(m, "GroupStats")
        .def_readonly("total_pages", &GroupStats::total_pages)
        .def_readonly("used_pages", &GroupStats::used_pages)
        .def_readonly("free_pages", &GroupStats::free_pages)
        .def_readonly("high_water", &GroupStats::high_water);

    py::class_<StepItem>(m, "StepItem")
        .def(py::init([](int slot, std::vector<int32_t> tokens, std::vector<int32_t> want) {
                 StepItem it; it.slot = slot; it.tokens = std::move(tokens); it.want = std::move(want); return it;
             }), py::arg("slot"), py::arg("tokens"), py::arg("want"))
        .def_readwrite("slot", &StepItem::slot)
        .def_readwrite("tokens", &StepItem::tokens)
        .def_readwrite("want", &StepItem::want);

    py::class_<StepLayout>(m, "StepLayout")
        .def_readonly("num_tokens", &StepLayout::num_tokens)
        .def_readonly("num_requests", &StepLayout::num_requests)
        .def_readonly("num_wanted", &StepLayout::num_wanted)
        .def_readonly("num_groups", &StepLayout::num_groups)
        .def_readonly("max_q_len", &StepLayout::max_q_len)
        .def_readonly("max_kv_len", &StepLayout::max_kv_len)
        .def_readonly("num_single", &StepLayout::num_single)
        .def_readonly("table_width", &StepLayout::table_width)
        .def_readonly("off_tokens", &StepLayout::off_tokens)
        .def_readonly("off_positions", &StepLayout::off_positions)
        .def_readonly("off_token_req", &StepLayout::off_token_req)
        .def_readonly("off_cu_q", &StepLayout::off_cu_q)
        .def_readonly("off_kv_len", &StepLayout::off_kv_len)
        .def_readonly("off_state_slot", &StepLayout::off_state_slot)
        .def_readonly("off_logit_rows", &StepLayout::off_logit_rows)
        .def_readonly("off_slots", &StepLayout::off_slots)
        .def_readonly("off_table", &StepLayout::off_table)
        .def_readonly("total", &StepLayout::total);

    py::class_<CacheManager>(m, "CacheManager")
        .def(py::init<std::vector<GroupSpec>, int>(), py::arg("groups"), py::arg("num_slots"))
        .def_property_readonly("num_groups", &CacheManager::num_groups)
        .def_property_readonly("num_slots", &CacheManager::num_slots)
        .def_property_readonly("free_slots", &CacheManager::free_slots)
        .def("group", &CacheManager::group)
        .def("open", &CacheManager::open)
        .def("close", &CacheManager::close)
        .def("is_open", &CacheManager::is_open)
        .def("length", &CacheManager::length)
        .def("pages_needed", &CacheManager::pages_needed)
        .def("max_appendable", &CacheManager::max_appendable, py::arg("slot"), py::arg("n"), py::arg("reserve") = 0)
        .def("append", &CacheManager::append)
        .def("can_append", &CacheManager::can_append)
        .def("table", &CacheManager::table)
        .def("stats", &CacheManager::stats)
        .def("free_pages", &CacheManager::free_pages)
        .def("plan_layout", &CacheManager::plan_layout, py::arg("items"), py::arg("min_table_width") = 0,
             py::arg("pad_requests") = 0)
        .def("pack",
             [](const CacheManager& c, const std::vector<StepItem>& items, const StepLayout& lay, uintptr_t out,
                size_t capacity) {
                 if ((size_t)lay.total > capacity) throw std::invalid_argument("metadata buffer is too small");
                 c.pack(items, lay, reinterpret_cast<int32_t*>(out));
             },
             py::arg("items"), py::arg("layout"), py::arg("out_ptr"), py::arg("capacity"))
        .def("pack_decode",
             // a step in which every request brings one token and wants its logits: `pack` without the items
             [](const CacheManager& c, const std::vector<int>& slots, const std::vector<int32_t>& tokens,
                const StepLayout& lay, uintptr_t out, size_t capacity) {
                 if ((size_t)lay.total > capacity) throw std::invalid_argument("metadata buffer is too small");
                 if (slots.size() != tokens.size() || (int)slots.size() > lay.num_requests ||
                     lay.num_tokens != lay.num_requests || lay.num_wanted != lay.num_requests)
                     throw std::invalid_argument("the step does not fit the fixed metadata layout");
                 std::vector<StepItem> items(slots.size());
                 for (size_t i = 0; i < slots.size(); ++i) {
                     items[i].slot = slots[i];
                     items[i].tokens.assign(1, tokens[i]);
                     items[i].want.assign(1, 0);
                     for (int g = 0; g < c.num_groups(); ++g)
                         if ((int)c.table(slots[i], g).size() > lay.table_width[g])
                             throw std::invalid_argument("a request's block table is wider than the layout's");
                 }
                 c.pack(items, lay, reinterpret_cast<int32_t*>(out));
             },
             py::arg("slots"), py::arg("tokens"), py::arg("layout"), py::arg("out_ptr"), py::arg("capacity"))
        .def("max_length",
             [](const CacheManager& c, const std::vector<int>& slots) {
                 int m = 0;
                 for (int s : slots) m = std::max(m, c.length(s));
                 return m;
             })
        .def("check", &CacheManager::check);

    py::class_<SchedulerConfig>(m, "SchedulerConfig")
        .def(py::init([](int max_step_tokens, int max_step_requests, int max_context, int vocab_size) {
                 SchedulerConfig c;
                 c.max_step_tokens = max_step_tokens; c.max_step_requests = max_step_requests;
                 c.max_context = max_context; c.vocab_size = vocab_size;
                 return c;
             }), py::arg("max_step_tokens") = 2048, py::arg("max_step_requests") = 64,
             py::arg("max_context") = 4096, py::arg("vocab_size") = 0)
        .def_readwrite("max_step_tokens", &SchedulerConfig::max_step_tokens)
        .def_readwrite("max_step_requests", &SchedulerConfig::max_step_requests)
        .def_readwrite("max_context", &SchedulerConfig::max_context)
        .def_readwrite("vocab_size", &SchedulerConfig::vocab_size);

    py::class_<PlannedItem>(m, "PlannedItem")
        .def_readonly("id", &PlannedItem::id)
        .def_readonly("slot", &PlannedItem::slot)
        .def_readonly("start", &PlannedItem::start)
        .def_readonly("tokens", &PlannedItem::tokens)
        .def_readonly("sample", &PlannedItem::sample);

    py::class_<Plan>(m, "Plan")
        .def_readonly("items", &Plan::items)
        .def_readonly("preempted", &Plan::preempted)
        .def_readonly("failed", &Plan::failed);

    py::class_<FinishedRequest>(m, "FinishedRequest")
        .def_readonly("id", &FinishedRequest::id)
        .def_readonly("output", &FinishedRequest::output)
        .def_readonly("reason", &FinishedRequest::reason);

    py::class_<SchedulerStats>(m, "SchedulerStats")
        .def_readonly("steps", &SchedulerStats::steps)
        .def_readonly("prompt_tokens", &SchedulerStats::prompt_tokens)
        .def_readonly("decode_tokens", &SchedulerStats::decode_tokens)
        .def_readonly("preemptions", &SchedulerStats::preemptions)
        .def_readonly("finished", &SchedulerStats::finished);

    py::class_<Scheduler>(m, "Scheduler")
        .def(py::init<CacheManager*, SchedulerConfig>(), py::arg("cache"), py::arg("config"),
             py::keep_alive<1, 2>())
        .def("submit", &Scheduler::submit, py::arg("id"), py::arg("prompt"), py::arg("max_new_tokens"),
             py::arg("eos") = std::vector<int32_t>{})
        .def("abort", &Scheduler::abort)
        .def("has_work", &Scheduler::has_work)
        .def_property_readonly("num_waiting", &Scheduler::num_waiting)
        .def_property_readonly("num_running", &Scheduler::num_running)
        .def("plan", &Scheduler::plan)
        .def("commit", &Scheduler::commit)
        .def("drain_finished", &Scheduler::drain_finished)
        .def("stats", &Scheduler::stats)
        .def("output_of", &Scheduler::output_of);
}
