// pybind11 bindings of the host runtime (cache manager, scheduler).
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "runtime.hpp"
#include "step_pack.hpp"

namespace py = pybind11;
using namespace aie;

PYBIND11_MODULE(_aie_host, m) {
    m.doc() = "host runtime: page pool, block tables, state slots, scheduler";

    py::class_<PagePool>(m, "PagePool")
        .def(py::init<int>())
        .def_property_readonly("num_pages", &PagePool::num_pages)
        .def_property_readonly("free_count", &PagePool::free_count)
        .def_property_readonly("in_use", &PagePool::in_use)
        .def_property_readonly("high_water", &PagePool::high_water)
        .def_property_readonly("total_allocations", &PagePool::total_allocations)
        .def("is_held", &PagePool::is_held)
        .def("alloc", [](PagePool& p, int n) -> py::object {
            std::vector<int> out;
            if (!p.alloc(n, out)) return py::none();
            return py::cast(out);
        })
        .def("release", &PagePool::release);

    py::class_<GroupSpec>(m, "GroupSpec")
        .def(py::init([](int page_size, int num_pages, int window) {
                 GroupSpec g; g.page_size = page_size; g.num_pages = num_pages; g.window = window; return g;
             }), py::arg("page_size"), py::arg("num_pages"), py::arg("window") = 0)
        .def_readwrite("page_size", &GroupSpec::page_size)
        .def_readwrite("num_pages", &GroupSpec::num_pages)
        .def_readwrite("window", &GroupSpec::window);

    py::class_<CacheManager>(m, "CacheManager")
        .def(py::init<std::vector<GroupSpec>, int, int>(), py::arg("groups"), py::arg("max_seqs"), py::arg("max_pages_per_seq"))
        .def_property_readonly("num_groups", &CacheManager::num_groups)
        .def_property_readonly("max_seqs", &CacheManager::max_seqs)
        .def_property_readonly("max_pages_per_seq", &CacheManager::max_pages_per_seq)
        .def_property_readonly("free_slots", &CacheManager::free_slots)
        .def("group", &CacheManager::group)
        .def("free_pages", [](const CacheManager& c, int g) { return c.pool(g).free_count(); })
        .def("pages_in_use", [](const CacheManager& c, int g) { return c.pool(g).in_use(); })
        .def("high_water", [](const CacheManager& c, int g) { return c.pool(g).high_water(); })
        .def("total_allocations", [](const CacheManager& c, int g) { return c.pool(g).total_allocations(); })
        .def("slot_live", &CacheManager::slot_live)
        .def("admit", &CacheManager::admit)
        .def("ensure", &CacheManager::ensure)
        .def("tokens_that_fit", &CacheManager::tokens_that_fit)
        .def("advance", &CacheManager::advance)
        .def("release_pages", &CacheManager::release_pages)
        .def("finish", &CacheManager::finish)
        .def("pages", &CacheManager::pages)
        .def("first_live", &CacheManager::first_live)
        .def("check_invariants", &CacheManager::check_invariants)
        .def("fill_block_table", [](const CacheManager& c, int g, std::vector<int> slots, int width,
                                    py::array_t<int32_t, py::array::c_style> out) {
            auto buf = out.mutable_unchecked<2>();
            if (buf.shape(0) < (py::ssize_t)slots.size() || buf.shape(1) != width)
                throw std::invalid_argument("fill_block_table: out must be [>= len(slots), width]");
            c.fill_block_table(g, slots.data(), (int)slots.size(), width, out.mutable_data());
        });

    // The step function's packing: (packed int32 array, segment lengths, T, R, N, max_q_len, max_total_len, width,
    // has_src).  A fault in the entries raises ValueError with the message the step function reports.
    m.def("pack_step", [](const CacheManager& cache, const std::vector<int>& slots, const std::vector<int>& starts,
                          const std::vector<std::vector<long long>>& tokens, const std::vector<std::vector<int>>& wants,
                          const std::vector<int>& srcs, int n_live, int page_size, bool bucket_width) {
        if (slots.size() != tokens.size()) throw std::invalid_argument("pack_step: the entries' fields differ in number");
        const StepShape s = step_shape(cache, starts, tokens, wants, srcs, page_size, bucket_width);
        py::array_t<int32_t> out(s.total);
        pack_step(cache, s, slots, starts, tokens, wants, srcs, n_live, out.mutable_data());
        return py::make_tuple(out, s.lengths, s.T, s.R, s.N, s.max_q_len, s.max_total_len, s.width, s.has_src);
    }, py::arg("cache"), py::arg("slots"), py::arg("starts"), py::arg("tokens"), py::arg("wants"), py::arg("srcs"),
       py::arg("n_live"), py::arg("page_size"), py::arg("bucket_width"));

    // The attention kernels' work lists of a step: (decode_tokens, other_tokens, tiles [n, 2], pairs [m, 2],
    // n_decode, max_decode_len).
    m.def("attention_lists", [](py::array_t<int32_t, py::array::c_style | py::array::forcecast> q_start,
                                py::array_t<int32_t, py::array::c_style | py::array::forcecast> q_len,
                                py::array_t<int32_t, py::array::c_style | py::array::forcecast> ctx_len, int tile) {
        const int R = (int)q_len.size();
        if ((int)q_start.size() != R || (int)ctx_len.size() != R || tile < 1)
            throw std::invalid_argument("attention_lists: arrays differ in length");
        const AttentionLists a = attention_lists(q_start.data(), q_len.data(), ctx_len.data(), R, tile);
        auto arr = [](const std::vector<int32_t>& v) {
            py::array_t<int32_t> o((py::ssize_t)v.size());
            std::copy(v.begin(), v.end(), o.mutable_data());
            return o;
        };
        py::array_t<int32_t> tiles = arr(a.tiles), pairs = arr(a.pairs);
        tiles.resize({(py::ssize_t)a.tiles.size() / 2, (py::ssize_t)2});
        pairs.resize({(py::ssize_t)a.pairs.size() / 2, (py::ssize_t)2});
        return py::make_tuple(arr(a.decode_tokens), arr(a.other_tokens), tiles, pairs, a.n_decode, a.max_decode_len);
    });

    py::class_<StepEntry>(m, "StepEntry")
        .def_readonly("id", &StepEntry::id)
        .def_readonly("slot", &StepEntry::slot)
        .def_readonly("start", &StepEntry::start)
        .def_readonly("n_tokens", &StepEntry::n_tokens)
        .def_readonly("sample", &StepEntry::sample)
        .def("__repr__", [](const StepEntry& e) {
            return "StepEntry(id=" + std::to_string(e.id) + ", slot=" + std::to_string(e.slot) + ", start=" + std::to_string(e.start) +
                   ", n_tokens=" + std::to_string(e.n_tokens) + ", sample=" + (e.sample ? "True" : "False") + ")";
        });

    py::class_<StepPlan>(m, "StepPlan")
        .def_readonly("entries", &StepPlan::entries)
        .def_readonly("preempted", &StepPlan::preempted)
        .def_readonly("admitted", &StepPlan::admitted);

    py::class_<Scheduler>(m, "Scheduler")
        .def(py::init<CacheManager*, int, int, int>(), py::arg("cache"), py::arg("max_num_seqs"),
             py::arg("max_num_batched_tokens"), py::arg("max_seq_len"), py::keep_alive<1, 2>())
        .def("add", &Scheduler::add)
        .def("has_work", &Scheduler::has_work)
        .def_property_readonly("num_running", &Scheduler::num_running)
        .def_property_readonly("num_waiting", &Scheduler::num_waiting)
        .def("schedule", &Scheduler::schedule)
        .def("commit", &Scheduler::commit)
        .def("on_token", &Scheduler::on_token)
        .def("finish", &Scheduler::finish)
        .def("computed", &Scheduler::computed)
        .def("generated", &Scheduler::generated)
        .def("slot", &Scheduler::slot)
        .def("running", &Scheduler::running)
        .def("waiting", &Scheduler::waiting)
        .def("stats", [](const Scheduler& s) {
            const auto& st = s.stats();
            py::dict d;
            d["steps"] = st.steps; d["prompt_tokens"] = st.prompt_tokens; d["decode_tokens"] = st.decode_tokens;
            d["preemptions"] = st.preemptions; d["admitted"] = st.admitted; d["finished"] = st.finished;
            return d;
        });
}
