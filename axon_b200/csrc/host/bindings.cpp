// Python bindings of the host library (module `axon_host`).
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "cache_manager.h"
#include "sampler.h"
#include "scheduler.h"

namespace py = pybind11;
using namespace axon;

PYBIND11_MODULE(axon_host, m) {
    m.doc() = "axon_b200 host library: pages, cache manager, scheduler, sampler";

    py::register_exception<CacheError>(m, "CacheError");
    py::register_exception<SchedulerError>(m, "SchedulerError");

    py::class_<PageAllocator>(m, "PageAllocator")
        .def(py::init<int, uint64_t>(), py::arg("n_pages"), py::arg("shuffle_seed") = 0)
        .def("alloc", &PageAllocator::alloc)
        .def("retain", &PageAllocator::retain)
        .def("release", &PageAllocator::release)
        .def("flush", &PageAllocator::flush)
        .def("refs", &PageAllocator::refs)
        .def("check", &PageAllocator::check)
        .def_property_readonly("n_pages", &PageAllocator::n_pages)
        .def_property_readonly("n_free", &PageAllocator::n_free)
        .def_property_readonly("n_retired", &PageAllocator::n_retired)
        .def_property_readonly("n_held", &PageAllocator::n_held);

    py::class_<GroupConfig>(m, "GroupConfig")
        .def(py::init([](int page_size, int n_pages, int window) {
                 GroupConfig c;
                 c.page_size = page_size;
                 c.n_pages = n_pages;
                 c.window = window;
                 return c;
             }),
             py::arg("page_size"), py::arg("n_pages"), py::arg("window") = 0)
        .def_readwrite("page_size", &GroupConfig::page_size)
        .def_readwrite("n_pages", &GroupConfig::n_pages)
        .def_readwrite("window", &GroupConfig::window);

    py::class_<CacheManager>(m, "CacheManager")
        .def(py::init<std::vector<GroupConfig>, int, int, uint64_t>(), py::arg("groups"),
             py::arg("max_slots"), py::arg("max_positions"), py::arg("shuffle_seed") = 0)
        .def_property_readonly("n_groups", &CacheManager::n_groups)
        .def_property_readonly("max_slots", &CacheManager::max_slots)
        .def_property_readonly("max_positions", &CacheManager::max_positions)
        .def_property_readonly("n_open", &CacheManager::n_open)
        .def("group", &CacheManager::group)
        .def("table_stride", &CacheManager::table_stride)
        .def("sink_page", &CacheManager::sink_page)
        .def("open_slot", &CacheManager::open_slot)
        .def("close_slot", &CacheManager::close_slot)
        .def("is_open", &CacheManager::is_open)
        .def("length", &CacheManager::length)
        .def("reserved_length", &CacheManager::reserved_length)
        .def("pages_short", &CacheManager::pages_short)
        .def("reserve", &CacheManager::reserve)
        .def("commit", &CacheManager::commit)
        .def("flush", &CacheManager::flush)
        .def("free_pages", &CacheManager::free_pages)
        .def("retired_pages", &CacheManager::retired_pages)
        .def("held_pages", &CacheManager::held_pages)
        .def("slot_pages", &CacheManager::slot_pages)
        .def("pages_for", &CacheManager::pages_for)
        .def("pages_needed", &CacheManager::pages_needed)
        .def("coverable", &CacheManager::coverable)
        .def("could_ever_hold", &CacheManager::could_ever_hold)
        .def("version", &CacheManager::version)
        .def("check", &CacheManager::check)
        // a step of single tokens laid out in one call; see cache_manager.h
        .def("stage_decode", [](CacheManager& c, const std::vector<int>& slots, const std::vector<int>& tokens,
                                const std::vector<unsigned char>& wanted, int vocab,
                                py::array_t<int32_t, py::array::c_style> out) {
            const int n = (int)slots.size();
            if (tokens.size() != slots.size() || wanted.size() != slots.size()) throw CacheError("stage_decode: lists of different lengths");
            if (out.size() < (py::ssize_t)(10 * (size_t)n)) throw CacheError("stage_decode: the output block is too small");
            int bad = -1;
            const int rc = c.stage_decode(slots.data(), tokens.data(), wanted.data(), n, vocab, out.mutable_data(), &bad);
            return py::make_tuple(rc, bad);
        })
        .def("commit_decode", [](CacheManager& c, const std::vector<int>& slots) { c.commit_decode(slots.data(), (int)slots.size()); })
        // any step laid out in one call; see cache_manager.h.  Returns (status, failing entry, tokens,
        // entries, wanted places, 1 when every entry brings one token, values written to `out`).
        .def("stage_step", [](CacheManager& c, py::array_t<int32_t, py::array::c_style | py::array::forcecast> slots,
                              py::array_t<int32_t, py::array::c_style | py::array::forcecast> tok_off,
                              py::array_t<int32_t, py::array::c_style | py::array::forcecast> tokens,
                              py::array_t<int32_t, py::array::c_style | py::array::forcecast> want_off,
                              py::array_t<int32_t, py::array::c_style | py::array::forcecast> wants, int vocab,
                              int max_step_tokens, py::array_t<int32_t, py::array::c_style> out) {
            const int n = (int)slots.size();
            if (tok_off.size() != n + 1 || want_off.size() != n + 1) throw CacheError("stage_step: offsets need one value more than there are entries");
            if (n > 0 && (tokens.size() < tok_off.data()[n] || wants.size() < want_off.data()[n]))
                throw CacheError("stage_step: offsets reach past the token or wanted-place lists");
            CacheManager::StepLayout lay;
            int bad = -1;
            const int rc = c.stage_step(slots.data(), tok_off.data(), tokens.data(), want_off.data(), wants.data(), n, vocab,
                                        max_step_tokens, out.mutable_data(), (long long)out.size(), &lay, &bad);
            return py::make_tuple(rc, bad, lay.n_tokens, lay.n_entries, lay.n_want, lay.decode_only, lay.total);
        })
        .def("commit_step", [](CacheManager& c, py::array_t<int32_t, py::array::c_style | py::array::forcecast> segments, int n) {
            if (segments.size() < 4 * (py::ssize_t)n) throw CacheError("commit_step: segments are [4][entries]");
            c.commit_step(segments.data(), n);
        })
        // the host block table of a group as a numpy view [max_slots][stride] (no copy)
        .def("table", [](CacheManager& c, int g) {
            return py::array_t<int32_t>({(py::ssize_t)c.max_slots(), (py::ssize_t)c.table_stride(g)},
                                        {(py::ssize_t)(c.table_stride(g) * sizeof(int32_t)), (py::ssize_t)sizeof(int32_t)},
                                        c.table_mut(g), py::cast(&c));
        });

    py::class_<SampleConfig>(m, "SampleConfig")
        .def(py::init<>())
        .def_readwrite("temp", &SampleConfig::temp)
        .def_readwrite("top_k", &SampleConfig::top_k)
        .def_readwrite("top_p", &SampleConfig::top_p)
        .def_readwrite("min_p", &SampleConfig::min_p)
        .def_readwrite("repeat_penalty", &SampleConfig::repeat_penalty)
        .def_readwrite("repeat_last_n", &SampleConfig::repeat_last_n)
        .def_readwrite("seed", &SampleConfig::seed);

    py::class_<Rng>(m, "Rng")
        .def(py::init<uint64_t>())
        .def("next_u64", &Rng::next_u64)
        .def("uniform", &Rng::uniform)
        .def("state", &Rng::state);

    py::class_<Sampler>(m, "Sampler")
        .def(py::init<SampleConfig>())
        .def_property_readonly("config", &Sampler::config)
        .def("uniform", &Sampler::uniform)
        .def("pick", [](Sampler& s, py::array_t<float, py::array::c_style | py::array::forcecast> logits,
                        py::array_t<int32_t, py::array::c_style | py::array::forcecast> ids) {
            if (logits.ndim() != 1 || ids.ndim() != 1 || logits.shape(0) != ids.shape(0) || logits.shape(0) == 0)
                throw std::invalid_argument("pick needs equally long, non-empty candidate arrays");
            return s.pick(logits.data(), ids.data(), (int)logits.shape(0));
        });

    m.def("kept", [](const SampleConfig& c, py::array_t<float, py::array::c_style | py::array::forcecast> logits) {
        return kept(c, logits.data(), (int)logits.shape(0));
    });
    m.def("pick_at", [](const SampleConfig& c, py::array_t<float, py::array::c_style | py::array::forcecast> logits,
                        py::array_t<int32_t, py::array::c_style | py::array::forcecast> ids, double u) {
        return pick_at(c, logits.data(), ids.data(), (int)logits.shape(0), u);
    });
    m.def("penalty_ids", &penalty_ids);

    py::class_<SchedulerConfig>(m, "SchedulerConfig")
        .def(py::init([](int max_batch_tokens, int max_running, int prefill_chunk) {
                 SchedulerConfig c;
                 c.max_batch_tokens = max_batch_tokens;
                 c.max_running = max_running;
                 c.prefill_chunk = prefill_chunk;
                 return c;
             }),
             py::arg("max_batch_tokens") = 2048, py::arg("max_running") = 16, py::arg("prefill_chunk") = 0)
        .def_readwrite("max_batch_tokens", &SchedulerConfig::max_batch_tokens)
        .def_readwrite("max_running", &SchedulerConfig::max_running)
        .def_readwrite("prefill_chunk", &SchedulerConfig::prefill_chunk);

    py::enum_<Phase>(m, "Phase")
        .value("Waiting", Phase::Waiting)
        .value("Prefill", Phase::Prefill)
        .value("Decode", Phase::Decode)
        .value("Finished", Phase::Finished);
    py::enum_<Finish>(m, "Finish")
        .value("NotFinished", Finish::None)
        .value("Stop", Finish::Stop)
        .value("Length", Finish::Length)
        .value("Aborted", Finish::Aborted);

    py::class_<Request>(m, "Request")
        .def_readonly("id", &Request::id)
        .def_readonly("tokens", &Request::tokens)
        .def_readonly("prompt_len", &Request::prompt_len)
        .def_readonly("max_new", &Request::max_new)
        .def_readonly("phase", &Request::phase)
        .def_readonly("finish", &Request::finish)
        .def_readonly("slot", &Request::slot)
        .def_readonly("fed", &Request::fed)
        .def_readonly("generated", &Request::generated)
        .def_readonly("preemptions", &Request::preemptions);

    py::class_<PlanEntry>(m, "PlanEntry")
        .def_readonly("id", &PlanEntry::id)
        .def_readonly("slot", &PlanEntry::slot)
        .def_readonly("start", &PlanEntry::start)
        .def_readonly("tokens", &PlanEntry::tokens)
        .def_readonly("want_logits", &PlanEntry::want_logits);

    py::class_<Plan>(m, "Plan")
        .def_readonly("entries", &Plan::entries)
        .def_readonly("preempted", &Plan::preempted)
        .def_readonly("n_tokens", &Plan::n_tokens)
        .def_property_readonly("n_entries", [](const Plan& p) { return (int)p.entries.size(); })
        // The plan as arrays, for the step function's native staging: request ids and slots of the
        // entries, token offsets (entries + 1) and the tokens, offsets of wanted places (entries + 1)
        // and the places (the last token of an entry that wants logits).
        .def("flat", [](const Plan& p) {
            const py::ssize_t n = (py::ssize_t)p.entries.size();
            py::array_t<int64_t> ids(n);
            py::ssize_t n_want = 0, n_tok = 0;
            for (const PlanEntry& e : p.entries) { n_want += e.want_logits ? 1 : 0; n_tok += (py::ssize_t)e.tokens.size(); }
            py::array_t<int32_t> slots(n), tok_off(n + 1), want_off(n + 1), tokens(n_tok);
            py::array_t<int32_t> wants(n_want);
            int64_t* idp = ids.mutable_data();
            int32_t *sp = slots.mutable_data(), *to = tok_off.mutable_data(), *wo = want_off.mutable_data();
            int32_t *tp = tokens.mutable_data(), *wp = wants.mutable_data();
            int at = 0, w = 0;
            to[0] = wo[0] = 0;
            for (py::ssize_t i = 0; i < n; ++i) {
                const PlanEntry& e = p.entries[(size_t)i];
                idp[i] = e.id; sp[i] = e.slot;
                for (int32_t t : e.tokens) tp[at++] = t;
                if (e.want_logits) wp[w++] = (int32_t)e.tokens.size() - 1;
                to[i + 1] = at; wo[i + 1] = w;
            }
            return py::make_tuple(ids, slots, tok_off, tokens, want_off, wants);
        });

    py::class_<Done>(m, "Done").def_readonly("id", &Done::id).def_readonly("finish", &Done::finish);

    py::class_<Scheduler>(m, "Scheduler")
        .def(py::init<CacheManager*, SchedulerConfig>(), py::arg("cache"), py::arg("config"),
             py::keep_alive<1, 2>())
        .def("add", &Scheduler::add, py::arg("id"), py::arg("prompt"), py::arg("max_new"),
             py::arg("stop") = std::vector<int32_t>())
        .def("abort", &Scheduler::abort)
        .def("plan", &Scheduler::plan)
        .def("commit", &Scheduler::commit)
        .def("commit_in_order", [](Scheduler& s, const Plan& plan, py::array_t<int32_t, py::array::c_style | py::array::forcecast> picks) {
            return s.commit_in_order(plan, picks.data(), (int)picks.size());
        })
        .def("idle", &Scheduler::idle)
        .def("request", &Scheduler::request, py::return_value_policy::copy)
        .def("take_output", &Scheduler::take_output)
        .def_property_readonly("n_waiting", &Scheduler::n_waiting)
        .def_property_readonly("n_running", &Scheduler::n_running)
        .def_property_readonly("config", &Scheduler::config);
}
