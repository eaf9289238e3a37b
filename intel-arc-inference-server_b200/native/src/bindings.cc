// pybind11 module `b200host`: the native host components exposed to the Python framework layer.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "http_server.h"
#include "json.h"
#include "kv_pool.h"
#include "openai.h"
#include "prefix_cache.h"
#include "prompt_lookup.h"
#include "safetensors.h"
#include "scheduler.h"
#include "spec.h"
#include "draft_policy.h"
#include "tokenizer.h"
#include "toolcall.h"

namespace py = pybind11;
using namespace b2host;

namespace {

py::object to_py(const Json& j) {
  switch (j.type()) {
    case Json::Null: return py::none();
    case Json::Bool: return py::bool_(j.as_bool());
    case Json::Int: return py::int_(j.as_int());
    case Json::Float: return py::float_(j.as_double());
    case Json::String: return py::str(j.as_string());
    case Json::Array: {
      py::list l;
      for (const Json& e : j.items()) l.append(to_py(e));
      return std::move(l);
    }
    case Json::Object: {
      py::dict d;  // Python dicts keep insertion order
      for (const auto& m : j.members()) d[py::str(m.first)] = to_py(m.second);
      return std::move(d);
    }
  }
  return py::none();
}

Json from_py(const py::handle& o) {
  if (o.is_none()) return Json();
  if (py::isinstance<py::bool_>(o)) return Json(o.cast<bool>());
  if (py::isinstance<py::int_>(o)) return Json((int64_t)o.cast<long long>());
  if (py::isinstance<py::float_>(o)) return Json(o.cast<double>());
  if (py::isinstance<py::str>(o)) return Json(o.cast<std::string>());
  if (py::isinstance<py::dict>(o)) {
    Json j = Json::object();
    for (auto kv : o.cast<py::dict>()) j[py::str(kv.first).cast<std::string>()] = from_py(kv.second);
    return j;
  }
  if (py::isinstance<py::list>(o) || py::isinstance<py::tuple>(o)) {
    Json j = Json::array();
    for (auto e : o) j.push_back(from_py(e));
    return j;
  }
  throw std::invalid_argument("value is not JSON-serialisable");
}

using FArr = py::array_t<float, py::array::c_style | py::array::forcecast>;
using UArr = py::array_t<uint32_t, py::array::c_style | py::array::forcecast>;

Sampling make_sampling(float temperature, uint32_t top_k, float top_p) {
  Sampling s;
  s.temperature = temperature;
  s.top_k = top_k;
  s.top_p = top_p;
  return s;
}

py::dict delta_to_py(const Delta& d) {
  py::dict o;
  o["kind"] = d.kind == Delta::Reasoning ? "reasoning" : (d.kind == Delta::Content ? "content" : "call");
  o["text"] = d.text;
  if (d.kind == Delta::Call) {
    o["id"] = d.call.id;
    o["name"] = d.call.name;
    o["arguments"] = to_py(d.call.arguments);
    o["arguments_json"] = d.call.arguments.dump();
    o["index"] = d.index;
  }
  return o;
}

ToolCall call_from_py(const py::dict& d) {
  ToolCall c;
  c.id = d["id"].cast<std::string>();
  c.name = d["name"].cast<std::string>();
  c.arguments = d.contains("arguments_json") ? Json::parse(d["arguments_json"].cast<std::string>()) : from_py(d["arguments"]);
  return c;
}

}  // namespace

PYBIND11_MODULE(b200host, m) {
  m.doc() = "native host components of b200serve";
  py::register_exception<BadRequest>(m, "BadRequest", PyExc_ValueError);

  // ------------------------------------------------------------ JSON
  m.def("json_loads", [](const std::string& s) { return to_py(Json::parse(s)); });
  m.def("json_dumps", [](const py::object& o) { return from_py(o).dump(); });

  // ------------------------------------------------------------ KV pool
  py::class_<KvPool>(m, "KvPool")
      .def(py::init<int, int, int>())
      .def("free_pages", &KvPool::free_pages)
      .def("table", &KvPool::table)
      .def("refcount", &KvPool::refcount)
      .def("ensure", &KvPool::ensure)
      .def("truncate", &KvPool::truncate)
      .def("release", &KvPool::release)
      .def("share", &KvPool::share)
      .def("adopt", &KvPool::adopt)
      .def("pin", &KvPool::pin)
      .def("unpin", &KvPool::unpin);

  // ------------------------------------------------------------ prompt lookup
  py::class_<PromptLookup>(m, "PromptLookup")
      .def(py::init<uint32_t, uint32_t, uint32_t>(), py::arg("max_match") = 64, py::arg("max_candidates") = 64,
           py::arg("max_steps") = 1024)
      .def("clear", &PromptLookup::clear)
      .def("append", &PromptLookup::append)
      .def("extend", &PromptLookup::append_many)
      .def("boundary", &PromptLookup::boundary)
      .def("truncate", &PromptLookup::truncate)
      .def("size", &PromptLookup::size)
      .def("ids", &PromptLookup::ids)
      .def("match",
           [](const PromptLookup& l, uint32_t min_n, uint32_t source_before) {
             auto mm = l.match(min_n, source_before);
             return py::make_tuple(mm.end == PromptLookup::kNone ? -1 : (long long)mm.end, mm.length, mm.steps, mm.truncated);
           },
           py::arg("min_n"), py::arg("source_before") = PromptLookup::kNone)
      .def("propose",
           [](const PromptLookup& l, uint32_t max_k, uint32_t min_n, uint32_t source_before) {
             return l.propose(max_k, min_n, nullptr, source_before);
           },
           py::arg("max_k"), py::arg("min_n"), py::arg("source_before") = PromptLookup::kNone);
  py::class_<LookupPolicy>(m, "LookupPolicy")
      .def(py::init<>())
      .def("active", &LookupPolicy::active)
      .def("width", &LookupPolicy::width)
      .def("decide", &LookupPolicy::decide)
      .def("observe", &LookupPolicy::observe);

  // ------------------------------------------------------------ sampling / acceptance
  // the samplers read `vocab_used` floats from the row: a shorter row (a vocabulary shard, say) is refused
  auto need_row = [](size_t have, uint32_t vocab_used) {
    if (have < vocab_used) throw std::invalid_argument("logits row is shorter than the vocabulary in use");
  };
  m.def("filter_probs", [need_row](FArr logits, uint32_t vocab_used, float temperature, uint32_t top_k, float top_p) {
    need_row((size_t)logits.size(), vocab_used);
    auto f = filter_probs(logits.data(), vocab_used, make_sampling(temperature, top_k, top_p));
    return py::make_tuple(f.ids, f.probs, f.mass);
  });
  m.def("apply_repetition_penalty", [need_row](py::array_t<float, py::array::c_style> logits, uint32_t vocab_used,
                                        const std::vector<uint32_t>& ids, float penalty) {
    need_row((size_t)logits.size(), vocab_used);
    apply_repetition_penalty(logits.mutable_data(), vocab_used, ids, penalty);
  });
  m.def("sample", [need_row](FArr logits, uint32_t vocab_used, float temperature, uint32_t top_k, float top_p, uint64_t seed) {
    need_row((size_t)logits.size(), vocab_used);
    std::mt19937_64 rng(seed);
    return draw(filter_probs(logits.data(), vocab_used, make_sampling(temperature, top_k, top_p)), rng);
  });
  m.def("argmax_low_tie", [need_row](FArr logits, uint32_t n) {
    need_row((size_t)logits.size(), n);
    return argmax_low_tie(logits.data(), n);
  });
  m.def("accept_greedy", [](const std::vector<uint32_t>& verify_argmax, const std::vector<uint32_t>& drafts) {
    if (verify_argmax.size() < drafts.size() + 1) throw std::invalid_argument("need k + 1 verify rows");
    auto r = accept_greedy(verify_argmax.data(), drafts.data(), (uint32_t)drafts.size());
    return py::make_tuple(r.accepted, r.next_token);
  });
  m.def("accept_sampled", [](FArr p_rows, FArr q_rows, const std::vector<uint32_t>& drafts, uint32_t vocab_used,
                             float temperature, uint32_t top_k, float top_p, uint64_t seed) {
    std::mt19937_64 rng(seed);
    const size_t stride = (size_t)p_rows.shape(1);
    auto r = accept_sampled(p_rows.data(), q_rows.data(), drafts.data(), (uint32_t)drafts.size(), vocab_used, stride,
                            make_sampling(temperature, top_k, top_p), rng);
    return py::make_tuple(r.accepted, r.next_token);
  });
  m.def("accept_point_mass", [](FArr p_rows, const std::vector<uint32_t>& drafts, uint32_t vocab_used,
                                float temperature, uint32_t top_k, float top_p, uint64_t seed) {
    std::mt19937_64 rng(seed);
    auto r = accept_point_mass(p_rows.data(), drafts.data(), (uint32_t)drafts.size(), vocab_used,
                               (size_t)p_rows.shape(1), make_sampling(temperature, top_k, top_p), rng);
    return py::make_tuple(r.accepted, r.next_token);
  });
  m.def("accept_sparse", [](FArr p_rows, UArr cand, FArr scores, const std::vector<uint32_t>& drafts,
                            uint32_t vocab_used, float temperature, uint32_t top_k, float top_p, uint64_t seed) {
    std::mt19937_64 rng(seed);
    const uint32_t k = (uint32_t)drafts.size(), n = (uint32_t)cand.shape(1);
    std::vector<SparseQ> q(k);
    const Sampling s = make_sampling(temperature, top_k, top_p);
    for (uint32_t i = 0; i < k; ++i) q[i] = sparse_q(cand.data() + (size_t)i * n, scores.data() + (size_t)i * n, n, s.temperature);
    auto r = accept_sparse(p_rows.data(), q.data(), drafts.data(), k, vocab_used, (size_t)p_rows.shape(1), s, rng);
    return py::make_tuple(r.accepted, r.next_token);
  });

  py::class_<StepCosts>(m, "StepCosts")
      .def(py::init<>())
      .def(py::init<std::vector<double>, std::vector<double>>(), py::arg("verify_rows"), py::arg("draft_depth"))
      .def_readwrite("verify_rows", &StepCosts::verify_rows)
      .def_readwrite("draft_depth", &StepCosts::draft_depth)
      .def("deepest", &StepCosts::deepest)
      .def("iteration", &StepCosts::iteration)
      .def("free_drafts", &StepCosts::free_drafts);
  py::class_<DraftLengthOptions>(m, "DraftLengthOptions")
      .def(py::init<>())
      .def_readwrite("deepest", &DraftLengthOptions::deepest)
      .def_readwrite("prior_accept", &DraftLengthOptions::prior_accept)
      .def_readwrite("prior_trials", &DraftLengthOptions::prior_trials)
      .def_readwrite("forget", &DraftLengthOptions::forget)
      .def_readwrite("settle", &DraftLengthOptions::settle)
      .def_readwrite("switch_margin", &DraftLengthOptions::switch_margin)
      .def_readwrite("probe_wait", &DraftLengthOptions::probe_wait)
      .def_readwrite("probe_wait_max", &DraftLengthOptions::probe_wait_max)
      .def_readwrite("costs", &DraftLengthOptions::costs);
  py::class_<DraftLengthPolicy>(m, "DraftLengthPolicy")
      .def(py::init<const DraftLengthOptions&>(), py::arg("options") = DraftLengthOptions())
      .def("next", &DraftLengthPolicy::next)
      .def("observe", &DraftLengthPolicy::observe)
      .def("current", &DraftLengthPolicy::current)
      .def("deepest", &DraftLengthPolicy::deepest)
      .def("acceptance", &DraftLengthPolicy::acceptance)
      .def("expected_tokens", &DraftLengthPolicy::expected_tokens)
      .def("tokens_per_cost", &DraftLengthPolicy::tokens_per_cost)
      .def("best_depth", &DraftLengthPolicy::best_depth);
  py::class_<ConfidenceModel>(m, "ConfidenceModel")
      .def(py::init<double>(), py::arg("learning_rate") = 0.05)
      .def("accept_prob", &ConfidenceModel::accept_prob)
      .def("learn", &ConfidenceModel::learn)
      .def("bias", &ConfidenceModel::bias)
      .def("slope", &ConfidenceModel::slope);
  py::class_<ConfidenceStop>(m, "ConfidenceStop")
      .def(py::init<const StepCosts&, uint32_t, ConfidenceModel&>(), py::keep_alive<1, 4>())
      .def("begin", &ConfidenceStop::begin)
      .def("after_draft", &ConfidenceStop::after_draft)
      .def("observe", &ConfidenceStop::observe)
      .def("verified", &ConfidenceStop::verified)
      .def("deepest", &ConfidenceStop::deepest)
      .def("typical", &ConfidenceStop::typical);

  // ------------------------------------------------------------ prefix cache
  py::class_<PrefixCache>(m, "PrefixCache")
      .def(py::init<int>())
      .def("block_tokens", &PrefixCache::block_tokens)
      .def("num_nodes", &PrefixCache::num_nodes)
      .def("root", &PrefixCache::root)
      .def("match", &PrefixCache::match)
      .def("plan",
           [](PrefixCache& c, int root, const std::vector<uint32_t>& prompt, const std::vector<uint32_t>& resident,
              bool split_last) {
             auto p = c.plan(root, prompt, resident, split_last);
             py::dict d;
             d["kind"] = p.kind == PrefixCache::Cold ? "cold" : (p.kind == PrefixCache::Continue ? "continue" : "restore");
             d["matched_tokens"] = p.matched_tokens;
             d["resident_tokens"] = p.resident_tokens;
             d["path"] = p.path;
             return d;
           })
      .def("insert", &PrefixCache::insert)
      .def("pin", &PrefixCache::pin)
      .def("unpin", &PrefixCache::unpin)
      .def("set_host_slot", &PrefixCache::set_host_slot)
      .def("set_device_pages", &PrefixCache::set_device_pages)
      .def("device_pages", [](const PrefixCache& c, int id) { return c.node(id).device_pages; })
      .def("host_slot", [](const PrefixCache& c, int id) { return c.node(id).host_slot; })
      .def("parent", [](const PrefixCache& c, int id) { return c.node(id).parent; })
      .def("device_victim", &PrefixCache::device_victim)
      .def("leaf_victim", &PrefixCache::leaf_victim)
      .def("remove", &PrefixCache::remove);

  // ------------------------------------------------------------ tool calls
  py::class_<OutputStream>(m, "OutputStream")
      .def(py::init([](bool thinking, const py::object& tools, const std::string& format, uint64_t seed) {
             return new OutputStream(thinking, from_py(tools), format == "hermes" ? OutputStream::Hermes : OutputStream::QwenXml, seed);
           }),
           py::arg("thinking"), py::arg("tools") = py::none(), py::arg("format") = "qwen_xml", py::arg("seed") = 0)
      .def("set_drop_cut_calls", &OutputStream::set_drop_cut_calls)
      .def("push",
           [](OutputStream& s, const std::string& piece) {
             py::list out;
             for (const auto& d : s.push(piece)) out.append(delta_to_py(d));
             return out;
           })
      .def("finish", [](OutputStream& s) {
        py::list out;
        for (const auto& d : s.finish()) out.append(delta_to_py(d));
        return out;
      });
  m.def("parse_output", [](const std::string& text, bool thinking, const py::object& tools, const std::string& format) {
    auto po = parse_output(text, thinking, from_py(tools), format == "hermes" ? 1 : 0);
    py::dict d;
    d["reasoning"] = po.reasoning;
    d["content"] = po.content;
    py::list calls;
    for (const auto& c : po.tool_calls) {
      py::dict cd;
      cd["id"] = c.id;
      cd["name"] = c.name;
      cd["arguments"] = to_py(c.arguments);
      cd["arguments_json"] = c.arguments.dump();
      calls.append(cd);
    }
    d["tool_calls"] = calls;
    return d;
  }, py::arg("text"), py::arg("thinking"), py::arg("tools") = py::none(), py::arg("format") = "qwen_xml");
  m.def("escape_raw_controls", [](const std::string& s) {
    std::string out;
    const bool changed = escape_raw_controls(s, out);
    return py::make_tuple(changed, out);
  });
  m.def("tag_prefix_suffix", &tag_prefix_suffix);
  m.def("make_call_id", &make_call_id);

  // ------------------------------------------------------------ tokenizer
  py::class_<Tokenizer>(m, "Tokenizer")
      .def_static("from_file", &Tokenizer::from_file)
      .def_static("from_json", &Tokenizer::from_json)
      .def("encode", &Tokenizer::encode)
      .def("decode", [](const Tokenizer& t, const std::vector<uint32_t>& ids, bool skip_special) {
             return py::bytes(t.decode(ids, skip_special));
           }, py::arg("ids"), py::arg("skip_special") = false)
      .def("token_bytes", [](const Tokenizer& t, uint32_t id) { return py::bytes(t.token_bytes(id)); })
      .def("token_to_id", &Tokenizer::token_to_id)
      .def("is_special", &Tokenizer::is_special)
      .def("vocab_size", &Tokenizer::vocab_size)
      .def("pre_tokenize", &Tokenizer::pre_tokenize);
  py::class_<Streamer>(m, "Streamer")
      .def(py::init<const Tokenizer*, bool>(), py::arg("tokenizer"), py::arg("skip_special") = true, py::keep_alive<1, 2>())
      .def("push", [](Streamer& s, uint32_t id) { return py::bytes(s.push(id)); })
      .def("finish", [](Streamer& s) { return py::bytes(s.finish()); });

  // ------------------------------------------------------------ HTTP + OpenAI schema
  py::class_<HttpServer>(m, "HttpServer")
      .def(py::init<const std::string&, int, int>(), py::arg("host"), py::arg("port"), py::arg("max_waiting") = 4)
      .def("port", &HttpServer::port)
      .def("stop", &HttpServer::stop, py::call_guard<py::gil_scoped_release>())
      .def("next",
           [](HttpServer& s, int timeout_ms) -> py::object {
             HttpRequest r;
             {
               py::gil_scoped_release rel;
               r = s.next(timeout_ms);
             }
             if (r.id == 0) return py::none();
             py::dict d;
             d["id"] = r.id;
             d["method"] = r.method;
             d["path"] = r.path;
             d["body"] = py::bytes(r.body);
             d["headers"] = r.headers;
             return std::move(d);
           })
      .def("waiting", &HttpServer::waiting)
      .def("cancelled", &HttpServer::cancelled)
      .def("close", &HttpServer::close)
      .def("active", &HttpServer::active)
      .def("respond", &HttpServer::respond, py::call_guard<py::gil_scoped_release>())
      .def("begin_stream", &HttpServer::begin_stream, py::call_guard<py::gil_scoped_release>())
      .def("send_event", &HttpServer::send_event, py::call_guard<py::gil_scoped_release>())
      .def("end_stream", &HttpServer::end_stream, py::call_guard<py::gil_scoped_release>());

  py::class_<ChatRequest>(m, "ChatRequest")
      .def_readonly("chat", &ChatRequest::chat)
      .def_readonly("model", &ChatRequest::model)
      .def_property_readonly("messages", [](const ChatRequest& r) { return to_py(r.messages); })
      .def_readonly("prompt", &ChatRequest::prompt)
      .def_readonly("prompt_ids", &ChatRequest::prompt_ids)
      .def_property_readonly("tools", [](const ChatRequest& r) { return to_py(r.tools); })
      .def_property_readonly("template_kwargs", [](const ChatRequest& r) { return to_py(r.template_kwargs); })
      .def_readwrite("max_tokens", &ChatRequest::max_tokens)
      .def_readonly("min_tokens", &ChatRequest::min_tokens)
      .def_readonly("ignore_eos", &ChatRequest::ignore_eos)
      .def_readonly("stream", &ChatRequest::stream)
      .def_readonly("include_usage", &ChatRequest::include_usage)
      .def_readonly("return_token_ids", &ChatRequest::return_token_ids)
      .def_readonly("stop", &ChatRequest::stop)
      .def_readonly("has_seed", &ChatRequest::has_seed)
      .def_readonly("seed", &ChatRequest::seed)
      .def_readonly("greedy", &ChatRequest::greedy)
      .def_readonly("temperature", &ChatRequest::temperature)
      .def_readonly("top_k", &ChatRequest::top_k)
      .def_readonly("top_p", &ChatRequest::top_p)
      .def_readonly("repetition_penalty", &ChatRequest::repetition_penalty);
  m.def("parse_request", &parse_request, py::arg("body"), py::arg("chat"));
  m.def("error_body", &error_body);
  m.def("models_response", &models_response);
  m.def("completion_response",
        [](const ChatRequest& req, const std::string& id, int64_t created, const std::string& model,
           const std::string& content, const std::string& reasoning, const py::list& calls,
           const std::string& finish_reason, int prompt_tokens, int completion_tokens, int cached_tokens,
           const std::vector<uint32_t>& token_ids) {
          std::vector<ToolCall> cs;
          for (auto c : calls) cs.push_back(call_from_py(c.cast<py::dict>()));
          Usage u{prompt_tokens, completion_tokens, cached_tokens};
          return completion_response(req, id, created, model, content, reasoning, cs, finish_reason, u, token_ids);
        });
  m.def("stream_frame",
        [](const ChatRequest& req, const std::string& id, int64_t created, const std::string& model,
           const std::string& kind, const std::string& text, const py::object& call, uint32_t call_index,
           const std::string& finish_reason, const py::object& usage, const std::vector<uint32_t>& token_ids) {
          static const std::map<std::string, int> kinds{{"role", 0}, {"content", 1}, {"reasoning", 2},
                                                        {"call", 3},  {"finish", 4},  {"usage", 5}};
          ToolCall tc;
          const bool has_call = !call.is_none();
          if (has_call) tc = call_from_py(call.cast<py::dict>());
          Usage u;
          const bool has_usage = !usage.is_none();
          if (has_usage) {
            auto t = usage.cast<py::tuple>();
            u = Usage{t[0].cast<int>(), t[1].cast<int>(), t[2].cast<int>()};
          }
          return stream_frame(req, id, created, model, kinds.at(kind), text, has_call ? &tc : nullptr, call_index,
                              finish_reason, has_usage ? &u : nullptr, token_ids.empty() ? nullptr : &token_ids);
        },
        py::arg("req"), py::arg("id"), py::arg("created"), py::arg("model"), py::arg("kind"), py::arg("text") = "",
        py::arg("call") = py::none(), py::arg("call_index") = 0, py::arg("finish_reason") = "",
        py::arg("usage") = py::none(), py::arg("token_ids") = std::vector<uint32_t>());
  py::class_<StopMatcher>(m, "StopMatcher")
      .def(py::init<std::vector<std::string>>())
      .def("push",
           [](StopMatcher& s, const std::string& piece) {
             bool hit = false;
             std::string out = s.push(piece, &hit);
             return py::make_tuple(out, hit);
           })
      .def("finish", &StopMatcher::finish);

  // ------------------------------------------------------------ scheduler
  py::class_<SchedOptions>(m, "SchedOptions")
      .def(py::init<>())
      .def_readwrite("max_slots", &SchedOptions::max_slots)
      .def_readwrite("max_queue", &SchedOptions::max_queue)
      .def_readwrite("prefill_chunk", &SchedOptions::prefill_chunk)
      .def_readwrite("row_budget", &SchedOptions::row_budget)
      .def_readwrite("interleave", &SchedOptions::interleave);
  py::class_<Scheduler>(m, "Scheduler")
      .def(py::init<const SchedOptions&>())
      .def("submit", &Scheduler::submit, py::arg("req"), py::arg("prompt_len"), py::arg("max_new"),
           py::arg("preferred_slot") = -1, py::arg("want_rows") = 1)
      .def("cancel", &Scheduler::cancel)
      .def("waiting", &Scheduler::waiting)
      .def("active", &Scheduler::active)
      .def("idle", &Scheduler::idle)
      .def("slot_of", &Scheduler::slot_of)
      .def("set_cached", &Scheduler::set_cached)
      .def("set_rows", &Scheduler::set_rows)
      .def("prefill_done", &Scheduler::prefill_done)
      .def("tokens", &Scheduler::tokens)
      .def("fail", &Scheduler::fail)
      .def("tick", [](Scheduler& s) {
        py::list out;
        static const char* names[] = {"release", "grant", "prefill", "decode", "reject"};
        for (const auto& a : s.tick()) {
          py::dict d;
          d["kind"] = names[a.kind];
          d["req"] = a.req;
          d["slot"] = a.slot;
          d["begin"] = a.begin;
          d["end"] = a.end;
          d["last"] = a.last;
          d["slots"] = a.slots;
          d["rows"] = a.rows;
          out.append(d);
        }
        return out;
      });

  // ------------------------------------------------------------ safetensors
  py::class_<SafetensorsFile>(m, "SafetensorsFile")
      .def(py::init<const std::string&>())
      .def("names", &SafetensorsFile::names)
      .def("has", &SafetensorsFile::has)
      .def("dtype", [](const SafetensorsFile& f, const std::string& n) { return f.info(n).dtype; })
      .def("shape", [](const SafetensorsFile& f, const std::string& n) { return f.info(n).shape; })
      .def("metadata", &SafetensorsFile::metadata)
      .def("view", [](py::object self, const std::string& n) {
        // a zero-copy byte view of the mapped tensor; the file object is kept alive by the view
        const SafetensorsFile& f = self.cast<const SafetensorsFile&>();
        return py::memoryview::from_memory(const_cast<uint8_t*>(f.data(n)), (py::ssize_t)f.nbytes(n), true);
      }, py::keep_alive<0, 1>());
}
