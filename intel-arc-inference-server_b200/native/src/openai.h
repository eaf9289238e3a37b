// OpenAI-compatible request parsing and response / SSE frame building.
//
// Field surface follows the reference's schema (src/server/openai.h:16-93, openai.cc:200-285):
// max_tokens (or max_completion_tokens), min_tokens, ignore_eos, stream,
// stream_options.include_usage, stop (string or list), return_token_ids, seed, temperature
// (absent = greedy), top_k, top_p, repetition_penalty, tools, chat_template_kwargs,
// reasoning_effort; responses carry reasoning_content, tool_calls, finish_reason in
// {stop, length, tool_calls} and usage.prompt_tokens_details.cached_tokens.  A malformed request
// raises BadRequest, which the server answers with an OpenAI error body and status 400.
#pragma once
#include <stdexcept>
#include <string>
#include <vector>

#include "json.h"
#include "toolcall.h"

namespace b2host {

struct BadRequest : std::runtime_error {
  using std::runtime_error::runtime_error;
};

struct ChatRequest {
  bool chat = true;            // /v1/chat/completions (false: /v1/completions)
  std::string model;
  Json messages;               // chat: the messages array, as given (ordered)
  std::string prompt;          // completions: text prompt
  std::vector<uint32_t> prompt_ids;  // completions: a prompt given as token ids
  Json tools;                  // null when absent
  Json template_kwargs;        // chat_template_kwargs (+ reasoning_effort folded in)
  int max_tokens = 0;          // 0: the server's default
  int min_tokens = 0;
  bool ignore_eos = false;
  bool stream = false;
  bool include_usage = false;
  bool return_token_ids = false;
  std::vector<std::string> stop;
  bool has_seed = false;
  uint64_t seed = 0;
  bool greedy = true;          // temperature absent or 0
  double temperature = 0.0;
  int top_k = 0;
  double top_p = 1.0;
  double repetition_penalty = 1.0;
};

inline std::string error_body(const std::string& message, const std::string& type, int code) {
  Json e = Json::object();
  e["message"] = message;
  e["type"] = type;
  e["param"] = Json();
  e["code"] = code;
  Json j = Json::object();
  j["error"] = e;
  return j.dump();
}

inline ChatRequest parse_request(const std::string& body, bool chat) {
  Json j;
  if (!Json::try_parse(body, j) || !j.is_object()) throw BadRequest("request body is not a JSON object");
  ChatRequest r;
  r.chat = chat;
  auto num = [&](const char* k, double lo, double hi, double dflt) {
    const Json* v = j.find(k);
    if (!v || v->is_null()) return dflt;
    if (!v->is_number()) throw BadRequest(std::string(k) + " must be a number");
    const double d = v->as_double();
    if (d < lo || d > hi) throw BadRequest(std::string(k) + " is out of range");
    return d;
  };
  auto boolean = [&](const char* k, bool dflt) {
    const Json* v = j.find(k);
    if (!v || v->is_null()) return dflt;
    if (!v->is_bool()) throw BadRequest(std::string(k) + " must be a boolean");
    return v->as_bool();
  };
  if (const Json* m = j.find("model"))
    if (m->is_string()) r.model = m->as_string();
  if (chat) {
    const Json* msgs = j.find("messages");
    if (!msgs || !msgs->is_array() || msgs->size() == 0) throw BadRequest("messages must be a non-empty array");
    for (const Json& m : msgs->items()) {
      if (!m.is_object() || !m.contains("role") || !m.at("role").is_string())
        throw BadRequest("every message needs a string role");
    }
    r.messages = *msgs;
  } else {
    const Json* p = j.find("prompt");
    if (!p) throw BadRequest("prompt is required");
    if (p->is_string()) r.prompt = p->as_string();
    else if (p->is_array() && p->size() > 0 && (*p)[0].is_int()) {
      for (const Json& t : p->items()) {
        if (!t.is_int() || t.as_int() < 0) throw BadRequest("prompt token ids must be non-negative integers");
        r.prompt_ids.push_back((uint32_t)t.as_int());
      }
    } else if (p->is_array() && p->size() == 1 && (*p)[0].is_string()) r.prompt = (*p)[0].as_string();
    else throw BadRequest("prompt must be a string or a list of token ids");
  }
  r.max_tokens = (int)num("max_tokens", 1, 1e9, 0);
  if (r.max_tokens == 0) r.max_tokens = (int)num("max_completion_tokens", 1, 1e9, 0);
  r.min_tokens = (int)num("min_tokens", 0, 1e9, 0);
  r.ignore_eos = boolean("ignore_eos", false);
  r.stream = boolean("stream", false);
  r.return_token_ids = boolean("return_token_ids", false);
  if (const Json* so = j.find("stream_options"))
    if (so->is_object())
      if (const Json* iu = so->find("include_usage")) r.include_usage = iu->as_bool();
  if (const Json* st = j.find("stop")) {
    if (st->is_string()) r.stop.push_back(st->as_string());
    else if (st->is_array()) {
      for (const Json& s : st->items()) {
        if (!s.is_string()) throw BadRequest("stop must be a string or a list of strings");
        r.stop.push_back(s.as_string());
      }
    } else if (!st->is_null()) throw BadRequest("stop must be a string or a list of strings");
    for (const auto& s : r.stop)
      if (s.empty()) throw BadRequest("stop strings must not be empty");
  }
  if (const Json* sd = j.find("seed"))
    if (!sd->is_null()) {
      if (!sd->is_int()) throw BadRequest("seed must be an integer");
      r.has_seed = true;
      r.seed = (uint64_t)sd->as_int();
    }
  const Json* temp = j.find("temperature");
  r.temperature = num("temperature", 0.0, 100.0, 0.0);
  r.greedy = !temp || temp->is_null() || r.temperature == 0.0;
  r.top_k = (int)num("top_k", -1, 1e9, 0);
  if (r.top_k < 0) r.top_k = 0;
  r.top_p = num("top_p", 0.0, 1.0, 1.0);
  if (r.top_p <= 0.0) throw BadRequest("top_p must be in (0, 1]");
  r.repetition_penalty = num("repetition_penalty", 0.01, 100.0, 1.0);
  if (const Json* t = j.find("tools")) {
    if (t->is_array() && t->size() > 0) r.tools = *t;
    else if (!t->is_null() && !t->is_array()) throw BadRequest("tools must be an array");
  }
  r.template_kwargs = Json::object();
  if (const Json* kw = j.find("chat_template_kwargs")) {
    if (kw->is_object()) r.template_kwargs = *kw;
    else if (!kw->is_null()) throw BadRequest("chat_template_kwargs must be an object");
  }
  if (const Json* re = j.find("reasoning_effort"))
    if (re->is_string()) r.template_kwargs["reasoning_effort"] = re->as_string();
  return r;
}

struct Usage {
  int prompt_tokens = 0, completion_tokens = 0, cached_tokens = 0;
  Json to_json() const {
    Json u = Json::object();
    u["prompt_tokens"] = prompt_tokens;
    u["completion_tokens"] = completion_tokens;
    u["total_tokens"] = prompt_tokens + completion_tokens;
    Json d = Json::object();
    d["cached_tokens"] = cached_tokens;
    u["prompt_tokens_details"] = d;
    return u;
  }
};

inline Json tool_calls_json(const std::vector<ToolCall>& calls, bool with_index, uint32_t first_index = 0) {
  Json arr = Json::array();
  uint32_t i = first_index;
  for (const ToolCall& c : calls) {
    Json t = Json::object();
    if (with_index) t["index"] = i++;
    t["id"] = c.id;
    t["type"] = "function";
    Json f = Json::object();
    f["name"] = c.name;
    f["arguments"] = c.arguments.dump();  // a string holding the object, keys in the model's order
    t["function"] = f;
    arr.push_back(t);
  }
  return arr;
}

// Whole (non-stream) response of either endpoint.
inline std::string completion_response(const ChatRequest& req, const std::string& id, int64_t created,
                                       const std::string& model, const std::string& content,
                                       const std::string& reasoning, const std::vector<ToolCall>& calls,
                                       const std::string& finish_reason, const Usage& usage,
                                       const std::vector<uint32_t>& token_ids) {
  Json j = Json::object();
  j["id"] = id;
  j["object"] = req.chat ? "chat.completion" : "text_completion";
  j["created"] = created;
  j["model"] = model;
  Json choice = Json::object();
  choice["index"] = 0;
  if (req.chat) {
    Json msg = Json::object();
    msg["role"] = "assistant";
    msg["content"] = (content.empty() && !calls.empty()) ? Json() : Json(content);
    if (!reasoning.empty()) msg["reasoning_content"] = reasoning;
    if (!calls.empty()) msg["tool_calls"] = tool_calls_json(calls, false);
    choice["message"] = msg;
  } else {
    choice["text"] = content;
  }
  if (req.return_token_ids) {
    Json ids = Json::array();
    for (uint32_t t : token_ids) ids.push_back(Json(t));
    choice["token_ids"] = ids;
  }
  choice["finish_reason"] = finish_reason;
  Json choices = Json::array();
  choices.push_back(choice);
  j["choices"] = choices;
  j["usage"] = usage.to_json();
  return j.dump();
}

// One SSE frame (the JSON after "data: ").  kind: 0 role frame, 1 content, 2 reasoning, 3 tool call,
// 4 final frame with finish_reason, 5 usage-only frame.
inline std::string stream_frame(const ChatRequest& req, const std::string& id, int64_t created,
                                const std::string& model, int kind, const std::string& text,
                                const ToolCall* call, uint32_t call_index, const std::string& finish_reason,
                                const Usage* usage, const std::vector<uint32_t>* token_ids) {
  Json j = Json::object();
  j["id"] = id;
  j["object"] = req.chat ? "chat.completion.chunk" : "text_completion";
  j["created"] = created;
  j["model"] = model;
  Json choices = Json::array();
  if (kind != 5) {
    Json choice = Json::object();
    choice["index"] = 0;
    if (req.chat) {
      Json delta = Json::object();
      if (kind == 0) {
        delta["role"] = "assistant";
        delta["content"] = "";
      } else if (kind == 1) delta["content"] = text;
      else if (kind == 2) delta["reasoning_content"] = text;
      else if (kind == 3 && call) delta["tool_calls"] = tool_calls_json({*call}, true, call_index);
      choice["delta"] = delta;
    } else {
      choice["text"] = kind == 1 ? text : "";
    }
    if (token_ids && !token_ids->empty()) {
      Json ids = Json::array();
      for (uint32_t t : *token_ids) ids.push_back(Json(t));
      choice["token_ids"] = ids;
    }
    choice["finish_reason"] = kind == 4 ? Json(finish_reason) : Json();
    choices.push_back(choice);
  }
  j["choices"] = choices;
  if (usage) j["usage"] = usage->to_json();
  return j.dump();
}

inline std::string models_response(const std::string& model, int64_t created, int max_len) {
  Json m = Json::object();
  m["id"] = model;
  m["object"] = "model";
  m["created"] = created;
  m["owned_by"] = "b200serve";
  m["max_model_len"] = max_len;
  Json data = Json::array();
  data.push_back(m);
  Json j = Json::object();
  j["object"] = "list";
  j["data"] = data;
  return j.dump();
}

// Stop strings over streamed text: text that may still become a stop string is held back.
class StopMatcher {
 public:
  explicit StopMatcher(std::vector<std::string> stops) : stops_(std::move(stops)) {}
  // returns the text that is safe to emit; sets hit when a stop string completed (text before it is returned)
  std::string push(const std::string& piece, bool* hit) {
    *hit = false;
    buf_ += piece;
    if (stops_.empty()) {
      std::string out;
      out.swap(buf_);
      return out;
    }
    size_t first = std::string::npos;
    for (const auto& s : stops_) {
      const size_t p = buf_.find(s);
      if (p != std::string::npos && p < first) first = p;
    }
    if (first != std::string::npos) {
      *hit = true;
      std::string out = buf_.substr(0, first);
      buf_.clear();
      return out;
    }
    size_t hold = 0;
    for (const auto& s : stops_) hold = std::max(hold, tag_prefix_suffix(buf_, s));
    std::string out = buf_.substr(0, buf_.size() - hold);
    buf_.erase(0, buf_.size() - hold);
    return out;
  }
  std::string finish() {
    std::string out;
    out.swap(buf_);
    return out;
  }

 private:
  std::vector<std::string> stops_;
  std::string buf_;
};

}  // namespace b2host
