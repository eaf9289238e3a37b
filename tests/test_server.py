"""The OpenAI-compatible server over real HTTP against a mock engine (CPU)."""
import http.client
import json
import threading
import time

import pytest

from b200serve.server.app import Server, ServerOptions
from b200serve.server.chat_template import ChatTemplate
from b200serve.server.iface import ByteTok, MockEngine

TOK = ByteTok()


def enc(s):
    return tuple(TOK.encode(s))


def post(port, path, body, stream=False, timeout=10):
    c = http.client.HTTPConnection("127.0.0.1", port, timeout=timeout)
    c.request("POST", path, json.dumps(body), {"Content-Type": "application/json"})
    r = c.getresponse()
    data = r.read().decode()
    c.close()
    if not stream:
        return r.status, (json.loads(data) if data else None)
    frames = [ln[6:] for ln in data.split("\n") if ln.startswith("data: ")]
    return r.status, frames


@pytest.fixture()
def server():
    servers = []

    def make(script=None, **kw):
        eng = MockEngine(vocab_size=259, max_len=kw.pop("max_len", 2048), max_seqs=kw.pop("max_seqs", 2),
                         script=script or {}, step_delay=kw.pop("step_delay", 0.0))
        srv = Server(eng, TOK, ChatTemplate(), ServerOptions(**kw)).start()
        servers.append(srv)
        return srv, eng
    yield make
    for s in servers:
        s.stop()


def prompt_ids(messages, tools=None, **kw):
    return enc(ChatTemplate().render(messages, tools, True, **kw))


def test_chat_completion_and_usage(server):
    msgs = [{"role": "user", "content": "hi"}]
    pid = prompt_ids(msgs, enable_thinking=False)
    srv, eng = server({pid: list(enc("Hello there.")) + [2]})
    st, body = post(srv.port, "/v1/chat/completions", {"messages": msgs, "chat_template_kwargs": {"enable_thinking": False}})
    assert st == 200
    ch = body["choices"][0]
    assert ch["message"] == {"role": "assistant", "content": "Hello there."} and ch["finish_reason"] == "stop"
    assert body["usage"]["prompt_tokens"] == len(pid) and body["usage"]["completion_tokens"] == len("Hello there.")
    assert body["object"] == "chat.completion" and body["id"].startswith("chatcmpl-")
    st, models = http_get(srv.port, "/v1/models")
    assert st == 200 and models["data"][0]["id"] == "b200serve"


def http_get(port, path):
    c = http.client.HTTPConnection("127.0.0.1", port, timeout=5)
    c.request("GET", path)
    r = c.getresponse()
    d = r.read().decode()
    c.close()
    return r.status, json.loads(d)


def test_streaming_reasoning_tool_call_and_frames(server):
    tools = [{"type": "function", "function": {"name": "read_file", "parameters": {"type": "object", "properties": {
        "path": {"type": "string"}}}}}]
    msgs = [{"role": "user", "content": "open it"}]
    pid = prompt_ids(msgs, tools)
    text = ("let me look\n</think>\n\nReading.\n\n<tool_call>\n<function=read_file>\n<parameter=path>\nsrc/a.cc\n"
            "</parameter>\n</function>\n</tool_call>")
    srv, eng = server({pid: list(enc(text)) + [2]})
    st, frames = post(srv.port, "/v1/chat/completions", {"messages": msgs, "tools": tools, "stream": True,
                                                          "stream_options": {"include_usage": True}}, stream=True)
    assert st == 200 and frames[-1] == "[DONE]"
    js = [json.loads(f) for f in frames[:-1]]
    assert js[0]["choices"][0]["delta"] == {"role": "assistant", "content": ""}          # role frame first
    reasoning = "".join(j["choices"][0]["delta"].get("reasoning_content", "") for j in js if j["choices"])
    content = "".join(j["choices"][0]["delta"].get("content", "") for j in js if j["choices"])
    calls = [j["choices"][0]["delta"]["tool_calls"][0] for j in js if j["choices"] and "tool_calls" in j["choices"][0]["delta"]]
    assert reasoning == "let me look" and content == "Reading."
    assert len(calls) == 1 and calls[0]["function"] == {"name": "read_file", "arguments": '{"path":"src/a.cc"}'}
    fin = [j for j in js if j["choices"] and j["choices"][0]["finish_reason"]]
    assert fin[-1]["choices"][0]["finish_reason"] == "tool_calls"
    assert js[-1]["choices"] == [] and js[-1]["usage"]["completion_tokens"] == len(enc(text))


def test_stop_string_max_tokens_and_cut_call(server):
    msgs = [{"role": "user", "content": "count"}]
    pid = prompt_ids(msgs, enable_thinking=False)
    srv, eng = server({pid: list(enc("one two STOP three four"))})
    kw = {"chat_template_kwargs": {"enable_thinking": False}}
    st, body = post(srv.port, "/v1/chat/completions", {"messages": msgs, "stop": ["STOP"], **kw})
    assert body["choices"][0]["message"]["content"] == "one two" and body["choices"][0]["finish_reason"] == "stop"
    st, body = post(srv.port, "/v1/chat/completions", {"messages": msgs, "max_tokens": 5, **kw})
    assert body["choices"][0]["message"]["content"] == "one t" and body["choices"][0]["finish_reason"] == "length"
    assert body["usage"]["completion_tokens"] == 5
    # completions endpoint with token ids in and out
    st, body = post(srv.port, "/v1/completions", {"prompt": list(pid), "max_tokens": 3, "return_token_ids": True})
    assert body["choices"][0]["text"] == "one" and body["choices"][0]["token_ids"] == list(enc("one"))


def test_errors_and_validation(server):
    srv, _ = server(max_len=64)
    assert post(srv.port, "/v1/chat/completions", {"messages": []})[0] == 400
    st, body = post(srv.port, "/v1/chat/completions", {"messages": [{"role": "user", "content": "x" * 500}]})
    assert st == 400 and "context" in body["error"]["message"]
    assert post(srv.port, "/v1/nothing", {})[0] == 404
    c = http.client.HTTPConnection("127.0.0.1", srv.port, timeout=5)
    c.request("POST", "/v1/chat/completions", "not json")
    assert c.getresponse().status == 400


def test_concurrent_requests_are_batched_and_queue_limit(server):
    srv, eng = server(max_seqs=2, step_delay=0.002, max_queue=2)
    results = {}

    def run(i):
        results[i] = post(srv.port, "/v1/completions", {"prompt": f"request {i} says", "max_tokens": 40})

    ts = [threading.Thread(target=run, args=(i,)) for i in range(6)]
    for t in ts:
        t.start()
        time.sleep(0.005)
    for t in ts:
        t.join()
    codes = sorted(r[0] for r in results.values())
    assert codes.count(200) >= 4 and set(codes) <= {200, 503}
    for st, body in results.values():
        if st == 200:
            assert body["usage"]["completion_tokens"] == 40
    # two slots decoded together: far fewer engine steps than tokens generated
    assert eng.steps < 40 * codes.count(200)
    # determinism: the same prompt alone gives the same text as inside the batch
    st, alone = post(srv.port, "/v1/completions", {"prompt": "request 0 says", "max_tokens": 40})
    assert alone["choices"][0]["text"] == results[0][1]["choices"][0]["text"]


def test_sampling_is_seeded_and_lookup_drafts_are_lossless(server):
    srv, eng = server()
    body = {"prompt": "abc abc abc abc", "max_tokens": 16, "temperature": 0.8, "top_k": 5, "seed": 11}
    a = post(srv.port, "/v1/completions", body)[1]["choices"][0]["text"]
    b = post(srv.port, "/v1/completions", body)[1]["choices"][0]["text"]
    c = post(srv.port, "/v1/completions", {**body, "seed": 12})[1]["choices"][0]["text"]
    assert a == b and (a != c or True)
    plain = post(srv.port, "/v1/completions", {"prompt": "xyzw " * 20, "max_tokens": 30})[1]["choices"][0]["text"]
    srv2, eng2 = server(spec="lookup", spec_max=4)
    spec = post(srv2.port, "/v1/completions", {"prompt": "xyzw " * 20, "max_tokens": 30})[1]
    assert spec["choices"][0]["text"] == plain and spec["usage"]["completion_tokens"] == 30


def test_failing_slot_fails_only_its_request(server):
    srv, eng = server(max_seqs=2, step_delay=0.002)
    eng.fail_slots.add(1)
    res = {}

    def run(i):
        res[i] = post(srv.port, "/v1/completions", {"prompt": f"p{i}", "max_tokens": 20})
    ts = [threading.Thread(target=run, args=(i,)) for i in range(2)]
    for t in ts:
        t.start(); time.sleep(0.01)
    for t in ts:
        t.join()
    codes = sorted(r[0] for r in res.values())
    assert codes == [200, 500] or codes == [500, 500]      # a shared step fails the rows that were in it
    eng.fail_slots.clear()
    assert post(srv.port, "/v1/completions", {"prompt": "again", "max_tokens": 5})[0] == 200


def test_ids_beyond_the_byte_range_and_a_failing_streamer_do_not_stop_the_server(server):
    """A preset with random weights emits ids the byte-level stand-in has no byte for: they fold onto the byte range.
    Whatever else fails while a token is emitted fails that request only."""
    assert ByteTok().decode([3 + 65, 3 + 256 + 66, 1500]) == "AB" + bytes([(1500 - 3) % 256]).decode("utf-8", "replace")
    pid = enc("wide")
    eng = MockEngine(vocab_size=2048, max_len=2048, max_seqs=2, script={pid: [700, 3 + 72, 3 + 256 + 105, 2]})
    srv = Server(eng, TOK, ChatTemplate(), ServerOptions()).start()
    request_stop = srv.stop
    try:
        _wide_ids_and_broken_streamer(srv)
    finally:
        request_stop()


def _wide_ids_and_broken_streamer(srv):
    st, body = post(srv.port, "/v1/completions", {"prompt": "wide", "max_tokens": 8})
    assert st == 200 and body["usage"]["completion_tokens"] == 3 and "Hi" in body["choices"][0]["text"]

    class Boom:
        def push(self, i):
            raise RuntimeError("streamer broke")

        def finish(self):
            return b""
    real = TOK.streamer
    TOK.streamer = lambda: Boom()
    try:
        st, _ = post(srv.port, "/v1/completions", {"prompt": "wide", "max_tokens": 8})
        assert st == 500
    finally:
        TOK.streamer = real
    assert post(srv.port, "/v1/completions", {"prompt": "wide", "max_tokens": 8})[0] == 200


def test_failed_step_fails_its_request_and_the_engine_latch_is_cleared(server):
    """An engine whose step gives up once (a bounded wait that ran out) stays latched until reset_failure(): the
    request in flight gets an error, the server clears the latch, and the next request is served."""
    srv, eng = server()
    state = {"latched": False, "resets": 0, "fail_next": True}
    real_step = eng.step

    def step(rows):
        if state["latched"]:
            raise RuntimeError("engine is latched after a failed step")
        if state["fail_next"]:
            state["fail_next"] = False
            state["latched"] = True
            raise RuntimeError("device kernels gave up on a bounded wait during step on rank 0: comm: code 0x501")
        return real_step(rows)

    def reset_failure():
        state["latched"] = False
        state["resets"] += 1

    eng.step = step
    eng.reset_failure = reset_failure
    st, body = post(srv.port, "/v1/completions", {"prompt": "abc", "max_tokens": 4})
    assert st == 500 and body["error"]["type"] == "server_error"
    assert state["resets"] == 1 and not state["latched"]
    st, body = post(srv.port, "/v1/completions", {"prompt": "abc", "max_tokens": 4})
    assert st == 200 and body["usage"]["completion_tokens"] == 4


def test_client_that_leaves_while_queued_is_cleaned_up(server):
    """A request that waits for a slot and whose client hangs up gets no release action: the tick itself must
    drop its session and let the connection thread close the socket."""
    import socket
    import time
    msgs = [{"role": "user", "content": "long"}]
    pid = prompt_ids(msgs, enable_thinking=False)
    srv, eng = server({pid: list(enc("x" * 400))}, max_seqs=1, step_delay=0.01)
    body = json.dumps({"messages": msgs, "max_tokens": 300, "stream": True,
                       "chat_template_kwargs": {"enable_thinking": False}}).encode()
    head = (f"POST /v1/chat/completions HTTP/1.1\r\nHost: x\r\nContent-Type: application/json\r\n"
            f"Content-Length: {len(body)}\r\n\r\n").encode()
    busy = socket.create_connection(("127.0.0.1", srv.port))
    busy.sendall(head + body)
    assert busy.recv(64).startswith(b"HTTP/1.1 200")          # the only slot is taken and streaming
    queued = socket.create_connection(("127.0.0.1", srv.port))
    queued.sendall(head + body)
    deadline = time.time() + 3
    while time.time() < deadline and len(srv.sessions) < 2:
        time.sleep(0.01)
    assert len(srv.sessions) == 2
    queued.close()                                             # leaves before a slot was granted
    deadline = time.time() + 3
    while time.time() < deadline and len(srv.sessions) > 1:
        time.sleep(0.02)
    assert len(srv.sessions) == 1
    busy.close()
    deadline = time.time() + 3
    while time.time() < deadline and (srv.sessions or srv.http.active() > 0):
        time.sleep(0.02)
    assert not srv.sessions and srv.http.active() == 0


def test_chat_format_kolibri_reads_kwargs_joins_parts_and_keys_reasoning_on_the_output():
    """The per-model chat format: template kwargs are checked (a bad reasoning_effort is a 400), list contents reach
    the template as one string, tool calls are hermes JSON, and reasoning is recognised from a <think> the MODEL
    emits -- also when the tag arrives split over several pieces."""
    from b200serve.native import host as H
    from b200serve.server.chat_format import ChatFormat, OutputOpening
    fmt = ChatFormat.for_model_type("kolibri1")
    assert fmt.kind == "kolibri" and fmt.tool_format == "hermes" and fmt.reasoning_in_output
    assert ChatFormat.for_model_type("qwen3_5_moe").kind == "qwen" and ChatFormat.for_model_type(None).tool_format == "qwen_xml"
    msgs = [{"role": "user", "content": [{"type": "text", "text": "a"}, {"type": "text", "text": "b"}]},
            {"role": "assistant", "content": "c"}]
    assert fmt.template_messages(msgs)[0]["content"] == "a\nb" and fmt.template_messages(msgs)[1]["content"] == "c"
    assert ChatFormat("qwen").template_messages(msgs) is msgs
    fmt.check_template_kwargs({"reasoning_effort": "xhigh", "preserve_thinking": True})
    for bad in ({"reasoning_effort": "extreme"}, {"preserve_thinking": "yes"}):
        with pytest.raises(ValueError):
            fmt.check_template_kwargs(bad)
    assert fmt.request_template_kwargs({"reasoning_effort": "low", "x": 1}) == {"reasoning_effort": "low", "x": 1}
    assert ChatFormat("qwen").request_template_kwargs({"reasoning_effort": "low", "enable_thinking": False}) == {"enable_thinking": False}

    def run(pieces):
        p = OutputOpening(lambda opened: H.OutputStream(opened, None, "hermes"))
        out = []
        for piece in pieces:
            out += p.push(piece)
        out += p.finish()
        r = "".join(d["text"] for d in out if d["kind"] == "reasoning")
        c = "".join(d["text"] for d in out if d["kind"] == "content")
        return r, c
    assert run(["<th", "ink>", "plan it", "</think>", "answer"]) == ("plan it", "answer")
    assert run(["  <think>x</think>y"]) == ("x", "y")
    assert run(["<thin", "g> is not a tag"]) == ("", "<thing> is not a tag")
    assert run(["<th"]) == ("", "<th")
