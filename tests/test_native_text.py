"""Native text path: tokenizer parity with the `tokenizers` library, streamer, tool-call stream
parser (split invariance), stop strings, OpenAI schema, HTTP transport.  CPU only."""
import json
import os
import random
import socket
import threading
import time

import pytest

from b200serve.native import host as H

PAT = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+"
       r"|\s+(?!\S)|\s+")

CORPUS = [
    "Hello world!  It's a test.\n\n  def f(x):\n\treturn x+1  \n",
    "naïve café 123456 — 日本語のテキスト 😀 end",
    "<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\n",
    "a  b   c\n \n  d", "x'S y'LL z'd", "   ", "tab\t\ttab \n", "", "\n", " \n\n\n ", "1 2 33 4444",
    "The quick brown fox jumps over the lazy dog. " * 3,
    "for (int i = 0; i < n; ++i) { a[i] += b[i] * 2; }  // loop\r\n",
    "مرحبا بالعالم Привет мир γειά σου κόσμε", "emoji 👩‍👩‍👧‍👦 zwj", "ends with space ", "ＦＵＬＬ width １２３",
]


@pytest.fixture(scope="module")
def trained(tmp_path_factory):
    tk = pytest.importorskip("tokenizers")
    from tokenizers import Regex, Tokenizer, decoders, models, pre_tokenizers, trainers
    tok = Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.Sequence([
        pre_tokenizers.Split(Regex(PAT), behavior="isolated"),
        pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    tok.decoder = decoders.ByteLevel()
    rnd = random.Random(0)
    words = ["alpha", "beta", "gamma", "tensor", "core", "memory", "page", "token", "the", "of", "and", "kv",
             "cache", "def", "return", "int", "float", "日本", "語", "café", "naïve", "123", "42", "{", "}", "(", ")",
             "==", "+=", "\n", "  ", "\t", "'s", "'ll", "!", "?", ".", ","]
    text = [" ".join(rnd.choice(words) for _ in range(rnd.randrange(3, 30))) for _ in range(400)] + CORPUS
    trainer = trainers.BpeTrainer(vocab_size=1200, special_tokens=["<|endoftext|>", "<|im_start|>", "<|im_end|>"],
                                  initial_alphabet=pre_tokenizers.ByteLevel.alphabet())
    tok.train_from_iterator(text, trainer)
    path = str(tmp_path_factory.mktemp("tok") / "tokenizer.json")
    tok.save(path)
    return tok, H.Tokenizer.from_file(path), text


def test_tokenizer_matches_reference_library(trained):
    ref, mine, text = trained
    for s in CORPUS + text[:200]:
        assert mine.encode(s) == ref.encode(s, add_special_tokens=False).ids, repr(s)
        assert mine.decode(mine.encode(s)).decode("utf-8") == s


def test_tokenizer_random_strings(trained):
    ref, mine, _ = trained
    rnd = random.Random(1)
    alphabet = "ab c\n\t1'.,é日😀 -_(){}" + "\r"
    for _ in range(300):
        s = "".join(rnd.choice(alphabet) for _ in range(rnd.randrange(0, 40)))
        assert mine.encode(s) == ref.encode(s, add_special_tokens=False).ids, repr(s)


# the reference checkout, when there is one beside this repository (or where REFERENCE_DIR points)
REF_TOK_DIR = os.path.join(os.environ.get("REFERENCE_DIR") or os.path.join(
    os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference"), "tests")


def test_tokenizer_parity_over_the_reference_corpus(tmp_path):
    """Every line of the reference's tokenizer parity corpus (10,240 cases: prose, code, numbers, scripts, whitespace
    runs) through both libraries, with a vocabulary trained on part of that corpus and the pre-tokeniser pattern
    read from the reference's own tokenizer file.  (The reference's expected ids belong to a full vocabulary that is
    not available here, so the library it wraps decides what is right.)"""
    import json
    corpus = os.path.join(REF_TOK_DIR, "tokenizer", "corpus.txt")
    tokjson = os.path.join(REF_TOK_DIR, "model", "qwen4exp-q38tok", "tokenizer.json")
    if not (os.path.exists(corpus) and os.path.exists(tokjson)):
        pytest.skip("the reference's tokenizer corpus is not on this machine")
    pytest.importorskip("tokenizers")
    from tokenizers import Regex, Tokenizer, decoders, models, pre_tokenizers, trainers
    with open(tokjson) as f:
        pat = json.load(f)["pre_tokenizer"]["pretokenizers"][0]["pattern"]["Regex"]
    with open(corpus, encoding="utf-8") as f:
        lines = f.read().split("\n")
    tok = Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.Sequence([
        pre_tokenizers.Split(Regex(pat), behavior="isolated"),
        pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    tok.decoder = decoders.ByteLevel()
    trainer = trainers.BpeTrainer(vocab_size=4000, special_tokens=["<|endoftext|>", "<|im_start|>", "<|im_end|>"],
                                  initial_alphabet=pre_tokenizers.ByteLevel.alphabet())
    tok.train_from_iterator(lines[::3], trainer)
    path = str(tmp_path / "tokenizer.json")
    tok.save(path)
    mine = H.Tokenizer.from_file(path)
    bad = []
    for i, s in enumerate(lines):
        want = tok.encode(s, add_special_tokens=False).ids
        got = mine.encode(s)
        if got != want:
            bad.append((i, s[:80]))
            if len(bad) > 5:
                break
    assert not bad, bad
    # the whole file as one text too: line ends meet the whitespace rules of the pattern
    blob = "\n".join(lines[:2000])
    assert mine.encode(blob) == tok.encode(blob, add_special_tokens=False).ids
    assert mine.decode(mine.encode(blob)).decode("utf-8") == blob


def test_special_tokens_and_streamer(trained):
    _, mine, _ = trained
    ids = mine.encode("<|im_start|>héllo 😀<|im_end|>")
    assert ids[0] == mine.token_to_id("<|im_start|>") and ids[-1] == mine.token_to_id("<|im_end|>")
    assert mine.is_special(ids[0])
    st = H.Streamer(mine, True)
    pieces = [st.push(i) for i in ids] + [st.finish()]
    for p in pieces:
        p.decode("utf-8")                      # every streamed piece is whole characters
    assert b"".join(pieces).decode() == "héllo 😀"
    assert mine.decode(ids, True).decode() == "héllo 😀"


# ----------------------------------------------------------------------------- tool calls
TOOLS = [{"type": "function", "function": {"name": "read_file", "parameters": {"type": "object", "properties": {
    "path": {"type": "string"}, "limit": {"type": "integer"}, "opts": {"type": "object"},
    "note": {"type": ["string", "null"]}}}}}]

XML = ("thinking about it\n</think>\n\nI'll read it.\n\n<tool_call>\n<function=read_file>\n<parameter=path>\n/tmp/a b.txt\n"
       "</parameter>\n<parameter=limit>\n20\n</parameter>\n<parameter=opts>\n{\"z\": 1, \"a\": [true, null]}\n</parameter>\n"
       "<parameter=note>\n123\n</parameter>\n</function>\n</tool_call>\n<tool_call>\n<function=read_file>\n<parameter=path>\nx\n"
       "</parameter>\n</function>\n</tool_call>")


def test_parse_output_xml_types_and_order():
    po = H.parse_output(XML, True, TOOLS)
    assert po["reasoning"] == "thinking about it"
    assert po["content"] == "I'll read it."
    c0, c1 = po["tool_calls"]
    assert c0["name"] == "read_file"
    assert c0["arguments"] == {"path": "/tmp/a b.txt", "limit": 20, "opts": {"z": 1, "a": [True, None]}, "note": "123"}
    assert list(c0["arguments"]) == ["path", "limit", "opts", "note"]            # the model's key order
    assert c0["arguments_json"].startswith('{"path":"/tmp/a b.txt","limit":20,"opts":{"z":1')
    assert c0["id"].startswith("call_") and len(c0["id"]) == 29 and c0["id"] != c1["id"]
    assert c1["arguments"] == {"path": "x"}


def _fold(deltas, acc):
    for d in deltas:
        if d["kind"] == "call":
            acc["calls"].append((d["name"], d["arguments_json"], d["index"]))
        else:
            acc[d["kind"]] += d["text"]


def test_stream_split_invariance():
    whole = {"reasoning": "", "content": "", "calls": []}
    s = H.OutputStream(True, TOOLS, "qwen_xml", 7)
    _fold(s.push(XML), whole); _fold(s.finish(), whole)
    rnd = random.Random(3)
    for _ in range(60):
        acc = {"reasoning": "", "content": "", "calls": []}
        s = H.OutputStream(True, TOOLS, "qwen_xml", 7)
        pos = 0
        while pos < len(XML):
            n = rnd.randrange(1, 9)
            _fold(s.push(XML[pos: pos + n]), acc)
            pos += n
        _fold(s.finish(), acc)
        assert acc == whole
    assert len(whole["calls"]) == 2 and [c[2] for c in whole["calls"]] == [0, 1]


def test_cut_call_is_dropped_and_no_tools_means_text():
    cut = "ok\n<tool_call>\n<function=read_file>\n<parameter=path>\n/tmp/x\n</parameter>\n<parameter=limit>\n5"
    po = H.parse_output(cut, False, TOOLS)
    assert po["content"] == "ok" and po["tool_calls"] == []
    closed = cut + "\n</parameter>\n</function>"
    assert len(H.parse_output(closed, False, TOOLS)["tool_calls"]) == 1         # </function> had closed: complete
    txt = "a <tool_call> b"
    assert H.parse_output(txt, False, None)["content"] == txt                   # no tools: tags are text


def test_hermes_calls_and_raw_newlines():
    body = '<tool_call>\n{"name": "read_file", "arguments": {"path": "line1\nline2\tend", "limit": "7"}}\n</tool_call>'
    po = H.parse_output(body, False, TOOLS, "hermes")
    (c,) = po["tool_calls"]
    assert c["arguments"] == {"path": "line1\nline2\tend", "limit": "7"}
    changed, out = H.escape_raw_controls('{"a": "x\ny", "b": 1}')
    assert changed and json.loads(out) == {"a": "x\ny", "b": 1}
    assert H.escape_raw_controls('{"a": "cut')[0] is False
    bad = "<tool_call>\nnot json\n</tool_call> tail"
    assert "not json" in H.parse_output(bad, False, TOOLS, "hermes")["content"]
    assert H.tag_prefix_suffix("abc<tool", "<tool_call>") == 5


def test_stop_matcher_holds_back_partial_stop():
    m = H.StopMatcher(["END", "\n\nUser:"])
    out, hit = m.push("hello E")
    assert (out, hit) == ("hello ", False)
    out, hit = m.push("N")
    assert (out, hit) == ("", False)
    out, hit = m.push("Dless")
    assert (out, hit) == ("", True)
    m = H.StopMatcher(["END"])
    out, hit = m.push("an EN")
    assert out == "an "
    out2, hit = m.push("x")
    assert (out2, hit) == ("ENx", False)


# ----------------------------------------------------------------------------- OpenAI schema
def test_parse_request_fields_and_errors():
    body = json.dumps({"model": "m", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 5, "stream": True,
                       "stream_options": {"include_usage": True}, "stop": "x", "seed": 3, "temperature": 0.7,
                       "top_k": 20, "top_p": 0.9, "repetition_penalty": 1.1, "min_tokens": 2, "ignore_eos": True,
                       "return_token_ids": True, "tools": TOOLS, "chat_template_kwargs": {"enable_thinking": False},
                       "reasoning_effort": "low"})
    r = H.parse_request(body, True)
    assert (r.max_tokens, r.stream, r.include_usage, r.stop, r.seed, r.greedy) == (5, True, True, ["x"], 3, False)
    assert (r.top_k, r.min_tokens, r.ignore_eos, r.return_token_ids) == (20, 2, True, True)
    assert r.template_kwargs == {"enable_thinking": False, "reasoning_effort": "low"}
    assert r.tools[0]["function"]["name"] == "read_file"
    assert H.parse_request(json.dumps({"messages": [{"role": "user", "content": "x"}]}), True).greedy
    for bad in ("nope", json.dumps({"messages": []}), json.dumps({"messages": [{"content": "x"}]}),
                json.dumps({"messages": [{"role": "user"}], "top_p": 0}),
                json.dumps({"messages": [{"role": "user"}], "stop": [""]}),
                json.dumps({"messages": [{"role": "user"}], "max_tokens": "many"})):
        with pytest.raises(ValueError):
            H.parse_request(bad, True)
    r = H.parse_request(json.dumps({"prompt": [1, 2, 3]}), False)
    assert r.prompt_ids == [1, 2, 3]
    e = json.loads(H.error_body("bad", "invalid_request_error", 400))
    assert e["error"]["message"] == "bad" and e["error"]["code"] == 400


def test_response_and_frames():
    r = H.parse_request(json.dumps({"messages": [{"role": "user", "content": "x"}], "return_token_ids": True}), True)
    call = {"id": "call_x", "name": "f", "arguments": {"b": 1, "a": 2}}
    full = json.loads(H.completion_response(r, "id1", 5, "m", "", "why", [call], "tool_calls", 10, 4, 8, [7, 8]))
    ch = full["choices"][0]
    assert ch["message"]["content"] is None and ch["message"]["reasoning_content"] == "why"
    assert ch["message"]["tool_calls"][0]["function"]["arguments"] == '{"b":1,"a":2}'
    assert ch["finish_reason"] == "tool_calls" and ch["token_ids"] == [7, 8]
    assert full["usage"] == {"prompt_tokens": 10, "completion_tokens": 4, "total_tokens": 14,
                             "prompt_tokens_details": {"cached_tokens": 8}}
    role = json.loads(H.stream_frame(r, "id1", 5, "m", "role"))
    assert role["choices"][0]["delta"] == {"role": "assistant", "content": ""} and role["choices"][0]["finish_reason"] is None
    c = json.loads(H.stream_frame(r, "id1", 5, "m", "call", "", call, 1))
    assert c["choices"][0]["delta"]["tool_calls"][0]["index"] == 1
    fin = json.loads(H.stream_frame(r, "id1", 5, "m", "finish", "", None, 0, "stop"))
    assert fin["choices"][0]["finish_reason"] == "stop" and fin["choices"][0]["delta"] == {}
    us = json.loads(H.stream_frame(r, "id1", 5, "m", "usage", "", None, 0, "", (3, 2, 1)))
    assert us["choices"] == [] and us["usage"]["total_tokens"] == 5


# ----------------------------------------------------------------------------- HTTP transport
def _http(port, method, path, body=b"", read_all=True):
    s = socket.create_connection(("127.0.0.1", port), timeout=5)
    s.sendall(f"{method} {path} HTTP/1.1\r\nHost: x\r\nContent-Length: {len(body)}\r\n\r\n".encode() + body)
    if not read_all:
        return s
    data = b""
    while True:
        chunk = s.recv(65536)
        if not chunk:
            break
        data += chunk
    s.close()
    return data


def test_http_plain_stream_and_queue_limit():
    srv = H.HttpServer("127.0.0.1", 0, 2)
    port = srv.port()
    results = {}

    def client(name, body):
        results[name] = _http(port, "POST", "/v1/chat/completions", body)

    t1 = threading.Thread(target=client, args=("a", b'{"n":1}')); t1.start()
    r = None
    for _ in range(100):
        r = srv.next(50)
        if r is not None:
            break
    assert r["method"] == "POST" and r["path"] == "/v1/chat/completions" and r["body"] == b'{"n":1}'
    assert srv.respond(r["id"], 200, "application/json", '{"ok":true}')
    t1.join()
    assert results["a"].startswith(b"HTTP/1.1 200 OK") and results["a"].endswith(b'{"ok":true}')
    # stream
    t2 = threading.Thread(target=client, args=("b", b"{}")); t2.start()
    r = srv.next(2000)
    assert srv.begin_stream(r["id"]) and srv.send_event(r["id"], '{"x":1}') and srv.end_stream(r["id"])
    t2.join()
    assert b"text/event-stream" in results["b"] and b'data: {"x":1}\n\n' in results["b"]
    assert results["b"].rstrip().endswith(b"0") and b"data: [DONE]" in results["b"]
    # a third waiting request beyond the bound of two is refused with 503
    socks = [_http(port, "POST", "/v1/completions", b"{}", read_all=False) for _ in range(2)]
    for _ in range(100):
        if srv.waiting() == 2:
            break
        time.sleep(0.01)
    assert _http(port, "POST", "/v1/completions", b"{}").startswith(b"HTTP/1.1 503")
    # a client that goes away is reported as cancelled
    r = srv.next(1000)
    socks[0].close(); socks[1].close()          # whichever of the two it is, its client is gone
    for _ in range(100):
        if srv.cancelled(r["id"]):
            break
        time.sleep(0.02)
    assert srv.cancelled(r["id"])
    srv.respond(r["id"], 200, "text/plain", "late")
    r2 = srv.next(1000)
    srv.respond(r2["id"], 404, "application/json", "{}")
    srv.stop()
