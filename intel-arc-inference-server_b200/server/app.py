"""The OpenAI-compatible server: request handling, continuous batching, streaming.

One serving loop owns the engine.  It takes parsed HTTP requests from the native transport,
submits them to the native scheduler, executes each tick's plan on the engine (at most one
prefill chunk, then one decode / verify step over every generating slot) and streams text as
it is produced: role frame first, content / reasoning / tool-call deltas through the native
incremental parsers, a final frame with ``finish_reason``, an optional usage frame, ``[DONE]``.
Behaviour follows the reference's server (src/server/server.cc:313-354 generate, :359-424
TextRouter, :426-650 generate_tail, :717-769 handle): the first token is emitted before the
first decode step, stop strings are held back until they cannot match, a tool call cut by
``max_tokens`` is dropped, a client that goes away cancels its request, a full queue answers 503.
"""
from __future__ import annotations

import json
import os
import sys
import threading
import time
import uuid
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import numpy as np

from ..native import host as H
from .chat_template import ChatTemplate
from .iface import EngineIface, TokIface


@dataclass
class ServerOptions:
    model_name: str = "b200serve"
    default_max_tokens: int = 512
    max_queue: int = 4
    prefill_chunk: int = 4096
    row_budget: int = 64
    tool_format: str = "qwen_xml"
    chat_format: Optional[object] = None     # server.chat_format.ChatFormat; None: the Qwen format with ``tool_format``
    log_requests: Optional[str] = None
    spec: str = "off"                 # off | lookup | mtp | dflash (drafting is done by the engine adapter)
    spec_max: int = 3
    prefix_split_last: bool = False
    spec_adaptive: bool = True        # per-request draft length from the acceptance seen so far (native DraftLengthPolicy)
    spec_costs: Optional[tuple] = None   # (verify_rows, draft_depth) in plain steps, measured at start-up; None: B200 defaults


@dataclass
class Session:
    http_id: int
    req: object
    prompt_ids: List[int]
    slot: int = -1
    out_ids: List[int] = field(default_factory=list)
    pending: Optional[int] = None      # token produced but not yet fed to the engine
    streamer: object = None
    parser: object = None
    stopper: object = None
    thinking: bool = False
    stream_started: bool = False
    finished: bool = False
    finish_reason: str = "stop"
    content: str = ""
    reasoning: str = ""
    calls: list = field(default_factory=list)
    cached_tokens: int = 0
    rng_seed: int = 0
    rid: str = ""
    created: int = 0
    t0: float = 0.0
    t_first: float = 0.0
    lookup: object = None
    klen: object = None                # DraftLengthPolicy of this request
    copy: object = None                # LookupPolicy (spec = dflash-lookup): copy steps inside a block drafter
    copy_step: bool = False            # the drafts of the step in flight came from the copy proposer


class Server:
    def __init__(self, engine: EngineIface, tok: TokIface, template: ChatTemplate, options: ServerOptions = None,
                 host: str = "127.0.0.1", port: int = 0, prefix=None):
        self.engine, self.tok, self.template = engine, tok, template
        self.o = options or ServerOptions()
        self.http = H.HttpServer(host, port, self.o.max_queue)
        so = H.SchedOptions()
        so.max_slots, so.max_queue = engine.max_seqs, self.o.max_queue
        so.prefill_chunk, so.row_budget = self.o.prefill_chunk, self.o.row_budget
        self.sched = H.Scheduler(so)
        self.sessions: Dict[int, Session] = {}          # by scheduler request id (= http id)
        self.by_slot: Dict[int, Session] = {}
        self.prefix = prefix
        self._stop = False
        self._thread: Optional[threading.Thread] = None

    @property
    def port(self) -> int:
        return self.http.port()

    # ------------------------------------------------------------------ lifecycle
    def start(self):
        self._thread = threading.Thread(target=self.serve_forever, daemon=True)
        self._thread.start()
        return self

    def stop(self):
        self._stop = True
        if self._thread:
            self._thread.join(timeout=10)
        self.http.stop()

    def serve_forever(self):
        while not self._stop:
            busy = not self.sched.idle()
            r = self.http.next(0 if busy else 50)
            while r is not None:
                self._intake(r)
                r = self.http.next(0)
            if not self.sched.idle():
                self._tick()

    # ------------------------------------------------------------------ intake
    def _error(self, http_id, status, message, etype="invalid_request_error"):
        self.http.respond(http_id, status, "application/json", H.error_body(message, etype, status))

    def _intake(self, r):
        hid, path, method = r["id"], r["path"], r["method"]
        if method == "GET" and path in ("/v1/models", "/models"):
            self.http.respond(hid, 200, "application/json",
                              H.models_response(self.o.model_name, int(time.time()), self.engine.max_len))
            return
        if method == "GET" and path in ("/health", "/"):
            self.http.respond(hid, 200, "application/json", '{"status":"ok"}')
            return
        if path not in ("/v1/chat/completions", "/v1/completions"):
            return self._error(hid, 404, f"no route {method} {path}", "not_found_error")
        if method != "POST":
            return self._error(hid, 405, "use POST")
        chat = path == "/v1/chat/completions"
        try:
            req = H.parse_request(r["body"].decode("utf-8", "replace"), chat)
        except ValueError as e:
            return self._error(hid, 400, str(e))
        fmt = self.o.chat_format
        try:
            thinking = False
            if chat:
                messages, kwargs = req.messages, (req.template_kwargs or {})
                if fmt is not None:
                    fmt.check_template_kwargs(kwargs)
                    messages, kwargs = fmt.template_messages(messages), fmt.request_template_kwargs(kwargs)
                prompt = self.template.render(messages, req.tools, True, **kwargs)
                thinking = self.template.thinking_opened(prompt)
                ids = self.tok.encode(prompt)
            else:
                ids = list(req.prompt_ids) or self.tok.encode(req.prompt)
        except Exception as e:  # noqa: BLE001  (template errors are the client's)
            return self._error(hid, 400, f"cannot render the prompt: {e}")
        if not ids:
            return self._error(hid, 400, "the prompt is empty")
        max_new = req.max_tokens or self.o.default_max_tokens
        if len(ids) + 1 > self.engine.max_len:
            return self._error(hid, 400, f"the prompt has {len(ids)} tokens; the context holds {self.engine.max_len}")
        max_new = min(max_new, self.engine.max_len - len(ids))
        s = Session(hid, req, ids, thinking=thinking, rid=("chatcmpl-" if chat else "cmpl-") + uuid.uuid4().hex[:24],
                    created=int(time.time()), t0=time.time())
        s.rng_seed = req.seed if req.has_seed else int.from_bytes(os.urandom(6), "little")
        s.streamer = self.tok.streamer()
        tool_format = fmt.tool_format if fmt is not None else self.o.tool_format
        if chat and fmt is not None and fmt.reasoning_in_output:
            from .chat_format import OutputOpening
            s.parser = OutputOpening(lambda opened, tools=req.tools, tf=tool_format: H.OutputStream(opened, tools, tf))
        else:
            s.parser = H.OutputStream(thinking, req.tools, tool_format) if chat else None
        s.stopper = H.StopMatcher(list(req.stop))
        req.max_tokens = max_new
        preferred = self.prefix.preferred_slot(ids) if self.prefix else -1
        want_rows = 1 + (self.o.spec_max if self.o.spec != "off" else 0)
        if not self.sched.submit(hid, len(ids), max_new, preferred, want_rows):
            return self._error(hid, 503, "server is busy: too many requests waiting", "server_error")
        self.sessions[hid] = s

    # ------------------------------------------------------------------ one scheduler tick
    def _tick(self):
        for s in list(self.sessions.values()):
            if not s.finished and self.http.cancelled(s.http_id):
                self.sched.cancel(s.http_id)
                s.finished = True
                s.finish_reason = "cancelled"
                if s.slot < 0:      # still waiting for a slot: no release action will come for it
                    self.http.close(s.http_id)
                    self.sessions.pop(s.http_id, None)
        for a in self.sched.tick():
            try:
                self._act(a)
            except Exception as e:  # noqa: BLE001   (whatever a request trips over fails that request, not the server)
                slots = [a["slot"]] if "slot" in a else list(a.get("slots", ()))
                for slot in slots:
                    s = self.by_slot.get(slot)
                    if s is not None and not s.finished:
                        self._fail(s, e)

    def _act(self, a):
        if True:
            kind = a["kind"]
            if kind == "release":
                s = self.by_slot.pop(a["slot"], None)
                if s is not None:
                    self._finish(s)
            elif kind == "grant":
                s = self.sessions[a["req"]]
                s.slot = a["slot"]
                self.by_slot[s.slot] = s
                cached = self.prefix.begin(s.slot, s.prompt_ids, self.o.prefix_split_last) if self.prefix else 0
                if not self.prefix:
                    self.engine.reset(s.slot)
                s.cached_tokens = cached
                if cached:
                    self.sched.set_cached(s.slot, cached)
            elif kind == "prefill":
                self._prefill(a)
            elif kind == "decode":
                self._decode(a)

    def _prefill(self, a):
        s = self.by_slot[a["slot"]]
        try:
            tok = self.engine.prefill(s.slot, s.prompt_ids[a["begin"]: a["end"]])
        except Exception as e:  # noqa: BLE001
            self._fail(s, e)
            return self._recover_engine()
        self.sched.prefill_done(s.slot, a["end"])
        if a["last"]:
            if self.prefix:
                self.prefix.after_prefill(s.slot, s.prompt_ids)
            if not s.req.greedy:
                tok = self._sample(s)
            s.t_first = time.time()
            self._emit_token(s, tok)       # the first token goes out before the first decode step

    def _sample(self, s: Session, logits=None, row: int = 0) -> int:
        """The request's next token from its logits row: on the device when the engine has a sampler (only the
        token comes back), else -- or when the kernel leaves the row to the host -- over the logits read back."""
        r = s.req
        seed = (s.rng_seed * 1000003 + len(s.out_ids)) & 0xFFFFFFFFFFFFFFFF
        dev = getattr(self.engine, "sample", None) if logits is None else None
        if dev is not None:
            tok = dev(s.slot, row, 0.0 if r.greedy else r.temperature, r.top_k, r.top_p, seed, r.repetition_penalty,
                      s.prompt_ids + s.out_ids if r.repetition_penalty != 1.0 else ())
            if tok is not None:
                return int(tok)
        if logits is None:
            logits = self.engine.logits(s.slot, row)
        lg = np.array(logits, dtype=np.float32, copy=True)
        if r.repetition_penalty != 1.0:
            H.apply_repetition_penalty(lg, self.engine.vocab_size, s.prompt_ids + s.out_ids, r.repetition_penalty)
        if r.greedy:
            return int(H.argmax_low_tie(lg, self.engine.vocab_size))
        return int(H.sample(lg, self.engine.vocab_size, r.temperature, r.top_k, r.top_p, seed))

    def _decode(self, a):
        rows = {}
        ask = {}       # slot -> (pending, k, temperature, seed): drafts the engine's head makes, all slots in one call
        for slot, n in zip(a["slots"], a["rows"]):
            s = self.by_slot.get(slot)
            if s is None or s.finished or s.pending is None:
                continue
            drafts = self._draft(s, self._draft_budget(s, n - 1)) if n > 1 else []
            if isinstance(drafts, int):       # the engine's draft head is to make this many
                sampled = self.o.spec != "mtp" and not s.req.greedy and s.req.repetition_penalty == 1.0
                seed = (s.rng_seed * 1000003 + len(s.out_ids)) & 0x7FFFFFFF
                ask[slot] = (s.pending, drafts, s.req.temperature if sampled else 0.0, seed)
                drafts = []
            rows[slot] = [s.pending] + drafts
        s_q = {}
        if ask:
            many = getattr(self.engine, "draft_many", None)
            made = many(ask) if many is not None else {sl: self.engine.draft(sl, rq[0], rq[1]) for sl, rq in ask.items()}
            for slot, drafts in made.items():
                rows[slot] = rows[slot] + [int(t) for t in drafts]
                if ask[slot][2] > 0 and hasattr(self.engine, "draft_q"):
                    s_q[slot] = self.engine.draft_q(slot)
        if not rows:
            return
        try:
            res = self.engine.step(rows)
        except Exception as e:  # noqa: BLE001   (a failing step fails its rows, not the server)
            for slot in rows:
                self._fail(self.by_slot[slot], e)
            self._recover_engine()
            return
        for slot, toks in rows.items():
            s = self.by_slot[slot]
            out = res[slot]
            drafts = toks[1:]
            host_rule = (not s.req.greedy) or s.req.repetition_penalty != 1.0
            if drafts and not host_rule:
                acc, nxt = H.accept_greedy(out, drafts)
            elif drafts:
                p_rows = np.stack([self.engine.logits(slot, i) for i in range(len(toks))])
                seed = (s.rng_seed * 1000003 + len(s.out_ids)) & 0xFFFFFFFFFFFFFFFF
                q = s_q.get(slot)
                if q is not None:
                    # the drafts were drawn from a sparse q (a block drafter's candidates): the lossless rule for it
                    acc, nxt = H.accept_sparse(p_rows, q[0][: len(drafts)], q[1][: len(drafts)], drafts,
                                               self.engine.vocab_size, s.req.temperature, s.req.top_k, s.req.top_p, seed)
                else:
                    acc, nxt = H.accept_point_mass(p_rows, drafts, self.engine.vocab_size, s.req.temperature,
                                                   s.req.top_k, s.req.top_p, seed)
            else:
                acc, nxt = 0, (self._sample(s) if host_rule else out[0])
            self._observe_drafts(s, len(drafts), acc)
            if acc < len(drafts):       # rejected rows leave the cache
                self.engine.truncate(slot, self.engine.length(slot) - (len(drafts) - acc))
            emitted = 0
            for t in drafts[:acc]:
                if s.finished:
                    break
                self._emit_token(s, t)
                emitted += 1
            if not s.finished:
                self._emit_token(s, nxt)
                emitted += 1
            if not s.finished:
                self.sched.tokens(slot, emitted, False)

    def _step_costs(self):
        if self.o.spec_costs is not None:
            return H.StepCosts(list(self.o.spec_costs[0]), list(self.o.spec_costs[1]))
        return H.StepCosts()

    def _draft_budget(self, s: Session, k: int) -> int:
        """Drafts this step may spend: the scheduler's row budget, cut by the request's draft-length policy (which
        pauses speculation while drafts keep being rejected and probes now and then)."""
        if k <= 0 or not self.o.spec_adaptive or self.o.spec == "off":
            return k
        if s.klen is None:
            o = H.DraftLengthOptions()
            o.deepest = min(self.o.spec_max, k) if self.o.spec_max > 0 else k
            costs = self._step_costs()
            # copied drafts cost nothing to make; a block drafter makes all its drafts in one pass
            o.costs = costs.free_drafts() if self.o.spec == "lookup" else costs
            s.klen = H.DraftLengthPolicy(o)
        return min(k, s.klen.next()) if self.o.spec != "dflash-lookup" else k

    def _observe_drafts(self, s: Session, proposed: int, accepted: int):
        if s.copy_step:
            s.copy.observe(proposed, accepted)
            s.copy_step = False
        elif s.klen is not None:
            s.klen.observe(proposed, accepted)

    def _lookup(self, s: Session):
        if s.lookup is None:
            s.lookup = H.PromptLookup()
            s.lookup.extend(s.prompt_ids + s.out_ids)
        return s.lookup

    def _recover_engine(self):
        """A step that gave up on a bounded wait latches the engine (its rows were failed above); clearing the latch
        lets the other requests and later ones run."""
        fn = getattr(self.engine, "reset_failure", None)
        if fn is not None:
            try:
                fn()
            except Exception as e:  # noqa: BLE001
                sys.stderr.write(f"engine recovery failed: {e}\n")

    def _draft(self, s: Session, k: int):
        """The step's drafts for ``s`` (a list), or how many the engine's draft head should make (an int)."""
        if k <= 0:
            return []
        room = s.req.max_tokens - len(s.out_ids) - 1
        if room <= 0:
            return []
        if self.o.spec == "dflash-lookup":
            # the copy proposer takes the step while the context repeats an earlier stretch (enter at 8 matching
            # tokens, stay down to 3) and widens its verify as whole copies are accepted; else the block drafter drafts
            if s.copy is None:
                s.copy = H.LookupPolicy()
            lk = self._lookup(s)
            width = s.copy.decide(lk.match(2)[1]) if lk.size() >= 2 else 0
            if width > 0:
                # a lone request may use the step's whole row budget for a wide copy; with company it keeps its share
                cap = self.o.row_budget - 1 if len(self.by_slot) == 1 else k
                drafts = list(lk.propose(min(width - 1, cap, room), 3))
                if drafts:
                    s.copy_step = True
                    return drafts
        if self.o.spec in ("mtp", "dflash", "dflash-lookup") and hasattr(self.engine, "draft"):
            return min(k, room)     # a learned draft head on the engine side
        if self.o.spec not in ("lookup", "dflash-lookup"):
            return []
        return list(self._lookup(s).propose(min(k, room), 2))

    # ------------------------------------------------------------------ output
    def _emit_token(self, s: Session, tok: int):
        """``tok`` was produced: record it, stream its text, decide whether the request ends."""
        r = s.req
        is_eos = tok in self.engine.eos_ids
        n_before = len(s.out_ids)
        if is_eos and not r.ignore_eos and n_before >= r.min_tokens:
            s.pending = None
            return self._end(s, "stop")
        s.out_ids.append(tok)
        if s.lookup is not None:
            s.lookup.append(tok)
        s.pending = tok
        piece = bytes(s.streamer.push(tok)).decode("utf-8", "replace")
        self._emit_text(s, piece, [tok])
        if not s.finished and len(s.out_ids) >= r.max_tokens:
            self._end(s, "length")

    def _emit_text(self, s: Session, piece: str, tok_ids=()):
        if s.finished:
            return
        text, hit = s.stopper.push(piece)
        self._route(s, text, tok_ids)
        if hit:
            self._end(s, "stop", flush=False)

    def _route(self, s: Session, text: str, tok_ids=()):
        deltas = s.parser.push(text) if s.parser is not None else ([{"kind": "content", "text": text}] if text else [])
        self._deliver(s, deltas, tok_ids)

    def _deliver(self, s: Session, deltas, tok_ids=()):
        r = s.req
        if r.stream and not s.stream_started:
            s.stream_started = True
            self.http.begin_stream(s.http_id)
            self.http.send_event(s.http_id, H.stream_frame(r, s.rid, s.created, self.o.model_name, "role"))
        ids = list(tok_ids) if r.return_token_ids else []
        for d in deltas:
            if d["kind"] == "content":
                s.content += d["text"]
            elif d["kind"] == "reasoning":
                s.reasoning += d["text"]
            else:
                s.calls.append(d)
            if r.stream:
                self.http.send_event(s.http_id, H.stream_frame(
                    r, s.rid, s.created, self.o.model_name, d["kind"], d.get("text", ""),
                    d if d["kind"] == "call" else None, d.get("index", 0), "", None, ids))
                ids = []

    def _end(self, s: Session, reason: str, flush: bool = True):
        """Ends generation.  ``flush``: text still held by the detokeniser and the stop matcher is
        output (EOS, length); after a stop string it is not (it lies behind the stop)."""
        if s.finished:
            return
        if flush:
            tail = bytes(s.streamer.finish()).decode("utf-8", "replace")
            text, hit = s.stopper.push(tail)
            if not hit:
                text += s.stopper.finish()
            if text:
                self._route(s, text)
        if s.parser is not None:
            self._deliver(s, s.parser.finish())
        s.finished = True
        s.finish_reason = "tool_calls" if s.calls and reason == "stop" else reason
        if s.slot >= 0:
            self.sched.tokens(s.slot, 0, True)

    def _fail(self, s: Session, exc: Exception):
        sys.stderr.write(f"request {s.rid}: failed: {exc}\n")
        s.finished = True
        s.finish_reason = "error"
        if s.slot >= 0:
            self.sched.fail(s.slot)

    def _finish(self, s: Session):
        """The slot was released: send the tail of the response and log the request."""
        r = s.req
        self.sessions.pop(s.http_id, None)
        usage = (len(s.prompt_ids), len(s.out_ids), s.cached_tokens)
        if self.prefix:
            self.prefix.end(s.slot, s.prompt_ids + s.out_ids)
        if s.finish_reason == "error":
            if s.stream_started:
                self.http.end_stream(s.http_id)
            else:
                self._error(s.http_id, 500, "generation failed", "server_error")
        elif s.finish_reason != "cancelled":
            if r.stream:
                if not s.stream_started:
                    self._deliver(s, [])
                self.http.send_event(s.http_id, H.stream_frame(r, s.rid, s.created, self.o.model_name, "finish", "",
                                                               None, 0, s.finish_reason))
                if r.include_usage:
                    self.http.send_event(s.http_id, H.stream_frame(r, s.rid, s.created, self.o.model_name, "usage", "",
                                                                   None, 0, "", usage))
                self.http.end_stream(s.http_id)
            else:
                body = H.completion_response(r, s.rid, s.created, self.o.model_name, s.content, s.reasoning, s.calls,
                                             s.finish_reason, usage[0], usage[1], usage[2], s.out_ids)
                self.http.respond(s.http_id, 200, "application/json", body)
        else:
            self.http.respond(s.http_id, 499, "application/json", "{}")
        dt = time.time() - s.t0
        n = len(s.out_ids)
        sys.stderr.write(f"gen: {s.rid} prompt {usage[0]} (cached {usage[2]}) -> {n} tokens, {s.finish_reason}, "
                         f"ttft {1e3 * (s.t_first - s.t0 if s.t_first else 0):.1f} ms, "
                         f"{1e3 * dt / max(n, 1):.2f} ms/token\n")
        if self.o.log_requests:
            os.makedirs(self.o.log_requests, exist_ok=True)
            with open(os.path.join(self.o.log_requests, s.rid + ".json"), "w") as f:
                json.dump({"id": s.rid, "prompt_tokens": usage[0], "cached_tokens": usage[2], "completion_tokens": n,
                           "finish_reason": s.finish_reason, "seconds": dt, "content": s.content,
                           "reasoning": s.reasoning, "tool_calls": [c.get("name") for c in s.calls],
                           "output_ids": s.out_ids}, f)
