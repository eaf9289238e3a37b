"""The server over the real engine on a GPU: HTTP in, tokens out, equal to the engine's own greedy decode;
learned-draft speculation and the prefix store switched on must not change a token."""
import http.client
import json

import pytest
import torch

from b200serve.models.config import preset
from b200serve.models.weights import random_weights

pytestmark = pytest.mark.gpu


def post(port, path, body, timeout=60):
    c = http.client.HTTPConnection("127.0.0.1", port, timeout=timeout)
    c.request("POST", path, json.dumps(body), {"Content-Type": "application/json"})
    r = c.getresponse()
    data = r.read().decode()
    c.close()
    return r.status, json.loads(data)


def _cfg():
    import dataclasses
    return dataclasses.replace(preset("small-dense"), mtp_layers=1, vocab=259, name="small-dense-bytes")


@pytest.mark.parametrize("spec,prefix", [("off", False), ("mtp", False), ("lookup", True), ("dflash", True)])
def test_completions_match_engine_greedy(spec, prefix):
    from b200serve.runtime.engine import Engine
    from b200serve.runtime.spec import SpecAdapter
    from b200serve.server.adapter import EngineAdapter
    from b200serve.server.app import Server, ServerOptions
    from b200serve.server.chat_template import ChatTemplate
    from b200serve.server.iface import ByteTok
    from b200serve.server.prefix import PrefixStore
    cfg = _cfg()
    w = random_weights(cfg, device="cuda", seed=8)
    tok = ByteTok()
    text = "The quick brown fox jumps over the lazy dog. " * 9       # ~400 byte tokens: the GEMM prompt pass
    ids = tok.encode(text)
    plain = Engine(w, max_seqs=1, max_len=1024, use_graphs=False)
    want = plain.generate(ids, 20)

    def near_greedy(got):
        """Every produced token is the plain engine's arg-max at its position or within a whisker of it:
        verify rows and cached prefixes run other kernels than single-row decode, they round differently, and
        random-init weights have near-ties."""
        from b200serve.runtime.engine import Row
        plain.reset(0)
        plain.prefill(0, ids)
        lg = plain.logits(1)[0].float()
        for i, t in enumerate(got):
            assert float(lg.max() - lg[t]) < 0.05, (i, t, int(lg.argmax()), float(lg.max() - lg[t]))
            plain.forward_rows([Row(0, plain.seq_len[0], int(t))])
            lg = plain.logits(1)[0].float()
    eng = Engine(w, max_seqs=2, max_len=1024, extra_kv_layers=2)
    adapter = EngineAdapter(eng, eos_ids=())
    if spec in ("mtp", "dflash"):
        adapter = SpecAdapter(adapter, spec, 3)
    store = PrefixStore(eng, host_gb=0.05, block_tokens=64) if prefix else None
    srv = Server(adapter, tok, ChatTemplate(), ServerOptions(model_name=cfg.name, spec=spec, spec_max=3),
                 prefix=store).start()
    try:
        body = {"model": cfg.name, "prompt": text, "max_tokens": 20, "temperature": 0, "ignore_eos": True,
                "return_token_ids": True}
        for attempt in range(2):                   # the second request hits the prefix store when it is on
            status, res = post(srv.port, "/v1/completions", body)
            assert status == 200, res
            got = res["choices"][0].get("token_ids")
            if got is None:
                got = tok.encode(res["choices"][0]["text"])
                assert got == [t for t in want if t >= 3][: len(got)]
            else:
                if got != want:
                    near_greedy(got)
            assert res["usage"]["completion_tokens"] == 20
            if prefix and attempt == 1:
                assert res["usage"]["prompt_tokens_details"]["cached_tokens"] >= 64
        if spec == "dflash":
            # sampled requests: the block drafter draws its drafts from 16 candidates per row and the server applies
            # the sparse-q accept rule; the same seed gives the same text
            texts = []
            for _ in range(2):
                status, res = post(srv.port, "/v1/completions", dict(body, temperature=0.8, seed=5))
                assert status == 200, res
                assert res["usage"]["completion_tokens"] == 20
                texts.append(res["choices"][0].get("token_ids") or res["choices"][0]["text"])
            assert texts[0] == texts[1]
            assert adapter.stats["drafted"] > 0
    finally:
        srv.stop()
