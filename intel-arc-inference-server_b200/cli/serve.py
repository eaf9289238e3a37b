"""``b200-serve``: the OpenAI-compatible server.

    python -m b200serve.cli.serve <snapshot-or-preset> [--spec mtp|dflash|lookup] [--kv-cache int8]
        [--prefill-backend int8] [--parallel tp2|ep8|replica|pp] [--max-num-seqs N] [--max-len auto|L] ...

Start-up order as in the reference (src/cli/b70_serve.cc:929-1498): flags, hardware gate, snapshot
and config, mode selection, memory plan (refusing with the numbers when it cannot fit), load,
engine, adapters, server.
"""
from __future__ import annotations

import signal
import sys

from .flags import ServeFlags, parse


def main(argv=None):
    f = parse(ServeFlags, argv, "b200-serve", __doc__)
    if not f.model:
        raise SystemExit("give a snapshot directory, a hub repo id, or a preset name")
    import torch
    from ..models.config import PRESETS, preset
    from ..runtime.engine import Engine
    from ..runtime.memory_plan import plan
    from ..server.adapter import EngineAdapter
    from ..server.app import Server, ServerOptions
    from ..server.chat_template import ChatTemplate
    from . import common

    par = f.parallel
    if par == "auto" and not torch.cuda.is_available():
        par = "1"           # the hardware gate below says what is missing
    if par == "auto":
        par = common.parallel_auto(common.peek_config(f.model), torch.cuda.device_count() if torch.cuda.is_available() else 0,
                                   torch.cuda.get_device_properties(0).total_memory if torch.cuda.is_available() else 0,
                                   f.max_num_seqs, f.kv_cache, f.int8_head)
        sys.stderr.write(f"placement: --parallel auto -> {par}\n")
    world = int(par[2:]) if par[:2] in ("tp", "ep") and par[2:].isdigit() else (2 if par in ("tp", "ep", "pp") else 1)
    common.hardware_gate(world if par != "replica" else 1)
    if world > 1 or par == "replica":
        from ..parallel.launch import serve_parallel
        return serve_parallel(f, par, world)
    torch.cuda.set_device(0)
    weights = common.load_model(f.model, "cuda", f.seed, f.int8_head)
    cfg = weights.cfg
    backend = {"l0": "bf16", "l0-int8": "int8"}.get(f.prefill_backend, f.prefill_backend)
    mp = plan(cfg, f.max_num_seqs, f.max_len if f.max_len == "auto" else int(f.max_len), f.kv_cache, f.int8_head,
              backend, budget=torch.cuda.get_device_properties(0).total_memory)
    sys.stderr.write(mp.line() + "\n")
    engine = Engine(weights, max_seqs=f.max_num_seqs, max_len=mp.max_len, kv_dtype=f.kv_cache,
                    int8_head=f.int8_head, prefill_backend=backend, num_pages=mp.num_pages)
    tok = common.find_tokenizer(f.model)
    template = ChatTemplate.from_snapshot(f.model) if f.model not in PRESETS else ChatTemplate()
    eos = []
    if hasattr(tok, "token_to_id"):
        eos = [i for i in (tok.token_to_id("<|im_end|>"), tok.token_to_id("<|endoftext|>")) if i is not None and i >= 0]
    spec = f.spec if f.spec != "auto" else ("mtp" if weights.mtp is not None else "off")
    hybrid = cfg.n_gdn_layers > 0
    if hybrid and f.prefix_cache_gb != "0":
        # a reused prefix needs the recurrent state at its end, which is not stored (rejected draft rows are
        # handled: the engine keeps the state from before the last multi-row step and replays the kept rows)
        sys.stderr.write("serve: gated delta-net layers keep a recurrent state per slot: the prefix cache is switched "
                         "off for this model\n")
    adapter = EngineAdapter(engine, eos_ids=eos or (2,))
    if spec in ("mtp", "dflash", "dflash-lookup"):
        from ..runtime.spec import SpecAdapter
        adapter = SpecAdapter(adapter, spec, f.spec_max, f.draft_model, f.draft_vocab, f.draft_vocab_ids,
                              candidate_head_int8=f.candidate_head_int8)
    prefix = None
    if f.prefix_cache_gb != "0" and not hybrid:
        from ..server.prefix import PrefixStore
        prefix = PrefixStore(engine, f.prefix_cache_gb)
    opts = ServerOptions(model_name=cfg.name, log_requests=f.log_requests, spec=spec, spec_max=f.spec_max,
                         tool_format=f.tool_format, prefix_split_last=f.prefix_split_last,
                         chat_format=common.chat_format_for(f.model))
    srv = Server(adapter, tok, template, opts, host=f.host, port=f.port, prefix=prefix)
    sys.stderr.write(f"serving {cfg.name} on http://{f.host}:{srv.port}/v1 (spec {spec}, {f.max_num_seqs} slots, "
                     f"context {mp.max_len})\n")
    signal.signal(signal.SIGINT, lambda *_: setattr(srv, "_stop", True))
    signal.signal(signal.SIGTERM, lambda *_: setattr(srv, "_stop", True))
    try:
        srv.serve_forever()
    finally:
        srv.http.stop()


if __name__ == "__main__":
    main()
