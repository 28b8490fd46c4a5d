"""Trace replay: feed given token ids through a model step by step and write the logits of chosen positions.

The runner samples nothing and owns no model code: it resolves the model class from ``config.json`` through the
registry, opens request batches with the engine's token-at-a-time stream (`B200Engine.begin_stream`: left-padded
static batch, prefill, decode state and cache) and advances them with `EngineStream.step(feed=...)` — the
CUDA-graph-replayed decode step that `generate` uses — reading the logits the step leaves on the device.

Input, one JSON object per line on standard input::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

`entries` bring each request's next tokens; `want` are the places among them whose logits are written, as
little-endian float32 ``[wanted, vocab]`` in ``<out>/<step>.f32``, in the order of the entries.  Requests that first
appear in a step form one batch; later steps continue them token by token; `end` lists the requests whose cache and
state are given back after the step.  After every step the runner prints ``done <step>``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Any, Dict, List, Optional

PAD_ID = 0


class Batch:
    """One live request batch: its stream and which row each request occupies."""

    def __init__(self, stream: Any, rows: Dict[str, int]):
        self.stream, self.rows = stream, rows
        self.live = set(rows)


def _open_batch(engine: Any, entries: List[Dict[str, Any]], max_tokens: int) -> Any:
    import torch

    B = len(entries)
    S = max(len(e["tokens"]) for e in entries)
    ids = torch.full((B, S), PAD_ID, dtype=torch.long)
    mask = torch.zeros((B, S), dtype=torch.int32)
    want_rows: List[int] = []
    for b, e in enumerate(entries):
        n = len(e["tokens"])
        ids[b, S - n:] = torch.tensor(e["tokens"], dtype=torch.long)
        mask[b, S - n:] = 1
        want_rows += [b * S + (S - n) + int(w) for w in e.get("want", [])]
    # slots of the batch: the longest prompt plus what the token budget leaves for decoding, one to spare; never more than the
    # model has positions for
    max_len = S + max(int(max_tokens) - S, 1) + 1
    limit = getattr(engine, "position_limit", None)
    if limit is not None and S <= limit:
        max_len = min(max_len, int(limit) + 1)            # the last slot holds a token that is never fed back
    while (B, max_len) in engine._decode_states:          # a live batch of the same shape keeps its own state
        max_len += 1
    dev = engine.device
    stream = engine.begin_stream(ids.to(dev), mask.to(dev), max_length=max_len, do_sample=False, pad_token_id=PAD_ID,
                                 eos_token_id=-1, logit_rows=torch.tensor(want_rows, dtype=torch.long))
    return stream


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--out", required=True, help="folder for the <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, default=4096,
                    help="most tokens live requests hold at any time; bounds the cache length of a batch")
    a = ap.parse_args(argv)

    from .models import registry
    from .ops import _lib

    arch, _, _ = registry.resolve(a.model)
    if a.dtype not in registry.gpu_dtypes(arch):
        print(f"the {arch} engine does not run in {a.dtype}", file=sys.stderr)
        return 3
    subset = registry.kernel_subset(arch)
    if subset:
        _lib.use_subset(subset)

    import torch

    if not torch.cuda.is_available():
        print("trace_run needs a CUDA device", file=sys.stderr)
        return 2
    _lib.lib()                                             # builds the native library at the first call in a fresh tree
    model = registry.load_pretrained(a.model, dtype=getattr(torch, a.dtype), device="cuda")
    engine = model._engine_for(model.params)
    os.makedirs(a.out, exist_ok=True)
    batches: List[Batch] = []
    where: Dict[str, Batch] = {}

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        entries = step.get("entries", [])
        results: Dict[str, Any] = {}
        fresh = [e for e in entries if e["id"] not in where]
        if fresh:
            stream = _open_batch(engine, fresh, a.max_tokens)
            batch = Batch(stream, {e["id"]: b for b, e in enumerate(fresh)})
            batches.append(batch)
            got, at = stream.prompt_logits(), 0
            for e in fresh:
                where[e["id"]] = batch
                n = len(e.get("want", []))
                results[e["id"]] = got[at:at + n]
                at += n
        for batch in batches:
            mine = [e for e in entries if where.get(e["id"]) is batch and e not in fresh]
            if not mine:
                continue
            count = max(len(e["tokens"]) for e in mine)
            rows_out: Dict[str, List[Any]] = {e["id"]: [] for e in mine}
            for j in range(count):
                feed = torch.full((batch.stream.st.B,), PAD_ID, dtype=torch.int32).pin_memory()
                for e in mine:
                    if j < len(e["tokens"]):
                        feed[batch.rows[e["id"]]] = int(e["tokens"][j])
                batch.stream.step(feed)
                logits = batch.stream.logits()
                for e in mine:
                    if j in e.get("want", []):
                        rows_out[e["id"]].append(logits[batch.rows[e["id"]]].clone())
            for e in mine:
                v = engine.config.vocab_size
                results[e["id"]] = torch.stack(rows_out[e["id"]]) if rows_out[e["id"]] else \
                    torch.empty((0, v), dtype=torch.float32, device=engine.device)
        parts = [results[e["id"]] for e in entries if e["id"] in results and results[e["id"]].shape[0] > 0]
        if parts:
            out = torch.cat([p.float() for p in parts], 0).cpu().numpy().astype("<f4")
            tmp = os.path.join(a.out, f".{step['step']}.part")
            out.tofile(tmp)
            os.replace(tmp, os.path.join(a.out, f"{step['step']}.f32"))
        for rid in step.get("end", []):
            batch = where.pop(rid, None)
            if batch is not None:
                batch.live.discard(rid)
                if not batch.live:
                    batch.stream.close()
                    batches.remove(batch)
        torch.cuda.synchronize()
        print(f"done {step['step']}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
