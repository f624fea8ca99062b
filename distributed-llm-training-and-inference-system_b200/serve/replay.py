"""Token-level trace replay: feed given token ids through a served model step by step and write the logits that
are asked for.  Nothing is sampled.  A step lists, per request, its next tokens and the offsets whose logits are
wanted; all entries of a step run as ONE batch through ``InferenceEngine.forward_portions`` — the step function of the
generation path — against the engine's block manager and caches.  Requests are admitted at their first entry, may
skip steps, and give their cache blocks back when a step names them in ``end``.

    llmctl replay trace --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N  < steps.jsonl
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step that wants something, ``DIR/<step>.f32`` holds the logits [wanted, vocab] as little-endian float32 in
entry order; after every step ``done <step>`` is printed.

Reference: reference llmctl/cli/commands/replay.py:9-13 is a stub; the reference has no token-level replay."""
from __future__ import annotations

import json
import sys
from pathlib import Path
from typing import Dict, IO, List, Optional

import numpy as np
import torch

MAX_LIVE_REQUESTS = 4
PAGE_TOKENS = 64


class TraceReplayer:
    def __init__(self, model_dir: str, dtype: str = "bfloat16", max_tokens: int = 4096, device: Optional[str] = None,
                 max_live: int = MAX_LIVE_REQUESTS, page_tokens: int = PAGE_TOKENS):
        from .engine import InferenceEngine
        td = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
        if td == torch.float32:
            # true fp32: no TF32 in any library matrix product
            torch.backends.cuda.matmul.allow_tf32 = False
            torch.backends.cudnn.allow_tf32 = False
            torch.set_float32_matmul_precision("highest")
        blocks = max((int(max_tokens) + page_tokens - 1) // page_tokens, 1)
        # the pool holds exactly what live requests may hold: pages are handed out again as soon as a request ends
        self.engine = InferenceEngine(model_dir, max_batch_size=max_live, max_batch_tokens=max(int(max_tokens), page_tokens),
                                      device=device, kv_block_size=page_tokens, num_kv_blocks=blocks, dtype=td, kv_watermark=0.0,
                                      cuda_graphs=False)
        if not self.engine.ragged:
            raise SystemExit("trace replay needs a model that runs ragged batches")
        self.max_live = max_live
        self.live: Dict[str, List[int]] = {}        # request name -> [engine sequence id, tokens held]
        self._next = 1

    def step(self, obj: dict) -> Optional[torch.Tensor]:
        eng = self.engine
        portions, wanted = [], 0
        for e in obj.get("entries", []):
            name, toks, want = str(e["id"]), [int(t) for t in e["tokens"]], [int(w) for w in e.get("want", [])]
            if not toks:
                continue
            st = self.live.get(name)
            if st is None:
                if len(self.live) >= self.max_live:
                    raise RuntimeError(f"more than {self.max_live} live requests")
                st = self.live[name] = [self._next, 0]
                self._next += 1
            if not eng.kv.allocate(st[0], st[1] + len(toks)):
                raise RuntimeError(f"cache pool exhausted at request {name!r} ({st[1]} + {len(toks)} tokens)")
            portions.append(eng.portion(st[0], toks, st[1], want))
            st[1] += len(toks)
            wanted += len(want)
        logits = eng.forward_portions(portions) if portions else None
        for name in obj.get("end", []):
            st = self.live.pop(str(name), None)
            if st is not None:
                eng.kv.free(st[0])
        return logits if wanted else None


def run(model: str, dtype: str, out: str, max_tokens: int, device: Optional[str] = None, stdin: IO = sys.stdin,
        stdout: IO = sys.stdout) -> int:
    rp = TraceReplayer(model, dtype, max_tokens, device)
    outdir = Path(out)
    outdir.mkdir(parents=True, exist_ok=True)
    for line in stdin:
        line = line.strip()
        if not line:
            continue
        obj = json.loads(line)
        logits = rp.step(obj)
        if logits is not None:
            a = logits.detach().to("cpu", torch.float32).contiguous().numpy().astype("<f4", copy=False)
            tmp = outdir / f".{obj['step']}.part"
            a.tofile(tmp)
            tmp.replace(outdir / f"{obj['step']}.f32")
        elif rp.engine.device.type == "cuda":
            torch.cuda.synchronize(rp.engine.device)
        stdout.write(f"done {obj['step']}\n")
        stdout.flush()
    return 0


def main(argv: Optional[List[str]] = None) -> int:
    import argparse
    ap = argparse.ArgumentParser(prog="trace_run", description="Replay a token-level trace through the serving engine")
    ap.add_argument("--model", required=True, help="directory with config.json and model.safetensors")
    ap.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    ap.add_argument("--out", required=True, help="directory for <step>.f32 logit files")
    ap.add_argument("--max-tokens", type=int, required=True, help="cache pool size in tokens (rounded up to pages of 64)")
    ap.add_argument("--device", default=None)
    a = ap.parse_args(argv)
    return run(a.model, a.dtype, a.out, a.max_tokens, a.device)
