"""Trace replay: feeds given token ids through a model step by step and writes the logits of the
positions a step asks for — no sampling.  It drives the serving path itself: requests are `Req`s in
a `ScheduleBatch`, a step's entries are ONE batch prepared by `prepare_for_extend` (portions of
prompts beside single tokens of running requests, i.e. a mixed chunked-prefill batch) or, when every
entry is one token of a running request, by `prepare_for_decode` (which replays the captured decode
CUDA graphs); the batch runs through `TpModelWorker.forward_batch_generation`, the KV runs come from
`TokenToKVPoolAllocator` and the request / recurrent-state slots from `ReqToTokenPool`, and a
finished request gives both back.

    python -m semi_pd_b200.trace_runner --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

stdin, one JSON object per line:  {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}],
"end": ["a"]}.  For a step with wanted positions, OUT/<step>.f32 holds their logits ([wanted, vocab]
little-endian fp32, in entry order); after every step `done <step>` is printed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Dict, List

import numpy as np
import torch


def build_worker(model: str, dtype: str, max_tokens: int, max_requests: int, cuda_graph: bool):
    from .configs import ServerArgs, get_model_config
    from .memory_pool import DEFAULT_RUN_LEN
    from .tp_worker import TpModelWorker

    # live requests hold their tokens in whole runs of the allocator; the budget counts 64-token units
    pool_tokens = max_tokens + max_requests * max(DEFAULT_RUN_LEN - 64, 0)
    pool_tokens = -(-pool_tokens // DEFAULT_RUN_LEN) * DEFAULT_RUN_LEN
    ctx = max_tokens + 64
    cfg = get_model_config(model)
    if ctx > cfg.max_position_embeddings:  # position tables are built for the longest request the pool can hold
        cfg = get_model_config(model, max_position_embeddings=ctx)
    sa = ServerArgs(model_path=model, dtype=dtype, load_format="auto", max_total_tokens=pool_tokens,
                    # the request pool adds one spare slot to what is asked for
                    max_running_requests=max(max_requests - 1, 1), context_length=ctx,
                    disable_cuda_graph=not cuda_graph, cuda_graph_bs=[b for b in (1, 2, 4, 8) if b <= max_requests])
    return TpModelWorker(sa, gpu_id=0, tp_rank=0, model_config=cfg)


class TraceSession:
    def __init__(self, worker):
        from .schedule_batch import ScheduleBatch
        self.worker = worker
        self.ScheduleBatch = ScheduleBatch
        self.req_to_token_pool, self.allocator = worker.get_memory_pool()
        self.device = worker.device
        self.reqs: Dict[str, object] = {}

    def _req(self, rid: str):
        from .schedule_batch import Req, SamplingParams
        r = self.reqs.get(rid)
        if r is None:
            r = self.reqs[rid] = Req(rid, [], SamplingParams(max_new_tokens=1 << 30))
        return r

    def step(self, entries: List[dict]) -> torch.Tensor:
        """Run one step; → fp32 logits [wanted, vocab] (entry order, then `want` order)."""
        reqs, news = [], []
        for e in entries:
            if not e["tokens"]:
                continue
            reqs.append(self._req(e["id"]))
            news.append(e)
        if not reqs:
            return torch.empty((0, self.worker.model_config.vocab_size))
        batch = self.ScheduleBatch.init_new(reqs, self.req_to_token_pool, self.allocator, self.device)
        decode = all(len(e["tokens"]) == 1 and len(r.origin_input_ids) > 0 for r, e in zip(reqs, news))
        if decode:
            lens = [len(r.origin_input_ids) for r in reqs]
            batch.req_pool_indices = torch.tensor([r.req_pool_idx for r in reqs], dtype=torch.int64, device=self.device)
            batch.seq_lens = torch.tensor(lens, dtype=torch.int64, device=self.device)
            batch.seq_lens_host = lens
            batch.seq_lens_sum = sum(lens)
            batch.output_ids = torch.tensor([e["tokens"][0] for e in news], dtype=torch.int64, device=self.device)
            batch.prepare_for_decode()
            rows = [i for i, e in enumerate(news) for _ in e["want"]]
        else:
            rows, start = [], 0
            for r, e in zip(reqs, news):
                r.prefix_indices = [0] * len(r.origin_input_ids)
                r.fill_ids = r.origin_input_ids + list(e["tokens"])
                r.extend_input_len = len(e["tokens"])
                rows += [start + int(p) for p in e["want"]]
                start += len(e["tokens"])
            batch.extend_logit_rows = torch.tensor(rows, dtype=torch.int64, device=self.device)
            batch.prepare_for_extend()
        for r, e in zip(reqs, news):
            r.origin_input_ids = r.origin_input_ids + list(e["tokens"])
        out, _ = self.worker.forward_batch_generation(batch.get_model_worker_batch(), skip_sample=True)
        logits = out.next_token_logits
        if decode:
            logits = logits[torch.tensor(rows, dtype=torch.int64, device=self.device)] if rows else logits[:0]
        return logits.float()

    def end(self, rids: List[str]):
        for rid in rids:
            r = self.reqs.pop(rid, None)
            if r is None or r.req_pool_idx is None:
                continue
            self.allocator.free_req(r.req_pool_idx)
            self.req_to_token_pool.free(r.req_pool_idx)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Replay a token trace through the serving path and write logits.")
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float16", "float32"])
    ap.add_argument("--out", required=True)
    ap.add_argument("--max-tokens", type=int, required=True, help="tokens live requests hold at any time (64-token units)")
    ap.add_argument("--max-requests", type=int, default=4, help="live requests at any time")
    ap.add_argument("--disable-cuda-graph", action="store_true")
    a = ap.parse_args(argv)
    os.makedirs(a.out, exist_ok=True)
    worker = build_worker(a.model, a.dtype, a.max_tokens, a.max_requests, not a.disable_cuda_graph)
    session = TraceSession(worker)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        msg = json.loads(line)
        logits = session.step(msg.get("entries", []))
        if logits.shape[0]:
            arr = logits.cpu().numpy().astype("<f4", copy=False)
            tmp = os.path.join(a.out, f".{msg['step']}.f32.part")
            with open(tmp, "wb") as f:
                f.write(np.ascontiguousarray(arr).tobytes())
            os.replace(tmp, os.path.join(a.out, f"{msg['step']}.f32"))
        else:
            torch.cuda.synchronize()
        session.end(msg.get("end", []))
        sys.stdout.write(f"done {msg['step']}\n")
        sys.stdout.flush()
    return 0


if __name__ == "__main__":
    sys.exit(main())
