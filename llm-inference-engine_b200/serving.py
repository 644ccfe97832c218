"""Serving a layer-list model: the scheduler (Batcher: page allocator, state slots, mixed plan) bound to a model's engine.

Two ways in:
  * generate(): requests go through the scheduler's own queue -- admission, prompts read in portions beside decoding sequences,
    preemption, top-k sampling -- one mixed batch per iteration (b200_batcher_step_hybrid);
  * open() / feed() / close(): the caller decides which tokens every sequence brings to every step (a replayed trace, prompts that
    are still arriving) and reads logits; pages and state slots still come from the same allocator, the step is the same engine call."""
import importlib

import numpy as np


def _mod():
    return importlib.import_module(__package__ or "llm-inference-engine_b200")


class Session:
    def __init__(self, model, pool_tokens, max_seqs=4, max_batch_tokens=None, poison=False):
        m = _mod()
        self.model, self.engine = model, model.engine
        pages = (int(pool_tokens) + m.KV_PAGE_SIZE - 1) // m.KV_PAGE_SIZE
        self.mpps = self.engine.cfg.max_pages_per_seq
        self.batcher = m.Batcher(max_seqs, pages, self.mpps, int(max_batch_tokens or self.engine.cfg.max_tokens))
        self.batcher.set_state_slots(max_seqs)
        self.engine.set_pools(pages, max_seqs, poison=poison)

    # ---- caller-driven sequences
    def open(self):
        return self.batcher.attach()

    def close(self, request):
        self.batcher.release(request)

    def feed(self, entries, trace=False):
        """entries: [(request, tokens, want)] -- `want` are indices into that entry's tokens.  One engine call for all of them.
        Returns device fp32 logits [total wanted, vocab], in the order of the entries and of their `want`."""
        ids, starts, pos0, slots, bt, rows = [], [0], [], [], [], []
        for request, tokens, want in entries:
            p0 = self.batcher.extend(request, tokens)
            row, slot = self.batcher.seq_pages(request)
            rows += [len(ids) + int(w) for w in want]
            ids += [int(t) for t in tokens]
            starts.append(len(ids)), pos0.append(p0), slots.append(max(slot, 0)), bt.append(row)
        return self.engine.forward(ids, starts, pos0, slots, np.concatenate(bt) if bt else np.zeros(0, np.int32), rows, trace=trace)

    # ---- scheduler-driven generation
    def generate(self, prompts, max_new_tokens, top_k=1, end_id=-1, chunk=0):
        """Greedy (top_k=1) or top-k sampled continuation of every prompt; returns one id list per prompt."""
        self.batcher.set_chunk(chunk)
        rids = [self.batcher.submit(p, max_new_tokens) for p in prompts]
        while self.batcher.pending():
            self.batcher.step_hybrid(self.engine, top_k=top_k, end_id=end_id)
        return [self.batcher.result(r, capacity=max_new_tokens + 1)[0].tolist() for r in rids]
