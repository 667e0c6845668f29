"""Token sampling on (tensor-parallel sharded) logits.

Reference behaviour kept (engine/model_runner.py:917-1083, 1151-1169): repetition penalty over the
tokens already in the sequence, constraints applied to the rank-local vocabulary shard, sharded
argmax for greedy requests, and for sampling a per-rank top-k whose candidates are gathered and
merged, then temperature / top-k / top-p / multinomial.  As in the reference a request without
top_k samples from the best `default_candidates` tokens.

Differences: every rank draws from the same seeded generator, so all ranks pick the same token and
no broadcast from rank 0 is needed; sampling over the candidates is vectorised over the batch
(no per-sequence `.item()`); only the last position of a prefill chunk ever reaches this code.
"""
from __future__ import annotations

import torch

from .constraints import init_constraint_state


class Sampler:
    default_candidates = 64

    def __init__(self, comm, vocab_start: int, eos_ids, seed: int = 0, full_vocab_gather: bool = False):
        # full_vocab_gather: the measuring baseline: every rank gathers the WHOLE logit row of every rank and runs
        # top-k over the full vocabulary (the structure the reference had before its top-k exchange,
        # engine/model_runner.py:1130-1133); tp * V floats per row on the wire instead of tp * k pairs
        self.full_vocab_gather = full_vocab_gather
        self.comm = comm
        self.vocab_start = vocab_start
        self.eos_ids = tuple(eos_ids)
        self.gen = torch.Generator(device="cpu")
        self.gen.manual_seed(seed)
        self._v_local = 0               # size of this rank's vocabulary shard (set by the runner)

    # ---- logits editing ---------------------------------------------------
    def _penalise(self, logits: torch.Tensor, seqs):
        n = logits.shape[-1]
        for i, seq in enumerate(seqs):
            rp = seq.repetition_penalty
            if rp == 1.0:
                continue
            ids = torch.tensor(sorted(set(seq.token_ids)), dtype=torch.long) - self.vocab_start
            ids = ids[(ids >= 0) & (ids < n)].to(logits.device)
            if ids.numel() == 0:
                continue
            v = logits[i, ids]
            logits[i, ids] = torch.where(v > 0, v / rp, v * rp)

    def _constrain(self, logits: torch.Tensor, seqs):
        for i, seq in enumerate(seqs):
            if seq.constraint is None:
                continue
            init_constraint_state(seq)
            seq.constraint.apply(logits[i], seq.constraint_state, self.vocab_start, self.eos_ids)

    max_device_candidates = 64      # the top-k kernels keep at most 64 candidates per rank

    def edit_rows(self, seqs) -> list:
        """Indices of the sequences whose logits are edited before the top-k (penalty, bias, masks, grammar)."""
        return [i for i, s in enumerate(seqs) if s.repetition_penalty != 1.0 or s.constraint is not None]

    def device_spec(self, seqs, edit_rows) -> dict:
        """Everything the device sampler needs for one step, built on the host: per-row temperature / top-k /
        top-p, one uniform number per sampling row drawn from the generator every rank seeds alike (drawn in
        row order, only for rows that sample, exactly as `sample_from_candidates` does), and for edited rows
        the additive logit row (what the constraint does to a row of zeros: 0, a bias, or -inf) and the
        sorted rank-local ids that get the repetition penalty."""
        n = len(seqs)
        rows = [i for i, s in enumerate(seqs) if s.temperature > 0 and s.top_k != 1]
        u = [0.0] * n
        if rows:
            draw = torch.rand(len(rows), 1, generator=self.gen)
            for j, i in enumerate(rows):
                u[i] = float(draw[j, 0])
        edits = []
        for i in edit_rows:
            seq = seqs[i]
            add = pen = None
            if seq.constraint is not None:
                init_constraint_state(seq)
                add = torch.zeros(self.v_local(seq), dtype=torch.float32)
                seq.constraint.apply(add, seq.constraint_state, self.vocab_start, self.eos_ids)
            if seq.repetition_penalty != 1.0:
                ids = torch.tensor(sorted(set(seq.token_ids)), dtype=torch.int32) - self.vocab_start
                pen = ids[(ids >= 0) & (ids < self.v_local(seq))]
            edits.append((i, add, pen, seq.repetition_penalty))
        return {"temperature": [s.temperature for s in seqs], "top_k": [s.top_k for s in seqs],
                "top_p": [s.top_p for s in seqs], "u": u, "edits": edits}

    def v_local(self, seq=None) -> int:
        return self._v_local

    def needs_full_logits(self, seqs) -> bool:
        return any(s.repetition_penalty != 1.0 or s.constraint is not None for s in seqs)

    def num_candidates(self, seqs) -> int:
        k = 1
        for s in seqs:
            if s.temperature > 0 and s.top_k != 1:
                k = max(k, s.top_k if s.top_k > 0 else self.default_candidates)
        return k

    # ---- sampling ---------------------------------------------------------
    def sample(self, logits: torch.Tensor, seqs) -> list:
        """logits: [n, V_local] fp32 (this rank's shard).  Returns one token id per sequence."""
        if self.needs_full_logits(seqs):
            logits = logits.clone()
            self._penalise(logits, seqs)
            self._constrain(logits, seqs)
        if self.full_vocab_gather and self.comm.world_size > 1:
            full = torch.cat(self.comm.all_gather(logits.float().contiguous()), dim=-1)   # shards are in rank order
            k = min(self.num_candidates(seqs), full.shape[-1])
            vals, idx = torch.topk(full, k, dim=-1)
            return self.sample_from_candidates(vals, idx, seqs, gathered=True)
        k = min(self.num_candidates(seqs), logits.shape[-1])
        vals, idx = torch.topk(logits, k, dim=-1)              # local candidates
        idx = idx + self.vocab_start
        return self.sample_from_candidates(vals, idx, seqs)

    def sample_from_candidates(self, vals: torch.Tensor, idx: torch.Tensor, seqs, gathered: bool = False) -> list:
        """vals/idx: [n, k] local candidates (global token ids).  Gathers over TP (unless the fused
        lm_head kernel already exchanged them: `gathered`) and samples."""
        if self.comm.world_size > 1 and not gathered:
            vals = torch.cat(self.comm.all_gather(vals.float().contiguous()), dim=-1)
            idx = torch.cat(self.comm.all_gather(idx.long().contiguous()), dim=-1)
        vals, idx = vals.float().cpu(), idx.long().cpu()
        # order by (value desc, token id asc): deterministic and identical on every rank
        order = torch.argsort(idx, dim=-1, stable=True)
        vals, idx = vals.gather(-1, order), idx.gather(-1, order)
        order = torch.argsort(vals, dim=-1, descending=True, stable=True)
        vals, idx = vals.gather(-1, order), idx.gather(-1, order)
        n, kk = vals.shape
        out = idx[:, 0].clone()
        rows = [i for i, s in enumerate(seqs) if s.temperature > 0 and s.top_k != 1]
        if rows:
            r = torch.tensor(rows)
            v = vals[r]
            temp = torch.tensor([seqs[i].temperature for i in rows]).unsqueeze(1)
            topk = torch.tensor([seqs[i].top_k if seqs[i].top_k > 0 else kk for i in rows]).unsqueeze(1)
            topp = torch.tensor([seqs[i].top_p for i in rows]).unsqueeze(1)
            ar = torch.arange(kk).unsqueeze(0)
            v = (v / temp).masked_fill(ar >= topk, float("-inf"))
            p = torch.softmax(v, dim=-1)
            csum = p.cumsum(-1)
            keep = (csum - p) < topp                       # smallest prefix reaching top_p
            p = torch.where(keep, p, torch.zeros_like(p))
            p = p / p.sum(-1, keepdim=True)
            u = torch.rand(len(rows), 1, generator=self.gen)
            pick = (p.cumsum(-1) < u).sum(-1).clamp_(max=kk - 1)
            # never land on a zero-probability tail entry
            pick = torch.minimum(pick, (p > 0).sum(-1) - 1)
            out[r] = idx[r].gather(-1, pick.unsqueeze(1)).squeeze(1)
        return out.tolist()
