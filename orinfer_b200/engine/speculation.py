"""Speculative decoding rounds: draft -> verify -> commit, distribution preserving.

Drafts come from request-local prompt lookup (copies of an earlier continuation) and, when
the model carries one, the MTP draft head.  One verification packet runs the target model
over ``[pending, d1, ..., dk]`` of every speculating request (plain decoders ride along
with one row); greedy requests commit the longest matching prefix plus the target's own
next token, sampled requests use exact rejection sampling with separate counter streams,
so the committed text never depends on whether speculation ran.  Rejected rows need no
rollback: their KV sits beyond the request's cursor and is overwritten later.  The width
of a round is chosen by the adaptive controller from measured round costs and
per-position acceptance.  Mirrors crates/orinfer-engine/src/runtime/requests/speculation.rs
:243-403,1361-1906 and mtp.rs:10-22,48-97 of the reference.
"""

from __future__ import annotations

import os
import time
from typing import Dict, List, Optional, Tuple

import numpy as np

from ..config import MAX_MTP_DRAFTS
from ..core import policy as P
from ..core import sampling as S
from .request import Phase, Request

WIDTHS = (2, 3, 4, 6, 8, 12, 16, 32)


class Speculator:
    def __init__(self, engine, max_drafts: Optional[int], prompt_lookup: bool):
        self.engine = engine
        self.max_drafts = MAX_MTP_DRAFTS if max_drafts is None else max_drafts
        if max_drafts is None:
            self.max_drafts = 3                        # "auto": up to three drafts
        self.prompt_lookup = prompt_lookup
        # the contract: which widths and batch shapes speculation may use for this model
        from ..contracts import MtpSpec
        self.contract = MtpSpec.for_config(engine.cfg, self.max_drafts, engine.sched.max_active,
                                           engine.max_rows)
        self.lookups: Dict[int, P.PromptLookup] = {}
        self.acceptance = P.Acceptance()
        # round cost per (batch bucket, verification width); plain-step cost per batch bucket
        # (the minimum of the last few: a decode step never gets faster than its kernels, so
        # outliers are host noise), and the call at which it was last measured
        self.costs: Dict[tuple, P.Timing] = {}
        self.last_used: Dict[tuple, int] = {}
        self.normal: Dict[int, list] = {}
        self.normal_last: Dict[int, int] = {}
        self.calls = 0
        self.rounds = self.proposed = self.accepted = self.committed = 0
        self.trace = os.environ.get("ORINFER_MTP_TRACE") == "1"
        self.policy = os.environ.get("ORINFER_SINGLE_MTP_POLICY", "auto")
        # how a round's draft rows are placed on its requests: "adaptive" gives the rows of a
        # width-w round (batch x (w - 1)) to the requests whose drafts survive most often,
        # "uniform" gives every request w - 1
        self.allocation = os.environ.get("ORINFER_MTP_ALLOCATION", "adaptive")
        self.local: Dict[int, List[float]] = {}       # rid -> [draft positions tested, accepted]

    @property
    def backlog(self) -> Dict[int, list]:
        """rid -> [(first position, hidden rows)] not yet seen by the draft head.  The rows are
        device data, so the engine keeps them (on every rank of a multi-rank engine)."""
        return self.engine._mtp_backlog

    @property
    def enabled(self) -> bool:
        return self.max_drafts > 0 and (self.prompt_lookup or self.engine.runner_has_mtp())

    # ------------------------------------------------------------------ width selection
    @staticmethod
    def _bucket(batch: int) -> int:
        b = 1
        while b < batch:
            b *= 2
        return b

    def observe_normal(self, batch: int, seconds: float) -> None:
        """A plain decode step of ``batch`` requests took ``seconds`` (replayed graph or
        direct packet, not a warm-up or capture step)."""
        key = self._bucket(batch)
        recent = self.normal.setdefault(key, [])
        recent.append(seconds)
        del recent[:-8]
        self.normal_last[key] = self.calls

    def choose_width(self, batch: int, remaining: int) -> int:
        """Verification width (rows per speculating request); 1 = plain decode."""
        if self.policy.startswith("fixed"):
            return 1 + min(int(self.policy[5:] or 0), self.max_drafts)
        key = self._bucket(batch)
        recent = self.normal.get(key)
        if not recent or len(recent) < 2:
            return 1                       # no plain step of this batch size measured yet
        normal = min(recent)
        cands = []
        for w in WIDTHS:
            if w - 1 > self.max_drafts:
                break
            t = self.costs.get((key, w))
            exp = self.acceptance.expected(w - 1)
            mean = t.mean if t and t.samples else normal * (1 + 0.05 * (w - 1))
            upper = t.upper if t and t.samples else mean * 1.5
            cands.append(P.Candidate(w, w, exp * batch, w * batch, remaining, mean, upper,
                                     samples=t.samples if t else 0,
                                     last=self.last_used.get((key, w))))
        cid, exploring, calibrating = P.mtp_select(
            normal, batch, self.engine.sched.target_tpot_ms / 1e3, cands,
            available_s=normal, calibration_s=4 * normal, calls=self.calls,
            normal_last=self.normal_last.get(key))
        if self.trace:
            print(f"MTP choose batch={batch} normal={normal:.5f} -> {cid} "
                  f"exploring={exploring} calibrating={calibrating}", flush=True)
        return cid or 1

    # ------------------------------------------------------------------ drafting
    def drafts_for(self, r: Request, count: int) -> List[int]:
        if count <= 0 or r.constraint is not None:
            return []
        if self.prompt_lookup:
            lk = self.lookups.setdefault(r.rid, P.PromptLookup())
            got = lk.propose(r.history, count, confident=not r.sampling.is_greedy)
            if got:
                return got
        return []

    def forget(self, r: Request) -> None:
        self.lookups.pop(r.rid, None)
        self.local.pop(r.rid, None)
        self.engine._mtp_forget(r.rid)

    # ------------------------------------------------------------------ MTP draft head
    def capture(self, rows_info, hidden) -> None:
        """Remember the target hidden states of freshly computed rows: the draft head must
        see (next token, hidden) of every position before it can draft past it."""
        if not self.engine.runner_has_mtp() or self.max_drafts <= 0:
            return
        keep = [(r.rid, int(row0), int(n), int(pos0)) for r, row0, n, pos0 in rows_info
                if n > 0 and not r.finished and r.constraint is None]
        if keep:
            self.engine._mtp_capture(keep, hidden)

    def mtp_drafts(self, reqs: List[Request], count: int) -> Dict[int, List[int]]:
        """Batched draft loop: one head pass over the backlog rows (catch-up + first draft),
        then ``count - 1`` single-row passes feeding the head's own hidden state back."""
        eng = self.engine
        live = [r for r in reqs if self.backlog.get(r.rid)]
        if not live or count <= 0:
            return {}
        cap = self.contract.draft_capacity(len(live))
        if len(live) > cap:                              # more requests than the largest profile
            out: Dict[int, List[int]] = {}
            for lo in range(0, len(live), cap):
                out.update(self.mtp_drafts(live[lo:lo + cap], count))
            return out
        toks, rreq, rpos, last = [], [], [], []
        for r in live:
            hist = r.history
            for pos0, h in self.backlog[r.rid]:
                n = h.shape[0]
                toks += [hist[pos0 + i + 1] for i in range(n)]
                rreq += [r.slot] * n
                rpos += list(range(pos0, pos0 + n))
            last.append(len(toks) - 1)
        if len(toks) > eng.max_rows:
            for r in live:
                eng._mtp_forget(r.rid)
            return {}
        plan = dict(rids=[r.rid for r in live], slots=[r.slot for r in live], toks=toks,
                    rreq=rreq, rpos=rpos, last=last, count=int(count),
                    offsets=[r.offset for r in live])
        out: Dict[int, List[int]] = {r.rid: [] for r in live}
        for step in eng._mtp_draft(plan):                # one device tensor per draft position
            for r, t in zip(live, step.cpu().tolist()):
                out[r.rid].append(int(t))
        return out

    # ------------------------------------------------------------------ draft rows per request
    LOCAL_PRIOR = 4.0            # draft positions' worth of weight of the engine-wide rate
    MIN_YIELD = 0.05             # a draft row expected to commit fewer tokens is not spent

    def local_rate(self, r: Request) -> float:
        """Probability that a draft of this request is accepted given the one before was:
        its own history, started from the engine-wide first-position rate."""
        tested, accepted = self.local.get(r.rid, (0.0, 0.0))
        prior = self.acceptance.rate(0, 0.7)
        return (self.LOCAL_PRIOR * prior + accepted) / (self.LOCAL_PRIOR + tested)

    def allocate(self, decoders: List[Request], width: int) -> Dict[int, int]:
        """rid -> draft rows of a width-``width`` round.  One request, fixed-width policies'
        first rounds and ``ORINFER_MTP_ALLOCATION=uniform`` give everyone ``width - 1``; else
        the same total is placed where it is expected to commit most tokens (a request whose
        drafts keep failing decodes plainly inside the packet, one that keeps being right
        gets up to the draft limit)."""
        uniform = {r.rid: width - 1 for r in decoders}
        if len(decoders) < 2 or self.allocation != "adaptive":
            return uniform
        caps = [0 if r.constraint is not None else
                max(min(self.max_drafts, r.max_new - len(r.generated) - 1), 0) for r in decoders]
        counts = P.mtp_allocate([self.local_rate(r) for r in decoders], caps,
                                len(decoders) * (width - 1), self.MIN_YIELD)
        return {r.rid: c for r, c in zip(decoders, counts)}

    def observe_local(self, r: Request, proposed: int, accepted: int) -> None:
        """``proposed`` drafts of ``r`` were verified and ``accepted`` of them kept; a round in
        which the request was given none lets its history fade towards the prior, so a text
        that turns predictable is tried again."""
        loc = self.local.setdefault(r.rid, [0.0, 0.0])
        if proposed <= 0:
            loc[0] *= 0.9
            loc[1] *= 0.9
            return
        loc[0] += min(accepted + 1, proposed)
        loc[1] += accepted

    # ------------------------------------------------------------------ inside prefill packets
    def plan_mixed(self, decoders: List[Request], room: int) -> Optional[Dict[int, List[int]]]:
        """Drafts of the greedy decoders for a packet that also carries prompt chunks:
        rid -> drafts, at most ``room`` draft rows in all; None when nobody drafts.  The
        width is the controller's choice for this many decoders (its round costs are learnt
        from pure verification rounds only)."""
        eng = self.engine
        if room <= 0 or not decoders:
            return None
        remaining = min(r.max_new - len(r.generated) for r in decoders)
        width = self.choose_width(len(decoders), remaining)
        self.calls += 1
        if width < 2:
            return None
        plain = [r for r in decoders if eng._plain(r)]
        plans: Dict[int, List[int]] = {}
        for r in plain:
            plans[r.rid] = self.drafts_for(r, min(width - 1, r.max_new - len(r.generated) - 1))
        if eng.runner_has_mtp():
            need = [r for r in plain if not plans[r.rid]]
            cap = min([r.max_new - len(r.generated) - 1 for r in need], default=0)
            for rid, d in self.mtp_drafts(need, min(width - 1, cap)).items():
                plans[rid] = d
        out: Dict[int, List[int]] = {}
        for r in plain:
            d = plans.get(r.rid) or []
            d = d[:max(room, 0)]
            if d:
                out[r.rid] = d
                room -= len(d)
        return out or None

    def observe_mixed(self, r: Request, drafts: List[int], accepted: int) -> None:
        self.observe_local(r, len(drafts), accepted)
        self.acceptance.observe([(len(drafts), accepted)])
        self.rounds += 1
        self.proposed += len(drafts)
        self.accepted += accepted
        self.committed += 1
        if r.rid in self.lookups:
            self.lookups[r.rid].observe(accepted, len(drafts), len(r.history))

    # ------------------------------------------------------------------ one round
    def run(self, decoders: List[Request]) -> Optional[List[Request]]:
        """Runs one verification packet; None when no request had a draft (caller falls
        back to the ordinary decode path)."""
        eng = self.engine
        remaining = min(r.max_new - len(r.generated) for r in decoders)
        width = self.choose_width(len(decoders), remaining)
        self.calls += 1
        if width < 2:
            return None
        share = self.allocate(decoders, width)
        plans: List[Tuple[Request, List[int]]] = []
        for r in decoders:
            room = r.max_new - len(r.generated) - 1
            plans.append((r, self.drafts_for(r, min(share[r.rid], room))))
        if eng.runner_has_mtp():
            need = [r for r, d in plans if not d and r.constraint is None and share[r.rid] > 0]
            room = min([r.max_new - len(r.generated) - 1 for r in need], default=0)
            most = max([share[r.rid] for r in need], default=0)
            got = self.mtp_drafts(need, min(most, room))
            plans = [(r, d or got.get(r.rid, [])[:share[r.rid]]) for r, d in plans]
        if not any(d for _, d in plans):
            return None
        t0 = time.monotonic()
        ids, rows_req, pos, max_kv = [], [], [], 1
        for r, drafts in plans:
            toks = [r.pending] + drafts
            ids += toks
            rows_req += [r.slot] * len(toks)
            pos += list(range(r.offset, r.offset + len(toks)))
            max_kv = max(max_kv, r.offset + len(toks))
        need = any(not eng._plain(r) for r, _ in plans)
        # recurrent layers must only keep the accepted prefix of each request's rows
        seg_lens = [1 + len(d) for _r, d in plans] if eng.recurrent else None
        packet = eng._verify_packet(ids, rows_req, pos, max_kv, need, seg_lens)
        tok_dev, logits = eng.runner.greedy(packet, need_logits=need)
        eng._status_enqueue()
        tokens = tok_dev.cpu().tolist()
        eng._status_check()
        produced, row = [], 0
        counts = []
        kept_rows = []
        hidden = eng.runner.final_hidden(len(ids)) if eng.runner_has_mtp() else None
        for r, drafts in plans:
            n = 1 + len(drafts)
            if eng._plain(r):
                commit = S.greedy_commit(drafts, tokens[row:row + n]) if drafts else [tokens[row]]
            elif drafts:
                lg = logits[row:row + n].float().cpu().numpy()
                commit = S.sampled_commit(drafts, None, lg, r.history, r.sampling,
                                          len(r.generated))
            else:
                tok = eng._sample_or_fail(r, tokens, logits, row)
                commit = [] if tok is None else [tok]
            if any(int(t) < 0 for t in commit):          # the device found no finite logit
                eng._fail_request(r, "FloatingPointError: non-finite logits")
                commit = []
            accepted = max(len(commit) - 1, 0)
            kept_rows.append(1 + accepted)
            self.observe_local(r, len(drafts), accepted)
            if drafts:
                counts.append((len(drafts), accepted))
                if r.rid in self.lookups:
                    self.lookups[r.rid].observe(accepted, len(drafts), len(r.history))
            if hidden is not None:
                self.capture([(r, row, 1 + accepted, r.offset)], hidden)
            r.offset += 1 + accepted
            for tok in commit:
                if r.finished:
                    break
                eng._deliver(r, int(tok))
            produced.append(r)
            row += n
        if packet.tentative:
            eng._verify_commit(kept_rows)
        if counts:
            self.acceptance.observe(counts)
            self.rounds += 1
            self.proposed += sum(c[0] for c in counts)
            self.accepted += sum(c[1] for c in counts)
        self.committed += sum(1 for _ in produced)
        dt = time.monotonic() - t0
        key = (self._bucket(len(decoders)), width)
        self.costs.setdefault(key, P.Timing()).observe(dt)
        self.last_used[key] = self.calls
        eng.stats.decode_tokens += len(ids)
        return produced

    def statistics(self) -> dict:
        return {"rounds": self.rounds, "proposed_tokens": self.proposed,
                "accepted_draft_tokens": self.accepted,
                "acceptance_rate": self.accepted / self.proposed if self.proposed else 0.0}
