"""Continuous-batching engine: admission, chunked prefill, mixed packets, decode
CUDA graphs, prefix reuse and per-request sampling.

One iteration (``step``) is one forward packet, as in the reference's
``advance_requests_with`` (crates/orinfer-engine/src/runtime/requests.rs:1386-1658):

1. retire finished / cancelled requests (store their prefix, free pages);
2. admit waiting requests while slots, pages and the memory reserve allow
   (``can_admit``: prospective KV for prompt + max_new, requests.rs:392-459),
   evicting cached prefixes under pressure;
3. select work: decode rows of every running request plus prefill chunks up to
   the packet budget (latency policy keeps chunks within the prefill budget;
   throughput policy fills the packet);
4. run the packet (captured CUDA graph when it is pure decode and graphs are on);
5. commit: greedy rows read tokens written by the device argmax in one readback,
   other rows go through the host sampling law with counter RNG keyed by
   (seed, committed position).

Requests never share mutable state: KV pages are private except for read-only
full prefix pages, and sampling depends only on the request's own history.
"""

from __future__ import annotations

import collections
import dataclasses
import os
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence

import numpy as np
import torch

from ..config import PAGE_TOKENS, GraphMode, LoadOptions, ModelConfig, Phase as ExecPhase, Policy, \
    SchedulerOptions
from ..core import sampling as S
from ..core.prefix import RadixPrefixCache
from ..utils import trace
from ..models.runner import KVPool, Packet
from ..models.weights import ModelWeights
from .pages import OutOfPages, PagePool
from .request import Phase, Request

DECODE_BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128)


@dataclass
class EngineStatistics:
    iterations: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0
    graph_hits: int = 0
    graph_captures: int = 0
    direct_packets: int = 0
    packed_uploads: int = 0                   # packets whose index arrays went up in one copy
    admitted: int = 0
    deferred_admissions: int = 0
    finished: int = 0
    cancelled: int = 0
    capture_s: float = 0.0
    replay_s: float = 0.0
    direct_s: float = 0.0
    batch_inputs_s: float = 0.0
    batch_commit_s: float = 0.0
    evicted_pages: int = 0
    device_samples: int = 0
    offloaded_pages: int = 0
    restored_pages: int = 0
    sharded_samples: int = 0                  # rows drawn from a sharded head's candidates
    layered_decode_steps: int = 0             # decode steps taken inside paused prefill packets
    mixed_verify_packets: int = 0             # prefill packets that also verified drafts
    failed_requests: int = 0                  # requests ended by an error of their own
    resident_steps: int = 0                   # decode steps that needed no input upload
    stored_snapshots: int = 0                 # recurrent-state endpoints kept for the prefix cache
    restored_snapshots: int = 0

    def as_dict(self) -> dict:
        return dict(self.__dict__)


class _DecodeGraph:
    """Static buffers + captured graph of a pure-decode packet of ``rows`` rows."""

    def __init__(self, engine: "Engine", rows: int):
        dev = engine.device
        z = lambda *s, dt=torch.int32: torch.zeros(*s, dtype=dt, device=dev)
        self.rows = rows
        self.ids, self.req, self.pos = z(rows), z(rows), z(rows)
        self.tokens = z(rows)
        # Device-resident step control: the captured step ends by writing its own next inputs
        # (ids <- sampled tokens, pos <- pos + live), so a step over the same requests needs
        # no upload at all; ``members`` / ``host_pos`` are the host's record of what the
        # device buffers hold (kernels/cuda/model/control.py:9,27 of the reference keeps
        # position, length and token on the device in the same way).
        self.live = z(rows)
        self.members: Optional[tuple] = None
        self.host_pos: List[int] = []
        self.logits = torch.zeros(rows, engine.cfg.vocab, dtype=torch.float32, device=dev)
        self.packet = Packet(self.ids, self.req, self.pos, engine.page_table_dev, rows,
                             engine.max_context)
        if engine.recurrent:
            # every decode row is its own run; the state slot is read from ``req`` on the device
            ar = torch.arange(rows, dtype=torch.int32, device=dev)
            self.packet.row_first = ar
            self.packet.segments = torch.stack(
                [ar, torch.ones_like(ar), torch.zeros_like(ar), torch.zeros_like(ar)], 1).contiguous()
            self.packet.n_segments = rows
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.trials = 0


class Engine:
    def __init__(self, weights: ModelWeights, *, load: Optional[LoadOptions] = None,
                 sched: Optional[SchedulerOptions] = None, kv_pages: Optional[int] = None,
                 max_context: Optional[int] = None, max_rows: Optional[int] = None,
                 runner=None, channel=None):
        # ``channel``: a parallel.rank_channel.LeaderChannel when this engine leads follower
        # ranks: every device command (page-table row, packet, graph replay, sharded
        # sampling) is published to them before it runs here, and they replay it through
        # ``apply`` on an engine of their own that takes no decisions.
        self.channel = channel
        self.w = weights
        self.cfg: ModelConfig = weights.config
        self.load = load or LoadOptions()
        self.sched = sched or SchedulerOptions()
        self.load.validate()
        self.sched.validate()
        self.device = weights.embed_q.device
        self.on_gpu = self.device.type == "cuda"
        # The kernel library keeps its status word, decode tables and workspaces per device
        # and answers for the device that is current on the calling thread: make the model's
        # device current before anything is launched, and keep a pinned mirror of the status
        # word that every step's token readback refreshes.
        self.failed: Optional[Exception] = None
        self._step_was_replay = False
        self._status = None
        if self.on_gpu:
            from ..ops import native
            torch.cuda.set_device(self.device)
            native.init()
            native.expect_device(self.device)
            self._status = native.StatusReader()
        # Recurrent (GDN) layers keep per-request state that cannot be rebuilt from KV pages.
        # A cached prefix of a hybrid model is therefore usable only at an endpoint where the
        # state was snapshotted (prompt end, periodic checkpoints): prefill chunks are cut at
        # those positions and ``_snapshots`` maps the radix node of the endpoint's last page
        # to the copy.  Speculation: verification packets are tentative and the runner commits
        # the accepted prefix of every request afterwards.
        self.recurrent = self.cfg.arch == "hybrid"
        self._snapshots: "collections.OrderedDict[int, tuple]" = collections.OrderedDict()
        self._snapshot_bytes = 0
        # the copies themselves: handle -> this rank's tensors (every rank of a multi-rank
        # engine keeps its own shard under the handle the leader chose)
        self._state_copies: Dict[int, tuple] = {}
        self._state_handles = 0
        self._tentative: Optional[Packet] = None     # verification packet awaiting its commit
        # hidden rows the draft head has not seen yet: rid -> [(first position, rows)]
        self._mtp_backlog: Dict[int, list] = {}
        # decoders of the current direct packet that verify drafts: rid -> (drafts, first row)
        self._verify: Dict[int, tuple] = {}
        self._direct_rows = 0
        self.max_context = max_context or min(self.cfg.max_context, 32768)
        self.max_pages_per_req = (self.max_context + PAGE_TOKENS - 1) // PAGE_TOKENS
        self.max_rows = max_rows or max(self.sched.prefill_chunk + self.sched.max_active, 256)
        extra = self.cfg.mtp_layers
        if kv_pages is None:
            kv_pages = self._auto_pages(extra)
        # Bounded expert residency: a packet of r rows routes to at most r x top_k experts of
        # a layer, so packets are capped at resident // top_k rows; the launch sequence depends
        # on data read back per layer, so graphs and speculation are off.
        self.row_cap = self.max_rows
        self.paging = bool(self.cfg.experts) and 0 < self.load.resident_experts < self.cfg.experts
        if self.paging:
            if self.load.resident_experts < self.cfg.top_k:
                raise ValueError("resident_experts must be at least top_k")
            cap = self.row_cap = self.load.resident_experts // self.cfg.top_k
            self.sched = dataclasses.replace(self.sched, max_active=min(self.sched.max_active, cap),
                                             prefill_chunk=min(self.sched.prefill_chunk, cap))
            self.load = dataclasses.replace(self.load, cuda_graph=GraphMode.OFF, mtp_drafts=0,
                                            prompt_lookup=False)
        self.pool = PagePool(kv_pages)
        self.kv = KVPool.allocate(self.cfg, kv_pages, self.device, extra_layers=extra)
        if runner is not None:
            self.runner = runner(weights, self.kv, self.max_rows)
        elif getattr(weights, "tp", None) is not None:
            from ..parallel.tp_runner import TPRunner, TPTorchRunner
            from ..parallel import fused
            if self.on_gpu:
                cls = fused.FusedTPRunner if fused.enabled() else TPRunner
            else:
                cls = TPTorchRunner
            self.runner = cls(weights, self.kv, self.max_rows)
        elif self.on_gpu:
            from ..models.runner import ModelRunner
            self.runner = ModelRunner(weights, self.kv, self.max_rows)
        else:
            from ..models.torch_runner import TorchRunner
            self.runner = TorchRunner(weights, self.kv, self.max_rows)
        if self.paging and hasattr(self.runner, "enable_expert_pager"):
            self.runner.enable_expert_pager(self.load.resident_experts)
        slots = self.sched.max_active + 1                      # last slot = padding target
        self.page_table_host = np.zeros((slots, self.max_pages_per_req), np.int32)
        self.page_table_dev = torch.zeros(slots, self.max_pages_per_req, dtype=torch.int32,
                                          device=self.device)
        self.free_slots: List[int] = list(range(self.sched.max_active - 1, -1, -1))
        self.pad_slot = self.sched.max_active
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.prefix = RadixPrefixCache(PAGE_TOKENS) if self.load.prefix_cache_bytes > 0 else None
        self._prefix_nodes: Dict[int, List[int]] = {}
        self.host_kv = None
        if self.prefix is not None and self.load.kv_offload_bytes > 0:
            from .offload import HostKvStore
            self.host_kv = HostKvStore(self.kv, self.load.kv_offload_bytes)
            if self.host_kv.slots == 0:
                self.host_kv = None
        self.stats = EngineStatistics()
        self._graphs: Dict[int, _DecodeGraph] = {}
        self._next_rid = 1
        self._pin = {}
        self._stage = None                       # pinned staging ring of ``_upload_many``
        self._packed_uploads = os.environ.get("ORINFER_PACKED_UPLOAD", "1") != "0"
        # verification rows inside prompt packets (ORINFER_MIXED_VERIFY=0: decoders take plain
        # single rows while prompts are being prefilled)
        self._mixed_verify = os.environ.get("ORINFER_MIXED_VERIFY", "1") != "0"
        from .speculation import Speculator
        self.spec = Speculator(self, self.load.mtp_drafts, self.load.prompt_lookup)
        self.tpot_ewma: Optional[float] = None
        from ..core.policy import CostCurves
        self.costs = CostCurves()

    # ------------------------------------------------------------------ sizing
    def _auto_pages(self, extra_layers: int) -> int:
        per_page = KVPool.bytes_per_page(self.cfg, extra_layers)
        if self.on_gpu:
            free, _total = torch.cuda.mem_get_info(self.device)
            budget = max(free - self.sched.memory_reserve_bytes - (8 << 30), per_page * 64)
            budget = min(budget, 64 << 30)
        else:
            budget = 64 << 20
        want = self.sched.max_active * self.max_pages_per_req + 1
        return int(max(4, min(budget // per_page, want)))

    # ------------------------------------------------------------------ public API
    def submit(self, prompt: Sequence[int], max_new: int = 16,
               sampling: Optional[S.SamplingOptions] = None, **kw) -> Request:
        if len(prompt) == 0:
            raise ValueError("empty prompt")
        if self.cfg.bidirectional:
            raise ValueError("an encoder model embeds its input; it does not generate")
        if len(prompt) + max_new > self.max_context:
            raise ValueError(
                f"request of {len(prompt)} + {max_new} tokens exceeds the context window "
                f"({self.max_context})")
        sampling = sampling or S.SamplingOptions(temperature=0.0)
        sampling.validate()
        req = Request(self._next_rid, list(map(int, prompt)), int(max_new), sampling, **kw)
        if req.media or req.rope_positions is not None:
            if not getattr(self.runner, "supports_media", False):
                raise ValueError("this runner takes no media inputs")
            for m in req.media:
                if not (0 <= m.start < m.end <= len(req.prompt)) or \
                        tuple(m.features.shape) != (m.end - m.start, self.cfg.hidden):
                    raise ValueError("media span does not fit the prompt or the hidden size")
            if req.rope_positions is not None and \
                    tuple(req.rope_positions.shape) != (3, len(req.prompt)):
                raise ValueError("rope_positions must be [3, prompt length]")
        self._next_rid += 1
        self.waiting.append(req)
        return req

    def encode(self, tokens: Sequence[int]):
        """One bidirectional-free encoder pass of the decoder over ``tokens`` outside the
        request queue: returns (mean-pooled, L2-normalised final hidden state fp32 [hidden],
        fp32 logits of the last position).  Used by the embeddings and rerank endpoints.
        Needs one free request slot and enough free KV pages (evicting cached prefixes)."""
        if self.channel is not None:
            raise ValueError("encoder passes are not supported by a multi-rank engine")
        n = len(tokens)
        if n == 0 or n > min(self.max_context, self.max_rows):
            raise ValueError(f"encoder input of {n} tokens is outside 1..{min(self.max_context, self.max_rows)}")
        need = (n + PAGE_TOKENS - 1) // PAGE_TOKENS
        if need > self.pool.available:
            self._reclaim(need)
        if not self.free_slots or need > self.pool.available:
            raise MemoryError("no free slot or KV pages for an encoder pass")
        slot = self.free_slots.pop()
        pages = self.pool.take(need)
        try:
            row = self.page_table_host[slot]
            row[:] = 0
            row[:need] = pages
            self.page_table_dev[slot].copy_(torch.from_numpy(row))
            packet = Packet(self._upload("ids", list(tokens)), self._upload("req", [slot] * n),
                            self._upload("pos", list(range(n))), self.page_table_dev, n, n,
                            self._upload("sel", [n - 1]).long())
            if self.cfg.bidirectional:
                # every row sees the whole input: keys are written first, then read with the
                # last position as each row's horizon (row kernel; no causal tile kernel)
                packet.attend_pos = self._upload("see", [n - 1] * n)
            elif self.on_gpu and n > 1:
                packet.chunks = self._upload("chunks", [0, n, 0, slot]).view(-1, 4)
                packet.max_q_len = n
            _tok, lg = self.runner.greedy(packet, need_logits=True)
            hidden = (self.runner.final_hidden(n) if hasattr(self.runner, "final_hidden")
                      else self.runner._final[:n]).float()
            pooled = {"mean": hidden.mean(0), "last": hidden[-1], "first": hidden[0]}[
                self.cfg.pooling]
            pooled = pooled / pooled.norm().clamp_min(1e-12)
            return pooled.cpu(), lg[0].float().cpu()
        finally:
            self.pool.release(pages)
            self.free_slots.append(slot)

    def prefill_device(self, ids: torch.Tensor) -> torch.Tensor:
        """Prefill of one fresh prompt whose token ids are already on the device, up to its
        first greedy token, without any host synchronisation: returns the device tensor that
        will hold the token (valid once the stream has run).  The prompt takes a free request
        slot and KV pages for the duration of the call only (nothing is cached), and runs
        through the same full-graph prefill path as a queued request.  For device-timed
        measurements and for callers that keep their own token stream on the GPU."""
        if not self.on_gpu or self.recurrent or self.channel is not None:
            raise ValueError("prefill_device needs a single-process CUDA engine of a "
                             "non-recurrent model")
        n = int(ids.numel())
        if n < 1 or n > min(self.max_context, self.max_rows):
            raise ValueError(f"prompt of {n} tokens is outside 1..{min(self.max_context, self.max_rows)}")
        need = (n + PAGE_TOKENS - 1) // PAGE_TOKENS
        if need > self.pool.available:
            self._reclaim(need)
        if not self.free_slots or need > self.pool.available:
            raise MemoryError("no free slot or KV pages")
        slot = self.free_slots.pop()
        pages = self.pool.take(need)
        try:
            row = self.page_table_host[slot]
            if list(row[:need]) != list(pages) or row[need:].any():
                row[:] = 0
                row[:need] = pages
                self.page_table_dev[slot].copy_(torch.from_numpy(row), non_blocking=True)
            cache = self.__dict__.setdefault("_pd_cache", {})
            fixed = cache.get((n, slot))
            if fixed is None:
                dev = self.device
                fixed = cache[(n, slot)] = (
                    torch.full((n,), slot, dtype=torch.int32, device=dev),
                    torch.arange(n, dtype=torch.int32, device=dev),
                    torch.tensor([n - 1], device=dev),
                    torch.tensor([[0, n, 0, slot]], dtype=torch.int32, device=dev))
            req_rows, pos, sel, chunks = fixed
            packet = Packet(ids.to(torch.int32), req_rows, pos, self.page_table_dev, n, n, sel,
                            chunks=chunks, max_q_len=n)
            out = None
            if (self.cfg.head_dim in (64, 128, 256)
                    and self.load.cuda_graph.uses_graph(ExecPhase.PREFILL)
                    and getattr(self.runner, "stage_hook", None) is None):
                plan = self._prefill_pool().plan(((n,), 1, False))
                out = self._prefill_graph(packet, False, *plan)
            if out is None:
                out = self.runner.greedy(packet, need_logits=False)
            self.stats.prefill_tokens += n
            return out[0]
        finally:
            self.pool.release(pages)
            self.free_slots.append(slot)

    def close(self, collective: bool = True) -> None:
        """Releases what must go before the process group and the CUDA context do: captured
        graphs first (they hold the collective and peer-memory work they recorded), then the
        runner's peer mappings.  With several ranks every rank calls this at the same point
        (the runner's close meets its peers at a barrier); ``collective=False`` skips that
        meeting when a rank is known to be gone."""
        self._graphs.clear()
        pool = self.__dict__.pop("_prefill_graphs", None)
        if pool is not None:
            pool.clear()
        if self.on_gpu:
            torch.cuda.synchronize()
        closer = getattr(self.runner, "close", None)
        if closer is not None:
            import inspect
            if "collective" in inspect.signature(closer).parameters:
                closer(collective=collective)
            else:
                closer()

    def cancel(self, req: Request) -> None:
        req.cancelled = True

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def generate(self, prompts: Sequence[Sequence[int]], max_new: int = 16,
                 sampling: Optional[S.SamplingOptions] = None, **kw) -> List[List[int]]:
        reqs = [self.submit(p, max_new, sampling, **kw) for p in prompts]
        while any(not r.finished for r in reqs):
            self.step()
        return [r.generated for r in reqs]

    def generate_reference(self, prompt: Sequence[int], max_new: int = 16,
                           chunk: Optional[int] = None) -> List[int]:
        """Greedy generation of one request on its own, outside the queue: the prompt runs as
        full chunks of ``chunk`` tokens, its tail and every new token as single-row packets, so
        no padding row ever enters attention, convolution or recurrent state.  This is the
        isolation oracle that batched, chunked, graph-replayed and speculative runs are checked
        against (the reference's crates/orinfer-engine/src/runtime/reference_generation.rs:5-6).
        No prefix cache, no graphs, no speculation; needs an idle engine."""
        if self.channel is not None:
            raise ValueError("generate_reference is not supported by a multi-rank engine")
        if self.running or self.waiting:
            raise RuntimeError("generate_reference needs an idle engine")
        prompt = list(map(int, prompt))
        total = len(prompt) + max_new
        if not prompt or total > self.max_context:
            raise ValueError("prompt is empty or prompt + max_new exceeds the context window")
        chunk = min(chunk or self.sched.prefill_chunk, self.max_rows)
        need = (total + PAGE_TOKENS - 1) // PAGE_TOKENS
        if need > self.pool.available:
            self._reclaim(need)
        if not self.free_slots or need > self.pool.available:
            raise MemoryError("no free slot or KV pages for a reference run")
        slot = self.free_slots.pop()
        pages = self.pool.take(need)
        try:
            row = self.page_table_host[slot]
            row[:] = 0
            row[:need] = pages
            self.page_table_dev[slot].copy_(torch.from_numpy(row))

            def run(tokens: List[int], start: int) -> int:
                n = len(tokens)
                p = Packet(self._upload("ids", tokens), self._upload("req", [slot] * n),
                           self._upload("pos", list(range(start, start + n))),
                           self.page_table_dev, n, start + n, self._upload("sel", [n - 1]).long())
                if self.recurrent:
                    p.segments = self._upload("segs", [0, n, 0, 0]).view(-1, 4)
                    p.row_first = self._upload("first", [0] * n)
                    p.n_segments = 1
                if self.on_gpu and n > 1:
                    p.chunks = self._upload("chunks", [0, n, start, slot]).view(-1, 4)
                    p.max_q_len = n
                tok, _ = self.runner.greedy(p, need_logits=False)
                return int(tok[0])

            at, full = 0, len(prompt) // chunk * chunk
            last = -1
            while at < full:
                last = run(prompt[at:at + chunk], at)
                at += chunk
            for t in prompt[full:]:
                last = run([t], at)
                at += 1
            out = [last]
            while len(out) < max_new:
                out.append(run([out[-1]], at))
                at += 1
            return out[:max_new]
        finally:
            self.pool.release(pages)
            self.free_slots.append(slot)

    # ------------------------------------------------------------------ admission
    def _pages_needed(self, req: Request) -> int:
        return (req.context_needed() + PAGE_TOKENS - 1) // PAGE_TOKENS

    def can_admit(self, req: Request, shared_pages: int = 0) -> bool:
        return bool(self.free_slots) and \
            self._pages_needed(req) - shared_pages <= self.pool.available

    def _reclaim(self, pages: int) -> None:
        """Evict cached prefixes (lowest utility first) until ``pages`` are free."""
        if self.prefix is None:
            return
        short = pages - self.pool.available
        if short <= 0:
            return
        if self.host_kv is not None:
            # move the least useful pages to pinned host memory; their nodes stay indexed
            if self.host_kv.available < short:
                for h in self.prefix.drop_host(short - self.host_kv.available):
                    self._host_kv("free", h)
            victims = self.prefix.evict(min(short, self.host_kv.available), to_host=True)
            for node, page in victims:
                # a node that was offloaded before and re-adopted a device page still owns
                # its old host slot: give it back before the new copy takes one
                stale = self.prefix.host_handle(node)
                if stale >= 0:
                    self._host_kv("free", stale)
                self.prefix.set_host(node, self._host_kv("save", page))
            if victims:
                self._host_kv("sync")               # pages are reused right after this
            self.pool.release([p for _, p in victims])
            self.stats.evicted_pages += len(victims)
            self.stats.offloaded_pages += len(victims)
            short -= len(victims)
            if short <= 0:
                return
        victims = self.prefix.evict(short, to_host=False)
        self.pool.release([p for _, p in victims])
        self.stats.evicted_pages += len(victims)

    def _host_kv(self, op: str, *args):
        """One operation of the host KV tier, published first: every rank moves its own shard
        of the page between its own device pool and its own host slab.  The stores hand out
        slots in the same order on every rank, so a handle means the same slot everywhere;
        ``save`` carries the leader's handle so that a follower can check that."""
        if op == "save":
            handle = self.host_kv.save(*args)
            self._publish("host_kv", (op, *args, handle))
            return handle
        self._publish("host_kv", (op, *args))
        return getattr(self.host_kv, op)(*args)

    def _restore_host_pages(self, node_ids: List[int], pages: List[int]) -> int:
        """Brings the host-resident nodes of a matched prefix back into device pages, in
        order; returns how many leading nodes are usable (device-resident) afterwards."""
        for i, (node, page) in enumerate(zip(node_ids, pages)):
            if page >= 0:
                continue
            if self.host_kv is None:
                return i
            if self.pool.available == 0:
                self._reclaim(1)
            if self.pool.available == 0:
                return i
            handle = self.prefix.host_handle(node)
            if handle < 0:
                return i
            new = self.pool.take(1)[0]
            self._host_kv("load", handle, new)
            if not self.prefix.restore(node, new):
                self.pool.release([new])
                return i
            self.prefix.set_host(node, -1)
            self._host_kv("free", handle)
            pages[i] = new
            self.stats.restored_pages += 1
        return len(pages)

    def _admit(self) -> None:
        started = time.monotonic()
        admitted = 0
        while self.waiting and len(self.running) < self.sched.max_active:
            req = self.waiting[0]
            if req.cancelled:
                self.waiting.popleft()
                self._finish(req, "cancelled")
                continue
            node_ids, pages = [], []
            if self.prefix is not None and req.cache_prompt:
                node_ids, pages = self.prefix.match(
                    req.prompt, limit_tokens=len(req.prompt) - 1,
                    media=req.page_media(PAGE_TOKENS, len(req.prompt) // PAGE_TOKENS + 1))
                snapshot = None
                if self.recurrent and node_ids:               # usable only up to a kept endpoint
                    cut, snapshot = self._snapshot_for(req.prompt, node_ids)
                    self.prefix.release(node_ids[cut:])
                    node_ids, pages = node_ids[:cut], pages[:cut]
                if any(pg < 0 for pg in pages):              # host-resident nodes: restore or cut
                    cut = self._restore_host_pages(node_ids, pages)
                    if self.recurrent and cut < len(pages):
                        cut = 0                               # the endpoint itself was lost
                    self.prefix.release(node_ids[cut:])
                    node_ids, pages = node_ids[:cut], pages[:cut]
            need = self._pages_needed(req) - len(pages)
            if need > self.pool.available:
                self._reclaim(need)
            if not self.free_slots or need > self.pool.available:
                if node_ids:
                    self.prefix.abandon(node_ids)        # the retry will match (and count) again
                self.stats.deferred_admissions += 1
                break
            self.waiting.popleft()
            for pg in pages:
                self.pool.share(pg)
            req.pages = list(pages) + self.pool.take(need)
            req.slot = self.free_slots.pop()
            req.offset = req.cached_tokens = len(pages) * PAGE_TOKENS
            if self.recurrent and pages:
                self._state_copy("restore", snapshot, req.slot)
                self.stats.restored_snapshots += 1
            req.phase = Phase.PREFILL
            self._prefix_nodes[req.rid] = node_ids
            self._set_page_row(req.slot, req.pages)
            self.running.append(req)
            self.stats.admitted += 1
            admitted += 1
            trace.line("admit", rid=req.rid, prompt=len(req.prompt), cached=req.cached_tokens,
                       pages=len(req.pages), slot=req.slot, waiting=len(self.waiting))
            if self._should_yield(admitted, time.monotonic() - started):
                break

    def _should_yield(self, admitted: int, elapsed: float) -> bool:
        has_decoders = any(r.phase is Phase.DECODE for r in self.running)
        if has_decoders:
            return admitted >= 8 or elapsed >= 0.100
        return admitted >= 32 or elapsed >= 3.0

    # ------------------------------------------------------------------ retirement
    def _finish(self, req: Request, reason: str) -> None:
        req.finish_reason = req.finish_reason or reason
        req.phase = Phase.FINISHED
        req.finished_at = time.monotonic()
        if req.slot >= 0:
            if self.prefix is not None and req.cache_prompt and reason != "error":
                # index the full pages of prompt + generated tokens whose KV is in the cache
                toks = req.history[:req.offset]
                adopted, ids = self.prefix.insert(
                    toks, req.pages[:len(toks) // PAGE_TOKENS],
                    media=req.page_media(PAGE_TOKENS, len(toks) // PAGE_TOKENS + 1))
                for pg, took, node in zip(req.pages, adopted, ids):
                    if took:
                        self.pool.share(pg)
                        # a host-resident node that adopts a fresh device page needs its host
                        # copy no longer: give the slot back now (an eviction that removes
                        # the node later would lose it)
                        stale = self.prefix.host_handle(node) if self.host_kv is not None else -1
                        if stale >= 0:
                            self.prefix.set_host(node, -1)
                            self._host_kv("free", stale)
                for at in sorted(req.snapshots):
                    if at // PAGE_TOKENS <= len(ids):
                        self._store_snapshot(ids[at // PAGE_TOKENS - 1], toks[:at],
                                             req.snapshots.pop(at))
            for handle in req.snapshots.values():            # endpoints that were not indexed
                self._state_copy("drop", handle)
            req.snapshots = {}
            if self.prefix is not None:
                self.prefix.release(self._prefix_nodes.pop(req.rid, []))
            self.pool.release(req.pages)
            req.pages = []
            self.free_slots.append(req.slot)
            req.slot = -1
        if reason == "cancelled":
            self.stats.cancelled += 1
        else:
            self.stats.finished += 1
        if req in self.running:
            self.running.remove(req)
        self.spec.forget(req)

    # ------------------------------------------------------------------ work selection
    def _select(self):
        decoders = [r for r in self.running if r.phase is Phase.DECODE]
        prefills = [r for r in self.running if r.phase is Phase.PREFILL]
        budget = max(min(self.max_rows, self.row_cap) - len(decoders), 0)
        budget = min(budget, self.sched.prefill_chunk)
        chunks = []
        if self.sched.policy is Policy.LATENCY and decoders and self.tpot_ewma is not None:
            # keep prompt progress within the prefill budget while decoders are live
            # measured packet costs size the chunk against the prefill budget (cold: the
            # running tokens/s estimate)
            ctx = max((r.offset for r in prefills), default=0) + 1
            dctx = max(r.offset for r in decoders) + 1
            if self.costs.cells:
                fit = self.costs.fit_tokens(self.sched.prefill_budget_ms / 1e3, budget, 16,
                                            context=ctx, decode_rows=len(decoders),
                                            decode_context=dctx)
                budget = min(budget, max(fit, 16))
            else:
                rate = self._prefill_rate()
                if rate:
                    budget = min(budget,
                                 max(int(rate * self.sched.prefill_budget_ms / 1e3), 16))
        prefills.sort(key=lambda r: (r.last_prefill_at or r.arrived))
        for r in prefills:
            if budget <= 0:
                break
            n = min(r.remaining_prefill, budget)
            if self.recurrent and self.prefix is not None and r.cache_prompt:
                n = min(n, self._next_endpoint(r) - r.offset)
            chunks.append((r, n))
            budget -= n
        if chunks and trace.enabled("prefill_choose"):
            trace.line("prefill_choose", decoders=len(decoders),
                       chunks=[[r.rid, r.offset, n] for r, n in chunks], budget_left=budget,
                       tpot_ms=None if self.tpot_ewma is None else round(self.tpot_ewma * 1e3, 3),
                       cost_cells=self.costs.cells)
        return decoders, chunks

    # ------------------------------------------------------------------ recurrent snapshots
    CHECKPOINT_TOKENS = 8192

    def _endpoints(self, prompt_len: int) -> List[int]:
        """Positions (page multiples) at which a hybrid model's recurrent state is kept: the
        last page boundary a later request with the same prompt may match (one token is always
        left to compute), and every ``CHECKPOINT_TOKENS`` before it."""
        last = (prompt_len - 1) // PAGE_TOKENS * PAGE_TOKENS
        pts = list(range(self.CHECKPOINT_TOKENS, last, self.CHECKPOINT_TOKENS))
        if last > 0:
            pts.append(last)
        return pts

    def _next_endpoint(self, r: Request) -> int:
        for at in self._endpoints(len(r.prompt)):
            if at > r.offset:
                return at
        return len(r.prompt)

    def _capture_snapshots(self, chunks) -> None:
        if not (self.recurrent and self.prefix is not None):
            return
        for r, _n in chunks:
            if r.cache_prompt and r.slot >= 0 and r.offset in self._endpoints(len(r.prompt)) \
                    and r.offset > r.cached_tokens:
                self._state_handles += 1
                r.snapshots[r.offset] = self._state_copy("take", self._state_handles, r.slot)

    def _state_copy(self, op: str, handle: int, slot: int = -1) -> int:
        """Recurrent-state copies live on each rank under a handle that the leader chose:
        ``take`` copies the state of one request slot (every recurrent layer), ``restore``
        writes a copy back into a slot, ``drop`` forgets it.  The command is published, so
        every rank does the same to its own shard of the state."""
        self._publish("state_copy", (op, int(handle), int(slot)))
        if op == "take":
            self._state_copies[handle] = self.runner.gdn_snapshot(slot)
        elif op == "restore":
            if handle not in self._state_copies:
                raise ValueError(f"no recurrent-state copy under handle {handle} on this rank")
            self.runner.gdn_restore(slot, self._state_copies[handle], self.page_table_dev.shape[0])
        elif op == "drop":
            self._state_copies.pop(handle, None)
        else:
            raise ValueError(f"unknown state-copy operation {op!r}")
        return handle

    @staticmethod
    def _token_digest(tokens) -> bytes:
        import hashlib
        import numpy as np
        return hashlib.blake2b(np.asarray(tokens, dtype=np.uint32).tobytes(),
                               digest_size=16).digest()

    @staticmethod
    def _nbytes(snap) -> int:
        total = 0
        for part in snap:
            for t in (part if isinstance(part, (list, tuple)) else [part]):
                if torch.is_tensor(t):
                    total += t.numel() * t.element_size()
        return total

    def _store_snapshot(self, node: int, tokens, handle: int) -> None:
        """Keeps the state copy ``handle`` for the radix node ``node`` (the last page of
        ``tokens``); the token digest guards against a node id that the tree has recycled
        since.  The store is an LRU bounded by a quarter of the prefix-cache budget (counted in
        this rank's bytes; shards are equal)."""
        digest = self._token_digest(tokens)
        old = self._snapshots.pop(node, None)
        if old is not None:
            self._snapshot_bytes -= old[2]
            self._state_copy("drop", old[1])
        size = self._nbytes(self._state_copies[handle])
        self._snapshots[node] = (digest, handle, size)
        self._snapshot_bytes += size
        self.stats.stored_snapshots += 1
        limit = max(self.load.prefix_cache_bytes // 4, size)
        while self._snapshot_bytes > limit and len(self._snapshots) > 1:
            _node, (_d, gone, sz) = self._snapshots.popitem(last=False)
            self._snapshot_bytes -= sz
            self._state_copy("drop", gone)

    def _snapshot_for(self, prompt, node_ids):
        """-> (pages of the matched prefix that can be used, handle of the state copy at that
        endpoint)."""
        for i in range(len(node_ids) - 1, -1, -1):
            hit = self._snapshots.get(node_ids[i])
            if hit is None:
                continue
            if hit[0] != self._token_digest(prompt[:(i + 1) * PAGE_TOKENS]):
                self._snapshot_bytes -= hit[2]                # recycled node id: stale entry
                del self._snapshots[node_ids[i]]
                self._state_copy("drop", hit[1])
                continue
            self._snapshots.move_to_end(node_ids[i])
            return i + 1, hit[1]
        return 0, None

    def _prefill_rate(self) -> Optional[float]:
        return getattr(self, "_prefill_tok_s", None)

    # ------------------------------------------------------------------ one iteration
    def _status_enqueue(self) -> None:
        """Queue the status-word copy behind the step's kernels (no synchronisation)."""
        if self._status is not None:
            self._status.enqueue()

    def _status_check(self) -> None:
        """After the step's readback: a bounded device wait that ran out (peer flag, TMA or
        MMA barrier) or a rejected index left its code in the status word.  The step's output
        cannot be trusted and peers' counters may be out of step, so the engine fails closed:
        this raises a fatal error now and on every later step."""
        if self._status is None:
            return
        word = self._status.value()
        if word:
            from ..core.policy import EngineError, ErrorKind
            code, detail = word >> 16, word & 0xffff
            kind = ErrorKind.NCCL if code == 5 else ErrorKind.CUDA
            names = {1: "TMA wait", 2: "MMA wait", 3: "epilogue wait", 4: "decode wait",
                     5: "peer wait", 6: "rejected index"}
            self.failed = EngineError(
                kind, f"device status {word:#x}: {names.get(code, 'code %d' % code)} "
                      f"(detail {detail:#x}); the engine is failed closed", word)
            raise self.failed

    def step(self) -> List[Request]:
        """Run one packet; returns the requests that produced tokens."""
        if self.failed is not None:
            raise self.failed
        self._verify = {}
        for r in list(self.running):
            if r.cancelled:
                self._finish(r, "cancelled")
        self._admit()
        decoders, chunks = self._select()
        if not decoders and not chunks:
            return []
        self.stats.iterations += 1
        t0 = time.monotonic()
        pure_decode = not chunks
        # media rows (feature overlay, shifted rotary positions) ride only in direct packets
        has_media = any(r.rope_delta for r in decoders) or \
            any(r.media or r.rope_positions is not None for r, _ in chunks)
        if has_media:
            tokens, logits, order = self._run_direct(decoders, chunks)
            produced = self._commit(order, tokens, logits)
            self._capture_snapshots(chunks)
            return produced
        if pure_decode and self.spec.enabled:
            produced = self.spec.run(decoders)
            if produced is not None:
                return produced
        use_graph = (self.on_gpu and pure_decode and
                     self.load.cuda_graph.uses_graph(ExecPhase.DECODE) and
                     len(decoders) <= DECODE_BUCKETS[-1])
        early: List[Request] = []
        if use_graph:
            tokens, logits, order = self._run_decode_graph(decoders)
        elif (decoders and self.sched.prefill_stages > 1
              and sum(n for _, n in chunks) >= self.sched.layered_min_rows
              and getattr(self.runner, "supports_stages", False)):
            tokens, logits, order = self._run_layered(decoders, chunks, early)
        else:
            # prompt chunks do not stop speculation: greedy decoders bring their drafts into
            # the same packet as verification rows (attention-only models)
            drafts = None
            if chunks and decoders and self.spec.enabled and not self.recurrent \
                    and self._mixed_verify:
                room = min(self.max_rows, self.row_cap) - len(decoders) - sum(n for _, n in chunks)
                drafts = self.spec.plan_mixed(decoders, room)
            tokens, logits, order = self._run_direct(decoders, chunks, drafts)
        t1 = time.monotonic()
        produced = early + [r for r in self._commit(order, tokens, logits) if r not in early]
        self._capture_snapshots(chunks)
        t2 = time.monotonic()
        self.stats.batch_commit_s += t2 - t1
        if pure_decode:
            dt = t2 - t0
            self.tpot_ewma = dt if self.tpot_ewma is None else 0.8 * self.tpot_ewma + 0.2 * dt
            if not use_graph or self._step_was_replay:     # warm-up / capture steps say nothing
                self.spec.observe_normal(len(decoders), dt)
        elif chunks:
            toks = sum(n for _, n in chunks)
            rate = toks / max(t2 - t0, 1e-6)
            prev = getattr(self, "_prefill_tok_s", None)
            self._prefill_tok_s = rate if prev is None else 0.8 * prev + 0.2 * rate
            self.costs.observe(t2 - t0, tokens=toks,
                               context=max(r.offset for r, _ in chunks),
                               decode_rows=len(decoders),
                               decode_context=max((r.offset for r in decoders), default=0) + 1)
        return produced

    # ------------------------------------------------------------------ execution
    def _pinned(self, name: str, n: int) -> torch.Tensor:
        buf = self._pin.get(name)
        if buf is None or buf.numel() < n:
            buf = torch.empty(max(n, 1024), dtype=torch.int32)
            if self.on_gpu:
                buf = buf.pin_memory()
            self._pin[name] = buf
        return buf

    def _upload(self, name: str, values: List[int]) -> torch.Tensor:
        n = len(values)
        host = self._pinned(name, n)
        host[:n] = torch.tensor(values, dtype=torch.int32)
        if not self.on_gpu:
            return host[:n].clone()
        return host[:n].to(self.device, non_blocking=True)

    STAGE_BYTES = 4 << 20

    def _upload_many(self, parts: Dict[str, Optional[List[int]]]) -> Dict[str, torch.Tensor]:
        """All index arrays of one packet in ONE host-to-device copy: the arrays are written
        at 128-byte aligned offsets into a region of a pinned staging ring (regions are handed
        out in submission order and reused only after the copy that read them has completed),
        copied as one block, and returned as int32 views of that block.  ``None`` entries are
        skipped.  Packets too large for the ring, and engines started with
        ``ORINFER_PACKED_UPLOAD=0``, upload every array on its own."""
        names = [k for k, v in parts.items() if v is not None]
        if self._packed_uploads:
            try:
                return self._upload_packed(parts, names)
            except Exception as exc:               # noqa: BLE001 - the plain path always works
                import sys
                print(f"packed uploads switched off after {type(exc).__name__}: {exc}",
                      file=sys.stderr, flush=True)
                self._packed_uploads = False
        return {k: self._upload(k, parts[k]) for k in names}

    def _upload_packed(self, parts, names) -> Dict[str, torch.Tensor]:
        offs, total = {}, 0
        for k in names:
            offs[k] = total
            total += (4 * len(parts[k]) + 127) // 128 * 128
        if total == 0 or total > self.STAGE_BYTES // 4:
            return {k: self._upload(k, parts[k]) for k in names}
        from ..core import transfers
        if self._stage is None:
            self._stage = torch.empty(self.STAGE_BYTES, dtype=torch.uint8)
            if self.on_gpu:
                self._stage = self._stage.pin_memory()
            self._stage_np = self._stage.numpy()
            self._stage_ring = transfers.StagingRing(self.STAGE_BYTES, 256)
            self._stage_inflight: Deque[tuple] = collections.deque()
        while self._stage_inflight and self._stage_inflight[0][1].query():
            self._stage_ring.retire_through(self._stage_inflight.popleft()[0])
        got = self._stage_ring.acquire(total)
        if got is None:                          # ring full: wait for the copies in flight
            while self._stage_inflight:
                ticket, event = self._stage_inflight.popleft()
                event.synchronize()
                self._stage_ring.retire_through(ticket)
            got = self._stage_ring.acquire(total)
            if got is None:
                return {k: self._upload(k, parts[k]) for k in names}
        ticket, base = got
        image = self._stage_np[base:base + total]
        ranges = transfers.pack_inputs(
            image, [(offs[k], np.asarray(parts[k], dtype=np.int32)) for k in names],
            merge_gap=128)
        if not ranges:
            self._stage_ring.retire_through(ticket)
            return {k: self._upload(k, parts[k]) for k in names}
        lo, hi = ranges[0][0], ranges[-1][0] + ranges[-1][1]
        block = self._stage[base + lo:base + hi]
        if self.on_gpu:
            dev = block.to(self.device, non_blocking=True)
            event = torch.cuda.Event()
            event.record()
            self._stage_inflight.append((ticket, event))
        else:
            dev = block.clone()
            self._stage_ring.retire_through(ticket)
        self.stats.packed_uploads += 1
        out = {}
        for k in names:
            o, n = offs[k] - lo, 4 * len(parts[k])
            out[k] = dev[o:o + n].view(torch.int32) if n else \
                torch.empty(0, dtype=torch.int32, device=dev.device)
        return out

    # ------------------------------------------------------------------ device commands
    def _publish(self, op: str, payload=None) -> None:
        if self.channel is not None:
            self.channel.publish(op, payload)

    def _set_page_row(self, slot: int, pages: Sequence[int]) -> None:
        pages = [int(p) for p in pages]
        self._publish("page_row", (slot, pages))
        row = self.page_table_host[slot]
        row[:] = 0
        row[:len(pages)] = pages
        self.page_table_dev[slot].copy_(torch.from_numpy(row), non_blocking=True)

    def apply(self, op: str, payload) -> None:
        """Follower side: executes one published device command.  A follower engine takes no
        decisions of its own and reads nothing back but its status word."""
        if op == "page_row":
            self._set_page_row(*payload)
        elif op == "direct":
            self._exec_direct(self._build_packet(payload), payload, False)
        elif op == "decode":
            self._exec_decode(*payload)
        elif op == "verify":
            packet = self._verify_packet(*payload)
            self.runner.greedy(packet, need_logits=bool(payload[4]))
        elif op == "verify_commit":
            self._verify_commit(payload)
        elif op == "state_copy":
            self._state_copy(*payload)
        elif op == "mtp_capture":
            self._mtp_capture(payload)
        elif op == "mtp_draft":
            self._mtp_draft(payload)
        elif op == "mtp_forget":
            self._mtp_forget(payload)
        elif op == "host_kv":
            kind, *args = payload
            if self.host_kv is None:
                raise ValueError("host KV command without a host KV store on this rank")
            if kind == "save":
                page, expected = args
                if self.host_kv.save(page) != expected:
                    raise ValueError("host KV slots of this rank are out of step with the leader")
            else:
                getattr(self.host_kv, kind)(*args)
        elif op == "sharded":
            rows, options, uniforms = payload
            self.runner.sample_sharded(rows, options, uniforms)
        else:
            raise ValueError(f"unknown device command {op!r}")
        self._status_enqueue()

    def _verify_packet(self, ids, rows_req, pos, max_kv: int, need: bool,
                       seg_lens: Optional[Sequence[int]] = None) -> Packet:
        """Packet of a verification round (every row's token is read back).  With follower
        ranks the round is published first; they run the same packet through ``apply`` and
        take part in its collectives.  ``seg_lens`` (recurrent models): rows per request; the
        packet then runs tentatively, recurrent layers journal their rows, and
        ``_verify_commit`` keeps the accepted prefix of every request."""
        seg_lens = [int(n) for n in seg_lens] if seg_lens else None
        if seg_lens and sum(seg_lens) != len(ids):
            raise ValueError("segment lengths do not add up to the packet's rows")
        self._publish("verify", (list(ids), list(rows_req), list(pos), int(max_kv), bool(need),
                                 seg_lens))
        segs, first, start = [], [], 0
        for n in seg_lens or ():
            segs += [start, n, 0, 0]
            first += [start] * n
            start += n
        dev = self._upload_many({"ids": list(ids), "req": list(rows_req), "pos": list(pos),
                                 "segs": segs if seg_lens else None,
                                 "first": first if seg_lens else None})
        packet = Packet(dev["ids"], dev["req"], dev["pos"], self.page_table_dev, len(ids), max_kv)
        if seg_lens:
            packet.segments = dev["segs"].view(-1, 4)
            packet.row_first = dev["first"]
            packet.n_segments = len(seg_lens)
            packet.tentative = True
            self._tentative = packet
        return packet

    # Draft head: the hidden rows it consumes and the KV it writes are per-rank device data, so
    # the three things that touch them are published like packets.
    def _mtp_capture(self, keep, hidden=None) -> None:
        """``keep``: [(rid, first row, rows, first position)] of the packet that just ran; the
        rows' final hidden states are copied into the draft backlog."""
        keep = [tuple(int(v) for v in item) for item in keep]
        self._publish("mtp_capture", keep)
        if hidden is None:
            hidden = self.runner.final_hidden(max(row0 + n for _rid, row0, n, _pos in keep))
        for rid, row0, n, pos0 in keep:
            self._mtp_backlog.setdefault(rid, []).append((pos0, hidden[row0:row0 + n].clone()))

    def _mtp_forget(self, rid: int) -> None:
        if rid in self._mtp_backlog:
            self._publish("mtp_forget", int(rid))
            del self._mtp_backlog[rid]

    def _mtp_draft(self, plan: dict) -> List[torch.Tensor]:
        """One batched draft round: a head pass over the backlog rows of ``plan["rids"]``
        (catch-up plus the first draft, read at row ``last[i]`` of request i), then
        ``count - 1`` single-row passes that feed the head's own hidden state back.  Returns
        one token tensor [requests] per draft position."""
        self._publish("mtp_draft", plan)
        hids = []
        for rid in plan["rids"]:
            if rid not in self._mtp_backlog:
                raise ValueError(f"no draft backlog for request {rid} on this rank")
            hids += [h for _pos0, h in self._mtp_backlog.pop(rid)]
        rows = len(plan["toks"])
        if sum(h.shape[0] for h in hids) != rows:
            raise ValueError("the draft backlog of this rank is out of step with the leader")
        p = Packet(self._upload("mids", plan["toks"]), self._upload("mreq", plan["rreq"]),
                   self._upload("mpos", plan["rpos"]), self.page_table_dev, rows,
                   max(plan["rpos"]) + 1)
        dtok, dhid = self.runner.mtp_rows(p.ids, torch.cat(hids, dim=0), p)
        sel = torch.tensor(plan["last"], device=dtok.device)
        cur_tok, cur_hid = dtok[sel], dhid[sel]
        out = [cur_tok]
        live = len(plan["slots"])
        for j in range(1, plan["count"]):
            pos = [o - 1 + j for o in plan["offsets"]]
            p = Packet(cur_tok.to(torch.int32).contiguous(), self._upload("mreq", plan["slots"]),
                       self._upload("mpos", pos), self.page_table_dev, live, max(pos) + 1)
            cur_tok, cur_hid = self.runner.mtp_rows(p.ids, cur_hid, p)
            out.append(cur_tok)
        return out

    def _verify_commit(self, kept_rows: Sequence[int]) -> None:
        """Keeps the first ``kept_rows[i]`` rows of request ``i`` of the tentative packet in
        every recurrent layer, on every rank."""
        packet, self._tentative = self._tentative, None
        if packet is None:
            raise ValueError("commit without a tentative verification packet")
        kept_rows = [int(k) for k in kept_rows]
        if len(kept_rows) != packet.n_segments:
            raise ValueError("one kept-row count per request of the tentative packet")
        self._publish("verify_commit", kept_rows)
        self.runner.gdn_commit(packet, kept_rows)

    def _build_packet(self, spec: dict) -> Packet:
        rows = len(spec["ids"])
        chunked = bool(spec["chunks"] and self.on_gpu)
        dev = self._upload_many({
            "ids": spec["ids"], "req": spec["req"], "pos": spec["pos"], "sel": spec["sel"],
            "segs": spec["segs"] if self.recurrent else None,
            "first": spec["first"] if self.recurrent else None,
            "chunks": spec["chunks"] if chunked else None})
        packet = Packet(dev["ids"], dev["req"], dev["pos"], self.page_table_dev, rows,
                        spec["max_kv"], dev["sel"].long())
        if self.recurrent:
            packet.segments = dev["segs"].view(-1, 4)
            packet.row_first = dev["first"]
            packet.n_segments = len(spec["segs"]) // 4
        if chunked:
            packet.chunks = dev["chunks"].view(-1, 4)
            packet.max_q_len = max(spec["chunks"][1::4])
            packet.decode_rows = spec["n_decode"]
        return packet

    def _graph_eligible(self, spec: dict) -> bool:
        """A pure-prefill packet of a non-recurrent model in full-graph mode."""
        return bool(self.on_gpu and spec["n_decode"] == 0 and spec["chunks"]
                    and not self.recurrent
                    and getattr(self.runner, "stage_hook", None) is None
                    and self.cfg.head_dim in (64, 128, 256)
                    and self.load.cuda_graph.uses_graph(ExecPhase.PREFILL))

    @staticmethod
    def _geometry(spec: dict) -> tuple:
        return (tuple(spec["chunks"][1::4]), len(spec["sel"]), bool(spec["need"]))

    def _prefill_pool(self):
        pool = self.__dict__.get("_prefill_graphs")
        if pool is None:
            from ..parallel.graph_registry import GraphPool
            pool = self._prefill_graphs = GraphPool(self.PREFILL_GRAPHS, 2)
        return pool

    def _plan_prefill_graph(self, spec: dict):
        """Leading (or only) rank, before the packet is published: how this packet runs
        (None = not a graph candidate, else the registry's decision), so that every rank
        takes the same path.  Geometries a follower could not replay are dropped first: all
        ranks then capture them again."""
        if not self._graph_eligible(spec):
            return None
        pool = self._prefill_pool()
        if self.channel is not None:
            for key in self.channel.take_misses():
                pool.evict(key)
        decision, key, held, epoch = pool.plan(self._geometry(spec))
        self._graph_plan = (decision, key, held, epoch)
        return decision

    def take_graph_misses(self) -> list:
        """Follower side: keys of geometries this rank was asked to replay but holds no graph
        of (it ran them directly); reported to the leader with the acknowledgement."""
        out, self._graph_misses = getattr(self, "_graph_misses", []), []
        return out

    def _exec_direct(self, packet: Packet, spec: dict, has_media: bool):
        need = spec["need"]
        plan, self._graph_plan = getattr(self, "_graph_plan", None), None
        graphed = None
        if spec.get("graph") is not None and not has_media:
            if plan is None:                         # follower: carry out the leader's decision
                from ..parallel.graph_registry import key_of
                d, key, held, epoch, missed = self._prefill_pool().follow(
                    self._geometry(spec), spec["graph"])
                if missed:
                    self.__dict__.setdefault("_graph_misses", []).append(key)
                plan = (d, key, held, epoch)
            graphed = self._prefill_graph(packet, need, *plan)
        return graphed if graphed is not None else self.runner.greedy(packet, need_logits=need)

    def _run_direct(self, decoders: List[Request], chunks, drafts: Optional[dict] = None):
        """``drafts``: rid -> draft tokens of decoders that verify them in this packet (their
        rows are ``[pending, d1, ..]`` at consecutive positions, every row's token is read
        back, and ``_commit`` keeps the accepted prefix)."""
        t0 = time.monotonic()
        ids, req_rows, pos, logit_rows, order, chunk_rows = [], [], [], [], [], []
        max_kv = 1
        self._verify = {}
        for r in decoders:
            toks = [r.pending] + list((drafts or {}).get(r.rid, ()))
            first = len(ids)
            ids += toks
            req_rows += [r.slot] * len(toks)
            pos += list(range(r.offset, r.offset + len(toks)))
            logit_rows += list(range(first, first + len(toks)))
            order.append((r, len(toks), True))
            if len(toks) > 1:
                self._verify[r.rid] = (toks[1:], first)
            max_kv = max(max_kv, r.offset + len(toks))
        n_decode = len(ids)
        if self._verify:
            self.stats.mixed_verify_packets += 1
        for r, n in chunks:
            chunk_rows.append([len(ids), n, r.offset, r.slot])
            ids += r.prompt[r.offset:r.offset + n]
            req_rows += [r.slot] * n
            pos += list(range(r.offset, r.offset + n))
            last = r.offset + n == len(r.prompt)
            if last:
                logit_rows.append(len(ids) - 1)
            order.append((r, n, last))
            max_kv = max(max_kv, r.offset + n)
        rows = len(ids)
        if not logit_rows:
            logit_rows = [rows - 1]                 # keep shapes simple; result unused
            dummy_logits = True
        else:
            dummy_logits = False
        spec = dict(ids=ids, req=req_rows, pos=pos, sel=logit_rows, max_kv=max_kv,
                    n_decode=n_decode, chunks=[v for c in chunk_rows for v in c],
                    need=any(self._needs_logits(r) for r, _n, has in order if has))
        if self.recurrent:
            segs = [[i, 1, 0, 0] for i in range(n_decode)] + [[c[0], c[1], 0, 0] for c in chunk_rows]
            spec["segs"] = [v for g in segs for v in g]
            spec["first"] = list(range(n_decode)) + [c[0] for c in chunk_rows for _ in range(c[1])]
        media = self._has_media(decoders, chunks)
        spec["graph"] = None if media else self._plan_prefill_graph(spec)
        self._publish("direct", spec)
        packet = self._build_packet(spec)
        has_media = self._attach_media(packet, decoders, chunks, chunk_rows, pos)
        if has_media and self.channel is not None:
            raise ValueError("media inputs are not supported by a multi-rank engine")
        t1 = time.monotonic()
        self.stats.batch_inputs_s += t1 - t0
        tok, lg = self._exec_direct(packet, spec, has_media)
        self._status_enqueue()
        tokens = tok.cpu()                           # one readback (synchronises)
        self._status_check()
        self._direct_rows = rows
        if self.spec.enabled and self.runner_has_mtp():
            info, row0 = [], 0
            for r, n, _has in order:
                if r.rid not in self._verify:       # verified rows: captured once accepted
                    info.append((r, row0, n, r.offset))
                row0 += n
            self.spec.capture(info, self.runner.final_hidden(rows))
        self.stats.direct_packets += 1
        self.stats.direct_s += time.monotonic() - t1
        self.stats.prefill_tokens += sum(n for _, n in chunks)
        if dummy_logits:
            return None, None, order
        return tokens, lg, order

    @staticmethod
    def _has_media(decoders, chunks) -> bool:
        return bool(any(r.rope_delta for r in decoders)
                    or any(r.media or r.rope_positions is not None for r, _ in chunks))

    def _attach_media(self, packet: Packet, decoders, chunks, chunk_rows, pos) -> bool:
        """Feature overlay rows and (t, h, w) rotary positions of a direct packet."""
        if not self._has_media(decoders, chunks):
            return False
        rope = torch.tensor([pos, pos, pos], dtype=torch.int32)
        rows_idx, feats = [], []
        for i, r in enumerate(decoders):
            rope[:, i] += r.rope_delta
        for (r, n), (first, _n, off, _slot) in zip(chunks, chunk_rows):
            if r.rope_positions is not None:
                rope[:, first:first + n] = torch.as_tensor(
                    r.rope_positions[:, off:off + n], dtype=torch.int32)
            for m in r.media:
                lo, hi = max(m.start, off), min(m.end, off + n)
                if lo < hi:
                    rows_idx += list(range(first + lo - off, first + hi - off))
                    feats.append(m.features[lo - m.start:hi - m.start])
        packet.mrope = rope.to(self.device)
        if rows_idx:
            packet.overlay_rows = torch.tensor(rows_idx, dtype=torch.int64, device=self.device)
            packet.overlay = torch.cat(feats).to(self.device)
        return True

    def _run_layered(self, decoders: List[Request], chunks, produced: List[Request]):
        """Layered prefill: the prompt rows run as their own packet, paused at
        ``prefill_stages - 1`` layer boundaries; at every pause the live decoders take one
        ordinary step (graph replay where enabled) and their tokens are delivered, so a long
        prompt costs the decoders one stage, not one full forward, between tokens."""
        def between():
            live = [r for r in decoders if r.phase is Phase.DECODE and not r.cancelled]
            if not live:
                return
            if self.on_gpu:
                torch.cuda.current_stream().synchronize()   # the outer packet's uploads landed
            if (self.on_gpu and self.load.cuda_graph.uses_graph(ExecPhase.DECODE)
                    and len(live) <= DECODE_BUCKETS[-1]):
                tok, lg, order = self._run_decode_graph(live)
            else:
                tok, lg, order = self._run_direct(live, [])
            for r in self._commit(order, tok, lg):
                if r not in produced:
                    produced.append(r)
            self.stats.layered_decode_steps += 1
            trace.line("layered", decoders=len(live), prompt_rows=sum(n for _, n in chunks))

        self.runner.stage_hook = (self.sched.prefill_stages, between)
        try:
            return self._run_direct([], chunks)
        finally:
            self.runner.stage_hook = None

    PREFILL_GRAPHS = 16

    def _prefill_graph(self, packet: Packet, need: bool, decision: int, key: int, held, epoch: int):
        """Full-graph mode: a pure-prefill packet is replayed from a graph keyed by its launch
        geometry (chunk lengths, selected rows); token ids, positions, page-table rows and
        chunk offsets are data in static buffers.  The graph registry decides: a geometry is
        captured at its second use, the least recently used of PREFILL_GRAPHS entries is
        dropped.  Whatever the decision, the packet's kernels run exactly once in this call,
        so ranks that decide differently still issue the same collectives.  Returns (tokens,
        logits), or None when the packet must run directly."""
        from ..ops import native
        from ..parallel.graph_registry import CAPTURE, REPLAY
        if decision == REPLAY:
            e = held
            st = e["packet"]
            st.ids.copy_(packet.ids, non_blocking=True)
            st.row_req.copy_(packet.row_req, non_blocking=True)
            st.row_pos.copy_(packet.row_pos, non_blocking=True)
            st.logit_rows.copy_(packet.logit_rows, non_blocking=True)
            st.chunks.copy_(packet.chunks, non_blocking=True)
            e["graph"].replay()
            native.count_launches(e["launches"])         # kernels the replay launches
            self.stats.graph_hits += 1
            return e["tok"], e["lg"]
        if decision != CAPTURE:
            return None
        st = Packet(packet.ids.clone(), packet.row_req.clone(), packet.row_pos.clone(),
                    packet.page_table, packet.rows, packet.max_kv_len,
                    packet.logit_rows.clone(), chunks=packet.chunks.clone(),
                    max_q_len=packet.max_q_len, decode_rows=0)
        out = self.runner.greedy(st, need_logits=need)       # this step's run, outside capture
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        before = native.launches()
        with torch.cuda.graph(graph):                        # records only: nothing runs here
            tok, lg = self.runner.greedy(st, need_logits=need)
        entry = dict(graph=graph, packet=st, tok=tok, lg=lg, launches=native.launches() - before)
        native.count_launches(-entry["launches"])            # recorded, not launched
        if self._prefill_pool().commit(key, epoch, entry):
            self.stats.graph_captures += 1
        return out

    def _exec_decode(self, bucket: int, need: bool, ids, slots, pos, live) -> "_DecodeGraph":
        """One pure-decode packet of ``bucket`` rows (padded): warm, capture at the second
        use, replay afterwards.  ``ids is None``: the device buffers already hold this step's
        inputs (written by the previous step).  Returns the record holding the outputs."""
        t1 = time.monotonic()
        g = self._graphs.get((bucket, need))
        if g is None:
            g = self._graphs[(bucket, need)] = _DecodeGraph(self, bucket)
        if ids is not None:
            g.ids.copy_(self._upload("ids", ids), non_blocking=True)
            g.req.copy_(self._upload("req", slots), non_blocking=True)
            g.pos.copy_(self._upload("pos", pos), non_blocking=True)
            g.live.copy_(self._upload("live", live), non_blocking=True)

        def body():
            self.runner.greedy(g.packet, g.logits, g.tokens, need_logits=need)
            torch.clamp(g.tokens, min=0, out=g.ids)      # next step's inputs, on the device
            g.pos.add_(g.live)

        self._step_was_replay = g.graph is not None
        if g.graph is None:
            g.trials += 1
            body()                                       # warm
            if g.trials >= 2:
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                from ..ops import native
                before = native.launches()
                with torch.cuda.graph(graph):            # records only: nothing runs here
                    body()
                g.graph = graph
                g.local = getattr(self.runner, "_last_local", None)
                g.launches = native.launches() - before
                self.stats.graph_captures += 1
                self.stats.capture_s += time.monotonic() - t1
        else:
            g.graph.replay()
            if getattr(g, "local", None) is not None:
                self.runner._last_local = g.local        # this graph's sharded logits
            from ..ops import native
            native.count_launches(getattr(g, "launches", 0))
            self.stats.graph_hits += 1
        return g

    def _run_decode_graph(self, decoders: List[Request]):
        t0 = time.monotonic()
        n = len(decoders)
        bucket = next(b for b in DECODE_BUCKETS if b >= n)
        need = any(self._needs_logits(r) for r in decoders)
        pad = bucket - n
        g = self._graphs.get((bucket, need))
        members = tuple(r.slot for r in decoders)
        resident = (g is not None and g.graph is not None and g.members == members
                    and all(self._plain(r) for r in decoders)
                    and all(r.offset == p for r, p in zip(decoders, g.host_pos)))
        if resident:
            self._publish("decode", (bucket, need, None, None, None, None))
            args = (None, None, None, None)
            self.stats.resident_steps += 1
        else:
            args = ([r.pending for r in decoders] + [0] * pad,
                    [r.slot for r in decoders] + [self.pad_slot] * pad,
                    [r.offset for r in decoders] + [0] * pad, [1] * n + [0] * pad)
            self._publish("decode", (bucket, need, *args))
        t1 = time.monotonic()
        self.stats.batch_inputs_s += t1 - t0
        g = self._exec_decode(bucket, need, *args)
        g.members = members
        g.host_pos = [r.offset + 1 for r in decoders]    # what the device holds after this step
        self._status_enqueue()
        tokens = g.tokens[:n].cpu()
        self._status_check()
        if self.spec.enabled and self.runner_has_mtp():
            self.spec.capture([(r, i, 1, r.offset) for i, r in enumerate(decoders)],
                              self.runner.final_hidden(n))
        self.stats.replay_s += time.monotonic() - t1
        order = [(r, 1, True) for r in decoders]
        return tokens, g.logits, order

    # ------------------------------------------------------------------ commit
    def _sharded(self, r: Request) -> bool:
        """Under a vocabulary-sharded head: drawn from per-rank candidates, no logit gather."""
        return (hasattr(self.runner, "sample_sharded") and not self._plain(r)
                and r.constraint is None and not r.want_logprobs and r.sampling.device_topk)

    def _needs_logits(self, r: Request) -> bool:
        return not self._plain(r) and not self._sharded(r)

    def _sharded_samples(self, order) -> Dict[int, int]:
        rows, reqs, sel = [], [], 0
        for r, n, has_logits in order:
            if not has_logits:
                continue
            if self._sharded(r):
                rows.append(sel)
                reqs.append(r)
            sel += self._logit_rows(r, n)
        if not rows:
            return {}
        options = [r.sampling for r in reqs]
        uniforms = [S.counter_uniform(r.sampling.seed, 0, len(r.generated)) for r in reqs]
        self._publish("sharded", (rows, options, uniforms))
        toks = self.runner.sample_sharded(rows, options, uniforms)
        self.stats.sharded_samples += len(rows)
        return dict(zip(rows, toks))

    def _device_samples(self, order, logits) -> Dict[int, int]:
        """Rows whose sampling options need no host state are drawn by one launch of the
        device top-k sampler (same counter-RNG uniform as the host law); only their tokens
        cross PCIe instead of a full row of logits each."""
        if not self.on_gpu or logits is None or not logits.is_cuda:
            return {}
        rows, reqs, sel = [], [], 0
        for r, n, has_logits in order:
            if not has_logits:
                continue
            if (not self._plain(r) and not self._sharded(r) and r.constraint is None
                    and not r.want_logprobs and r.sampling.device_topk):
                rows.append(sel)
                reqs.append(r)
            sel += self._logit_rows(r, n)
        if not rows:
            return {}
        from ..ops import functional as F
        dev = self.device
        f64 = lambda v: torch.tensor(v, dtype=torch.float64, device=dev)
        idx = torch.tensor(rows, dtype=torch.int64, device=dev)
        tok, flag = F.sample_topk(
            logits.index_select(0, idx).float().contiguous(),
            torch.tensor([r.sampling.top_k for r in reqs], dtype=torch.int32, device=dev),
            f64([r.sampling.temperature for r in reqs]), f64([r.sampling.top_p for r in reqs]),
            f64([S.counter_uniform(r.sampling.seed, 0, len(r.generated)) for r in reqs]))
        tok, flag = tok.cpu().tolist(), flag.cpu().tolist()
        self.stats.device_samples += len(rows)
        return {row: t for row, t, f in zip(rows, tok, flag) if not f}

    def _logit_rows(self, r: Request, n: int) -> int:
        """Rows of the logit selection that belong to an entry with logits: every row of a
        decoder that verifies drafts, else one."""
        return n if r.rid in self._verify else 1

    def _commit_verified(self, r: Request, n: int, tokens, sel: int) -> None:
        """A greedy decoder's verification rows inside a mixed packet: keep the longest draft
        prefix the model agrees with plus its own next token."""
        drafts, first = self._verify[r.rid]
        commit = S.greedy_commit(drafts, tokens[sel:sel + n])
        accepted = len(commit) - 1
        self.spec.observe_mixed(r, drafts, accepted)
        if self.runner_has_mtp():
            self.spec.capture([(r, first, 1 + accepted, r.offset)],
                              self.runner.final_hidden(self._direct_rows))
        r.offset += 1 + accepted
        self.stats.decode_tokens += n
        for tok in commit:
            if r.finished:
                break
            self._deliver(r, int(tok))

    def _commit(self, order, tokens, logits) -> List[Request]:
        produced = []
        sel = 0
        now = time.monotonic()
        drawn = self._sharded_samples(order)
        drawn.update(self._device_samples(order, logits))
        if isinstance(tokens, torch.Tensor):      # one conversion, not one tensor index per row
            tokens = tokens.tolist()
        for r, n, has_logits in order:
            was_decode = r.phase is Phase.DECODE
            if was_decode and r.rid in self._verify:
                self._commit_verified(r, n, tokens, sel)
                sel += n
                produced.append(r)
                continue
            r.offset += n
            if not was_decode:
                r.last_prefill_at = now
            if not has_logits:
                continue
            row = sel
            sel += 1
            if was_decode:
                self.stats.decode_tokens += 1
            tok = drawn[row] if row in drawn else self._sample_or_fail(r, tokens, logits, row)
            if tok is not None:
                self._deliver(r, tok)
            produced.append(r)
        self._verify = {}
        return produced

    def _deliver(self, r: Request, tok: int) -> None:
        """Commit one sampled token: history, callbacks, stop conditions."""
        r.pending = tok
        r.generated.append(tok)
        if r.first_token_at is None:
            r.first_token_at = time.monotonic()
        r.phase = Phase.DECODE
        if r.on_token is not None:
            r.on_token(r, tok)
        if tok in r.stop_ids and not r.ignore_eos:
            self._finish(r, "stop")
        elif len(r.generated) >= r.max_new:
            self._finish(r, "length")
        elif r.constraint is not None and getattr(r.constraint, "finished", lambda: False)():
            self._finish(r, "stop")

    def runner_has_mtp(self) -> bool:
        return (self.w.mtp is not None and hasattr(self.runner, "mtp_rows")
                and self.load.mtp_drafts != 0)

    @staticmethod
    def _plain(r: Request) -> bool:
        """Greedy, unconstrained, no probability report: the device argmax is the answer."""
        return (r.sampling.is_greedy and r.constraint is None and not r.want_logprobs
                and r.sampling.top_logprobs is None)

    def _sample_or_fail(self, r: Request, tokens, logits, row: int) -> Optional[int]:
        """The next token of ``r``, or None after the request was failed: what goes wrong
        while one request's token is chosen (its constraint rejects every token or cannot
        follow the grammar, its logits are not finite) ends that request with an error its
        client sees; the engine and the other requests carry on."""
        try:
            return self._sample(r, tokens, logits, row)
        except Exception as exc:                       # noqa: BLE001 - any failure of this row
            first = (str(exc).strip().splitlines() or [""])[0]
            self._fail_request(r, f"{type(exc).__name__}: {first}")
            return None

    def _fail_request(self, r: Request, message: str) -> None:
        r.error = message[:300]
        self.stats.failed_requests += 1
        self._finish(r, "error")

    def _sample(self, r: Request, tokens, logits, row: int) -> int:
        if self._plain(r):
            tok = int(tokens[row])
            if tok < 0:
                raise FloatingPointError("non-finite logits")
            return tok
        lg = logits[row].float().cpu().numpy()
        mask = None
        if r.constraint is not None:
            mask = r.constraint.mask(self.cfg.vocab)
        step = len(r.generated)
        u = S.counter_uniform(r.sampling.seed, 0, step)
        tok = S.sample(lg, r.history, r.sampling, u, mask)
        if r.want_logprobs or r.sampling.top_logprobs is not None:
            lp, top = S.logprobs(lg, r.history, r.sampling, tok, r.sampling.top_logprobs or 0,
                                 mask)
            r.logprobs.append((tok, lp, top))
        if r.constraint is not None:
            r.constraint.consume(tok)
        return tok
