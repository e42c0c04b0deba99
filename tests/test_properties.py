"""Property tests (hypothesis): user text can never become control tokens; DSML calls survive
any chunking of the stream; the staging ring never hands out overlapping live regions."""
import json

from hypothesis import given, settings, strategies as st

from orinfer_b200.api import dsml
from orinfer_b200.api.chat_codec import ByteTokenizer
from orinfer_b200.api.token_boundary import Boundary

TOK = ByteTokenizer(1024)
BOUNDARY = Boundary(TOK)
SPELLINGS = list(TOK.special_ids)
text_with_controls = st.lists(
    st.one_of(st.text(max_size=12), st.sampled_from(SPELLINGS), st.just(BOUNDARY.prefix),
              st.just(BOUNDARY.prefix + "3;")), max_size=8).map("".join)


@settings(max_examples=200, deadline=None)
@given(text_with_controls)
def test_user_text_is_only_ever_plain_tokens(text):
    ids = BOUNDARY.encode(BOUNDARY.escape(text))
    assert all(i < 256 for i in ids)                              # no control token at all
    assert bytes(ids).decode("utf-8") == text                      # and nothing is lost


@settings(max_examples=200, deadline=None)
@given(text_with_controls, text_with_controls)
def test_template_controls_survive_next_to_user_text(before, after):
    rendered = (BOUNDARY.control("<|im_start|>") + BOUNDARY.escape(before)
                + BOUNDARY.control("<|im_end|>") + BOUNDARY.escape(after))
    ids = BOUNDARY.encode(rendered)
    controls = [i for i in ids if i >= 256]
    assert controls == [TOK.special_ids["<|im_start|>"], TOK.special_ids["<|im_end|>"]]
    assert bytes(i for i in ids if i < 256).decode("utf-8") == before + after


values = st.one_of(st.text(alphabet=st.characters(blacklist_categories=("Cs",),
                                                  blacklist_characters="<"), max_size=20),
                   st.integers(-10 ** 6, 10 ** 6), st.booleans(),
                   st.lists(st.integers(0, 9), max_size=4))
arguments = st.dictionaries(st.text(alphabet="abcdefgh_", min_size=1, max_size=6), values,
                            max_size=4)


@settings(max_examples=150, deadline=None)
@given(st.lists(st.tuples(st.sampled_from(["edit", "noop", "search"]), arguments), min_size=1,
                max_size=3), st.integers(1, 17))
def test_dsml_calls_round_trip_under_any_chunking(calls, step):
    text = dsml.render_calls([{"function": {"name": n, "arguments": json.dumps(a)}}
                              for n, a in calls])[len(dsml.OPEN):]
    machine = dsml.DsmlCalls()
    events = []
    for i in range(0, len(text), step):
        events += machine.feed(text[i:i + step])
    assert events[-1] == ("close",)
    got, current = [], None
    for ev in events:
        if ev[0] == "begin":
            current = [ev[1], ""]
        elif ev[0] == "arguments":
            current[1] += ev[1]
        elif ev[0] == "end":
            got.append((current[0], json.loads(current[1])))
    assert got == calls


@settings(max_examples=60, deadline=None)
@given(st.lists(st.one_of(st.integers(1, 500), st.just(-1)), min_size=1, max_size=80))
def test_staging_ring_regions_never_overlap(ops):
    from orinfer_b200.core.transfers import StagingRing
    ring = StagingRing(1024, 64)
    live = []
    for op in ops:
        if op < 0:
            if live:
                ring.retire_through(live[len(live) // 2][0])
                live = live[len(live) // 2 + 1:]
            continue
        got = ring.acquire(op)
        if got is None:
            continue
        ticket, off = got
        size = -(-op // 64) * 64
        assert off + size <= 1024
        for _, o, s in live:
            assert off + size <= o or o + s <= off
        live.append((ticket, off, size))


@settings(max_examples=150, deadline=None)
@given(st.integers(1, 500), st.integers(1, 9), st.data())
def test_row_plans_partition_unique_rows_by_owner(table_rows, ranks, data):
    import numpy as np
    from orinfer_b200.core.host_rows import RowPlan, row_shard
    ids = data.draw(st.lists(st.integers(0, table_rows - 1), max_size=60))
    plan = RowPlan.build(ids, table_rows, ranks)
    assert plan.rows[plan.restore].tolist() == ids if ids else plan.rows.size == 0
    assert len(set(plan.rows.tolist())) == plan.rows.size == len(set(ids))
    seen = []
    for r in range(ranks):
        first, count = row_shard(table_rows, ranks, r)
        mine = plan.for_rank(r).tolist()
        assert all(first <= x < first + count for x in mine)
        seen += mine
    assert seen == plan.rows.tolist()


@settings(max_examples=100, deadline=None)
@given(st.lists(st.integers(0, 15), min_size=1, max_size=30), st.integers(0, 29))
def test_ngram_addresses_do_not_depend_on_the_chunk_cut(tokens, cut):
    import numpy as np
    from orinfer_b200.core.host_rows import HashLayer, NgramHasher
    h = NgramHasher(list(range(16)), 0, [15], 2, [HashLayer(0, 5 + 7 + 11 + 13 + 17 + 19,
                                                            [3, 5, 7, 9], [5, 7, 11, 13, 17, 19])])
    cut = min(cut, len(tokens))
    whole, valid = h.hash([], tokens)
    a, va = h.hash([], tokens[:cut])
    b, vb = h.hash(tokens[:cut], tokens[cut:])
    assert np.array_equal(np.concatenate([a, b]), whole)
    assert np.array_equal(np.concatenate([va, vb]), valid)
    assert valid.tolist() == [t != 15 for t in tokens]


@settings(max_examples=200, deadline=None)
@given(st.integers(8, 4000), st.integers(8, 4000))
def test_resize_geometry_stays_on_the_grid_and_in_budget(h, w):
    from orinfer_b200.models import vision as V
    if max(h, w) / min(h, w) > 200:
        return
    lo, hi = 64 * 64, 1024 * 1024
    nh, nw = V.smart_resize(h, w, 32, lo, hi)
    assert nh % 32 == 0 and nw % 32 == 0 and nh >= 32 and nw >= 32
    assert nh * nw <= hi or min(nh, nw) == 32              # very thin images keep one row of patches
    assert nh * nw >= lo
    assert abs((nh / nw) / (h / w) - 1) < 0.35 or min(nh, nw) <= 64    # rounding to the grid


@settings(max_examples=100, deadline=None)
@given(st.lists(st.tuples(st.integers(0, 6), st.integers(1, 4), st.integers(1, 4)), max_size=4),
       st.integers(0, 6))
def test_rotary_positions_of_prompts_with_images(images, tail):
    """(text run, merged grid height, merged grid width) per image, then a text tail."""
    import numpy as np
    from orinfer_b200.models import vision as V
    spec = V.VisionSpec(hidden=8, image_token_id=9, vision_start_token_id=7, vision_end_token_id=8)
    tokens, spans, grids = [], [], []
    for run, gh, gw in images:
        tokens += [1] * run
        spans.append((len(tokens), len(tokens) + gh * gw))
        tokens += [9] * (gh * gw)
        grids.append((gh * 2, gw * 2))
    tokens += [1] * tail
    pos, delta = V.mrope_positions(spec, tokens, spans, grids)
    assert pos.shape == (3, len(tokens)) and delta <= 0
    assert np.all(np.diff(pos[0]) >= 0)                           # time never runs backwards
    text = np.array([t != 9 for t in tokens], dtype=bool)
    assert np.all(pos[0][text] == pos[1][text]) and np.all(pos[1][text] == pos[2][text])
    if not images:
        assert pos[0].tolist() == list(range(len(tokens))) and delta == 0
    for (a, b), (gh, gw) in zip(spans, grids):
        assert len(set(pos[0, a:b].tolist())) == 1                # one time step per image
        cells = set(zip(pos[1, a:b].tolist(), pos[2, a:b].tolist()))
        assert len(cells) == b - a                                # every feature its own cell
    assert int(pos.max(initial=-1)) + 1 == len(tokens) + delta    # where decoding continues


@settings(max_examples=25, deadline=None)
@given(st.integers(1, 40), st.sampled_from([(1, 1), (1, 2), (2, 4)]), st.sampled_from([8, 16]),
       st.integers(1, 20), st.integers(0, 2 ** 31 - 1))
def test_chunkwise_gated_delta_rule_is_the_sequential_one(t, heads, d, chunk, seed):
    import torch
    from orinfer_b200.ref import gdn_ref as G
    g = torch.Generator().manual_seed(seed)
    hk, hv = heads
    q = torch.nn.functional.normalize(torch.randn(t, hk, d, generator=g), dim=-1)
    k = torch.nn.functional.normalize(torch.randn(t, hk, d, generator=g), dim=-1)
    v = torch.randn(t, hv, d, generator=g)
    decay = -torch.rand(t, hv, generator=g)
    beta = torch.rand(t, hv, generator=g)
    s0 = torch.randn(hv, d, d, generator=g) * 0.2
    o1, s1 = G.recurrence(q, k, v, decay, beta, s0)
    o2, s2 = G.recurrence_chunked(q, k, v, decay, beta, s0, chunk)
    assert torch.allclose(o1, o2, atol=5e-5, rtol=1e-4) and torch.allclose(s1, s2, atol=5e-5, rtol=1e-4)


@settings(max_examples=60, deadline=None)
@given(st.lists(st.tuples(st.sampled_from(["insert", "match", "release", "evict"]),
                          st.integers(0, 5), st.integers(1, 4)), min_size=1, max_size=60))
def test_prefix_cache_never_evicts_a_page_in_use_and_matches_what_it_indexed(ops):
    """Random traffic on the radix prefix cache (4-token pages, six prompt families that share
    prefixes): a page handed out by a match is never evicted while held, a match returns pages
    that were indexed for exactly those tokens, and every adopted page is evicted at most once."""
    from orinfer_b200.core.prefix import RadixPrefixCache
    cache = RadixPrefixCache(page_tokens=4)
    family = lambda f, pages: [(f % 3) * 100 + i // 4 if i < 4 else f * 1000 + i // 4
                               for i in range(pages * 4)]     # families share their first page
    page_of = {}                      # (tuple of tokens up to a page end) -> page id
    held = {}                         # node id -> leases
    handles = []                      # node-id lists still to release
    evicted, next_page = set(), [1]
    for op, f, pages in ops:
        toks = family(f, pages)
        if op == "insert":
            ids = list(range(next_page[0], next_page[0] + pages))
            next_page[0] += pages
            adopted, _nodes = cache.insert(toks, ids)
            for i, (took, pg) in enumerate(zip(adopted, ids)):
                if took:
                    page_of[tuple(toks[:(i + 1) * 4])] = pg
        elif op == "match":
            nodes, got = cache.match(toks)
            for i, pg in enumerate(got):
                assert page_of[tuple(toks[:(i + 1) * 4])] == pg
                assert pg not in evicted
            for n in nodes:
                held[n] = held.get(n, 0) + 1
            if nodes:
                handles.append(nodes)
        elif op == "release" and handles:
            nodes = handles.pop(f % len(handles))
            cache.release(nodes)
            for n in nodes:
                held[n] -= 1
        elif op == "evict":
            for node, pg in cache.evict(pages):
                assert held.get(node, 0) == 0, "evicted a page that a request still reads"
                assert pg not in evicted
                evicted.add(pg)
                page_of = {k: v for k, v in page_of.items() if v != pg}
    st_ = cache.statistics()
    assert st_.device_pages == len(page_of) and st_.evicted == len(evicted)


@settings(max_examples=60, deadline=None)
@given(st.lists(st.tuples(st.sampled_from(["insert", "offload", "restore", "drop", "evict"]),
                          st.integers(0, 5), st.integers(1, 4)), min_size=1, max_size=80))
def test_host_tier_slots_are_never_lost_or_shared(ops):
    """Random traffic that moves pages between the device and a host slab of eight slots the
    way the engine does (offload = evict to host + record the slot; a hit restores and frees
    it; re-adoption of a host-resident node frees its stale slot; pressure drops host-only
    leaves): every slot is always either free or owned by exactly one indexed node."""
    from orinfer_b200.core.prefix import RadixPrefixCache
    cache = RadixPrefixCache(page_tokens=4)
    family = lambda f, pages: [(f % 3) * 100 + i // 4 if i < 4 else f * 1000 + i // 4
                               for i in range(pages * 4)]
    free = list(range(8))
    owner = {}                        # slot -> node id
    next_page = [1]

    def check():
        assert len(free) + len(owner) == 8 and not set(free) & set(owner)
        assert cache.statistics().host_pages == len(owner)
        for slot, node in owner.items():
            assert cache.host_handle(node) == slot

    for op, f, pages in ops:
        toks = family(f, pages)
        if op == "insert":
            ids = list(range(next_page[0], next_page[0] + pages))
            next_page[0] += pages
            adopted, nodes = cache.insert(toks, ids)
            for took, node in zip(adopted, nodes):
                stale = cache.host_handle(node) if took else -1
                if stale >= 0:                         # re-adopted: the host copy is redundant
                    cache.set_host(node, -1)
                    free.append(owner_pop(owner, stale, node))
        elif op == "offload":
            if not free:
                for slot in cache.drop_host(pages):
                    del owner[slot]
                    free.append(slot)
            for node, _page in cache.evict(min(pages, len(free)), to_host=True):
                slot = free.pop()
                cache.set_host(node, slot)
                owner[slot] = node
        elif op == "restore":
            nodes, got = cache.match(toks, acquire=False)
            for node, page in zip(nodes, got):
                if page >= 0:
                    continue
                slot = cache.host_handle(node)
                if slot < 0 or not cache.restore(node, next_page[0]):
                    break
                next_page[0] += 1
                cache.set_host(node, -1)
                free.append(owner_pop(owner, slot, node))
        elif op == "drop":
            for slot in cache.drop_host(pages):
                del owner[slot]
                free.append(slot)
        elif op == "evict":
            for node, _page in cache.evict(pages):
                assert cache.host_handle(node) < 0 and node not in owner.values()
        check()


def owner_pop(owner, slot, node):
    assert owner.pop(slot) == node
    return slot
