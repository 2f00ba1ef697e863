"""Scheduler / LLM API on CPU: batching, chunked prefill, prefix cache, preemption, n-gram speculation exactness."""
import pytest
import torch

from blaze_b200.config import named_config
from blaze_b200.llm import LLM
from blaze_b200.sampler import SamplingParams
from blaze_b200.sched import PrefixCache, SpecCost, Acceptance, ngram_propose


def _llm(**kw):
    base = dict(device="cpu", dtype=torch.float32, max_seqs=8, max_model_len=256, use_graphs=False, seed=0)
    base.update(kw)
    return LLM(named_config("tiny"), **base)


def _prompts(n, L, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, 1024, (n, L), generator=g).tolist()


GREEDY = SamplingParams(temperature=0.0, max_tokens=12)


def test_generate_matches_single_request_runs():
    llm = _llm()
    ps = _prompts(5, 20)
    batch = llm.generate(ps, GREEDY)
    for p, o in zip(ps, batch):
        solo = _llm().generate([p], GREEDY)[0]
        assert o.token_ids == solo.token_ids
        assert o.finish_reason == "length" and len(o.token_ids) == 12


def test_chunked_prefill_equals_unchunked():
    ps = _prompts(3, 70, seed=1)
    a = _llm(chunk=2048).generate(ps, GREEDY)
    b = _llm(chunk=16).generate(ps, GREEDY)
    assert [o.token_ids for o in a] == [o.token_ids for o in b]


def test_prefix_cache_hit_gives_same_tokens():
    llm = _llm()
    base = _prompts(1, 64, seed=2)[0]
    first = llm.generate([base + [5, 6, 7]], GREEDY)[0]
    assert llm.sched.cache.entries, "the finished request should have left a snapshot"
    second = llm.generate([base + [5, 6, 7] + first.token_ids[:4] + [9]], GREEDY)[0]
    assert second.cached_tokens >= 64
    cold = _llm(enable_prefix_caching=False).generate([base + [5, 6, 7] + first.token_ids[:4] + [9]], GREEDY)[0]
    assert second.token_ids == cold.token_ids


def test_preemption_under_kv_pressure_keeps_outputs():
    ps = _prompts(6, 40, seed=3)
    want = [o.token_ids for o in _llm().generate(ps, SamplingParams(temperature=0.0, max_tokens=30))]
    small = _llm(kv_tokens=16 * 16, enable_prefix_caching=False)   # 16 pages: cannot hold six 70-token sequences
    got = small.generate(ps, SamplingParams(temperature=0.0, max_tokens=30))
    assert [o.token_ids for o in got] == want
    assert small.sched.stats.preemptions > 0
    assert small.engine.pages.free_count == small.engine.num_pages - 1


def test_ngram_speculation_is_exact():
    rep = [3, 4, 5, 6, 7, 8] * 6
    ps = [rep, _prompts(1, 30, seed=4)[0]]
    want = [o.token_ids for o in _llm().generate(ps, SamplingParams(temperature=0.0, max_tokens=24))]
    spec = _llm(spec_method="ngram")
    got = spec.generate(ps, SamplingParams(temperature=0.0, max_tokens=24))
    assert [o.token_ids for o in got] == want
    assert spec.sched.stats.draft_tokens > 0


def test_chain_drafts_padded_to_one_length_stay_exact():
    """When the engine says that a uniform verify step can replay a captured graph, the scheduler pads every draft of the
    step to the longest one.  The filler rows are verified like any draft, so the streams do not change, and only the
    drafter's own tokens are counted as drafted."""
    rep = [3, 4, 5, 6, 7, 8] * 6
    ps = [rep, _prompts(1, 30, seed=4)[0], rep[2:] + rep[:2]]
    sp = SamplingParams(temperature=0.0, max_tokens=24)
    want = [o.token_ids for o in _llm().generate(ps, sp)]
    plain = _llm(spec_method="ngram")
    plain.generate(ps, sp)
    spec = _llm(spec_method="ngram")
    asked = []
    spec.engine.verify_graphable = lambda seqs, rows: (asked.append((seqs, rows)), True)[1]
    shapes = []
    fwd = spec.engine.forward
    spec.engine.forward = lambda chunks, mode="greedy", hidden_in=None, feedback=False: (
        shapes.append([len(c.tokens) for c in chunks]), fwd(chunks, mode, hidden_in, feedback))[1]
    got = spec.generate(ps, sp)
    assert [o.token_ids for o in got] == want
    assert asked and any(len(set(sh)) == 1 and sh[0] > 1 and len(sh) == 3 for sh in shapes), "no uniform verify step was planned"
    # the second prompt has nothing to look up: without padding its steps would have had one row
    assert spec.sched.stats.draft_tokens <= plain.sched.stats.draft_tokens + 3 * 24
    assert spec.sched.stats.accepted_tokens <= spec.sched.stats.draft_tokens


def test_sampled_generation_is_seeded():
    ps = _prompts(2, 16, seed=5)
    sp = SamplingParams(temperature=0.8, top_k=20, top_p=0.9, seed=7, max_tokens=8)
    a = [o.token_ids for o in _llm().generate(ps, sp)]
    b = [o.token_ids for o in _llm().generate(ps, sp)]
    assert a == b
    c = [o.token_ids for o in _llm().generate(ps, SamplingParams(temperature=0.8, top_k=20, top_p=0.9, seed=8, max_tokens=8))]
    assert a != c


def test_stop_token_and_logprobs():
    llm = _llm()
    p = _prompts(1, 10, seed=6)[0]
    free = llm.generate([p], SamplingParams(temperature=0.0, max_tokens=10, logprobs=3))[0]
    assert len(free.logprobs) == 10 and all(len(l["top"]) == 3 for l in free.logprobs)
    assert all(l["logprob"] <= 0 for l in free.logprobs)
    stop_at = free.token_ids[4]
    cut = llm.generate([p], SamplingParams(temperature=0.0, max_tokens=10, stop_token_ids=(stop_at,)))[0]
    assert cut.finish_reason == "stop" and cut.token_ids[-1] == stop_at and len(cut.token_ids) <= 5


def test_spec_cost_and_ngram_helpers():
    assert ngram_propose([1, 2, 3, 9, 1, 2, 3], 2) == [9, 1]
    assert ngram_propose([1, 2, 3], 2) == []
    acc = Acceptance()
    for _ in range(20):
        acc.record(4, 4)
    bad = Acceptance()
    for _ in range(20):
        bad.record(4, 0)
    cost = SpecCost()
    for rows in (1, 2, 4, 8, 16):
        cost.observe(rows, 10.0 * rows)
    k = cost.choose([acc, bad], [4, 4])
    assert k[0] >= k[1] and k[1] <= 1
    for rows in (1, 2, 4, 8, 16):
        for _ in range(30):
            cost.observe(rows, 10.0)
    k = cost.choose([acc, bad], [4, 4])
    assert k[0] >= 3


def test_mtp_drafter_keeps_outputs_exact():
    from blaze_b200.models.drafter import ChainDrafter
    ps = _prompts(3, 24, seed=9)
    want = [o.token_ids for o in _llm().generate(ps, SamplingParams(temperature=0.0, max_tokens=14))]
    llm = _llm(spec_method="mtp")
    d = ChainDrafter.random_init(llm.model, seed=3, max_seqs=8, max_model_len=256, kv_dtype="fp32")
    llm.sched.drafter = d
    got = llm.generate(ps, SamplingParams(temperature=0.0, max_tokens=14))
    assert [o.token_ids for o in got] == want
    assert llm.sched.stats.draft_tokens > 0 and d.proposed > 0
    assert not d.states and d.engine.pages.free_count == d.engine.num_pages - 1


def test_mtp_drafter_catch_up_feed_in_pieces():
    """The drafter's first pass over a prompt's confirmed (token, hidden) pairs is cut into passes of bounded rows (a step
    must fit the tensor-parallel exchange buffers); the pieces, including requests cut in the middle, give the same drafts."""
    from blaze_b200.models.drafter import ChainDrafter
    ps = _prompts(3, 37, seed=9)
    sp = SamplingParams(temperature=0.0, max_tokens=10)
    outs = []
    for limit in (4096, 4):
        llm = _llm(spec_method="mtp")
        d = ChainDrafter.random_init(llm.model, seed=3, max_seqs=8, max_model_len=256, kv_dtype="fp32")
        d.MAX_FEED_ROWS = limit
        llm.sched.drafter = d
        fed = []
        fwd = d.engine.forward
        d.engine.forward = lambda chunks, mode="greedy", hidden_in=None, feedback=False: (
            fed.append(sum(len(c.tokens) for c in chunks)), fwd(chunks, mode, hidden_in, feedback))[1]
        toks = [o.token_ids for o in llm.generate(ps, sp)]
        outs.append((toks, llm.sched.stats.draft_tokens, llm.sched.stats.accepted_tokens, max(fed)))
    assert outs[0][0] == outs[1][0]
    assert outs[0][1:3] == outs[1][1:3]                      # same drafts, same acceptance
    assert outs[0][3] > 4 >= outs[1][3]


def _ahead_llm(**kw):
    llm = _llm(**kw)
    llm.engine.ecfg.feedback_eager = True        # token feedback without captured graphs, so the loop runs on CPU
    return llm


def test_run_ahead_decode_is_exact_and_used():
    ps = _prompts(5, 20, seed=11)
    want = [o.token_ids for o in _llm().generate(ps, GREEDY)]
    llm = _ahead_llm()
    fed = []
    fwd = llm.engine.forward
    llm.engine.forward = lambda chunks, mode="greedy", hidden_in=None, feedback=False: (fed.append(feedback), fwd(chunks, mode, hidden_in, feedback))[1]
    got = llm.generate(ps, GREEDY)
    assert [o.token_ids for o in got] == want
    assert sum(fed) >= 8, "decode steps should have been launched ahead of the host"
    assert llm.engine.pages.free_count + sum(len(e.snap.pages) for e in llm.sched.cache.entries) >= 1


def test_run_ahead_stops_on_eos_seen_late_and_admits_new_requests():
    ps = _prompts(4, 24, seed=12)
    ref = _llm().generate(ps, SamplingParams(temperature=0.0, max_tokens=20))
    # make a token that request 0 produces mid-way its stop token: the host learns of it one step late
    stop = ref[0].token_ids[7]
    sp = [SamplingParams(temperature=0.0, max_tokens=20, stop_token_ids=[stop])] + [SamplingParams(temperature=0.0, max_tokens=20)] * 3
    want = _llm().generate(ps, sp)
    llm = _ahead_llm(max_seqs=4)
    extra = _prompts(1, 10, seed=13)[0]
    outs = {}

    def late(ev):
        outs.setdefault(ev.request_id, []).extend(ev.tokens or [])

    from blaze_b200.sched import GenRequest
    n = {"steps": 0}
    orig = llm.sched.step

    def step():
        n["steps"] += 1
        if n["steps"] == 6:      # arrives while steps are in flight
            llm.sched.submit(GenRequest("late", extra, SamplingParams(temperature=0.0, max_tokens=6), sink=late))
        orig()

    llm.sched.step = step
    got = llm.generate(ps, sp)
    assert [o.token_ids for o in got] == [o.token_ids for o in want]
    assert got[0].finish_reason == "stop" and len(got[0].token_ids) <= 8
    solo = _llm().generate([extra], SamplingParams(temperature=0.0, max_tokens=6))[0]
    assert outs["late"] == solo.token_ids
    llm.sched.cache.clear()
    assert llm.engine.pages.free_count == llm.engine.num_pages - 1


def test_host_kv_tier_restores_evicted_snapshots():
    """With one device cache slot, a second conversation pushes the first one's snapshot to the host tier; when the first
    conversation comes back its prefix is restored from there and the tokens equal a cold run."""
    a = _prompts(1, 64, seed=21)[0]
    b = _prompts(1, 64, seed=22)[0]
    follow = a + [5, 6, 7, 8, 9]
    cold = _llm(enable_prefix_caching=False).generate([follow], GREEDY)[0]
    llm = _llm(cache_slots=1, kv_host_tokens=64 * 16)
    llm.generate([a], GREEDY)
    llm.generate([b], GREEDY)                       # evicts a's snapshot(s) to the host
    cache = llm.sched.cache
    assert cache.host is not None and cache.host_entries and cache.host.spilled_pages > 0
    free_before = llm.engine.pages.free_count
    got = llm.generate([follow], GREEDY)[0]
    assert cache.host_hits == 1 and cache.host.restored_pages > 0
    assert got.cached_tokens >= 48
    assert got.token_ids == cold.token_ids
    # nothing leaks: dropping every snapshot returns every page and every host page
    cache.clear()
    assert llm.engine.pages.free_count == llm.engine.num_pages - 1
    assert cache.host.free_pages == cache.host.capacity
    assert free_before > 0


def test_prefill_first_schedule_keeps_tokens_and_defers_decode_rows():
    ps = _prompts(6, 40, seed=31)
    sp = SamplingParams(temperature=0.0, max_tokens=10)
    want = [o.token_ids for o in _llm(chunk=48).generate(ps, sp)]
    llm = _llm(chunk=48, schedule="prefill_first")
    llm.sched.cfg.max_decode_stall = 3600.0           # never force decode rows into a prefill step in this test
    mixed = []
    fwd = llm.engine.forward

    def spy(chunks, mode="greedy", hidden_in=None, feedback=False):
        lens = [len(c.tokens) for c in chunks]
        mixed.append(any(n == 1 for n in lens) and any(n > 1 for n in lens))
        return fwd(chunks, mode, hidden_in, feedback)
    llm.engine.forward = spy
    got = [o.token_ids for o in llm.generate(ps, sp)]
    assert got == want
    assert sum(mixed) <= 1, "decode rows should sit out while prompts are being read"


def test_steps_left_in_flight_give_the_same_results():
    """Chunked prefill, KV pressure with preemption and prefix-cache reuse with launched-but-unread steps (the overlap the
    GPU path uses) must give the tokens of the step-by-step scheduler."""
    ps = _prompts(6, 70, seed=41)
    sp = SamplingParams(temperature=0.0, max_tokens=14)
    want = [o.token_ids for o in _llm(chunk=32).generate(ps, sp)]
    for schedule in ("interleave", "prefill_first"):
        llm = _ahead_llm(chunk=32, schedule=schedule)
        seen_pending = []
        orig = llm.sched.step

        def step(orig=orig, llm=llm, seen_pending=seen_pending):
            orig()
            seen_pending.append(llm.sched._pending is not None)
        llm.sched.step = step
        got = [o.token_ids for o in llm.generate(ps, sp)]
        assert got == want, schedule
        assert any(seen_pending), "some steps should have been left in flight"
    # KV pressure: preemption may hit a request whose step is still unread
    want2 = [o.token_ids for o in _llm().generate(_prompts(6, 40, seed=3), SamplingParams(temperature=0.0, max_tokens=30))]
    small = _ahead_llm(kv_tokens=16 * 16, enable_prefix_caching=False)
    got2 = [o.token_ids for o in small.generate(_prompts(6, 40, seed=3), SamplingParams(temperature=0.0, max_tokens=30))]
    assert got2 == want2 and small.sched.stats.preemptions > 0
    assert small.engine.pages.free_count == small.engine.num_pages - 1
    # prefix cache across requests
    llm = _ahead_llm()
    base = _prompts(1, 64, seed=2)[0]
    first = llm.generate([base + [5, 6, 7]], GREEDY)[0]
    second = llm.generate([base + [5, 6, 7] + first.token_ids[:4] + [9]], GREEDY)[0]
    cold = _llm(enable_prefix_caching=False).generate([base + [5, 6, 7] + first.token_ids[:4] + [9]], GREEDY)[0]
    assert second.cached_tokens >= 64 and second.token_ids == cold.token_ids


def test_cuda_sampler_eligibility_rules():
    from blaze_b200.sampler_cuda import eligible
    from blaze_b200.sampler import parse_pipeline
    assert eligible(SamplingParams(temperature=0.8, top_k=40, top_p=0.9))
    assert eligible(SamplingParams(temperature=0.0))
    assert not eligible(SamplingParams(temperature=0.8, top_p=0.9))                      # no top_k: full sort needed
    assert not eligible(SamplingParams(temperature=0.8, top_k=100))
    assert not eligible(SamplingParams(temperature=0.8, top_k=10, pipeline=parse_pipeline("top_k,temperature")))
    assert not eligible(SamplingParams(top_k=10, top_nsigma=0.5, pipeline=parse_pipeline("top_k,top_nsigma")))


def test_drafter_with_reduced_vocabulary_stays_exact():
    """A drafter that can only propose a subset of the vocabulary changes acceptance, never the tokens."""
    from blaze_b200.models.drafter import ChainDrafter
    ps = _prompts(3, 24, seed=9)
    sp = SamplingParams(temperature=0.0, max_tokens=14)
    want = [o.token_ids for o in _llm().generate(ps, sp)]
    llm = _llm(spec_method="mtp")
    d = ChainDrafter.random_init(llm.model, seed=3, max_seqs=8, max_model_len=256, kv_dtype="fp32")
    d.use_draft_vocab(range(0, 1024, 3))
    llm.sched.drafter = d
    got = llm.generate(ps, sp)
    assert [o.token_ids for o in got] == want
    assert d.proposed > 0 and d.draft_head.N == len(range(0, 1024, 3))


def test_ngram_tree_speculation_is_exact():
    """With branching n-gram drafts (several continuations of the same suffix, verified as one tree) greedy and seeded
    sampled outputs stay those of plain decoding, and some branch rows are accepted."""
    from blaze_b200.sched import ngram_propose_many
    from blaze_b200.tree import merge_chains
    assert ngram_propose_many([1, 2, 7, 7, 1, 2, 8, 8, 1, 2], 2, 3) == [[8, 8], [7, 7]]
    t = merge_chains([[5, 6, 7], [5, 9], [4]])
    assert t.token[1:] == [5, 6, 7, 9, 4] and t.parent == [-1, 0, 1, 2, 1, 0]
    # a history where "3 4" continues in two ways keeps offering a two-branch tree
    rep = [3, 4, 5, 6, 3, 4, 9, 6] * 5
    ps = [rep, _prompts(1, 30, seed=4)[0], [3, 4, 5, 3, 4, 7, 3, 4, 5, 3, 4]]
    for sp in (SamplingParams(temperature=0.0, max_tokens=24), SamplingParams(temperature=0.7, top_k=8, seed=11, max_tokens=16)):
        want = [o.token_ids for o in _llm().generate(ps, sp)]
        spec = _llm(spec_method="ngram", draft_tree_width=3)
        got = spec.generate(ps, sp)
        assert [o.token_ids for o in got] == want
        if sp.temperature == 0.0:
            assert spec.sched.stats.draft_tokens > 0
    assert spec.engine.pages.free_count > 0


def test_tree_rows_in_the_step_batch():
    """Depth positions, row-order KV slots and ancestor bit masks of a draft tree; causal masks for the other rows."""
    import numpy as np
    from blaze_b200.batch import SeqChunk, build_batch, tree_depths, tree_masks
    parents = [-1, 0, 0, 1, 2, 2]
    assert tree_depths(parents).tolist() == [0, 1, 1, 2, 2, 2]
    assert [int(m) & 0xFFFFFFFF for m in tree_masks(parents)] == [0b1, 0b11, 0b101, 0b1011, 0b10101, 0b100101]
    table = np.arange(1, 9, dtype=np.int32).reshape(2, 4)
    b = build_batch([SeqChunk(0, [9] * 6, 14, want_logits=6, parents=parents), SeqChunk(1, [7, 8], 3, want_logits=2)], table, "cpu")
    assert b.positions.tolist() == [14, 15, 15, 16, 16, 16, 3, 4]
    assert b.slot_mapping.tolist() == [1 * 16 + 14, 1 * 16 + 15, 2 * 16, 2 * 16 + 1, 2 * 16 + 2, 2 * 16 + 3, 5 * 16 + 3, 5 * 16 + 4]
    assert b.tree_mask.tolist() == [0b1, 0b11, 0b101, 0b1011, 0b10101, 0b100101, 0b1, 0b11]
    assert build_batch([SeqChunk(1, [7, 8], 3)], table, "cpu").tree_mask is None
    with pytest.raises(ValueError):
        tree_depths([-1, 1])


def test_speculation_on_a_recurrent_hybrid_is_exact():
    """Gated DeltaNet layers carry a recurrent state: verify rows must not advance it past rejected drafts.  The state
    update of speculative rows is deferred and replayed over the accepted rows, so n-gram speculation gives the tokens of
    plain decoding, rejected drafts included."""
    def hy(**kw):
        base = dict(device="cpu", dtype=torch.float32, max_seqs=8, max_model_len=256, use_graphs=False, seed=0)
        base.update(kw)
        return LLM(named_config("tiny-hybrid"), **base)
    rep = [3, 4, 5, 6, 7, 8] * 6
    ps = [rep, _prompts(1, 30, seed=4)[0], [9, 9, 9, 9, 9, 9, 9, 9, 9, 9, 9, 9]]
    sp = SamplingParams(temperature=0.0, max_tokens=24)
    want = [o.token_ids for o in hy().generate(ps, sp)]
    spec = hy(spec_method="ngram")
    got = spec.generate(ps, sp)
    assert [o.token_ids for o in got] == want
    st = spec.sched.stats
    assert st.draft_tokens > 0 and st.accepted_tokens < st.draft_tokens, "the test needs rejected drafts to mean anything"


def test_device_status_error_fails_the_step_and_serving_continues():
    """A kernel that gives up on a bounded wait leaves a code in the device status word.  The engine reads the word with
    every step's results: the running requests end with an error, the word is cleared, and the next request is served.
    (The device word is replaced by a host-side stand-in here; the kernels' side is tested against a silent peer on the GPU.)"""
    llm = _llm()
    ps = _prompts(2, 20, seed=9)
    want = [o.token_ids for o in llm.generate(ps, GREEDY)]
    codes = [0, 0, 2]          # the third status read of the next run reports "a peer rank's flag never arrived"

    def status():
        return codes.pop(0) if codes else 0
    llm.engine.status_source = status
    bad = llm.generate(ps, GREEDY)
    assert all(o.finish_reason == "error" and "device status 2" in (o.error or "") for o in bad)
    assert llm.sched.stats.failed == 1 and llm.engine.status_errors == 1 and llm.sched.health.errors == 1
    assert not llm.sched.active and llm.engine.pages.free_count == llm.engine.num_pages - 1 - sum(len(e.snap.pages) for e in llm.sched.cache.entries)
    good = llm.generate(ps, GREEDY)
    assert [o.token_ids for o in good] == want and all(o.finish_reason == "length" for o in good)


def test_watchdog_reports_a_step_that_does_not_return():
    import time
    llm = _llm()
    llm.engine.ecfg.hang_secs = 0.2
    seen = []
    llm.engine.start_watchdog(on_hang=seen.append)
    llm.engine.last_step_started = time.monotonic() - 1.0      # a step that has been running for a second
    llm.engine.last_step_what = "greedy rows=1 seqs=1"
    for _ in range(40):
        if seen:
            break
        time.sleep(0.05)
    assert seen and "engine hang" in seen[0] and llm.engine.hangs == 1


def test_multimodal_request_gets_mrope_positions_and_image_rows():
    """An image in the prompt: its pad tokens take the vision tower's rows as embeddings, rotary positions follow the
    three-axis layout (text after the image resumes from the block's largest position + 1), chunked prefill cuts through
    the image without changing the result, and the prefix cache tells two different images apart."""
    from blaze_b200.config import named_config
    from blaze_b200.mm import ImageEmbeds, MmInput
    from blaze_b200.sched import GenRequest
    cfg = named_config("tiny")
    cfg.rope.mrope_section = [8, 12, 12]                       # half of head_dim 64
    PAD = 1000

    def run(chunk, img_seed, cache=False):
        llm = LLM(cfg, device="cpu", dtype=torch.float32, max_seqs=4, max_model_len=256, use_graphs=False, seed=0, chunk=chunk,
                  enable_prefix_caching=cache)
        g = torch.Generator().manual_seed(img_seed)
        emb = torch.randn(12, cfg.hidden_size, generator=g) * 0.05          # a 3 x 4 grid of image tokens
        outs = []
        for rep in range(2 if cache else 1):
            mm = MmInput([ImageEmbeds(emb, (3, 4), 7000 + img_seed)], PAD)
            got = []
            llm.sched.submit(GenRequest(f"mm{rep}", [5, 6, 7, PAD, 8, 9, 10, 11], SamplingParams(temperature=0.0, max_tokens=8),
                                        mm=mm, sink=lambda ev: got.extend(ev.tokens or [])))
            llm.sched.run_until_idle()
            outs.append(got)
        return llm, outs
    llm, (a,) = run(64, 1)
    _, (b,) = run(5, 1)                       # prefill chunks of 5 rows cut through the 12-row image block
    assert a == b and len(a) == 8
    _, (c,) = run(64, 2)
    assert c != a, "a different image must change the continuation"
    # the rotary positions: 3 text rows, a 3 x 4 image block at temporal position 3, text resumes at 3 + max(3, 4) = 7
    mm = MmInput([ImageEmbeds(torch.zeros(12, 4), (3, 4), 1)], PAD)
    toks = mm.expand([5, 6, 7, PAD, 8, 9])
    p3 = mm.positions3(toks)
    assert p3[:, :3].tolist() == [[0, 1, 2]] * 3
    assert p3[0, 3:15].tolist() == [3] * 12 and p3[1, 3:15].tolist() == [3, 3, 3, 3, 4, 4, 4, 4, 5, 5, 5, 5]
    assert p3[2, 3:15].tolist() == [3, 4, 5, 6] * 3 and p3[:, 15].tolist() == [7, 7, 7]
    # same image twice: the second request reuses the cached prefix and gives the same tokens
    llm2, (x, y) = run(64, 1, cache=True)
    assert x == y == a


@pytest.mark.parametrize("kind,tree", [("eagle", 1), ("eagle", 3), ("dflash", 1)])
def test_eagle_and_dflash_drafters_keep_outputs_exact(kind, tree):
    """EAGLE-style (chains and level-by-level trees from its low-rank candidate head) and DFlash-style (one block pass)
    drafters through the product path (``LLM(spec_method=...)``): greedy and seeded sampled outputs are those of plain
    decoding, drafts are proposed, the drafter's pages are all returned."""
    ps = _prompts(3, 24, seed=21) + [[3, 4, 5, 6] * 6]
    for sp in (SamplingParams(temperature=0.0, max_tokens=14), SamplingParams(temperature=0.8, top_k=10, seed=5, max_tokens=10)):
        want = [o.token_ids for o in _llm().generate(ps, sp)]
        llm = _llm(spec_method=kind, draft_tree_width=tree, draft_tree_depth=3)
        assert llm.drafter is not None and llm.drafter.kind == kind
        got = llm.generate(ps, sp)
        assert [o.token_ids for o in got] == want
        assert llm.sched.stats.draft_tokens > 0 and llm.drafter.proposed > 0
        d = llm.drafter
        assert not d.states and d.engine.pages.free_count == d.engine.num_pages - 1
    if kind == "eagle":
        assert llm.model.capture_layers == d.capture_layers and len(d.capture_layers) >= 1


def test_spec_benchmark_harness_imposes_acceptance_and_checks_exactness():
    """The speculative benchmark's synthetic acceptance: the drafter still runs, its proposals are rewritten so that the first
    j are right (j seeded, uniform in 0..k), the streams equal the non-speculative ones, and a shared prompt prefix is
    served from the prefix cache."""
    from blaze_b200.benchmarks import spec
    llm = _llm(spec_method="mtp", max_draft=4, cache_slots=8)
    g = torch.Generator().manual_seed(2)
    shared = torch.randint(0, 1024, (64,), generator=g).tolist()
    prompts = [shared + torch.randint(0, 1024, (9,), generator=g).tolist() for _ in range(5)]
    r = spec.run(llm, prompts, out_tokens=20, k=4, seed=4, shared=64)
    assert r["exact"] and r["agreement"] == 1.0 and r["output_tokens"] == 100
    assert r["draft_tokens"] > 0 and 0.2 < r["acceptance"] < 0.8            # uniform j in 0..4 accepts half of the drafts on average
    assert sum(r["accepted_per_step_hist"]) > 0 and r["cached_prompt_tokens_spec"] >= 5 * 64
    assert r["cached_prompt_tokens_plain"] >= 5 * 64          # the shared head is in the cache before either timed pass
    assert r["steps"] < 5 * 20            # fewer target steps than tokens
