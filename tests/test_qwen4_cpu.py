"""Hyper-connections and the per-layer n-gram embedding (Qwen4-Exp): every formula against a scalar restatement in the
manner of the reference's kernel tests (``kernels/tests/test_qwen4.cu``, ``test_hc_mix.cu``), the hash against big-integer
arithmetic, and the model through the engine: chunked prefill, decode, prefix reuse and speculation agree with one pass."""
import math

import pytest
import torch

from blaze_b200.config import ModelConfig, named_config
from blaze_b200.llm import LLM
from blaze_b200.models import qwen4
from blaze_b200.sampler import SamplingParams


def test_config_reads_the_extras():
    raw = {"architectures": ["Qwen4ExpForConditionalGeneration"], "text_config": {
        "model_type": "qwen4_exp", "hidden_size": 64, "num_hidden_layers": 4, "num_attention_heads": 2, "head_dim": 32,
        "layer_types": ["linear_attention", "full_attention"] * 2, "linear_num_value_heads": 2, "linear_num_key_heads": 1,
        "linear_key_head_dim": 32, "linear_value_head_dim": 32, "hc_count": 4, "hc_lowrank": 8, "ple_layer_ids": [1, 3],
        "ngram_size": 3, "heads_per_ngram": 8, "ple_embed_dim": 32, "output_gate_type": "sigmoid", "eos_token_id": 7,
        "indexer_n_heads": 4, "indexer_head_dim": 64, "indexer_budget": 2048, "indexer_compress_ratio": 4}}
    c = ModelConfig.from_json(raw)
    assert c.has_hc and c.hc_count == 4 and c.hc_lowrank == 8 and c.ple_layers == [0, 2]
    assert (c.ngram_size, c.heads_per_ngram, c.ple_embed_dim, c.ple_conv_kernel) == (3, 8, 32, 4)
    assert c.gdn_output_gate == "sigmoid" and c.attn_output_gate and c.zero_centered_norm
    assert c.indexer_heads == 4 and c.indexer_budget == 2048
    assert not ModelConfig.from_json({"hc_count": 1}).has_hc


def test_grouped_norm_mix_and_combine_against_loops():
    g = torch.Generator().manual_seed(5)
    rows, HC, H, R, eps = 3, 4, 24, 6, 1e-6
    x = torch.randn(rows, HC * H, generator=g)
    w = torch.randn(HC * H, generator=g) * 0.1
    got = qwen4.grouped_norm(x, w, HC, eps)
    for r in range(rows):
        for c in range(HC):
            seg = x[r, c * H:(c + 1) * H].double()
            inv = 1.0 / math.sqrt(float((seg * seg).sum() / H) + eps)
            want = seg * inv * (1.0 + w[c * H:(c + 1) * H].double())
            assert torch.allclose(got[r, c * H:(c + 1) * H].double(), want, atol=1e-5)
    blk = qwen4.HcBlock()
    blk.norm = torch.zeros(HC * H)
    blk.down = torch.randn(R, HC * H, generator=g) * 0.2
    blk.up = torch.randn(HC * H, R, generator=g) * 0.5
    blk.inject = torch.randn(HC, HC * H, generator=g) * 0.1
    out, n = qwen4.hc_mix(x, blk, HC, eps)
    assert torch.allclose(n, qwen4.grouped_norm(x, blk.norm, HC, eps))
    for m in range(rows):
        t = []
        for k in range(R):
            a = float((n[m].double() * blk.down[k].double()).sum()) / HC
            t.append(a / (1.0 + math.exp(-a)))
        for j in range(H):
            o = 0.0
            for c in range(HC):
                u = sum(t[k] * float(blk.up[c * H + j, k]) for k in range(R))
                o += 1.0 / (1.0 + math.exp(-u)) * float(n[m, c * H + j])
            assert abs(float(out[m, j]) - o / HC) < 1e-5
    y = torch.randn(rows, H, generator=g)
    comb = qwen4.hc_combine(x, n, blk, y, HC)
    for r in range(rows):
        for c in range(HC):
            a = 2.0 / (1.0 + math.exp(-float((n[r].double() * blk.inject[c].double()).sum()) / HC))
            want = x[r, c * H:(c + 1) * H].double() + a * y[r].double()
            assert torch.allclose(comb[r, c * H:(c + 1) * H].double(), want, atol=1e-5)


def test_ngram_hash_against_big_integers():
    """Two sequences with end-of-sequence tokens inside and a carried history (the case of ``test_qwen4.cu``)."""
    eos = 248044
    mult = [123456789123, 98765432101, 55555555555]
    sizes = [20000003 + 2 * h for h in range(16)]
    offs = [sum(sizes[:h]) for h in range(16)]
    P = qwen4.Ple()
    P.mult, P.sizes, P.offs = torch.tensor(mult), torch.tensor(sizes), torch.tensor(offs)
    seqs = [([300, 301], [11, 12, eos, 13, 14, 15]), ([eos, eos], [7, eos, eos, 9])]
    mask = (1 << 64) - 1

    def s64(v):
        v &= mask
        return v - (1 << 64) if v >= 1 << 63 else v
    for hist, toks in seqs:
        win = hist + toks
        want = []
        for i in range(2, len(win)):
            w0, w1, w2 = win[i - 2], win[i - 1], win[i]
            reach = 0 if w1 == eos else (1 if w0 == eos else 2)
            t1 = w1 if reach >= 1 else eos
            t2 = w0 if reach >= 2 else eos
            m2 = s64((w2 * mult[0]) ^ (t1 * mult[1]))
            m3 = s64(m2 ^ (t2 * mult[2]))
            want.append([((m2 if h < 8 else m3) % sizes[h]) + offs[h] for h in range(16)])
        got = qwen4.ngram_ids(torch.tensor(win[2:]), torch.tensor(win[1:-1]), torch.tensor(win[:-2]), eos, P, 8)
        assert got.tolist() == want


def test_ple_gate_and_conv_carry_state_across_chunks():
    g = torch.Generator().manual_seed(3)
    HC, H, T, dil = 2, 16, 7, 3
    C = HC * H
    P = qwen4.Ple()
    P.norm_key = torch.randn(C, generator=g) * 0.1
    P.norm_query = torch.randn(C, generator=g) * 0.1
    key, streams, val = torch.randn(T, C, generator=g), torch.randn(T, C, generator=g), torch.randn(T, H, generator=g)
    gated = qwen4.ple_gate(key, streams, val, P, HC, 1e-6)
    kn, qn = qwen4.grouped_norm(key, P.norm_key, HC, 1e-6), qwen4.grouped_norm(streams, P.norm_query, HC, 1e-6)
    for t in range(T):
        for c in range(HC):
            d = float((kn[t, c * H:(c + 1) * H].double() * qn[t, c * H:(c + 1) * H].double()).sum()) / math.sqrt(H)
            sq = math.copysign(math.sqrt(max(abs(d), 1e-6)), d)
            gate = 1.0 / (1.0 + math.exp(-sq))
            assert torch.allclose(gated[t, c * H:(c + 1) * H].double(), gate * val[t].double(), atol=1e-5)
    # the convolution over one pass equals two chunks with the history carried over
    gn = torch.randn(T, C, generator=g)
    w = torch.randn(C, 4, generator=g) * 0.3
    zero = torch.zeros(3 * dil, C)
    whole = qwen4.ple_conv(gn, zero, w, dil)
    for t in range(T):
        want = sum(w[:, j].double() * (gn[t - (3 - j) * dil].double() if t - (3 - j) * dil >= 0 else 0.0) for j in range(4))
        assert torch.allclose(whole[t].double(), want, atol=1e-5)
    first = qwen4.ple_conv(gn[:4], zero, w, dil)
    hist = torch.cat([zero, gn[:4]])[-3 * dil:]
    second = qwen4.ple_conv(gn[4:], hist, w, dil)
    assert torch.allclose(torch.cat([first, second]), whole, atol=1e-6)


def _llm(**kw):
    base = dict(device="cpu", dtype=torch.float32, max_seqs=8, max_model_len=256, use_graphs=False, seed=0)
    base.update(kw)
    return LLM(named_config("tiny-qwen4"), **base)


def _prompts():
    g = torch.Generator().manual_seed(11)
    ps = [torch.randint(2, 1024, (n,), generator=g).tolist() for n in (37, 5, 18)]
    ps[2][6] = 1          # an end-of-sequence token inside a prompt cuts the n-gram window
    return ps


GREEDY = SamplingParams(temperature=0.0, max_tokens=20, ignore_eos=True)


def test_the_model_runs_and_the_extras_matter():
    llm = _llm()
    m = llm.model
    assert m.hc_final is not None and m.layers[0].ple is not None and m.layers[1].ple is None and llm.engine.kv.ple is not None
    out = [o.token_ids for o in llm.generate(_prompts(), GREEDY)]
    assert all(len(t) == 20 for t in out)
    # without the n-gram rows the model says something else: the embedding is part of the computation
    for L in m.layers:
        if L.ple is not None:
            L.ple.table.zero_()
    assert [o.token_ids for o in llm.generate(_prompts(), GREEDY)] != out
    with pytest.raises(ValueError):
        from blaze_b200.models.qwen3 import Model, TPInfo
        Model(named_config("tiny-qwen4"), tp=TPInfo(0, 2))


def test_chunked_prefill_decode_and_prefix_reuse_agree():
    ps = _prompts()
    want = [o.token_ids for o in _llm(chunk=256).generate(ps, GREEDY)]
    assert [o.token_ids for o in _llm(chunk=8).generate(ps, GREEDY)] == want, "prefill in chunks of 8"
    one = _llm()
    assert [one.generate([p], GREEDY)[0].token_ids for p in ps] == want, "one request at a time"
    # a second request that shares a prefix starts from the cached state rows (token window and conv history included)
    again = one.generate([ps[0] + [5, 6, 7]], GREEDY)[0].token_ids
    fresh = _llm().generate([ps[0] + [5, 6, 7]], GREEDY)[0].token_ids
    assert again == fresh


def test_speculation_keeps_the_ngram_state_exact():
    """Verify rows must not move the token window or the convolution history past rejected drafts.  Drafts are scripted:
    the next two tokens of the known continuation, then two wrong ones, so that every verify step accepts a part."""
    ps = [[3, 4, 5, 6, 7, 8] * 6, _prompts()[0], [9] * 12]
    sp = SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True)
    want = [o.token_ids for o in _llm().generate(ps, sp)]
    spec = _llm(spec_method="ngram", spec_fixed=True)

    def scripted(decoders):
        out = {}
        for a in decoders:
            seq = want[ps.index(list(a.tokens[:a.n_prompt]))]
            n = len(a.generated)
            room = min(4, sp.max_tokens - n - 1)
            d = seq[n:n + 2] + [(seq[-1] + 1) % 1024] * 2
            if room > 0:
                out[id(a)] = d[:room]
        return out
    spec.sched._draft = scripted
    assert [o.token_ids for o in spec.generate(ps, sp)] == want
    st = spec.sched.stats
    assert st.accepted_tokens > 0 and st.accepted_tokens < st.draft_tokens


def test_a_checkpoint_with_the_reference_names_loads(tmp_path):
    """Every tensor of the extras under the names of ``scripts/ref_qwen4.py`` (hyper-connections, sharded n-gram table,
    projections, norms, conv), next to the hybrid decoder's: the loaded model computes what the written one does."""
    import synthetic_checkpoint
    from blaze_b200.models.qwen3 import Model
    src = _llm(dtype=torch.bfloat16, kv_cache_dtype="bf16")
    synthetic_checkpoint.write(src.model, str(tmp_path))
    loaded = LLM(str(tmp_path), device="cpu", dtype=torch.bfloat16, kv_cache_dtype="bf16", max_seqs=8, max_model_len=256, use_graphs=False)
    m = loaded.model
    assert isinstance(m, Model) and m.cfg.hc_count == 2 and m.cfg.ple_layers == [0, 2] and m.layers[2].ple.table.shape == src.model.layers[2].ple.table.shape
    ps = _prompts()[:2]
    assert [o.token_ids for o in loaded.generate(ps, GREEDY)] == [o.token_ids for o in src.generate(ps, GREEDY)]


# ----------------------------------------------------------------------------------- sparse-attention indexer
def test_indexer_scores_and_selection_against_loops():
    """Compressed keys, block scores and the selected tokens as ``kernels/tests/test_qsa_index.cu`` states them."""
    g = torch.Generator().manual_seed(9)
    D, HEADS, RATIO, ROT, eps = 32, 3, 4, 16, 1e-6
    n, top = 45, 5
    inv = torch.tensor([1.0 / (1e7 ** (2.0 * i / ROT)) for i in range(ROT // 2)])
    I = qwen4.Indexer()
    I.q_norm, I.k_norm = torch.randn(D, generator=g) * 0.1, torch.randn(D, generator=g) * 0.1
    kraw = torch.randn(n, D, generator=g)
    qraw = torch.randn(n, HEADS, D, generator=g)

    def norm_rope(v, w, pos):
        v = v.double()
        v = v / math.sqrt(float((v * v).sum() / D) + eps) * (1.0 + w.double())
        o = v.clone()
        for i in range(ROT // 2):
            c, s = math.cos(pos * float(inv[i])), math.sin(pos * float(inv[i]))
            o[i] = v[i] * c - v[i + ROT // 2] * s
            o[i + ROT // 2] = v[i + ROT // 2] * c + v[i] * s
        return o
    comp = qwen4.compressed_keys(kraw, I, RATIO, inv, ROT, eps, 1.0)
    assert comp.shape == (n // RATIO, D)
    for b in range(n // RATIO):
        want = norm_rope(kraw[b * RATIO:(b + 1) * RATIO].double().sum(0) / RATIO, I.k_norm, b * RATIO)
        assert torch.allclose(comp[b].double(), want, atol=1e-4)
    pos = torch.arange(n)
    iq = qwen4._norm_rope(qraw, I.q_norm, pos, inv, ROT, eps, 1.0, torch.float32)
    for r in (0, 17, 44):
        for h in range(HEADS):
            assert torch.allclose(iq[r, h].double(), norm_rope(qraw[r, h], I.q_norm, r), atol=1e-4)
    sc = qwen4.block_scores(iq, comp)
    sc[:, 3] = sc[:, 7]                     # equal scores: the earlier block wins
    sel = qwen4.select_keys(sc, pos, RATIO, top, n)
    for r in range(n):
        nvis = (r + 1) // RATIO
        for b in range(n // RATIO):
            d = sum(max(float((iq[r, h].double() * comp[b].double()).sum()), 0.0) for h in range(HEADS)) / math.sqrt(D)
            if b not in (3, 7):
                assert abs(d - float(sc[r, b])) < 1e-4
        order = sorted(range(nvis), key=lambda b: (-float(sc[r, b]), b))[:top]
        want = set()
        for b in order:
            want.update(range(b * RATIO, (b + 1) * RATIO))
        want.update(range(nvis * RATIO, r + 1))
        assert set(torch.nonzero(sel[r]).flatten().tolist()) == want, r


def _sparse_llm(budget, **kw):
    cfg = named_config("tiny-qwen4")
    cfg.indexer_heads, cfg.indexer_head_dim, cfg.indexer_budget, cfg.indexer_compress_ratio = 2, 32, budget, 4
    base = dict(device="cpu", dtype=torch.float32, max_seqs=8, max_model_len=256, use_graphs=False, seed=0)
    base.update(kw)
    return LLM(cfg, **base)


def test_sparse_attention_through_the_engine():
    g = torch.Generator().manual_seed(21)
    ps = [torch.randint(2, 1024, (n,), generator=g).tolist() for n in (90, 20, 61)]
    # within the budget every key is selected: the tokens of the model whose budget is never reached
    dense = [o.token_ids for o in _sparse_llm(4096).generate(ps, GREEDY)]
    assert [o.token_ids for o in _sparse_llm(128).generate(ps, GREEDY)] == dense
    # beyond it rows see their best blocks only: another answer, and the same one however the prompt is cut into steps
    sparse = [o.token_ids for o in _sparse_llm(32, chunk=256).generate(ps, GREEDY)]
    assert sparse != dense and sparse[1] == dense[1], "the 20-token prompt stays within a budget of 32"
    assert [o.token_ids for o in _sparse_llm(32, chunk=16).generate(ps, GREEDY)] == sparse
    one = _sparse_llm(32)
    assert [one.generate([p], GREEDY)[0].token_ids for p in ps] == sparse
    # a shared prefix brings its index keys with its pages
    again = one.generate([ps[0] + [5, 6, 7]], GREEDY)[0]
    assert again.token_ids == _sparse_llm(32).generate([ps[0] + [5, 6, 7]], GREEDY)[0].token_ids


def test_a_checkpoint_with_an_indexer_loads(tmp_path):
    import synthetic_checkpoint
    src = _sparse_llm(32, dtype=torch.bfloat16, kv_cache_dtype="bf16")
    synthetic_checkpoint.write(src.model, str(tmp_path))
    loaded = LLM(str(tmp_path), device="cpu", dtype=torch.bfloat16, kv_cache_dtype="bf16", max_seqs=8, max_model_len=256, use_graphs=False)
    assert loaded.model.cfg.indexer_budget == 32 and loaded.model.layers[1].attn.index is not None
    p = torch.randint(2, 1024, (70,), generator=torch.Generator().manual_seed(2)).tolist()
    assert loaded.generate([p], GREEDY)[0].token_ids == src.generate([p], GREEDY)[0].token_ids


def test_model_drafters_are_refused_for_stream_models():
    with pytest.raises(ValueError, match="hyper-connection"):
        _llm(spec_method="mtp")
