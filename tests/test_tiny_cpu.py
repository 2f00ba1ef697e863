"""BASELINE config 1: tiny Qwen3-architecture decoder on CPU fp32 through the engine's paged path,
checked against a from-scratch dense recomputation (no KV cache, no paging)."""
import pytest
import torch

from blaze_b200.config import named_config
from blaze_b200.engine import Engine, EngineConfig
from blaze_b200.models.qwen3 import Model
from blaze_b200.ops import ref


def dense_logits(m: Model, toks: torch.Tensor) -> torch.Tensor:
    """Plain causal transformer over the whole sequence, written independently of the engine path."""
    cfg = m.cfg
    x = m.embed[toks].float()
    T = toks.numel()
    pos = torch.arange(T)
    cos, sin = ref.rope_cos_sin(pos, m.inv_freq)
    for L in m.layers:
        h, _ = ref.rmsnorm(x, L.input_norm, cfg.rms_norm_eps)
        qkv = h @ L.attn.qkv.dequant().t()
        q, k, v, _ = ref.attn_prep(qkv, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, L.attn.q_norm, L.attn.k_norm,
                                   cfg.rms_norm_eps, cos, sin)
        g = cfg.num_heads // cfg.num_kv_heads
        k, v = k.repeat_interleave(g, 1), v.repeat_interleave(g, 1)
        s = torch.einsum("qhd,khd->hqk", q, k) * cfg.head_dim ** -0.5
        s = s.masked_fill(~torch.tril(torch.ones(T, T, dtype=torch.bool)), float("-inf"))
        o = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), v).reshape(T, -1)
        x = x + o @ L.attn.o.dequant().t()
        h, _ = ref.rmsnorm(x, L.post_norm, cfg.rms_norm_eps)
        x = x + ref.silu_mul(h @ L.mlp.gate_up.dequant().t()) @ L.mlp.down.dequant().t()
    h, _ = ref.rmsnorm(x, m.final_norm, cfg.rms_norm_eps)
    return h @ m.lm_head.dequant().t()


def test_tiny_qwen3_greedy_matches_dense_reference():
    torch.manual_seed(0)
    cfg = named_config("tiny")
    m = Model.random_init(cfg, seed=0, device="cpu", dtype=torch.float32)
    eng = Engine(m, EngineConfig(max_seqs=8, max_model_len=64, kv_dtype="fp32", use_graphs=False))
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, cfg.vocab_size, (4, 32), generator=g)
    seqs = [eng.open_from() for _ in range(4)]
    # prefill all four prompts in one step
    chunks = eng.plan([(s, prompts[i].tolist(), 1) for i, s in enumerate(seqs)])
    logits = eng.forward(chunks, "logits")
    streams = [prompts[i].tolist() for i in range(4)]
    for i in range(4):
        want = dense_logits(m, prompts[i])[-1]
        assert torch.allclose(logits[i], want, atol=1e-4, rtol=1e-4)
    nxt = ref.argmax_lowest(logits)
    for step in range(16):
        for i in range(4):
            streams[i].append(int(nxt[i]))
        if step == 15:
            break
        chunks = eng.plan([(s, [int(nxt[i])], 1) for i, s in enumerate(seqs)])
        logits = eng.forward(chunks, "logits")
        if step in (0, 7, 14):
            for i in range(4):
                want = dense_logits(m, torch.tensor(streams[i]))[-1]
                assert torch.allclose(logits[i], want, atol=1e-4, rtol=1e-4)
        nxt = ref.argmax_lowest(logits)
    # identical greedy streams against the dense recomputation
    for i in range(4):
        toks = prompts[i].tolist()
        for _ in range(16):
            toks.append(int(torch.argmax(dense_logits(m, torch.tensor(toks))[-1])))
        assert toks == streams[i]
    for s in seqs:
        eng.close(s)
    assert eng.pages.free_count == eng.num_pages - 1


def test_kv_rotation_keeps_the_output():
    """Rotating q and k by the same orthogonal map changes the stored keys but not the scores: generation with
    ``kv_rotate`` gives the tokens of the plain run."""
    from blaze_b200.llm import LLM
    from blaze_b200.ops import ref
    from blaze_b200.sampler import SamplingParams
    x, y = torch.randn(4, 3, 64), torch.randn(4, 3, 64)
    rx, ry = ref.hadamard_rotate(x), ref.hadamard_rotate(y)
    assert torch.allclose((rx * ry).sum(-1), (x * y).sum(-1), atol=1e-4)
    assert not torch.allclose(rx, x, atol=1e-2)
    outs = []
    for rot in (False, True):
        llm = LLM("tiny", device="cpu", dtype=torch.float32, kv_cache_dtype="fp32", kv_rotate=rot, seed=3, max_seqs=4,
                  max_model_len=128)
        outs.append(llm.generate([[5, 6, 7, 8, 9, 10, 11], [40, 41, 42]], SamplingParams(max_tokens=12, temperature=0.0)))
    assert [o.token_ids for o in outs[0]] == [o.token_ids for o in outs[1]]


def test_draft_tree_rows_match_their_chains_and_commit_compacts_the_path():
    """A draft tree verified in one step: every node's logits equal those of its root-to-node chain run on its own, and
    after ``commit_tree`` the sequence continues as if only the accepted path had ever been fed."""
    from blaze_b200.config import named_config
    from blaze_b200.engine import Engine, EngineConfig
    from blaze_b200.models.qwen3 import Model
    from blaze_b200.quant import Format
    cfg = named_config("tiny")
    model = Model.random_init(cfg, Format.DENSE, 0, "cpu", torch.float32)
    eng = Engine(model, EngineConfig(max_seqs=8, max_model_len=128, kv_dtype="fp32", kv_tokens=1024, use_graphs=False))
    prompt = list(range(7, 30))                       # 23 tokens: the tree straddles a page boundary
    toks = [100, 201, 202, 301, 302, 303]             # root, two children, then 301 under 201, 302 and 303 under 202
    parents = [-1, 0, 0, 1, 2, 2]

    def chain_logits(path_tokens):
        s = eng.open_from()
        eng.forward(eng.plan([(s, prompt, 0)]), "none")
        out = eng.forward(eng.plan([(s, path_tokens, len(path_tokens))]), "logits")
        return s, out

    seq = eng.open_from()
    eng.forward(eng.plan([(seq, prompt, 0)]), "none")
    base = seq.length
    tree_logits = eng.forward(eng.plan_tree([(seq, toks, parents)]), "logits")
    assert tree_logits.shape[0] == len(toks) and seq.length == base + len(toks)
    for node in range(len(toks)):
        path, i = [], node
        while i >= 0:
            path.append(i)
            i = parents[i]
        path = path[::-1]
        s, want = chain_logits([toks[i] for i in path])
        assert torch.allclose(tree_logits[node], want[-1], atol=2e-4), node
        eng.close(s)
    # accept root -> 202 -> 303 (rows 2 and 5), then decode one more token
    eng.commit_tree([(seq, base, [2, 5])])
    assert seq.length == base + 3
    nxt = eng.forward(eng.plan([(seq, [400], 1)]), "logits")
    s, _ = chain_logits([100, 202, 303])
    want = eng.forward(eng.plan([(s, [400], 1)]), "logits")
    assert torch.allclose(nxt, want, atol=2e-4)
    with pytest.raises(ValueError):
        eng.plan_tree([(seq, [1, 2], [0, 0])])


def test_nvfp4_kv_rows_and_the_scale_search():
    """KV rows in NVFP4 (``--kv-cache-dtype nvfp4`` / ``nvfp4_4over6``): 4-bit codes plus one E4M3 scale per 16 elements.  The
    searched scale never does worse than the plain one on any block, a block whose values sit on the grid comes back exactly,
    and decoding over such a cache stays close to the fp32 cache."""
    from blaze_b200.quant import nvfp4_kv_dequantize, nvfp4_kv_quantize
    g = torch.Generator().manual_seed(0)
    x = torch.randn(64, 2, 64, generator=g) * torch.rand(64, 2, 1, generator=g) * 3
    plain, best = nvfp4_kv_quantize(x), nvfp4_kv_quantize(x, search=True)
    assert plain.shape == (64, 2, 64 // 2 + 64 // 16) and plain.dtype == torch.uint8
    e_plain = ((nvfp4_kv_dequantize(plain, 64) - x) ** 2).view(64, 2, 4, 16).sum(-1)
    e_best = ((nvfp4_kv_dequantize(best, 64) - x) ** 2).view(64, 2, 4, 16).sum(-1)
    assert (e_best <= e_plain + 1e-6).all() and e_best.sum() < 0.95 * e_plain.sum()
    rel = (nvfp4_kv_dequantize(best, 64) - x).norm() / x.norm()
    assert rel < 0.12
    grid = torch.tensor([0.0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.5, -1, -1.5, -2, -3, -4, -6, 6]).repeat(4) * 0.25
    assert torch.equal(nvfp4_kv_dequantize(nvfp4_kv_quantize(grid[None]), 64)[0], grid)
    # through the engine: prefill, then a decode step over the cache, fp32 pages against the 4-bit ones
    ps = torch.randint(0, 1024, (3, 40), generator=g).tolist()
    cfg = named_config("tiny")
    m = Model.random_init(cfg, seed=0, device="cpu", dtype=torch.float32)
    out = {}
    for kvd in ("fp32", "nvfp4", "nvfp4_4over6"):
        eng = Engine(m, EngineConfig(max_seqs=4, max_model_len=128, kv_dtype=kvd, use_graphs=False))
        seqs = [eng.open_from() for _ in ps]
        eng.forward(eng.plan([(s, p, 1) for s, p in zip(seqs, ps)]), "logits")
        out[kvd] = eng.forward(eng.plan([(s, [7], 1) for s in seqs]), "logits")
        if kvd != "fp32":
            assert eng.kv.k[0].dtype == torch.uint8 and eng.kv.k[0].shape[-1] == 64 // 2 + 64 // 16
    cos = {k: torch.nn.functional.cosine_similarity(out[k], out["fp32"], dim=1).min().item() for k in ("nvfp4", "nvfp4_4over6")}
    assert cos["nvfp4"] > 0.97 and cos["nvfp4_4over6"] > 0.97, cos


@pytest.mark.parametrize("fmt,want,lo", [("nvfp4", "NVFP4", 0.90), ("nvfp4_modelopt", "NVFP4", 0.90), ("mxfp8", "MXFP8", 0.99),
                                         ("fp8_block", "FP8_BLOCK", 0.99), ("fp8_channel", "FP8_CHANNEL", 0.99),
                                         ("fp8_tensor", "FP8_CHANNEL", 0.98)])
def test_checkpoints_in_every_weight_format_load(tmp_path, fmt, want, lo):
    """A local checkpoint whose projections are stored in each supported format (tensor names as the quantisation tools
    write them) loads into that format: the stored codes and scales arrive unchanged (the loaded weight dequantises to what
    was written), and the model's logits follow the bf16 model's within the format's error."""
    import synthetic_checkpoint
    from blaze_b200.quant import Format
    cfg = named_config("tiny")
    dense = Model.random_init(cfg, seed=3, device="cpu", dtype=torch.float32)
    synthetic_checkpoint.write(dense, str(tmp_path), prefix="model.", fmt=fmt)
    m = Model.load(str(tmp_path), device="cpu", dtype=torch.float32)
    L0 = m.layers[0]
    assert L0.attn.qkv.fmt == getattr(Format, want) and L0.mlp.down.fmt == getattr(Format, want) and m.lm_head.fmt == Format.DENSE
    # exactness of the round trip: dequantising the loaded module gives the dequantisation of what the writer stored
    w = dense.layers[0].mlp.down.dequant()
    stored = synthetic_checkpoint.quantised("x", w, fmt)
    from blaze_b200 import quant
    if fmt.startswith("nvfp4"):
        g = stored.get("x.weight_scale_2")
        g = g if g is not None else 1.0 / stored["x.weight_global_scale"]
        ref_w = quant.nvfp4_dequantize(stored.get("x.weight_packed", stored.get("x.weight")), stored["x.weight_scale"], g[0])
    elif fmt == "mxfp8":
        ref_w = quant.mxfp8_dequantize(stored["x.weight"], stored["x.weight_scale"])
    elif fmt == "fp8_block":
        ref_w = quant.fp8_block_dequantize(stored["x.weight"], stored["x.weight_scale_inv"])
    else:
        ref_w = stored["x.weight"].float() * stored["x.weight_scale"].float().reshape(-1, 1)
    assert torch.allclose(L0.mlp.down.dequant().float(), ref_w.float(), atol=1e-6)
    assert (ref_w - w).norm() / w.norm() < (0.15 if fmt.startswith("nvfp4") else 0.05)
    toks = torch.randint(0, cfg.vocab_size, (24,), generator=torch.Generator().manual_seed(1))
    out = {}
    for name, model in (("dense", dense), ("loaded", m)):
        eng = Engine(model, EngineConfig(max_seqs=2, max_model_len=64, kv_dtype="fp32", use_graphs=False))
        s = eng.open_from()
        out[name] = eng.forward(eng.plan([(s, toks.tolist(), len(toks))]), "logits")
    cos = torch.nn.functional.cosine_similarity(out["loaded"], out["dense"], dim=1)
    assert cos.min().item() > lo, (fmt, cos.min().item())


def test_a_hybrid_moe_checkpoint_with_mxfp8_projections_loads(tmp_path):
    """The hybrid family (Gated DeltaNet + gated attention + MoE with a shared expert) from a checkpoint whose attention,
    expert and shared-expert projections are MXFP8 while the GDN projections, router and gates are bf16."""
    import synthetic_checkpoint
    from blaze_b200.quant import Format
    cfg = named_config("tiny-hybrid")
    dense = Model.random_init(cfg, seed=3, device="cpu", dtype=torch.float32)
    synthetic_checkpoint.write(dense, str(tmp_path), fmt="mxfp8")
    m = Model.load(str(tmp_path), device="cpu", dtype=torch.float32)
    assert m.cfg.layer_types == cfg.layer_types and m.cfg.num_experts == 8
    assert m.layers[1].attn.qkv.fmt == Format.MXFP8 and m.layers[0].mlp.experts.gate_up[3].fmt == Format.MXFP8
    assert m.layers[0].mlp.shared.down.fmt == Format.MXFP8 and m.layers[0].gdn.in_proj.fmt == Format.DENSE
    assert m.layers[0].mlp.router.fmt == Format.DENSE
    toks = torch.randint(0, cfg.vocab_size, (24,), generator=torch.Generator().manual_seed(1)).tolist()
    out = {}
    for name, model in (("dense", dense), ("loaded", m)):
        eng = Engine(model, EngineConfig(max_seqs=2, max_model_len=64, kv_dtype="fp32", use_graphs=False))
        s = eng.open_from()
        out[name] = eng.forward(eng.plan([(s, toks, len(toks))]), "logits")
    cos = torch.nn.functional.cosine_similarity(out["loaded"], out["dense"], dim=1)
    # a row whose routing flips an expert under the 8-bit weights moves further than the others
    assert cos.mean().item() > 0.985 and cos.min().item() > 0.9, (cos.mean().item(), cos.min().item())
