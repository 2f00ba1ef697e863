"""Draft-tree verification on the GPU: the tree mask of the verify attention kernel against the oracle, the KV row move
kernel against the host path over the same page layout, and an engine-level check that every tree row's logits are those
of its own root-to-node chain."""
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


@pytest.fixture(scope="module")
def ops():
    from blaze_b200.ops import get_ops
    o = get_ops(DEV)
    assert o.is_cuda, "kernel library not loaded"
    return o


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-6)).item()


@pytest.mark.parametrize("Hq,Hkv,ctxs,qlens,parents", [
    (8, 2, [300, 77], [6, 4], [[-1, 0, 0, 1, 2, 2], [-1, 0, 1, 1]]),               # 24 and 16 rows per KV head
    (32, 8, [1024, 130, 40], [8, 2, 1], [[-1, 0, 1, 2, 0, 4, 0, 6], [-1, 0], None]),  # with a chain pair and a plain decode row
    (4, 4, [200], [20], [[-1] + [max(i - 3, 0) for i in range(1, 20)]]),           # group 1, wide tree
])
def test_tree_mask_attention(ops, Hq, Hkv, ctxs, qlens, parents):
    from test_gpu_kernels import _attention_case
    o, want = _attention_case(ops, Hq, Hkv, ctxs, qlens, parents=parents)
    assert torch.isfinite(o.float()).all()
    assert _rel(o, want) < 0.06
    # the mask matters: the same rows without it give something else
    plain, _ = _attention_case(ops, Hq, Hkv, ctxs, qlens)
    assert _rel(plain, want) > 0.01


def test_kv_row_moves_match_the_host_path(ops):
    from blaze_b200.config import ModelConfig, RopeConfig
    from blaze_b200.kv import KVCache
    cfg = ModelConfig(hidden_size=512, num_heads=8, num_kv_heads=2, head_dim=128, num_layers=2, rope=RopeConfig(theta=1e6))
    cfg.layer_types = ["full_attention"] * 2
    g = torch.Generator(device=DEV).manual_seed(3)
    kv = KVCache(cfg, 12, 4, 8, "fp8", DEV, "umma")
    for i in kv.attn_layers:
        kv.kv[i].copy_(torch.randint(0, 255, kv.kv[i].shape, dtype=torch.uint8, device=DEV, generator=g))
    before = {i: kv.kv[i].clone() for i in kv.attn_layers}
    # sequence 0: rows 2 -> 1 then 5 -> 2 of a tree that starts at slot 30 (crosses pages 1 and 2); sequence 1: 100 -> 97
    moves = [[(32, 31), (35, 32)], [(100, 97)]]
    kv.move_rows(moves, ops)
    torch.cuda.synchronize()
    assert ops.take_status() == 0
    host = KVCache(cfg, 12, 4, 8, "fp8", DEV, "umma")
    for i in host.attn_layers:
        host.kv[i].copy_(before[i])
    host.move_rows(moves, None)
    for i in kv.attn_layers:
        assert torch.equal(kv.kv[i], host.kv[i])
        assert not torch.equal(kv.kv[i], before[i])
        kl, _ = kv.logical_kv(i)
        kb = before[i]
        # row 35 of the old pool (page 2, offset 3) now also sits at slot 32 (page 2, offset 0)
        old_k = KVCache.unpack_umma_page(kb[2, 0], 128)[0].view(torch.uint8)
        assert torch.equal(kl[2, 0, 0].view(torch.uint8), old_k[3])


def test_engine_tree_rows_match_their_chains():
    from blaze_b200.config import ModelConfig, RopeConfig
    from blaze_b200.engine import Engine, EngineConfig
    from blaze_b200.models.qwen3 import Model
    from blaze_b200.quant import Format
    cfg = ModelConfig(vocab_size=2048, hidden_size=512, num_layers=2, num_heads=8, num_kv_heads=2, head_dim=128,
                      intermediate_size=1024, rope=RopeConfig(theta=1e6))
    cfg.layer_types = ["full_attention"] * 2
    model = Model.random_init(cfg, fmt=Format.NVFP4, seed=0, device="cuda:0")
    eng = Engine(model, EngineConfig(max_seqs=16, max_model_len=256, kv_dtype="fp8", kv_tokens=4096, use_graphs=False))
    prompt = torch.randint(0, 2048, (45,), generator=torch.Generator().manual_seed(5)).tolist()
    toks = [100, 201, 202, 301, 302, 303]
    parents = [-1, 0, 0, 1, 2, 2]

    def chain(path_tokens):
        s = eng.open_from()
        eng.forward(eng.plan([(s, prompt, 0)]), "none")
        return s, eng.forward(eng.plan([(s, path_tokens, len(path_tokens))]), "logits")

    seq = eng.open_from()
    eng.forward(eng.plan([(seq, prompt, 0)]), "none")
    base = seq.length
    tree_logits = eng.forward(eng.plan_tree([(seq, toks, parents)]), "logits")
    for node in range(len(toks)):
        path, i = [], node
        while i >= 0:
            path.append(i)
            i = parents[i]
        s, want = chain([toks[i] for i in path[::-1]])
        assert _rel(tree_logits[node], want[-1]) < 0.05, node
        eng.close(s)
    eng.commit_tree([(seq, base, [2, 5])])
    nxt = eng.forward(eng.plan([(seq, [400], 1)]), "logits")
    s, _ = chain([100, 202, 303])
    want = eng.forward(eng.plan([(s, [400], 1)]), "logits")
    assert _rel(nxt, want) < 0.05
    torch.cuda.synchronize()
    assert model.ops.take_status() == 0
