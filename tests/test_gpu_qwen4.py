"""The Qwen4-Exp extras on the GPU: hyper-connection streams and the n-gram embedding run as torch ops on the device around
the attention, Gated DeltaNet and MLP kernels.  Same weights through the kernels and through the PyTorch oracle ops:
prefill logits of every prompt row (three sequences, so the per-sequence state rows are exercised), then decode steps over
the state the prefill left."""
import pytest
import torch

from blaze_b200.config import ModelConfig, RopeConfig

pytestmark = pytest.mark.gpu


def _cfg():
    cfg = ModelConfig(architecture="Qwen4ExpForCausalLM", model_type="qwen4_exp", vocab_size=2048, hidden_size=512, num_layers=4,
                      num_heads=4, num_kv_heads=2, head_dim=128, intermediate_size=1024, linear_num_key_heads=2,
                      linear_num_value_heads=4, linear_key_head_dim=128, linear_value_head_dim=128, linear_conv_kernel_dim=4,
                      attn_output_gate=True, zero_centered_norm=True, rope=RopeConfig(theta=1e6, partial_rotary_factor=0.25))
    cfg.layer_types = ["linear_attention", "full_attention"] * 2
    cfg.hc_count, cfg.hc_lowrank = 2, 16
    cfg.ple_layers, cfg.ngram_size, cfg.heads_per_ngram, cfg.ple_embed_dim, cfg.ple_conv_kernel = [0, 2], 3, 2, 32, 4
    cfg.eos_token_ids = [1]
    return cfg


@pytest.mark.parametrize("gate,indexer", [("silu", False), ("sigmoid", False), ("silu", True)])
def test_streams_and_ngram_embedding_match_the_oracle_ops(gate, indexer):
    from blaze_b200.engine import Engine, EngineConfig
    from blaze_b200.models.qwen3 import Model
    from blaze_b200.ops.ref_ops import RefOps
    cfg = _cfg()
    cfg.gdn_output_gate = gate          # the Gated DeltaNet output gate a checkpoint names (output_gate_type)
    if indexer:
        # a sparse-attention indexer whose budget the contexts stay within: its keys are written, attention is dense
        cfg.indexer_heads, cfg.indexer_head_dim, cfg.indexer_budget, cfg.indexer_compress_ratio = 2, 64, 2048, 4
    mk = Model.random_init(cfg, seed=5, device="cuda")
    mr = Model.random_init(cfg, seed=5, device="cuda", ops=RefOps())
    assert mk.ops.is_cuda and not mr.ops.is_cuda and mk.layers[0].ple is not None and mk.hc_final is not None
    ek = Engine(mk, EngineConfig(max_seqs=4, max_model_len=256, kv_dtype="fp8", kv_tokens=2048, use_graphs=True))
    er = Engine(mr, EngineConfig(max_seqs=4, max_model_len=256, kv_dtype="fp8", kv_tokens=2048, use_graphs=False))
    assert not ek.ecfg.use_graphs, "nothing of a hyper-connection model is captured"
    prompts = torch.randint(2, 2048, (3, 70), generator=torch.Generator().manual_seed(11)).tolist()
    prompts[1][30] = 1          # an end-of-sequence token inside a prompt cuts the n-gram window
    sk = [ek.open_from() for _ in prompts]
    sr = [er.open_from() for _ in prompts]
    lk = ek.forward(ek.plan([(s, p, len(p)) for s, p in zip(sk, prompts)]), "logits").float()
    lr = er.forward(er.plan([(s, p, len(p)) for s, p in zip(sr, prompts)]), "logits").float()
    cos = torch.nn.functional.cosine_similarity(lk, lr, dim=1)
    print(f"[qwen4] prefill rows {lk.shape[0]}: cosine min {cos.min().item():.5f} mean {cos.mean().item():.5f}")
    assert cos.min().item() >= 0.995 and cos.mean().item() >= 0.999      # measured on B200: 0.99998 / 0.99999
    toks = lr[[70 * (i + 1) - 1 for i in range(3)]].argmax(1).tolist()
    for step in range(4):
        lk = ek.forward(ek.plan([(s, [t], 1) for s, t in zip(sk, toks)]), "logits").float()
        lr = er.forward(er.plan([(s, [t], 1) for s, t in zip(sr, toks)]), "logits").float()
        cos = torch.nn.functional.cosine_similarity(lk, lr, dim=1)
        print(f"[qwen4] decode step {step}: cosine min {cos.min().item():.5f}")
        assert cos.min().item() >= 0.995
        toks = lr.argmax(1).tolist()
    # the token window and the convolution history moved alike on both sides
    for a, b in ((ek.kv.ple.hist, er.kv.ple.hist),):
        assert torch.equal(a[[s.row for s in sk]], b[[s.row for s in sr]])
    if indexer:
        # both sides wrote the same index keys (the same torch ops on the same projection kernel's output)
        pk, pr = ek.kv.idx_k[1], er.kv.idx_k[1]
        rows_k = pk[ek.kv.block_table[sk[0].row, :4].long()].float()
        rows_r = pr[er.kv.block_table[sr[0].row, :4].long()].float()
        assert rows_k.abs().sum() > 0 and torch.nn.functional.cosine_similarity(rows_k.flatten(), rows_r.flatten(), dim=0) > 0.999
    torch.cuda.synchronize()
    assert mk.ops.take_status() == 0
