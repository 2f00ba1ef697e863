"""Routing heat of mixture-of-experts models: collection during generation, the profile file, per-stage merges, and the
placement statistics (``blaze_b200/expert_heat.py``; reference ``kernels/src/runtime/swap.cpp`` ``HeatProfile``)."""
import numpy as np
import torch

from blaze_b200.config import named_config
from blaze_b200.expert_heat import ExpertHeat
from blaze_b200.llm import LLM
from blaze_b200.sampler import SamplingParams


def _tiny_moe():
    cfg = named_config("tiny-hybrid")
    return cfg


def test_collection_counts_every_routed_row(tmp_path):
    cfg = _tiny_moe()
    path = str(tmp_path / "heat.bin")
    llm = LLM(cfg, device="cpu", dtype=torch.float32, max_seqs=4, max_model_len=128, chunk=64, expert_heat=path, use_graphs=False)
    assert llm.heat is not None and llm.model.heat is llm.heat
    prompts = [[1, 2, 3, 4, 5, 6, 7], [9, 8, 7]]
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))
    llm.save_expert_heat()
    # every token that went through the model was routed top_k times in every mixture-of-experts layer
    rows = sum(len(p) for p in prompts) + sum(len(o.token_ids) - 1 for o in outs)
    moe_layers = [i for i, L in enumerate(llm.model.layers) if hasattr(L.mlp, "experts")]
    assert moe_layers
    per_layer = llm.heat.longterm.sum(axis=1)
    for l in moe_layers:
        assert per_layer[l] == rows * cfg.num_experts_per_tok
    assert per_layer.sum() == len(moe_layers) * rows * cfg.num_experts_per_tok
    # the file holds what was collected; a second run starts from it and adds to it
    again = ExpertHeat.load(path, cfg.num_layers, cfg.num_experts)
    assert again is not None and np.array_equal(again.longterm, llm.heat.longterm)
    llm2 = LLM(cfg, device="cpu", dtype=torch.float32, max_seqs=4, max_model_len=128, chunk=64, expert_heat=path, use_graphs=False)
    llm2.generate([[1, 2, 3]], SamplingParams(temperature=0.0, max_tokens=2, ignore_eos=True))
    llm2.save_expert_heat()
    assert ExpertHeat.load(path, cfg.num_layers, cfg.num_experts).longterm.sum() == per_layer.sum() + len(moe_layers) * 4 * cfg.num_experts_per_tok


def test_profile_file_roundtrip_shapes_and_stage_merge(tmp_path):
    path = str(tmp_path / "p.bin")
    h = ExpertHeat(4, 8)
    h.observe(1, torch.tensor([[0, 3], [3, 5]]))
    h.observe(3, torch.tensor([[7, 7]]))
    h.save(path)
    got = ExpertHeat.load(path, 4, 8)
    assert got.longterm[1].tolist() == [1, 0, 0, 2, 0, 1, 0, 0] and got.longterm[3, 7] == 2
    assert ExpertHeat.load(path, 4, 16) is None                       # another expert count: not this model's profile
    more = ExpertHeat.load(path, 5, 8)                                # a layer added: the known layers are kept, the new one is cold
    assert more.longterm[:4].sum() == 6 and more.longterm[4].sum() == 0
    assert ExpertHeat.load(str(tmp_path / "absent.bin"), 4, 8) is None
    (tmp_path / "junk.bin").write_bytes(b"not a profile")
    assert ExpertHeat.load(str(tmp_path / "junk.bin"), 4, 8) is None
    # a pipeline stage that owns layers 2..3 replaces only those
    stage = ExpertHeat.open(path, 4, 8)
    stage.layer_range = (2, 4)
    stage.longterm[:] = 0
    stage.recent[:] = 0
    stage.observe(2, torch.tensor([[1, 1, 1]]))
    stage.observe(1, torch.tensor([[6]]))                             # not its layer: must not reach the file
    stage.save()
    merged = ExpertHeat.load(path, 4, 8)
    assert merged.longterm[1].tolist() == [1, 0, 0, 2, 0, 1, 0, 0]
    assert merged.longterm[2, 1] == 3 and merged.longterm[3].sum() == 0


def test_recent_score_forgets_and_longterm_does_not():
    h = ExpertHeat(1, 4, half_life=8.0)
    h.observe(0, torch.tensor([[0] * 8]))
    h.fold()
    h.observe(0, torch.tensor([[1] * 8]))
    h.fold()
    assert h.longterm[0].tolist() == [8, 8, 0, 0]
    assert h.recent[0, 1] == 8 and abs(h.recent[0, 0] - 4.0) < 1e-9   # eight rows later the first burst counts half


def test_placement_evens_out_what_contiguous_ranks_concentrate():
    h = ExpertHeat(2, 16)
    load = np.ones(16)
    load[:4] = 20.0                       # the four hot experts sit on rank 0 of four under the contiguous placement
    h.longterm[0] = h.recent[0] = load
    h.fold()
    cont = h.imbalance(4)
    where = h.placement(4)
    bal = h.imbalance(4, where)
    assert cont[0] > 3.4 and bal[0] < 1.05
    assert cont[1] == 1.0 and bal[1] == 1.0                            # no observations: reported as even
    assert all(np.bincount(where[0], minlength=4) == 4)                # every rank holds the same number of experts
    rep = h.report(4)
    assert rep["observed_layers"] == 1 and rep["imbalance_contiguous"]["worst"] > rep["imbalance_balanced"]["worst"]
    assert rep["hottest_in_first_layer"][0][0] in (0, 1, 2, 3)
    try:
        h.placement(3)
        raise AssertionError("16 experts over 3 ranks must be refused")
    except ValueError:
        pass


def test_inspect_reports_a_profile(tmp_path, capsys):
    from blaze_b200.cli import main
    cfg = _tiny_moe()
    path = str(tmp_path / "heat.bin")
    h = ExpertHeat(cfg.num_layers, cfg.num_experts)
    h.observe(0, torch.arange(cfg.num_experts).view(1, -1))
    h.observe(0, torch.zeros(1, 6, dtype=torch.long))
    h.save(path)
    assert main(["inspect", "--model", "tiny-hybrid", "--expert-heat", path, "--ranks", "2"]) == 0
    text = capsys.readouterr().out
    assert '"observed_layers": 1' in text and "busiest-rank load over mean" in text
    assert main(["inspect", "--model", "tiny", "--expert-heat", path]) == 1
