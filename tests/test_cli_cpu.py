"""The command line on the CPU: offline generation, the self-speculation check of the verify / commit path, the drafter
check, and the flags that are refused loudly instead of being ignored."""
import json

import pytest

from blaze_b200 import cli

IDS = "5,6,7,8,9,10,11,12,13"


def _run(capsys, argv):
    rc = cli.main(argv)
    return rc, capsys.readouterr().out.strip().splitlines()


def test_generate_prints_tokens(capsys):
    rc, out = _run(capsys, ["generate", "--model", "tiny", "--device", "cpu", "--prompt-ids", IDS, "--max-tokens", "6"])
    line = json.loads(out[-1])
    assert rc == 0 and len(line["token_ids"]) == 6 and line["finish_reason"] == "length"


def test_self_spec_verify_rounds_reproduce_greedy_decoding(capsys):
    """Drafts are the greedy continuation with a wrong token at pseudo-random places: every round accepts up to the wrong
    token, commits, truncates the rest; all tokens must match and rounds must be fewer than tokens."""
    rc, out = _run(capsys, ["self-spec", "--model", "tiny", "--device", "cpu", "--prompt-ids", IDS, "--max-tokens", "48", "--draft", "5"])
    assert rc == 0
    assert out[-1].startswith("48/48 tokens match the reference")
    rounds = int(out[-1].split(";")[1].split()[0])
    assert rounds < 30


def test_self_spec_on_the_recurrent_hybrid(capsys):
    """Same check on a model with Gated DeltaNet layers: rejected rows must not have advanced the recurrent state."""
    rc, out = _run(capsys, ["self-spec", "--model", "tiny-hybrid", "--device", "cpu", "--prompt-ids", IDS, "--max-tokens", "24", "--draft", "4"])
    assert rc == 0 and out[-1].startswith("24/24 tokens match the reference")


def test_eagle_test_reports_rounds_and_parting_point(capsys):
    rc, out = _run(capsys, ["eagle-test", "--model", "tiny", "--device", "cpu", "--spec-method", "mtp", "--prompt-ids", IDS,
                            "--max-tokens", "20"])
    line = json.loads(out[-1])
    assert rc == 0 and line["tokens"] == 20 and line["match_until"] == 20 and line["drafter"] == "mtp" and line["rounds"] > 0


def test_eagle_test_needs_a_drafter(capsys):
    assert cli.main(["eagle-test", "--model", "tiny", "--device", "cpu", "--prompt-ids", IDS]) == 2


def test_reference_engine_flags_carry_over_or_are_refused_with_a_reason(capsys):
    """Launch scripts written for the reference keep working where the flag's neutral value is what this engine does anyway;
    a value it cannot honour ends the command with the reason instead of being ignored."""
    base = ["generate", "--model", "tiny", "--device", "cpu", "--prompt-ids", IDS, "--max-tokens", "3"]
    rc, out = _run(capsys, base + ["--gemm", "auto", "--attn-f16-acc", "off", "--prefill-attention", "auto", "--verify-attention", "auto",
                                   "--prefill-a16", "none", "--l2-prefetch-mib", "0", "--draft-head-vram", "auto",
                                   "--ple-threads", "8", "--ple-cache-gib", "2"])
    assert rc == 0 and len(json.loads(out[-1])["token_ids"]) == 3
    for extra, word in ((["--gemm", "bf16"], "weight format"), (["--attn-f16-acc", "on"], "fp32"),
                        (["--l2-prefetch-mib", "4"], "prefetch"), (["--pp-remote", "1=host:9000"], "torch.distributed"),
                        (["--prefill-a16", "kv"], "16-bit"),
                        (["--mtp-model", "/nowhere", "--spec-method", "eagle"], "--spec-method mtp")):
        with pytest.raises(SystemExit) as e:
            cli.main(base + extra)
        assert word in str(e.value), (extra, str(e.value))
