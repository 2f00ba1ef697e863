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
