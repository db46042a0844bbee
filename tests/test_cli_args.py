"""The command line's arguments: the reference's names, defaults and error wording (src/cli/main.cpp:26-37,
:196-247), without a GPU."""
import pytest

from citlali_b200.cli import REFERENCE_ONLY, parse_args


def test_defaults_are_the_references():
    a = parse_args(["citlali_cli", "--model", "m", "--prompt-ids", "1,2,3"])
    assert (a.model_path, a.prompts, a.max_new_tokens, a.max_context) == ("m", [[1, 2, 3]], 256, 2048)
    assert a.temperature == 0.0 and a.stop_ids is None and a.dtype == "bfloat16" and not a.info and not a.help


def test_options_and_their_aliases():
    a = parse_args(["citlali_cli", "--model", "m", "--prompt-ids", "1,2", "--prompt-ids", "7", "--ctx", "512",
                    "--max-new-tokens", "9", "--temperature", "0.8", "--seed", "5", "--stop-ids", "3,4",
                    "--dtype", "float32", "--slots", "2", "--json"])
    assert a.prompts == [[1, 2], [7]] and a.max_context == 512 and a.max_new_tokens == 9
    assert a.temperature == 0.8 and a.seed == 5 and a.stop_ids == [3, 4] and a.dtype == "float32" and a.slots == 2 and a.json
    assert parse_args(["citlali_cli", "--context", "64"]).max_context == 64
    assert parse_args(["citlali_cli", "-h"]).help and parse_args(["citlali_cli", "--help"]).help
    assert parse_args(["citlali_cli", "--model", "m", "--info"]).info


def test_errors_are_worded_as_in_the_reference():
    with pytest.raises(RuntimeError, match="^unknown argument: --frobnicate$"):
        parse_args(["citlali_cli", "--frobnicate"])
    with pytest.raises(RuntimeError, match="^missing value for --model$"):
        parse_args(["citlali_cli", "--model"])


@pytest.mark.parametrize("flag", sorted(REFERENCE_ONLY))
def test_the_references_other_options_say_why_they_are_not_here(flag):
    with pytest.raises(RuntimeError, match=flag + ": .*(no tokenizer|not part of this library)"):
        parse_args(["citlali_cli", "--model", "m", flag, "x"])
