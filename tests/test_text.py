"""Text in and out: the byte-level BPE read from a hand-made tokenizer.json (both ways, added
tokens, split behaviours, `ignore_merges`, streaming without cutting characters), the stop set
and sampling defaults read from a checkpoint's side files, the request meter, the pool sized
from free memory, and the command line's choice of sampling options."""

from __future__ import annotations

import json

import pytest

from mlx_omnia_b200.engine.engine import pool_tokens
from mlx_omnia_b200.engine.meter import Meter
from mlx_omnia_b200.text import ByteLevelBPE, Detokenizer, SamplingDefaults, generation_defaults, read_tokenizer
from mlx_omnia_b200.text.bpe import BYTE_TO_CHAR, CHAR_TO_BYTE


def tokenizer_json(**model_extra) -> dict:
    """256 byte symbols, a few merges ("hello", " world", "ab"), two added tokens."""
    vocab = {char: value for value, char in enumerate(BYTE_TO_CHAR)}
    merges = []
    for left, right in [("h", "e"), ("l", "l"), ("he", "ll"), ("hell", "o"), ("Ġ", "w"), ("Ġw", "o"), ("r", "l"),
                        ("Ġwo", "rl"), ("Ġworl", "d"), ("a", "b")]:
        vocab[left + right] = len(vocab)
        merges.append(f"{left} {right}")
    added = [{"id": len(vocab), "content": "<|end|>", "special": True},
             {"id": len(vocab) + 1, "content": "<|end|>!", "special": True}]
    return {"model": {"type": "BPE", "vocab": vocab, "merges": merges, **model_extra}, "added_tokens": added,
            "pre_tokenizer": {"type": "Sequence", "pretokenizers": [
                {"type": "Split", "pattern": {"Regex": r" ?\p{L}+| ?\p{N}+|\s+|[^\s\p{L}\p{N}]+"}, "behavior": "Isolated"},
                {"type": "ByteLevel", "add_prefix_space": False, "use_regex": False}]}}


def test_byte_alphabet_is_a_bijection_of_printable_characters():
    assert len(set(BYTE_TO_CHAR)) == 256 and all(CHAR_TO_BYTE[c] == b for b, c in enumerate(BYTE_TO_CHAR))
    assert BYTE_TO_CHAR[ord("A")] == "A" and BYTE_TO_CHAR[ord(" ")] == "Ġ" and BYTE_TO_CHAR[0] == "Ā"


def test_bpe_round_trip_merges_and_added_tokens(tmp_path):
    (tmp_path / "tokenizer.json").write_text(json.dumps(tokenizer_json()), encoding="utf-8")
    tok = read_tokenizer(tmp_path)
    vocab = tok.vocab
    assert tok.encode("hello world") == [vocab["hello"], vocab["Ġworld"]]
    # merges apply by rank, not left to right: "hell" + "o" only after "he" + "ll"
    assert tok.encode("hel") == [vocab["he"], ord("l")]
    # an added token is cut out first, the longer one where one starts another; text around it is split on its own
    ids = tok.encode("ab<|end|>!ab<|end|>")
    assert ids == [vocab["ab"], tok.added["<|end|>!"], vocab["ab"], tok.added["<|end|>"]]
    text = "hello world<|end|> héllo ☃ 12 \n\tx"
    assert tok.decode(tok.encode(text)) == text
    assert tok.vocab_size == len(vocab) + 2
    with pytest.raises(ValueError, match="not in the tokenizer"):
        tok.decode([10 ** 6])


def test_streaming_decode_never_cuts_a_character(tmp_path):
    tok = ByteLevelBPE.from_file(_written(tmp_path, tokenizer_json()))
    ids = tok.encode("é☃𝄞!")
    pieces = Detokenizer(tok)
    out = [pieces.feed(i) for i in ids]
    assert "".join(out) + pieces.flush() == "é☃𝄞!" and all("�" not in piece for piece in out)
    assert out[0] == "" and out[1] == "é"  # the first byte of a two-byte character waits for the second


def _written(folder, declared):
    path = folder / "tokenizer.json"
    path.write_text(json.dumps(declared), encoding="utf-8")
    return path


def test_split_behaviours_and_ignore_merges(tmp_path):
    declared = tokenizer_json(ignore_merges=True)
    declared["model"]["vocab"]["xyz"] = 999  # a whole pre-token in the vocabulary, unreachable by merges
    declared["pre_tokenizer"] = {"type": "Split", "pattern": {"Regex": r"\n"}, "behavior": "MergedWithNext"}
    tok = ByteLevelBPE.from_file(_written(tmp_path, declared))
    assert tok.stages[0].cut("a\nb\n\nc") == ["a", "\nb", "\n", "\nc"]
    assert tok.encode("xyz") == [999]
    declared["model"]["ignore_merges"] = False
    assert ByteLevelBPE.from_file(_written(tmp_path, declared)).encode("xyz") == [ord("x"), ord("y"), ord("z")]
    declared["pre_tokenizer"] = {"type": "Split", "pattern": {"Regex": r","}, "behavior": "MergedWithPrevious"}
    assert ByteLevelBPE.from_file(_written(tmp_path, declared)).stages[0].cut("a,b,,c") == ["a,", "b,", ",", "c"]
    declared["pre_tokenizer"] = {"type": "Split", "pattern": {"Regex": r","}, "behavior": "Removed"}
    assert ByteLevelBPE.from_file(_written(tmp_path, declared)).stages[0].cut("a,b,,c") == ["a", "b", "c"]
    declared["pre_tokenizer"] = {"type": "Whitespace"}
    with pytest.raises(ValueError, match="not read"):
        ByteLevelBPE.from_file(_written(tmp_path, declared))
    assert read_tokenizer(tmp_path / "nowhere") is None


def test_stop_set_and_sampling_defaults_come_from_the_side_files(tmp_path):
    assert generation_defaults(tmp_path, (7,)).stop == (7,) and generation_defaults(tmp_path).sampling == SamplingDefaults()
    (tmp_path / "generation_config.json").write_text(json.dumps(
        {"eos_token_id": [9, 7, 11], "temperature": 0.6, "top_p": 0.95, "top_k": 20, "min_p": 0, "do_sample": True}))
    (tmp_path / "tokenizer_config.json").write_text(json.dumps({"eos_token": {"content": "<|end|>"}}))
    declared = tokenizer_json()
    _written(tmp_path, declared)
    end = declared["added_tokens"][0]["id"]
    found = generation_defaults(tmp_path, (7,))
    assert found.stop == (7, 9, 11, end)  # in load order, without repeats; only ever widened
    assert found.sampling == SamplingDefaults(temperature=0.6, top_p=0.95, top_k=20)  # min_p 0 means "not declared"
    (tmp_path / "generation_config.json").write_text(json.dumps({"do_sample": False, "temperature": 0.6, "eos_token_id": 3}))
    greedy = generation_defaults(tmp_path)
    assert greedy.sampling == SamplingDefaults(temperature=0.0) and greedy.stop == (3, end)


def test_command_line_options_prefer_flags_then_the_checkpoint_then_the_reference_s_defaults():
    from mlx_omnia_b200.cli.main import _options, _parser

    args = _parser().parse_args(["run", "-m", "x", "hi"])
    plain = _options(args, SamplingDefaults())
    assert plain.sampler.temperature == 1.0 and plain.sampler.top_k == 0 and plain.max_tokens == 512
    declared = SamplingDefaults(temperature=0.6, top_p=0.95, top_k=20, repetition_penalty=1.1)
    taken = _options(args, declared)
    assert (taken.sampler.temperature, taken.sampler.top_p, taken.sampler.top_k) == (0.6, 0.95, 20)
    assert taken.penalty.value == 1.1
    assert _options(args, SamplingDefaults(temperature=0.0)).sampler.greedy
    flagged = _options(_parser().parse_args(["run", "-m", "x", "--temperature", "0.9", "--top-k", "5", "hi"]), declared)
    assert (flagged.sampler.temperature, flagged.sampler.top_k, flagged.sampler.top_p) == (0.9, 5, 0.95)
    assert _options(_parser().parse_args(["run", "-m", "x", "--temperature", "0", "hi"]), declared).sampler.greedy


def test_meter_separates_the_first_token_from_the_decode_rate(monkeypatch):
    import mlx_omnia_b200.engine.meter as meter_module

    clock = iter([10.0, 10.5, 10.6, 10.8])
    monkeypatch.setattr(meter_module.time, "perf_counter", lambda: next(clock))
    meter = Meter()
    meter.begin(7)
    assert meter.ttft is None and meter.tokens_per_second is None
    for _ in range(3):
        meter.token()
    assert meter.prompt_tokens == 7 and meter.completion_tokens == 3
    assert meter.ttft == pytest.approx(0.5) and meter.decode_seconds == pytest.approx(0.3)
    assert meter.tokens_per_second == pytest.approx(2 / 0.3)  # the first token belongs to the time to first token
    assert "prompt 7 tokens" in meter.line() and "500.0 ms" in meter.line()


def test_pool_is_sized_in_whole_pages_from_free_memory():
    assert pool_tokens(10_000_000, 1000, 16, 0.8) == 8000 - 8000 % 16
    assert pool_tokens(100, 1000, 16, 0.8) == 16  # never less than a page
    assert pool_tokens(1 << 30, 0, 16, 0.8) == 16  # a model that keeps no pages
