"""Constrained decoding: automata, token masks on vocabulary shards, end-to-end guided generation."""
import json

import pytest
import torch

from tileinfer_b200.engine.constraints import (ChoiceFSM, JsonFSM, RegexFSM, VocabIndex, make_constraint)
from tileinfer_b200.engine.llm import LLM
from tileinfer_b200.engine.sampling_params import SamplingParams
from tileinfer_b200.utils.tokenizer import ByteTokenizer


def _accepts(fsm, text):
    st = fsm.start
    for ch in text:
        st = fsm.step(st, ch)
        if st is None:
            return False
    return fsm.accepting(st)


def _prefix_ok(fsm, text):
    st = fsm.start
    for ch in text:
        st = fsm.step(st, ch)
        if st is None:
            return False
    return True


@pytest.mark.parametrize("pattern,good,bad", [
    (r"\d{3}-\d{4}", ["555-1234"], ["55-1234", "555-12345", "abc-1234"]),
    (r"(cat|dog)s?", ["cat", "dogs"], ["cats?", "bird", ""]),
    (r"[a-c]+x*", ["abcabc", "ax", "cxxx"], ["", "x", "ad"]),
    (r"[^0-9]+", ["abc", "-_"], ["a1", ""]),
    (r"a.c", ["abc", "a c"], ["ac", "a\nc"]),
    (r"(ab){2,3}", ["abab", "ababab"], ["ab", "abababab"]),
    (r"\w+@\w+\.com", ["me@host.com"], ["me@host.org", "@host.com"]),
    (r"-?(0|[1-9]\d*)(\.\d+)?", ["0", "-12.50", "7"], ["01", "1.", "--1"]),
])
def test_regex_language(pattern, good, bad):
    fsm = RegexFSM(pattern)
    for g in good:
        assert _accepts(fsm, g), (pattern, g)
    for b in bad:
        assert not _accepts(fsm, b), (pattern, b)


def test_json_automaton():
    fsm = JsonFSM()
    good = ['{}', '{"a":1}', '{"a": [1, 2.5e-3, true, null, "x\\n\\u00e9"], "b": {"c": -0.1}}', '{"k":"v" , "z":[]}']
    for g in good:
        assert _accepts(fsm, g), g
        json.loads(g)
    for b in ['', '[1]', '{"a":}', '{"a":01}', '{a:1}', '{"a":1,}', '{"a":1} x', '{"a":tru}', '{"a":  1}']:
        assert not _accepts(fsm, b), b
    assert _prefix_ok(fsm, '{"a": [1, {"b": "unfinished')
    assert not _prefix_ok(fsm, '{"a" 1')
    deep = '{"a":' * 13
    assert not _prefix_ok(fsm, deep)          # nesting is capped


def test_choice_automaton():
    fsm = ChoiceFSM(["yes", "no", "north"])
    assert _accepts(fsm, "no") and _accepts(fsm, "north") and not _accepts(fsm, "nor")
    assert fsm.can_continue("no") and not fsm.can_continue("yes")


def test_masks_on_vocab_shards_agree_with_full_vocab():
    tok = ByteTokenizer(1024)
    sp = SamplingParams(guided_regex=r"[ab]+c", logit_bias={5: 2.0}, bad_token_ids=[ord("a")])
    c = make_constraint(sp, tok)
    st = c.initial_state()
    full = torch.zeros(1024)
    c.apply(full, st, 0, eos_ids=(1023,))
    parts = []
    for r in range(4):
        shard = torch.zeros(256)
        c.apply(shard, st, r * 256, eos_ids=(1023,))
        parts.append(shard)
    assert torch.equal(torch.cat(parts), full)
    allowed = set(torch.nonzero(full > float("-inf")).flatten().tolist())
    assert allowed == {ord("b")}                                    # 'a' is denied, 'c' needs a prefix first
    st = c.advance(st, ord("b"))
    full = torch.zeros(1024)
    c.apply(full, st, 0, eos_ids=(1023,))
    assert set(torch.nonzero(full > float("-inf")).flatten().tolist()) == {ord("b"), ord("c")}
    st = c.advance(st, ord("c"))
    assert c.is_complete(st)


def test_vocab_index_multichar_tokens():
    class Tok:
        vocab_size = 6
        all_special_ids = [5]
        words = ["ab", "a", "b", "abc", "c", "<eos>"]

        def __len__(self):
            return 6

        def decode(self, ids, skip_special_tokens=False):
            return "".join(self.words[i] for i in ids)
    vi = VocabIndex(Tok())
    fsm = RegexFSM("abc")
    assert sorted(vi.admissible(fsm, fsm.start)) == [0, 1, 3]       # "ab", "a", "abc"
    st = fsm.step(fsm.start, "a")
    assert sorted(vi.admissible(fsm, st)) == [2]                     # only "b"


def test_guided_generation_end_to_end():
    llm = LLM("preset:tiny-hybrid", device="cpu", quantization="bf16", num_kvcache_blocks=64, max_num_seqs=4)
    out = llm.generate(["pick"], SamplingParams(temperature=0.0, max_tokens=20, guided_choice=["alpha", "beta"]))[0]
    assert out["text"] in ("alpha", "beta") and out["finish_reason"] == "stop"
    out = llm.generate(["num"], SamplingParams(temperature=0.7, max_tokens=30, guided_regex=r"\d{2}:\d{2}"))[0]
    assert len(out["text"]) == 5 and out["text"][2] == ":" and out["text"].replace(":", "").isdigit()
    out = llm.generate(["json"], SamplingParams(temperature=0.8, max_tokens=60, guided_json=True))[0]
    if out["finish_reason"] == "stop":
        assert isinstance(json.loads(out["text"]), dict)
    else:                                                           # ran out of tokens: still a valid JSON prefix
        assert _prefix_ok(JsonFSM(), out["text"])
    out = llm.generate_token_ids(["x"], SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True,
                                                       allowed_token_ids=[7, 8]))[0]
    assert set(out) <= {7, 8}
    with pytest.raises(ValueError):
        make_constraint(SamplingParams(guided_regex="a", guided_json=True), llm.tokenizer)
