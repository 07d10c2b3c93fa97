"""Grammar-constrained decoding end to end on CPU (regex, JSON schema, EBNF) with a tokenizer
trained in memory; a random model must still emit only strings of the grammar
(reference tests: `python/sgl_jax/test/srt/test_json_constrained.py`, `test_regex_constrained.py`)."""

import json
import re

import pytest

pytest.importorskip("llguidance")


@pytest.fixture(scope="module")
def engine(tmp_path_factory):
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers
    from transformers import PreTrainedTokenizerFast
    from sglang_jax_b200.entrypoints.engine import Engine
    from sglang_jax_b200.parallel import state as ps
    from sglang_jax_b200.utils.tiny_models import TINY_QWEN3, write_tiny_qwen3_checkpoint
    tok = Tokenizer(models.BPE(unk_token=None))
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = decoders.ByteLevel()
    tr = trainers.BpeTrainer(vocab_size=600, special_tokens=["<|endoftext|>"],
                             initial_alphabet=pre_tokenizers.ByteLevel.alphabet())
    tok.train_from_iterator(['{"name": "alice", "age": 31}', "hello world 12345 yes no true false null",
                             '[1, 2, 3] {"a": [true]}'] * 50, tr)
    d = str(tmp_path_factory.mktemp("gram"))
    write_tiny_qwen3_checkpoint(d, config=dict(TINY_QWEN3, vocab_size=640, eos_token_id=0))
    PreTrainedTokenizerFast(tokenizer_object=tok, eos_token="<|endoftext|>").save_pretrained(d)
    ps.reset_state()
    eng = Engine(model_path=d, device="cpu", enable_single_process=True, page_size=4, max_total_tokens=4096,
                 dtype="float32", log_level="error", constrained_json_disable_any_whitespace=True)
    yield eng
    eng.shutdown()


def test_regex(engine):
    pat = r"(yes|no) [0-9]{3}"
    outs = engine.generate(prompt=["Give me a number:", "Another:"],
                           sampling_params={"temperature": 0.0, "max_new_tokens": 24, "regex": pat})
    for o in outs:
        assert re.fullmatch(pat, o["text"]), o["text"]
        assert o["meta_info"]["finish_reason"]["type"] == "stop"
    sampled = engine.generate(prompt="x", sampling_params={"temperature": 1.0, "max_new_tokens": 24, "regex": pat})
    assert re.fullmatch(pat, sampled["text"])


def test_json_schema_and_overlap_with_plain_requests(engine):
    schema = {"type": "object", "properties": {"name": {"type": "string", "maxLength": 4}, "ok": {"type": "boolean"},
                                               "n": {"type": "integer", "minimum": 0, "maximum": 9}},
              "required": ["name", "ok", "n"], "additionalProperties": False}
    outs = engine.generate(prompt=["json:", "free text"],
                           sampling_params=[{"temperature": 0.0, "max_new_tokens": 64, "json_schema": json.dumps(schema)},
                                            {"temperature": 0.0, "max_new_tokens": 8, "ignore_eos": True}])
    obj = json.loads(outs[0]["text"])
    assert set(obj) == {"name", "ok", "n"} and isinstance(obj["ok"], bool) and 0 <= obj["n"] <= 9
    assert len(outs[1]["output_ids"]) == 8


def test_ebnf_and_invalid_grammar(engine):
    o = engine.generate(prompt="x:", sampling_params={"temperature": 0.0, "max_new_tokens": 12,
                                                      "ebnf": 'root ::= "a" root | "b"'})
    assert re.fullmatch(r"a*b?", o["text"]) and o["text"]
    with pytest.raises(Exception):
        engine.generate(prompt="x", sampling_params={"max_new_tokens": 4, "regex": "(unclosed"})
