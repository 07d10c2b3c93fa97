"""Small utilities: template helpers, tiktoken adapter, trace diff, EPLB tools, named scopes."""

import base64
import json
import os

import numpy as np
import pytest


def test_template_content_format_and_processing():
    from sglang_jax_b200.jinja_template_utils import (detect_template_content_format,
                                                      process_content_for_template_format, render_template)
    plain = "{% for m in messages %}{{ m.role }}: {{ m.content }}\n{% endfor %}"
    rich = "{% for m in messages %}{% for c in m.content %}{% if c.type == 'text' %}{{ c.text }}{% endif %}{% endfor %}{% endfor %}"
    assert detect_template_content_format(plain) == "string" and detect_template_content_format(rich) == "openai"
    msg = {"role": "user", "content": [{"type": "text", "text": "look"}, {"type": "image_url", "image_url": {"url": "u"}},
                                       {"type": "text", "text": "here"}]}
    imgs = []
    s = process_content_for_template_format(msg, "string", imgs)
    assert s["content"] == "look here" and imgs == ["u"]
    o = process_content_for_template_format(msg, "openai")
    assert [c["type"] for c in o["content"]] == ["text", "image", "text"]
    assert render_template(plain, messages=[{"role": "user", "content": "hi"}]) == "user: hi\n"
    from sglang_jax_b200.conversation import Conversation
    c = Conversation(system="be brief")
    c.add_message("user", "hi")
    assert c.get_prompt() == "system: be brief\nuser: hi\nassistant:"


def test_tiktoken_adapter(tmp_path):
    pytest.importorskip("tiktoken")
    from sglang_jax_b200.utils.tiktoken_tokenizer import TiktokenTokenizer
    path = tmp_path / "tok.tiktoken"
    toks = [bytes([i]) for i in range(256)] + [b"he", b"ll", b"hell", b"hello", b" wor", b" world"]
    path.write_bytes(b"\n".join(base64.b64encode(t) + b" " + str(i).encode() for i, t in enumerate(toks)))
    (tmp_path / "tokenizer_config.json").write_text(json.dumps(
        {"chat_template": "{% for m in messages %}<{{ m.role }}>{{ m.content }}{% endfor %}"}))
    t = TiktokenTokenizer(str(path))
    ids = t.encode("hello world")
    assert ids == [259, 261] and t.decode(ids) == "hello world"
    assert t.decode(ids + [t.eos_token_id]) == "hello world" and t.vocab_size == 263
    assert t.apply_chat_template([{"role": "user", "content": "hello"}], tokenize=False) == "<user>hello"


def test_trace_diff_finds_first_divergence(tmp_path):
    from sglang_jax_b200.utils.trace_diff import diff, load, main
    a, b = tmp_path / "a.jsonl", tmp_path / "b.jsonl"
    recs = [{"forward": 0, "stage": "EXTEND", "name": "layer_residual", "layer": i, "mean": 0.1 * i, "std": 1.0,
             "abs_max": 3.0} for i in range(4)]
    a.write_text("\n".join(json.dumps(r) for r in recs))
    recs[2]["std"] = 1.5
    b.write_text("\n".join(json.dumps(r) for r in recs))
    rows = diff(load(str(a)), load(str(b)))
    assert [r["ok"] for r in rows] == [True, True, False, True]
    assert main([str(a), str(a)]) == 0 and main([str(a), str(b)]) == 1


def test_eplb_tools_report_improvement(tmp_path, capsys):
    from sglang_jax_b200.eplb.tools import device_imbalance, hot_experts, main
    rng = np.random.RandomState(0)
    counts = rng.poisson(50, size=(3, 16)).astype(np.float64)
    counts[:, 0] *= 20                                   # one very hot expert
    p = tmp_path / "c.npy"
    np.save(p, counts)
    assert hot_experts(counts, 2)[0][0][0] == 0
    assert device_imbalance(counts, 4).min() > 2.0
    assert main(["rebalance", str(p), "--num-devices", "4", "--redundant", "4"]) == 0
    out = capsys.readouterr().out
    before = float(out.split("before: mean device max/mean ")[1].split()[0])
    after = float(out.split("after : mean device max/mean ")[1].split()[0])
    assert after < before
    assert main(["inspect", str(p), "--topk", "3"]) == 0 and main(["hot", str(p), "--num-devices", "4"]) == 0


def test_named_scope_and_timeit():
    from sglang_jax_b200.utils.perf import multiple_iteration_timeit
    from sglang_jax_b200.utils.profiling_utils import named_scope

    @named_scope
    def f(x):
        return x + 1

    @named_scope(name="g-scope")
    def g(x):
        return x * 2

    with named_scope("block"):
        assert f(1) == 2 and g(2) == 4
    r = multiple_iteration_timeit(lambda: sum(range(1000)), warmup=1, iters=3, device="cpu")
    assert r["iters"] == 3 and r["min_ms"] <= r["median_ms"]


def test_accuracy_evals_score_known_samplers(tmp_path):
    """MMLU / GSM8K harness: an oracle sampler scores 1, a wrong one 0, a half-right one 0.5."""
    import csv
    import json
    from sglang_jax_b200.test.eval.simple_eval_common import SamplerBase, make_report, normalize_number
    from sglang_jax_b200.test.eval.simple_eval_gsm8k import GSM8KEval
    from sglang_jax_b200.test.eval.simple_eval_mmlu import MMLUEval
    rows = [dict(Question=f"q{i}?", A="a", B="b", C="c", D="d", Answer="ABCD"[i % 4],
                 Subject=["abstract_algebra", "philosophy"][i % 2]) for i in range(8)]
    p = tmp_path / "mmlu.csv"
    with open(p, "w", newline="") as f:
        w = csv.DictWriter(f, fieldnames=list(rows[0]))
        w.writeheader()
        w.writerows(rows)

    class Oracle(SamplerBase):
        def __init__(self, right):
            self.right = right

        def __call__(self, messages):
            q = messages[-1]["content"]
            i = int(q.split("q")[-1].split("?")[0]) if "?" in q else 0
            return f"thinking...\nAnswer: {'ABCD'[i % 4] if self.right(i) else 'ABCD'[(i + 1) % 4]}"

    assert MMLUEval(str(p), num_threads=2)(Oracle(lambda i: True)).score == 1.0
    assert MMLUEval(str(p), num_threads=1)(Oracle(lambda i: False)).score == 0.0
    half = MMLUEval(str(p))(Oracle(lambda i: i % 2 == 0))
    assert half.score == 0.5 and half.metrics["stem"] == 1.0 and half.metrics["humanities"] == 0.0
    assert "score: 0.5" in make_report(half)
    g = tmp_path / "gsm.jsonl"
    with open(g, "w") as f:
        for i in range(9):
            f.write(json.dumps({"question": f"what is {i}+{i}?", "answer": f"work\n#### {2 * i:,}"}) + "\n")

    class Adder(SamplerBase):
        def __call__(self, messages):
            a = int(messages[-1]["content"].rsplit("what is ", 1)[1].split("+")[0])
            assert messages[-1]["content"].count("Question:") == 4            # 3 shots + the question
            return f"{a}+{a}\nAnswer: ${2 * a}.0"

    ev = GSM8KEval(str(g), num_shots=3, num_threads=2)
    assert len(ev.examples) == 6 and ev(Adder()).score == 1.0
    assert normalize_number("1,234.0") == "1234" and normalize_number("about 12 apples") == "12"


def test_varlen_page_packing_and_reference_attention():
    """The page layout the varlen attention kernel reads (every sequence on its own pages, page 0 a zero dummy) and
    the PyTorch statement of bidirectional packed attention (sequences do not see each other)."""
    import torch
    from sglang_jax_b200 import ops
    from sglang_jax_b200.ops.native import pack_varlen_pages
    torch.manual_seed(0)
    lens = [5, 64, 130, 0, 1]
    T = sum(lens)
    k, v = torch.randn(T, 2, 8), torch.randn(T, 2, 8)
    cache, pt, lens_t, cu, n_pages, max_pages = pack_varlen_pages(k, v, lens, 64)
    assert cache.shape == (7, 2, 2, 64, 8) and n_pages == 7 and max_pages == 3
    assert pt.tolist() == [[1, 0, 0], [2, 0, 0], [3, 4, 5], [0, 0, 0], [6, 0, 0]]
    assert cu.tolist() == [0, 5, 69, 199, 199, 200] and lens_t.tolist() == lens
    assert not cache[0].any()
    o = 0
    for b, n in enumerate(lens):
        if n:
            pages = pt[b, : (n + 63) // 64].long()
            assert torch.equal(cache[pages, 0].permute(0, 2, 1, 3).reshape(-1, 2, 8)[:n], k[o:o + n])
            assert torch.equal(cache[pages, 1].permute(0, 2, 1, 3).reshape(-1, 2, 8)[:n], v[o:o + n])
        o += n
    q = torch.randn(T, 4, 8)
    out = ops.varlen_attention(q, k, v, lens, 8 ** -0.5)
    alone = ops.varlen_attention(q[5:69], k[5:69], v[5:69], [64], 8 ** -0.5)
    assert torch.allclose(out[5:69], alone, atol=1e-6)
    sd = torch.nn.functional.scaled_dot_product_attention(
        q[5:69].transpose(0, 1)[None], k[5:69].transpose(0, 1).repeat_interleave(2, 0)[None],
        v[5:69].transpose(0, 1).repeat_interleave(2, 0)[None])[0].transpose(0, 1)
    assert torch.allclose(alone, sd, atol=1e-5)


def test_fused_residual_dataflow_is_chosen_per_model():
    """A LoRA adapter on a row-parallel projection cannot feed the fused reduce: the whole model then keeps the
    replicated residual stream; bias and quantised weights still qualify (their local product is a partial sum)."""
    import torch
    from sglang_jax_b200.layers.fused_block import model_supports_fused_residual, row_linear_qualifies
    from sglang_jax_b200.layers.linear import RowParallelLinear

    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.o_proj = RowParallelLinear(64, 32, True, torch.float32, tp_size=2, tp_rank=0)
            self.down_proj = RowParallelLinear(64, 32, False, torch.float32, tp_size=2, tp_rank=0)

    m = Block()
    assert model_supports_fused_residual(m)
    m.o_proj.lora = object()
    assert not row_linear_qualifies(m.o_proj) and not model_supports_fused_residual(m)
    m.o_proj.lora = None
    m.down_proj.qweight = object()
    assert model_supports_fused_residual(m)


def test_bench_serving_dataset_samplers(tmp_path):
    import json
    from sglang_jax_b200 import bench_serving as bs
    lengths = bs._Lengths(None)
    sg = tmp_path / "sg.json"
    sg.write_text(json.dumps([{"conversations": [{"from": "human", "value": f"question number {i} please"},
                                                 {"from": "gpt", "value": "an answer of six words here"}]}
                              for i in range(6)] + [{"conversations": [{"from": "human", "value": "x"}]}]))
    reqs = bs.sample_sharegpt_requests(str(sg), 4, lengths)
    assert len(reqs) == 4 and all(o == 6 and p.startswith("question") for p, o in reqs)
    assert bs.sample_sharegpt_requests(str(sg), 4, lengths, fixed_output_len=9)[0][1] == 9
    cu = tmp_path / "c.jsonl"
    cu.write_text("\n".join([json.dumps({"prompt": "a b c", "output_len": 7}), json.dumps({"input_ids": [1, 2, 3]}),
                             json.dumps({"conversations": [{"content": "hi"}, {"content": "hello you"}]})]))
    assert bs.sample_custom_requests(str(cu), 10, lengths) == [("a b c", 7), ([1, 2, 3], 128), ("hi", 2)]
    mc = tmp_path / "m.jsonl"
    mc.write_text("\n".join(json.dumps({"timestamp": 250 * i, "input_length": 600, "output_length": 3,
                                        "hash_ids": [7, 100 + i]}) for i in range(3)))
    tr = bs.sample_mooncake_requests(str(mc), 3, 1000, block_tokens=512)
    assert [(len(a), b, c) for a, b, c in tr] == [(600, 3, 0.0), (600, 3, 0.25), (600, 3, 0.5)]
    assert tr[0][0][:512] == tr[1][0][:512] and tr[0][0][512:] != tr[1][0][512:]      # shared first block only
    msgs, out = bs.sample_image_requests(1, 2, "32x16", 8, 4)[0]
    kinds = [c["type"] for c in msgs[0]["content"]]
    assert kinds == ["image_url", "image_url", "text"] and out == 4
    import base64
    png = base64.b64decode(msgs[0]["content"][0]["image_url"]["url"].split(",", 1)[1])
    assert png[:8] == b"\x89PNG\r\n\x1a\n" and png[16:24] == (32).to_bytes(4, "big") + (16).to_bytes(4, "big")
    # peak output throughput: tokens per one-second bucket of chunk arrivals
    o = bs.RequestFuncOutput(success=True, latency=2.0, ttft=0.1, itl=[0.1] * 9, prompt_len=5, output_len=10, start=0.0,
                             chunk_times=[0.1 * (i + 1) for i in range(10)])
    m = bs.calculate_metrics([o], 2.0)
    assert m["peak_output_throughput"] >= 9 and m["output_throughput"] == 5.0


def test_gemm_plan_is_measured_once_and_persisted(tmp_path):
    """The tuning cache measures a decode-sized GEMM shape the first time it is met, keeps the winner on disk and
    answers from the table afterwards (also in a fresh process: a second instance on the same file)."""
    from sglang_jax_b200.model_executor.tuning_cache import GemmPlan
    path = str(tmp_path / "plan.json")
    calls = []
    plan = GemmPlan(path, measure=False)
    assert plan.mode_for(128, 5120, 1024, lambda m: calls.append(m)) == -1 and not calls   # nothing known, no measuring
    plan.table["128x5120x1024"] = 0
    plan.dirty = True
    plan.save()
    again = GemmPlan(path, measure=True)
    assert again.mode_for(100, 5120, 1024, lambda m: calls.append(m)) == 0 and not calls    # bucket 128, from disk
    assert again.mode_for(4096, 5120, 1024, lambda m: calls.append(m)) == -1               # prefill sizes: default


def test_suite_runner_checks_floors_on_the_cpu_smoke_suite():
    """The named-suite runner: cases run through the engine, metrics are compared with floors, a floor that is out of
    reach fails the case (reference `test/srt/nightly/single_host/suite_runner.py`)."""
    from sglang_jax_b200.parallel import state as ps
    from sglang_jax_b200.test import suite_runner as sr
    assert {"perf-text-models-b200-1", "perf-moe-models-b200", "smoke-cpu"} <= set(sr.SUITES)
    big = sr.SUITES["perf-text-models-b200-1"]
    assert [c.kind for c in big] == ["decode", "decode", "prefill"] and big[1].floors == {"out_tps": 865.6}
    ps.reset_state()
    res = sr.run_suite("smoke-cpu")
    assert len(res) == 3 and all(r["passed"] for r in res)
    assert res[0]["requests"] == 4 and res[-1]["kind"] == "prefill" and res[-1]["in_tps"] > res[-1]["out_tps"]
    ps.reset_state()
    import dataclasses
    hard = sr.run_case(dataclasses.replace(sr.SUITES["smoke-cpu"][0], floors={"out_tps": 1e12}))
    assert not hard["passed"] and "out_tps" in hard["violations"]
    ps.reset_state()


def test_further_accuracy_evals_score_scripted_samplers(tmp_path):
    """MATH / AIME / GPQA / HumanEval / MGSM / C-SimpleQA against samplers with scripted replies: extraction rules,
    option shuffling, sandboxed execution with a time limit, grader labels."""
    import csv
    import json
    from sglang_jax_b200.test.eval import simple_eval_more as m
    from sglang_jax_b200.test.run_eval import build_eval
    # MATH: last "Answer:" line, LaTeX normalisation, checker only asked when strings differ
    with open(tmp_path / "math.csv", "w", newline="") as f:
        w = csv.writer(f)
        w.writerows([["Question", "Answer"], ["1/2 + 1/4?", "\\frac{3}{4}"], ["2+2?", "4"], ["sqrt(16)?", "4"]])
    replies = {"1/2": "think...\nAnswer: $\\dfrac{3}{4}$", "2+2": "Answer: 5", "sqrt": "no final line"}
    asked = []
    res = m.MathEval(str(tmp_path / "math.csv"), equality_checker=lambda msgs: asked.append(1) or "No")(
        lambda msgs: next(v for k, v in replies.items() if k in msgs[0]["content"]))
    assert abs(res.score - 1 / 3) < 1e-9 and abs(res.metrics["invalid"] - 1 / 3) < 1e-9 and len(asked) == 1
    # AIME: nested braces, integer compare
    assert m.boxed_answer("so \\boxed{\\frac{1}{2}} then \\boxed{042}") == "042" and m.same_integer("42", "042")
    (tmp_path / "aime.jsonl").write_text(json.dumps({"problem": "p1", "answer": 42}) + "\n" + json.dumps({"question": "p2", "answer": "7"}) + "\n")
    res = build_eval("aime25", str(tmp_path / "aime.jsonl"), None, 1)(lambda msgs: "\\boxed{42}")
    assert res.score == 0.5
    # GPQA: the correct option moves with the seeded permutation; a sampler that finds it by text scores 1
    with open(tmp_path / "gpqa.csv", "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["Question", "Correct Answer", "Incorrect Answer 1", "Incorrect Answer 2", "Incorrect Answer 3"])
        for i in range(6):
            w.writerow([f"q{i}", f"right{i}", "w1", "w2", "w3"])

    def finder(msgs):
        lines = msgs[0]["content"].splitlines()
        return "Answer: " + next(l[0] for l in lines if "right" in l)
    ev = m.GPQAEval(str(tmp_path / "gpqa.csv"))
    assert ev(finder).score == 1.0 and ev(lambda msgs: "Answer: A").score < 1.0
    assert len({tuple(e["permutation"]) for e in ev.examples}) > 1
    # HumanEval: fenced code is extracted and run; wrong code and endless loops fail within the limit
    task = {"task_id": "t/0", "prompt": "def add(a, b):\n    \"\"\"sum\"\"\"\n", "entry_point": "add",
            "test": "def check(f):\n    assert f(2, 3) == 5\n"}
    (tmp_path / "he.jsonl").write_text(json.dumps(task) + "\n")
    he = m.HumanEvalEval(str(tmp_path / "he.jsonl"), timeout=3.0, num_threads=1)
    assert he(lambda msgs: "```python\ndef add(a, b):\n    return a + b\n```").score == 1.0
    assert he(lambda msgs: "    return a + b\n").score == 1.0                       # bare body continues the stub
    assert he(lambda msgs: "```python\ndef add(a, b):\n    return a - b\n```").score == 0.0
    assert he(lambda msgs: "```python\ndef add(a, b):\n    while True:\n        pass\n```").score == 0.0
    # MGSM: per-language prefix
    (tmp_path / "mgsm_en.tsv").write_text("q1\t18\nq2\t3\n")
    (tmp_path / "mgsm_de.tsv").write_text("f1\t5\n")
    mg = m.MGSMEval(str(tmp_path))
    res = mg(lambda msgs: "Antwort: 5" if msgs[0]["content"].startswith("Löse") else "steps\nAnswer: 18.")
    assert res.metrics["de"] == 1.0 and res.metrics["en"] == 0.5 and abs(res.score - 2 / 3) < 1e-9
    # C-SimpleQA: grader letters -> correct / incorrect / not attempted, F1 of accuracy-given-attempted and correct
    (tmp_path / "sqa.jsonl").write_text("".join(json.dumps({"question": f"q{i}", "answer": f"a{i}"}) + "\n" for i in range(4)))
    grades = iter(["A", "B: INCORRECT", "C", "A"])
    res = m.CSimpleQAEval(str(tmp_path / "sqa.jsonl"), grader=lambda msgs: next(grades), num_threads=1)(lambda msgs: "x")
    assert res.score == 0.5 and res.metrics["is_not_attempted"] == 0.25
    assert abs(res.metrics["accuracy_given_attempted"] - 2 / 3) < 1e-9 and abs(res.metrics["f1"] - 4 / 7) < 1e-9


def test_penalty_state_restart_and_decode_updates():
    """The device-side count table: a (re)starting request seeds its slot with the tokens it already generated (a
    retracted request prefills again over prompt + output), decode steps add their input ids, other slots stay."""
    import numpy as np
    import torch
    from sglang_jax_b200.sampling.penaltylib import PenaltyInfo, PenaltyState
    st = PenaltyState(4, 16, torch.device("cpu"))
    info = PenaltyInfo(np.array([1.0, 0.0], np.float32), np.array([0.5, 0.0], np.float32), np.array([0, 3], np.int32),
                       np.array([3, 0], np.int32), np.array([[-1, -1], [7, 9]], np.int32),
                       np.array([0, 1], np.int32), [[5, 5, 2], []])
    out = st.apply(torch.zeros(2, 16), info, [2, 0], None, False)
    assert st.counts[2].tolist()[2] == 1 and st.counts[2].tolist()[5] == 2 and int(st.counts[0].sum()) == 0
    assert out[0, 5] == -2.5 and out[0, 2] == -1.5 and out[0, 0] == 0.0
    assert out[1, 7] == float("-inf") and out[1, 9] == float("-inf") and out[1, 8] == 0.0     # min_new_tokens
    dec = PenaltyInfo(info.frequency, info.presence, info.min_new_tokens, np.array([4, 3], np.int32), info.stop_ids,
                      np.empty(0, np.int32), [])
    out = st.apply(torch.zeros(2, 16), dec, [2, 0], torch.tensor([5, 7]), True)
    assert st.counts[2, 5] == 3 and st.counts[0, 7] == 1 and out[0, 5] == -3.5 and out[1, 7] == 0.0
    assert int(st.counts[1].sum()) == 0 and int(st.counts[3].sum()) == 0


def test_residual_dataflow_token_window():
    """The fused NVLink dataflow is chosen for forwards inside the token window only (decode-sized ones by default)."""
    from types import SimpleNamespace
    from sglang_jax_b200.layers import fused_block
    from sglang_jax_b200.model_executor.model_runner import ModelRunner
    model = SimpleNamespace(model=SimpleNamespace(layers_to_capture=None), capture_aux_hidden_states=False)
    r = SimpleNamespace(fused_residual_ok=True, fused_min_tokens=0, fused_max_tokens=512, model=model)
    fb = lambda n: SimpleNamespace(num_tokens=n, extras={})
    try:
        assert ModelRunner.select_residual_dataflow(r, fb(128)) is True
        assert fused_block._FUSED_RESIDUAL is True
        assert ModelRunner.select_residual_dataflow(r, fb(1300)) is False
        assert fused_block._FUSED_RESIDUAL is False
        r.fused_min_tokens = 256
        assert ModelRunner.select_residual_dataflow(r, fb(128)) is False
        assert ModelRunner.select_residual_dataflow(r, fb(300)) is True
        assert ModelRunner.select_residual_dataflow(r, SimpleNamespace(num_tokens=300, extras={"deepstack": 1})) is False
    finally:
        fused_block.set_fused_residual(True)


def test_kv_pool_canary_pages_catch_a_write_past_the_pool(monkeypatch):
    """Guard pages behind every layer's KV buffer (the stand-in for a memory checker on the pools)."""
    import pytest
    import torch
    from sglang_jax_b200.mem_cache.memory_pool import MHATokenToKVPool
    pool = MHATokenToKVPool(32, 4, torch.float32, 2, 8, 2, "cpu", canary_pages=2)
    assert pool.kv_buffer[0].shape[0] == pool.num_pages and pool.kv_buffer[0].is_contiguous()
    loc = torch.arange(4, 36)
    pool.set_kv_buffer(0, loc, torch.randn(32, 2, 8), torch.randn(32, 2, 8))       # every legal slot
    pool.check_canaries()
    # a page id one past the pool (what a kernel with a bad page-table entry would write through)
    whole = pool.kv_buffer[1]._base
    whole[pool.num_pages, 0, 0, 0, 0] = 1.0
    with pytest.raises(RuntimeError, match=f"guard page {pool.num_pages} of layer 1"):
        pool.check_canaries()
    # the environment switch is the default source of the page count; without it nothing is added
    monkeypatch.setenv("SGLB_KV_CANARY_PAGES", "1")
    assert MHATokenToKVPool(8, 4, torch.float32, 1, 8, 1, "cpu").canary_pages == 1
    monkeypatch.delenv("SGLB_KV_CANARY_PAGES")
    plain = MHATokenToKVPool(8, 4, torch.float32, 1, 8, 1, "cpu")
    assert plain.canary_pages == 0 and plain.kv_buffer[0]._base is None
    plain.check_canaries()


def test_checked_kernel_build_compiles(tmp_path):
    """The -DSGLB_BOUNDS_CHECK variant of the KV-write kernel keeps compiling for sm_100a (it cannot run here)."""
    import os
    import shutil
    import subprocess
    from sglang_jax_b200.csrc import build as b
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not available")
    src = os.path.join(b.HERE, "elementwise.cu")
    flags = [f for f in b.NVCC_FLAGS if f not in ("-shared", "-DSGLB_BOUNDS_CHECK")]
    r = subprocess.run([nvcc, *flags, "-DSGLB_BOUNDS_CHECK", "-I", b.HERE, "-c", src, "-o", str(tmp_path / "e.o")],
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert r.returncode == 0, r.stdout
    syms = subprocess.run(["nm", "-C", str(tmp_path / "e.o")], stdout=subprocess.PIPE, text=True).stdout
    assert "sglb_debug_set_kv_pages" in syms


def test_moe_parity_tool_on_a_tiny_checkpoint(tmp_path, capsys):
    """`utils/moe_parity.py`: one MoE layer's checkpoint weights through the framework's expert FFN against an fp32
    expert-by-expert loop; per-expert and fused checkpoint layouts, key listing, quantised experts, npz dump."""
    import json
    import numpy as np
    import torch
    from safetensors.torch import save_file
    from sglang_jax_b200.parallel import state as ps
    from sglang_jax_b200.utils import moe_parity
    ps.reset_state()
    E, H, I = 8, 64, 32
    g = torch.Generator().manual_seed(0)
    sd = {"model.layers.1.mlp.gate.weight": torch.randn(E, H, generator=g) * 0.2,
          "model.layers.1.post_attention_layernorm.weight": 1 + 0.1 * torch.randn(H, generator=g)}
    for e in range(E):
        for n, shape in (("gate_proj", (I, H)), ("up_proj", (I, H)), ("down_proj", (H, I))):
            sd[f"model.layers.1.mlp.experts.{e}.{n}.weight"] = torch.randn(*shape, generator=g) * 0.1
    d = tmp_path / "per_expert"
    d.mkdir()
    save_file(sd, str(d / "model.safetensors"))
    (d / "config.json").write_text(json.dumps(dict(num_experts=E, num_experts_per_tok=2, norm_topk_prob=True)))
    common = ["--model-dir", str(d), "--from-config", "--layer-idx", "1", "--num-tokens", "24", "--device", "cpu"]
    assert moe_parity.main(common + ["--dtype", "float32", "--atol", "1e-4", "--tokens-apply-rmsnorm",
                                     "--dump-npz", str(tmp_path / "o.npz"), "--debug-topn", "2"]) == 0
    out = capsys.readouterr().out
    rep = json.loads(out.splitlines()[0])
    assert rep["experts"] == E and rep["hidden"] == H and rep["intermediate"] == I and rep["max_abs"] < 1e-4
    assert "token" in out.splitlines()[1]
    z = np.load(tmp_path / "o.npz")
    assert z["framework"].shape == (24, H) and np.allclose(z["framework"], z["reference"], atol=1e-4)
    # key listing with a filter
    assert moe_parity.main(["--model-dir", str(d), "--list-keys", "--match", r"experts\.3\."]) == 0
    assert "3 keys" in capsys.readouterr().out
    # the fused checkpoint layout gives the same layer
    fused = {"model.layers.1.mlp.gate.weight": sd["model.layers.1.mlp.gate.weight"],
             "model.layers.1.mlp.experts.gate_up_proj": torch.stack([torch.cat(
                 [sd[f"model.layers.1.mlp.experts.{e}.gate_proj.weight"],
                  sd[f"model.layers.1.mlp.experts.{e}.up_proj.weight"]], 0) for e in range(E)]),
             "model.layers.1.mlp.experts.down_proj": torch.stack(
                 [sd[f"model.layers.1.mlp.experts.{e}.down_proj.weight"] for e in range(E)])}
    d2 = tmp_path / "fused"
    d2.mkdir()
    save_file(fused, str(d2 / "model.safetensors"))
    (d2 / "config.json").write_text((d / "config.json").read_text())
    assert moe_parity.main(["--model-dir", str(d2), "--from-config", "--layer-idx", "1", "--num-tokens", "24",
                            "--device", "cpu", "--dtype", "float32", "--atol", "1e-4"]) == 0
    capsys.readouterr()
    # quantised experts: the report is the recipe's error on this layer (small, not zero), bf16 tokens
    assert moe_parity.main(common + ["--moe-weight-dtype", "float8_e4m3fn", "--deterministic-router"]) == 0
    q = json.loads(capsys.readouterr().out.splitlines()[0])
    assert 1e-5 < q["rel_fro"] < 0.1 and q["cosine"] > 0.99 and q["experts_hit"] == E


def test_recurrent_state_pool_sizing_rules():
    """`--max-recurrent-state-size` (total slots, request slots included) wins; without prefix sharing there are no
    checkpoint slots; an explicit `--recurrent-snapshot-slots` is taken as is; `-1` derives the pool from the share
    `ratio / (1 + ratio)` of the available memory."""
    import pytest
    import torch
    from sglang_jax_b200.mem_cache.recurrent_state_pool import RecurrentStatePool, plan_state_slots, slot_bytes
    spec = dict(num_layers=3, conv_dim=64, conv_kernel=4, num_heads=4, head_k_dim=8, head_v_dim=8)
    per = slot_bytes(**spec)
    pool = RecurrentStatePool(5, snapshot_slots=2, **spec)
    assert pool.size_bytes() == (5 + 1 + 2) * per
    assert plan_state_slots(16, per, 0, 40, 7, 0.9, True) == (24, (16 + 1 + 24) * per)
    assert plan_state_slots(16, per, 0, 10, 7, 0.9, True)[0] == 0            # smaller than the request slots
    assert plan_state_slots(16, per, 0, None, 7, 0.9, False)[0] == 0
    assert plan_state_slots(16, per, 0, None, 7, 0.9, True)[0] == 7
    avail = 1000 * per
    snap, used = plan_state_slots(16, per, avail, None, -1, 1.0, True)       # half of the memory -> 500 slots
    assert snap == 500 - 16 and used == (16 + 1 + snap) * per
    with pytest.raises(ValueError):
        plan_state_slots(16, per, avail, None, -1, 0.0, True)


def test_hub_ids_resolve_through_download_dir_and_draft_revision(tmp_path, monkeypatch):
    """A model path that is not a directory is fetched into `--download-dir` at the configured revision; the draft
    model of speculative decoding uses `--speculative-draft-model-revision`."""
    import json
    import sys
    import types
    from sglang_jax_b200.configs.model_config import ModelConfig
    from sglang_jax_b200.server_args import ServerArgs
    from sglang_jax_b200.utils.tiny_models import TINY_QWEN3
    local = tmp_path / "snap"
    local.mkdir()
    (local / "config.json").write_text(json.dumps(dict(TINY_QWEN3)))
    calls = []
    fake = types.ModuleType("huggingface_hub")

    def snapshot_download(repo_id, cache_dir=None, revision=None, allow_patterns=None, **kw):
        calls.append((repo_id, cache_dir, revision))
        return str(local)

    fake.snapshot_download = snapshot_download
    monkeypatch.setitem(sys.modules, "huggingface_hub", fake)
    sa = ServerArgs(model_path="org/tiny-model", download_dir=str(tmp_path / "dl"), revision="r1",
                    speculative_draft_model_revision="d7", skip_tokenizer_init=True, device="cpu")
    mc = ModelConfig.from_server_args(sa)
    assert mc.model_path == str(local) and calls[-1] == ("org/tiny-model", str(tmp_path / "dl"), "r1")
    ModelConfig.from_server_args(sa, model_path="org/tiny-draft", is_draft_model=True)
    assert calls[-1] == ("org/tiny-draft", str(tmp_path / "dl"), "d7")
    ModelConfig.from_server_args(sa, model_path=str(local))             # a directory is used as is
    assert len(calls) == 2


def test_sequence_parallel_flag_selects_the_token_sharded_dataflow(monkeypatch):
    """`--enable-sequence-parallel` turns the token-sharded (reduce-scatter) residual dataflow on for every forward;
    the default window is empty; the environment variables override both."""
    from types import SimpleNamespace
    from sglang_jax_b200.model_executor.model_runner import fused_token_window
    monkeypatch.delenv("SGLB_FUSED_MAX_TOKENS", raising=False)
    monkeypatch.delenv("SGLB_FUSED_MIN_TOKENS", raising=False)
    assert fused_token_window(SimpleNamespace(enable_sequence_parallel=False)) == (0, -1)
    assert fused_token_window(SimpleNamespace(enable_sequence_parallel=True)) == (0, 1000000)
    monkeypatch.setenv("SGLB_FUSED_MAX_TOKENS", "512")
    monkeypatch.setenv("SGLB_FUSED_MIN_TOKENS", "64")
    assert fused_token_window(SimpleNamespace(enable_sequence_parallel=True)) == (64, 512)


def test_bench_py_contract_on_cpu():
    """`bench.py` end to end on CPU with a one-layer debug model: one JSON line with the keys the driver reads, the
    per-kind step breakdown, and the `invalid` mark of a debug run."""
    import json
    import subprocess
    import sys
    root = os.path.join(os.path.dirname(__file__), "..")
    r = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--model", "qwen3-8b", "--layers", "1",
                        "--concurrency", "4", "--input-len-min", "16", "--input-len-max", "32", "--output-len", "8",
                        "--steps", "6", "--warmup", "3", "--no-latency", "--no-e2e"],
                       stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=900, cwd=root)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    for k in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
              "vs_baseline", "dtype", "data", "config", "clocks", "e2e", "gpu_launches", "step_breakdown"):
        assert k in d, k
    assert d["steps"] == 6 and d["warmup"] == 3 and d["n_gpus"] == 1 and d["value"] > 0 and d["invalid"]
    sb = d["step_breakdown"]
    assert sb["decode"]["steps"] + sb["prefill"]["steps"] == 6 and d["config"]["tp_dataflow"] is None
    ref = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference"],
                         stdout=subprocess.PIPE, text=True, timeout=300, cwd=root)
    out = json.loads([l for l in ref.stdout.splitlines() if l.startswith("{")][-1])
    assert ref.returncode == 0 and out["impl"] == "reference" and "unavailable" in out


def test_bench_serving_client_options_against_a_fake_server(tmp_path):
    """The serving benchmark client against a recording server: non-streaming requests, adapters spread over the
    requests, routing keys of shared-prefix groups, extra headers, warm-up requests, tags and per-request details."""
    import asyncio
    import json
    import threading
    from aiohttp import web
    from sglang_jax_b200 import bench_serving as bs
    from sglang_jax_b200.utils.common import get_free_port
    seen = []

    async def generate(request):
        body = await request.json()
        seen.append((body, request.headers.get("X-Test")))
        n = body["sampling_params"]["max_new_tokens"]
        meta = {"completion_tokens": n, "prompt_tokens": len(body.get("input_ids") or [])}
        if body.get("stream"):
            resp = web.StreamResponse(headers={"Content-Type": "text/event-stream"})
            await resp.prepare(request)
            for i in range(1, n + 1):
                await resp.write(("data: " + json.dumps({"meta_info": dict(meta, completion_tokens=i)}) + "\n\n").encode())
            await resp.write(b"data: [DONE]\n\n")
            return resp
        return web.json_response({"meta_info": meta})

    port = get_free_port()
    loop = asyncio.new_event_loop()
    app = web.Application()
    app.router.add_post("/generate", generate)
    runner = web.AppRunner(app)

    def serve():
        asyncio.set_event_loop(loop)
        loop.run_until_complete(runner.setup())
        loop.run_until_complete(web.TCPSite(runner, "127.0.0.1", port).start())
        loop.run_forever()

    t = threading.Thread(target=serve, daemon=True)
    t.start()
    import time
    time.sleep(0.5)
    out = tmp_path / "res.jsonl"
    try:
        args = bs.build_parser().parse_args([
            "--port", str(port), "--dataset-name", "generated-shared-prefix", "--gsp-num-groups", "2",
            "--gsp-prompts-per-group", "3", "--gsp-system-prompt-len", "8", "--gsp-question-len", "4",
            "--gsp-output-len", "5", "--gsp-ordered", "--gsp-send-routing-key", "--disable-stream",
            "--lora-name", "a", "b", "--lora-request-distribution", "distinct", "--header", "X-Test=yes",
            "--warmup-requests", "1", "--tag", "run-7", "--output-details", "--output-file", str(out),
            "--return-logprob", "--disable-ignore-eos"])
        m = bs.run_benchmark(args)
        assert m["completed"] == 6 and m["failed"] == 0 and m["tag"] == "run-7" and len(m["details"]) == 6
        timed = seen[1:]                                             # the first request is the warm-up
        assert len(seen) == 7 and all(h == "yes" for _, h in seen)
        assert [b["lora_path"] for b, _ in timed] == ["a", "b", "a", "b", "a", "b"]
        assert [b["routing_key"] for b, _ in timed] == ["group-0"] * 3 + ["group-1"] * 3
        assert all(b["stream"] is False and b["return_logprob"] is True for b, _ in timed)
        assert all(b["sampling_params"]["ignore_eos"] is False for b, _ in timed)
        assert json.loads(out.read_text().splitlines()[-1])["tag"] == "run-7"
        # the streaming path still measures inter-token times
        seen.clear()
        args = bs.build_parser().parse_args(["--port", str(port), "--dataset-name", "random", "--num-prompts", "3",
                                             "--random-input-len", "6", "--random-output-len", "4"])
        m = bs.run_benchmark(args)
        assert m["completed"] == 3 and m["total_output_tokens"] == 12 and all(b["stream"] for b, _ in seen)
    finally:
        loop.call_soon_threadsafe(loop.stop)
        t.join(timeout=5)


def test_offline_throughput_bench_on_a_tiny_model(tmp_path):
    """`bench_offline_throughput` through the in-process engine: random and shared-prefix datasets, result file."""
    import json
    from sglang_jax_b200 import bench_offline_throughput as bo
    from sglang_jax_b200.parallel import state as ps
    from sglang_jax_b200.utils.tiny_models import write_tiny_qwen3_checkpoint
    ckpt = write_tiny_qwen3_checkpoint(str(tmp_path / "m"))
    out = tmp_path / "r.jsonl"
    common = ["--model-path", ckpt, "--device", "cpu", "--dtype", "float32", "--skip-tokenizer-init",
              "--enable-single-process", "--page-size", "16", "--max-total-tokens", "4096", "--log-level", "error"]
    ps.reset_state()
    r = bo.main(common + ["--num-prompts", "5", "--random-input-len", "24", "--random-output-len", "6",
                          "--result-filename", str(out)])
    assert r["successful_requests"] == 5 and r["total_output_tokens"] == 30 and r["output_throughput"] > 0
    ps.reset_state()
    r = bo.main(common + ["--dataset-name", "generated-shared-prefix", "--gsp-num-groups", "2",
                          "--gsp-prompts-per-group", "2", "--gsp-system-prompt-len", "32", "--gsp-question-len", "8",
                          "--gsp-output-len", "4", "--skip-warmup", "--result-filename", str(out)])
    assert r["successful_requests"] == 4 and r["total_input_tokens"] == 4 * 40
    recs = [json.loads(l) for l in out.read_text().splitlines()]
    assert [x["dataset_name"] for x in recs] == ["random", "generated-shared-prefix"]


def test_bench_one_batch_options_and_correctness_test(tmp_path, capsys):
    """`bench_one_batch`: result file with the run name, decode-step logging, and `--correctness-test` (prefill in
    one piece against a cached prefix plus the rest)."""
    import json
    from sglang_jax_b200 import bench_one_batch as b1
    from sglang_jax_b200.parallel import state as ps
    from sglang_jax_b200.utils.tiny_models import write_tiny_qwen3_checkpoint
    ckpt = write_tiny_qwen3_checkpoint(str(tmp_path / "m"))
    common = ["--model-path", ckpt, "--device", "cpu", "--dtype", "float32", "--skip-tokenizer-init",
              "--enable-single-process", "--page-size", "16", "--max-total-tokens", "4096", "--log-level", "error"]
    ps.reset_state()
    out = tmp_path / "one.jsonl"
    recs = b1.main(common + ["--batch-size", "2", "--input-len", "32", "--output-len", "4", "--run-name", "r1",
                             "--result-filename", str(out), "--log-decode-step", "2"])
    assert recs[0]["run_name"] == "r1" and recs[0]["batch_size"] == 2 and recs[0]["median_decode_latency_s"] > 0
    assert "decode step 2:" in capsys.readouterr().out
    assert json.loads(out.read_text().splitlines()[0])["input_len"] == 32
    ps.reset_state()
    res = b1.main(common + ["--correctness-test", "--cut-len", "16", "--output-len", "5"])[0]
    assert res["passed"] and max(res["split_cached"]) == 16 and all(len(o) == 5 for o in res["whole"])


def test_bench_one_batch_server_against_a_fake_server(tmp_path, capsys):
    """`bench_one_batch_server`: streamed batches against a recording server, unequal prompt lengths, report, file."""
    import asyncio
    import json
    import threading
    import time
    from aiohttp import web
    from sglang_jax_b200 import bench_one_batch_server as b
    from sglang_jax_b200.utils.common import get_free_port
    seen = []

    async def generate(request):
        body = await request.json()
        seen.append(body)
        resp = web.StreamResponse(headers={"Content-Type": "text/event-stream"})
        await resp.prepare(request)
        for i in range(body["sampling_params"]["max_new_tokens"]):
            await resp.write(("data: " + json.dumps({"meta_info": {"completion_tokens": i + 1}}) + "\n\n").encode())
        await resp.write(b"data: [DONE]\n\n")
        return resp

    port = get_free_port()
    loop = asyncio.new_event_loop()
    app = web.Application()
    app.router.add_post("/generate", generate)
    runner = web.AppRunner(app)

    def serve():
        asyncio.set_event_loop(loop)
        loop.run_until_complete(runner.setup())
        loop.run_until_complete(web.TCPSite(runner, "127.0.0.1", port).start())
        loop.run_forever()

    t = threading.Thread(target=serve, daemon=True)
    t.start()
    time.sleep(0.5)
    out = tmp_path / "srv.jsonl"
    try:
        rows = b.main(["--base-url", f"http://127.0.0.1:{port}", "--batch-size", "2", "4", "--input-len", "40",
                       "--output-len", "3", "--input-len-step-percentage", "0.5", "--run-name", "s1", "--show-report",
                       "--result-filename", str(out), "--return-logprob"])
    finally:
        loop.call_soon_threadsafe(loop.stop)
        t.join(timeout=5)
    assert [r["batch_size"] for r in rows] == [2, 4] and all(r["run_name"] == "s1" and r["ttft_s"] for r in rows)
    assert len(seen) == 3 and len(seen[0]["input_ids"]) == 1                      # the warm-up request comes first
    assert [len(x) for x in seen[2]["input_ids"]] == [40, 35, 30, 25] and seen[2]["return_logprob"] is True
    assert "out tok/s" in capsys.readouterr().out and len(out.read_text().splitlines()) == 2


def test_framework_debug_listing_of_parameters(monkeypatch, capsys):
    """`SGLANG_FRAMEWORK_LOG_LEVEL>=3`: every parameter with its local shape, dtype and tensor-parallel slice."""
    import torch
    from sglang_jax_b200.layers.linear import ColumnParallelLinear
    from sglang_jax_b200.parallel import state as ps
    from sglang_jax_b200.utils import debug_utils as du
    ps.reset_state()
    m = torch.nn.Module()
    m.proj = ColumnParallelLinear(8, 16, False, torch.float32)
    lines = du.parameter_shardings(m)
    assert lines == ["proj.weight: shape=(16, 8) dtype=float32 device=cpu replicated"]
    monkeypatch.setenv("SGLANG_FRAMEWORK_LOG_LEVEL", "0")
    du.print_parameter_shardings(m)
    assert capsys.readouterr().out == ""
    monkeypatch.setenv("SGLANG_FRAMEWORK_LOG_LEVEL", "3")
    du.print_parameter_shardings(m)
    assert "proj.weight" in capsys.readouterr().out

    @du.log_shapes("f")
    def f(x):
        return x.sum(0), 3

    f(torch.zeros(2, 5))
    out = capsys.readouterr().out
    assert "f input[0]: (2, 5) float32 cpu" in out and "f output[0]: (5,) float32 cpu" in out
