"""Serving benchmark client (reference `python/sgl_jax/bench_serving.py`): an asyncio load generator
against the native `/generate`, the OpenAI `/v1/completions` or the `/v1/chat/completions` endpoint with the
datasets of the reference's `get_dataset` (:780): `random` (synthetic ids), `generated-shared-prefix` (:1778),
`sharegpt` (:1177, a local ShareGPT json), `custom` (a jsonl of prompts / conversations), `mooncake` (a jsonl
trace replayed at its own timestamps), `image` (:1624, synthetic images attached to chat requests) and `mmmu`
(:1092, a local copy of the benchmark), a request rate / max-concurrency limiter, and the
reference's metric definitions (`calculate_metrics` :1942-2117): TTFT = latency of the first streamed
chunk, ITL = gaps between chunks, TPOT = (latency - TTFT) / (output_len - 1), throughput =
tokens / duration, percentiles p50/p90/p99, peak output tok/s from 1-second buckets.  Request shaping and reporting
options of the reference client: `--disable-stream`, `--disable-ignore-eos`, `--apply-chat-template`,
`--prompt-suffix`, `--header`, `--served-model-name`, `--lora-name` with `--lora-request-distribution` /
`--lora-zipf-alpha`, `--return-logprob`, `--return-routed-experts`, `--gsp-ordered`, `--gsp-send-routing-key`,
`--warmup-requests`, `--tokenize-prompt`, `--print-requests`, `--output-details`, `--tag`.

    python -m sglang_jax_b200.bench_serving --backend sglang --dataset-name random \
        --random-input-len 1024 --random-output-len 512 --num-prompts 1024 --max-concurrency 64
"""

from __future__ import annotations

import argparse
import asyncio
import json
import random
import sys
import time
from dataclasses import dataclass, field

import numpy as np


@dataclass
class RequestFuncOutput:
    success: bool = False
    latency: float = 0.0
    ttft: float = 0.0
    itl: list[float] = field(default_factory=list)
    prompt_len: int = 0
    output_len: int = 0
    error: str = ""
    start: float = 0.0
    chunk_times: list[float] = field(default_factory=list)


def sample_random_requests(input_len: int, output_len: int, num_prompts: int, range_ratio: float, vocab_size: int,
                           seed: int = 1) -> list[tuple[list[int], int]]:
    rng = np.random.RandomState(seed)
    lo_i, lo_o = max(int(input_len * range_ratio), 1), max(int(output_len * range_ratio), 1)
    ins = rng.randint(lo_i, input_len + 1, size=num_prompts)
    outs = rng.randint(lo_o, output_len + 1, size=num_prompts)
    return [(rng.randint(0, vocab_size, size=int(n)).tolist(), int(o)) for n, o in zip(ins, outs)]


def sample_generated_shared_prefix_requests(num_groups: int, prompts_per_group: int, system_prompt_len: int,
                                            question_len: int, output_len: int, vocab_size: int, seed: int = 1,
                                            ordered: bool = False):
    """`(ids, output_len, None, group)`: the third slot is the departure offset of trace datasets (none here), the
    fourth names the group whose system prompt the request shares (`--gsp-send-routing-key`); `ordered` keeps the
    groups together instead of shuffling the requests."""
    rng = np.random.RandomState(seed)
    reqs = []
    for g in range(num_groups):
        sys_ids = rng.randint(0, vocab_size, size=system_prompt_len).tolist()
        for _ in range(prompts_per_group):
            reqs.append((sys_ids + rng.randint(0, vocab_size, size=question_len).tolist(), output_len, None, g))
    if not ordered:
        random.Random(seed).shuffle(reqs)
    return reqs


class _Lengths:
    """Token counts of text prompts: a HF tokenizer when `--tokenizer` names one, else whitespace words
    (good enough to size a load; the server reports exact counts in its usage fields)."""

    def __init__(self, path: str | None):
        self.tok = None
        if path:
            from transformers import AutoTokenizer
            self.tok = AutoTokenizer.from_pretrained(path)

    def __call__(self, text: str) -> int:
        return len(self.tok.encode(text)) if self.tok is not None else max(len(text.split()), 1)


def sample_sharegpt_requests(path: str, num_prompts: int, lengths: _Lengths, fixed_output_len: int | None = None,
                             context_len: int | None = None, seed: int = 1):
    """ShareGPT json: a list of `{"conversations": [{"from": "human", "value": ...}, {"from": "gpt", ...}]}`.
    The first human turn is the prompt, the length of the first reply the output length (reference :1177)."""
    with open(path) as f:
        data = json.load(f)
    data = [d for d in data if len(d.get("conversations", d.get("conversation", []))) >= 2]
    random.Random(seed).shuffle(data)
    reqs = []
    for d in data:
        conv = d.get("conversations", d.get("conversation"))
        prompt, reply = conv[0]["value"], conv[1]["value"]
        n_in = lengths(prompt)
        n_out = fixed_output_len or lengths(reply)
        if n_in < 2 or n_out < 2 or (context_len and n_in + n_out > context_len):
            continue
        reqs.append((prompt, n_out))
        if len(reqs) == num_prompts:
            break
    return reqs


def sample_custom_requests(path: str, num_prompts: int, lengths: _Lengths, fixed_output_len: int | None = None,
                           seed: int = 1):
    """jsonl, one request per line: `{"prompt": str | [ids], "output_len": int}` or
    `{"conversations": [...]}` in the ShareGPT turn format."""
    reqs = []
    with open(path) as f:
        for line in f:
            line = line.strip()
            if not line:
                continue
            d = json.loads(line)
            if "conversations" in d:
                conv = d["conversations"]
                prompt = conv[0].get("value", conv[0].get("content", ""))
                n_out = fixed_output_len or (lengths(conv[1].get("value", conv[1].get("content", ""))) if len(conv) > 1 else 128)
            else:
                prompt = d.get("prompt", d.get("input_ids"))
                n_out = fixed_output_len or int(d.get("output_len", d.get("max_tokens", 128)))
            reqs.append((prompt, n_out))
            if len(reqs) == num_prompts:
                break
    return reqs


def sample_mooncake_requests(path: str, num_prompts: int, vocab_size: int, block_tokens: int = 512, seed: int = 1):
    """Mooncake trace jsonl: `{"timestamp": ms, "input_length": n, "output_length": m, "hash_ids": [...]}`.
    Each hash id stands for one block of `block_tokens` tokens, so equal ids reproduce the trace's prefix sharing;
    returns `(ids, output_len, arrival_s)` triples."""
    reqs = []
    with open(path) as f:
        for line in f:
            if not line.strip():
                continue
            d = json.loads(line)
            ids: list[int] = []
            for h in d.get("hash_ids", []):
                ids.extend(np.random.RandomState(int(h) % (2 ** 31)).randint(0, vocab_size, size=block_tokens).tolist())
            n = int(d["input_length"])
            if len(ids) < n:
                ids.extend(np.random.RandomState(seed + len(reqs)).randint(0, vocab_size, size=n - len(ids)).tolist())
            reqs.append((ids[:n], int(d["output_length"]), float(d.get("timestamp", 0)) / 1000.0))
            if len(reqs) == num_prompts:
                break
    return reqs


def _png_data_url(width: int, height: int, rng) -> str:
    """A random RGB image as a base64 PNG data URL (stored-deflate blocks, no imaging library needed)."""
    import base64
    import struct
    import zlib
    raw = b"".join(b"\x00" + rng.bytes(width * 3) for _ in range(height))

    def chunk(kind: bytes, data: bytes) -> bytes:
        return struct.pack(">I", len(data)) + kind + data + struct.pack(">I", zlib.crc32(kind + data) & 0xFFFFFFFF)

    png = b"\x89PNG\r\n\x1a\n" + chunk(b"IHDR", struct.pack(">IIBBBBB", width, height, 8, 2, 0, 0, 0)) + \
        chunk(b"IDAT", zlib.compress(raw, 1)) + chunk(b"IEND", b"")
    return "data:image/png;base64," + base64.b64encode(png).decode()


def sample_image_requests(num_prompts: int, image_count: int, resolution: str, input_len: int, output_len: int,
                          seed: int = 1):
    """Chat requests with `image_count` synthetic images of `resolution` (`WxH`, or 360p/720p/1080p/4k) and a random
    text of about `input_len` words (reference :1624); returns `(messages, output_len)` pairs."""
    presets = {"360p": (640, 360), "720p": (1280, 720), "1080p": (1920, 1080), "4k": (3840, 2160)}
    w, h = presets[resolution] if resolution in presets else tuple(int(x) for x in resolution.lower().split("x"))
    rng = np.random.RandomState(seed)
    reqs = []
    for _ in range(num_prompts):
        content = [{"type": "image_url", "image_url": {"url": _png_data_url(w, h, rng)}} for _ in range(image_count)]
        content.append({"type": "text", "text": " ".join(f"w{int(x)}" for x in rng.randint(0, 5000, size=input_len))})
        reqs.append(([{"role": "user", "content": content}], output_len))
    return reqs


def sample_mmmu_requests(path: str, num_prompts: int, output_len: int):
    """A local MMMU split as jsonl (`{"question": ..., "options": [...], "image": <path or data url>}`); the hub
    copy cannot be fetched offline (reference :1092 downloads it)."""
    reqs = []
    with open(path) as f:
        for line in f:
            if not line.strip():
                continue
            d = json.loads(line)
            img = d.get("image") or d.get("image_1")
            if img and not str(img).startswith("data:"):
                import base64
                with open(img, "rb") as g:
                    img = "data:image/png;base64," + base64.b64encode(g.read()).decode()
            text = d["question"] + "".join(f"\n({chr(65 + i)}) {o}" for i, o in enumerate(d.get("options", [])))
            content = ([{"type": "image_url", "image_url": {"url": img}}] if img else []) + [{"type": "text", "text": text}]
            reqs.append(([{"role": "user", "content": content}], output_len))
            if len(reqs) == num_prompts:
                break
    return reqs


async def _request_openai_chat(session, url, messages, out_len, extra, model) -> RequestFuncOutput:
    out = RequestFuncOutput(prompt_len=sum(len(str(m.get("content", ""))) for m in messages) // 4)
    body = {"model": model, "messages": messages, "max_tokens": out_len, "temperature": 0.0, "stream": True,
            "ignore_eos": True, "stream_options": {"include_usage": True}, **extra}
    out.start = st = time.perf_counter()
    last, n = st, 0
    try:
        async with session.post(url + "/v1/chat/completions", json=body) as resp:
            if resp.status != 200:
                out.error = f"HTTP {resp.status}"
                return out
            async for raw in resp.content:
                line = raw.decode().strip()
                if not line.startswith("data:") or line.endswith("[DONE]"):
                    continue
                d = json.loads(line[5:])
                now = time.perf_counter()
                if d.get("usage"):
                    out.output_len = d["usage"]["completion_tokens"]
                    out.prompt_len = d["usage"].get("prompt_tokens", out.prompt_len)
                if d.get("choices") and (d["choices"][0].get("delta") or {}).get("content"):
                    if n == 0:
                        out.ttft = now - st
                    else:
                        out.itl.append(now - last)
                    out.chunk_times.append(now)
                    last = now
                    n += 1
        out.latency = time.perf_counter() - st
        out.output_len = out.output_len or n
        out.success = n > 0
    except Exception as e:
        out.error = repr(e)
    return out


async def _request_sglang_generate(session, url, ids, out_len, extra, opt=None) -> RequestFuncOutput:
    opt = opt or {}
    out = RequestFuncOutput(prompt_len=len(ids) if not isinstance(ids, str) else max(len(ids.split()), 1))
    body = {("text" if isinstance(ids, str) else "input_ids"): ids, "stream": not opt.get("disable_stream"),
            "sampling_params": {"temperature": 0.0, "max_new_tokens": out_len,
                                "ignore_eos": not opt.get("disable_ignore_eos"), **extra}}
    for k in ("lora_path", "return_logprob", "return_routed_experts", "routing_key"):
        if opt.get(k) is not None:
            body[k] = opt[k]
    if opt.get("disable_stream"):
        out.start = st = time.perf_counter()
        try:
            async with session.post(url + "/generate", json=body) as resp:
                if resp.status != 200:
                    out.error = f"HTTP {resp.status}: {await resp.text()}"
                    return out
                d = await resp.json()
            out.latency = out.ttft = time.perf_counter() - st
            out.output_len = d["meta_info"]["completion_tokens"]
            out.prompt_len = d["meta_info"].get("prompt_tokens", out.prompt_len)
            out.chunk_times.append(time.perf_counter())
            out.success = out.output_len > 0
        except Exception as e:
            out.error = repr(e)
        return out
    out.start = st = time.perf_counter()
    last = st
    n_tok = 0
    try:
        async with session.post(url + "/generate", json=body) as resp:
            if resp.status != 200:
                out.error = f"HTTP {resp.status}: {await resp.text()}"
                return out
            async for raw in resp.content:
                line = raw.decode().strip()
                if not line.startswith("data:"):
                    continue
                payload = line[5:].strip()
                if payload == "[DONE]":
                    break
                d = json.loads(payload)
                if "error" in d:
                    out.error = str(d["error"])
                    return out
                now = time.perf_counter()
                n_new = d["meta_info"]["completion_tokens"]
                out.prompt_len = d["meta_info"].get("prompt_tokens", out.prompt_len)
                if n_new > n_tok:
                    if n_tok == 0:
                        out.ttft = now - st
                    else:
                        out.itl.extend([(now - last) / (n_new - n_tok)] * (n_new - n_tok))
                    out.chunk_times.append(now)
                    last = now
                    n_tok = n_new
        out.latency = time.perf_counter() - st
        out.output_len = n_tok
        out.success = n_tok > 0
    except Exception as e:  # connection errors are data, not crashes
        out.error = repr(e)
    return out


async def _request_openai_completions(session, url, ids, out_len, extra, model) -> RequestFuncOutput:
    out = RequestFuncOutput(prompt_len=len(ids) if not isinstance(ids, str) else max(len(ids.split()), 1))
    body = {"model": model, "prompt": ids, "max_tokens": out_len, "temperature": 0.0, "stream": True,
            "ignore_eos": True, "stream_options": {"include_usage": True}, **extra}
    out.start = st = time.perf_counter()
    last = st
    n = 0
    try:
        async with session.post(url + "/v1/completions", json=body) as resp:
            if resp.status != 200:
                out.error = f"HTTP {resp.status}"
                return out
            async for raw in resp.content:
                line = raw.decode().strip()
                if not line.startswith("data:") or line.endswith("[DONE]"):
                    continue
                d = json.loads(line[5:])
                now = time.perf_counter()
                if d.get("usage"):
                    out.output_len = d["usage"]["completion_tokens"]
                if d.get("choices"):
                    if n == 0:
                        out.ttft = now - st
                    else:
                        out.itl.append(now - last)
                    out.chunk_times.append(now)
                    last = now
                    n += 1
        out.latency = time.perf_counter() - st
        out.output_len = out.output_len or n
        out.success = n > 0
    except Exception as e:
        out.error = repr(e)
    return out


def calculate_metrics(outputs: list[RequestFuncOutput], duration: float) -> dict:
    ok = [o for o in outputs if o.success]
    ttfts = [o.ttft for o in ok]
    itls = [x for o in ok for x in o.itl]
    tpots = [(o.latency - o.ttft) / (o.output_len - 1) for o in ok if o.output_len > 1]
    e2e = [o.latency for o in ok]
    total_in = sum(o.prompt_len for o in ok)
    total_out = sum(o.output_len for o in ok)

    def pct(xs, q):
        return float(np.percentile(xs, q)) * 1000 if xs else 0.0

    # peak output throughput over 1-second buckets of chunk arrival times
    peak = 0.0
    if ok:
        t0 = min(o.start for o in ok)
        buckets: dict[int, int] = {}
        for o in ok:
            per = o.output_len / max(len(o.chunk_times), 1)
            for t in o.chunk_times:
                buckets[int(t - t0)] = buckets.get(int(t - t0), 0) + per
        peak = max(buckets.values()) if buckets else 0.0
    m = {"completed": len(ok), "failed": len(outputs) - len(ok), "duration_s": duration,
         "total_input_tokens": total_in, "total_output_tokens": total_out,
         "request_throughput": len(ok) / duration, "input_throughput": total_in / duration,
         "output_throughput": total_out / duration, "total_throughput": (total_in + total_out) / duration,
         "peak_output_throughput": peak, "concurrency": sum(e2e) / duration if duration else 0.0}
    for name, xs in (("ttft", ttfts), ("itl", itls), ("tpot", tpots), ("e2e_latency", e2e)):
        m[f"mean_{name}_ms"] = float(np.mean(xs)) * 1000 if xs else 0.0
        m[f"median_{name}_ms"] = pct(xs, 50)
        m[f"p90_{name}_ms"] = pct(xs, 90)
        m[f"p99_{name}_ms"] = pct(xs, 99)
    return m


async def benchmark(args, reqs) -> dict:
    import aiohttp
    url = args.base_url or f"http://{args.host}:{args.port}"
    extra = json.loads(args.extra_request_body) if args.extra_request_body else {}
    sem = asyncio.Semaphore(args.max_concurrency) if args.max_concurrency else None
    timeout = aiohttp.ClientTimeout(total=6 * 3600)
    conn = aiohttp.TCPConnector(limit=0)
    headers = dict(h.split("=", 1) for h in (args.header or []))
    async with aiohttp.ClientSession(timeout=timeout, connector=conn, headers=headers or None) as session:
        if args.flush_cache:
            async with session.post(url + "/flush_cache"):
                pass

        model = args.served_model_name or args.model or "default"
        lora_rng = np.random.RandomState(args.seed)

        def pick_lora(i: int):
            """`--lora-name a b c` with `--lora-request-distribution`: uniform draws, distinct = round robin, skewed =
            Zipf over the list (`--lora-zipf-alpha`)."""
            names = args.lora_name or []
            if not names:
                return None
            if args.lora_request_distribution == "distinct":
                return names[i % len(names)]
            if args.lora_request_distribution == "skewed":
                w = 1.0 / np.arange(1, len(names) + 1) ** args.lora_zipf_alpha
                return names[int(lora_rng.choice(len(names), p=w / w.sum()))]
            return names[int(lora_rng.randint(len(names)))]

        async def one(ids, out_len, index=0, routing_key=None):
            opt = {"disable_stream": args.disable_stream, "disable_ignore_eos": args.disable_ignore_eos,
                   "lora_path": pick_lora(index), "return_logprob": True if args.return_logprob else None,
                   "return_routed_experts": True if args.return_routed_experts else None,
                   "routing_key": routing_key if args.gsp_send_routing_key else None}
            if isinstance(ids, str) and args.prompt_suffix:
                ids = ids + args.prompt_suffix
            if args.print_requests:
                print(json.dumps({"index": index, "prompt": ids if isinstance(ids, str) else f"<{len(ids)} items>",
                                  "output_len": out_len, "lora": opt["lora_path"]}))

            async def call():
                if isinstance(ids, list) and ids and isinstance(ids[0], dict):       # chat messages (image datasets)
                    return await _request_openai_chat(session, url, ids, out_len, extra, model)
                if args.backend == "sglang":
                    return await _request_sglang_generate(session, url, ids, out_len, extra, opt)
                if args.backend == "sglang-oai-chat" or (args.apply_chat_template and isinstance(ids, str)):
                    msgs = [{"role": "user", "content": ids if isinstance(ids, str) else " ".join(map(str, ids))}]
                    return await _request_openai_chat(session, url, msgs, out_len, extra, model)
                return await _request_openai_completions(session, url, ids, out_len, extra, model)
            if sem is None:
                return await call()
            async with sem:
                return await call()

        for w in range(min(args.warmup_requests, len(reqs))):      # untimed, one at a time
            await one(reqs[w][0], min(reqs[w][1], 16), w)
        if args.profile:
            async with session.post(url + "/start_profile", json={"num_steps": args.profile_num_steps}):
                pass
        t0 = time.perf_counter()
        tasks = []
        for i, req in enumerate(reqs):
            ids, out_len = req[0], req[1]
            if len(req) > 2 and req[2] is not None:
                # trace replay: the request leaves at its recorded offset (scaled by --mooncake-slowdown-factor)
                wait = req[2] * args.mooncake_slowdown_factor - (time.perf_counter() - t0)
                if wait > 0:
                    await asyncio.sleep(wait)
            tasks.append(asyncio.create_task(one(ids, out_len, i, f"group-{req[3]}" if len(req) > 3 else None)))
            if (len(req) == 2 or req[2] is None) and args.request_rate != float("inf"):
                await asyncio.sleep(np.random.exponential(1.0 / args.request_rate))
        outputs = await asyncio.gather(*tasks)
        duration = time.perf_counter() - t0
    m = calculate_metrics(outputs, duration)
    m.update(backend=args.backend, dataset_name=args.dataset_name, request_rate=args.request_rate,
             max_concurrency=args.max_concurrency)
    if args.tag:
        m["tag"] = args.tag
    if args.output_details:
        m["details"] = [{"prompt_len": o.prompt_len, "output_len": o.output_len, "ttft": o.ttft, "latency": o.latency,
                         "itl": o.itl, "error": o.error} for o in outputs]
    errs = [o.error for o in outputs if not o.success][:3]
    if errs:
        m["errors"] = errs
    return m


def print_metrics(m: dict):
    w = 50
    print("=" * w + "\n" + " Serving Benchmark Result ".center(w, "=") + "\n")
    for k in ("backend", "max_concurrency", "completed", "failed", "duration_s", "total_input_tokens",
              "total_output_tokens", "request_throughput", "input_throughput", "output_throughput",
              "peak_output_throughput", "total_throughput", "concurrency"):
        v = m.get(k)
        print(f"{k:<36}{v:>14.2f}" if isinstance(v, float) else f"{k:<36}{str(v):>14}")
    for name in ("ttft", "tpot", "itl", "e2e_latency"):
        print(f"--- {name} (ms): mean {m[f'mean_{name}_ms']:.2f}  median {m[f'median_{name}_ms']:.2f}  "
              f"p90 {m[f'p90_{name}_ms']:.2f}  p99 {m[f'p99_{name}_ms']:.2f}")
    print("=" * w)


def run_benchmark(args) -> dict:
    random.seed(args.seed)
    np.random.seed(args.seed)
    if args.dataset_name == "random":
        reqs = sample_random_requests(args.random_input_len, args.random_output_len, args.num_prompts,
                                      args.random_range_ratio, args.vocab_size, args.seed)
    elif args.dataset_name == "generated-shared-prefix":
        reqs = sample_generated_shared_prefix_requests(args.gsp_num_groups, args.gsp_prompts_per_group,
                                                       args.gsp_system_prompt_len, args.gsp_question_len,
                                                       args.gsp_output_len, args.vocab_size, args.seed,
                                                       args.gsp_ordered)
    elif args.dataset_name in ("sharegpt", "custom", "mooncake", "mmmu"):
        if not args.dataset_path:
            raise SystemExit(f"dataset {args.dataset_name} reads a local file (there is no network to fetch it): "
                             f"pass --dataset-path")
        lengths = _Lengths(args.tokenizer)
        if args.dataset_name == "sharegpt":
            reqs = sample_sharegpt_requests(args.dataset_path, args.num_prompts, lengths, args.sharegpt_output_len,
                                            args.sharegpt_context_len, args.seed)
        elif args.dataset_name == "custom":
            reqs = sample_custom_requests(args.dataset_path, args.num_prompts, lengths, args.sharegpt_output_len,
                                          args.seed)
        elif args.dataset_name == "mooncake":
            reqs = sample_mooncake_requests(args.dataset_path, args.num_prompts, args.vocab_size,
                                            args.mooncake_block_tokens, args.seed)
        else:
            reqs = sample_mmmu_requests(args.dataset_path, args.num_prompts, args.random_output_len)
    elif args.dataset_name == "image":
        reqs = sample_image_requests(args.num_prompts, args.image_count, args.image_resolution,
                                     args.random_input_len, args.random_output_len, args.seed)
    else:
        raise SystemExit(f"unknown dataset {args.dataset_name}")
    if args.tokenize_prompt:
        # send token ids instead of text (needs --tokenizer): the server's tokenizer is left out of the measurement
        if not args.tokenizer:
            raise SystemExit("--tokenize-prompt needs --tokenizer")
        from transformers import AutoTokenizer
        tok = AutoTokenizer.from_pretrained(args.tokenizer)
        reqs = [((tok.encode(r[0]) if isinstance(r[0], str) else r[0]), *r[1:]) for r in reqs]
    m = asyncio.run(benchmark(args, reqs))
    print_metrics(m)
    if args.output_file:
        with open(args.output_file, "a") as f:
            f.write(json.dumps(m) + "\n")
    return m


def build_parser():
    p = argparse.ArgumentParser()
    p.add_argument("--backend", default="sglang", choices=["sglang", "sglang-oai", "sglang-oai-chat", "vllm"])
    p.add_argument("--base-url", default=None)
    p.add_argument("--host", default="127.0.0.1")
    p.add_argument("--port", type=int, default=30000)
    p.add_argument("--model", default=None)
    p.add_argument("--dataset-name", default="random",
                   choices=["random", "generated-shared-prefix", "sharegpt", "custom", "mooncake", "image", "mmmu"])
    p.add_argument("--dataset-path", default=None, help="local file of the sharegpt / custom / mooncake / mmmu datasets")
    p.add_argument("--tokenizer", default=None, help="HF tokenizer directory used to size text prompts")
    p.add_argument("--sharegpt-output-len", type=int, default=None)
    p.add_argument("--sharegpt-context-len", type=int, default=None)
    p.add_argument("--mooncake-slowdown-factor", type=float, default=1.0)
    p.add_argument("--mooncake-block-tokens", type=int, default=512)
    p.add_argument("--image-count", type=int, default=1)
    p.add_argument("--image-resolution", default="360p")
    p.add_argument("--num-prompts", type=int, default=1000)
    p.add_argument("--random-input-len", type=int, default=1024)
    p.add_argument("--random-output-len", type=int, default=1024)
    p.add_argument("--random-range-ratio", type=float, default=1.0)
    p.add_argument("--vocab-size", type=int, default=32000)
    p.add_argument("--request-rate", type=float, default=float("inf"))
    p.add_argument("--max-concurrency", type=int, default=None)
    p.add_argument("--gsp-num-groups", type=int, default=64)
    p.add_argument("--gsp-prompts-per-group", type=int, default=16)
    p.add_argument("--gsp-system-prompt-len", type=int, default=2048)
    p.add_argument("--gsp-question-len", type=int, default=128)
    p.add_argument("--gsp-output-len", type=int, default=256)
    p.add_argument("--seed", type=int, default=1)
    p.add_argument("--disable-stream", action="store_true", help="non-streaming requests (TTFT equals the latency)")
    p.add_argument("--disable-ignore-eos", action="store_true")
    p.add_argument("--apply-chat-template", action="store_true", help="text prompts go through the chat route")
    p.add_argument("--prompt-suffix", default="", help="appended to every text prompt")
    p.add_argument("--header", nargs="*", default=None, help="extra HTTP headers, KEY=VALUE")
    p.add_argument("--served-model-name", default=None)
    p.add_argument("--lora-name", nargs="*", default=None, help="adapters the requests are spread over")
    p.add_argument("--lora-request-distribution", default="uniform", choices=["uniform", "distinct", "skewed"])
    p.add_argument("--lora-zipf-alpha", type=float, default=1.5)
    p.add_argument("--return-logprob", action="store_true")
    p.add_argument("--return-routed-experts", action="store_true")
    p.add_argument("--gsp-ordered", action="store_true", help="keep the groups together instead of shuffling")
    p.add_argument("--gsp-send-routing-key", action="store_true",
                   help="generated-shared-prefix: requests of one group carry the group's routing key")
    p.add_argument("--warmup-requests", type=int, default=0)
    p.add_argument("--tokenize-prompt", action="store_true")
    p.add_argument("--print-requests", action="store_true")
    p.add_argument("--output-details", action="store_true", help="per-request records in the output file")
    p.add_argument("--tag", default=None, help="label copied into the result record")
    p.add_argument("--extra-request-body", default=None)
    p.add_argument("--output-file", default=None)
    p.add_argument("--flush-cache", action="store_true")
    p.add_argument("--profile", action="store_true")
    p.add_argument("--profile-num-steps", type=int, default=5)
    return p


if __name__ == "__main__":
    run_benchmark(build_parser().parse_args())
