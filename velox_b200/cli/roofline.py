"""How close decode steps come to the memory roofline, and prompt portions to the matrix-product
peak, per layer, over sizes, batches and contexts.

    python -m velox_b200.cli.roofline --model-size 1.5b,7b --batch 1,8,64 --context 512,4096,32000
    python -m velox_b200.cli.roofline --model-size 1.5b,7b --prefill 512,2048 --context 0,8192,30000

For every named configuration two models with random weights are built, with ``--layers A,B``
layers (2 and 6 unless told otherwise); for every batch and context each runs decode steps whose
sequences hold that many keys, and the difference of the two step times over B - A is what one
layer costs: embedding, head, sampling and the host's share of a step cancel.  A layer has to read
its matrices once and the keys and values of the live requests; those bytes over the layer's time,
against the measured copy bandwidth, is the fraction printed.  The reference has no counterpart;
its benchmark reports tokens per second only (benchmark.py:233-262 of that project).

The cache is not filled through the model (the keys are whatever the pool holds): the step's work
does not depend on their values.  Steps are queued back to back, each fed the tokens the step
before it sampled (on the device), so the device never waits for the host.

With ``--prefill T,...`` the steps are portions of T prompt tokens of one sequence behind
``--context`` keys instead: a layer's floating-point operations (two per weight and token, four
per query, key and head dimension under the causal mask) over its time, against the measured
library bf16 rate.
"""
from __future__ import annotations

import argparse
import json
import sys
import tempfile
from typing import Dict, List, Optional, Tuple


def parse_args(argv: Optional[List[str]] = None) -> argparse.Namespace:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--model-size", default="1.5b", help="named configurations, comma separated")
    parser.add_argument("--batch", default="1,8,64")
    parser.add_argument("--context", default="512,4096")
    parser.add_argument("--prefill", default=None, metavar="T,...",
                        help="time prompt portions of so many tokens behind --context keys instead of decode steps")
    parser.add_argument("--layers", default="2,6", help="the two layer counts whose difference is taken")
    parser.add_argument("--block-size", type=int, default=16)
    parser.add_argument("--steps", type=int, default=24)
    parser.add_argument("--warmup", type=int, default=4)
    parser.add_argument("--output-json", default=None)
    return parser.parse_args(argv)


def _latent_layers(config_json: Dict) -> Optional[List[Dict]]:
    """The per-layer entries of a configuration that lists its layers (latent attention and a
    dense feed-forward with gates), or None for a configuration of uniform Qwen2 layers."""
    return config_json.get("layers")


def _is_redalix(config_json: Dict) -> bool:
    return config_json.get("architecture") == "Redalix" or "Redalix" in (config_json.get("architectures") or [])


def _redalix_attention(m: Dict, width: int) -> Tuple[int, int, int]:
    """(weights, cached values per key, rounded head size) of one windowed attention mixer."""
    head = -(-max(m["dim"], m["vdim"]) // 16) * 16
    weights = width * (m["heads"] * m["dim"] + m["kv_heads"] * (m["dim"] + m["vdim"])) + m["heads"] * m["vdim"] * width
    if "rot" in m:
        weights += m["heads"] * width  # the gate per head
    return weights, 2 * m["kv_heads"] * head, head


def _redalix_layer(entry: Dict, width: int, tokens: int, batch: int, context: int):
    """(weights read, bytes of cache and state touched, operations) of one layer for ``tokens``
    new tokens of each of ``batch`` sequences behind ``context`` keys.  Experts: as many as the
    step's tokens can name; a window bounds the keys a token reads; a state is read and written."""
    kind, m = entry["type"], entry["mixer"]
    weights = cache = 0
    flops = 0.0
    rows = batch * tokens

    def attention(a):
        nonlocal weights, cache, flops
        w, per_key, head = _redalix_attention(a, width)
        weights += w
        reach = a["mask"]["size"] + a["mask"].get("keep_first", 0)
        cache += batch * min(context + tokens, reach + tokens) * per_key * 2
        pairs = sum(min(context + i + 1, reach) for i in range(tokens)) if tokens <= 4096 else tokens * reach
        flops += 2.0 * rows * w + 4.0 * batch * pairs * a["heads"] * head

    if kind == "attention":
        attention(m)
    elif kind == "parallel":
        attention(m["left"])
        r = m["right"]
        part = r["width"] // r["blocks"]
        weights += 3 * r["width"] * width
        flops += 2.0 * rows * 3 * r["width"] * width + 2.0 * rows * 2 * r["width"] * part
        weights += 2 * 2 * r["width"] * part  # the two gate matrices are float32
        cache += batch * r["conv"] * r["width"] * 4 * 2
    else:
        inner = m["heads"] * m["vdim"]
        rows_in = 2 * inner + 2 * m["groups"] * m["state"] + m["heads"]
        weights += rows_in * width + inner * width
        flops += 2.0 * rows * (rows_in + inner) * width + 6.0 * rows * inner * m["state"]
        cache += batch * (m["heads"] * m["state"] * m["vdim"] + (m["conv"] - 1) * (inner + 2 * m["groups"] * m["state"])) * 4 * 2
    mlp = entry.get("mlp")
    if mlp is not None:
        if mlp["kind"] == "dense":
            weights += 2 * mlp["ff"] * width
            flops += 2.0 * rows * 2 * mlp["ff"] * width
        else:
            used = min(mlp["router"]["experts"], rows * mlp["router"]["top"])
            weights += used * 2 * mlp["expert"]["ff"] * width
            flops += 2.0 * rows * mlp["router"]["top"] * 2 * mlp["expert"]["ff"] * width
            if mlp.get("shared"):
                weights += (2 * mlp["shared"]["ff"] + 1) * width
                flops += 2.0 * rows * 2 * mlp["shared"]["ff"] * width
    return 2 * weights, cache, flops


def _is_lizizen(config_json: Dict) -> bool:
    return config_json.get("architecture") == "Lizizen" or "Lizizen" in (config_json.get("architectures") or [])


def _lizizen_layer(entry: Dict, width: int, tokens: int, batch: int, context: int):
    """(bytes of weights read, bytes of cache and state touched, operations) of one Lizizen layer
    for ``tokens`` new tokens of each of ``batch`` sequences behind ``context`` keys.  A cached
    row is as wide as the attention kernels' head: both maps' keys side by side for
    ``attention_2``, whose chunked mask bounds the keys a token reads and whose two maps are two
    score products over one set of values."""
    m = entry["mixer"]
    rows = batch * tokens
    maps = 2 if entry["type"] == "attention_2" else 1
    head = -(-max(maps * m["dim"], m["vdim"]) // 16) * 16
    weights = width * (m["heads"] * maps * m["dim"] + m["kv_heads"] * (maps * m["dim"] + m["vdim"])) + m["heads"] * m["vdim"] * width
    if maps == 2:
        weights += m["heads"] * m["vdim"] * width  # the output gate
    reach = (m.get("mask") or {}).get("size") or (context + tokens)
    if tokens <= 4096:
        if maps == 2 and m.get("mask"):
            pairs = sum((context + i) % reach + 1 for i in range(tokens))
        else:
            pairs = sum(context + i + 1 for i in range(tokens))
    else:
        pairs = tokens * min(reach, context + tokens) / 2
    cache = batch * min(context + tokens, reach + tokens) * 2 * m["kv_heads"] * head * 2
    cache += batch * width * 4 * 2  # the shift's row, read and written
    flops = 2.0 * rows * weights + 4.0 * batch * pairs * maps * m["heads"] * head
    mlp = entry.get("mlp")
    if mlp is not None:
        weights += 3 * mlp["ff"] * width
        flops += 2.0 * rows * 3 * mlp["ff"] * width
    return 2 * weights, cache, flops


def _is_mamivik(config_json: Dict) -> bool:
    return config_json.get("architecture") == "Mamivik" or "Mamivik" in (config_json.get("architectures") or [])


def _mamivik_layer(entry: Dict, width: int, tokens: int, batch: int, context: int):
    """(bytes of weights read, bytes of cache and state touched, operations) of one Mamivik layer
    for ``tokens`` new tokens of each of ``batch`` sequences behind ``context`` keys.  A window
    bounds the keys a token reads; the latent layer's scores and sums run over the cached rows, as
    the engine computes them; the delta rule's state is read and written once a step and costs six
    operations per entry and token; the decay's inner size is the random-weights default."""
    from ..config.model_config import DeltaRuleConfig
    from ..models.mamivik import default_decay_rank

    m = entry["mixer"]
    rows = batch * tokens
    cache = batch * 3 * width * 4 * 2  # the convolution's rows (at most; read and written)
    flops = 0.0

    def pairs_within(reach):
        if tokens <= 4096:
            return sum(min(context + i + 1, reach) for i in range(tokens))
        return tokens * min(reach, context + tokens / 2)

    if entry["type"] == "latent_attention":
        heads, q_head, row = m["heads"], m["dim"] + m["rot_dim"], m["kv_rank"] + m["rot_dim"]
        padded = -(-row // 16) * 16
        weights = ((m["q_rank"] + row + heads * m["vdim"]) * width + heads * q_head * m["q_rank"]
                   + heads * (m["dim"] + m["vdim"]) * m["kv_rank"] + width * heads * m["vdim"])
        reach = m["mask"]["size"]
        cache += batch * min(context + tokens, reach + tokens) * padded * 2
        flops += 2.0 * rows * weights + 4.0 * batch * pairs_within(reach) * heads * padded
    else:
        a, d = m["left"], m["right"]
        head = -(-a["dim"] // 16) * 16
        inner = d["heads"] * d["dim"]
        rank = default_decay_rank(DeltaRuleConfig(d["heads"], d["dim"]))
        weights = (width * (a["heads"] + a["kv_heads"]) * a["dim"] + a["heads"] * a["dim"] * width
                   + (5 * inner + rank) * width + inner * rank + inner * width)
        reach = a["mask"]["size"]
        cache += batch * min(context + tokens, reach + tokens) * 2 * a["kv_heads"] * head * 2
        cache += batch * inner * d["dim"] * 4 * 2
        flops += 2.0 * rows * weights + 4.0 * batch * pairs_within(reach) * a["heads"] * head
        flops += 6.0 * rows * inner * d["dim"]
    mlp = entry.get("mlp")
    if mlp is not None:
        weights += 3 * mlp["ff"] * width
        flops += 2.0 * rows * 3 * mlp["ff"] * width
    return 2 * weights, cache, flops


def _listed_layer(config_json: Dict):
    """The per-layer accounting of a design whose layers differ in kind, or None."""
    if _is_redalix(config_json):
        return _redalix_layer
    if _is_lizizen(config_json):
        return _lizizen_layer
    if _is_mamivik(config_json):
        return _mamivik_layer
    return None


def layer_bytes(config_json: Dict, batch: int, context: int) -> Tuple[int, int]:
    """(bytes of one layer's matrices in bfloat16, bytes of ``batch`` x ``context`` cached rows of
    one layer: keys and values, or the latent rows that serve as both), averaged over the layers
    of a configuration that lists them."""
    entries = _latent_layers(config_json)
    if entries is not None and _listed_layer(config_json) is not None:
        parts = [_listed_layer(config_json)(entry, config_json["width"], 1, batch, context) for entry in entries]
        return sum(p[0] for p in parts) // len(parts), sum(p[1] for p in parts) // len(parts)
    if entries is not None:
        width = config_json["width"]
        weights = cache = 0
        for entry in entries:
            m = entry["mixer"]
            heads, q_head, row = m["heads"], m["dim"] + m["rot_dim"], m["kv_rank"] + m["rot_dim"]
            rows_in = heads * q_head + heads + width + (row if m.get("kv_from") is None else 0)
            weights += 2 * (rows_in * width + heads * (m["dim"] + m["vdim"]) * m["kv_rank"] + width * heads * m["vdim"])
            if entry.get("mlp") is not None:
                weights += 2 * ((entry["mlp"]["ff"] + width) * width + width * entry["mlp"]["ff"])
            cache += batch * context * (-(-row // 16) * 16) * 2
        return weights // len(entries), cache // len(entries)
    width, heads, kv_heads = config_json["hidden_size"], config_json["num_attention_heads"], config_json["num_key_value_heads"]
    inner = config_json["intermediate_size"]
    head_dim = config_json.get("head_dim") or width // heads
    weights = 2 * (width * (heads + 2 * kv_heads) * head_dim + heads * head_dim * width + 3 * width * inner)
    cache = batch * context * kv_heads * head_dim * 2 * 2
    return weights, cache


def layer_flops(config_json: Dict, tokens: int, context: int) -> float:
    """Floating-point operations of one layer on a portion of ``tokens`` behind ``context`` keys
    (for latent attention: as the engine computes it, scores and sums over the cached rows)."""
    entries = _latent_layers(config_json)
    pairs = tokens * (context + (tokens + 1) / 2.0)
    if entries is not None and _listed_layer(config_json) is not None:
        return sum(_listed_layer(config_json)(entry, config_json["width"], tokens, 1, context)[2] for entry in entries) / len(entries)
    if entries is not None:
        weights, _ = layer_bytes(config_json, 0, 0)
        attention = 0.0
        for entry in entries:
            m = entry["mixer"]
            attention += 2.0 * pairs * m["heads"] * (2 * m["kv_rank"] + m["rot_dim"])
        return 2.0 * tokens * (weights / 2) + attention / len(entries)
    width, heads, kv_heads = config_json["hidden_size"], config_json["num_attention_heads"], config_json["num_key_value_heads"]
    inner = config_json["intermediate_size"]
    head_dim = config_json.get("head_dim") or width // heads
    weights = width * (heads + 2 * kv_heads) * head_dim + heads * head_dim * width + 3 * width * inner
    return 2.0 * tokens * weights + 4.0 * pairs * heads * head_dim


def launch_times(config_json: Dict, layers: int, args, batch: int = 0, tokens: int = 0, context: int = 0,
                 repeats: int = 5) -> Dict[str, float]:
    """Microseconds of every kind of launch, summed over one step of a model of ``layers`` layers
    (``batch`` single tokens behind ``context`` keys each, or one portion of ``tokens``): the step
    is launched kernel by kernel behind a queued delay with a CUDA event after every launch
    (``ops.kernels.launch_events``); the median over ``repeats`` steps."""
    import torch

    from ..config import EngineConfig
    from ..config.presets import with_layers
    from ..engine.engine import Engine
    from ..engine.runner import StepChunk
    from ..ops import kernels
    from ..weights import write_random_model

    seqs_n, per_seq = (batch, 1) if batch else (1, tokens)
    most_keys = context + per_seq + 8
    with tempfile.TemporaryDirectory(prefix="velox_roofline_") as folder:
        write_random_model(folder, with_layers(config_json, layers), seed=0, dtype="bfloat16")
        engine = Engine.from_pretrained(EngineConfig(
            model=folder, dtype="bfloat16", max_model_len=most_keys, max_num_seqs=max(seqs_n, 2),
            max_num_batched_tokens=max(256, per_seq, seqs_n), max_prefill_chunk_size=max(256, per_seq),
            block_size=args.block_size, num_gpu_blocks=max(seqs_n, 2) * (-(-most_keys // args.block_size) + 1) + 8,
            seed=0, enable_cuda_graphs=False))
    runner, cache = engine.runner, engine.cache
    seqs = []
    for index in range(seqs_n):
        seq = cache.new_sequence(f"k{index}")
        if not (cache.acquire_slot(seq) and cache.append_slots(seq, context + per_seq)):
            raise RuntimeError(f"the pool does not hold {seqs_n} sequences of {context + per_seq} keys")
        cache.advance(seq, context)
        seqs.append(seq)
    chunks = [StepChunk(seq, [1 + (i % 97) for i in range(per_seq)], (per_seq - 1,)) for seq in seqs]
    runs = []
    for _ in range(repeats + 2):
        ctx, ids, rows, count = runner.prepare(chunks)
        torch.cuda.synchronize()
        torch.cuda._sleep(40_000_000)
        first = torch.cuda.Event(enable_timing=True)
        first.record()
        kernels.launch_events = []
        try:
            runner.model.forward(ctx, runner.layer_caches, ids, rows, count)
        finally:
            events, kernels.launch_events = kernels.launch_events, None
        torch.cuda.synchronize()
        took, previous = [], first
        for name, event in events:
            took.append((name, previous.elapsed_time(event) * 1000.0))
            previous = event
        runs.append(took)
    runs = runs[2:]
    out: Dict[str, float] = {}
    for index, (name, _) in enumerate(runs[0]):
        values = sorted(run[index][1] for run in runs)
        out[name] = out.get(name, 0.0) + values[len(values) // 2]
    runner.check_status()
    del engine, runner, cache
    torch.cuda.empty_cache()
    return out


def layer_launch_times(config_json: Dict, few: int, many: int, args, **step) -> Dict[str, float]:
    """Microseconds one layer spends in every kind of launch: ``launch_times`` of a model of
    ``many`` layers minus that of one of ``few``, over the difference (what is outside the layers
    cancels)."""
    short = launch_times(config_json, few, args, **step)
    long = launch_times(config_json, many, args, **step)
    return {name: round((long[name] - short.get(name, 0.0)) / (many - few), 2) for name in long}


def portion_times(config_json: Dict, layers: int, portions: List[int], contexts: List[int], args) -> Dict[Tuple[int, int], float]:
    """Milliseconds of a step that is one portion of a prompt, for every (portion, context)."""
    import torch

    from ..config import EngineConfig
    from ..engine.engine import Engine
    from ..engine.runner import StepChunk
    from ..config.presets import with_layers
    from ..weights import write_random_model

    most_tokens, most_keys = max(portions), max(contexts) + max(portions) + 8
    with tempfile.TemporaryDirectory(prefix="velox_roofline_") as folder:
        write_random_model(folder, with_layers(config_json, layers), seed=0, dtype="bfloat16")
        engine = Engine.from_pretrained(EngineConfig(
            model=folder, dtype="bfloat16", max_model_len=most_keys, max_num_seqs=2,
            max_num_batched_tokens=most_tokens, max_prefill_chunk_size=most_tokens, block_size=args.block_size,
            num_gpu_blocks=2 * (-(-most_keys // args.block_size) + 1) + 8, seed=0))
    runner, cache = engine.runner, engine.cache
    times: Dict[Tuple[int, int], float] = {}
    for tokens in portions:
        ids = [1 + (i % 97) for i in range(tokens)]
        for context in contexts:
            measured = []
            for repeat in range(args.warmup + 3):
                seq = cache.new_sequence(f"p{tokens}_{context}_{repeat}")
                if not (cache.acquire_slot(seq) and cache.append_slots(seq, context + tokens)):
                    raise RuntimeError(f"the pool does not hold {context + tokens} keys")
                cache.advance(seq, context)
                start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                start.record()
                runner.step([StepChunk(seq, ids, (tokens - 1,))])
                end.record()
                torch.cuda.synchronize()
                cache.free(seq)
                cache.release_slot(seq)
                if repeat >= args.warmup:
                    measured.append(start.elapsed_time(end))
            times[(tokens, context)] = sorted(measured)[len(measured) // 2]
    runner.check_status()
    del engine, runner, cache
    torch.cuda.empty_cache()
    return times


def step_times(config_json: Dict, layers: int, batches: List[int], contexts: List[int], args) -> Dict[Tuple[int, int], float]:
    """Milliseconds of a decode step for every (batch, context), with ``layers`` layers."""
    import torch

    from ..config import EngineConfig
    from ..engine.engine import Engine
    from ..engine.runner import StepChunk
    from ..sampling.params import SamplingParams
    from ..config.presets import with_layers
    from ..weights import write_random_model

    most_seqs, most_keys = max(batches), max(contexts) + args.steps + args.warmup + 2
    with tempfile.TemporaryDirectory(prefix="velox_roofline_") as folder:
        write_random_model(folder, with_layers(config_json, layers), seed=0, dtype="bfloat16")
        engine = Engine.from_pretrained(EngineConfig(
            model=folder, dtype="bfloat16", max_model_len=most_keys, max_num_seqs=most_seqs,
            max_num_batched_tokens=max(256, most_seqs), max_prefill_chunk_size=256, block_size=args.block_size,
            num_gpu_blocks=most_seqs * (-(-most_keys // args.block_size) + 1) + 8, seed=0))
    runner, cache, sampler = engine.runner, engine.cache, engine.sampler
    times: Dict[Tuple[int, int], float] = {}
    for batch in batches:
        params = [SamplingParams(temperature=0.0, max_tokens=1)] * batch
        names = [f"s{i}" for i in range(batch)]
        for context in contexts:
            seqs = []
            for name in names:
                seq = cache.new_sequence(name)
                if not (cache.acquire_slot(seq) and cache.append_slots(seq, context)):
                    raise RuntimeError(f"the pool does not hold {batch} sequences of {context} keys")
                cache.advance(seq, context)
                seqs.append(seq)

            def one_step(ids):
                chunks = []
                for seq, token in zip(seqs, ids):
                    cache.append_slots(seq, 1)
                    chunks.append(StepChunk(seq, [token], (0,)))
                logits = runner.step(chunks)
                sampler.sample(logits, params, names, [0] * batch)
                for seq in seqs:
                    cache.advance(seq, 1)

            for _ in range(args.warmup):
                one_step([1] * batch)
            fed = [-1 - row for row in range(batch)]
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            for _ in range(args.steps):
                one_step(fed)
            end.record()
            torch.cuda.synchronize()
            times[(batch, context)] = start.elapsed_time(end) / args.steps
            for seq in seqs:
                cache.free(seq)
                cache.release_slot(seq)
    runner.check_status()
    del engine, runner, cache, sampler
    torch.cuda.empty_cache()
    return times


def main(argv: Optional[List[str]] = None) -> int:
    args = parse_args(argv)
    from ..config.presets import model_size
    from .benchmark import bf16_peak_tflops, hbm_peak_gbs

    batches = [int(v) for v in args.batch.split(",")]
    contexts = [int(v) for v in args.context.split(",")]
    few, many = (int(v) for v in args.layers.split(","))
    if not 0 < few < many:
        raise SystemExit("--layers A,B needs 0 < A < B")
    rows = []
    if args.prefill:
        portions = [int(v) for v in args.prefill.split(",")]
        rate = bf16_peak_tflops()
        print(f"{'size':>6} {'tokens':>6} {'context':>7} {'us/layer':>9} {'TFLOP/s':>8} {'fraction':>8}")
        for name in args.model_size.split(","):
            config_json = model_size(name)
            short = portion_times(config_json, few, portions, contexts, args)
            long = portion_times(config_json, many, portions, contexts, args)
            for tokens in portions:
                for context in contexts:
                    seconds = (long[(tokens, context)] - short[(tokens, context)]) / (many - few) * 1e-3
                    achieved = layer_flops(config_json, tokens, context) / seconds / 1e12 if seconds > 0 else 0.0
                    row = {"size": name, "tokens": tokens, "context": context, "us_per_layer": round(seconds * 1e6, 1),
                           "tflops": round(achieved, 1), "bf16_frac": round(achieved / rate, 3), "bf16_peak_tflops": rate,
                           "kv_block_size": args.block_size}
                    rows.append(row)
                    print(f"{name:>6} {tokens:>6} {context:>7} {row['us_per_layer']:>9.1f} {row['tflops']:>8.1f} "
                          f"{row['bf16_frac']:>8.3f}", flush=True)
        if args.output_json:
            with open(args.output_json, "w", encoding="utf-8") as handle:
                json.dump(rows, handle, indent=1)
        return 0
    peak = hbm_peak_gbs()
    print(f"{'size':>6} {'batch':>5} {'context':>7} {'us/layer':>9} {'by bytes':>9} {'fraction':>8}  cache share")
    for name in args.model_size.split(","):
        config_json = model_size(name)
        short = step_times(config_json, few, batches, contexts, args)
        long = step_times(config_json, many, batches, contexts, args)
        for batch in batches:
            for context in contexts:
                # the sequences grow while they are timed: count the keys of the middle step
                keys = context + args.warmup + args.steps // 2
                weights, cached = layer_bytes(config_json, batch, keys)
                seconds = (long[(batch, context)] - short[(batch, context)]) / (many - few) * 1e-3
                ideal = (weights + cached) / (peak * 1e9)
                row = {"size": name, "batch": batch, "context": context, "us_per_layer": round(seconds * 1e6, 1),
                       "us_by_bytes": round(ideal * 1e6, 1), "hbm_frac": round(ideal / seconds, 3) if seconds > 0 else None,
                       "cache_share": round(cached / (weights + cached), 2), "hbm_peak_gbs": peak,
                       "kv_block_size": args.block_size}
                rows.append(row)
                print(f"{name:>6} {batch:>5} {context:>7} {row['us_per_layer']:>9.1f} {row['us_by_bytes']:>9.1f} "
                      f"{row['hbm_frac']:>8.3f}  {row['cache_share']:.2f}", flush=True)
    if args.output_json:
        with open(args.output_json, "w", encoding="utf-8") as handle:
            json.dump(rows, handle, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
